// Host orchestration of the batched Muon step: groups weights by Newton-Schulz
// shape, owns the packed bf16 scratch and issues, per group,
//   momentum (1 launch) -> Frobenius normalise (2) -> ns_steps x 3 GEMM phases -> update (1)
// on the caller's stream, with no host synchronisation.  This is the role of
// BatchedProjMuon / ResidentMuon / the expert branch of GroupedMoEFFN.step in the
// reference (ancora/optim/muon.py:180-201,256-277; ancora/kernels/moe.py:578-588),
// except that a whole shape group is batched at once: a B200 has the HBM for it and
// the GEMM kernel's tile scheduler needs thousands of tiles to fill 148 SMs.
#include <algorithm>
#include <map>
#include <math.h>
#include <vector>
#include "anc_internal.h"

namespace {

struct Group {
  int M, Nn;                       // Newton-Schulz orientation, M <= Nn
  std::vector<int> widx;           // plan weight indices, in registration order
  anc_mom_entry *d_mom = nullptr;  // device tables, one entry per weight
  anc_upd_entry *d_upd = nullptr;
  anc_upd_extra *d_ext = nullptr;  // optional extra outputs of the update (nullptr: none in this group)
  anc_tmap *d_maps = nullptr;      // three 64x64-box tensor maps per weight (momentum buffer, gradient, master
                                   // weight): how the sweeps fetch the tiles of tall (K > N) weights
  anc_tmap omap[2];                // the packed operands X and Y seen as slots of (M, Nn) bf16, for the same sweeps
  double scale_tall = 1.0;         // sqrt(max(1, K/N)) for the K > N members
};

struct TimedSpan {
  int phase;
  cudaEvent_t a, b;
};

}  // namespace

struct anc_muon_plan {
  anc_ctx *ctx;
  int grad_dtype;
  int max_batch;
  std::vector<anc_muon_weight> weights;   // owned weights only
  std::vector<anc_muon_outputs> outputs;  // parallel to weights (all-null entries when unused)
  std::vector<Group> groups;
  uint16_t *X = nullptr, *Y = nullptr, *A = nullptr, *B = nullptr;
  float *recip = nullptr;
  float *partial = nullptr;       // per-tile sums of squares written by the momentum kernel
  uint32_t *sched = nullptr;      // scheduler words of the chain kernel: 2 + largest batch
  uint64_t scratch_bytes = 0;
  bool timing = false;
  std::vector<TimedSpan> spans;
  double last_flops = 0.0;
  double last_flops_executed = 0.0;
  int last_launches = 0;
};

// The chain on an UN-normalised X: the Frobenius factor r[e] = recip[e] enters through the
// epilogues of the first iteration (A = r^2 X X^T, Y = r (B' X)), which equals the chain on r*X
// without ever writing r*X back to memory.  The iteration's a*X term is folded into the
// polynomial, B' = b A + c A A + a I, so that the new iterate is the plain product B' X
// (the reference forms a*X + B X in the last epilogue, ancora/kernels/muon_ns.py:268-273).
// sched: the chain kernel's scheduler words (cleared by the Frobenius finalize kernel); when it
// is NULL, or the shape is outside the chain kernel's reach, every phase is its own launch.
static int ns_chain(anc_ctx *ctx, uint16_t *&X, uint16_t *A, uint16_t *B, uint16_t *&Y, int E, int M,
                    int N, int steps, const float *coeffs, const float *recip, uint32_t *sched,
                    cudaStream_t st) {
  if (sched && anc_ns_chain_supported(ctx, M, N, steps)) {
    int rc = anc_launch_ns_chain(ctx, X, Y, A, B, E, M, N, steps, coeffs, recip, sched, 0, st);
    if (rc) return rc;
    if (steps & 1) std::swap(X, Y);
    return ANC_OK;
  }
  for (int k = 0; k < steps; ++k) {
    const float a = coeffs[3 * k], b = coeffs[3 * k + 1], c = coeffs[3 * k + 2];
    const float *ms = (k == 0) ? recip : nullptr;
    int rc = anc_launch_ns_gemm(ctx, 0, X, nullptr, A, E, M, N, 0.f, 1.f, 0.f, ms, st);
    if (rc) return rc;
    rc = anc_launch_ns_gemm(ctx, 1, A, nullptr, B, E, M, N, b, c, a, nullptr, st);   // B' = bA + cAA + aI
    if (rc) return rc;
    rc = anc_launch_ns_gemm(ctx, 2, B, X, Y, E, M, N, 0.f, 1.f, 0.f, ms, st);        // X' = B' X
    if (rc) return rc;
    std::swap(X, Y);
  }
  return ANC_OK;
}

static void plan_free(anc_muon_plan *pl) {
  for (auto &g : pl->groups) {
    if (g.d_maps) cudaFree(g.d_maps);
    if (g.d_mom) cudaFree(g.d_mom);
    if (g.d_upd) cudaFree(g.d_upd);
    if (g.d_ext) cudaFree(g.d_ext);
  }
  for (void *p : {(void *)pl->X, (void *)pl->Y, (void *)pl->A, (void *)pl->B, (void *)pl->recip,
                  (void *)pl->partial, (void *)pl->sched})
    if (p) cudaFree(p);
  for (auto &s : pl->spans) {
    cudaEventDestroy(s.a);
    cudaEventDestroy(s.b);
  }
  delete pl;
}

extern "C" {

int anc_muon_plan_create(anc_ctx *ctx, const anc_muon_weight *weights, int n_weights, int grad_dtype,
                         int my_rank, int max_batch, anc_muon_plan **out) {
  return anc_muon_plan_create_ex(ctx, weights, nullptr, n_weights, grad_dtype, my_rank, max_batch, out);
}

int anc_muon_plan_create_ex(anc_ctx *ctx, const anc_muon_weight *weights, const anc_muon_outputs *outputs,
                            int n_weights, int grad_dtype, int my_rank, int max_batch,
                            anc_muon_plan **out) {
  ANC_REQUIRE(ctx && out && (weights || n_weights == 0), "NULL argument");
  ANC_REQUIRE(grad_dtype == ANC_GRAD_BF16 || grad_dtype == ANC_GRAD_F32, "bad grad_dtype");
  *out = nullptr;
  anc_device_guard guard(ctx->device);
  anc_muon_plan *pl = new anc_muon_plan();
  pl->ctx = ctx;
  pl->grad_dtype = grad_dtype;
  pl->max_batch = max_batch;
  std::map<std::pair<int, int>, int> gindex;
  for (int i = 0; i < n_weights; ++i) {
    const anc_muon_weight &w = weights[i];
    if (w.owner >= 0 && w.owner != my_rank) continue;
    if (!w.buf || !w.g || !w.p32 || !w.p16) {
      anc_set_error("Muon weight %d has a NULL pointer", i);
      plan_free(pl);
      return ANC_E_INVALID;
    }
    if (w.K <= 0 || w.N <= 0 || w.K % 128 || w.N % 128) {
      anc_set_error("Muon weight (%d,%d) tile-misaligned: K and N must be multiples of 128", w.K, w.N);
      plan_free(pl);
      return ANC_E_INVALID;
    }
    const int M = std::min(w.K, w.N), Nn = std::max(w.K, w.N);
    auto key = std::make_pair(M, Nn);
    auto it = gindex.find(key);
    if (it == gindex.end()) {
      gindex[key] = (int)pl->groups.size();
      Group g;
      g.M = M;
      g.Nn = Nn;
      g.scale_tall = pow((double)Nn / (double)M, 0.5);   // Python's max(1, K/N) ** 0.5
      pl->groups.push_back(g);
      it = gindex.find(key);
    }
    pl->groups[it->second].widx.push_back((int)pl->weights.size());
    pl->weights.push_back(w);
    anc_muon_outputs o = {nullptr, nullptr, nullptr, nullptr, nullptr};
    if (outputs) o = outputs[i];
    if ((o.fp8 == nullptr) != (o.fp8_scale == nullptr) || (o.fp8_t == nullptr) != (o.fp8_scale_t == nullptr)) {
      anc_set_error("Muon weight %d: an fp8 output and its scale output must be given together", i);
      plan_free(pl);
      return ANC_E_INVALID;
    }
    if (((uintptr_t)o.fp8 & 7) || ((uintptr_t)o.fp8_t & 15) || ((uintptr_t)o.p16_t & 15)) {
      anc_set_error("Muon weight %d: fp8 needs 8-byte, fp8_t and p16_t 16-byte alignment", i);
      plan_free(pl);
      return ANC_E_INVALID;
    }
    pl->outputs.push_back(o);
  }
  {
    int rc = anc_elem_kernels_prepare(ctx);
    if (rc) {
      plan_free(pl);
      return rc;
    }
  }
  // scratch: sized for the largest batch over all groups
  size_t xe = 0, ae = 0, emax = 0;
  for (auto &g : pl->groups) {
    const size_t E = pl->max_batch > 0 ? std::min<size_t>(pl->max_batch, g.widx.size()) : g.widx.size();
    xe = std::max(xe, E * (size_t)g.M * g.Nn);
    ae = std::max(ae, E * (size_t)g.M * g.M);
    emax = std::max(emax, E);
    std::vector<anc_mom_entry> mom;
    std::vector<anc_upd_entry> upd;
    std::vector<anc_upd_extra> ext;
    std::vector<anc_tmap> maps(3 * g.widx.size());
    bool any_ext = false;
    for (size_t s = 0; s < g.widx.size(); ++s) {
      const anc_muon_weight &w = pl->weights[g.widx[s]];
      if (w.K > w.N) {
        const int gb = grad_dtype == ANC_GRAD_F32 ? 4 : 2;
        int rc = anc_encode_tile_map(&maps[3 * s], w.buf, 4, (uint64_t)w.N, (uint64_t)w.K, 0, 64, 64);
        if (!rc) rc = anc_encode_tile_map(&maps[3 * s + 1], w.g, gb, (uint64_t)w.N, (uint64_t)w.K, 0, 64, 64);
        if (!rc) rc = anc_encode_tile_map(&maps[3 * s + 2], w.p32, 4, (uint64_t)w.N, (uint64_t)w.K, 0, 64, 64);
        if (rc) {
          plan_free(pl);
          return rc;
        }
      }
      mom.push_back({w.buf, w.g, w.K, w.N, w.K > w.N ? 1 : 0, 0});
      upd.push_back({w.p32, w.p16, w.K, w.N, w.K > w.N ? 1 : 0, 0});
      const anc_muon_outputs &o = pl->outputs[g.widx[s]];
      ext.push_back({o.fp8, o.fp8_scale, o.p16_t, o.fp8_t, o.fp8_scale_t, 0});
      any_ext = any_ext || o.fp8 || o.p16_t || o.fp8_t;
    }
    if (any_ext) {
      cudaError_t ee = cudaMalloc((void **)&g.d_ext, ext.size() * sizeof(anc_upd_extra));
      if (ee == cudaSuccess)
        ee = cudaMemcpy(g.d_ext, ext.data(), ext.size() * sizeof(anc_upd_extra), cudaMemcpyHostToDevice);
      if (ee != cudaSuccess) {
        plan_free(pl);
        return anc_cuda_fail(ee, "muon output table");
      }
    }
    cudaError_t e = cudaMalloc((void **)&g.d_mom, mom.size() * sizeof(anc_mom_entry));
    if (e == cudaSuccess) e = cudaMalloc((void **)&g.d_upd, upd.size() * sizeof(anc_upd_entry));
    if (e == cudaSuccess) e = cudaMalloc((void **)&g.d_maps, maps.size() * sizeof(anc_tmap));
    if (e == cudaSuccess)
      e = cudaMemcpy(g.d_maps, maps.data(), maps.size() * sizeof(anc_tmap), cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
      e = cudaMemcpy(g.d_mom, mom.data(), mom.size() * sizeof(anc_mom_entry), cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
      e = cudaMemcpy(g.d_upd, upd.data(), upd.size() * sizeof(anc_upd_entry), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      plan_free(pl);
      return anc_cuda_fail(e, "muon tables");
    }
  }
  if (xe) {
    cudaError_t e = cudaMalloc((void **)&pl->X, xe * 2);
    if (e == cudaSuccess) e = cudaMalloc((void **)&pl->Y, xe * 2);
    if (e == cudaSuccess) e = cudaMalloc((void **)&pl->A, ae * 2);
    if (e == cudaSuccess) e = cudaMalloc((void **)&pl->B, ae * 2);
    if (e == cudaSuccess) e = cudaMalloc((void **)&pl->recip, emax * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc((void **)&pl->partial, (xe / 4096) * 8 * sizeof(float));   // 8 warp sums per 64x64 tile
    if (e == cudaSuccess) e = cudaMalloc((void **)&pl->sched, (emax + 2) * sizeof(uint32_t));
    if (e != cudaSuccess) {
      plan_free(pl);
      return anc_cuda_fail(e, "muon scratch");
    }
    pl->scratch_bytes = 4 * xe + 4 * ae + emax * sizeof(float) + (xe / 4096) * 8 * sizeof(float);
    for (auto &g : pl->groups) {
      const size_t E = pl->max_batch > 0 ? std::min<size_t>(pl->max_batch, g.widx.size()) : g.widx.size();
      int rc = anc_encode_tile_map(&g.omap[0], pl->X, 2, (uint64_t)g.Nn, (uint64_t)g.M, E, 64, 64);
      if (!rc) rc = anc_encode_tile_map(&g.omap[1], pl->Y, 2, (uint64_t)g.Nn, (uint64_t)g.M, E, 64, 64);
      if (rc) {
        plan_free(pl);
        return rc;
      }
    }
  }
  *out = pl;
  return ANC_OK;
}

}  // extern "C"

namespace {

struct ChunkRef {
  int group, w0, count;
};

// Chunks in execution order: shape groups in order of first appearance, each cut into
// batches of at most max_batch matrices.
std::vector<ChunkRef> plan_chunks(const anc_muon_plan *pl) {
  std::vector<ChunkRef> out;
  for (size_t gi = 0; gi < pl->groups.size(); ++gi) {
    const int total = (int)pl->groups[gi].widx.size();
    const int cap = pl->max_batch > 0 ? std::min(pl->max_batch, total) : total;
    for (int w0 = 0; w0 < total; w0 += cap) out.push_back({(int)gi, w0, std::min(cap, total - w0)});
  }
  return out;
}

int step_chunk(anc_muon_plan *pl, const ChunkRef &c, double lr, float momentum, int nesterov,
               int ns_steps, const float *coeffs, float eps, cudaStream_t st) {
  anc_ctx *ctx = pl->ctx;
  Group &g = pl->groups[c.group];
  auto begin_span = [&](int phase) {
    if (!pl->timing) return;
    TimedSpan sp;
    sp.phase = phase;
    cudaEventCreate(&sp.a);
    cudaEventCreate(&sp.b);
    cudaEventRecord(sp.a, st);
    pl->spans.push_back(sp);
  };
  auto end_span = [&]() {
    if (!pl->timing) return;
    cudaEventRecord(pl->spans.back().b, st);
  };
  const int epw = g.M * g.Nn;
  // lr * sqrt(max(1, K/N)) in double, then one float32 rounding (ancora/optim/muon.py:176,200)
  const float scale_wide = (float)(lr * 1.0);
  const float scale_tall = (float)(lr * g.scale_tall);
  const int E = c.count;
  uint16_t *X = pl->X, *Y = pl->Y;
  begin_span(0);
  int rc = anc_launch_momentum_group(ctx, g.d_mom + c.w0, g.d_maps + 3 * (size_t)c.w0, X, E, epw, pl->grad_dtype,
                                     momentum, nesterov, pl->partial, st);
  end_span();
  if (rc) return rc;
  begin_span(1);
  if (ns_steps > 0)   // 1/(||u||_F + eps) per matrix from the momentum kernel's tile sums
    rc = anc_launch_fro_finalize(ctx, pl->partial, pl->recip, E, epw / 4096, 1, eps, pl->sched, st);
  else                // no iteration to fold the factor into: normalise in place
    rc = anc_launch_fro_normalize(ctx, X, pl->recip, E, g.M, g.Nn, eps, st);
  end_span();
  if (rc) return rc;
  begin_span(2);
  rc = ns_chain(ctx, X, pl->A, pl->B, Y, E, g.M, g.Nn, ns_steps, coeffs, pl->recip, pl->sched, st);
  end_span();
  if (rc) return rc;
  pl->last_flops +=
      (double)E * ns_steps * (4.0 * g.M * (double)g.M * g.Nn + 2.0 * g.M * (double)g.M * g.M);
  // executed by the tensor cores: the symmetric phases compute the pair tiles on or below the
  // diagonal only (mb2*(mb2+1)/2 of mb2^2 tiles of 256x256), the apply phase everything
  {
    const double nb = (g.M % 256 == 0) ? g.M / 256.0 : g.M / 128.0;   // tile rows: CTA-pair or single-CTA kernel
    const double sym_frac = (nb + 1.0) / (2.0 * nb);
    pl->last_flops_executed += (double)E * ns_steps *
                               (sym_frac * (2.0 * g.M * (double)g.M * g.Nn + 2.0 * g.M * (double)g.M * g.M) +
                                2.0 * g.M * (double)g.M * g.Nn);
  }
  pl->last_launches += (ns_steps > 0 && anc_ns_chain_supported(ctx, g.M, g.Nn, ns_steps)) ? 1 : 3 * ns_steps;
  begin_span(3);
  rc = anc_launch_update_group(ctx, g.d_upd + c.w0, g.d_maps + 3 * (size_t)c.w0, &g.omap[X == pl->X ? 0 : 1],
                               g.d_ext ? (const void *)(g.d_ext + c.w0) : nullptr, X, E, epw, scale_wide,
                               scale_tall, st);
  end_span();
  return rc;
}

}  // namespace

extern "C" {

int anc_muon_step(anc_muon_plan *pl, double lr, float momentum, int nesterov, int ns_steps,
                  const float *coeffs, float eps, void *stream) {
  ANC_REQUIRE(pl && (coeffs || ns_steps == 0), "NULL argument");
  ANC_REQUIRE(ns_steps >= 0 && ns_steps <= 64, "bad ns_steps %d", ns_steps);
  anc_device_guard guard(pl->ctx->device);
  cudaStream_t st = anc_pick_stream(pl->ctx, stream);
  for (const ChunkRef &c : plan_chunks(pl)) {
    int rc = step_chunk(pl, c, lr, momentum, nesterov, ns_steps, coeffs, eps, st);
    if (rc) return rc;
  }
  return ANC_OK;
}

int anc_muon_plan_num_groups(anc_muon_plan *pl, int *n) {
  ANC_REQUIRE(pl && n, "NULL argument");
  *n = (int)pl->groups.size();
  return ANC_OK;
}

int anc_muon_plan_group_info(anc_muon_plan *pl, int group, int32_t info[4]) {
  ANC_REQUIRE(pl && info, "NULL argument");
  ANC_REQUIRE(group >= 0 && group < (int)pl->groups.size(), "group %d out of range", group);
  const Group &g = pl->groups[group];
  info[0] = (int)g.widx.size();
  info[1] = pl->max_batch > 0 ? std::min(pl->max_batch, (int)g.widx.size()) : (int)g.widx.size();
  info[2] = g.M;
  info[3] = g.Nn;
  return ANC_OK;
}

int anc_muon_step_range(anc_muon_plan *pl, int group, int first, int count, double lr, float momentum,
                        int nesterov, int ns_steps, const float *coeffs, float eps, void *stream) {
  ANC_REQUIRE(pl && (coeffs || ns_steps == 0), "NULL argument");
  ANC_REQUIRE(ns_steps >= 0 && ns_steps <= 64, "bad ns_steps %d", ns_steps);
  ANC_REQUIRE(group >= 0 && group < (int)pl->groups.size(), "group %d out of range", group);
  const int total = (int)pl->groups[group].widx.size();
  const int cap = pl->max_batch > 0 ? std::min(pl->max_batch, total) : total;
  ANC_REQUIRE(first >= 0 && count > 0 && first + count <= total, "range [%d,+%d) outside the group's %d weights",
              first, count, total);
  ANC_REQUIRE(count <= cap, "range of %d matrices exceeds the scratch batch of %d", count, cap);
  anc_device_guard guard(pl->ctx->device);
  ChunkRef c = {group, first, count};
  return step_chunk(pl, c, lr, momentum, nesterov, ns_steps, coeffs, eps,
                    anc_pick_stream(pl->ctx, stream));
}

int anc_muon_plan_set_timing(anc_muon_plan *pl, int on) {
  ANC_REQUIRE(pl, "plan is NULL");
  pl->timing = on != 0;
  return ANC_OK;
}

int anc_muon_plan_last_timing(anc_muon_plan *pl, float ms[4], double ns_flops[2], int *ns_launches) {
  ANC_REQUIRE(pl && ms, "NULL argument");
  anc_device_guard guard(pl->ctx->device);
  for (int i = 0; i < 4; ++i) ms[i] = 0.f;
  for (auto &s : pl->spans) {
    ANC_CUDA(cudaEventSynchronize(s.b));
    float t = 0.f;
    ANC_CUDA(cudaEventElapsedTime(&t, s.a, s.b));
    ms[s.phase] += t;
  }
  if (ns_flops) {
    ns_flops[0] = pl->last_flops;            // dense count: steps * (4 M^2 N + 2 M^3) per matrix
    ns_flops[1] = pl->last_flops_executed;   // what the tensor cores ran (lower pair tiles only in the symmetric phases)
  }
  if (ns_launches) *ns_launches = pl->last_launches;
  for (auto &s : pl->spans) {
    cudaEventDestroy(s.a);
    cudaEventDestroy(s.b);
  }
  pl->spans.clear();
  pl->last_flops = 0.0;
  pl->last_flops_executed = 0.0;
  pl->last_launches = 0;
  return ANC_OK;
}

int anc_muon_plan_scratch_bytes(anc_muon_plan *pl, uint64_t *bytes) {
  ANC_REQUIRE(pl && bytes, "NULL argument");
  *bytes = pl->scratch_bytes;
  return ANC_OK;
}

int anc_muon_plan_destroy(anc_muon_plan *pl) {
  if (!pl) return ANC_OK;
  anc_device_guard guard(pl->ctx->device);
  cudaStreamSynchronize(pl->ctx->stream);
  plan_free(pl);
  return ANC_OK;
}

int anc_ns_batched(anc_ctx *ctx, uint16_t *X, uint16_t *A, uint16_t *B, uint16_t *Y, float *recip,
                   int E, int M, int N, int steps, const float *coeffs, float eps, void *stream) {
  return anc_ns_batched_ex(ctx, X, A, B, Y, recip, E, M, N, steps, coeffs, eps, 1, stream);
}

int anc_ns_batched_ex(anc_ctx *ctx, uint16_t *X, uint16_t *A, uint16_t *B, uint16_t *Y, float *recip,
                      int E, int M, int N, int steps, const float *coeffs, float eps, int single_launch,
                      void *stream) {
  ANC_REQUIRE(ctx && X && A && B && Y && recip && (coeffs || steps == 0), "NULL argument");
  ANC_REQUIRE(M <= N, "Newton-Schulz needs M <= N (got %d x %d); transpose tall weights first", M, N);
  ANC_REQUIRE(M % 128 == 0 && N % 128 == 0, "NS shape (%d,%d) must be multiples of 128", M, N);
  anc_device_guard guard(ctx->device);
  cudaStream_t st = anc_pick_stream(ctx, stream);
  if (steps == 0) return anc_launch_fro_normalize(ctx, X, recip, E, M, N, eps, st);
  // block sums of squares -> recip; the factor itself is applied inside the first iteration
  const size_t bpm = ((size_t)M * N) / 16384;
  // workspace: E * bpm partial sums, then the chain kernel's 2 + E scheduler words
  const size_t sched_off = ((size_t)E * bpm * sizeof(float) + 255) / 256 * 256;
  const size_t need = sched_off + ((size_t)E + 2) * sizeof(uint32_t);
  if (need > ctx->work_bytes) {
    ANC_CUDA(cudaStreamSynchronize(st));
    ANC_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->d_work) cudaFree(ctx->d_work);
    ctx->d_work = nullptr;
    ctx->work_bytes = 0;
    ANC_CUDA(cudaMalloc(&ctx->d_work, need * 2));
    ctx->work_bytes = need * 2;
  }
  int rc = anc_launch_fro_partial(ctx, X, (float *)ctx->d_work, E, M, N, st);
  if (rc) return rc;
  uint32_t *sched = (uint32_t *)((char *)ctx->d_work + sched_off);
  rc = anc_launch_fro_finalize(ctx, (const float *)ctx->d_work, recip, E, (int)bpm, 0, eps, sched, st);
  if (rc) return rc;
  uint16_t *x = X, *y = Y;
  rc = ns_chain(ctx, x, A, B, y, E, M, N, steps, coeffs, recip, single_launch ? sched : nullptr, st);
  if (rc) return rc;
  if (x != X)   // odd number of steps: result sits in Y, copy it home (muon_ns.py:274-276)
    ANC_CUDA(cudaMemcpyAsync(X, x, (size_t)E * M * N * 2, cudaMemcpyDeviceToDevice, st));
  return ANC_OK;
}

}  // extern "C"
