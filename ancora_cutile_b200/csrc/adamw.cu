// Multi-tensor fused AdamW for sm_100a: one launch sweeps every tensor of the
// arena once (28 B/param with bf16 grads: read g 2 + p 4 + m 4 + v 4, write
// p 4 + m 4 + v 4 + p16 2).
//
// Arithmetic: the operation order of the reference kernel
// (ancora/optim/adamw.py:34-37), every product/sum/quotient/root a separate
// round-to-nearest float32 operation (__fmul_rn/__fadd_rn/__fdiv_rn/__fsqrt_rn are
// never contracted into FMAs), so the fp32 state is bit-identical to a numpy
// float32 evaluation.  The bf16 copy is rounded either to nearest even
// (adamw.py:41) or stochastically: (bits + dither16) >> 16 (bit rule of
// ancora/kernels/fused.py:159-161) with the dither taken from Philox4x32-10 keyed
// by (seed, step, global element index / 8).  One Philox call serves the eight
// elements of one 128-bit bf16 vector, so the stream depends only on the element's
// position in the arena, never on grid, chunking or sharding.
#include <cuda_bf16.h>
#include <vector>
#include "anc_internal.h"
#include "philox.cuh"

namespace {

struct TensorEntry {   // 64 bytes, device resident
  const void *g;
  float *p;
  float *m;
  float *v;
  uint16_t *p16;
  uint64_t numel;
  uint64_t elem_offset;
  float wd;
  uint32_t vec_ok;      // all five pointers 16-byte aligned
};

struct Chunk {          // 16 bytes
  uint64_t start;       // first element inside the tensor (multiple of 8)
  uint32_t tensor;
  uint32_t count;
};

constexpr int kThreads = 256;
constexpr int kChunkElems = 8192;   // 4 passes of 256 threads x 8 elements

struct Scalars {
  float b1, omb1, b2, omb2, eps, lr, ibc1, ibc2;
};

__device__ __forceinline__ void adamw_elem(float g, float &p, float &m, float &v, float wd,
                                           const Scalars &s) {
  const float mn = __fadd_rn(__fmul_rn(s.b1, m), __fmul_rn(s.omb1, g));
  const float vn = __fadd_rn(__fmul_rn(s.b2, v), __fmul_rn(__fmul_rn(s.omb2, g), g));
  const float num = __fmul_rn(mn, s.ibc1);
  const float den = __fadd_rn(__fsqrt_rn(__fmul_rn(vn, s.ibc2)), s.eps);
  const float upd = __fadd_rn(__fdiv_rn(num, den), __fmul_rn(wd, p));
  p = __fsub_rn(p, __fmul_rn(s.lr, upd));
  m = mn;
  v = vn;
}

template <bool kGradF32>
__device__ __forceinline__ void load_grad8(const void *g, uint64_t i, float out[8]) {
  if constexpr (kGradF32) {
    const float4 a = __ldcs(reinterpret_cast<const float4 *>((const float *)g + i));
    const float4 b = __ldcs(reinterpret_cast<const float4 *>((const float *)g + i) + 1);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
    const uint4 r = __ldcs(reinterpret_cast<const uint4 *>((const uint16_t *)g + i));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      out[2 * k] = __uint_as_float(w[k] << 16);
      out[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
    }
  }
}

template <bool kGradF32, bool kSR>
__global__ void __launch_bounds__(kThreads)
adamw_multi_kernel(const TensorEntry *__restrict__ tensors, const Chunk *__restrict__ chunks,
                   uint32_t n_chunks, uint32_t n_tensors, Scalars s, uint32_t seed_lo,
                   uint32_t seed_hi, uint32_t step_lo, uint32_t step_hi, uint32_t *status,
                   const Scalars *__restrict__ sched, const unsigned long long *__restrict__ counter,
                   unsigned long long sched_first, uint32_t sched_len) {
  if (sched) {
    // device-resident schedule: the step number lives in device memory and selects this step's
    // scalars from a table the host filled in advance, so the launch can be replayed from a graph
    const unsigned long long t = *counter;
    const unsigned long long k = t - sched_first;
    if (k >= sched_len) {
      if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, ANC_DEV_BAD_INDEX);
      return;
    }
    s = sched[k];
    step_lo = (uint32_t)t;
    step_hi = (uint32_t)(t >> 32);
  }
  for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
    const Chunk ch = chunks[c];
    if (ch.tensor >= n_tensors) {   // table corruption guard: record and skip
      if (threadIdx.x == 0) atomicOr(status, ANC_DEV_BAD_INDEX);
      continue;
    }
    const TensorEntry t = tensors[ch.tensor];
    const uint32_t groups = ch.count >> 3;           // full 8-element groups
    if (t.vec_ok) {
      for (uint32_t gi = threadIdx.x; gi < groups; gi += kThreads) {
        const uint64_t i = ch.start + (uint64_t)gi * 8;
        float g[8], p[8], m[8], v[8];
        load_grad8<kGradF32>(t.g, i, g);
        const float4 p0 = __ldcs(reinterpret_cast<const float4 *>(t.p + i));
        const float4 p1 = __ldcs(reinterpret_cast<const float4 *>(t.p + i) + 1);
        const float4 m0 = __ldcs(reinterpret_cast<const float4 *>(t.m + i));
        const float4 m1 = __ldcs(reinterpret_cast<const float4 *>(t.m + i) + 1);
        const float4 v0 = __ldcs(reinterpret_cast<const float4 *>(t.v + i));
        const float4 v1 = __ldcs(reinterpret_cast<const float4 *>(t.v + i) + 1);
        p[0] = p0.x; p[1] = p0.y; p[2] = p0.z; p[3] = p0.w; p[4] = p1.x; p[5] = p1.y; p[6] = p1.z; p[7] = p1.w;
        m[0] = m0.x; m[1] = m0.y; m[2] = m0.z; m[3] = m0.w; m[4] = m1.x; m[5] = m1.y; m[6] = m1.z; m[7] = m1.w;
        v[0] = v0.x; v[1] = v0.y; v[2] = v0.z; v[3] = v0.w; v[4] = v1.x; v[5] = v1.y; v[6] = v1.z; v[7] = v1.w;
#pragma unroll
        for (int k = 0; k < 8; ++k) adamw_elem(g[k], p[k], m[k], v[k], t.wd, s);
        uint32_t h[8];
        if constexpr (kSR) {
          const uint64_t blk = (t.elem_offset + i) >> 3;
          uint32_t w[4];
          philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), step_lo, step_hi, seed_lo, seed_hi, w);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            h[2 * k] = bf16_sr(p[2 * k], w[k] & 0xFFFFu);
            h[2 * k + 1] = bf16_sr(p[2 * k + 1], w[k] >> 16);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) h[k] = bf16_rne(p[k]);
        }
        __stcs(reinterpret_cast<float4 *>(t.p + i), make_float4(p[0], p[1], p[2], p[3]));
        __stcs(reinterpret_cast<float4 *>(t.p + i) + 1, make_float4(p[4], p[5], p[6], p[7]));
        __stcs(reinterpret_cast<float4 *>(t.m + i), make_float4(m[0], m[1], m[2], m[3]));
        __stcs(reinterpret_cast<float4 *>(t.m + i) + 1, make_float4(m[4], m[5], m[6], m[7]));
        __stcs(reinterpret_cast<float4 *>(t.v + i), make_float4(v[0], v[1], v[2], v[3]));
        __stcs(reinterpret_cast<float4 *>(t.v + i) + 1, make_float4(v[4], v[5], v[6], v[7]));
        *reinterpret_cast<uint4 *>(t.p16 + i) =
            make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
      }
    }
    // scalar path: the ragged tail of a tensor, or a tensor whose pointers are not
    // 16-byte aligned.  Same arithmetic, same Philox block per 8 elements.
    const uint32_t first = t.vec_ok ? (groups << 3) : 0u;
    for (uint32_t e = first + threadIdx.x; e < ch.count; e += kThreads) {
      const uint64_t i = ch.start + e;
      float g;
      if constexpr (kGradF32) g = ((const float *)t.g)[i];
      else g = __uint_as_float((uint32_t)((const uint16_t *)t.g)[i] << 16);
      float p = t.p[i], m = t.m[i], v = t.v[i];
      adamw_elem(g, p, m, v, t.wd, s);
      uint32_t h;
      if constexpr (kSR) {
        const uint64_t gidx = t.elem_offset + i;
        const uint64_t blk = gidx >> 3;
        const uint32_t lane = (uint32_t)(gidx & 7);
        uint32_t w[4];
        philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), step_lo, step_hi, seed_lo, seed_hi, w);
        const uint32_t word = w[lane >> 1];
        h = bf16_sr(p, (lane & 1) ? (word >> 16) : (word & 0xFFFFu));
      } else {
        h = bf16_rne(p);
      }
      t.p[i] = p; t.m[i] = m; t.v[i] = v;
      t.p16[i] = (uint16_t)h;
    }
  }
}

__global__ void adamw_advance_kernel(unsigned long long *counter) { *counter += 1ull; }

}  // namespace

struct anc_adamw_plan {
  anc_ctx *ctx;
  int grad_dtype;
  std::vector<TensorEntry> tensors;
  uint64_t arena_elems;     // max(elem_offset + numel)
  uint64_t owned_elems;
  TensorEntry *d_tensors;
  Chunk *d_chunks;
  uint32_t n_chunks;
  uint32_t chunk_capacity;
  Scalars *d_sched = nullptr;              // optional device-resident schedule
  unsigned long long *d_counter = nullptr;
  unsigned long long sched_first = 0;
  uint32_t sched_len = 0;
};

static int adamw_build_chunks(anc_adamw_plan *pl, uint64_t begin, uint64_t end) {
  std::vector<Chunk> chunks;
  uint64_t owned = 0;
  for (uint32_t ti = 0; ti < pl->tensors.size(); ++ti) {
    const TensorEntry &t = pl->tensors[ti];
    const uint64_t lo = t.elem_offset > begin ? t.elem_offset : begin;
    const uint64_t hi = (t.elem_offset + t.numel) < end ? (t.elem_offset + t.numel) : end;
    if (lo >= hi) continue;
    owned += hi - lo;
    for (uint64_t s = lo; s < hi; s += kChunkElems) {
      Chunk c;
      c.start = s - t.elem_offset;
      c.tensor = ti;
      c.count = (uint32_t)((hi - s) < (uint64_t)kChunkElems ? (hi - s) : (uint64_t)kChunkElems);
      chunks.push_back(c);
    }
  }
  if (chunks.size() > pl->chunk_capacity) {
    if (pl->d_chunks) cudaFree(pl->d_chunks);
    pl->d_chunks = nullptr;
    pl->chunk_capacity = (uint32_t)chunks.size();
    ANC_CUDA(cudaMalloc((void **)&pl->d_chunks, sizeof(Chunk) * chunks.size()));
  }
  if (!chunks.empty())
    ANC_CUDA(cudaMemcpy(pl->d_chunks, chunks.data(), sizeof(Chunk) * chunks.size(),
                        cudaMemcpyHostToDevice));
  pl->n_chunks = (uint32_t)chunks.size();
  pl->owned_elems = owned;
  return ANC_OK;
}

extern "C" {

int anc_adamw_plan_create(anc_ctx *ctx, const anc_adamw_tensor *tensors, int n_tensors,
                          int grad_dtype, anc_adamw_plan **out) {
  ANC_REQUIRE(ctx && out && (tensors || n_tensors == 0), "NULL argument");
  ANC_REQUIRE(n_tensors >= 0, "n_tensors < 0");
  ANC_REQUIRE(grad_dtype == ANC_GRAD_BF16 || grad_dtype == ANC_GRAD_F32, "bad grad_dtype %d",
              grad_dtype);
  *out = nullptr;
  anc_device_guard guard(ctx->device);
  anc_adamw_plan *pl = new anc_adamw_plan();
  pl->ctx = ctx;
  pl->grad_dtype = grad_dtype;
  pl->arena_elems = 0;
  pl->d_tensors = nullptr;
  pl->d_chunks = nullptr;
  pl->n_chunks = 0;
  pl->chunk_capacity = 0;
  for (int i = 0; i < n_tensors; ++i) {
    const anc_adamw_tensor &a = tensors[i];
    if (!a.g || !a.p32 || !a.m || !a.v || !a.p16) {
      anc_set_error("tensor %d has a NULL pointer", i);
      delete pl;
      return ANC_E_INVALID;
    }
    if (a.elem_offset % 8 != 0) {
      anc_set_error("tensor %d: elem_offset %llu is not a multiple of 8", i,
                    (unsigned long long)a.elem_offset);
      delete pl;
      return ANC_E_INVALID;
    }
    TensorEntry t;
    t.g = a.g; t.p = a.p32; t.m = a.m; t.v = a.v; t.p16 = a.p16;
    t.numel = a.numel; t.elem_offset = a.elem_offset; t.wd = a.wd;
    const uintptr_t bits = (uintptr_t)a.g | (uintptr_t)a.p32 | (uintptr_t)a.m | (uintptr_t)a.v |
                           (uintptr_t)a.p16;
    t.vec_ok = (bits & 15) == 0 ? 1u : 0u;
    pl->tensors.push_back(t);
    if (a.elem_offset + a.numel > pl->arena_elems) pl->arena_elems = a.elem_offset + a.numel;
  }
  if (n_tensors > 0) {
    cudaError_t e = cudaMalloc((void **)&pl->d_tensors, sizeof(TensorEntry) * n_tensors);
    if (e == cudaSuccess)
      e = cudaMemcpy(pl->d_tensors, pl->tensors.data(), sizeof(TensorEntry) * n_tensors,
                     cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      delete pl;
      return anc_cuda_fail(e, "adamw tensor table");
    }
  }
  int rc = adamw_build_chunks(pl, 0, UINT64_MAX);
  if (rc != ANC_OK) {
    anc_adamw_plan_destroy(pl);
    return rc;
  }
  *out = pl;
  return ANC_OK;
}

int anc_adamw_plan_set_range(anc_adamw_plan *plan, uint64_t begin, uint64_t end) {
  ANC_REQUIRE(plan, "plan is NULL");
  ANC_REQUIRE(begin % 8 == 0 && (end % 8 == 0 || end == UINT64_MAX) && begin <= end,
              "slice [%llu,%llu) must be 8-aligned", (unsigned long long)begin,
              (unsigned long long)end);
  anc_device_guard guard(plan->ctx->device);
  ANC_CUDA(cudaStreamSynchronize(plan->ctx->stream));
  return adamw_build_chunks(plan, begin, end);
}

int anc_adamw_plan_total(anc_adamw_plan *plan, uint64_t *arena_elems, uint64_t *owned_elems) {
  ANC_REQUIRE(plan, "plan is NULL");
  if (arena_elems) *arena_elems = plan->arena_elems;
  if (owned_elems) *owned_elems = plan->owned_elems;
  return ANC_OK;
}

int anc_adamw_step(anc_adamw_plan *plan, const anc_adamw_scalars *sc, int rounding, uint64_t seed,
                   uint64_t step, void *stream) {
  ANC_REQUIRE(plan && sc, "NULL argument");
  ANC_REQUIRE(rounding == ANC_ROUND_RNE || rounding == ANC_ROUND_SR, "bad rounding %d", rounding);
  if (plan->n_chunks == 0) return ANC_OK;
  anc_ctx *ctx = plan->ctx;
  anc_device_guard guard(ctx->device);
  cudaStream_t st = anc_pick_stream(ctx, stream);
  Scalars s = {sc->beta1, sc->one_minus_beta1, sc->beta2, sc->one_minus_beta2,
               sc->eps,   sc->lr,              sc->ibc1,  sc->ibc2};
  uint32_t grid = plan->n_chunks;
  const uint32_t cap = (uint32_t)ctx->sm_count * 16u;
  if (grid > cap) grid = cap;
  const uint32_t nt = (uint32_t)plan->tensors.size();
  const uint32_t sl = (uint32_t)seed, sh = (uint32_t)(seed >> 32);
  const uint32_t tl = (uint32_t)step, th = (uint32_t)(step >> 32);
#define ANC_ADAMW_LAUNCH(F32, SR)                                                              \
  adamw_multi_kernel<F32, SR><<<grid, kThreads, 0, st>>>(plan->d_tensors, plan->d_chunks,      \
                                                         plan->n_chunks, nt, s, sl, sh, tl, th, \
                                                         ctx->d_status, nullptr, nullptr, 0ull, 0u)
  const bool f32 = plan->grad_dtype == ANC_GRAD_F32;
  const bool sr = rounding == ANC_ROUND_SR;
  if (f32 && sr) ANC_ADAMW_LAUNCH(true, true);
  else if (f32) ANC_ADAMW_LAUNCH(true, false);
  else if (sr) ANC_ADAMW_LAUNCH(false, true);
  else ANC_ADAMW_LAUNCH(false, false);
#undef ANC_ADAMW_LAUNCH
  ANC_CUDA(cudaGetLastError());
  return ANC_OK;
}

int anc_adamw_plan_set_schedule(anc_adamw_plan *plan, const anc_adamw_scalars *table, int n,
                                uint64_t first_step) {
  ANC_REQUIRE(plan && table && n > 0, "bad argument");
  anc_device_guard guard(plan->ctx->device);
  ANC_CUDA(cudaStreamSynchronize(plan->ctx->stream));
  if (plan->d_sched) cudaFree(plan->d_sched);
  plan->d_sched = nullptr;
  static_assert(sizeof(Scalars) == sizeof(anc_adamw_scalars), "scalar layout");
  ANC_CUDA(cudaMalloc((void **)&plan->d_sched, sizeof(Scalars) * (size_t)n));
  ANC_CUDA(cudaMemcpy(plan->d_sched, table, sizeof(Scalars) * (size_t)n, cudaMemcpyHostToDevice));
  if (!plan->d_counter) ANC_CUDA(cudaMalloc((void **)&plan->d_counter, sizeof(unsigned long long)));
  unsigned long long t0 = first_step;
  ANC_CUDA(cudaMemcpy(plan->d_counter, &t0, sizeof(t0), cudaMemcpyHostToDevice));
  plan->sched_first = first_step;
  plan->sched_len = (uint32_t)n;
  return ANC_OK;
}

int anc_adamw_plan_set_counter(anc_adamw_plan *plan, uint64_t step, void *stream) {
  ANC_REQUIRE(plan, "plan is NULL");
  ANC_REQUIRE(plan->d_sched && plan->d_counter, "no schedule: call anc_adamw_plan_set_schedule first");
  ANC_REQUIRE(step >= plan->sched_first && step < plan->sched_first + plan->sched_len,
              "step %llu is outside the uploaded schedule [%llu, %llu)", (unsigned long long)step,
              (unsigned long long)plan->sched_first, (unsigned long long)(plan->sched_first + plan->sched_len));
  anc_device_guard guard(plan->ctx->device);
  cudaStream_t st = anc_pick_stream(plan->ctx, stream);
  ANC_CUDA(cudaStreamSynchronize(st));      // no launch that reads the counter is still in flight
  unsigned long long t0 = step;
  ANC_CUDA(cudaMemcpy(plan->d_counter, &t0, sizeof(t0), cudaMemcpyHostToDevice));
  return ANC_OK;
}

int anc_adamw_step_scheduled(anc_adamw_plan *plan, int rounding, uint64_t seed, int advance,
                             void *stream) {
  ANC_REQUIRE(plan, "plan is NULL");
  ANC_REQUIRE(plan->d_sched && plan->d_counter, "no schedule: call anc_adamw_plan_set_schedule first");
  ANC_REQUIRE(rounding == ANC_ROUND_RNE || rounding == ANC_ROUND_SR, "bad rounding %d", rounding);
  anc_ctx *ctx = plan->ctx;
  anc_device_guard guard(ctx->device);
  cudaStream_t st = anc_pick_stream(ctx, stream);
  if (plan->n_chunks) {
    Scalars s = {};
    uint32_t grid = plan->n_chunks;
    const uint32_t cap = (uint32_t)ctx->sm_count * 16u;
    if (grid > cap) grid = cap;
    const uint32_t nt = (uint32_t)plan->tensors.size();
    const uint32_t sl = (uint32_t)seed, sh = (uint32_t)(seed >> 32);
#define ANC_ADAMW_LAUNCH_S(F32, SR)                                                                 \
  adamw_multi_kernel<F32, SR><<<grid, kThreads, 0, st>>>(                                           \
      plan->d_tensors, plan->d_chunks, plan->n_chunks, nt, s, sl, sh, 0u, 0u, ctx->d_status,        \
      plan->d_sched, plan->d_counter, plan->sched_first, plan->sched_len)
    const bool f32 = plan->grad_dtype == ANC_GRAD_F32;
    const bool sr = rounding == ANC_ROUND_SR;
    if (f32 && sr) ANC_ADAMW_LAUNCH_S(true, true);
    else if (f32) ANC_ADAMW_LAUNCH_S(true, false);
    else if (sr) ANC_ADAMW_LAUNCH_S(false, true);
    else ANC_ADAMW_LAUNCH_S(false, false);
#undef ANC_ADAMW_LAUNCH_S
    ANC_CUDA(cudaGetLastError());
  }
  if (advance) {
    adamw_advance_kernel<<<1, 1, 0, st>>>(plan->d_counter);
    ANC_CUDA(cudaGetLastError());
  }
  return ANC_OK;
}

int anc_adamw_plan_destroy(anc_adamw_plan *plan) {
  if (!plan) return ANC_OK;
  anc_device_guard guard(plan->ctx->device);
  cudaStreamSynchronize(plan->ctx->stream);
  if (plan->d_sched) cudaFree(plan->d_sched);
  if (plan->d_counter) cudaFree(plan->d_counter);
  if (plan->d_tensors) cudaFree(plan->d_tensors);
  if (plan->d_chunks) cudaFree(plan->d_chunks);
  delete plan;
  return ANC_OK;
}

}  // extern "C"
