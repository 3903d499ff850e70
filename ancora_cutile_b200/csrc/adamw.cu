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
#include "stream_ring.cuh"

namespace {

struct TensorEntry {   // host side only
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

// One stage of work: at most kChunkElems consecutive elements of one tensor.  Self-contained
// (the pointers are those of the chunk's first element) so that the thread that feeds the
// ring needs one table read per stage, issued a stage ahead.
struct Chunk {          // 64 bytes, device resident
  const void *g;
  float *p;
  float *m;
  float *v;
  uint16_t *p16;
  uint64_t gidx;        // arena index of the first element (a multiple of 8): the Philox position
  uint32_t count;
  float wd;
  uint32_t aligned;     // the five addresses are 16-byte aligned
  uint32_t bulk;        // aligned and count a multiple of 8: the stage is filled by bulk copies
};
static_assert(sizeof(Chunk) == 64, "chunk record");

constexpr int kThreads = 256;       // computing threads of one group
constexpr int kGroups = 1;          // groups of computing threads taking the stages in turn (two groups: 96
                                    // registers per thread, spills, 0.91 instead of 0.73 ms on the full arena)
constexpr int kBlock = kGroups * kThreads + 32;   // one more warp feeds the ring
constexpr int kChunkElems = 2048;   // 256 threads x 8 elements
constexpr int kHdrBytes = 128;      // the chunk record travels with its stage

template <bool kGradF32>
struct Ring {
  static constexpr int kStages = kGradF32 ? 6 : 7;
  static constexpr uint32_t kGradBytes = kGradF32 ? 4u : 2u;
  static constexpr uint32_t kStageBytes = kHdrBytes + kChunkElems * (12u + kGradBytes);
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes;   // 201,600 / 197,376 bytes
};

struct Scalars {
  float b1, omb1, b2, omb2, eps, lr, ibc1, ibc2;
};

__device__ __forceinline__ void adamw_elem(float g, float &p, float &m, float &v, float wd,
                                           const Scalars &s) {
  const float mn = __fadd_rn(__fmul_rn(s.b1, m), __fmul_rn(s.omb1, g));
  const float vn = __fadd_rn(__fmul_rn(s.b2, v), __fmul_rn(__fmul_rn(s.omb2, g), g));
  const float num = __fmul_rn(mn, s.ibc1);
  // Rows of an embedding that no token of the step touched have g = m = v = 0 for ever.  The correctly
  // rounded square root and division leave their fast paths on zero operands (a subroutine per element,
  // which the few computing warps of this kernel cannot hide: the sweep ran 2.3 times slower on an arena
  // of zeros), so zeros go through as 1 and the exact result is put back: sqrt(+-0) = +-0, and
  // (+-0) / den = (+-0) * (1 / den), NaN and infinity in den included.
  const float x = __fmul_rn(vn, s.ibc2);
  const float rt0 = __fsqrt_rn(x == 0.f ? 1.f : x);
  const float den = __fadd_rn(x == 0.f ? x : rt0, s.eps);
  const float q0 = __fdiv_rn(num == 0.f ? 1.f : num, den);
  const float upd = __fadd_rn(num == 0.f ? __fmul_rn(num, q0) : q0, __fmul_rn(wd, p));
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

// The update of one 8-element group held in registers and its stores (i = offset inside the chunk).
template <bool kSR>
__device__ __forceinline__ void finish8(const Chunk &ch, uint32_t i, float g[8], float p[8], float m[8],
                                        float v[8], const Scalars &s, uint32_t seed_lo, uint32_t seed_hi,
                                        uint32_t step_lo, uint32_t step_hi) {
#pragma unroll
  for (int k = 0; k < 8; ++k) adamw_elem(g[k], p[k], m[k], v[k], ch.wd, s);
  uint32_t h[8];
  if constexpr (kSR) {
    const uint64_t blk = (ch.gidx + i) >> 3;
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
  __stcs(reinterpret_cast<float4 *>(ch.p + i), make_float4(p[0], p[1], p[2], p[3]));
  __stcs(reinterpret_cast<float4 *>(ch.p + i) + 1, make_float4(p[4], p[5], p[6], p[7]));
  __stcs(reinterpret_cast<float4 *>(ch.m + i), make_float4(m[0], m[1], m[2], m[3]));
  __stcs(reinterpret_cast<float4 *>(ch.m + i) + 1, make_float4(m[4], m[5], m[6], m[7]));
  __stcs(reinterpret_cast<float4 *>(ch.v + i), make_float4(v[0], v[1], v[2], v[3]));
  __stcs(reinterpret_cast<float4 *>(ch.v + i) + 1, make_float4(v[4], v[5], v[6], v[7]));
  *reinterpret_cast<uint4 *>(ch.p16 + i) =
      make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
}

// A chunk the bulk copies cannot serve (a tensor whose pointers are not 16-byte aligned, or the
// ragged last chunk of a tensor): plain loads, 128-bit where the alignment allows, then
// element by element.  Same arithmetic, same Philox block per 8 elements.
template <bool kGradF32, bool kSR>
__device__ __forceinline__ void direct_chunk(const Chunk &ch, int tid, const Scalars &s, uint32_t seed_lo,
                                             uint32_t seed_hi, uint32_t step_lo, uint32_t step_hi) {
  const uint32_t groups = ch.aligned ? (ch.count >> 3) : 0u;
  for (uint32_t gi = tid; gi < groups; gi += kThreads) {
    const uint32_t i = gi * 8;
    float g[8], p[8], m[8], v[8];
    load_grad8<kGradF32>(ch.g, i, g);
    const float4 p0 = __ldcs(reinterpret_cast<const float4 *>(ch.p + i));
    const float4 p1 = __ldcs(reinterpret_cast<const float4 *>(ch.p + i) + 1);
    const float4 m0 = __ldcs(reinterpret_cast<const float4 *>(ch.m + i));
    const float4 m1 = __ldcs(reinterpret_cast<const float4 *>(ch.m + i) + 1);
    const float4 v0 = __ldcs(reinterpret_cast<const float4 *>(ch.v + i));
    const float4 v1 = __ldcs(reinterpret_cast<const float4 *>(ch.v + i) + 1);
    p[0] = p0.x; p[1] = p0.y; p[2] = p0.z; p[3] = p0.w; p[4] = p1.x; p[5] = p1.y; p[6] = p1.z; p[7] = p1.w;
    m[0] = m0.x; m[1] = m0.y; m[2] = m0.z; m[3] = m0.w; m[4] = m1.x; m[5] = m1.y; m[6] = m1.z; m[7] = m1.w;
    v[0] = v0.x; v[1] = v0.y; v[2] = v0.z; v[3] = v0.w; v[4] = v1.x; v[5] = v1.y; v[6] = v1.z; v[7] = v1.w;
    finish8<kSR>(ch, i, g, p, m, v, s, seed_lo, seed_hi, step_lo, step_hi);
  }
  for (uint32_t i = (groups << 3) + tid; i < ch.count; i += kThreads) {
    float g;
    if constexpr (kGradF32) g = ((const float *)ch.g)[i];
    else g = __uint_as_float((uint32_t)((const uint16_t *)ch.g)[i] << 16);
    float p = ch.p[i], m = ch.m[i], v = ch.v[i];
    adamw_elem(g, p, m, v, ch.wd, s);
    uint32_t h;
    if constexpr (kSR) {
      const uint64_t gidx = ch.gidx + i;
      const uint64_t blk = gidx >> 3;
      const uint32_t ln = (uint32_t)(gidx & 7);
      uint32_t w[4];
      philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), step_lo, step_hi, seed_lo, seed_hi, w);
      const uint32_t word = w[ln >> 1];
      h = bf16_sr(p, (ln & 1) ? (word >> 16) : (word & 0xFFFFu));
    } else {
      h = bf16_rne(p);
    }
    ch.p[i] = p; ch.m[i] = m; ch.v[i] = v;
    ch.p16[i] = (uint16_t)h;
  }
}

// One CTA per SM.  The last warp's first lane walks this CTA's chunks (blockIdx.x, + gridDim.x, ...),
// copies each chunk's record into the stage's header and starts the four bulk copies (p, m, v,
// g) that fill it; the eight computing warps wait for the
// stage, take eight elements per thread from shared memory, hand the stage back and update + store
// from registers.
template <bool kGradF32, bool kSR>
__global__ void __launch_bounds__(kBlock, 1)
adamw_multi_kernel(const Chunk *__restrict__ chunks, uint32_t n_chunks, Scalars s, uint32_t seed_lo,
                   uint32_t seed_hi, uint32_t step_lo, uint32_t step_hi, uint32_t *status,
                   const Scalars *__restrict__ sched, const unsigned long long *__restrict__ counter,
                   unsigned long long sched_first, uint32_t sched_len) {
  using R = Ring<kGradF32>;
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t bars[2 * R::kStages];
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
  const uint32_t full0 = anc_ring::smem_u32(&bars[0]), empty0 = anc_ring::smem_u32(&bars[R::kStages]);
  if (threadIdx.x == 0) {
    for (int i = 0; i < R::kStages; ++i) {
      anc_ring::mbar_init(full0 + 8 * i, 1);
      anc_ring::mbar_init(empty0 + 8 * i, kThreads / 32);
    }
    anc_ring::mbar_init_fence();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == kGroups * kThreads / 32) {
    if (lane != 0) return;
    uint32_t it = 0;
    uint32_t c = blockIdx.x;
    Chunk nxt = chunks[c];                      // the grid never exceeds n_chunks
    for (; c < n_chunks; c += gridDim.x, ++it) {
      const Chunk ch = nxt;
      if (c + gridDim.x < n_chunks) nxt = chunks[c + gridDim.x];
      const uint32_t slot = it % R::kStages, ph = (it / R::kStages) & 1u;
      if (it >= (uint32_t)R::kStages && !anc_ring::mbar_wait(empty0 + 8 * slot, ph ^ 1u)) {
        atomicOr(status, ANC_DEV_TIMEOUT_TMA);
        anc_ring::drain_issued<R::kStages>(full0, it);
        return;
      }
      uint8_t *st = ring + (size_t)slot * R::kStageBytes;
      *reinterpret_cast<Chunk *>(st) = ch;
      if (ch.bulk) {
        const uint32_t dst = anc_ring::smem_u32(st + kHdrBytes);
        anc_ring::mbar_expect_tx(full0 + 8 * slot, ch.count * (12u + R::kGradBytes));
        anc_ring::bulk_load(dst, ch.p, ch.count * 4u, full0 + 8 * slot);
        anc_ring::bulk_load(dst + kChunkElems * 4u, ch.m, ch.count * 4u, full0 + 8 * slot);
        anc_ring::bulk_load(dst + kChunkElems * 8u, ch.v, ch.count * 4u, full0 + 8 * slot);
        anc_ring::bulk_load(dst + kChunkElems * 12u, ch.g, ch.count * R::kGradBytes, full0 + 8 * slot);
      } else {
        anc_ring::mbar_arrive(full0 + 8 * slot);
      }
    }
    return;
  }
  const uint32_t grp = (uint32_t)warp / (kThreads / 32);
  const int tid = threadIdx.x & (kThreads - 1);          // thread within its group
  uint32_t it = grp;
  for (uint32_t c = blockIdx.x + grp * gridDim.x; c < n_chunks; c += kGroups * gridDim.x, it += kGroups) {
    const uint32_t slot = it % R::kStages, ph = (it / R::kStages) & 1u;
    if (!anc_ring::mbar_wait(full0 + 8 * slot, ph)) {
      if (lane == 0) atomicOr(status, ANC_DEV_TIMEOUT_TMA);
      return;
    }
    const uint8_t *st = ring + (size_t)slot * R::kStageBytes;
    const Chunk ch = *reinterpret_cast<const Chunk *>(st);
    if (ch.bulk) {
      const int t = tid;
      const bool act = (uint32_t)t * 8u < ch.count;
      float g[8], p[8], m[8], v[8];
      if (act) {
        const float *sp = reinterpret_cast<const float *>(st + kHdrBytes);
        anc_ring::ld8(sp, t, lane, p);
        anc_ring::ld8(sp + kChunkElems, t, lane, m);
        anc_ring::ld8(sp + 2 * kChunkElems, t, lane, v);
        if constexpr (kGradF32) anc_ring::ld8(sp + 3 * kChunkElems, t, lane, g);
        else anc_ring::ld8_bf16(reinterpret_cast<const uint16_t *>(sp + 3 * kChunkElems), t, g);
      }
      __syncwarp();
      if (lane == 0) anc_ring::mbar_arrive(empty0 + 8 * slot);
      if (act) finish8<kSR>(ch, (uint32_t)t * 8u, g, p, m, v, s, seed_lo, seed_hi, step_lo, step_hi);
    } else {
      __syncwarp();
      if (lane == 0) anc_ring::mbar_arrive(empty0 + 8 * slot);
      direct_chunk<kGradF32, kSR>(ch, tid, s, seed_lo, seed_hi, step_lo, step_hi);
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
    const uint32_t gb = pl->grad_dtype == ANC_GRAD_F32 ? 4u : 2u;
    for (uint64_t s = lo; s < hi; s += kChunkElems) {
      const uint64_t first = s - t.elem_offset;       // inside the tensor, a multiple of 8
      Chunk c;
      c.g = (const uint8_t *)t.g + first * gb;
      c.p = t.p + first;
      c.m = t.m + first;
      c.v = t.v + first;
      c.p16 = t.p16 + first;
      c.gidx = s;
      c.count = (uint32_t)((hi - s) < (uint64_t)kChunkElems ? (hi - s) : (uint64_t)kChunkElems);
      c.wd = t.wd;
      c.aligned = t.vec_ok;
      c.bulk = (t.vec_ok && c.count % 8 == 0) ? 1u : 0u;
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
  {
    // the ring's shared memory is above the default per-launch limit
    cudaError_t e = cudaSuccess;
#define ANC_ADAMW_SMEM(F32, SR)                                                                      \
  if (e == cudaSuccess)                                                                              \
    e = cudaFuncSetAttribute(adamw_multi_kernel<F32, SR>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                             (int)Ring<F32>::kSmemBytes)
    ANC_ADAMW_SMEM(true, true);
    ANC_ADAMW_SMEM(true, false);
    ANC_ADAMW_SMEM(false, true);
    ANC_ADAMW_SMEM(false, false);
#undef ANC_ADAMW_SMEM
    if (e != cudaSuccess) {
      delete pl;
      return anc_cuda_fail(e, "adamw kernel attributes");
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
  uint32_t grid = plan->n_chunks;                   // one persistent CTA per SM
  if (grid > (uint32_t)ctx->sm_count) grid = (uint32_t)ctx->sm_count;
  const uint32_t sl = (uint32_t)seed, sh = (uint32_t)(seed >> 32);
  const uint32_t tl = (uint32_t)step, th = (uint32_t)(step >> 32);
#define ANC_ADAMW_LAUNCH(F32, SR)                                                                  \
  adamw_multi_kernel<F32, SR><<<grid, kBlock, Ring<F32>::kSmemBytes, st>>>(                 \
      plan->d_chunks, plan->n_chunks, s, sl, sh, tl, th, ctx->d_status, nullptr, nullptr, 0ull, 0u)
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
    if (grid > (uint32_t)ctx->sm_count) grid = (uint32_t)ctx->sm_count;
    const uint32_t sl = (uint32_t)seed, sh = (uint32_t)(seed >> 32);
#define ANC_ADAMW_LAUNCH_S(F32, SR)                                                                 \
  adamw_multi_kernel<F32, SR><<<grid, kBlock, Ring<F32>::kSmemBytes, st>>>(                  \
      plan->d_chunks, plan->n_chunks, s, sl, sh, 0u, 0u, ctx->d_status, plan->d_sched,              \
      plan->d_counter, plan->sched_first, plan->sched_len)
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
  if (plan->d_chunks) cudaFree(plan->d_chunks);
  delete plan;
  return ANC_OK;
}

}  // extern "C"
