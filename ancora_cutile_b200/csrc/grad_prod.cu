// Gradient producer for the optimizer step: accumulate one more contribution into the float32
// gradient accumulator and, in the same sweep, emit the bf16 gradient the step reads.
//
//   acc[i]  = src[i] + acc[i]                      one float32 add per element
//                                                  (ancora/kernels/fused.py:242-249 `_acc_f32`)
//   g16[i]  = bf16(acc[i] * scale)                 nearest-even, or stochastic with the bit rule
//                                                  (bits + dither16) >> 16 of fused.py:159-161
//   acc[i]  = 0 afterwards when asked (the accumulator is ready for the next step)
//
// The reference runs the accumulation and the downcast as separate sweeps (12 + 6 B/elem with
// float32 contributions); fused it is 14 B/elem (read src 4 + acc 4, write acc 4 + g16 2), or
// 12 with bf16 contributions.  HBM-bound: 8 elements per thread per pass, 128-bit accesses.
// The dither is 16 bits of Philox4x32-10 keyed by (seed, step, global element index / 8), the
// layout the AdamW kernel uses, so the bits depend only on the element's global position.
#include "anc_internal.h"
#include "philox.cuh"

namespace {

constexpr int kThreads = 256;

struct GradArgs {
  float *acc;
  const void *src;      // nullptr: no accumulation, downcast only
  uint16_t *g16;        // nullptr: accumulate only
  uint64_t numel;
  uint64_t elem_offset; // global index of element 0 (multiple of 8 on the vector path)
  float scale;
  uint32_t seed_lo, seed_hi, step_lo, step_hi;
  int zero_after;
};

template <bool kSrcF32>
__device__ __forceinline__ float load_src(const void *src, uint64_t i) {
  if constexpr (kSrcF32) return ((const float *)src)[i];
  else return __uint_as_float((uint32_t)((const uint16_t *)src)[i] << 16);
}

template <bool kSrcF32, bool kSR>
__global__ void __launch_bounds__(kThreads)
grad_accumulate_kernel(GradArgs a, int vec_ok) {
  const uint64_t groups = vec_ok ? (a.numel >> 3) : 0ull;
  const uint64_t stride = (uint64_t)gridDim.x * kThreads;
  for (uint64_t gi = (uint64_t)blockIdx.x * kThreads + threadIdx.x; gi < groups; gi += stride) {
    const uint64_t i = gi << 3;
    const float4 a0 = __ldcs(reinterpret_cast<const float4 *>(a.acc + i));
    const float4 a1 = __ldcs(reinterpret_cast<const float4 *>(a.acc + i) + 1);
    float v[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    if (a.src) {
      float s[8];
      if constexpr (kSrcF32) {
        const float4 s0 = __ldcs(reinterpret_cast<const float4 *>((const float *)a.src + i));
        const float4 s1 = __ldcs(reinterpret_cast<const float4 *>((const float *)a.src + i) + 1);
        s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w;
        s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
      } else {
        const uint4 r = __ldcs(reinterpret_cast<const uint4 *>((const uint16_t *)a.src + i));
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          s[2 * k] = __uint_as_float(w[k] << 16);
          s[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
        }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = __fadd_rn(s[k], v[k]);
    }
    if (a.g16) {
      uint32_t h[8];
      if constexpr (kSR) {
        const uint64_t blk = (a.elem_offset + i) >> 3;
        uint32_t w[4];
        philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), a.step_lo, a.step_hi, a.seed_lo, a.seed_hi, w);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          h[2 * k] = bf16_sr(__fmul_rn(v[2 * k], a.scale), w[k] & 0xFFFFu);
          h[2 * k + 1] = bf16_sr(__fmul_rn(v[2 * k + 1], a.scale), w[k] >> 16);
        }
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) h[k] = bf16_rne(__fmul_rn(v[k], a.scale));
      }
      *reinterpret_cast<uint4 *>(a.g16 + i) =
          make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
    }
    if (a.zero_after) {
      __stcs(reinterpret_cast<float4 *>(a.acc + i), make_float4(0.f, 0.f, 0.f, 0.f));
      __stcs(reinterpret_cast<float4 *>(a.acc + i) + 1, make_float4(0.f, 0.f, 0.f, 0.f));
    } else if (a.src) {
      __stcs(reinterpret_cast<float4 *>(a.acc + i), make_float4(v[0], v[1], v[2], v[3]));
      __stcs(reinterpret_cast<float4 *>(a.acc + i) + 1, make_float4(v[4], v[5], v[6], v[7]));
    }
  }
  // scalar path: the ragged tail, or everything when a pointer or the offset is unaligned.
  // Same arithmetic, same Philox block per 8 global elements.
  for (uint64_t i = (groups << 3) + (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < a.numel; i += stride) {
    float v = a.acc[i];
    if (a.src) v = __fadd_rn(load_src<kSrcF32>(a.src, i), v);
    if (a.g16) {
      const float x = __fmul_rn(v, a.scale);
      uint32_t h;
      if constexpr (kSR) {
        const uint64_t gidx = a.elem_offset + i;
        const uint64_t blk = gidx >> 3;
        const uint32_t lane = (uint32_t)(gidx & 7);
        uint32_t w[4];
        philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), a.step_lo, a.step_hi, a.seed_lo, a.seed_hi, w);
        const uint32_t word = w[lane >> 1];
        h = bf16_sr(x, (lane & 1) ? (word >> 16) : (word & 0xFFFFu));
      } else {
        h = bf16_rne(x);
      }
      a.g16[i] = (uint16_t)h;
    }
    if (a.zero_after) a.acc[i] = 0.f;
    else if (a.src) a.acc[i] = v;
  }
}

}  // namespace

extern "C" int anc_grad_accumulate(anc_ctx *ctx, float *acc, const void *src, int src_dtype, uint16_t *g16,
                                   uint64_t numel, uint64_t elem_offset, float scale, int round_mode,
                                   uint64_t seed, uint64_t step, int zero_after, void *stream) {
  ANC_REQUIRE(ctx && acc, "NULL argument");
  ANC_REQUIRE(src || g16, "neither a contribution nor a bf16 output was given");
  ANC_REQUIRE(src_dtype == ANC_GRAD_BF16 || src_dtype == ANC_GRAD_F32, "bad src_dtype %d", src_dtype);
  ANC_REQUIRE(round_mode == ANC_ROUND_RNE || round_mode == ANC_ROUND_SR, "bad round_mode %d", round_mode);
  ANC_REQUIRE(((uintptr_t)acc & 3) == 0 && ((uintptr_t)g16 & 1) == 0 &&
                  ((uintptr_t)src & (src_dtype == ANC_GRAD_F32 ? 3 : 1)) == 0,
              "pointer not aligned to its element size");
  if (numel == 0) return ANC_OK;
  anc_device_guard guard(ctx->device);
  cudaStream_t st = stream ? (cudaStream_t)stream : ctx->stream;
  GradArgs a;
  a.acc = acc; a.src = src; a.g16 = g16; a.numel = numel; a.elem_offset = elem_offset; a.scale = scale;
  a.seed_lo = (uint32_t)seed; a.seed_hi = (uint32_t)(seed >> 32);
  a.step_lo = (uint32_t)step; a.step_hi = (uint32_t)(step >> 32);
  a.zero_after = zero_after ? 1 : 0;
  const uintptr_t bits = (uintptr_t)acc | (uintptr_t)src | (uintptr_t)g16;
  const int vec_ok = ((bits & 15) == 0 && (elem_offset & 7) == 0) ? 1 : 0;
  const uint64_t work = vec_ok ? ((numel + 7) >> 3) : numel;
  uint64_t blocks = (work + kThreads - 1) / kThreads;
  const uint64_t cap = (uint64_t)ctx->sm_count * 16;       // 8 resident blocks per SM, two waves
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const dim3 grid((unsigned)blocks), block(kThreads);
  const bool f32 = src_dtype == ANC_GRAD_F32, sr = round_mode == ANC_ROUND_SR;
  if (f32 && sr) grad_accumulate_kernel<true, true><<<grid, block, 0, st>>>(a, vec_ok);
  else if (f32) grad_accumulate_kernel<true, false><<<grid, block, 0, st>>>(a, vec_ok);
  else if (sr) grad_accumulate_kernel<false, true><<<grid, block, 0, st>>>(a, vec_ok);
  else grad_accumulate_kernel<false, false><<<grid, block, 0, st>>>(a, vec_ok);
  ANC_CUDA(cudaGetLastError());
  return ANC_OK;
}
