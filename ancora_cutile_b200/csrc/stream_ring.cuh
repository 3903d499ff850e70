// Shared-memory staging ring of the HBM-bound sweeps (AdamW, Muon momentum / update): one
// thread issues untiled bulk copies (cp.async.bulk, the 1-D form of TMA) several stages ahead,
// their bytes complete an mbarrier per stage, the other warps wait on it, compute from shared
// memory and store their results straight from registers.  The bytes in flight per SM are then
// the ring's size (about 200 KB) instead of what the registers of the resident threads can hold,
// and no load instruction of the computing warps ever waits for HBM.
//
// A bulk copy wants both addresses 16-byte aligned and a size that is a multiple of 16 bytes;
// callers send anything else down a path with plain loads.  Every wait is bounded.
#pragma once
#include <stdint.h>

namespace anc_ring {

constexpr uint32_t kWaitTries = 1u << 19;   // each try may suspend ~2 us: about a second in all

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// the last operand is the time (ns) the hardware may keep the thread suspended in the instruction
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(2000u)
      : "memory");
  return ok != 0;
}
// false when the limit ran out
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t tries = kWaitTries) {
  for (uint32_t it = 0; it < tries; ++it)
    if (mbar_try(bar, parity)) return true;
  return false;
}
// For the feeding thread when it gives up at iteration `it`: waits (bounded) until the copies of the
// stages it issued last have landed, so that none is in flight when the CTA's shared memory is released.
template <int kStages>
__device__ __forceinline__ void drain_issued(uint32_t full0, uint32_t it) {
  const uint32_t lo = it > (uint32_t)kStages ? it - (uint32_t)kStages : 0u;
  for (uint32_t i = lo; i < it; ++i) mbar_wait(full0 + 8u * (i % kStages), (i / kStages) & 1u, 1u << 12);
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// One 2-D / 3-D box of a tiled tensor map that lives in global memory (written by the host before
// the launch).  The innermost coordinate times the element size must be a multiple of 16 bytes
// and the destination 128-byte aligned.
__device__ __forceinline__ void box_load_2d(uint32_t dst, const void *map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void box_load_3d(uint32_t dst, const void *map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
// barrier `id` (1, 2, ...) among the `count` threads of one group of computing warps
__device__ __forceinline__ void bar_compute(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// The same barrier with an OR over a predicate: every computing warp learns whether any of them
// gave up its wait, so that they leave together and nobody is left standing at a later barrier.
__device__ __forceinline__ bool bar_compute_or(int id, int count, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %3, 0;\n\t"
      "barrier.cta.red.or.pred q, %1, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(id), "r"(count), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

// Eight consecutive floats of a staged array, element index 8 * t, as two 16-byte reads.  A
// quarter warp reading chunks 2t and 2t+1 in the same order would hit every bank group twice;
// lanes 4-7 of each eight take the odd chunk first.
__device__ __forceinline__ void ld8(const float *base, int t, int lane, float out[8]) {
  const int sw = (lane >> 2) & 1;
  const float4 *q = reinterpret_cast<const float4 *>(base) + 2 * t;
  const float4 a = q[sw], b = q[sw ^ 1];
  const float4 lo = sw ? b : a, hi = sw ? a : b;
  out[0] = lo.x; out[1] = lo.y; out[2] = lo.z; out[3] = lo.w;
  out[4] = hi.x; out[5] = hi.y; out[6] = hi.z; out[7] = hi.w;
}
// Eight consecutive bf16 values (one 16-byte read), widened.
__device__ __forceinline__ void ld8_bf16(const uint16_t *base, int t, float out[8]) {
  const uint4 r = reinterpret_cast<const uint4 *>(base)[t];
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    out[2 * k] = __uint_as_float(w[k] << 16);
    out[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
  }
}

}  // namespace anc_ring
