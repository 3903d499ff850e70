// Batched Newton-Schulz GEMM phases for sm_100a: bf16 operands staged in shared
// memory by TMA, tcgen05.mma with fp32 accumulators in tensor memory (TMEM), fused
// axpy + bf16 rounding in the epilogue.  One persistent CTA per SM walks a static
// tile list; the accumulator is double-buffered in TMEM so the epilogue of one tile
// overlaps the MMAs of the next.
//
//   mode 0 (gram)  : C = RNE(P P^T)                    lower 128-blocks + mirrored store
//   mode 1 (poly)  : C = RNE(alpha*P + beta*(P P^T) [+ diag*I])   P symmetric, so P P^T = P P
//   mode 2 (apply) : C = RNE(alpha*Q + beta*(P Q))     full tiles, Q read N-major
//
// The optimizer's chain folds the iteration's a*X term into the polynomial: with
// B' = b*A + c*A*A + a*I (the diagonal added in fp32 before the one rounding of B') the new
// iterate is X' = B'*X, a plain product, so the apply phase fetches no axpy operand at all:
// a quarter less epilogue traffic on the phase that holds 70 % of the tiles.  Against the fp32
// chain the error is the same as with the separate a*X term (0.5 % relative Frobenius).
//
// which are the three launches per iteration of the reference's fused chain
// (ancora/kernels/muon_ns.py:261-273: _gemm_nt_tril+_mirror, _gemm_axpy_tril+_mirror,
// _gemm_axpy_bf16).  Every output element is produced by exactly one tile with a
// fixed K order (no split-K, no atomics), so results are bitwise independent of the
// grid and of which other matrices share the launch.
//
// All waits are bounded: a wait that runs out records a status bit, raises a CTA-wide
// abort flag and the kernel drains and returns (TMEM is always released).
#include <cuda.h>
#include <cuda_bf16.h>
#include <map>
#include <mutex>
#include <stdlib.h>
#include <vector>
#include "anc_internal.h"

namespace {

constexpr int BM = 128;            // tile rows (UMMA M)
constexpr int BK = 64;             // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;          // 16 KiB
constexpr int kBBytes = 256 * BK * 2;         // 32 KiB (tile width up to 256)
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/;
constexpr int kThreads = 192;      // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSpinLimit = 1u << 19;   // tries; each may suspend up to ~2 us: about a second

struct GemmParams {
  const uint16_t *D;      // axpy operand (modes 1, 2), same layout as C
  uint16_t *C;
  const uint32_t *tile_tab;
  const float *mscale;    // per-matrix factor folded into the epilogue (nullable)
  uint32_t *status;
  int E, M, ldc;          // matrices, rows per matrix, row pitch of C/D in elements
  int tiles_per_matrix, total_tiles, kblocks, mode;
  float alpha, beta;
  float diag;             // mode 1: added to the diagonal elements (0 = nothing added, bit for bit)
  int use_d;              // the axpy operand D is read (mode 1; mode 2 unless alpha == 0)
};

// ---- PTX wrappers ----------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// The last operand is the time (ns) the hardware may keep the thread suspended inside the
// instruction: a suspended thread uses no issue slots, unlike a loop around a test.
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
// Bounded wait.  Returns false when the limit ran out or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try(bar, parity)) return true;
    if (it > 64) {
      __nanosleep(128);
      if ((it & 255) == 0 && *abort_flag) return false;
    }
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld64(uint32_t taddr, uint32_t *r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Programmatic dependent launch: the next kernel on the stream may be scheduled while this one
// still runs; it blocks in pdl_wait() until every earlier grid has completed and its writes
// are visible.  Hides the launch latency between the chained phases.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading/stride byte
// offsets (all >> 4), version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo)) |
         ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi)) << 16);
}

__global__ void __launch_bounds__(kThreads, 1)
ns_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;             // stage buffers, 1024-aligned
  uint8_t *gen_base = smem_raw + (base - raw);
  uint64_t *bars = reinterpret_cast<uint64_t *>(gen_base + kStages * kStageBytes);
  const uint32_t bar0 = base + kStages * kStageBytes;
  // barrier slots: full[0..S), empty[S..2S), tmem_full[2S..2S+2), tmem_empty[2S+2..2S+4)
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 2 + b); };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // TMEM allocation: one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();                       // operands were written by the previous launch

  const bool nmajor_b = (p.mode == 2);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
        const int e = t / p.tiles_per_matrix;
        const uint32_t tt = p.tile_tab[t - e * p.tiles_per_matrix];
        const int i = tt & 0xFF, j = (tt >> 8) & 0xFF, w = (tt >> 16) & 0xFF;
        const int row0 = e * p.M;
        const uint32_t bytes = kABytes + (uint32_t)w * 128u * BK * 2u;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) {
            atomicOr(p.status, ANC_DEV_TIMEOUT_TMA);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kABytes;
          mbar_expect_tx(full_bar(s), bytes);
          tma_load_2d(sa, &tmA, kb * BK, row0 + i * BM, full_bar(s));
          if (!nmajor_b) {
            // K-major B operand: 128-row boxes of P, rows (j + h) * 128
            for (int h = 0; h < w; ++h)
              tma_load_2d(sb + h * (128 * BK * 2), &tmB, kb * BK, row0 + (j + h) * 128, full_bar(s));
          } else {
            // N-major B operand: boxes of 64 columns x 64 K-rows of Q
            for (int c = 0; c < 2 * w; ++c)
              tma_load_2d(sb + c * (64 * BK * 2), &tmB, j * 128 + c * 64, row0 + kb * BK, full_bar(s));
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x, ++acc_it) {
        const int e = t / p.tiles_per_matrix;
        const uint32_t tt = p.tile_tab[t - e * p.tiles_per_matrix];
        const int w = (tt >> 16) & 0xFF;
        const uint32_t n_dim = (uint32_t)w * 128u;
        // instruction descriptor: D=f32, A=B=bf16, A K-major, B K- or N-major, N, M=128
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((nmajor_b ? 1u : 0u) << 16) |
                               ((n_dim >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        const uint32_t buf = acc_it & 1;
        const uint32_t aph = (acc_it >> 1) & 1;
        if (!mbar_wait(tempty_bar(buf), aph ^ 1, abort_flag)) {
          atomicOr(p.status, ANC_DEV_TIMEOUT_MMA);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * 256u;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(full_bar(s), ph, abort_flag)) {
            atomicOr(p.status, ANC_DEV_TIMEOUT_MMA);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // A: K-major, 8-row groups 1024 B apart; K advance = 32 B inside the swizzle row
            const uint64_t da = make_desc(sa + k * (UMMA_K * 2), 16, 1024);
            // B: K-major like A, or N-major: 64-column chunks 8192 B apart (LBO),
            //    8-K-row groups 1024 B apart (SBO); K advance = 16 rows * 128 B
            const uint64_t db = nmajor_b ? make_desc(sb + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                         : make_desc(sb + k * (UMMA_K * 2), 16, 1024);
            tc_mma(tmem_d, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(empty_bar(s));   // frees the stage when these MMAs have read it
        }
        if (ok) tc_commit(tfull_bar(buf));   // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;                  // TMEM lane quarter this warp may read
    const int r = q * 32 + lane;             // row inside the 128-row tile
    uint32_t acc_it = 0;
    for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x, ++acc_it) {
      const int e = t / p.tiles_per_matrix;
      const uint32_t tt = p.tile_tab[t - e * p.tiles_per_matrix];
      const int i = tt & 0xFF, j = (tt >> 8) & 0xFF, w = (tt >> 16) & 0xFF;
      const uint32_t buf = acc_it & 1;
      const uint32_t aph = (acc_it >> 1) & 1;
      if (!mbar_wait(tfull_bar(buf), aph, abort_flag)) {
        if (lane == 0) atomicOr(p.status, ANC_DEV_TIMEOUT_EPI);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const size_t grow = (size_t)e * p.M + (size_t)i * BM + r;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256u;
      // optional per-matrix factor r: mode 0 scales the product by r^2, mode 2 both terms by r
      const bool scaled = p.mscale != nullptr && p.mode != 1;
      const float sc = scaled ? p.mscale[e] : 1.f;
      const float sc2 = __fmul_rn(sc, sc);
      const float al = scaled ? __fmul_rn(p.alpha, sc) : p.alpha;
      const float be = scaled ? __fmul_rn(p.beta, sc) : p.beta;
      for (int cc = 0; cc < 4 * w; ++cc) {
        uint32_t v[32];
        tc_ld32(taddr0 + cc * 32, v);
        tc_wait_ld();
        const int col = j * 128 + cc * 32;
        uint16_t *crow = p.C + grow * p.ldc + col;
        float f[32];
        if (p.mode == 0) {
#pragma unroll
          for (int k = 0; k < 32; ++k)
            f[k] = scaled ? __fmul_rn(sc2, __uint_as_float(v[k])) : __uint_as_float(v[k]);
        } else if (!p.use_d) {
#pragma unroll
          for (int k = 0; k < 32; ++k) f[k] = __fmul_rn(be, __uint_as_float(v[k]));
        } else {
          const uint4 *drow = reinterpret_cast<const uint4 *>(p.D + grow * p.ldc + col);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const uint4 d = drow[k4];
            const uint32_t dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float dlo = __uint_as_float(dw[k] << 16);
              const float dhi = __uint_as_float(dw[k] & 0xFFFF0000u);
              f[k4 * 8 + 2 * k] =
                  __fmaf_rn(be, __uint_as_float(v[k4 * 8 + 2 * k]), __fmul_rn(al, dlo));
              f[k4 * 8 + 2 * k + 1] =
                  __fmaf_rn(be, __uint_as_float(v[k4 * 8 + 2 * k + 1]), __fmul_rn(al, dhi));
            }
          }
        }
        if (p.mode == 1 && p.diag != 0.f) {   // the matrix's diagonal passes through this chunk?
          const int dk = i * BM + r - col;
#pragma unroll
          for (int k = 0; k < 32; ++k)
            if (k == dk) f[k] = __fadd_rn(f[k], p.diag);
        }
        uint32_t h[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) h[k] = pack_bf16(f[2 * k], f[2 * k + 1]);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          reinterpret_cast<uint4 *>(crow)[k4] =
              make_uint4(h[4 * k4], h[4 * k4 + 1], h[4 * k4 + 2], h[4 * k4 + 3]);
        if (p.mode != 2) {
          // mirror: the 128-block (i, hb) with hb < i also lands, transposed, at (hb, i)
          const int hb = j + (cc >> 2);
          if (hb < i) {
            uint16_t *mcol = p.C + ((size_t)e * p.M + (size_t)col) * p.ldc + (size_t)i * BM + r;
#pragma unroll
            for (int k = 0; k < 32; ++k)
              mcol[(size_t)k * p.ldc] = (uint16_t)((k & 1) ? (h[k >> 1] >> 16) : (h[k >> 1] & 0xFFFFu));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}


// ====================================================================================
// CTA-pair variant (tcgen05 cta_group::2).  Two CTAs of a 2-CTA cluster compute one
// 256x256 tile: CTA r owns rows [128r, 128r+128) of the tile (its accumulator lives in its
// own TMEM) and loads only its half of each operand per K block -- 128 rows of A and 128
// of the 256 B columns (16 KiB + 16 KiB per stage instead of 16 + 32) -- so the bytes an
// SM must keep in flight per FLOP drop by a third and six stages fit in shared memory.
// The leader CTA (cluster rank 0) issues every MMA; both CTAs' TMA loads complete on the
// leader's "full" barrier; stage release and accumulator-ready signals are multicast
// tcgen05.commit arrivals on both CTAs' barriers; the peer's epilogue warps arrive on the
// leader's "accumulator free" barrier through its cluster address.  No TMA load is
// multicast.
// ====================================================================================
constexpr int kStages2 = 5;
constexpr int kHalfBBytes = 128 * BK * 2;                 // 16 KiB
constexpr int kStageBytes2 = kABytes + kHalfBBytes;       // 32 KiB
constexpr int kEpiBoxBytes = 128 * 64 * 2;                // one 128-row x 64-column bf16 box
constexpr int kEpiBytes = 4 * kEpiBoxBytes;               // 128 x 256 staging tile, 64 KiB
constexpr int kSmemBytes2 = kStages2 * kStageBytes2 + kEpiBytes + 1024 + 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y,
                                                 uint32_t leader_bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(leader_bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask)
      : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map),
               "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void epi_bar(int id) {   // the 128 epilogue threads only
  asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory");
}

// Barrier of the 128 epilogue threads that also ORs a predicate, so that a decision taken on a
// flag other roles may raise at any moment is the same for all of them.
__device__ __forceinline__ bool epi_bar_or(int id, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %2, 0;\n\t"
      "barrier.cta.red.or.pred q, %1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(id), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}
// The same over the 256 epilogue threads of the chain kernel.
__device__ __forceinline__ bool epi_bar_or256(int id, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %2, 0;\n\t"
      "barrier.cta.red.or.pred q, %1, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(id), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

// tile_tab entries here are (I | J << 8) in units of 256 rows / 256 columns.
__global__ void __launch_bounds__(kThreads, 1)
ns_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmD,
                    const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gen_base = smem_raw + (base - raw);
  const uint32_t epi_base = base + kStages2 * kStageBytes2;      // 64 KiB staging, 1024-aligned
  uint8_t *epi_gen = gen_base + kStages2 * kStageBytes2;
  uint64_t *bars = reinterpret_cast<uint64_t *>(epi_gen + kEpiBytes);
  const uint32_t bar0 = epi_base + kEpiBytes;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages2 + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * kStages2 + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * kStages2 + 2 + b); };
  const uint32_t dfull_bar = bar0 + 8u * (2 * kStages2 + 4);     // axpy operand landed in staging
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages2 + 5);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();          // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(full_bar(s), 1);      // leader's copy is the one in use
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);    // 4 epilogue warps in each of the 2 CTAs (leader's copy in use)
    }
    mbar_init(dfull_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                // both CTAs' barriers exist before any remote signal
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();                        // operands were written by the previous launch
  const bool nmajor_b = (p.mode == 2);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair_id; ok && t < p.total_tiles; t += n_pairs) {
        const int e = t / p.tiles_per_matrix;
        const uint32_t tt = p.tile_tab[t - e * p.tiles_per_matrix];
        const int I = tt & 0xFF, J = (tt >> 8) & 0xFF;
        const int row0 = e * p.M;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % kStages2;
          const uint32_t ph = (it / kStages2) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) {
            atomicOr(p.status, ANC_DEV_TIMEOUT_TMA);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t sa = base + s * kStageBytes2;
          const uint32_t sb = sa + kABytes;
          const uint32_t lead_full = map_to_cta(full_bar(s), 0);
          if (crank == 0) mbar_expect_tx(full_bar(s), 2u * kStageBytes2);   // both CTAs' bytes
          tma_load_2d_pair(sa, &tmA, kb * BK, row0 + I * 256 + (int)crank * 128, lead_full);
          if (!nmajor_b) {
            tma_load_2d_pair(sb, &tmB, kb * BK, row0 + J * 256 + (int)crank * 128, lead_full);
          } else {
            for (int c = 0; c < 2; ++c)
              tma_load_2d_pair(sb + c * (64 * BK * 2), &tmB, J * 256 + (int)crank * 128 + c * 64,
                               row0 + kb * BK, lead_full);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && crank == 0) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      // D=f32, A=B=bf16, A K-major, B K- or N-major, N=256, M=256 (pair)
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((nmajor_b ? 1u : 0u) << 16) |
                             ((256u >> 3) << 17) | ((256u >> 4) << 24);
      for (int t = pair_id; ok && t < p.total_tiles; t += n_pairs, ++acc_it) {
        const uint32_t buf = acc_it & 1;
        const uint32_t aph = (acc_it >> 1) & 1;
        if (!mbar_wait(tempty_bar(buf), aph ^ 1, abort_flag)) {
          atomicOr(p.status, ANC_DEV_TIMEOUT_MMA);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * 256u;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % kStages2;
          const uint32_t ph = (it / kStages2) & 1;
          if (!mbar_wait(full_bar(s), ph, abort_flag)) {
            atomicOr(p.status, ANC_DEV_TIMEOUT_MMA);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = base + s * kStageBytes2;
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_desc(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = nmajor_b ? make_desc(sb + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                         : make_desc(sb + k * (UMMA_K * 2), 16, 1024);
            tc_mma_pair(tmem_d, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit_pair(empty_bar(s));
        }
        if (ok) tc_commit_pair(tfull_bar(buf));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, both CTAs)
    // Global traffic goes through a 128x256 bf16 staging tile in shared memory (four
    // 128-row x 64-column boxes, 128-byte swizzle): the axpy operand arrives by TMA while
    // the tile's MMAs still run, each thread combines its row in place, and the result
    // leaves by TMA store.  Only the mirrored (transposed) blocks of the symmetric phases
    // are stored from registers.
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const bool elected = (threadIdx.x == 64);
    uint32_t acc_it = 0;
    for (int t = pair_id; t < p.total_tiles; t += n_pairs, ++acc_it) {
      const int e = t / p.tiles_per_matrix;
      const uint32_t tt = p.tile_tab[t - e * p.tiles_per_matrix];
      const int I = tt & 0xFF, J = (tt >> 8) & 0xFF;
      const int i = 2 * I + (int)crank;       // this CTA's 128-row block
      const int j = 2 * J;                    // first 128-column block
      // symmetric phases keep the lower 128-blocks only (hb <= i); the upper block of a
      // diagonal tile is produced by the mirror of its transpose
      const int nblk = (p.mode == 2 || j + 1 <= i) ? 2 : 1;
      const uint32_t buf = acc_it & 1;
      const uint32_t aph = (acc_it >> 1) & 1;
      const int grow0 = e * p.M + i * BM;
      if (elected) {
        bulk_wait_read0();                    // previous tile's stores no longer read staging
        if (p.use_d) {
          mbar_expect_tx(dfull_bar, (uint32_t)nblk * 2u * kEpiBoxBytes);
          for (int b = 0; b < 2 * nblk; ++b)
            tma_load_2d(epi_base + b * kEpiBoxBytes, &tmD, j * 128 + b * 64, grow0, dfull_bar);
        }
      }
      epi_bar(2);                             // staging is free for this tile
      bool ok = mbar_wait(tfull_bar(buf), aph, abort_flag);
      if (ok && p.use_d) ok = mbar_wait(dfull_bar, acc_it & 1, abort_flag);
      ok = __all_sync(0xFFFFFFFFu, ok);       // the warp-wide TMEM loads below need a converged warp
      if (!ok) {
        if (lane == 0) atomicOr(p.status, ANC_DEV_TIMEOUT_EPI);
        *abort_flag = 1;
      } else {
        tc_fence_after();
        const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256u;
        uint8_t *my_row = epi_gen + r * 128;
        const bool scaled = p.mscale != nullptr && p.mode != 1;
        const float sc = scaled ? p.mscale[e] : 1.f;
        const float sc2 = __fmul_rn(sc, sc);
        const float al = scaled ? __fmul_rn(p.alpha, sc) : p.alpha;
        const float be = scaled ? __fmul_rn(p.beta, sc) : p.beta;
        for (int cc = 0; cc < 4 * nblk; ++cc) {
          uint32_t v[32];
          tc_ld32(taddr0 + cc * 32, v);
          tc_wait_ld();
          // this thread's 32 columns sit in box cc/2 as four 16-byte pieces, swizzled by row
          uint8_t *box_row = my_row + (cc >> 1) * kEpiBoxBytes;
          const int c16 = (cc & 1) * 4;
          uint32_t h[16];
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            uint4 *slot = reinterpret_cast<uint4 *>(box_row + (((c16 + k4) ^ (r & 7)) << 4));
            float f[8];
            if (p.mode == 0) {
#pragma unroll
              for (int k = 0; k < 8; ++k)
                f[k] = scaled ? __fmul_rn(sc2, __uint_as_float(v[k4 * 8 + k])) : __uint_as_float(v[k4 * 8 + k]);
            } else if (!p.use_d) {
#pragma unroll
              for (int k = 0; k < 8; ++k) f[k] = __fmul_rn(be, __uint_as_float(v[k4 * 8 + k]));
            } else {
              const uint4 d = *slot;
              const uint32_t dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float dlo = __uint_as_float(dw[k] << 16);
                const float dhi = __uint_as_float(dw[k] & 0xFFFF0000u);
                f[2 * k] = __fmaf_rn(be, __uint_as_float(v[k4 * 8 + 2 * k]), __fmul_rn(al, dlo));
                f[2 * k + 1] =
                    __fmaf_rn(be, __uint_as_float(v[k4 * 8 + 2 * k + 1]), __fmul_rn(al, dhi));
              }
            }
            if (p.mode == 1 && p.diag != 0.f) {   // the matrix's diagonal passes through these 8 columns?
              const int dk = i * BM + r - (j * 128 + cc * 32 + k4 * 8);
#pragma unroll
              for (int k = 0; k < 8; ++k)
                if (k == dk) f[k] = __fadd_rn(f[k], p.diag);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) h[k4 * 4 + k] = pack_bf16(f[2 * k], f[2 * k + 1]);
            *slot = make_uint4(h[k4 * 4], h[k4 * 4 + 1], h[k4 * 4 + 2], h[k4 * 4 + 3]);
          }
          const int hb = j + (cc >> 2);
          if (p.mode != 2 && hb < i) {
            const int col = j * 128 + cc * 32;
            uint16_t *mcol = p.C + ((size_t)e * p.M + (size_t)col) * p.ldc + (size_t)i * BM + r;
#pragma unroll
            for (int k = 0; k < 32; ++k)
              mcol[(size_t)k * p.ldc] = (uint16_t)((k & 1) ? (h[k >> 1] >> 16) : (h[k >> 1] & 0xFFFFu));
          }
        }
        // accumulator fully read: hand the TMEM buffer back before the stores go out
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0));
        fence_async_smem();                   // staging writes visible to the TMA store
      }
      // every row of the staging tile is final; the abort decision is made uniform by the barrier
      if (epi_bar_or(1, *abort_flag != 0)) break;
      if (elected) {
        for (int b = 0; b < 2 * nblk; ++b)
          tma_store_2d(&tmC, j * 128 + b * 64, grow0, epi_base + b * kEpiBoxBytes);
        bulk_commit();
      }
    }
    if (elected) bulk_wait0();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                // the peer's shared memory and barriers stay valid until here
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}


// ====================================================================================
// Whole Newton-Schulz chain in ONE persistent launch (CTA pairs as above).
//
// All 3 * steps phases of all E matrices form one tile queue, phase-major:
//   [iteration 0: gram tiles of matrix 0..E-1 | poly tiles 0..E-1 | apply tiles 0..E-1 | iteration 1 ...]
// CTA pairs claim tiles with an integer atomicAdd (dynamic scheduling: a pair that starts late,
// or shares its SMs with another stream's kernel, simply takes fewer tiles).  A tile of matrix
// e may start when every tile of e's previous phase has been stored, which is tracked by one
// completion counter per matrix; the same rule makes the reuse of A, B and the
// X/Y ping-pong buffers safe.  Tiles are claimed in queue order and only ever depend on
// earlier tiles, so the smallest unfinished tile can always run: waiting cannot deadlock.
// The tile -> output mapping and each tile's K order are those of the per-phase kernel, so
// the results are bitwise the same.
//
// Roles (384 threads): warps 0-7 epilogue; then four single-thread roles: TMA producer, MMA
// issuer (leader CTA), scheduler (leader CTA): it claims a tile, waits for the tile's
// dependencies, decodes it and publishes it to both CTAs through a small ring in shared
// memory; and a thread that raises the matrix's completion counter once the epilogue warps
// have stored their part of a tile (a release at GPU scope waits for the stores to be
// performed, which would otherwise stall the epilogue for a microsecond per tile).
//
// Shared memory holds nothing but the operand ring (7 stages of 32 KiB).  With 256x256 pair
// tiles the tensor cores read 64 B/clk of operands from shared memory and TMA writes another
// 64 B/clk into it, which is all the 128 B/clk an SM has; any staging of the epilogue through
// shared memory therefore takes time from the MMAs, and with K = M = 1024 a tile's epilogue
// moves a quarter as many bytes as its main loop.  So the epilogue works from registers:
// each of its 8 warps (two per TMEM lane quarter, one per half of the tile's columns) fetches
// its rows' 256 bytes of the axpy operand with 256-bit GPU-coherent loads while the tile's MMAs
// still run, then reads its half-row of the accumulator from TMEM in two 64-column loads
// (every TMEM load round trip is slow while MMAs are queued: eight 16-column loads took 4 us
// per tile, as long as the tile's MMAs) and writes the bf16 result with 256-bit stores (full
// 32-byte sectors).
// Every wait is bounded; a wait that runs out raises the launch-wide abort word, and all
// roles drain and return.
// ====================================================================================
constexpr int kChainThreads = 384;
// Warps 0-7 are the epilogue, 8-11 the four single-thread roles.  The roles spend most of their
// time polling barriers; as the lowest-numbered warps of their scheduler partitions they kept the
// issue slots from the epilogue warps (a 64-column combine took 2.7 kclk instead of a few hundred).
constexpr int kProducerWarp = 8, kMmaWarp = 9, kSchedWarp = 10, kSignalWarp = 11;
constexpr int kSchedSlots = 4;
constexpr int kMaxChainSteps = 16;
constexpr int kStages3 = 7;
constexpr uint32_t kTileDone = 0xFFFFFFFFu;
constexpr int kSmemBytes3 = kStages3 * kStageBytes2 + 1024 + 512;
constexpr uint32_t kSignalsPerTile = 2;    // one per CTA of the pair

struct alignas(64) ChainMaps {
  CUtensorMap xy128[2];   // the two ping-pong operand buffers, boxes of 64 columns x 128 rows
  CUtensorMap xy64[2];    // the same buffers, boxes of 64 x 64 (N-major operand of the apply phase)
  CUtensorMap a128, b128; // Gram matrix A and polynomial B, boxes of 64 columns x 128 rows
};

struct ChainParams {
  uint16_t *XY[2], *A, *B;             // the buffers the epilogue reads and writes directly
  const uint32_t *tab_sym, *tab_full;  // (I | J << 8) per local tile
  const float *mscale;                 // per-matrix Frobenius factor folded into iteration 0 (nullable)
  uint32_t *sched;                     // [0] next tile, [1] abort, [2 + e] completed half-tiles of matrix e
  uint32_t *status;
  int E, M, N, steps;
  int g, a;                            // tiles per matrix in a symmetric phase / in the apply phase
  uint32_t total_tiles;
  uint32_t spin_limit;
  float coef[3 * kMaxChainSteps];
};

// A published tile: iteration k, phase (0 gram, 1 poly, 2 apply), matrix e, pair-tile (I, J).
struct ChainTile {
  uint32_t t;
  int k, mode, e, I, J;
};

__device__ __forceinline__ ChainTile chain_decode(const ChainParams &p, uint32_t t) {
  const uint32_t per_it = (uint32_t)p.E * (2u * (uint32_t)p.g + (uint32_t)p.a);
  ChainTile ti;
  ti.t = t;
  ti.k = (int)(t / per_it);
  uint32_t r = t - (uint32_t)ti.k * per_it;
  const uint32_t eg = (uint32_t)p.E * (uint32_t)p.g;
  uint32_t per = (uint32_t)p.g;
  ti.mode = 0;
  if (r >= 2u * eg) {
    r -= 2u * eg;
    ti.mode = 2;
    per = (uint32_t)p.a;
  } else if (r >= eg) {
    r -= eg;
    ti.mode = 1;
  }
  ti.e = (int)(r / per);
  const uint32_t l = r - (uint32_t)ti.e * per;
  const uint32_t tt = (ti.mode == 2 ? p.tab_full : p.tab_sym)[l];
  ti.I = (int)(tt & 0xFF);
  ti.J = (int)((tt >> 8) & 0xFF);
  return ti;
}
// Ring slot: {t, k | mode << 8 | I << 16 | J << 24, e, 0}
__device__ __forceinline__ uint4 chain_pack(const ChainTile &ti) {
  return make_uint4(ti.t, (uint32_t)ti.k | ((uint32_t)ti.mode << 8) | ((uint32_t)ti.I << 16) | ((uint32_t)ti.J << 24),
                    (uint32_t)ti.e, 0u);
}
__device__ __forceinline__ ChainTile chain_unpack(const uint4 w) {
  ChainTile ti;
  ti.t = w.x;
  ti.k = (int)(w.y & 0xFF);
  ti.mode = (int)((w.y >> 8) & 0xFF);
  ti.I = (int)((w.y >> 16) & 0xFF);
  ti.J = (int)((w.y >> 24) & 0xFF);
  ti.e = (int)w.z;
  return ti;
}

__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(2000u)
      : "memory");
  return ok != 0;
}
// Bounded wait with cluster-scope acquire (the data it guards was written by the peer CTA).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                                  uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_cluster(bar, parity)) return true;
    if (it > 64) {
      __nanosleep(64);
      if ((it & 255) == 0 && *abort_flag) return false;
    }
  }
  return false;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, uint4 v) {
  asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.volatile.shared::cta.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *ptr) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t *ptr, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}
// Orders accesses made through the generic proxy (plain loads/stores, atomics) with accesses
// made through the async proxy (TMA) by this thread.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// 256-bit accesses to global memory (eight 32-bit words, 32-byte aligned).  The load is
// coherent at GPU scope: the data was written by other SMs earlier in this launch, and the same
// addresses held other values an iteration ago, so it must not be served from this SM's L1.
__device__ __forceinline__ void ld_gpu_256(const void *ptr, uint32_t (&r)[8]) {
  asm volatile("ld.relaxed.gpu.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "l"(ptr)
               : "memory");
}
__device__ __forceinline__ void st_256(void *ptr, const uint32_t *r) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// Optional per-role stall accounting (compiled in with -DANC_CHAIN_PROFILE only): every role adds
// the cycles it spent in each of its waits to a per-CTA row of a device array.
#ifdef ANC_CHAIN_PROFILE
__device__ unsigned long long g_chain_prof[512 * 5 * 8];
#define PROF_BEGIN() unsigned long long _pt = clock64(); unsigned long long _pa[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define PROF_LAP(k)                      \
  do {                                   \
    const unsigned long long _n = clock64(); \
    _pa[k] += _n - _pt;                  \
    _pt = _n;                            \
  } while (0)
#define PROF_END(role)                                                                      \
  do {                                                                                      \
    for (int _k = 0; _k < 8; ++_k)                                                          \
      atomicAdd(&g_chain_prof[((blockIdx.x % 512) * 5 + (role)) * 8 + _k], _pa[_k]);        \
  } while (0)
#else
#define PROF_BEGIN() do { } while (0)
#define PROF_LAP(k) do { } while (0)
#define PROF_END(role) do { } while (0)
#endif

__global__ void __launch_bounds__(kChainThreads, 1)
ns_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *gen_base = smem_raw + (base - raw);
  // after the operand ring: the tile ring (16-byte slots), then the barriers, then two words
  const uint32_t ring_addr = base + kStages3 * kStageBytes2;
  const uint32_t bar0 = ring_addr + 16u * kSchedSlots;
  uint64_t *bars = reinterpret_cast<uint64_t *>(gen_base + kStages3 * kStageBytes2 + 16 * kSchedSlots);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages3 + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * kStages3 + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * kStages3 + 2 + b); };
  auto sfull_bar = [&](int s) { return bar0 + 8u * (2 * kStages3 + 4 + s); };                 // tile published
  auto sempty_bar = [&](int s) { return bar0 + 8u * (2 * kStages3 + 4 + kSchedSlots + s); };  // slot read by all
  auto done_bar = [&](int s) { return bar0 + 8u * (2 * kStages3 + 4 + 2 * kSchedSlots + s); };  // tile stored by the 8 warps
  constexpr int kNumBars = 2 * kStages3 + 4 + 3 * kSchedSlots;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kNumBars);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t abort_addr = bar0 + 8u * kNumBars + 4u;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages3; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 16);   // 8 epilogue warps in each of the 2 CTAs (leader's copy in use)
    }
    for (int s = 0; s < kSchedSlots; ++s) {
      mbar_init(sfull_bar(s), 1);
      // readers of a slot: the leader's producer, MMA issuer, 8 epilogue warps and signaller (11),
      // the peer's producer, 8 epilogue warps and signaller (10); the leader's copy is in use
      mbar_init(sempty_bar(s), 21);
      mbar_init(done_bar(s), 8);     // one arrival per epilogue warp of this CTA
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();
  // Raises the abort state everywhere: this CTA, the peer CTA, and the launch-wide word that
  // the schedulers of the other pairs poll while they wait for a dependency.
  auto raise_abort = [&](uint32_t bit) {
    atomicOr(p.status, bit);
    *abort_flag = 1;
    st_cluster_u32(map_to_cta(abort_addr, crank ^ 1u), 1u);
    atomicExch(&p.sched[1], 1u);
  };
  auto release_slot = [&](int slot) {
    if (crank == 0) mbar_arrive(sempty_bar(slot));
    else mbar_arrive_cluster(map_to_cta(sempty_bar(slot), 0));
  };
  // n-th tile of this pair for the calling role; tile.t == kTileDone ends the role.  The
  // scheduler publishes a tile only after its dependency wait (bounded by p.spin_limit), so
  // this wait uses the long fixed bound: it must outlast the scheduler's.
  auto ring_get = [&](uint32_t n, bool arrive, uint32_t bit) -> ChainTile {
    const int slot = (int)(n % kSchedSlots);
    // the leader's roles share a CTA with the scheduler: CTA-scope waits and arrivals do
    const bool got = crank == 0 ? mbar_wait(sfull_bar(slot), (n / kSchedSlots) & 1u, abort_flag)
                                : mbar_wait_cluster(sfull_bar(slot), (n / kSchedSlots) & 1u, abort_flag, kSpinLimit);
    if (!got) {
      if (!*abort_flag) raise_abort(bit);
      ChainTile none;
      none.t = kTileDone;
      none.k = none.mode = none.e = none.I = none.J = 0;
      return none;
    }
    const ChainTile ti = chain_unpack(ld_shared_v4(ring_addr + 16u * slot));
    if (arrive) release_slot(slot);
    return ti;
  };

  if (warp == kSchedWarp) {
    // ------------------------------------------------------------ scheduler (leader only)
    if (lane == 0 && crank == 0) {
      const uint32_t limit = p.spin_limit;
      // completions per matrix and iteration, and before the poly / apply phase of an iteration
      const uint32_t per_e_it = kSignalsPerTile * (2u * (uint32_t)p.g + (uint32_t)p.a);
      const uint32_t after_gram = kSignalsPerTile * (uint32_t)p.g;
      PROF_BEGIN();
      for (uint32_t n = 0;; ++n) {
        const int slot = (int)(n % kSchedSlots);
        ChainTile ti;
        ti.t = kTileDone;
        ti.k = ti.mode = ti.e = ti.I = ti.J = 0;
        PROF_LAP(0);
        if (mbar_wait_cluster(sempty_bar(slot), ((n / kSchedSlots) & 1u) ^ 1u, abort_flag, kSpinLimit)) {
          PROF_LAP(1);                 // ring slot free
          const uint32_t t = atomicAdd(&p.sched[0], 1u);
          if (t < p.total_tiles) ti = chain_decode(p, t);
          PROF_LAP(2);                 // claim + decode
        } else if (!*abort_flag) {
          raise_abort(ANC_DEV_TIMEOUT_DEP);
        }
        if (ti.t != kTileDone) {
          const uint32_t need = (uint32_t)ti.k * per_e_it +
                                (ti.mode == 1 ? after_gram : (ti.mode == 2 ? 2u * after_gram : 0u));
          if (need) {
            const uint32_t *cnt = p.sched + 2 + ti.e;
            bool ready = false;
            for (uint32_t it = 0; it < limit; ++it) {
              if (ld_acquire_gpu(cnt) >= need) {
                ready = true;
                break;
              }
              if (it > 16) __nanosleep(32);
              if ((it & 63) == 63 && (ld_acquire_gpu(p.sched + 1) != 0 || *abort_flag)) break;
            }
            if (!ready) {
              if (ld_acquire_gpu(p.sched + 1) == 0 && !*abort_flag) raise_abort(ANC_DEV_TIMEOUT_DEP);
              ti.t = kTileDone;
            }
          }
        }
        PROF_LAP(3);                   // dependency wait
        const uint4 w = chain_pack(ti);
        st_cluster_v4(map_to_cta(ring_addr + 16u * slot, 1), w);
        mbar_arrive_cluster(map_to_cta(sfull_bar(slot), 1));
        asm volatile("st.shared::cta.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(ring_addr + 16u * slot), "r"(w.x),
                     "r"(w.y), "r"(w.z), "r"(w.w)
                     : "memory");
        mbar_arrive(sfull_bar(slot));
        if (ti.t == kTileDone) break;
      }
      PROF_END(4);
    }
  } else if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      PROF_BEGIN();
      for (uint32_t n = 0;; ++n) {
        PROF_LAP(0);
        const ChainTile ti = ring_get(n, true, ANC_DEV_TIMEOUT_TMA);
        PROF_LAP(1);                   // waiting for a tile
        if (ti.t == kTileDone) break;
        fence_proxy_async_all();      // the operands were written by other SMs' plain stores (previous phase)
        const int cur = ti.k & 1;
        const CUtensorMap *ma = ti.mode == 0 ? &maps.xy128[cur] : (ti.mode == 1 ? &maps.a128 : &maps.b128);
        const CUtensorMap *mb = ti.mode == 0 ? &maps.xy128[cur] : (ti.mode == 1 ? &maps.a128 : &maps.xy64[cur]);
        const int kblocks = (ti.mode == 0 ? p.N : p.M) / BK;
        const int row0 = ti.e * p.M;
        const int arow = row0 + ti.I * 256 + (int)crank * 128;
        const int brow = row0 + ti.J * 256 + (int)crank * 128;   // K-major B operand
        const int bcol = ti.J * 256 + (int)crank * 128;          // N-major B operand (apply)
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kStages3;
          const uint32_t ph = (it / kStages3) & 1;
          PROF_LAP(0);
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) {
            if (!*abort_flag) raise_abort(ANC_DEV_TIMEOUT_TMA);
            ok = false;
            break;
          }
          PROF_LAP(2);                 // waiting for a free stage
          const uint32_t sa = base + s * kStageBytes2;
          const uint32_t sb = sa + kABytes;
          const uint32_t lead_full = map_to_cta(full_bar(s), 0);
          if (crank == 0) mbar_expect_tx(full_bar(s), 2u * kStageBytes2);
          tma_load_2d_pair(sa, ma, kb * BK, arow, lead_full);
          if (ti.mode != 2) {
            tma_load_2d_pair(sb, mb, kb * BK, brow, lead_full);
          } else {
            for (int c = 0; c < 2; ++c)
              tma_load_2d_pair(sb + c * (64 * BK * 2), mb, bcol + c * 64, row0 + kb * BK, lead_full);
          }
        }
        if (!ok) break;
      }
      PROF_END(0);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && crank == 0) {
      uint32_t it = 0;
      PROF_BEGIN();
      for (uint32_t n = 0;; ++n) {
        PROF_LAP(0);
        const ChainTile ti = ring_get(n, true, ANC_DEV_TIMEOUT_MMA);
        PROF_LAP(1);                   // waiting for a tile
        if (ti.t == kTileDone) break;
        const bool nmajor_b = (ti.mode == 2);
        const int kblocks = (ti.mode == 0 ? p.N : p.M) / BK;
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((nmajor_b ? 1u : 0u) << 16) |
                               ((256u >> 3) << 17) | ((256u >> 4) << 24);
        const uint32_t buf = n & 1;
        const uint32_t aph = (n >> 1) & 1;
        if (!mbar_wait(tempty_bar(buf), aph ^ 1, abort_flag)) {
          if (!*abort_flag) raise_abort(ANC_DEV_TIMEOUT_MMA);
          break;
        }
        PROF_LAP(2);                   // waiting for a free accumulator (epilogue behind)
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * 256u;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kStages3;
          const uint32_t ph = (it / kStages3) & 1;
          PROF_LAP(0);
          if (!mbar_wait(full_bar(s), ph, abort_flag)) {
            if (!*abort_flag) raise_abort(ANC_DEV_TIMEOUT_MMA);
            ok = false;
            break;
          }
          PROF_LAP(3);                 // waiting for operands
          tc_fence_after();
          const uint32_t sa = base + s * kStageBytes2;
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_desc(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = nmajor_b ? make_desc(sb + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                         : make_desc(sb + k * (UMMA_K * 2), 16, 1024);
            tc_mma_pair(tmem_d, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit_pair(empty_bar(s));
        }
        if (!ok) break;
        tc_commit_pair(tfull_bar(buf));
      }
      PROF_END(1);
    }
  } else if (warp == kSignalWarp) {
    // ------------------------------------------------------------ completion signal (both CTAs)
    if (lane == 0) {
      PROF_BEGIN();
      for (uint32_t n = 0;; ++n) {
        PROF_LAP(0);
        const ChainTile ti = ring_get(n, false, ANC_DEV_TIMEOUT_EPI);
        PROF_LAP(1);
        if (ti.t == kTileDone) {
          release_slot((int)(n % kSchedSlots));
          break;
        }
        // The done barriers are indexed like the ring, and this thread gives its ring slot back only
        // after the wait: tile n + kSchedSlots cannot be published (so no warp can arrive for it on
        // the same barrier) before tile n's phase of the barrier has been observed here.
        if (!mbar_wait(done_bar((int)(n % kSchedSlots)), (n / kSchedSlots) & 1u, abort_flag)) {
          if (!*abort_flag) raise_abort(ANC_DEV_TIMEOUT_EPI);
          break;
        }
        release_slot((int)(n % kSchedSlots));
        PROF_LAP(2);                  // waiting for the epilogue warps
        // release at GPU scope: covers, through the barrier this thread acquired, the stores of all
        // epilogue threads of this CTA; the next phase reads them through TMA (async proxy)
        fence_proxy_async_all();
        red_release_gpu_add(p.sched + 2 + ti.e, 1u);
        PROF_LAP(3);                  // the release
      }
      PROF_END(3);
    }
  } else {
    // ------------------------------------------------------------ epilogue (8 warps, both CTAs)
    // Warp w reads TMEM lanes [32 (w & 3), +32) (the only ones it may touch) and, of the tile's
    // 256 columns, the half w / 4.  Thread = row.  The axpy operand of the whole half-row
    // (256 bytes) is requested before the wait for the accumulator.
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int half = warp >> 2;
    PROF_BEGIN();
    for (uint32_t n = 0;; ++n) {
      const ChainTile ti = ring_get(n, false, ANC_DEV_TIMEOUT_EPI);
      PROF_LAP(0);                  // waiting for a tile (+ loop overhead)
      // warp-uniform end of the role (a lane that gave up on the wait must take its warp along:
      // the TMEM loads below are warp-wide)
      if (__any_sync(0xFFFFFFFFu, ti.t == kTileDone)) break;
      const int slot = (int)(n % kSchedSlots);
      if (lane == 0) release_slot(slot);       // after the vote: every lane has read the slot
      const int mode = ti.mode;
      const int i = 2 * ti.I + (int)crank;
      const int j = 2 * ti.J;
      const int nblk = (mode == 2 || j + 1 <= i) ? 2 : 1;
      const bool active = half < nblk;    // a diagonal tile's upper block comes from the mirror
      const uint32_t buf = n & 1;
      const uint32_t aph = (n >> 1) & 1;
      const int cur = ti.k & 1;
      const int ld = mode == 2 ? p.N : p.M;                                   // row pitch of C and D
      const uint16_t *dbase = p.A;                                            // axpy operand (poly phase)
      uint16_t *cbase = mode == 0 ? p.A : (mode == 1 ? p.B : p.XY[cur ^ 1]);
      const size_t row_off = ((size_t)ti.e * p.M + (size_t)i * BM + r) * ld + (size_t)j * 128 + (size_t)half * 128;
      const uint16_t *drow = dbase + row_off;
      uint16_t *crow = cbase + row_off;
      uint32_t d[64];                     // the half-row of the axpy operand (poly phase): 128 bf16
      if (mode == 1 && active) {
#pragma unroll
        for (int s = 0; s < 8; ++s) ld_gpu_256(drow + s * 16, reinterpret_cast<uint32_t(&)[8]>(d[s * 8]));
      }
      PROF_LAP(1);                  // issuing the axpy operand loads
      bool ok = mbar_wait(tfull_bar(buf), aph, abort_flag);
      PROF_LAP(2);                  // waiting for the accumulator (MMA-bound when large)
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) {
        if (lane == 0 && !*abort_flag) raise_abort(ANC_DEV_TIMEOUT_EPI);
        break;
      }
      tc_fence_after();
      PROF_LAP(3);                  // warp vote + fence
      if (active) {
        const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256u + (uint32_t)half * 128u;
        const bool scaled = p.mscale != nullptr && ti.k == 0 && mode != 1;
        const float sc = scaled ? p.mscale[ti.e] : 1.f;
        const float sc2 = __fmul_rn(sc, sc);
        // poly: B' = b*A + c*(A A) + a*I; apply: X' = B' X (times the Frobenius factor in iteration 0)
        const float al = mode == 1 ? p.coef[3 * ti.k + 1] : 0.f;
        const float be = mode == 1 ? p.coef[3 * ti.k + 2] : sc;
        const float a_diag = p.coef[3 * ti.k];
        // the matrix's diagonal crosses this warp's 128 columns in the diagonal 128-block only,
        // at column r of the block
        const int dcol = (mode == 1 && i == j + half) ? r : -1;
        const bool mirror = mode != 2 && j + half < i;   // block (i, j + half) also lands, transposed, at (j + half, i)
        uint16_t *mcol0 = cbase + ((size_t)ti.e * p.M + (size_t)(j + half) * 128) * p.M + (size_t)i * BM + r;
        uint32_t v[64];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {                      // two round trips of 64 columns
          tc_ld64(taddr0 + hh * 64, v);
          tc_wait_ld();
          if (hh == 0) PROF_LAP(4); else PROF_LAP(6);   // TMEM round trips
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4) {
            const int s = hh * 4 + s4;
            uint32_t h[8];
            if (mode == 0) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const float lo = __uint_as_float(v[s4 * 16 + 2 * k]), hi = __uint_as_float(v[s4 * 16 + 2 * k + 1]);
                h[k] = scaled ? pack_bf16(__fmul_rn(sc2, lo), __fmul_rn(sc2, hi)) : pack_bf16(lo, hi);
              }
            } else if (mode == 2) {
#pragma unroll
              for (int k = 0; k < 8; ++k)
                h[k] = pack_bf16(__fmul_rn(be, __uint_as_float(v[s4 * 16 + 2 * k])),
                                 __fmul_rn(be, __uint_as_float(v[s4 * 16 + 2 * k + 1])));
            } else {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const uint32_t dw = d[s * 8 + k];
                const float dlo = __uint_as_float(dw << 16);
                const float dhi = __uint_as_float(dw & 0xFFFF0000u);
                float lo = __fmaf_rn(be, __uint_as_float(v[s4 * 16 + 2 * k]), __fmul_rn(al, dlo));
                float hi = __fmaf_rn(be, __uint_as_float(v[s4 * 16 + 2 * k + 1]), __fmul_rn(al, dhi));
                if (dcol == s * 16 + 2 * k) lo = __fadd_rn(lo, a_diag);
                if (dcol == s * 16 + 2 * k + 1) hi = __fadd_rn(hi, a_diag);
                h[k] = pack_bf16(lo, hi);
              }
            }
            st_256(crow + s * 16, h);
            if (mirror) {
              uint16_t *mcol = mcol0 + (size_t)(s * 16) * p.M;
#pragma unroll
              for (int k = 0; k < 16; ++k)
                mcol[(size_t)k * p.M] = (uint16_t)((k & 1) ? (h[k >> 1] >> 16) : (h[k >> 1] & 0xFFFFu));
            }
          }
          if (hh == 0) PROF_LAP(5);   // combine + stores of the first 64 columns
        }
      }
      PROF_LAP(7);                  // combine + stores of the last 64 columns
      // accumulator read: hand the TMEM buffer back; then pass this warp's part of the tile to the
      // signalling thread (the barrier orders the stores of all lanes before its release)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0));
        mbar_arrive(done_bar(slot));
      }
    }
    if (threadIdx.x == 0) PROF_END(2);
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

// ---- host side -------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void *sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || !sym) {
    cudaGetLastError();
    return nullptr;
  }
  fn = (EncodeTiledFn)sym;
  return fn;
}

// 2-D bf16 row-major tensor (rows, cols), box (box_cols=64, box_rows), 128-byte swizzle.
int make_map(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    anc_set_error("cuTensorMapEncodeTiled is not available from this driver");
    return ANC_E_CUDA;
  }
  if (((uintptr_t)ptr & 15) != 0 || (cols * 2) % 16 != 0) {
    anc_set_error("TMA operand must be 16-byte aligned with a 16-byte multiple row pitch");
    return ANC_E_INVALID;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    anc_set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return ANC_E_CUDA;
  }
  return ANC_OK;
}

}  // namespace

int anc_encode_tile_map(anc_tmap *out, const void *ptr, int elem_bytes, uint64_t inner, uint64_t rows,
                        uint64_t slices, uint32_t box_inner, uint32_t box_rows) {
  static_assert(sizeof(anc_tmap) == sizeof(CUtensorMap), "tensor map storage");
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    anc_set_error("cuTensorMapEncodeTiled is not available from this driver");
    return ANC_E_CUDA;
  }
  const uint64_t eb = (uint64_t)elem_bytes;
  if ((elem_bytes != 2 && elem_bytes != 4) || ((uintptr_t)ptr & 15) != 0 || (inner * eb) % 16 != 0 ||
      (box_inner * eb) % 16 != 0 || box_inner > 256 || box_rows > 256) {
    anc_set_error("tile map: operand must be 16-byte aligned with 16-byte multiple rows and boxes");
    return ANC_E_INVALID;
  }
  cuuint64_t dims[3] = {inner, rows, slices ? slices : 1};
  cuuint64_t strides[2] = {inner * eb, inner * rows * eb};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(reinterpret_cast<CUtensorMap *>(out),
                   elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                   slices ? 3 : 2, const_cast<void *>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    anc_set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return ANC_E_CUDA;
  }
  return ANC_OK;
}

namespace {

struct TileTab {
  uint32_t *d_tab;
  int count;
};
struct GemmCache {
  std::map<uint64_t, TileTab> tabs;
  bool attr_set = false;
  bool attr2_set = false;
  bool attr3_set = false;
};
std::map<anc_ctx *, GemmCache *> g_caches;
std::mutex g_caches_mu;   // contexts of different threads may launch concurrently

// Tile list of one matrix.  sym: lower-triangular 128-blocks of an (mb x mb) grid packed
// into 256-wide tiles; else the full (mb x nb) grid.
int get_tile_tab(anc_ctx *ctx, bool sym, bool pair, int mb, int nb, TileTab *out) {
  std::lock_guard<std::mutex> lock(g_caches_mu);
  GemmCache *&gc = g_caches[ctx];
  if (!gc) gc = new GemmCache();
  const uint64_t key = ((uint64_t)(sym ? 1 : 0) << 40) | ((uint64_t)(pair ? 1 : 0) << 41) |
                       ((uint64_t)mb << 20) | (uint64_t)nb;
  auto it = gc->tabs.find(key);
  if (it != gc->tabs.end()) {
    *out = it->second;
    return ANC_OK;
  }
  std::vector<uint32_t> tab;
  if (pair) {
    // units of 256 rows x 256 columns; sym keeps J <= I
    for (int i = 0; i < mb / 2; ++i)
      for (int j = 0; j < (sym ? i + 1 : nb / 2); ++j) tab.push_back((uint32_t)i | ((uint32_t)j << 8));
  }
  for (int i = 0; !pair && i < mb; ++i) {
    if (sym) {
      for (int j = 0; j <= i; j += 2) {
        const int w = (j + 1 <= i) ? 2 : 1;
        tab.push_back((uint32_t)i | ((uint32_t)j << 8) | ((uint32_t)w << 16));
      }
    } else {
      for (int j = 0; j < nb; j += 2) {
        const int w = (nb - j) >= 2 ? 2 : 1;
        tab.push_back((uint32_t)i | ((uint32_t)j << 8) | ((uint32_t)w << 16));
      }
    }
  }
  TileTab tt;
  tt.count = (int)tab.size();
  ANC_CUDA(cudaMalloc((void **)&tt.d_tab, tab.size() * sizeof(uint32_t)));
  ANC_CUDA(cudaMemcpy(tt.d_tab, tab.data(), tab.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
  gc->tabs[key] = tt;
  *out = tt;
  return ANC_OK;
}

}  // namespace

void anc_gemm_cache_destroy(anc_ctx *ctx) {
  std::lock_guard<std::mutex> lock(g_caches_mu);
  auto it = g_caches.find(ctx);
  if (it == g_caches.end()) return;
  for (auto &kv : it->second->tabs) cudaFree(kv.second.d_tab);
  delete it->second;
  g_caches.erase(it);
}

int anc_launch_ns_gemm(anc_ctx *ctx, int mode, const uint16_t *P, const uint16_t *Q, uint16_t *C,
                       int E, int M, int N, float alpha, float beta, float diag, const float *mscale,
                       cudaStream_t st) {
  ANC_REQUIRE(mode >= 0 && mode <= 2, "bad mode %d", mode);
  ANC_REQUIRE(E > 0 && M > 0 && N > 0 && M % 128 == 0 && N % 128 == 0,
              "Newton-Schulz shape (%d x %d x %d) must be multiples of 128", E, M, N);
  ANC_REQUIRE(M / 128 <= 255 && N / 128 <= 255, "matrix too large for the tile table");
  ANC_REQUIRE((size_t)E * M < (1u << 31), "E*M too large");
  // mode 0: P is (E*M, N), K = N.  modes 1/2: P is (E*M, M), K = M.
  const int Kdim = mode == 0 ? N : M;
  const int mb = M / 128;
  CUtensorMap tmA, tmB;
  int rc = make_map(&tmA, P, (uint64_t)E * M, (uint64_t)Kdim, 128);
  if (rc) return rc;
  if (mode == 2) {
    ANC_REQUIRE(Q, "mode 2 needs Q");
    rc = make_map(&tmB, Q, (uint64_t)E * M, (uint64_t)N, 64);
  } else {
    rc = make_map(&tmB, P, (uint64_t)E * M, (uint64_t)Kdim, 128);
  }
  if (rc) return rc;
  // CTA pairs need 256-row tiles (and 256-column tiles in the apply phase)
  const char *env = getenv("ANCORA_NS_CTA_PAIR");
  const bool pair = !(env && env[0] == '0') && M % 256 == 0 && (mode != 2 || N % 256 == 0) &&
                    ctx->sm_count >= 2;
  TileTab tt;
  rc = get_tile_tab(ctx, mode != 2, pair, mb, mode == 2 ? N / 128 : mb, &tt);
  if (rc) return rc;
  GemmCache *gc;
  {
    std::lock_guard<std::mutex> lock(g_caches_mu);
    gc = g_caches[ctx];
  }
  if (!gc->attr_set) {
    ANC_CUDA(cudaFuncSetAttribute(ns_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kSmemBytes));
    gc->attr_set = true;
  }
  GemmParams p;
  p.D = mode == 0 ? nullptr : (mode == 1 ? P : Q);
  p.C = C;
  p.tile_tab = tt.d_tab;
  p.mscale = mscale;
  p.status = ctx->d_status;
  p.E = E;
  p.M = M;
  p.ldc = mode == 2 ? N : M;
  p.tiles_per_matrix = tt.count;
  p.total_tiles = tt.count * E;
  p.kblocks = Kdim / BK;
  p.mode = mode;
  p.alpha = alpha;
  p.beta = beta;
  p.diag = mode == 1 ? diag : 0.f;
  p.use_d = (mode == 1 || (mode == 2 && alpha != 0.f)) ? 1 : 0;
  if (pair) {
    if (!gc->attr2_set) {
      ANC_CUDA(cudaFuncSetAttribute(ns_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBytes2));
      gc->attr2_set = true;
    }
    int pairs = ctx->sm_count / 2;
    if (p.total_tiles < pairs) pairs = p.total_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes2;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    CUtensorMap tmC, tmD;
    rc = make_map(&tmC, C, (uint64_t)E * M, (uint64_t)p.ldc, 128);
    if (rc) return rc;
    rc = make_map(&tmD, mode == 0 ? (const void *)C : (const void *)p.D, (uint64_t)E * M, (uint64_t)p.ldc, 128);
    if (rc) return rc;
    ANC_CUDA(cudaLaunchKernelEx(&cfg, ns_gemm_pair_kernel, tmA, tmB, tmC, tmD, p));
    return ANC_OK;
  }
  int grid = p.total_tiles < ctx->sm_count ? p.total_tiles : ctx->sm_count;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  ANC_CUDA(cudaLaunchKernelEx(&cfg, ns_gemm_kernel, tmA, tmB, p));
  return ANC_OK;
}

bool anc_ns_chain_supported(const anc_ctx *ctx, int M, int N, int steps) {
  const char *env = getenv("ANCORA_NS_CHAIN");
  if (env && env[0] == '0') return false;       // fall back to one launch per phase
  return steps >= 1 && steps <= kMaxChainSteps && M > 0 && M <= N && M % 256 == 0 && N % 256 == 0 &&
         M / 256 <= 255 && N / 256 <= 255 && ctx->sm_count >= 2;
}

// The whole chain of `steps` iterations on E packed matrices in one persistent launch.
// X holds the operand, Y is the second ping-pong buffer: the result is in X when steps is even,
// in Y when it is odd.  sched: 2 + E words that are ZERO when the kernel starts (the Frobenius
// finalize kernel clears them).  spin_limit = 0 selects the default bound of the waits.
int anc_launch_ns_chain(anc_ctx *ctx, uint16_t *X, uint16_t *Y, uint16_t *A, uint16_t *B, int E, int M, int N,
                        int steps, const float *coeffs, const float *mscale, uint32_t *sched,
                        uint32_t spin_limit, cudaStream_t st) {
  ANC_REQUIRE(anc_ns_chain_supported(ctx, M, N, steps), "shape (%d,%d) x %d steps not supported by the chain kernel",
              M, N, steps);
  ANC_REQUIRE(E > 0 && (size_t)E * M < (1u << 31), "bad batch %d", E);
  ANC_REQUIRE(sched, "scheduler words missing");
  ChainMaps maps;
  uint16_t *xy[2] = {X, Y};
  int rc;
  for (int b = 0; b < 2; ++b) {
    if ((rc = make_map(&maps.xy128[b], xy[b], (uint64_t)E * M, (uint64_t)N, 128))) return rc;
    if ((rc = make_map(&maps.xy64[b], xy[b], (uint64_t)E * M, (uint64_t)N, 64))) return rc;
  }
  if ((rc = make_map(&maps.a128, A, (uint64_t)E * M, (uint64_t)M, 128))) return rc;
  if ((rc = make_map(&maps.b128, B, (uint64_t)E * M, (uint64_t)M, 128))) return rc;
  TileTab ts, tf;
  if ((rc = get_tile_tab(ctx, true, true, M / 128, M / 128, &ts))) return rc;
  if ((rc = get_tile_tab(ctx, false, true, M / 128, N / 128, &tf))) return rc;
  GemmCache *gc;
  {
    std::lock_guard<std::mutex> lock(g_caches_mu);
    gc = g_caches[ctx];
  }
  if (!gc->attr3_set) {
    ANC_CUDA(cudaFuncSetAttribute(ns_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes3));
    gc->attr3_set = true;
  }
  ChainParams p;
  memset(&p, 0, sizeof(p));
  p.XY[0] = X;
  p.XY[1] = Y;
  p.A = A;
  p.B = B;
  p.tab_sym = ts.d_tab;
  p.tab_full = tf.d_tab;
  p.mscale = mscale;
  p.sched = sched;
  p.status = ctx->d_status;
  p.E = E;
  p.M = M;
  p.N = N;
  p.steps = steps;
  p.g = ts.count;
  p.a = tf.count;
  const uint64_t total = (uint64_t)steps * E * (2ull * ts.count + tf.count);
  ANC_REQUIRE(total < 0xFFFFFF00ull, "too many tiles");
  p.total_tiles = (uint32_t)total;
  p.spin_limit = spin_limit ? spin_limit : kSpinLimit;
  for (int i = 0; i < 3 * steps; ++i) p.coef[i] = coeffs[i];
  // SMs left free for kernels of other streams (a collective that overlaps the chain): the chain
  // CTAs are persistent and fill an SM each, so a kernel that arrives after them would otherwise
  // wait for the whole chain.  Set per context (anc_ctx_reserve_sms); 0 by default.
  int usable = ctx->sm_count - ctx->reserved_sms;
  if (usable < 2) usable = 2;
  uint64_t pairs = (uint64_t)(usable / 2);
  if (total < pairs) pairs = total;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(kChainThreads);
  cfg.dynamicSmemBytes = kSmemBytes3;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  ANC_CUDA(cudaLaunchKernelEx(&cfg, ns_chain_kernel, maps, p));
  return ANC_OK;
}

extern "C" int anc_ns_gemm_phase(anc_ctx *ctx, int mode, const uint16_t *P, const uint16_t *Q,
                                 uint16_t *C, int E, int M, int N, float alpha, float beta,
                                 void *stream) {
  ANC_REQUIRE(ctx && P && C, "NULL argument");
  anc_device_guard guard(ctx->device);
  return anc_launch_ns_gemm(ctx, mode, P, Q, C, E, M, N, alpha, beta, 0.f, nullptr,
                            anc_pick_stream(ctx, stream));
}

// Launches the chain kernel on a 256x256 matrix with the tile counter preset past the first
// phase, so the first claimed tile depends on a phase that never runs: its bounded wait must
// run out, set ANC_DEV_TIMEOUT_DEP in the context's status word and let every role drain.
extern "C" int anc_ns_chain_wait_selftest(anc_ctx *ctx, uint32_t spin_limit) {
  ANC_REQUIRE(ctx, "ctx is NULL");
  ANC_REQUIRE(spin_limit > 0 && spin_limit <= (1u << 20), "spin_limit must be in [1, 2^20]");
  anc_device_guard guard(ctx->device);
  const int M = 256;
  const size_t bytes = (size_t)M * M * 2;
  char *buf = nullptr;
  ANC_CUDA(cudaMalloc((void **)&buf, 4 * bytes + 256));
  cudaError_t e = cudaMemsetAsync(buf, 0, 4 * bytes + 256, ctx->stream);
  uint32_t *sched = (uint32_t *)(buf + 4 * bytes);
  const uint32_t first_tile = 1;     // tile 0 is the only gram tile; tile 1 (poly) waits for it
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(sched, &first_tile, sizeof(first_tile), cudaMemcpyHostToDevice, ctx->stream);
  int rc = e == cudaSuccess ? ANC_OK : anc_cuda_fail(e, "selftest set-up");
  const float coef[3] = {1.f, 1.f, 1.f};
  if (!rc)
    rc = anc_launch_ns_chain(ctx, (uint16_t *)buf, (uint16_t *)(buf + bytes), (uint16_t *)(buf + 2 * bytes),
                             (uint16_t *)(buf + 3 * bytes), 1, M, M, 1, coef, nullptr, sched, spin_limit,
                             ctx->stream);
  e = cudaStreamSynchronize(ctx->stream);
  cudaFree(buf);
  if (rc) return rc;
  if (e != cudaSuccess) return anc_cuda_fail(e, "selftest sync");
  return ANC_OK;
}

#ifdef ANC_CHAIN_PROFILE
// Reads (and clears) the stall counters: rows of 8 counters for (CTA, role), roles 0 producer,
// 1 MMA issuer, 2 epilogue (its elected thread), 3 store thread, 4 scheduler.
extern "C" __attribute__((visibility("default"))) int anc_debug_chain_prof(unsigned long long *out, int n_ctas) {
  const size_t bytes = (size_t)n_ctas * 5 * 8 * sizeof(unsigned long long);
  ANC_CUDA(cudaDeviceSynchronize());
  ANC_CUDA(cudaMemcpyFromSymbol(out, g_chain_prof, bytes));
  void *sym = nullptr;
  ANC_CUDA(cudaGetSymbolAddress(&sym, g_chain_prof));
  ANC_CUDA(cudaMemset(sym, 0, sizeof(g_chain_prof)));
  return ANC_OK;
}
#endif
