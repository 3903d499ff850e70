// Muon's elementwise kernels for sm_100a (HBM-bound sweeps):
//   momentum + Nesterov  -> packed bf16 Newton-Schulz input   (12 B/elem, bf16 grad)
//   Frobenius normalise  -> fixed-order two-level reduction, then scale in place
//   master update + bf16 refresh                               (12 B/elem)
// Arithmetic follows ancora/kernels/muon_ns.py:184-186 (nb = mu*b + g;
// u = RNE(g + mu*nb)) and :227-229 (pn = p - lr_scale*O; p16 = RNE(pn)) with
// separately rounded float32 operations, so results equal a numpy float32
// evaluation bit for bit.  Tall weights (K > N) store u transposed / read O
// transposed through a shared-memory tile, which is bit-identical to the untransposed
// kernel followed by a transpose (reference: _muon_mom_t, _muon_update_cast_t).
#include <cuda_bf16.h>
#include <mutex>
#include "anc_internal.h"
#include "stream_ring.cuh"

namespace {

constexpr int kTile = 64;
constexpr int kThreads = 256;
constexpr int kPad = 8;   // row pitch 72 bf16 = 144 B: 16-byte aligned rows, few bank conflicts

// Table entries.  The i-th entry of a launched range uses slot i of the packed Newton-Schulz
// operand: slot s starts at element s * K * N and holds (K,N) if !tr, else (N,K).
struct MomW {
  float *buf;
  const void *g;
  int K, N, tr, _pad;
};

struct UpdW {
  float *p32;
  uint16_t *p16;
  int K, N, tr, _pad;
};

__device__ __forceinline__ uint32_t rne16(float x) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x));
}
__device__ __forceinline__ float bf16_f32(uint32_t h) { return __uint_as_float(h << 16); }

// Column swizzle of the 64x64 transposition tile: element (row, col) lives in 8-element column
// group (col / 8) ^ ((row / 8) % 8).  Rows stay 16-byte vectors for the row-wise side, and the
// 16-bit column-wise side finds rows 8 or 16 apart in different banks (the 144-byte pitch alone
// maps them to the same bank: 4- and 8-way conflicts).
__device__ __forceinline__ int swz_col(int row, int col) {
  return ((((col >> 3) ^ (row >> 3)) & 7) << 3) | (col & 7);
}

// One 64x64 tile of one weight.  Thread t: columns 8*(t%8)..+7, rows t/8 and t/8 + 32,
// 128-bit accesses.  Returns this thread's sum of squares of the bf16-rounded u values
// (added in element order: first row left to right, then the second row).
template <bool kGradF32>
__device__ __forceinline__ float momentum_tile(const MomW &w, int slot, uint16_t *xbase, int ti, int tj,
                                               float mu, int nesterov, uint16_t (*sm)[kTile + kPad]) {
  uint16_t *wx = xbase + (size_t)slot * w.K * w.N;
  const int c8 = (threadIdx.x & 7) * 8;
  const int r0 = threadIdx.x >> 3;
  const int col = tj * kTile + c8;
  // A weight stored in its Newton-Schulz orientation is a flat copy: its "tile" is 4096
  // contiguous elements (streams like a memcpy).  A tall weight needs 64x64 tiles for the
  // transposed store.
  const size_t flat0 = ((size_t)ti * (w.N / kTile) + tj) * (kTile * kTile) + (size_t)threadIdx.x * 8;
  float ss = 0.f;
  // both rows' loads are issued before the first store: the stores could alias the second row's
  // loads as far as the compiler knows, and a thread with 96 instead of 48 bytes in flight is
  // what keeps HBM busy
  size_t idxs[2];
  float4 b0s[2], b1s[2];
  float gs[2][8];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int rl = r0 + 32 * k;
    const size_t idx = w.tr ? (size_t)(ti * kTile + rl) * w.N + col : flat0 + (size_t)k * (kThreads * 8);
    idxs[k] = idx;
    b0s[k] = __ldcs(reinterpret_cast<const float4 *>(w.buf + idx));
    b1s[k] = __ldcs(reinterpret_cast<const float4 *>(w.buf + idx) + 1);
    float *g = gs[k];
    if constexpr (kGradF32) {
      const float4 g0 = __ldcs(reinterpret_cast<const float4 *>((const float *)w.g + idx));
      const float4 g1 = __ldcs(reinterpret_cast<const float4 *>((const float *)w.g + idx) + 1);
      g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
    } else {
      const uint4 gv = __ldcs(reinterpret_cast<const uint4 *>((const uint16_t *)w.g + idx));
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        g[2 * j] = __uint_as_float(gw[j] << 16);
        g[2 * j + 1] = __uint_as_float(gw[j] & 0xFFFF0000u);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int rl = r0 + 32 * k;
    const size_t idx = idxs[k];
    const float4 b0 = b0s[k], b1 = b1s[k];
    const float *g = gs[k];
    const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    float nb[8];
    uint32_t h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      nb[j] = __fadd_rn(__fmul_rn(mu, bb[j]), g[j]);
      const float u = nesterov ? __fadd_rn(g[j], __fmul_rn(mu, nb[j])) : nb[j];
      h[j] = rne16(u);
      const float ur = bf16_f32(h[j]);
      ss = __fadd_rn(ss, __fmul_rn(ur, ur));
    }
    __stcs(reinterpret_cast<float4 *>(w.buf + idx), make_float4(nb[0], nb[1], nb[2], nb[3]));
    __stcs(reinterpret_cast<float4 *>(w.buf + idx) + 1, make_float4(nb[4], nb[5], nb[6], nb[7]));
    const uint4 pk = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16),
                                h[6] | (h[7] << 16));
    if (!w.tr) *reinterpret_cast<uint4 *>(wx + idx) = pk;
    else *reinterpret_cast<uint4 *>(&sm[rl][swz_col(rl, c8)]) = pk;
  }
  if (w.tr) {
    __syncthreads();
    // output tile: rows = source columns, cols = source rows.  Thread: row t/4, 16 elems.
    const int oc = threadIdx.x >> 2;
    const int rr = (threadIdx.x & 3) * 16;
    uint32_t pk[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int ra = rr + 2 * j;               // ra and ra + 1 share one swizzle
      const int sc = swz_col(ra, oc);
      pk[j] = (uint32_t)sm[ra][sc] | ((uint32_t)sm[ra + 1][sc] << 16);
    }
    uint16_t *dst = wx + (size_t)(tj * kTile + oc) * w.K + (size_t)ti * kTile + rr;
    reinterpret_cast<uint4 *>(dst)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    reinterpret_cast<uint4 *>(dst)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    __syncthreads();
  }
  return ss;
}

__device__ __forceinline__ void update_tile(const UpdW &w, int slot, const uint16_t *obase, float lr_scale,
                                            int ti, int tj, uint16_t (*sm)[kTile + kPad]) {
  const uint16_t *wo = obase + (size_t)slot * w.K * w.N;
  const int c8 = (threadIdx.x & 7) * 8;
  const int r0 = threadIdx.x >> 3;
  const int col = tj * kTile + c8;
  const size_t flat0 = ((size_t)ti * (w.N / kTile) + tj) * (kTile * kTile) + (size_t)threadIdx.x * 8;
  // all global loads of both rows before the first store (see momentum_tile)
  size_t idxs[2];
  float4 p0s[2], p1s[2];
  uint4 ovs[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int rl = r0 + 32 * k;
    const size_t idx = w.tr ? (size_t)(ti * kTile + rl) * w.N + col : flat0 + (size_t)k * (kThreads * 8);
    idxs[k] = idx;
    p0s[k] = __ldcs(reinterpret_cast<const float4 *>(w.p32 + idx));
    p1s[k] = __ldcs(reinterpret_cast<const float4 *>(w.p32 + idx) + 1);
    if (!w.tr) ovs[k] = *reinterpret_cast<const uint4 *>(wo + idx);
  }
  if (w.tr) {
    // stage O^T tile: source rows = columns of the weight tile
    const int oc = threadIdx.x >> 2;
    const int rr = (threadIdx.x & 3) * 16;
    const uint16_t *src = wo + (size_t)(tj * kTile + oc) * w.K + (size_t)ti * kTile + rr;
    const uint4 a = reinterpret_cast<const uint4 *>(src)[0];
    const uint4 b = reinterpret_cast<const uint4 *>(src)[1];
    *reinterpret_cast<uint4 *>(&sm[oc][swz_col(oc, rr)]) = a;
    *reinterpret_cast<uint4 *>(&sm[oc][swz_col(oc, rr + 8)]) = b;
    __syncthreads();
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int rl = r0 + 32 * k;
    const size_t idx = idxs[k];
    const float4 p0 = p0s[k], p1 = p1s[k];
    float o[8];
    if (!w.tr) {
      const uint4 ov = ovs[k];
      const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[2 * j] = __uint_as_float(ow[j] << 16);
        o[2 * j + 1] = __uint_as_float(ow[j] & 0xFFFF0000u);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = bf16_f32(sm[c8 + j][swz_col(c8 + j, rl)]);
    }
    const float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    float pn[8];
    uint32_t h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      pn[j] = __fsub_rn(pp[j], __fmul_rn(lr_scale, o[j]));
      h[j] = rne16(pn[j]);
    }
    __stcs(reinterpret_cast<float4 *>(w.p32 + idx), make_float4(pn[0], pn[1], pn[2], pn[3]));
    __stcs(reinterpret_cast<float4 *>(w.p32 + idx) + 1, make_float4(pn[4], pn[5], pn[6], pn[7]));
    *reinterpret_cast<uint4 *>(w.p16 + idx) = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16),
                                                         h[4] | (h[5] << 16), h[6] | (h[7] << 16));
  }
  if (w.tr) __syncthreads();
}

__device__ __forceinline__ float warp_tree_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// recip[e] = 1 / (sqrt(sum of the matrix's tile sums) + eps): one CTA per matrix.  The momentum
// kernel leaves eight warp sums per 64x64 tile; a tile's sum is those eight added in warp order,
// the matrix's sum the tile sums added thread-strided in index order, then the fixed tree.
__global__ void __launch_bounds__(kThreads)
fro_finalize_kernel(const float *__restrict__ partial, float *__restrict__ recip, int per_matrix,
                    int warp_sums, float eps, uint32_t *sched) {
  __shared__ float wsum[kThreads / 32];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (sched != nullptr && threadIdx.x == 0) {
    // scheduler words of the chain kernel that follows: tile counter, abort word, one
    // completion counter per matrix
    sched[2 + blockIdx.x] = 0u;
    if (blockIdx.x == 0) {
      sched[0] = 0u;
      sched[1] = 0u;
    }
  }
  float acc = 0.f;
  if (!warp_sums) {   // one value per block of the matrix (fro_partial_kernel)
    const float *p1 = partial + (size_t)blockIdx.x * per_matrix;
    for (int k = threadIdx.x; k < per_matrix; k += kThreads) acc = __fadd_rn(acc, p1[k]);
  }
  const float4 *pp = reinterpret_cast<const float4 *>(partial) + (size_t)blockIdx.x * per_matrix * 2;
  for (int k = threadIdx.x; warp_sums && k < per_matrix; k += kThreads) {
    const float4 a = pp[2 * k], b = pp[2 * k + 1];
    float t = __fadd_rn(a.x, a.y);
    t = __fadd_rn(t, a.z);
    t = __fadd_rn(t, a.w);
    t = __fadd_rn(t, b.x);
    t = __fadd_rn(t, b.y);
    t = __fadd_rn(t, b.z);
    t = __fadd_rn(t, b.w);
    acc = __fadd_rn(acc, t);
  }
  acc = warp_tree_sum_f(acc);
  if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = wsum[0];
#pragma unroll
    for (int k = 1; k < kThreads / 32; ++k) t = __fadd_rn(t, wsum[k]);
    recip[blockIdx.x] = __fdiv_rn(1.0f, __fadd_rn(__fsqrt_rn(t), eps));
  }
}

// ---- the two table-driven sweeps fed by a staging ring ------------------------------------
// One CTA per SM: the first lane of the last warp walks this CTA's tiles (blockIdx.x, + gridDim.x, ...) and
// fills a ring of stages several tiles ahead: a flat tile is one untiled bulk copy per array, a tile
// of a tall weight one 64x64 box per array through the weight's tensor maps (64 row-sized bulk
// copies per array instead ran at a third of the speed: the copy engine takes about 60 cycles per
// request whatever its size); one or two groups of eight computing warps take the stages in turn: wait for a
// stage, take their 16 elements from shared memory, hand the stage back, and compute and store
// from registers with the arithmetic of momentum_tile / update_tile (the single-weight kernels).
// Every weight in the table has the same K*N, hence the same number of tiles (tiles_per_w); tile b
// belongs to weight b / tiles_per_w.  lr_scale_wide applies to weights stored with K <= N,
// lr_scale_tall to K > N (lr * sqrt(max(1, K/N)), ancora/optim/muon.py:101,176).
// groups of 256 computing threads taking the stages in turn
constexpr int kMomGroups = 2;                 // measured: momentum 0.97 against 1.02 ms per step with two groups,
constexpr int kUpdGroups = 1;                 //           update 0.90 against 0.93 ms with one
constexpr int kRingHdr = 128;                 // table entry + tile coordinates travel with the stage
constexpr int kTileElems = kTile * kTile;
template <int kBytesPerElem>
struct TileRing {
  static constexpr uint32_t kStageBytes = kRingHdr + kTileElems * kBytesPerElem;
  static constexpr int kStages = (int)((200u * 1024u) / kStageBytes) > 7 ? 7 : (int)((200u * 1024u) / kStageBytes);
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 128;   // + room to align the base
};
__device__ __forceinline__ uint8_t *ring_base(uint8_t *raw) {
  return raw + ((128u - (anc_ring::smem_u32(raw) & 127u)) & 127u);   // box loads want 128-byte aligned stages
}

template <bool kGradF32, int kGroups>
__global__ void __launch_bounds__(kGroups * kThreads + 32, 1)
momentum_ring_kernel(const MomW *__restrict__ table, const anc_tmap *__restrict__ maps, uint16_t *xbase, int n_w,
                     int tiles_per_w, float mu, int nesterov, float *__restrict__ partial, uint32_t *status) {
  using R = TileRing<kGradF32 ? 8 : 6>;
  constexpr uint32_t kGB = kGradF32 ? 4u : 2u;
  extern __shared__ __align__(128) uint8_t ring_raw[];
  uint8_t *ring = ring_base(ring_raw);
  __shared__ __align__(16) uint16_t sm2[kGroups][kTile][kTile + kPad];
  __shared__ __align__(8) uint64_t bars[2 * R::kStages];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // the packed operand may still be read by the previous launch
  const uint32_t full0 = anc_ring::smem_u32(&bars[0]), empty0 = anc_ring::smem_u32(&bars[R::kStages]);
  if (threadIdx.x == 0) {
    for (int i = 0; i < R::kStages; ++i) {
      anc_ring::mbar_init(full0 + 8 * i, 1);
      anc_ring::mbar_init(empty0 + 8 * i, kThreads / 32);
    }
    anc_ring::mbar_init_fence();
  }
  __syncthreads();
  const int total = n_w * tiles_per_w;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == kGroups * kThreads / 32) {
    if (lane != 0) return;
    uint32_t it = 0;
    int b = blockIdx.x;                                  // the grid never exceeds the tile count
    MomW nxt = table[b / tiles_per_w];
    for (; b < total; b += gridDim.x, ++it) {
      const MomW w = nxt;
      const int wi = b / tiles_per_w, t = b - wi * tiles_per_w;
      if (b + (int)gridDim.x < total) nxt = table[(b + (int)gridDim.x) / tiles_per_w];
      const uint32_t slot = it % R::kStages, ph = (it / R::kStages) & 1u;
      if (it >= (uint32_t)R::kStages && !anc_ring::mbar_wait(empty0 + 8 * slot, ph ^ 1u)) {
        atomicOr(status, ANC_DEV_TIMEOUT_TMA);
        anc_ring::drain_issued<R::kStages>(full0, it);
        return;
      }
      const int tn = w.N / kTile, ti = t / tn, tj = t - ti * tn;
      uint8_t *st = ring + (size_t)slot * R::kStageBytes;
      const uint32_t bar = full0 + 8 * slot;
      *reinterpret_cast<MomW *>(st) = w;
      *reinterpret_cast<int4 *>(st + 32) = make_int4(wi, t, ti, tj);
      anc_ring::mbar_expect_tx(bar, kTileElems * (4u + kGB));
      const uint32_t db = anc_ring::smem_u32(st + kRingHdr), dg = db + kTileElems * 4u;
      if (!w.tr) {
        const size_t flat = (size_t)t * kTileElems;
        anc_ring::bulk_load(db, w.buf + flat, kTileElems * 4u, bar);
        anc_ring::bulk_load(dg, (const uint8_t *)w.g + flat * kGB, kTileElems * kGB, bar);
      } else {
        const anc_tmap *m = maps + 3 * (size_t)wi;
        anc_ring::box_load_2d(db, m, tj * kTile, ti * kTile, bar);
        anc_ring::box_load_2d(dg, m + 1, tj * kTile, ti * kTile, bar);
      }
    }
    return;
  }
  const int grp = warp / (kThreads / 32);                 // this warp's group of 256 threads
  const int tid = threadIdx.x & (kThreads - 1);           // thread within the group
  const int wig = warp & (kThreads / 32 - 1);             // warp within the group
  uint16_t (*sm)[kTile + kPad] = sm2[grp];
  const int c8 = (tid & 7) * 8;
  const int r0 = tid >> 3;
  uint32_t it = grp;
  for (int b = blockIdx.x + grp * (int)gridDim.x; b < total; b += kGroups * (int)gridDim.x, it += kGroups) {
    const uint32_t slot = it % R::kStages, ph = (it / R::kStages) & 1u;
    const bool gave_up = !anc_ring::mbar_wait(full0 + 8 * slot, ph);
    if (anc_ring::bar_compute_or(1 + grp, kThreads, gave_up)) {
      if (gave_up && lane == 0) atomicOr(status, ANC_DEV_TIMEOUT_TMA);
      return;
    }
    const uint8_t *st = ring + (size_t)slot * R::kStageBytes;
    const MomW w = *reinterpret_cast<const MomW *>(st);
    const int4 hv = *reinterpret_cast<const int4 *>(st + 32);
    const int wi = hv.x, t = hv.y, ti = hv.z, tj = hv.w;
    float bb[2][8], gg[2][8];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const float *sb = reinterpret_cast<const float *>(st + kRingHdr) + k * (kThreads * 8);
      anc_ring::ld8(sb, tid, lane, bb[k]);
      if constexpr (kGradF32)
        anc_ring::ld8(reinterpret_cast<const float *>(st + kRingHdr + kTileElems * 4) + k * (kThreads * 8),
                      tid, lane, gg[k]);
      else
        anc_ring::ld8_bf16(reinterpret_cast<const uint16_t *>(st + kRingHdr + kTileElems * 4) + k * (kThreads * 8),
                           tid, gg[k]);
    }
    __syncwarp();
    if (lane == 0) anc_ring::mbar_arrive(empty0 + 8 * slot);
    uint16_t *wx = xbase + (size_t)wi * w.K * w.N;
    const size_t flat0 = (size_t)t * kTileElems + (size_t)tid * 8;
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int rl = r0 + 32 * k;
      const size_t idx = w.tr ? (size_t)(ti * kTile + rl) * w.N + (size_t)tj * kTile + c8
                              : flat0 + (size_t)k * (kThreads * 8);
      float nb[8];
      uint32_t h[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        nb[j] = __fadd_rn(__fmul_rn(mu, bb[k][j]), gg[k][j]);
        const float u = nesterov ? __fadd_rn(gg[k][j], __fmul_rn(mu, nb[j])) : nb[j];
        h[j] = rne16(u);
        const float ur = bf16_f32(h[j]);
        ss = __fadd_rn(ss, __fmul_rn(ur, ur));
      }
      __stcs(reinterpret_cast<float4 *>(w.buf + idx), make_float4(nb[0], nb[1], nb[2], nb[3]));
      __stcs(reinterpret_cast<float4 *>(w.buf + idx) + 1, make_float4(nb[4], nb[5], nb[6], nb[7]));
      const uint4 pk = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16),
                                  h[6] | (h[7] << 16));
      if (!w.tr) *reinterpret_cast<uint4 *>(wx + idx) = pk;
      else *reinterpret_cast<uint4 *>(&sm[rl][swz_col(rl, c8)]) = pk;
    }
    if (w.tr) {
      anc_ring::bar_compute(1 + grp, kThreads);
      const int oc = tid >> 2;
      const int rr = (tid & 3) * 16;
      uint32_t pk[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int ra = rr + 2 * j;
        const int sc = swz_col(ra, oc);
        pk[j] = (uint32_t)sm[ra][sc] | ((uint32_t)sm[ra + 1][sc] << 16);
      }
      uint16_t *dst = wx + (size_t)(tj * kTile + oc) * w.K + (size_t)ti * kTile + rr;
      reinterpret_cast<uint4 *>(dst)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      reinterpret_cast<uint4 *>(dst)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      // the next tile's vote barrier keeps its writes to the transposition tile behind these reads
    }
    if (partial) {
      // partial[(slot * tiles_per_w + tile) * 8 + warp]: the warp's sum of squares of its bf16 u values
      // (thread sums in element order, then the shuffle tree); the finalize kernel adds the eight
      ss = warp_tree_sum_f(ss);
      if (lane == 0) partial[((size_t)wi * tiles_per_w + t) * 8 + wig] = ss;
    }
  }
}

template <int kGroups>
__global__ void __launch_bounds__(kGroups * kThreads + 32, 1)
update_ring_kernel(const UpdW *__restrict__ table, const anc_tmap *__restrict__ maps,
                   const __grid_constant__ anc_tmap omap, const uint16_t *obase, int n_w, int tiles_per_w,
                   float lr_scale_wide, float lr_scale_tall, uint32_t *status) {
  using R = TileRing<6>;
  extern __shared__ __align__(128) uint8_t ring_raw[];
  uint8_t *ring = ring_base(ring_raw);
  __shared__ __align__(16) uint16_t sm2[kGroups][kTile][kTile + kPad];
  __shared__ __align__(8) uint64_t bars[2 * R::kStages];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t full0 = anc_ring::smem_u32(&bars[0]), empty0 = anc_ring::smem_u32(&bars[R::kStages]);
  if (threadIdx.x == 0) {
    for (int i = 0; i < R::kStages; ++i) {
      anc_ring::mbar_init(full0 + 8 * i, 1);
      anc_ring::mbar_init(empty0 + 8 * i, kThreads / 32);
    }
    anc_ring::mbar_init_fence();
  }
  __syncthreads();
  const int total = n_w * tiles_per_w;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == kGroups * kThreads / 32) {
    if (lane != 0) return;
    uint32_t it = 0;
    int b = blockIdx.x;
    UpdW nxt = table[b / tiles_per_w];
    for (; b < total; b += gridDim.x, ++it) {
      const UpdW w = nxt;
      const int wi = b / tiles_per_w, t = b - wi * tiles_per_w;
      if (b + (int)gridDim.x < total) nxt = table[(b + (int)gridDim.x) / tiles_per_w];
      const uint32_t slot = it % R::kStages, ph = (it / R::kStages) & 1u;
      if (it >= (uint32_t)R::kStages && !anc_ring::mbar_wait(empty0 + 8 * slot, ph ^ 1u)) {
        atomicOr(status, ANC_DEV_TIMEOUT_TMA);
        anc_ring::drain_issued<R::kStages>(full0, it);
        return;
      }
      const int tn = w.N / kTile, ti = t / tn, tj = t - ti * tn;
      uint8_t *st = ring + (size_t)slot * R::kStageBytes;
      const uint32_t bar = full0 + 8 * slot;
      *reinterpret_cast<UpdW *>(st) = w;
      *reinterpret_cast<int4 *>(st + 32) = make_int4(wi, t, ti, tj);
      anc_ring::mbar_expect_tx(bar, kTileElems * 6u);
      const uint32_t dp = anc_ring::smem_u32(st + kRingHdr), dO = dp + kTileElems * 4u;
      if (!w.tr) {
        const size_t flat = (size_t)t * kTileElems;
        anc_ring::bulk_load(dp, w.p32 + flat, kTileElems * 4u, bar);
        anc_ring::bulk_load(dO, obase + (size_t)wi * w.K * w.N + flat, kTileElems * 2u, bar);
      } else {
        // the weight's tile, and the same tile of O^T: its rows are the tile's columns
        anc_ring::box_load_2d(dp, maps + 3 * (size_t)wi + 2, tj * kTile, ti * kTile, bar);
        anc_ring::box_load_3d(dO, &omap, ti * kTile, tj * kTile, wi, bar);
      }
    }
    return;
  }
  const int grp = warp / (kThreads / 32);                 // this warp's group of 256 threads
  const int tid = threadIdx.x & (kThreads - 1);           // thread within the group
  uint16_t (*sm)[kTile + kPad] = sm2[grp];
  const int c8 = (tid & 7) * 8;
  const int r0 = tid >> 3;
  uint32_t it = grp;
  for (int b = blockIdx.x + grp * (int)gridDim.x; b < total; b += kGroups * (int)gridDim.x, it += kGroups) {
    const uint32_t slot = it % R::kStages, ph = (it / R::kStages) & 1u;
    const bool gave_up = !anc_ring::mbar_wait(full0 + 8 * slot, ph);
    if (anc_ring::bar_compute_or(1 + grp, kThreads, gave_up)) {
      if (gave_up && lane == 0) atomicOr(status, ANC_DEV_TIMEOUT_TMA);
      return;
    }
    const uint8_t *st = ring + (size_t)slot * R::kStageBytes;
    const UpdW w = *reinterpret_cast<const UpdW *>(st);
    const int4 hv = *reinterpret_cast<const int4 *>(st + 32);
    const int t = hv.y, ti = hv.z, tj = hv.w;
    const float lr_scale = w.tr ? lr_scale_tall : lr_scale_wide;
    float pp[2][8], oo[2][8];
    const uint16_t *sO = reinterpret_cast<const uint16_t *>(st + kRingHdr + kTileElems * 4);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      anc_ring::ld8(reinterpret_cast<const float *>(st + kRingHdr) + k * (kThreads * 8), tid, lane, pp[k]);
      if (!w.tr) anc_ring::ld8_bf16(sO + k * (kThreads * 8), tid, oo[k]);
    }
    if (w.tr) {
      // staged O^T tile (row oc = the weight tile's column oc) into the swizzled transposition tile
      const int oc = tid >> 2;
      const int rr = (tid & 3) * 16;
      const int sw = (lane >> 2) & 1;
      const uint4 *q = reinterpret_cast<const uint4 *>(sO + oc * kTile + rr);
      const uint4 a = q[sw], c = q[sw ^ 1];
      *reinterpret_cast<uint4 *>(&sm[oc][swz_col(oc, rr + 8 * sw)]) = a;
      *reinterpret_cast<uint4 *>(&sm[oc][swz_col(oc, rr + 8 * (sw ^ 1))]) = c;
    }
    __syncwarp();
    if (lane == 0) anc_ring::mbar_arrive(empty0 + 8 * slot);
    if (w.tr) {
      anc_ring::bar_compute(1 + grp, kThreads);
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int rl = r0 + 32 * k;
#pragma unroll
        for (int j = 0; j < 8; ++j) oo[k][j] = bf16_f32(sm[c8 + j][swz_col(c8 + j, rl)]);
      }
    }
    const size_t flat0 = (size_t)t * kTileElems + (size_t)tid * 8;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int rl = r0 + 32 * k;
      const size_t idx = w.tr ? (size_t)(ti * kTile + rl) * w.N + (size_t)tj * kTile + c8
                              : flat0 + (size_t)k * (kThreads * 8);
      float pn[8];
      uint32_t h[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        pn[j] = __fsub_rn(pp[k][j], __fmul_rn(lr_scale, oo[k][j]));
        h[j] = rne16(pn[j]);
      }
      __stcs(reinterpret_cast<float4 *>(w.p32 + idx), make_float4(pn[0], pn[1], pn[2], pn[3]));
      __stcs(reinterpret_cast<float4 *>(w.p32 + idx) + 1, make_float4(pn[4], pn[5], pn[6], pn[7]));
      *reinterpret_cast<uint4 *>(w.p16 + idx) = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16),
                                                           h[4] | (h[5] << 16), h[6] | (h[7] << 16));
    }
    // the next tile's vote barrier keeps its writes to the transposition tile behind these reads
  }
}

// A stage nobody fills, waited for the way the ring's computing warps do: the bounded wait runs out, the
// warps agree on it at their barrier, one of them records it and all return.
__global__ void __launch_bounds__(kThreads)
ring_wait_selftest_kernel(uint32_t tries, uint32_t *status) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t full = anc_ring::smem_u32(&bar);
  if (threadIdx.x == 0) {
    anc_ring::mbar_init(full, 1);
    anc_ring::mbar_init_fence();
  }
  __syncthreads();
  const bool gave_up = !anc_ring::mbar_wait(full, 0, tries);
  if (anc_ring::bar_compute_or(1, kThreads, gave_up)) {
    if (gave_up && (threadIdx.x & 31) == 0) atomicOr(status, ANC_DEV_TIMEOUT_TMA);
    return;
  }
}

// ---- update with post-step consumers fused in ---------------------------------------------
// Optional extra outputs of the update, produced from the freshly rounded bf16 weight while it is
// still on chip (the reference runs them as separate sweeps after every optimizer step):
//   fp8 + scale : MXFP8 re-quantisation, blocks of 32 along K (rows), E8M0 scale byte =
//                 max(exponent(amax) - 7, 0), value = RNE_e4m3(w / 2^(byte-127))
//                 (ancora/kernels/quant.py:56-68 `_quant_mxfp8_w`; layout (K,N) u8 + (K/32,N) u8)
//   p16_t       : the transposed bf16 copy (N,K) a backward pass reads
//                 (ancora/kernels/moe.py:371-377 `_transpose_e`)
//   fp8_t + scale_t : the same MXFP8 bytes in the transposed layout a column-major B operand
//                 wants, (N,K) u8 + (N,K/32) u8 (ancora/kernels/quant.py:79-90 `_quant_mxfp8_w_cm`)
struct UpdX {
  uint8_t *fp8;
  uint8_t *scale;
  uint16_t *p16_t;
  uint8_t *fp8_t;
  uint8_t *scale_t;
  int64_t _pad;
};
constexpr int kQPad = 16;   // row pad of the byte staging tile (keeps rows 16-byte aligned)

__device__ __forceinline__ uint32_t e4m3_rn(float x) {
  // cvt.rn.satfinite.e4m3x2.f32 packs two values; the high one is zero here
  uint16_t r;
  asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %1, %2;\n\tmov.b16 %0, t;\n\t}" : "=h"(r) : "f"(0.f), "f"(x));
  return (uint32_t)(r & 0xFF);
}

// 64x64 tile, same thread mapping as update_tile (8 columns x rows r0, r0+32): the two rows of a
// thread fall into the tile's two 32-row quantisation blocks.
__device__ __forceinline__ void update_tile_extras(const UpdW &w, const UpdX &x, int slot,
                                                   const uint16_t *obase, float lr_scale, int ti, int tj,
                                                   uint16_t (*sm)[kTile + kPad], uint32_t (*wmax)[2][kTile],
                                                   uint8_t (*sbyte)[kTile], uint8_t (*sq)[kTile + kQPad]) {
  const uint16_t *wo = obase + (size_t)slot * w.K * w.N;
  const bool want_q = x.fp8 != nullptr || x.fp8_t != nullptr;
  const int c8 = (threadIdx.x & 7) * 8;
  const int r0 = threadIdx.x >> 3;
  const int col = tj * kTile + c8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (w.tr) {
    const int oc = threadIdx.x >> 2;
    const int rr = (threadIdx.x & 3) * 16;
    const uint16_t *src = wo + (size_t)(tj * kTile + oc) * w.K + (size_t)ti * kTile + rr;
    *reinterpret_cast<uint4 *>(&sm[oc][swz_col(oc, rr)]) = reinterpret_cast<const uint4 *>(src)[0];
    *reinterpret_cast<uint4 *>(&sm[oc][swz_col(oc, rr + 8)]) = reinterpret_cast<const uint4 *>(src)[1];
    __syncthreads();
  }
  uint32_t h[2][8];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int rl = r0 + 32 * k;
    const size_t idx = (size_t)(ti * kTile + rl) * w.N + col;
    const float4 p0 = __ldcs(reinterpret_cast<const float4 *>(w.p32 + idx));
    const float4 p1 = __ldcs(reinterpret_cast<const float4 *>(w.p32 + idx) + 1);
    float o[8];
    if (!w.tr) {
      const uint4 ov = *reinterpret_cast<const uint4 *>(wo + idx);
      const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[2 * j] = __uint_as_float(ow[j] << 16);
        o[2 * j + 1] = __uint_as_float(ow[j] & 0xFFFF0000u);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = bf16_f32(sm[c8 + j][swz_col(c8 + j, rl)]);
    }
    const float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    float pn[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      pn[j] = __fsub_rn(pp[j], __fmul_rn(lr_scale, o[j]));
      h[k][j] = rne16(pn[j]);
    }
    __stcs(reinterpret_cast<float4 *>(w.p32 + idx), make_float4(pn[0], pn[1], pn[2], pn[3]));
    __stcs(reinterpret_cast<float4 *>(w.p32 + idx) + 1, make_float4(pn[4], pn[5], pn[6], pn[7]));
    *reinterpret_cast<uint4 *>(w.p16 + idx) = make_uint4(h[k][0] | (h[k][1] << 16), h[k][2] | (h[k][3] << 16),
                                                         h[k][4] | (h[k][5] << 16), h[k][6] | (h[k][7] << 16));
  }
  __syncthreads();                       // every thread is done reading the staged O^T tile
  if (x.p16_t) {
#pragma unroll
    for (int k = 0; k < 2; ++k)
      *reinterpret_cast<uint4 *>(&sm[r0 + 32 * k][swz_col(r0 + 32 * k, c8)]) =
          make_uint4(h[k][0] | (h[k][1] << 16), h[k][2] | (h[k][3] << 16), h[k][4] | (h[k][5] << 16),
                     h[k][6] | (h[k][7] << 16));
  }
  if (want_q) {
    // column maxima of |w| per 32-row block: 4 rows per warp by shuffles, 8 warps through smem
#pragma unroll
    for (int k = 0; k < 2; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t a = h[k][j] & 0x7FFFu;                 // |bf16| bits order like the magnitudes
        a = max(a, __shfl_xor_sync(0xFFFFFFFFu, a, 8));
        a = max(a, __shfl_xor_sync(0xFFFFFFFFu, a, 16));
        if (lane < 8) wmax[warp][k][c8 + j] = a;
      }
  }
  __syncthreads();
  if (want_q && threadIdx.x < 2 * kTile) {
    const int k = threadIdx.x >> 6, c = threadIdx.x & 63;
    uint32_t a = wmax[0][k][c];
#pragma unroll
    for (int q = 1; q < kThreads / 32; ++q) a = max(a, wmax[q][k][c]);
    const uint32_t ea = (a >> 7) & 0xFF;                // exponent field of the bf16 = of the float
    const uint32_t byte = ea >= 7 ? ea - 7 : 0;
    sbyte[k][c] = (uint8_t)byte;
    if (x.fp8) x.scale[((size_t)(ti * 2 + k)) * w.N + (size_t)tj * kTile + c] = (uint8_t)byte;
    if (x.fp8_t) x.scale_t[((size_t)tj * kTile + c) * (size_t)(w.K / 32) + (size_t)(ti * 2 + k)] = (uint8_t)byte;
  }
  if (x.p16_t) {
    // transposed store of the bf16 tile: thread handles output row t/4, 16 elements
    const int oc = threadIdx.x >> 2;
    const int rr = (threadIdx.x & 3) * 16;
    uint32_t pk[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int ra = rr + 2 * j;
      const int sc = swz_col(ra, oc);
      pk[j] = (uint32_t)sm[ra][sc] | ((uint32_t)sm[ra + 1][sc] << 16);
    }
    uint16_t *dst = x.p16_t + (size_t)(tj * kTile + oc) * w.K + (size_t)ti * kTile + rr;
    reinterpret_cast<uint4 *>(dst)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    reinterpret_cast<uint4 *>(dst)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
  }
  __syncthreads();
  if (want_q) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      uint32_t q[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t byte = sbyte[k][c8 + j];
        const float inv = __uint_as_float((254u - byte) << 23);      // 2^(127 - byte), exact
        q[j] = e4m3_rn(__fmul_rn(bf16_f32(h[k][j]), inv));
      }
      const uint2 packed =
          make_uint2(q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24), q[4] | (q[5] << 8) | (q[6] << 16) | (q[7] << 24));
      if (x.fp8) {
        const size_t idx = (size_t)(ti * kTile + r0 + 32 * k) * w.N + col;
        *reinterpret_cast<uint2 *>(x.fp8 + idx) = packed;
      }
      if (x.fp8_t) *reinterpret_cast<uint2 *>(&sq[r0 + 32 * k][c8]) = packed;
    }
  }
  if (x.fp8_t) {
    // transposed store of the byte tile: thread handles output row t/4 (a column of the weight),
    // 16 consecutive K positions
    __syncthreads();
    const int oc = threadIdx.x >> 2;
    const int rr = (threadIdx.x & 3) * 16;
    uint32_t pk[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      pk[j] = (uint32_t)sq[rr + 4 * j][oc] | ((uint32_t)sq[rr + 4 * j + 1][oc] << 8) |
              ((uint32_t)sq[rr + 4 * j + 2][oc] << 16) | ((uint32_t)sq[rr + 4 * j + 3][oc] << 24);
    uint8_t *dst = x.fp8_t + (size_t)(tj * kTile + oc) * w.K + (size_t)ti * kTile + rr;
    *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kThreads)
update_extras_kernel(const UpdW *__restrict__ table, const UpdX *__restrict__ extras, const uint16_t *obase,
                     int n_w, int tiles_per_w, float lr_scale_wide, float lr_scale_tall) {
  __shared__ __align__(16) uint16_t sm[kTile][kTile + kPad];
  __shared__ uint32_t wmax[kThreads / 32][2][kTile];
  __shared__ uint8_t sbyte[2][kTile];
  __shared__ __align__(16) uint8_t sq[kTile][kTile + kQPad];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int total = n_w * tiles_per_w;
  for (int b = blockIdx.x; b < total; b += gridDim.x) {
    const int wi = b / tiles_per_w;
    const int t = b - wi * tiles_per_w;
    const UpdW w = table[wi];
    const UpdX x = extras[wi];
    const int tn = w.N / kTile;
    update_tile_extras(w, x, wi, obase, w.tr ? lr_scale_tall : lr_scale_wide, t / tn, t % tn, sm, wmax, sbyte, sq);
  }
}

// single-weight forms (table passed by value)
template <bool kGradF32>
__global__ void __launch_bounds__(kThreads)
momentum_one_kernel(MomW w, uint16_t *xbase, float mu, int nesterov) {
  __shared__ __align__(16) uint16_t sm[kTile][kTile + kPad];
  const int tn = w.N / kTile;
  const int total = (w.K / kTile) * tn;
  for (int t = blockIdx.x; t < total; t += gridDim.x)
    (void)momentum_tile<kGradF32>(w, 0, xbase, t / tn, t % tn, mu, nesterov, sm);
}

__global__ void __launch_bounds__(kThreads)
update_one_kernel(UpdW w, const uint16_t *obase, float lr_scale) {
  __shared__ __align__(16) uint16_t sm[kTile][kTile + kPad];
  const int tn = w.N / kTile;
  const int total = (w.K / kTile) * tn;
  for (int t = blockIdx.x; t < total; t += gridDim.x)
    update_tile(w, 0, obase, lr_scale, t / tn, t % tn, sm);
}

// ---- Frobenius normalisation ------------------------------------------------
// Each matrix is cut into blocks of kFroBlock contiguous elements.  Level 1: one
// CTA per block; a thread adds its 64 squares in index order, a warp combines with a
// xor-shuffle tree, warp 0 adds the 8 warp sums in order.  Level 2 (inside the scale
// kernel): the per-block sums of one matrix are added by one warp, lane-strided then
// the same shuffle tree.  The order never depends on the grid or on which other
// matrices share the launch.
constexpr int kFroBlock = 16384;

__device__ __forceinline__ float warp_tree_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

__global__ void __launch_bounds__(kThreads)
fro_partial_kernel(const uint16_t *__restrict__ X, float *__restrict__ partial, int total_blocks) {
  __shared__ float wsum[kThreads / 32];
  for (int b = blockIdx.x; b < total_blocks; b += gridDim.x) {
    const uint4 *src = reinterpret_cast<const uint4 *>(X + (size_t)b * kFroBlock);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < kFroBlock / (kThreads * 8); ++k) {
      const uint4 r = src[k * kThreads + threadIdx.x];
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
        acc = __fadd_rn(acc, __fmul_rn(lo, lo));
        acc = __fadd_rn(acc, __fmul_rn(hi, hi));
      }
    }
    acc = warp_tree_sum(acc);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = wsum[0];
#pragma unroll
      for (int k = 1; k < kThreads / 32; ++k) s = __fadd_rn(s, wsum[k]);
      partial[b] = s;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kThreads)
fro_scale_kernel(uint16_t *__restrict__ X, const float *__restrict__ partial,
                 float *__restrict__ recip, int blocks_per_matrix, int total_blocks, float eps) {
  __shared__ float s_r;
  for (int b = blockIdx.x; b < total_blocks; b += gridDim.x) {
    const int e = b / blocks_per_matrix;
    if (threadIdx.x < 32) {
      const float *pp = partial + (size_t)e * blocks_per_matrix;
      float acc = 0.f;
      for (int k = threadIdx.x; k < blocks_per_matrix; k += 32) acc = __fadd_rn(acc, pp[k]);
      acc = warp_tree_sum(acc);
      if (threadIdx.x == 0) {
        const float r = __fdiv_rn(1.0f, __fadd_rn(__fsqrt_rn(acc), eps));
        s_r = r;
        if (b - e * blocks_per_matrix == 0) recip[e] = r;
      }
    }
    __syncthreads();
    const float r = s_r;
    uint4 *dst = reinterpret_cast<uint4 *>(X + (size_t)b * kFroBlock);
#pragma unroll
    for (int k = 0; k < kFroBlock / (kThreads * 8); ++k) {
      uint4 v = dst[k * kThreads + threadIdx.x];
      uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __fmul_rn(__uint_as_float(w[j] << 16), r);
        const float hi = __fmul_rn(__uint_as_float(w[j] & 0xFFFF0000u), r);
        w[j] = rne16(lo) | (rne16(hi) << 16);
      }
      dst[k * kThreads + threadIdx.x] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    __syncthreads();
  }
}

}  // namespace

// ---- launchers -----------------------------------------------------------------

static int check_shape(int K, int N) {
  ANC_REQUIRE(K > 0 && N > 0 && K % 64 == 0 && N % 64 == 0,
              "Muon weight (%d,%d) tile-misaligned: K and N must be multiples of 64", K, N);
  return ANC_OK;
}

int anc_launch_momentum(anc_ctx *ctx, float *buf, const void *g, int grad_dtype, uint16_t *u, int K,
                        int N, float momentum, int nesterov, int transposed, cudaStream_t st) {
  int rc = check_shape(K, N);
  if (rc) return rc;
  MomW w = {buf, g, K, N, transposed ? 1 : 0, 0};
  int tiles = (K / kTile) * (N / kTile);
  int grid = tiles < ctx->sm_count * 8 ? tiles : ctx->sm_count * 8;
  if (grad_dtype == ANC_GRAD_F32)
    momentum_one_kernel<true><<<grid, kThreads, 0, st>>>(w, u, momentum, nesterov);
  else
    momentum_one_kernel<false><<<grid, kThreads, 0, st>>>(w, u, momentum, nesterov);
  ANC_CUDA(cudaGetLastError());
  return ANC_OK;
}

int anc_launch_update(anc_ctx *ctx, float *p32, uint16_t *p16, const uint16_t *O, int K, int N,
                      float lr_scale, int transposed, cudaStream_t st) {
  int rc = check_shape(K, N);
  if (rc) return rc;
  UpdW w = {p32, p16, K, N, transposed ? 1 : 0, 0};
  int tiles = (K / kTile) * (N / kTile);
  int grid = tiles < ctx->sm_count * 8 ? tiles : ctx->sm_count * 8;
  update_one_kernel<<<grid, kThreads, 0, st>>>(w, O, lr_scale);
  ANC_CUDA(cudaGetLastError());
  return ANC_OK;
}

int anc_launch_fro_normalize(anc_ctx *ctx, uint16_t *X, float *recip, int E, int M, int N, float eps,
                             cudaStream_t st) {
  ANC_REQUIRE(E > 0 && M > 0 && N > 0, "bad shape");
  ANC_REQUIRE(((size_t)M * N) % kFroBlock == 0, "matrix of %dx%d elements is not a multiple of %d",
              M, N, kFroBlock);
  const int bpm = (int)(((size_t)M * N) / kFroBlock);
  const size_t total = (size_t)E * bpm;
  ANC_REQUIRE(total < (1u << 30), "too many blocks");
  if (total * sizeof(float) > ctx->work_bytes) {
    ANC_CUDA(cudaStreamSynchronize(st));
    ANC_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->d_work) cudaFree(ctx->d_work);
    ctx->d_work = nullptr;
    ctx->work_bytes = 0;          // stays 0 if the allocation fails, so the next call retries
    ANC_CUDA(cudaMalloc(&ctx->d_work, total * sizeof(float) * 2));
    ctx->work_bytes = total * sizeof(float) * 2;
  }
  int grid = (int)(total < (size_t)ctx->sm_count * 8 ? total : (size_t)ctx->sm_count * 8);
  fro_partial_kernel<<<grid, kThreads, 0, st>>>(X, (float *)ctx->d_work, (int)total);
  ANC_CUDA(cudaGetLastError());
  fro_scale_kernel<<<grid, kThreads, 0, st>>>(X, (const float *)ctx->d_work, recip, bpm, (int)total,
                                              eps);
  ANC_CUDA(cudaGetLastError());
  return ANC_OK;
}

// Table-driven group launches used by the Muon plan.
static_assert(sizeof(anc_mom_entry) == sizeof(MomW), "table layout");
static_assert(sizeof(anc_upd_entry) == sizeof(UpdW), "table layout");

// Launch with programmatic stream serialization (the kernels above wait with griddepcontrol).
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl_ex(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t st,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), int grid, cudaStream_t st, Args... args) {
  return launch_pdl_ex(kernel, grid, kThreads, 0, st, args...);
}

// The ring kernels' shared memory is above the default per-launch limit: raised once per device.
static cudaError_t ring_kernels_ready(int device) {
  static std::mutex mu;
  static bool done[64] = {};
  std::lock_guard<std::mutex> lock(mu);
  if (device >= 0 && device < 64 && done[device]) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(momentum_ring_kernel<true, kMomGroups>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)TileRing<8>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(momentum_ring_kernel<false, kMomGroups>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)TileRing<6>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(update_ring_kernel<kUpdGroups>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)TileRing<6>::kSmemBytes);
  if (e == cudaSuccess && device >= 0 && device < 64) done[device] = true;
  return e;
}

// Called when a plan is created, so that the first step (which may run under stream capture) sets nothing.
int anc_elem_kernels_prepare(anc_ctx *ctx) {
  ANC_CUDA(ring_kernels_ready(ctx->device));
  return ANC_OK;
}

int anc_launch_fro_finalize(anc_ctx *ctx, const float *partial, float *recip, int E, int per_matrix,
                            int warp_sums, float eps, uint32_t *sched, cudaStream_t st) {
  (void)ctx;
  if (E <= 0) return ANC_OK;
  ANC_CUDA(launch_pdl(fro_finalize_kernel, E, st, partial, recip, per_matrix, warp_sums, eps, sched));
  return ANC_OK;
}

// Per-block sums of squares of packed bf16 matrices (blocks of 16384 elements) into `partial`.
int anc_launch_fro_partial(anc_ctx *ctx, const uint16_t *X, float *partial, int E, int M, int N,
                           cudaStream_t st) {
  const size_t total = (size_t)E * (((size_t)M * N) / kFroBlock);
  int grid = (int)(total < (size_t)ctx->sm_count * 8 ? total : (size_t)ctx->sm_count * 8);
  if (grid == 0) return ANC_OK;
  fro_partial_kernel<<<grid, kThreads, 0, st>>>(X, partial, (int)total);
  ANC_CUDA(cudaGetLastError());
  return ANC_OK;
}

int anc_launch_momentum_group(anc_ctx *ctx, const void *d_table, const anc_tmap *d_maps, uint16_t *xbase,
                              int n_w, int elems_per_w, int grad_dtype, float momentum, int nesterov,
                              float *partial, cudaStream_t st) {
  const int tpw = elems_per_w / (kTile * kTile);
  const long long total = (long long)n_w * tpw;
  int grid = (int)(total < (long long)ctx->sm_count ? total : (long long)ctx->sm_count);   // one CTA per SM
  if (grid == 0) return ANC_OK;
  ANC_CUDA(ring_kernels_ready(ctx->device));
  if (grad_dtype == ANC_GRAD_F32)
    ANC_CUDA(launch_pdl_ex(momentum_ring_kernel<true, kMomGroups>, grid, kMomGroups * kThreads + 32, TileRing<8>::kSmemBytes, st,
                           (const MomW *)d_table, d_maps, xbase, n_w, tpw, momentum, nesterov, partial,
                           ctx->d_status));
  else
    ANC_CUDA(launch_pdl_ex(momentum_ring_kernel<false, kMomGroups>, grid, kMomGroups * kThreads + 32, TileRing<6>::kSmemBytes, st,
                           (const MomW *)d_table, d_maps, xbase, n_w, tpw, momentum, nesterov, partial,
                           ctx->d_status));
  return ANC_OK;
}

static_assert(sizeof(anc_upd_extra) == sizeof(UpdX), "table layout");

int anc_launch_update_group(anc_ctx *ctx, const void *d_table, const anc_tmap *d_maps, const anc_tmap *omap,
                            const void *d_extras, const uint16_t *obase, int n_w, int elems_per_w,
                            float lr_scale_wide, float lr_scale_tall, cudaStream_t st) {
  if (d_extras) {
    const int tpw = elems_per_w / (kTile * kTile);
    const long long total = (long long)n_w * tpw;
    int grid = (int)(total < (long long)ctx->sm_count * 8 ? total : (long long)ctx->sm_count * 8);
    if (grid == 0) return ANC_OK;
    ANC_CUDA(launch_pdl(update_extras_kernel, grid, st, (const UpdW *)d_table, (const UpdX *)d_extras, obase,
                        n_w, tpw, lr_scale_wide, lr_scale_tall));
    return ANC_OK;
  }
  const int tpw = elems_per_w / (kTile * kTile);
  const long long total = (long long)n_w * tpw;
  int grid = (int)(total < (long long)ctx->sm_count ? total : (long long)ctx->sm_count);   // one CTA per SM
  if (grid == 0) return ANC_OK;
  ANC_CUDA(ring_kernels_ready(ctx->device));
  ANC_CUDA(launch_pdl_ex(update_ring_kernel<kUpdGroups>, grid, kUpdGroups * kThreads + 32, TileRing<6>::kSmemBytes, st,
                         (const UpdW *)d_table, d_maps, *omap, obase, n_w, tpw, lr_scale_wide, lr_scale_tall,
                         ctx->d_status));
  return ANC_OK;
}

// ---- allocation-free Frobenius normalisation -------------------------------------
// The per-block partial sums of squares live in this file-scope device array instead of a
// cudaMalloc'ed workspace.  Every GPU that loads the library carries these 256 KiB until the
// process exits.
#define ANC_FRO_STATIC_MAX_BLOCKS 65536
static __device__ __align__(256) float g_fro_static_partials[ANC_FRO_STATIC_MAX_BLOCKS];

namespace {
constexpr int kMaxDevices = 64;
struct StaticScratch {
  float *partials = nullptr;   // device address of g_fro_static_partials on this device
  int sm_count = 0;
};
StaticScratch g_static[kMaxDevices];
std::mutex g_static_mu;
}  // namespace

extern "C" {

int anc_ring_wait_selftest(anc_ctx *ctx, uint32_t tries) {
  ANC_REQUIRE(ctx, "ctx is NULL");
  ANC_REQUIRE(tries > 0 && tries <= (1u << 20), "tries %u outside 1..2^20", tries);
  anc_device_guard guard(ctx->device);
  ring_wait_selftest_kernel<<<1, kThreads, 0, ctx->stream>>>(tries, ctx->d_status);
  ANC_CUDA(cudaGetLastError());
  ANC_CUDA(cudaStreamSynchronize(ctx->stream));
  return ANC_OK;
}

int anc_muon_momentum(anc_ctx *ctx, float *buf, const void *g, int grad_dtype, uint16_t *u, int K,
                      int N, float momentum, int nesterov, int transposed, void *stream) {
  ANC_REQUIRE(ctx && buf && g && u, "NULL argument");
  anc_device_guard guard(ctx->device);
  return anc_launch_momentum(ctx, buf, g, grad_dtype, u, K, N, momentum, nesterov, transposed,
                             anc_pick_stream(ctx, stream));
}

int anc_muon_update(anc_ctx *ctx, float *p32, uint16_t *p16, const uint16_t *O, int K, int N,
                    float lr_scale, int transposed, void *stream) {
  ANC_REQUIRE(ctx && p32 && p16 && O, "NULL argument");
  anc_device_guard guard(ctx->device);
  return anc_launch_update(ctx, p32, p16, O, K, N, lr_scale, transposed,
                           anc_pick_stream(ctx, stream));
}

int anc_fro_normalize_static(int device, uint16_t *X, float *recip, int E, int M, int N, float eps,
                             void *stream) {
  ANC_REQUIRE(X && recip, "NULL argument");
  ANC_REQUIRE(device >= 0 && device < kMaxDevices, "bad device index %d", device);
  ANC_REQUIRE(E > 0 && M > 0 && N > 0, "bad shape (%d x %d x %d)", E, M, N);
  ANC_REQUIRE(((size_t)M * N) % kFroBlock == 0, "matrix of %dx%d elements is not a multiple of %d",
              M, N, kFroBlock);
  const size_t bpm = ((size_t)M * N) / kFroBlock;
  const size_t total = (size_t)E * bpm;
  ANC_REQUIRE(total <= ANC_FRO_STATIC_MAX_BLOCKS,
              "anc_fro_normalize_static: %zu blocks of %d elements exceed the built-in scratch of %d "
              "blocks (E*M*N <= 2^30 elements); use anc_fro_normalize",
              total, kFroBlock, ANC_FRO_STATIC_MAX_BLOCKS);
  int n_dev = 0;
  ANC_CUDA(cudaGetDeviceCount(&n_dev));
  ANC_REQUIRE(device < n_dev, "device %d does not exist (%d visible)", device, n_dev);
  // The kernels below must run on `device`: its scratch address is meaningless elsewhere.
  // So the switch is checked here instead of being left to a guard that ignores a failure.
  int prev_dev = -1;
  ANC_CUDA(cudaGetDevice(&prev_dev));
  if (prev_dev != device) ANC_CUDA(cudaSetDevice(device));
  struct Restore {
    int prev, cur;
    ~Restore() {
      if (prev != cur) cudaSetDevice(prev);
    }
  } restore = {prev_dev, device};
  StaticScratch sc;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static[device].partials) {
      // First call on this device: resolve the array's DEVICE address.  In host code the
      // symbol's name is only a handle, not something a kernel may dereference.
      float *ptr = nullptr;
      ANC_CUDA(cudaGetSymbolAddress((void **)&ptr, g_fro_static_partials));
      int sms = 0;
      ANC_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
      g_static[device].sm_count = sms;
      g_static[device].partials = ptr;
    }
    sc = g_static[device];
  }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t cap = (size_t)sc.sm_count * 8;
  const int grid = (int)(total < cap ? total : cap);
  fro_partial_kernel<<<grid, kThreads, 0, st>>>(X, sc.partials, (int)total);
  ANC_CUDA(cudaGetLastError());
  fro_scale_kernel<<<grid, kThreads, 0, st>>>(X, sc.partials, recip, (int)bpm, (int)total, eps);
  ANC_CUDA(cudaGetLastError());
  return ANC_OK;
}

int anc_fro_normalize(anc_ctx *ctx, uint16_t *X, float *recip, int E, int M, int N, float eps,
                      void *stream) {
  ANC_REQUIRE(ctx && X && recip, "NULL argument");
  anc_device_guard guard(ctx->device);
  return anc_launch_fro_normalize(ctx, X, recip, E, M, N, eps, anc_pick_stream(ctx, stream));
}

}  // extern "C"
