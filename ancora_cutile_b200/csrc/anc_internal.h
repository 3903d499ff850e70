// Internal declarations shared by the translation units of libancora_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include "../../include/ancora_b200.h"

struct anc_ctx {
  int device;
  cudaStream_t stream;
  bool own_stream;
  uint32_t *d_status;       // device status word: kernels OR error bits into it
  void *d_work;             // small device workspace (Frobenius partial sums)
  size_t work_bytes;
  void *d_flush;            // L2 flush buffer, allocated on first use
  size_t flush_bytes;
  int sm_count;
  int reserved_sms;         // SMs the persistent Newton-Schulz kernel leaves to other streams
};

// entries of the device tables the Muon plan builds for the group launches
struct anc_mom_entry { float *buf; const void *g; int K, N, tr, _pad; };
struct anc_upd_entry { float *p32; uint16_t *p16; int K, N, tr, _pad; };
struct anc_upd_extra { uint8_t *fp8; uint8_t *scale; uint16_t *p16_t; uint8_t *fp8_t; uint8_t *scale_t; int64_t _pad; };

// device status bits
#define ANC_DEV_TIMEOUT_TMA 0x1u     // producer/consumer mbarrier wait ran out
#define ANC_DEV_TIMEOUT_MMA 0x2u
#define ANC_DEV_TIMEOUT_EPI 0x4u
#define ANC_DEV_BAD_INDEX 0x8u       // a table index failed its bounds check
#define ANC_DEV_TIMEOUT_DEP 0x10u    // a tile's dependency (the matrix's previous phase) never completed

void anc_set_error(const char *fmt, ...);
int anc_cuda_fail(cudaError_t e, const char *what);

#define ANC_CUDA(call)                                           \
  do {                                                           \
    cudaError_t _e = (call);                                     \
    if (_e != cudaSuccess) return anc_cuda_fail(_e, #call);      \
  } while (0)

#define ANC_REQUIRE(cond, ...)                                   \
  do {                                                           \
    if (!(cond)) {                                               \
      anc_set_error(__VA_ARGS__);                                \
      return ANC_E_INVALID;                                      \
    }                                                            \
  } while (0)

static inline cudaStream_t anc_pick_stream(anc_ctx *ctx, void *stream) {
  return stream ? (cudaStream_t)stream : ctx->stream;
}

struct anc_device_guard {
  int prev;
  bool changed;
  explicit anc_device_guard(int dev) : prev(-1), changed(false) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) {
      changed = (cudaSetDevice(dev) == cudaSuccess);
    }
  }
  ~anc_device_guard() {
    if (changed) cudaSetDevice(prev);
  }
};

// ---- launchers implemented in the kernel translation units -----------------
int anc_launch_momentum(anc_ctx *ctx, float *buf, const void *g, int grad_dtype, uint16_t *u, int K,
                        int N, float momentum, int nesterov, int transposed, cudaStream_t st);
int anc_launch_update(anc_ctx *ctx, float *p32, uint16_t *p16, const uint16_t *O, int K, int N,
                      float lr_scale, int transposed, cudaStream_t st);
int anc_launch_fro_normalize(anc_ctx *ctx, uint16_t *X, float *recip, int E, int M, int N, float eps,
                             cudaStream_t st);
// Raises the shared-memory limit of the ring-fed sweeps on the context's device (idempotent).
int anc_elem_kernels_prepare(anc_ctx *ctx);
// Storage of one CUtensorMap (kept opaque here so that this header needs no driver types).
struct alignas(64) anc_tmap { unsigned char b[128]; };
// Tiled map over a dense row-major array of `slices` matrices of (rows, inner) elements of 2 or 4
// bytes (slices == 0: a single matrix, 2-D map), box (box_inner, box_rows[, 1]), no swizzle.
int anc_encode_tile_map(anc_tmap *out, const void *ptr, int elem_bytes, uint64_t inner, uint64_t rows,
                        uint64_t slices, uint32_t box_inner, uint32_t box_rows);
// d_maps: three maps per table entry (momentum buffer, gradient, master weight; 64x64 boxes) for
// the entries with tr != 0, unused storage for the others.
int anc_launch_momentum_group(anc_ctx *ctx, const void *d_table, const anc_tmap *d_maps, uint16_t *xbase,
                              int n_w, int elems_per_w, int grad_dtype, float momentum, int nesterov,
                              float *partial, cudaStream_t st);
// partial: per matrix, per_matrix sums of squares (warp_sums == 0: fro_partial's blocks) or per_matrix
// groups of eight warp sums (warp_sums != 0: the momentum kernel's 64x64 tiles).
// sched (nullable): 2 + E scheduler words of the chain kernel, cleared here
int anc_launch_fro_finalize(anc_ctx *ctx, const float *partial, float *recip, int E, int per_matrix,
                            int warp_sums, float eps, uint32_t *sched, cudaStream_t st);
int anc_launch_fro_partial(anc_ctx *ctx, const uint16_t *X, float *partial, int E, int M, int N,
                           cudaStream_t st);
// omap: 3-D map over the packed operand at obase seen as slots of (N, K) bf16, 64x64 boxes (host copy).
int anc_launch_update_group(anc_ctx *ctx, const void *d_table, const anc_tmap *d_maps, const anc_tmap *omap,
                            const void *d_extras, const uint16_t *obase, int n_w, int elems_per_w,
                            float lr_scale_wide, float lr_scale_tall, cudaStream_t st);
// mscale (nullable): per-matrix factor r[e] folded into the epilogue -- mode 0 stores
// RNE(r^2 * acc), mode 2 stores RNE((alpha*r)*Q + (beta*r)*acc); mode 1 ignores it.
// diag (mode 1): added to the diagonal of every matrix before the rounding (0 adds nothing).
// Mode 2 with alpha == 0 reads no axpy operand.
int anc_launch_ns_gemm(anc_ctx *ctx, int mode, const uint16_t *P, const uint16_t *Q, uint16_t *C,
                       int E, int M, int N, float alpha, float beta, float diag, const float *mscale,
                       cudaStream_t st);
// One persistent launch for the whole chain (M and N multiples of 256, at most 16 steps); the result is
// in X for an even number of steps, in Y for an odd one.  sched: 2 + E zeroed words.
bool anc_ns_chain_supported(const anc_ctx *ctx, int M, int N, int steps);
int anc_launch_ns_chain(anc_ctx *ctx, uint16_t *X, uint16_t *Y, uint16_t *A, uint16_t *B, int E, int M, int N,
                        int steps, const float *coeffs, const float *mscale, uint32_t *sched,
                        uint32_t spin_limit, cudaStream_t st);
void anc_gemm_cache_destroy(anc_ctx *ctx);
