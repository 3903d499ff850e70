// Peer-to-peer exchange over NVLink without using SMs for the payload: every rank maps the
// other ranks' bf16 parameter arenas through CUDA IPC and pushes its own slice into them
// with asynchronous device-to-device copies (copy engines), so the transfer overlaps the
// Newton-Schulz GEMMs, which occupy every SM.  Completion is signalled per destination
// by a one-word store into the peer's flag array issued on the same stream after the
// payload copy (stream order = the payload has landed first); the receiver waits with a
// bounded spin.  The reference is single-GPU and has no counterpart.
#include "anc_internal.h"

namespace {

__global__ void signal_kernel(volatile uint32_t *remote_flag, uint32_t value) {
  *remote_flag = value;
  __threadfence_system();
}

// Waits until flags[i] >= value for every i != skip.  Bounded: ~2 s, then records a status
// bit and returns.  The comparison is on the distance so the counter may wrap.
__global__ void wait_flags_kernel(const volatile uint32_t *flags, int n, int skip, uint32_t value,
                                  uint32_t *status) {
  const int i = threadIdx.x;
  if (i >= n || i == skip) return;
  for (uint32_t it = 0; it < (1u << 24); ++it) {
    const uint32_t f = flags[i];
    if ((int32_t)(f - value) >= 0) return;
    __nanosleep(100);
  }
  atomicOr(status, ANC_DEV_TIMEOUT_PEER);
}

}  // namespace

extern "C" {

int anc_ipc_export_mem(anc_ctx *ctx, void *dptr, void *handle64) {
  ANC_REQUIRE(ctx && dptr && handle64, "NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == ANC_IPC_HANDLE_BYTES, "ipc handle size");
  anc_device_guard g(ctx->device);
  ANC_CUDA(cudaIpcGetMemHandle((cudaIpcMemHandle_t *)handle64, dptr));
  return ANC_OK;
}

int anc_ipc_open_mem(anc_ctx *ctx, const void *handle64, void **peer_ptr) {
  ANC_REQUIRE(ctx && handle64 && peer_ptr, "NULL argument");
  anc_device_guard g(ctx->device);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  ANC_CUDA(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return ANC_OK;
}

int anc_ipc_close_mem(anc_ctx *ctx, void *peer_ptr) {
  ANC_REQUIRE(ctx, "ctx is NULL");
  if (!peer_ptr) return ANC_OK;
  anc_device_guard g(ctx->device);
  ANC_CUDA(cudaIpcCloseMemHandle(peer_ptr));
  return ANC_OK;
}

int anc_p2p_signal(anc_ctx *ctx, uint32_t *remote_flag, uint32_t value, void *stream) {
  ANC_REQUIRE(ctx && remote_flag, "NULL argument");
  anc_device_guard g(ctx->device);
  signal_kernel<<<1, 1, 0, anc_pick_stream(ctx, stream)>>>(remote_flag, value);
  ANC_CUDA(cudaGetLastError());
  return ANC_OK;
}

int anc_p2p_wait_flags(anc_ctx *ctx, const uint32_t *flags, int n, int skip, uint32_t value,
                       void *stream) {
  ANC_REQUIRE(ctx && flags && n > 0 && n <= 64, "bad argument");
  anc_device_guard g(ctx->device);
  wait_flags_kernel<<<1, 64, 0, anc_pick_stream(ctx, stream)>>>(flags, n, skip, value, ctx->d_status);
  ANC_CUDA(cudaGetLastError());
  return ANC_OK;
}

}  // extern "C"
