// ZeRO-1 exchange step: NCCL over NVLink, opened with dlopen so that the library
// loads (and every other entry point works) on machines without NCCL.  The reference
// is single-GPU and has no counterpart.  Collectives are issued on the caller's
// stream; payloads are sent as bytes so no NCCL datatype enum is relied on.
#include <dlfcn.h>
#include <mutex>
#include <nccl.h>
#include <string.h>
#include "anc_internal.h"

namespace {

struct NcclApi {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
NcclApi g_nccl;
std::mutex g_nccl_mu;   // guards the one-time load

int nccl_fail(ncclResult_t r, const char *what) {
  anc_set_error("NCCL error %d (%s) in %s", (int)r,
                g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?", what);
  return ANC_E_NCCL;
}

#define ANC_NCCL(call)                                     \
  do {                                                     \
    ncclResult_t _r = (call);                              \
    if (_r != ncclSuccess) return nccl_fail(_r, #call);    \
  } while (0)

template <typename T>
bool load_sym(T &fn, const char *name) {
  fn = (T)dlsym(g_nccl.handle, name);
  return fn != nullptr;
}

}  // namespace

struct anc_comm {
  anc_ctx *ctx;
  ncclComm_t comm;
  int rank, world;
  float *d_token;
};

extern "C" {

int anc_nccl_load(const char *path) {
  std::lock_guard<std::mutex> lk(g_nccl_mu);
  if (g_nccl.handle) return ANC_OK;
  const char *cands[4] = {path, getenv("ANC_NCCL_PATH"), "libnccl.so.2", "libnccl.so"};
  for (const char *c : cands) {
    if (!c || !*c) continue;
    g_nccl.handle = dlopen(c, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.handle) break;
  }
  if (!g_nccl.handle) {
    anc_set_error("cannot open NCCL (%s)", dlerror());
    return ANC_E_NCCL;
  }
  bool ok = load_sym(g_nccl.GetUniqueId, "ncclGetUniqueId") &&
            load_sym(g_nccl.CommInitRank, "ncclCommInitRank") &&
            load_sym(g_nccl.CommDestroy, "ncclCommDestroy") &&
            load_sym(g_nccl.AllGather, "ncclAllGather") &&
            load_sym(g_nccl.ReduceScatter, "ncclReduceScatter") &&
            load_sym(g_nccl.AllReduce, "ncclAllReduce") &&
            load_sym(g_nccl.GetErrorString, "ncclGetErrorString");
  if (!ok) {
    anc_set_error("NCCL library lacks a required symbol");
    dlclose(g_nccl.handle);
    g_nccl = NcclApi();
    return ANC_E_NCCL;
  }
  return ANC_OK;
}

int anc_nccl_unique_id(void *id128) {
  ANC_REQUIRE(id128, "id is NULL");
  int rc = anc_nccl_load(nullptr);
  if (rc) return rc;
  static_assert(sizeof(ncclUniqueId) == ANC_NCCL_UNIQUE_ID_BYTES, "unique id size");
  ncclUniqueId id;
  ANC_NCCL(g_nccl.GetUniqueId(&id));
  memcpy(id128, &id, sizeof(id));
  return ANC_OK;
}

int anc_comm_create(anc_ctx *ctx, const void *id128, int rank, int world, anc_comm **out) {
  ANC_REQUIRE(ctx && id128 && out, "NULL argument");
  ANC_REQUIRE(world >= 1 && rank >= 0 && rank < world, "bad rank %d of %d", rank, world);
  int rc = anc_nccl_load(nullptr);
  if (rc) return rc;
  anc_device_guard guard(ctx->device);
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  anc_comm *c = new anc_comm();
  c->ctx = ctx;
  c->rank = rank;
  c->world = world;
  c->d_token = nullptr;
  ncclResult_t r = g_nccl.CommInitRank(&c->comm, world, id, rank);
  if (r != ncclSuccess) {
    delete c;
    return nccl_fail(r, "ncclCommInitRank");
  }
  cudaError_t e = cudaMalloc((void **)&c->d_token, 256);
  if (e == cudaSuccess) e = cudaMemset(c->d_token, 0, 256);
  if (e != cudaSuccess) {
    g_nccl.CommDestroy(c->comm);
    delete c;
    return anc_cuda_fail(e, "comm token");
  }
  *out = c;
  return ANC_OK;
}

int anc_comm_destroy(anc_comm *c) {
  if (!c) return ANC_OK;
  anc_device_guard guard(c->ctx->device);
  cudaStreamSynchronize(c->ctx->stream);
  if (c->d_token) cudaFree(c->d_token);
  if (g_nccl.CommDestroy) g_nccl.CommDestroy(c->comm);
  delete c;
  return ANC_OK;
}

int anc_comm_allgather_bf16(anc_comm *c, uint16_t *arena, uint64_t elems_per_rank, void *stream) {
  ANC_REQUIRE(c && arena, "NULL argument");
  if (elems_per_rank == 0) return ANC_OK;
  anc_device_guard guard(c->ctx->device);
  cudaStream_t st = anc_pick_stream(c->ctx, stream);
  const size_t bytes = (size_t)elems_per_rank * 2;
  ANC_NCCL(g_nccl.AllGather((const char *)arena + (size_t)c->rank * bytes, arena, bytes, ncclUint8,
                            c->comm, st));
  return ANC_OK;
}

int anc_comm_reduce_scatter_grads(anc_comm *c, void *arena, uint64_t elems_per_rank, int grad_dtype,
                                  void *stream) {
  ANC_REQUIRE(c && arena, "NULL argument");
  ANC_REQUIRE(grad_dtype == ANC_GRAD_BF16 || grad_dtype == ANC_GRAD_F32, "bad grad_dtype");
  if (elems_per_rank == 0) return ANC_OK;
  anc_device_guard guard(c->ctx->device);
  cudaStream_t st = anc_pick_stream(c->ctx, stream);
  const size_t esz = grad_dtype == ANC_GRAD_BF16 ? 2 : 4;
  const ncclDataType_t dt = grad_dtype == ANC_GRAD_BF16 ? (ncclDataType_t)9 /* ncclBfloat16 */ : ncclFloat32;
  ANC_NCCL(g_nccl.ReduceScatter(arena, (char *)arena + (size_t)c->rank * elems_per_rank * esz,
                                (size_t)elems_per_rank, dt, ncclSum, c->comm, st));
  return ANC_OK;
}

int anc_comm_barrier(anc_comm *c, void *stream) {
  ANC_REQUIRE(c, "comm is NULL");
  anc_device_guard guard(c->ctx->device);
  cudaStream_t st = anc_pick_stream(c->ctx, stream);
  ANC_NCCL(g_nccl.AllReduce(c->d_token, c->d_token, 1, ncclFloat32, ncclSum, c->comm, st));
  ANC_CUDA(cudaStreamSynchronize(st));
  return ANC_OK;
}

}  // extern "C"
