// Context, device memory, events: the plumbing the reference does with
// cuda.bindings (cuMemAlloc / cuMemcpy* / cuMemFree in _DBuf, _Buf, _GpuArray).
#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif
#include <sched.h>
#include <stdlib.h>
#include <sys/syscall.h>
#include <unistd.h>
#include <string.h>
#include "anc_internal.h"

static thread_local char g_err[512] = "";

void anc_set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int anc_cuda_fail(cudaError_t e, const char *what) {
  anc_set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return e == cudaErrorMemoryAllocation ? ANC_E_NOMEM : ANC_E_CUDA;
}

extern "C" {

int anc_version(void) { return 100; }

const char *anc_last_error(void) { return g_err; }

int anc_device_count(int *count) {
  ANC_REQUIRE(count, "count is NULL");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  *count = n;
  return ANC_OK;
}

int anc_ctx_create(int device, void *stream, anc_ctx **out) {
  ANC_REQUIRE(out, "out is NULL");
  *out = nullptr;
  ANC_CUDA(cudaSetDevice(device));
  ANC_CUDA(cudaFree(0));
  anc_ctx *c = new anc_ctx();
  memset(c, 0, sizeof(*c));
  c->device = device;
  auto fail = [c](int rc) {          // release whatever was set up so far
    if (c->d_work) cudaFree(c->d_work);
    if (c->d_status) cudaFree(c->d_status);
    if (c->own_stream) cudaStreamDestroy(c->stream);
    delete c;
    return rc;
  };
  if (stream) {
    c->stream = (cudaStream_t)stream;
    c->own_stream = false;
  } else {
    cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return fail(anc_cuda_fail(e, "cudaStreamCreate"));
    c->own_stream = true;
  }
  int major = 0, minor = 0;
  cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) return fail(anc_cuda_fail(e, "cudaDeviceGetAttribute"));
  if (major != 10) {
    anc_set_error("device %d is sm_%d%d; this library holds sm_100a code only", device, major, minor);
    return fail(ANC_E_UNSUPPORTED);
  }
  c->work_bytes = 1 << 20;
  e = cudaMalloc(&c->d_work, c->work_bytes);
  if (e == cudaSuccess) e = cudaMalloc((void **)&c->d_status, 256);
  if (e == cudaSuccess) e = cudaMemset(c->d_status, 0, 256);
  if (e != cudaSuccess) return fail(anc_cuda_fail(e, "ctx workspace"));
  *out = c;
  return ANC_OK;
}

int anc_ctx_destroy(anc_ctx *ctx) {
  if (!ctx) return ANC_OK;
  anc_device_guard g(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  anc_gemm_cache_destroy(ctx);
  if (ctx->d_work) cudaFree(ctx->d_work);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->d_flush) cudaFree(ctx->d_flush);
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return ANC_OK;
}

int anc_ctx_reserve_sms(anc_ctx *ctx, int n_sms) {
  ANC_REQUIRE(ctx, "ctx is NULL");
  ANC_REQUIRE(n_sms >= 0 && n_sms <= ctx->sm_count - 2, "cannot reserve %d of %d SMs", n_sms, ctx->sm_count);
  ctx->reserved_sms = n_sms;
  return ANC_OK;
}

int anc_ctx_stream(anc_ctx *ctx, void **stream) {
  ANC_REQUIRE(ctx && stream, "NULL argument");
  *stream = (void *)ctx->stream;
  return ANC_OK;
}

int anc_ctx_sync(anc_ctx *ctx, void *stream) {
  ANC_REQUIRE(ctx, "ctx is NULL");
  anc_device_guard g(ctx->device);
  ANC_CUDA(cudaStreamSynchronize(anc_pick_stream(ctx, stream)));
  return ANC_OK;
}

int anc_ctx_status(anc_ctx *ctx, uint32_t *code) {
  ANC_REQUIRE(ctx && code, "NULL argument");
  anc_device_guard g(ctx->device);
  ANC_CUDA(cudaStreamSynchronize(ctx->stream));
  ANC_CUDA(cudaMemcpy(code, ctx->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (*code) ANC_CUDA(cudaMemset(ctx->d_status, 0, sizeof(uint32_t)));
  return ANC_OK;
}

int anc_malloc(anc_ctx *ctx, size_t bytes, void **dptr) {
  ANC_REQUIRE(ctx && dptr, "NULL argument");
  anc_device_guard g(ctx->device);
  *dptr = nullptr;
  if (bytes == 0) bytes = 256;
  cudaError_t e = cudaMalloc(dptr, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    anc_set_error("cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    return ANC_E_NOMEM;
  }
  return ANC_OK;
}

int anc_free(anc_ctx *ctx, void *dptr) {
  ANC_REQUIRE(ctx, "ctx is NULL");
  if (!dptr) return ANC_OK;
  anc_device_guard g(ctx->device);
  ANC_CUDA(cudaFree(dptr));
  return ANC_OK;
}

int anc_memset(anc_ctx *ctx, void *dptr, int byte, size_t bytes, void *stream) {
  ANC_REQUIRE(ctx && dptr, "NULL argument");
  anc_device_guard g(ctx->device);
  ANC_CUDA(cudaMemsetAsync(dptr, byte, bytes, anc_pick_stream(ctx, stream)));
  return ANC_OK;
}

int anc_h2d(anc_ctx *ctx, void *dptr, const void *hptr, size_t bytes, void *stream, int sync) {
  ANC_REQUIRE(ctx && dptr && hptr, "NULL argument");
  anc_device_guard g(ctx->device);
  cudaStream_t st = anc_pick_stream(ctx, stream);
  ANC_CUDA(cudaMemcpyAsync(dptr, hptr, bytes, cudaMemcpyHostToDevice, st));
  if (sync) ANC_CUDA(cudaStreamSynchronize(st));
  return ANC_OK;
}

int anc_d2h(anc_ctx *ctx, void *hptr, const void *dptr, size_t bytes, void *stream, int sync) {
  ANC_REQUIRE(ctx && dptr && hptr, "NULL argument");
  anc_device_guard g(ctx->device);
  cudaStream_t st = anc_pick_stream(ctx, stream);
  ANC_CUDA(cudaMemcpyAsync(hptr, dptr, bytes, cudaMemcpyDeviceToHost, st));
  if (sync) ANC_CUDA(cudaStreamSynchronize(st));
  return ANC_OK;
}

int anc_d2d(anc_ctx *ctx, void *dst, const void *src, size_t bytes, void *stream) {
  ANC_REQUIRE(ctx && dst && src, "NULL argument");
  anc_device_guard g(ctx->device);
  ANC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, anc_pick_stream(ctx, stream)));
  return ANC_OK;
}

int anc_host_alloc(size_t bytes, void **hptr) {
  ANC_REQUIRE(hptr, "hptr is NULL");
  *hptr = nullptr;
  cudaError_t e = cudaHostAlloc(hptr, bytes ? bytes : 64, cudaHostAllocDefault);
  if (e != cudaSuccess) {
    cudaGetLastError();
    anc_set_error("cudaHostAlloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    return ANC_E_NOMEM;
  }
  return ANC_OK;
}

// CPUs listed in a sysfs cpulist string ("0-13,56-69") into a cpu_set_t; false if none parsed.
static bool parse_cpulist(const char *s, cpu_set_t *set) {
  CPU_ZERO(set);
  bool any = false;
  while (*s) {
    char *end = nullptr;
    long a = strtol(s, &end, 10);
    if (end == s) break;
    long b = a;
    s = end;
    if (*s == '-') {
      b = strtol(s + 1, &end, 10);
      if (end == s + 1) break;
      s = end;
    }
    for (long c = a; c <= b && c < CPU_SETSIZE; ++c) {
      if (c >= 0) {
        CPU_SET((int)c, set);
        any = true;
      }
    }
    while (*s == ',' || *s == ' ' || *s == '\n') ++s;
  }
  return any;
}

int anc_host_alloc_near(int device, size_t bytes, void **hptr) {
  ANC_REQUIRE(hptr, "hptr is NULL");
  *hptr = nullptr;
  // Page-locked memory lands where the allocating thread's memory policy and CPU put it.  For the
  // duration of the allocation this thread prefers the GPU's NUMA node (set_mempolicy; works even
  // when the process may not run on that node's CPUs) and, where allowed, runs on the CPUs next
  // to the GPU, so that host<->device copies do not cross the socket interconnect.  Any failure on
  // the way falls back to a plain allocation.
  cpu_set_t saved, local;
  bool bound = false, policy = false;
  char busid[32] = {0};
  if (sched_getaffinity(0, sizeof(saved), &saved) == 0 &&
      cudaDeviceGetPCIBusId(busid, (int)sizeof(busid), device) == cudaSuccess) {
    for (char *c = busid; *c; ++c)
      if (*c >= 'A' && *c <= 'F') *c = (char)(*c - 'A' + 'a');
    char path[128];
    snprintf(path, sizeof(path), "/sys/bus/pci/devices/%s/numa_node", busid);
    FILE *fn = fopen(path, "r");
    if (fn) {
      int node = -1;
      if (fscanf(fn, "%d", &node) == 1 && node >= 0 && node < 1024) {
        unsigned long mask[16] = {0};
        mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
        policy = syscall(SYS_set_mempolicy, 1 /* MPOL_PREFERRED */, mask, 1024ul) == 0;
      }
      fclose(fn);
    }
    snprintf(path, sizeof(path), "/sys/bus/pci/devices/%s/local_cpulist", busid);
    FILE *f = fopen(path, "r");
    if (f) {
      char line[1024] = {0};
      if (fgets(line, sizeof(line), f) && parse_cpulist(line, &local)) {
        cpu_set_t both;
        CPU_AND(&both, &local, &saved);          // stay inside what this process may use
        if (CPU_COUNT(&both) > 0 && sched_setaffinity(0, sizeof(both), &both) == 0) bound = true;
      }
      fclose(f);
    }
  } else {
    cudaGetLastError();
  }
  int rc = anc_host_alloc(bytes, hptr);
  if (rc == ANC_OK && (bound || policy) && bytes) memset(*hptr, 0, bytes);   // touch while the placement holds
  if (bound) sched_setaffinity(0, sizeof(saved), &saved);
  if (policy) syscall(SYS_set_mempolicy, 0 /* MPOL_DEFAULT */, (unsigned long *)nullptr, 0ul);
  return rc;
}

int anc_host_free(void *hptr) {
  if (hptr) ANC_CUDA(cudaFreeHost(hptr));
  return ANC_OK;
}

int anc_event_create(void **ev) {
  ANC_REQUIRE(ev, "ev is NULL");
  cudaEvent_t e;
  ANC_CUDA(cudaEventCreate(&e));
  *ev = (void *)e;
  return ANC_OK;
}

int anc_event_record(void *ev, void *stream) {
  ANC_REQUIRE(ev, "ev is NULL");
  ANC_CUDA(cudaEventRecord((cudaEvent_t)ev, (cudaStream_t)stream));
  return ANC_OK;
}

int anc_event_sync(void *ev) {
  ANC_REQUIRE(ev, "ev is NULL");
  ANC_CUDA(cudaEventSynchronize((cudaEvent_t)ev));
  return ANC_OK;
}

int anc_event_elapsed_ms(void *start, void *stop, float *ms) {
  ANC_REQUIRE(start && stop && ms, "NULL argument");
  ANC_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
  return ANC_OK;
}

int anc_event_destroy(void *ev) {
  if (ev) ANC_CUDA(cudaEventDestroy((cudaEvent_t)ev));
  return ANC_OK;
}

int anc_stream_create(anc_ctx *ctx, void **stream) {
  ANC_REQUIRE(ctx && stream, "NULL argument");
  anc_device_guard g(ctx->device);
  cudaStream_t st;
  ANC_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  *stream = (void *)st;
  return ANC_OK;
}

int anc_stream_destroy(anc_ctx *ctx, void *stream) {
  ANC_REQUIRE(ctx, "ctx is NULL");
  if (!stream) return ANC_OK;
  anc_device_guard g(ctx->device);
  ANC_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  ANC_CUDA(cudaStreamDestroy((cudaStream_t)stream));
  return ANC_OK;
}

int anc_stream_wait_event(void *stream, void *ev) {
  ANC_REQUIRE(ev, "ev is NULL");
  ANC_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)ev, 0));
  return ANC_OK;
}

int anc_graph_begin(anc_ctx *ctx, void *stream) {
  ANC_REQUIRE(ctx, "ctx is NULL");
  anc_device_guard g(ctx->device);
  ANC_CUDA(cudaStreamBeginCapture(anc_pick_stream(ctx, stream), cudaStreamCaptureModeThreadLocal));
  return ANC_OK;
}

int anc_graph_end(anc_ctx *ctx, void *stream, void **graph_exec) {
  ANC_REQUIRE(ctx && graph_exec, "NULL argument");
  anc_device_guard g(ctx->device);
  *graph_exec = nullptr;
  cudaGraph_t graph = nullptr;
  ANC_CUDA(cudaStreamEndCapture(anc_pick_stream(ctx, stream), &graph));
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return anc_cuda_fail(e, "cudaGraphInstantiate");
  *graph_exec = (void *)exec;
  return ANC_OK;
}

int anc_graph_launch(anc_ctx *ctx, void *graph_exec, void *stream) {
  ANC_REQUIRE(ctx && graph_exec, "NULL argument");
  anc_device_guard g(ctx->device);
  ANC_CUDA(cudaGraphLaunch((cudaGraphExec_t)graph_exec, anc_pick_stream(ctx, stream)));
  return ANC_OK;
}

int anc_graph_destroy(void *graph_exec) {
  if (graph_exec) ANC_CUDA(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
  return ANC_OK;
}

__global__ void anc_flush_kernel(uint4 *p, size_t n16) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n16; i += stride) p[i] = make_uint4(0u, 0u, 0u, 0u);
}

int anc_flush_l2(anc_ctx *ctx, void *stream) {
  ANC_REQUIRE(ctx, "ctx is NULL");
  anc_device_guard g(ctx->device);
  if (!ctx->d_flush) {
    ctx->flush_bytes = (size_t)256 << 20;  // 256 MiB > 126 MB L2
    cudaError_t e = cudaMalloc(&ctx->d_flush, ctx->flush_bytes);
    if (e != cudaSuccess) {
      ctx->d_flush = nullptr;
      return anc_cuda_fail(e, "flush buffer");
    }
  }
  anc_flush_kernel<<<ctx->sm_count * 8, 256, 0, anc_pick_stream(ctx, stream)>>>(
      (uint4 *)ctx->d_flush, ctx->flush_bytes / 16);
  ANC_CUDA(cudaGetLastError());
  return ANC_OK;
}

}  // extern "C"
