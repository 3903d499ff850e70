/*
 * ancora_b200.h -- C ABI of libancora_b200.so: the Muon + AdamW hybrid optimizer
 * step of ancora-cutile (ancora/optim/{adamw,muon,hybrid}.py and
 * ancora/kernels/muon_ns.py) as hand-written CUDA for sm_100a.
 *
 * The reference has no C ABI for this path: its Python classes launch cuda.tile
 * kernels with ct.launch(stream_int, grid, kernel, args).  Each entry point below
 * names the reference call site(s) it replaces.  The calling style (opaque handle
 * from a create call, int status from every call, explicit free) is the one the
 * reference already uses for its only ctypes plug-in (ancora/model/resident.py:37-47).
 *
 * Conventions
 *   - every function returns 0 on success, a negative ANC_E_* code on failure, and
 *     never aborts the process; anc_last_error() gives the message for this thread.
 *   - device pointers are plain void* / typed pointers into CUDA device memory;
 *     "stream" is a CUstream / cudaStream_t passed as void* (NULL = the context's
 *     own stream).  The reference passes the same value as a Python int.
 *   - bf16 values travel as uint16_t bit patterns, as in the reference.
 *   - calls are asynchronous on the stream unless the name ends in _sync or the
 *     comment says otherwise (reference: ResidentLayerTrain.step is async,
 *     ancora/model/resident_train.py:336-339).
 */
#ifndef ANCORA_B200_H_
#define ANCORA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ANC_API __attribute__((visibility("default")))

/* status codes */
#define ANC_OK 0
#define ANC_E_INVALID (-1)    /* bad argument (shape, alignment, null pointer)          */
#define ANC_E_CUDA (-2)       /* a CUDA runtime / driver call failed                    */
#define ANC_E_NOMEM (-3)      /* device or host allocation failed                       */
#define ANC_E_DEVICE (-4)     /* a kernel reported a bounded-wait timeout / bad index   */
#define ANC_E_NCCL (-5)       /* NCCL missing or a collective failed                    */
#define ANC_E_UNSUPPORTED (-6)

/* gradient element type */
#define ANC_GRAD_BF16 0
#define ANC_GRAD_F32 1

/* bf16 rounding of the parameter copy */
#define ANC_ROUND_RNE 0 /* ancora/optim/adamw.py:41 */
#define ANC_ROUND_SR 1  /* Philox4x32-10 dither, bit rule of ancora/kernels/fused.py:159-161 */

typedef struct anc_ctx anc_ctx;
typedef struct anc_adamw_plan anc_adamw_plan;
typedef struct anc_muon_plan anc_muon_plan;
typedef struct anc_comm anc_comm;

/* ---------------------------------------------------------------- runtime ---- */

ANC_API int anc_version(void);
ANC_API const char *anc_last_error(void);
ANC_API int anc_device_count(int *count);

/* Context = (device, stream, small device workspace, device status word).
 * Replaces the reference's per-script bootstrap (cudart.cudaFree(0); Device(0);
 * create_stream(): tests/optim/test_adamw.py:15-17).  stream==NULL creates one. */
ANC_API int anc_ctx_create(int device, void *stream, anc_ctx **out);
ANC_API int anc_ctx_destroy(anc_ctx *ctx);
/* The persistent Newton-Schulz kernel fills every SM it is given for the length of a whole chain.
 * Reserving n SMs keeps it off them, so that a kernel of another stream (the NCCL all-gather that
 * overlaps the step) finds room at once.  0 by default; no counterpart in the reference. */
ANC_API int anc_ctx_reserve_sms(anc_ctx *ctx, int n_sms);
ANC_API int anc_ctx_stream(anc_ctx *ctx, void **stream);
ANC_API int anc_ctx_sync(anc_ctx *ctx, void *stream);
/* Reads and clears the device status word (0 = no kernel reported a problem). */
ANC_API int anc_ctx_status(anc_ctx *ctx, uint32_t *code);

/* Device buffers: replace cuMemAlloc / cuMemcpyHtoD / cuMemcpyDtoH / cuMemFree in
 * _DBuf (ancora/model/resident.py:52-94), _Buf (ancora/optim/adamw.py:51-60) and
 * _GpuArray (ancora/kernels/loss.py:277-294). */
ANC_API int anc_malloc(anc_ctx *ctx, size_t bytes, void **dptr);
ANC_API int anc_free(anc_ctx *ctx, void *dptr);
ANC_API int anc_memset(anc_ctx *ctx, void *dptr, int byte, size_t bytes, void *stream);
ANC_API int anc_h2d(anc_ctx *ctx, void *dptr, const void *hptr, size_t bytes, void *stream, int sync);
ANC_API int anc_d2h(anc_ctx *ctx, void *hptr, const void *dptr, size_t bytes, void *stream, int sync);
ANC_API int anc_d2d(anc_ctx *ctx, void *dst, const void *src, size_t bytes, void *stream);
ANC_API int anc_host_alloc(size_t bytes, void **hptr); /* pinned */
/* Pinned memory placed on the NUMA node next to `device` (the calling thread is bound to the
 * GPU's local CPUs while it allocates and touches the pages, then restored); falls back to
 * anc_host_alloc when the topology cannot be read. */
ANC_API int anc_host_alloc_near(int device, size_t bytes, void **hptr);
ANC_API int anc_host_free(void *hptr);

/* CUDA events on the caller's stream (timing in the benchmark). */
ANC_API int anc_event_create(void **ev);
ANC_API int anc_event_record(void *ev, void *stream);
ANC_API int anc_event_sync(void *ev);
ANC_API int anc_event_elapsed_ms(void *start, void *stop, float *ms);
ANC_API int anc_event_destroy(void *ev);
/* Stream capture into an executable CUDA graph and its replay (thread-local capture mode).
 * Run the work once eagerly first: first calls allocate tables and set kernel attributes. */
ANC_API int anc_graph_begin(anc_ctx *ctx, void *stream);
ANC_API int anc_graph_end(anc_ctx *ctx, void *stream, void **graph_exec);
ANC_API int anc_graph_launch(anc_ctx *ctx, void *graph_exec, void *stream);
ANC_API int anc_graph_destroy(void *graph_exec);
/* Extra streams for overlapping copies / collectives with compute. */
ANC_API int anc_stream_create(anc_ctx *ctx, void **stream);
ANC_API int anc_stream_destroy(anc_ctx *ctx, void *stream);
ANC_API int anc_stream_wait_event(void *stream, void *ev);

/* Writes `bytes` of device memory (larger than L2) to evict cached lines between
 * timed iterations. */
ANC_API int anc_flush_l2(anc_ctx *ctx, void *stream);

/* ------------------------------------------------------------------ AdamW ---- */

/* One tensor of the multi-tensor AdamW arena.  elem_offset is the index of the
 * tensor's first element in the global (un-sharded) arena and must be a multiple
 * of 8: it keys the stochastic-rounding stream, so results do not depend on how the
 * arena is sharded or launched. */
typedef struct anc_adamw_tensor {
  const void *g; /* gradient, bf16 bits or f32 (plan's grad_dtype)            */
  float *p32;    /* fp32 master, updated in place                              */
  float *m;      /* first moment                                               */
  float *v;      /* second moment                                              */
  uint16_t *p16; /* bf16 parameter copy the forward reads, written every step  */
  uint64_t numel;
  uint64_t elem_offset;
  float wd; /* decoupled weight decay for this tensor (0 for no_decay names) */
  float _pad;
} anc_adamw_tensor;

/* Scalars of one step, already float32 (the host materialises 1-beta and the bias
 * corrections once so that the kernel and the CPU oracle use identical values). */
typedef struct anc_adamw_scalars {
  float beta1, one_minus_beta1, beta2, one_minus_beta2, eps, lr, ibc1, ibc2;
} anc_adamw_scalars;

/* Builds the device tensor table + chunk table.  Replaces the per-tensor state dict
 * built in AdamW.__init__ (ancora/optim/adamw.py:74-86) and the per-tensor launch
 * loop in AdamW.step (adamw.py:92-97) / ResidentLayerTrain.step
 * (ancora/model/resident_train.py:349-353): one launch covers all tensors. */
ANC_API int anc_adamw_plan_create(anc_ctx *ctx, const anc_adamw_tensor *tensors, int n_tensors,
                                  int grad_dtype, anc_adamw_plan **out);
/* Restricts the plan to the arena slice [begin, end) (ZeRO-1 ownership; both
 * multiples of 8).  begin=0,end=UINT64_MAX restores the whole arena. */
ANC_API int anc_adamw_plan_set_range(anc_adamw_plan *plan, uint64_t begin, uint64_t end);
ANC_API int anc_adamw_plan_total(anc_adamw_plan *plan, uint64_t *arena_elems, uint64_t *owned_elems);
/* The fused step: replaces ct.launch(si, (R//otm,1,1), _adamw, ...) of
 * ancora/optim/adamw.py:23-41.  seed/step key the Philox stream (ANC_ROUND_SR). */
ANC_API int anc_adamw_step(anc_adamw_plan *plan, const anc_adamw_scalars *s, int rounding,
                           uint64_t seed, uint64_t step, void *stream);
/* Replayable form: the step number and the per-step scalars live in device memory, so the
 * same launch can be replayed from a CUDA graph.  The reference keeps its optimizer step
 * out of its captured graph because the bias corrections are kernel arguments that change
 * every step (ancora/model/resident_prefix_model.py:157-161).  table[k] holds the scalars
 * of step first_step + k (built by the host with the same float32 definitions as
 * anc_adamw_step); the device counter starts at first_step.  anc_adamw_step_scheduled uses
 * table[counter - first_step] and the counter as the SR step; advance != 0 appends a
 * one-thread kernel that increments the counter (give it on the last AdamW launch of a
 * step).  A counter outside the table sets status bit 0x8 and the launch does nothing. */
ANC_API int anc_adamw_plan_set_schedule(anc_adamw_plan *plan, const anc_adamw_scalars *table, int n,
                                        uint64_t first_step);
ANC_API int anc_adamw_step_scheduled(anc_adamw_plan *plan, int rounding, uint64_t seed, int advance,
                                     void *stream);
/* Points the device step counter at `step` (inside the uploaded table) without touching the
 * table, so a captured graph stays valid after eager steps or a restored state moved the
 * step number.  Synchronises `stream` first. */
ANC_API int anc_adamw_plan_set_counter(anc_adamw_plan *plan, uint64_t step, void *stream);
ANC_API int anc_adamw_plan_destroy(anc_adamw_plan *plan);

/* ------------------------------------------------------------------- Muon ---- */

/* One 2-D weight under Muon.  (K,N) is the stored orientation; Newton-Schulz runs
 * on the orientation with rows <= cols (ancora/optim/muon.py:72-74,99-100). */
typedef struct anc_muon_weight {
  float *buf;    /* momentum, f32 (K,N), the only persistent Muon state          */
  const void *g; /* gradient (K,N), bf16 bits or f32                             */
  float *p32;    /* fp32 master (K,N), updated in place                          */
  uint16_t *p16; /* bf16 weight (K,N) the forward reads, refreshed every step    */
  int32_t K, N;
  int32_t owner; /* ZeRO-1 owner rank of this matrix; -1 = always mine           */
  int32_t _pad;
} anc_muon_weight;

/* Groups weights by Newton-Schulz shape (min(K,N), max(K,N)), allocates the packed
 * bf16 scratch (X, Y, A, B per group, shared across groups) and encodes the TMA
 * tensor maps.  Replaces BatchedProjMuon.__init__ / MuonScratch / ExpertMuonScratch
 * (ancora/optim/muon.py:137-161,223-254; ancora/kernels/moe.py:404-421).
 * K and N must be multiples of 128 (reference: muon.py:98,172,233).
 * my_rank selects which weights this plan steps (owner == my_rank or owner < 0);
 * max_batch <= 0 batches a whole shape group at once. */
ANC_API int anc_muon_plan_create(anc_ctx *ctx, const anc_muon_weight *weights, int n_weights,
                                 int grad_dtype, int my_rank, int max_batch, anc_muon_plan **out);
/* Optional extra outputs the update writes from the freshly rounded bf16 weight (all
 * pointers may be NULL).  They replace sweeps the reference runs after every optimizer
 * step: the MXFP8 re-quantisation of the projection weights (ancora/kernels/quant.py:56-68
 * `_quant_mxfp8_w`, re-run because the step dirties them, model/resident_train.py:190-199,
 * 354-357) and the transposed expert weights for the backward (kernels/moe.py:371-377,593-596).
 *   fp8       (K,N) u8  E4M3 values, quantisation blocks of 32 along K
 *   fp8_scale (K/32,N) u8  E8M0 bytes: max(exponent(max|w| of the block) - 7, 0)
 *   p16_t     (N,K) bf16  transposed copy of p16
 *   fp8_t, fp8_scale_t  the same MXFP8 bytes transposed, (N,K) u8 + (N,K/32) u8, the layout of
 *             _quant_mxfp8_w_cm (ancora/kernels/quant.py:79-90) for a column-major B operand
 * fp8 needs 8-byte alignment, fp8_t and p16_t 16-byte; a values pointer and its scale pointer
 * are given together. */
typedef struct anc_muon_outputs {
  uint8_t *fp8;
  uint8_t *fp8_scale;
  uint16_t *p16_t;
  uint8_t *fp8_t;
  uint8_t *fp8_scale_t;
} anc_muon_outputs;
ANC_API int anc_muon_plan_create_ex(anc_ctx *ctx, const anc_muon_weight *weights,
                                    const anc_muon_outputs *outputs, int n_weights, int grad_dtype,
                                    int my_rank, int max_batch, anc_muon_plan **out);
/* One Muon step for every owned weight: momentum + Nesterov -> packed bf16 u
 * (transposed for tall weights) -> Frobenius normalisation -> ns_steps Newton-Schulz
 * iterations with coeffs[k] = (a,b,c) -> master update + bf16 refresh.  Replaces
 * BatchedProjMuon.step (ancora/optim/muon.py:256-277), ResidentMuon.step
 * (muon.py:180-201) and the expert branch of GroupedMoEFFN.step
 * (ancora/kernels/moe.py:578-588).  coeffs holds 3*ns_steps floats.  lr is a double
 * because the reference forms lr*sqrt(max(1,K/N)) in double before the single float32
 * rounding (muon.py:176,200). */
ANC_API int anc_muon_step(anc_muon_plan *plan, double lr, float momentum, int nesterov, int ns_steps,
                          const float *coeffs, float eps, void *stream);
/* The weights of a plan form shape groups (same Newton-Schulz shape), in order of first
 * registration; inside a group the weights keep their registration order.  A caller can step
 * any contiguous range of a group on its own -- to overlap that range's input copy, output
 * copy or exchange with the next range's compute using its own streams and events.
 * group_info = {weights in the group, largest range the scratch holds, M, N}.  Ranges share
 * the scratch, so they must be issued on ONE stream; every weight once per step.  Results do
 * not depend on how a group is cut into ranges. */
ANC_API int anc_muon_plan_num_groups(anc_muon_plan *plan, int *n);
ANC_API int anc_muon_plan_group_info(anc_muon_plan *plan, int group, int32_t info[4]);
ANC_API int anc_muon_step_range(anc_muon_plan *plan, int group, int first, int count, double lr,
                                float momentum, int nesterov, int ns_steps, const float *coeffs,
                                float eps, void *stream);
/* Per-phase device time accumulated over every anc_muon_step since the previous call
 * (timing enabled with anc_muon_plan_set_timing(plan, 1); CUDA events on the step's
 * stream, no synchronisation inside the step): ms spent in momentum, normalise,
 * Newton-Schulz GEMMs and update; ns_flops[0] the algorithmic (dense) FLOPs of those GEMMs,
 * ns_flops[1] the FLOPs the tensor cores executed (the symmetric phases compute only the
 * tiles on or below the diagonal); the launch count of the GEMM kernels.  The call waits
 * for the recorded events, then resets the accumulators. */
ANC_API int anc_muon_plan_set_timing(anc_muon_plan *plan, int on);
ANC_API int anc_muon_plan_last_timing(anc_muon_plan *plan, float ms[4], double ns_flops[2],
                                      int *ns_launches);
/* Self-test of the bounded waits (no counterpart in the reference): runs the chain kernel on
 * a zeroed 256x256 matrix with the first phase skipped, so that a tile waits for a
 * dependency nobody completes.  The wait gives up after `spin_limit` polls (<= 2^20), the
 * kernel drains and returns, and status bit 0x10 is set in the context's status word; the
 * context stays usable.  Synchronises the context's stream. */
ANC_API int anc_ns_chain_wait_selftest(anc_ctx *ctx, uint32_t spin_limit);
/* No reference counterpart.  The same for the staging ring of the AdamW / momentum / update sweeps:
 * one CTA waits, the way those kernels' computing warps do, for a stage nobody fills.  The wait gives
 * up after `tries` polls (<= 2^20, each may suspend about 2 us), status bit 0x1 is set, the kernel
 * returns and the context stays usable.  Synchronises the context's stream. */
ANC_API int anc_ring_wait_selftest(anc_ctx *ctx, uint32_t tries);
ANC_API int anc_muon_plan_scratch_bytes(anc_muon_plan *plan, uint64_t *bytes);
ANC_API int anc_muon_plan_destroy(anc_muon_plan *plan);

/* Bare batched Newton-Schulz on caller-owned packed buffers: replaces
 * newton_schulz_resident / newton_schulz_resident_e
 * (ancora/kernels/muon_ns.py:245-283,430-468).  X (E*M,N) bf16 bits is overwritten
 * with the result; A,B (E*M,M) and Y (E*M,N) are bf16 scratch; recip (E) f32.
 * M <= N, both multiples of 128.  All buffers 1024-byte aligned.
 * The whole chain is one persistent launch when M and N are multiples of 256 and
 * steps <= 16, else one launch per phase; both give the same bits. */
ANC_API int anc_ns_batched(anc_ctx *ctx, uint16_t *X, uint16_t *A, uint16_t *B, uint16_t *Y,
                           float *recip, int E, int M, int N, int steps, const float *coeffs,
                           float eps, void *stream);
/* Same, with the launch structure chosen by the caller: single_launch = 0 always runs one
 * launch per phase (what the reference's fused=False selects, muon_ns.py:277-283). */
ANC_API int anc_ns_batched_ex(anc_ctx *ctx, uint16_t *X, uint16_t *A, uint16_t *B, uint16_t *Y,
                              float *recip, int E, int M, int N, int steps, const float *coeffs,
                              float eps, int single_launch, void *stream);

/* One batched GEMM phase of the chain, exposed for kernel-level parity tests
 * (reference kernels: _e_gemm_nt_tril + _e_mirror, _e_gemm_axpy_tril + _e_mirror,
 * _e_gemm_axpy: ancora/kernels/muon_ns.py:331-384).
 *   mode 0: C = RNE(P P^T)                      P (E*M,K)  -> C (E*M,M), symmetric
 *   mode 1: C = RNE(alpha*P + beta*(P P^T))     P (E*M,M) symmetric -> C (E*M,M)
 *   mode 2: C = RNE(alpha*Q + beta*(P Q))       P (E*M,M), Q (E*M,N) -> C (E*M,N) */
ANC_API int anc_ns_gemm_phase(anc_ctx *ctx, int mode, const uint16_t *P, const uint16_t *Q,
                              uint16_t *C, int E, int M, int N, float alpha, float beta,
                              void *stream);

/* Muon elementwise kernels on their own (kernel-level parity tests; reference:
 * _muon_mom/_muon_mom_t and _muon_update_cast/_muon_update_cast_t,
 * ancora/kernels/muon_ns.py:177-242).  `transposed` selects the tall-weight forms
 * whose packed operand is (N,K). */
ANC_API int anc_muon_momentum(anc_ctx *ctx, float *buf, const void *g, int grad_dtype, uint16_t *u,
                              int K, int N, float momentum, int nesterov, int transposed,
                              void *stream);
ANC_API int anc_muon_update(anc_ctx *ctx, float *p32, uint16_t *p16, const uint16_t *O, int K, int N,
                            float lr_scale, int transposed, void *stream);
/* recip[e] = 1/(||X_e||_F + eps) by a fixed-order two-level reduction, then
 * X_e = RNE(X_e * recip[e]) in place (reference: _e_fro_recip + _e_scale,
 * ancora/kernels/muon_ns.py:387-406). */
ANC_API int anc_fro_normalize(anc_ctx *ctx, uint16_t *X, float *recip, int E, int M, int N, float eps,
                              void *stream);

/* Frobenius normalisation that allocates nothing.  No counterpart in the reference.
 *
 * Same kernels, same reduction order and therefore the same bits as anc_fro_normalize,
 * but the per-block partial sums go to a 256 KiB array built into the library's device
 * image rather than to a cudaMalloc'ed workspace, and no anc_ctx (whose creation
 * allocates) is needed.  It is for callers that must not enter the CUDA allocator at the
 * point of the call: a training loop whose device memory is owned entirely by a
 * framework's caching pool (a raw cudaMalloc there can fail for lack of un-pooled memory
 * or force a device-wide synchronisation), or a latency-critical step that has to stay
 * free of the implicit synchronisation cudaMalloc/cudaFree cause.  The caller still
 * supplies X (E*M rows of N bf16 values, normalised in place) and recip (E floats).
 *
 * Limits and rules:
 *   - E*M*N / 16384 must not exceed 65536 (2^30 elements per call); larger calls are
 *     rejected with ANC_E_INVALID and a message, nothing is launched.
 *   - The first call on each device looks up the array's device address (with that device
 *     made current) and remembers it; make that first call outside any stream capture.
 *   - All calls on one device share the one array.  Nothing in it has to start at zero
 *     (every slot is written before it is read within a call), but two calls whose
 *     kernels may overlap on the GPU (different streams, no dependency) would overwrite
 *     each other's partial sums: keep such calls ordered.
 *   - Every GPU that loads the library holds the 256 KiB until the process exits.
 * `device` is the CUDA device ordinal of X; `stream` a stream of that device (NULL = the
 * legacy default stream). */
ANC_API int anc_fro_normalize_static(int device, uint16_t *X, float *recip, int E, int M, int N,
                                     float eps, void *stream);

/* --------------------------------------------------------- gradient producer ---- */
/* One sweep that feeds the step its bf16 gradient:
 *   acc[i] = src[i] + acc[i]        (when src != NULL; one float32 add, the `_acc_f32` sweep of
 *                                    ancora/kernels/fused.py:242-249; src is f32 or bf16)
 *   g16[i] = bf16(acc[i] * scale)   (when g16 != NULL; ANC_ROUND_RNE, or ANC_ROUND_SR = the bit
 *                                    rule (bits + dither16) >> 16 of fused.py:159-161 that the
 *                                    reference applies in `_gemm_dx_sr`, dither from
 *                                    Philox4x32-10 keyed by (seed, step, (elem_offset + i) / 8))
 *   acc[i] = 0                      (when zero_after != 0: ready for the next accumulation)
 * The reference runs accumulation and downcast as separate sweeps.  `scale` is applied to
 * the bf16 output only (1/micro-batches, 1/world), never stored in acc.  elem_offset is the
 * global index of element 0, so a sharded arena draws the same bits as an unsharded one.
 * Use a seed different from the AdamW step's: both streams share the counter layout. */
ANC_API int anc_grad_accumulate(anc_ctx *ctx, float *acc, const void *src, int src_dtype, uint16_t *g16,
                                uint64_t numel, uint64_t elem_offset, float scale, int round_mode,
                                uint64_t seed, uint64_t step, int zero_after, void *stream);

/* ----------------------------------------------------------------- ZeRO-1 ---- */
/* No counterpart in the reference (single GPU, ancora README.md:93).  NCCL is
 * opened with dlopen at first use; nccl_path may be NULL (default search). */
#define ANC_NCCL_UNIQUE_ID_BYTES 128
ANC_API int anc_nccl_load(const char *nccl_path);
ANC_API int anc_nccl_unique_id(void *id128);
ANC_API int anc_comm_create(anc_ctx *ctx, const void *id128, int rank, int world, anc_comm **out);
ANC_API int anc_comm_destroy(anc_comm *comm);
/* In-place all-gather of equal contiguous slices: rank r owns
 * [r*elems_per_rank, (r+1)*elems_per_rank) of `arena` (bf16 elements). */
ANC_API int anc_comm_allgather_bf16(anc_comm *comm, uint16_t *arena, uint64_t elems_per_rank,
                                    void *stream);
/* In-place sum reduce-scatter of a gradient arena made of `world` equal contiguous slices
 * (bf16 or f32 elements): afterwards rank r's slice holds the sum over all ranks of that
 * slice (the other slices are unspecified).  Feeds the ZeRO-1 owner of each slice from
 * data-parallel replicas. */
ANC_API int anc_comm_reduce_scatter_grads(anc_comm *comm, void *arena, uint64_t elems_per_rank,
                                          int grad_dtype, void *stream);
ANC_API int anc_comm_barrier(anc_comm *comm, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ANCORA_B200_H_ */
