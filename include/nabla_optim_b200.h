/* nabla_optim_b200.h - C ABI of libnabla_optim_b200.so
 *
 * A B200 (sm_100a) implementation of the optimizer-step path of nabla-train:
 * SGD / momentum, Adam, AdamW, parameter groups, LR schedules, dynamic loss
 * scaling, global grad-norm clipping, a mixed-precision AdamW step and ZeRO-1
 * sharding over NCCL.  Every entry point replaces one Rust interface of the
 * reference; the citation beside each declaration is the file:line inside the
 * nabla project (v0.10.0) whose behaviour it reproduces.
 *
 * Conventions
 *   - Plain C99: opaque handle, pointers, sizes, doubles.  No exceptions, no
 *     abort() across the boundary.
 *   - Every function returns an nbo_status.  nbo_last_error() gives the text
 *     of the last failure on that handle (or of the last handle-less failure
 *     of the calling thread when passed NULL).
 *   - Parameter and gradient pointers are DEVICE pointers owned by the caller
 *     (what nabla's Tensor::device_ptr() returns,
 *     nabla-core/src/common/tensor/mod.rs:132-134); tensors are contiguous.
 *     The handle owns optimizer state (m, v, velocity, fp32 masters), its
 *     tables and its scratch, all on the device given to nbo_create.
 *   - Work is enqueued on the stream given to nbo_create (0 = the legacy
 *     default stream).  Functions that return a device-computed scalar
 *     (a norm, a skip decision) synchronise that stream before returning;
 *     all others are asynchronous.
 *   - One host thread drives a handle at a time.
 *   - There is no CPU fallback: without a CUDA device nbo_create fails.
 */
#ifndef NABLA_OPTIM_B200_H
#define NABLA_OPTIM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NBO_API __attribute__((visibility("default")))

typedef struct nbo_optimizer nbo_optimizer;

typedef enum {
    NBO_OK = 0,
    NBO_ERR_INVALID = 1, /* bad argument: null/misaligned pointer, count mismatch ... */
    NBO_ERR_CUDA = 2,    /* a CUDA runtime call failed                              */
    NBO_ERR_NCCL = 3,    /* an NCCL call failed                                     */
    NBO_ERR_TIMEOUT = 4, /* a bounded wait ran out                                  */
    NBO_ERR_STATE = 5,   /* call order violated (e.g. step before set_tensors)      */
    NBO_ERR_NOMEM = 6    /* device or host allocation failed                        */
} nbo_status;

/* OptimKind, same order as nabla-train/src/optim/core.rs:46-51. */
typedef enum { NBO_ADAMW = 0, NBO_ADAM = 1, NBO_SGD = 2 } nbo_kind;

/* Element type of the caller's params/grads. */
typedef enum {
    NBO_F32 = 0,       /* params, grads and state all fp32 (Optimizer<f32, Cuda>)     */
    NBO_MIXED_BF16 = 1, /* bf16 params+grads, fp32 master/m/v held by the handle      */
    NBO_MIXED_BF16_F32GRAD = 2 /* bf16 params, fp32 grads (e.g. accumulated over
                                  micro-batches in fp32), fp32 master/m/v                 */
} nbo_precision;

/* One parameter group = ParamGroupConfig (nabla-train/src/optim/groups.rs:40-51).
 * A plain optimizer is a handle with a single group. */
typedef struct {
    int32_t kind;        /* nbo_kind */
    double lr;
    double beta1;        /* Adam/AdamW; defaults .9  (alg.rs:29-37)  */
    double beta2;        /*             defaults .999                */
    double eps;          /*             defaults 1e-8                */
    double weight_decay; /* AdamW default 0.01; Sgd default 0; ignored by Adam */
    double momentum;     /* Sgd only (alg.rs:324-329)                */
} nbo_group_config;

/* GradScalerState (nabla-train/src/optim/core.rs:326-332). */
typedef struct {
    double scale;
    double growth_factor;
    double backoff_factor;
    uint64_t growth_interval;
    uint64_t consecutive_ok;
} nbo_scaler_state;

/* LrSchedule (nabla-train/src/optim/core.rs:101-121). */
typedef enum {
    NBO_SCHED_COSINE = 0,
    NBO_SCHED_LINEAR = 1,
    NBO_SCHED_ONECYCLE = 2,
    NBO_SCHED_STEP = 3
} nbo_schedule_kind;

typedef struct {
    int32_t kind;          /* nbo_schedule_kind               */
    uint64_t warmup_steps; /* cosine, linear                  */
    uint64_t total_steps;  /* cosine, linear, onecycle        */
    double min_lr;         /* cosine                          */
    double max_lr;         /* onecycle                        */
    double pct_start;      /* onecycle                        */
    uint64_t step_size;    /* step                            */
    double gamma;          /* step                            */
} nbo_lr_schedule;

/* Outcome of one mixed-precision / ZeRO-1 step. */
typedef struct {
    int32_t applied;      /* 1 = update applied, 0 = skipped (non-finite grads)       */
    int32_t nonfinite;    /* 1 = a non-finite gradient was seen                        */
    double grad_norm;     /* pre-clip global L2 norm of the unscaled grads; 0 when
                             max_norm <= 0 (no norm is taken then, trainer.rs:501-503) */
    double loss_scale;    /* scale to use for the NEXT backward pass                   */
    uint64_t step_count;  /* optimizer step count after this call (group 0)            */
} nbo_step_result;

/* ---- library ------------------------------------------------------------ */

/* ABI version of this header; bumps on any incompatible change. */
NBO_API int32_t nbo_abi_version(void);

/* Text of the last error on `h`; with h == NULL, the calling thread's last
 * handle-less error.  Never NULL. */
NBO_API const char *nbo_last_error(const nbo_optimizer *h);

/* ---- lifecycle ---------------------------------------------------------- */

/* Creates an optimizer bound to CUDA device `device` and to `stream`
 * (a cudaStream_t; NULL = legacy default stream; nabla's own stream is
 * cuda_compute_stream(), nabla-core/src/cuda_hip/cuda/core.rs:618-620).
 * Replaces the constructors Sgd::new / Adam::new / AdamW::new /
 * GroupOptimizer::from_named_params (alg.rs:20-40,181-201,319-331;
 * groups.rs:168-226) together with nbo_add_group and nbo_set_tensors. */
NBO_API int32_t nbo_create(int32_t device, void *stream, nbo_optimizer **out);
NBO_API int32_t nbo_destroy(nbo_optimizer *h);

/* Appends a parameter group; *group_id receives its index (0, 1, ...).
 * Must precede nbo_set_tensors.  (groups.rs:40-51, 204-218) */
NBO_API int32_t nbo_add_group(nbo_optimizer *h, const nbo_group_config *cfg, int32_t *group_id);

/* Declares the parameter list: `n` tensors with `numel[i]` elements, tensor i
 * belonging to group `group_ids[i]` (NULL = all in group 0).  Allocates and
 * zeroes the state (m, v / velocity; plus fp32 masters for NBO_MIXED_BF16),
 * as the constructors do from `param_shapes` (alg.rs:20-40).  Zero-element
 * tensors are allowed. */
NBO_API int32_t nbo_set_tensors(nbo_optimizer *h, uint64_t n, const uint64_t *numel,
                                const int32_t *group_ids, int32_t precision);

/* ---- Optimizer trait (nabla-train/src/optim/core.rs:9-44) ---------------- */

/* Optimizer::step(params, grads) for fp32 handles.  `n` must equal the count
 * given to nbo_set_tensors, else NBO_ERR_INVALID with the reference's
 * "params count mismatch" wording (alg.rs:110-119).  Pointers may change from
 * call to call; an unchanged set reuses the device-resident table.
 * A tensor whose parameter or gradient pointer is not 16-byte aligned (any
 * allocator's own blocks are) is still updated correctly, element by element,
 * at about a third of the speed of an aligned one.
 * SGD: alg.rs:382-416.  Adam: alg.rs:254-291.  AdamW: alg.rs:109-150. */
NBO_API int32_t nbo_step(nbo_optimizer *h, uint64_t n, void *const *params,
                         const void *const *grads);

/* adamw_step (alg.rs:431-469): AdamW on ONE fp32 tensor whose moments `m` and `v`
 * are owned by the caller (device pointers, n floats each); `step` is the
 * 1-based step number used for the bias corrections.  Needs no handle and
 * allocates nothing: the tensor description travels in the kernel arguments.
 * Asynchronous on `stream`. */
NBO_API int32_t nbo_adamw_step(int32_t device, void *stream, void *param, const void *grad, float *m,
                               float *v, uint64_t n, double lr, double beta1, double beta2, double eps,
                               double weight_decay, uint64_t step);

/* Optimizer::reset: zero the state and the Adam step counts (alg.rs:152-162). */
NBO_API int32_t nbo_reset(nbo_optimizer *h);

/* Optimizer::set_lr.  One group: overwrite lr (alg.rs:164-166).  Several
 * groups: group k gets base_lr[k] * lr / base_lr[0]; if base_lr[0] <= 0 every
 * group gets `lr` (groups.rs:301-312). */
NBO_API int32_t nbo_set_lr(nbo_optimizer *h, double lr);
NBO_API int32_t nbo_get_lr(const nbo_optimizer *h, int32_t group_id, double *lr);

/* zero_grad (nabla-ml/src/autograd/ops.rs:1668-1673): every gradient of the
 * bound list becomes +0 (one kernel over the table on the stream).  The element
 * size follows the handle's precision: bf16 gradients for NBO_MIXED_BF16, fp32
 * otherwise. */
NBO_API int32_t nbo_zero_grad(nbo_optimizer *h, uint64_t n, void *const *grads);

/* Gradient accumulation, accum[i] = accum[i] + grads[i] elementwise in fp32
 * (the `buf[i] = &buf[i] + g` loop of Trainer, nabla-train/src/trainer.rs:262-266).
 * The handle's table holds the accumulation buffers in its parameter column, so
 * use a handle of its own for this (any group kind; no optimizer state is touched).
 * Asynchronous. */
NBO_API int32_t nbo_accumulate_grads(nbo_optimizer *h, uint64_t n, void *const *accum,
                                     const void *const *grads);

/* ---- OptimState (nabla-train/src/optim/core.rs:64-79) -------------------- */

/* Step count of a group (AdamW::step_count, alg.rs:76-79). */
NBO_API int32_t nbo_step_count(const nbo_optimizer *h, int32_t group_id, uint64_t *count);
NBO_API int32_t nbo_set_step_count(nbo_optimizer *h, int32_t group_id, uint64_t count);
NBO_API int32_t nbo_get_group(const nbo_optimizer *h, int32_t group_id, nbo_group_config *cfg);
NBO_API int32_t nbo_set_group(nbo_optimizer *h, int32_t group_id, const nbo_group_config *cfg);

/* State tensors.  `which`: 0 = m (Adam/AdamW), 1 = v (Adam/AdamW) or the
 * velocity (SGD - the reference names it v{i} too, alg.rs:620-640),
 * 2 = fp32 master (mixed precision only).  `dst`/`src` are HOST buffers of
 * numel[tensor] floats.  Synchronous. */
NBO_API int32_t nbo_state_export(nbo_optimizer *h, uint64_t tensor, int32_t which, float *dst);
NBO_API int32_t nbo_state_import(nbo_optimizer *h, uint64_t tensor, int32_t which,
                                 const float *src);

/* ---- GradScaler / clip_grad_norm on fp32 gradients ----------------------- */

/* GradScaler state (core.rs:334-349,390-413).  A fresh handle holds the
 * defaults: 65536, x2 every 2000 clean steps, x0.5 on overflow. */
NBO_API int32_t nbo_scaler_get(const nbo_optimizer *h, nbo_scaler_state *out);
NBO_API int32_t nbo_scaler_set(nbo_optimizer *h, const nbo_scaler_state *in);

/* GradScaler::unscale_and_update (core.rs:351-388) on fp32 device gradients:
 * non-finite test on the still-scaled values; on a hit the scale backs off,
 * the counter resets, every gradient becomes zero and *ok = 0; otherwise each
 * element is multiplied by f32(1/scale), the counter advances (growing the
 * scale at the interval) and *ok = 1.  Synchronises the stream. */
NBO_API int32_t nbo_unscale_and_update(nbo_optimizer *h, uint64_t n, void *const *grads,
                                       int32_t *ok);

/* clip_grad_norm (nabla-train/src/trainer.rs:500-523) on fp32 device
 * gradients: *norm = sqrt(sum g^2) accumulated in f64; if norm > max_norm and
 * norm > 0 every element is multiplied by f32(max_norm / norm).  max_norm <= 0
 * returns 0.0 and changes nothing.  Synchronises the stream. */
NBO_API int32_t nbo_clip_grad_norm(nbo_optimizer *h, uint64_t n, void *const *grads,
                                   double max_norm, double *norm);

/* Trainer::has_non_finite (trainer.rs:387-400) plus the norm in one pass:
 * *nonfinite = 1 if any element is inf/NaN; *norm = global L2 norm (undefined
 * when non-finite).  Does not modify the gradients.  Synchronises. */
NBO_API int32_t nbo_grad_norm(nbo_optimizer *h, uint64_t n, const void *const *grads,
                              double *norm, int32_t *nonfinite);

/* The norm / non-finite pass for callers that must not allocate: code running
 * while a stream capture elsewhere in the process (global capture mode)
 * makes cudaMalloc illegal, under an allocator that owns all device memory
 * (nabla's pool allocator forbids raw cudaMalloc beside it), or with a fixed
 * memory budget.  It has no counterpart in the reference.  It needs no handle
 * and calls no cudaMalloc / cudaFree or any allocating routine: all scratch
 * (table, chunk list, per-CTA partials, ticket) lives in one fixed
 * ~536 KiB array in the library's device image, which every GPU that loads
 * the library holds until exit.
 *   grads     one contiguous DEVICE buffer of n elements, fp32 (NBO_F32) or
 *             bf16 (NBO_MIXED_BF16); n <= 134,217,728 (2^27), else
 *             NBO_ERR_INVALID - larger buffers need a handle and nbo_grad_norm
 *   inv_scale each element is multiplied by it (rounded to f32) before it is
 *             squared; the non-finite test is on the unmultiplied value
 *   out_dev   caller-owned DEVICE buffer of two doubles, written on `stream`:
 *             out_dev[0] = sum of squares (the norm is its sqrt),
 *             out_dev[1] = 1.0 if any element is inf/NaN else 0.0
 * Asynchronous on `stream`.  The first call on a device looks up the device
 * address of the scratch array (cudaGetSymbolAddress) and has the driver load
 * the kernels of both precisions, and should therefore be made - once per
 * device, either precision - before any stream capture begins and before the
 * caller's memory budget is fixed.  Every call shares the one scratch
 * array: calls that may overlap on the GPU (different streams without an
 * ordering between them) race on it and must be serialised by the caller. */
NBO_API int32_t nbo_grad_norm_noalloc(int32_t device, void *stream, const void *grads, uint64_t n,
                                      int32_t precision, float inv_scale, double *out_dev);

/* ---- mixed-precision AdamW step ----------------------------------------- */

/* Seeds the fp32 masters from the caller's bf16 params (exact widening), or
 * from fp32 host values via nbo_state_import(which = 2). */
NBO_API int32_t nbo_init_master_from_params(nbo_optimizer *h, uint64_t n,
                                            const void *const *params_bf16);

/* One fused training-step tail for NBO_MIXED_BF16 handles, in the order of
 * Trainer::train_epoch_with_max_steps (trainer.rs:230-283):
 *   GradScaler::unscale_and_update (if use_scaler) -> non-finite skip ->
 *   clip_grad_norm(max_norm) (if max_norm > 0) -> Adam/AdamW on the fp32
 *   masters -> bf16 params = round-to-nearest-even of the masters.
 * The gradients are read twice (norm/non-finite pass, update pass) and never
 * written.  A skipped step changes nothing but the scaler.  Synchronises the
 * stream to fill `result`. */
NBO_API int32_t nbo_step_mixed(nbo_optimizer *h, uint64_t n, void *const *params_bf16,
                               const void *const *grads_bf16, int32_t use_scaler,
                               double max_norm, nbo_step_result *result);

/* The same step without any host round trip, for callers that keep the GPU fed
 * (or capture the optimizer phase into a CUDA graph): step counters, bias
 * corrections and the GradScaler bookkeeping are computed on the device from a
 * device-resident copy of the state, so nothing is read back and every launch
 * has constant arguments.  A skipped step is decided and accounted for on the
 * device (trainer.rs:230-237).  Up to 32 groups; unsharded handles only.
 * The host-side view (nbo_step_count, nbo_scaler_get, nbo_get_lr ...) is
 * brought up to date by any of those calls or by nbo_step_mixed_collect, each
 * of which synchronises the stream; host-side changes (nbo_set_lr,
 * nbo_scaler_set ...) are sent down again by the next asynchronous step.
 * Arithmetic and results are identical to nbo_step_mixed. */
NBO_API int32_t nbo_step_mixed_async(nbo_optimizer *h, uint64_t n, void *const *params_bf16,
                                     const void *const *grads_bf16, int32_t use_scaler,
                                     double max_norm);

/* Outcome of the most recent asynchronous step (and the number of such steps
 * the device has completed since the last hand-over).  Synchronises. */
NBO_API int32_t nbo_step_mixed_collect(nbo_optimizer *h, nbo_step_result *result,
                                       uint64_t *steps_enqueued);

/* The same step for a caller whose gradients and parameters live in HOST
 * memory, as every tensor of nabla's CPU backend does (nabla-core/src/cpu/
 * mod.rs; the optimizer reads `grads[i]` and writes `params[i]` in place,
 * alg.rs:109-150).  `params_dev` / `grads_dev` are device staging buffers of
 * the declared sizes (what nbo_step_mixed takes); `params_host` /
 * `grads_host` hold one host pointer per tensor.  The chunk list is cut into
 * slices of about `slice_elems` elements (0 = 32 Mi) and pipelined over three
 * streams - gradients host->device, update, parameters device->host - so both
 * PCIe directions run at once and the update hides behind them; the fp32
 * master / m / v state stays in HBM.  With use_scaler or max_norm > 0 every
 * gradient is copied in first (the decision needs all of them); a skipped
 * step copies nothing out.  Host buffers should be page-locked, otherwise
 * the copies do not overlap.  The call returns when the host parameters are
 * complete.  Same kernels and arithmetic as nbo_step_mixed: results are
 * bit-identical.  Unsharded mixed-precision handles. */
NBO_API int32_t nbo_step_mixed_host(nbo_optimizer *h, uint64_t n, void *const *params_dev,
                                    const void *const *grads_dev, void *const *params_host,
                                    const void *const *grads_host, uint64_t slice_elems,
                                    int32_t use_scaler, double max_norm, nbo_step_result *result);

/* ---- LR schedules (pure host math) --------------------------------------- */

/* lr_at_step (nabla-train/src/optim/core.rs:130-173); `step` is the trainer's
 * step before its increment. */
NBO_API int32_t nbo_lr_at_step(const nbo_lr_schedule *schedule, double base_lr, uint64_t step,
                               double *lr);

/* ---- ZeRO-1 over NCCL (replaces nabla-train/src/dist.rs:7-44) ------------ */

/* 128-byte NCCL unique id; rank 0 creates it and ships it to the other ranks
 * by any host channel. */
NBO_API int32_t nbo_zero1_unique_id(uint8_t id_out[128]);

/* Shard geometry for `total` elements over `world` ranks: every rank owns
 * *shard_elems elements, a multiple of 8 (so bf16 shards are 16-byte aligned);
 * *padded_total = world * *shard_elems >= total.  Pure host arithmetic. */
NBO_API int32_t nbo_zero1_geometry(uint64_t total, int32_t world, uint64_t *shard_elems,
                                   uint64_t *padded_total);

/* Declares the parameter list as one flat bf16 bucket in list order (tensor i
 * starts where tensor i-1 ends; the bucket is padded_total elements long) and
 * joins the NCCL communicator.  The handle then holds state only for the
 * intersection of every tensor with this rank's shard
 * [rank*shard, (rank+1)*shard).  Replaces nbo_set_tensors.  world == 1 makes
 * no NCCL call at all. */
NBO_API int32_t nbo_zero1_init(nbo_optimizer *h, uint64_t n, const uint64_t *numel,
                               const int32_t *group_ids, int32_t rank, int32_t world,
                               const uint8_t unique_id[128]);

/* Host-side time limit (seconds, default 600) for joining the communicator and
 * for the completion of each sharded step.  When it runs out - a rank never
 * arrived, or stopped taking part - the communicator is aborted, the call
 * returns NBO_ERR_TIMEOUT, the CUDA context stays usable and later sharded
 * steps on this handle return NBO_ERR_STATE.  May be called before or after
 * nbo_zero1_init.  The reference's counterpart is the Err("send failed") of
 * its channel pair (nabla-train/src/dist.rs:37-40). */
NBO_API int32_t nbo_zero1_set_timeout(nbo_optimizer *h, double seconds);

/* Seeds this rank's fp32 master shard from the flat bf16 param bucket. */
NBO_API int32_t nbo_zero1_init_master(nbo_optimizer *h, const void *params_flat_bf16);

/* One ZeRO-1 step on the flat buckets (both padded_total bf16 elements):
 *   reduce-scatter(grads, sum or mean) -> shard norm^2 + non-finite flag ->
 *   all-gather of the per-rank scalars, combined in rank order -> scaler /
 *   skip / clip decision (identical on every rank) -> fused local update of
 *   the shard -> all-gather(params).
 * `average` != 0 divides the reduced gradients by `world` (ncclAvg). */
NBO_API int32_t nbo_zero1_step(nbo_optimizer *h, void *params_flat_bf16, void *grads_flat_bf16,
                               int32_t average, int32_t use_scaler, double max_norm,
                               nbo_step_result *result);

/* nbo_step_mixed_host for a ZeRO-1 handle: the caller's gradients and parameters are host tensors (one
 * pointer per tensor of the declared list, n = that list's length; alg.rs:109-150 reads `grads[i]` and
 * writes `params[i]` in host memory on nabla's CPU backend) and the two flat buckets are device staging.
 *   world == 1: exactly nbo_step_mixed_host on the flat buckets.
 *   world  > 1: the buckets must be the ones given to nbo_zero1_attach_symmetric.  Every rank passes its own
 *     gradients for the WHOLE list (data-parallel replicas) and receives the updated parameters of ITS
 *     shard (the elements nbo_zero1_shard reports) in `params_host`; the other elements of `params_host`
 *     are not written.  The shard is cut into slices of about `slice_elems` elements (0 = 32 Mi / world);
 *     per slice every rank copies in its gradients for that slice of every rank's shard, a stream-ordered
 *     barrier follows, the fused kernel reduces / updates / publishes the slice over NVLink, and the slice's
 *     parameters are copied out - so PCIe (both directions) and NVLink work at the same time.  With
 *     use_scaler or max_norm > 0 all gradients are copied in first and a skipped step copies nothing out.
 *     Results are bit-identical to nbo_zero1_step_fused on the same gradients.  One bounded host wait per
 *     step (nbo_zero1_set_timeout).
 * `average` as in nbo_zero1_step (ignored when world == 1). */
NBO_API int32_t nbo_zero1_step_host(nbo_optimizer *h, void *params_flat_dev, void *grads_flat_dev,
                                    uint64_t n, void *const *params_host,
                                    const void *const *grads_host, uint64_t slice_elems,
                                    int32_t average, int32_t use_scaler, double max_norm,
                                    nbo_step_result *result);

/* The same step with the two collectives fused into the kernels over NVLink /
 * NVSwitch peer memory instead of issued as separate NCCL passes.  Both flat
 * buckets must live in symmetric memory: every rank's bucket mapped into every
 * process (`*_peers[r]` = this process's mapping of rank r's bucket, with
 * `*_peers[rank] == *_local`), optionally with an NVSwitch multicast mapping
 * (`*_mc`, may be NULL).  transport: 0 = choose (multicast when available and
 * world >= 5, else peer), 1 = plain peer loads/stores, 2 = multimem
 * ld_reduce / st through the switch.  World 2..16.  Replaces
 * nabla-train/src/dist.rs:36-43 together with the update it feeds. */
NBO_API int32_t nbo_zero1_attach_symmetric(nbo_optimizer *h, void *grads_local,
                                           void *const *grads_peers, void *grads_mc,
                                           void *params_local, void *const *params_peers,
                                           void *params_mc, int32_t transport);

/* Symmetric buckets without any framework.  nbo_zero1_attach_symmetric needs every rank's bucket mapped
 * into every process; these calls make such buckets with the CUDA virtual-memory API: one allocation per
 * rank, mapped over NVLink into all ranks of the node and, where the fabric supports it (and
 * want_multicast != 0), bound to one NVSwitch multicast object.  The ranks are processes of one node.
 *   nbo_symm_token  rank 0 makes a 16-byte token and ships it to the other ranks by any host channel
 *                   (as with the NCCL unique id); one token serves any number of allocations.
 *   nbo_symm_alloc  collective: every rank calls it with the same token, tag, world and size.  The
 *                   allocations' shareable handles are file descriptors, which a byte channel cannot
 *                   carry, so the library passes them itself over abstract unix sockets named after
 *                   token and tag (two allocations alive at once need different tags).  Every wait is
 *                   bounded by timeout_s (<= 0: 60 s); on expiry NBO_ERR_TIMEOUT and nothing is kept.
 *   nbo_symm_pointers  this process's mappings: *local (== peers[rank]), peers[0..world), and *multicast
 *                   (NULL when the fabric has none) - the arguments of nbo_zero1_attach_symmetric.
 *   nbo_symm_free   unbinds from the multicast object, unmaps and releases.  Every rank must call it
 *                   (after its last use, e.g. after a barrier) before it exits: a process must not end
 *                   while its memory is bound to a multicast object.
 * The memory is ordinary device memory with undefined initial contents; world <= 16.  Replaces the in-process
 * channel pair of nabla-train/src/dist.rs:7-34 as the way replicas reach each other's buffers. */
typedef struct nbo_symm nbo_symm;
NBO_API int32_t nbo_symm_token(uint8_t token_out[16]);
NBO_API int32_t nbo_symm_alloc(int32_t device, int32_t rank, int32_t world, uint64_t bytes,
                               const uint8_t token[16], int32_t tag, int32_t want_multicast,
                               double timeout_s, nbo_symm **out);
NBO_API int32_t nbo_symm_pointers(const nbo_symm *s, void **local, void **peers, void **multicast);
NBO_API int32_t nbo_symm_free(nbo_symm *s);

/* One step on the attached buckets: stream-ordered barrier -> [reduce + norm
 * pass when loss scaling or clipping is on, per-rank scalars all-gathered and
 * combined in rank order] -> one kernel per group that reads the gradients of
 * this rank's shard from every rank, updates the fp32 state and writes the
 * bf16 params into every rank's bucket -> barrier.  Everything is enqueued
 * without waiting; the kernels that touch other ranks' memory verify on the
 * device that the barrier before them completed (and do nothing otherwise), and
 * the host waits once, at the end, with the nbo_zero1_set_timeout limit.  The
 * reduced gradients are left in this rank's slice of its own gradient bucket,
 * as nbo_zero1_step leaves them, unless nbo_zero1_keep_reduced_grads(h, 0).
 * Same result structure and skip semantics as nbo_zero1_step. */
NBO_API int32_t nbo_zero1_step_fused(nbo_optimizer *h, int32_t average, int32_t use_scaler,
                                     double max_norm, nbo_step_result *result);

/* nbo_zero1_step_fused without any host wait, the sharded counterpart of nbo_step_mixed_async: step
 * counters, bias corrections and the GradScaler bookkeeping advance in the handle's device-resident state,
 * every launch has constant arguments, and the skip decision (trainer.rs:230-237) is taken and accounted
 * for on the device from the all-gathered per-rank sums, identically on every rank.  The call returns as
 * soon as the work is enqueued, so the caller can go on to its next backward pass.
 * nbo_step_mixed_collect hands the state back and reports the last outcome; on a sharded handle its wait is
 * bounded by nbo_zero1_set_timeout, which is where a rank that stopped taking part is noticed.
 * Arithmetic and results are those of nbo_zero1_step_fused. */
NBO_API int32_t nbo_zero1_step_fused_async(nbo_optimizer *h, int32_t average, int32_t use_scaler,
                                           double max_norm);

/* Whether the fused step also writes the reduced gradient into this rank's
 * slice of its own gradient bucket (default 1, what an in-place reduce-scatter
 * leaves behind; nabla-train/src/dist.rs:36-43 hands the mean back to the
 * caller).  A caller that zeroes or overwrites the gradients after the step
 * anyway can switch it off and save 2 bytes of HBM writes per element; a step
 * with loss scaling or clipping always writes them (its two passes need them). */
NBO_API int32_t nbo_zero1_keep_reduced_grads(nbo_optimizer *h, int32_t on);

/* This rank's shard range in bucket elements and the number of table entries
 * (tensor pieces) it holds. */
NBO_API int32_t nbo_zero1_shard(const nbo_optimizer *h, uint64_t *begin, uint64_t *end,
                                uint64_t *pieces);

/* Copies this rank's fp32 state shard to a HOST buffer of shard_elems floats;
 * `which` as in nbo_state_export.  Synchronous. */
NBO_API int32_t nbo_zero1_state_export(nbo_optimizer *h, int32_t which, float *dst);

/* The reverse: loads this rank's fp32 state shard from a HOST buffer of
 * shard_elems floats (resume from a checkpoint; OptimState::load_state_tensors,
 * nabla-train/src/optim/alg.rs:487-518, applied to the slice this rank owns). */
NBO_API int32_t nbo_zero1_state_import(nbo_optimizer *h, int32_t which, const float *src);

/* ---- introspection ------------------------------------------------------- */

/* Device timing of the kernels inside nbo_step / nbo_step_mixed / nbo_zero1_step.
 * With `on` != 0 the handle records CUDA events on its stream around the norm
 * pass and around the update launches of every later step (two extra event
 * records each; no synchronisation is added).  nbo_profile_last returns the
 * elapsed milliseconds of the most recent step's norm pass (0 if it had none)
 * and update launches; it synchronises the stream.  No counterpart in the
 * reference, whose profiler wraps host timers around whole ops
 * (nabla-train/src/profiler.rs:177-197). */
NBO_API int32_t nbo_profile(nbo_optimizer *h, int32_t on);
NBO_API int32_t nbo_profile_last(nbo_optimizer *h, float *norm_ms, float *update_ms);

/* Plain device-to-device copy of `bytes` bytes with 128-bit loads and stores
 * issued by the SMs (persistent grid), asynchronous on `stream`; `src` or `dst`
 * may be another GPU's memory mapped into this process.  It is the yardstick
 * the NVLink share of the fused sharded step is measured against (same kind of
 * access, nothing else to do); it has no counterpart in the reference.
 * Pointers and size must be multiples of 16 bytes. */
NBO_API int32_t nbo_copy_probe(int32_t device, void *stream, void *dst, const void *src,
                               uint64_t bytes);

/* Number of kernels the handle has launched since creation (all entry
 * points), and the number of chunks in its multi-tensor table. */
NBO_API int32_t nbo_launch_count(const nbo_optimizer *h, uint64_t *launches);
NBO_API int32_t nbo_table_info(const nbo_optimizer *h, uint64_t *tensors, uint64_t *chunks,
                               uint64_t *uploads);

#ifdef __cplusplus
}
#endif
#endif /* NABLA_OPTIM_B200_H */
