// The one translation unit that holds the device code, plus the launchers the
// host code calls.  Grids are persistent: SM count x resident CTAs per SM
// (from the occupancy calculator), capped by the number of chunks.
#include <math.h>

#include <map>
#include <mutex>

#include "internal.h"
#include "kernels.cuh"
#include "fused_nvlink.cuh"

namespace nbo {

// max_per_sm caps the resident CTAs used per SM: the multi-stream update kernels stream fastest at 2
// (measured for SGD-momentum on 0.75 G elements: 6170 / 6443 / 6170 / 6115 GB/s at 1 / 2 / 3 / 4 CTAs per SM;
// the Adam kernels are register-limited to 2 anyway).
static int grid_for(const nbo_optimizer *h, uint32_t nchunks, const void *kernel, int max_per_sm = 0)
{
    static std::map<const void *, int> cache;  // resident CTAs per SM, per kernel
    static std::mutex cache_lock;               // handles may be driven from different host threads
    std::lock_guard<std::mutex> guard(cache_lock);
    int per_sm;
    auto it = cache.find(kernel);
    if (it == cache.end()) {
        per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kBlock, 0) != cudaSuccess ||
            per_sm < 1)
            per_sm = 1;
        cache[kernel] = per_sm;
    } else {
        per_sm = it->second;
    }
    if (max_per_sm > 0 && per_sm > max_per_sm) per_sm = max_per_sm;
    long long g = (long long)h->sm_count * per_sm;
    if (g > h->max_grid) g = h->max_grid;
    if (g > (long long)nchunks) g = nchunks;
    return (int)(g < 1 ? 1 : g);
}

static int32_t launched(nbo_optimizer *h)
{
    h->launches += 1;
    NBO_CUDA(h, cudaGetLastError());
    return NBO_OK;
}

int32_t launch_adam_f32(nbo_optimizer *h, uint32_t cb, uint32_t nc, const AdamHP &hp)
{
    if (nc == 0) return NBO_OK;
    int grid = grid_for(h, nc, (const void *)adam_f32_kernel);
    adam_f32_kernel<<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks + cb, nc, hp);
    return launched(h);
}

int32_t launch_sgd_f32(nbo_optimizer *h, uint32_t cb, uint32_t nc, const SgdHP &hp)
{
    if (nc == 0) return NBO_OK;
    if (hp.use_mu) {
        int grid = grid_for(h, nc, (const void *)sgd_f32_kernel<true>, 2);
        sgd_f32_kernel<true><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks + cb, nc, hp);
    } else {
        int grid = grid_for(h, nc, (const void *)sgd_f32_kernel<false>, 2);
        sgd_f32_kernel<false><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks + cb, nc, hp);
    }
    return launched(h);
}

template <bool kScaled, bool kGradF32>
static int32_t launch_adam_mixed_one(nbo_optimizer *h, uint32_t cb, uint32_t nc, const AdamHP &hp,
                                     const StepCtrl *ctrl, const AdamHP *hp_dev)
{
    int grid = grid_for(h, nc, (const void *)adam_mixed_kernel<kScaled, kGradF32>);
    adam_mixed_kernel<kScaled, kGradF32><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks + cb, nc, hp,
                                                                        ctrl, hp_dev);
    return launched(h);
}

int32_t launch_adam_mixed(nbo_optimizer *h, uint32_t cb, uint32_t nc, const AdamHP &hp, bool with_ctrl)
{
    if (nc == 0) return NBO_OK;
    const bool gf32 = h->precision == NBO_MIXED_BF16_F32GRAD;
    const StepCtrl *ctrl = with_ctrl ? h->d_ctrl : nullptr;
    if (with_ctrl || hp.inv_scale != 1.0f)
        return gf32 ? launch_adam_mixed_one<true, true>(h, cb, nc, hp, ctrl, nullptr)
                    : launch_adam_mixed_one<true, false>(h, cb, nc, hp, ctrl, nullptr);
    return gf32 ? launch_adam_mixed_one<false, true>(h, cb, nc, hp, nullptr, nullptr)
                : launch_adam_mixed_one<false, false>(h, cb, nc, hp, nullptr, nullptr);
}

// Every norm launch of a handle uses the same grid whichever kernel variant runs (generic, per-element flag,
// power-of-two scale) of the same element type: the per-thread accumulation order and the order of the per-CTA partials depend on the
// grid alone, so the synchronous and the asynchronous step, and a step before and after the loss scale leaves
// the power-of-two fast path, produce the same f64 sum for the same gradients.
static int norm_grid(const nbo_optimizer *h, bool bf16)
{
    uint32_t units = (h->nchunks + kNormBatch - 1) / kNormBatch;  // one loop iteration takes kNormBatch chunks
    long long g = (long long)h->sm_count * (bf16 ? kNormCtasPerSm : kNormCtasPerSmF32);
    if (g > h->max_grid) g = h->max_grid;
    if (g > (long long)units) g = units;
    return (int)(g < 1 ? 1 : g);
}

template <bool kBf16, bool kCheckEach>
static void launch_norm_one(nbo_optimizer *h, float inv_scale, double max_norm, int finalize, const NormOut &out,
                            const float *inv_scale_dev = nullptr)
{
    int grid = norm_grid(h, kBf16);
    norm_kernel<kBf16, kCheckEach><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks,
                                                                  inv_scale, max_norm, finalize, out, inv_scale_dev);
}

// k with inv_scale == 2^-k exactly and 0 <= k <= kPow2MaxK; -1 otherwise.  Up to k = 16 the f32 product
// g * 2^-k is exact for every finite bf16 g, so the scale may be applied to the sum instead of to each
// element without a second look; from 17 on (a loss scale that has grown past its initial 2^16) that holds
// for all but the tiniest nonzero values, which the guarded kernel finds and takes the long way.
constexpr int kPow2MaxK = 64;
static int pow2_unscale_exponent(float inv_scale)
{
    int e = 0;
    if (!(inv_scale > 0.0f) || frexpf(inv_scale, &e) != 0.5f) return -1;
    int k = 1 - e;  // inv_scale = 0.5 * 2^e = 2^(e-1)
    return (k >= 0 && k <= kPow2MaxK) ? k : -1;
}

int32_t launch_norm(nbo_optimizer *h, bool bf16, float inv_scale, double max_norm, int finalize)
{
    NormOut out{h->d_partial_sum, h->d_partial_bad, h->d_ticket, h->d_local, h->d_ctrl};
    const int k = bf16 ? pow2_unscale_exponent(inv_scale) : -1;
    if (k >= 0) {
        int grid = norm_grid(h, true);
        Pow2Guard gd{0u, inv_scale, ldexp(1.0, k)};
        if (k <= 16) {
            norm_pow2_bf16_kernel<false><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks,
                                                                       ldexp(1.0, -2 * k), max_norm, finalize, out, gd);
        } else {
            gd.limit = ((uint32_t)(k - 15) << 7) - 1u;
            norm_pow2_bf16_kernel<true><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks,
                                                                      ldexp(1.0, -2 * k), max_norm, finalize, out, gd);
        }
        return launched(h);
    }
    // the flag can be read off the sum only while the unscale factor cannot overflow a finite gradient
    bool each = !(inv_scale <= 1.0f);
    if (bf16) {
        if (each) launch_norm_one<true, true>(h, inv_scale, max_norm, finalize, out);
        else launch_norm_one<true, false>(h, inv_scale, max_norm, finalize, out);
    } else {
        if (each) launch_norm_one<false, true>(h, inv_scale, max_norm, finalize, out);
        else launch_norm_one<false, false>(h, inv_scale, max_norm, finalize, out);
    }
    return launched(h);
}

int32_t launch_nonfinite(nbo_optimizer *h, bool bf16)
{
    NormOut out{h->d_partial_sum, h->d_partial_bad, h->d_ticket, h->d_local, h->d_ctrl};
    uint32_t units = (h->nchunks + kNormBatch - 1) / kNormBatch;
    if (bf16) {
        int grid = grid_for(h, units, (const void *)nonfinite_kernel<true>);
        nonfinite_kernel<true><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks, out);
    } else {
        int grid = grid_for(h, units, (const void *)nonfinite_kernel<false>);
        nonfinite_kernel<false><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks, out);
    }
    return launched(h);
}

// Asynchronous step: the unscale factor is read from device memory, so the per-element flag test is kept
// (the host cannot know whether the factor exceeds 1).
int32_t launch_norm_dev(nbo_optimizer *h, const float *inv_scale_dev, double max_norm)
{
    NormOut out{h->d_partial_sum, h->d_partial_bad, h->d_ticket, h->d_local, h->d_ctrl};
    if (h->precision == NBO_MIXED_BF16_F32GRAD) launch_norm_one<false, true>(h, 1.0f, max_norm, 1, out, inv_scale_dev);
    else launch_norm_one<true, true>(h, 1.0f, max_norm, 1, out, inv_scale_dev);
    return launched(h);
}

int32_t launch_prepare(nbo_optimizer *h, int use_scaler)
{
    prepare_kernel<<<1, kMaxDevGroups, 0, h->stream>>>(h->d_state, h->d_hp, h->d_inv_scale, use_scaler);
    return launched(h);
}

int32_t launch_commit(nbo_optimizer *h, bool checked, int use_scaler)
{
    commit_kernel<<<1, 32, 0, h->stream>>>(h->d_state, checked ? h->d_ctrl : nullptr, use_scaler);
    return launched(h);
}

int32_t launch_adam_mixed_dev(nbo_optimizer *h, uint32_t cb, uint32_t nc, int group, bool with_ctrl)
{
    if (nc == 0) return NBO_OK;
    AdamHP unused{};
    const StepCtrl *ctrl = with_ctrl ? h->d_ctrl : nullptr;
    return h->precision == NBO_MIXED_BF16_F32GRAD
               ? launch_adam_mixed_one<true, true>(h, cb, nc, unused, ctrl, h->d_hp + group)
               : launch_adam_mixed_one<true, false>(h, cb, nc, unused, ctrl, h->d_hp + group);
}

int32_t launch_finalize_ranks(nbo_optimizer *h, const double *gathered, int world, double max_norm)
{
    finalize_ranks_kernel<<<1, 32, 0, h->stream>>>(gathered, world, max_norm, h->d_ctrl);
    return launched(h);
}

int32_t launch_scale_grads(nbo_optimizer *h, int mode, float factor)
{
    if (h->nchunks == 0) return NBO_OK;
    int grid = grid_for(h, h->nchunks, (const void *)scale_grads_kernel, 3);  // 6684 GB/s at 3, 5898 at 8
    scale_grads_kernel<<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks, mode, factor,
                                                       h->d_ctrl);
    return launched(h);
}

int32_t launch_zero_grads(nbo_optimizer *h, bool bf16)
{
    if (h->nchunks == 0) return NBO_OK;
    if (bf16) {
        int grid = grid_for(h, h->nchunks, (const void *)zero_grads_kernel<true>, 3);
        zero_grads_kernel<true><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks);
    } else {
        int grid = grid_for(h, h->nchunks, (const void *)zero_grads_kernel<false>, 3);  // 6889 GB/s at 3, 6037 at 8
        zero_grads_kernel<false><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks);
    }
    return launched(h);
}

int32_t launch_accumulate(nbo_optimizer *h)
{
    if (h->nchunks == 0) return NBO_OK;
    int grid = grid_for(h, h->nchunks, (const void *)accumulate_kernel, 2);  // 6613 GB/s at 2, 6369 at 8
    accumulate_kernel<<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks);
    return launched(h);
}

int32_t launch_init_master(nbo_optimizer *h)
{
    if (h->nchunks == 0) return NBO_OK;
    int grid = grid_for(h, h->nchunks, (const void *)init_master_kernel, 3);
    init_master_kernel<<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks);
    return launched(h);
}

}  // namespace nbo

// ---- adamw_step: one tensor, caller-owned moments, no handle ---------------------------------------

extern "C" int32_t nbo_adamw_step(int32_t device, void *stream, void *param, const void *grad, float *m,
                                  float *v, uint64_t n, double lr, double beta1, double beta2, double eps,
                                  double weight_decay, uint64_t step)
{
    using namespace nbo;
    if (n == 0) return NBO_OK;
    if (!param || !grad || !m || !v)
        return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_adamw_step: null device pointer");
    uintptr_t all = (uintptr_t)param | (uintptr_t)grad | (uintptr_t)m | (uintptr_t)v;
    if (all & 3u) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_adamw_step: pointer not aligned to f32");
    if (n > (uint64_t)0xfffffff0u * kChunkElems)
        return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_adamw_step: tensor too large");
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e == cudaSuccess && prev != device) e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail_cuda(nullptr, e, "cudaSetDevice");
    nbo_group_config cfg{NBO_ADAMW, lr, beta1, beta2, eps, weight_decay, 0.0};
    AdamHP hp = adam_hparams(cfg, step, 1.0f);
    TensorDesc d;
    d.p = param; d.g = grad; d.s0 = m; d.s1 = v; d.s2 = nullptr; d.n = n; d.group = 0;
    d.head = (all & 15u) ? 0xffffffffu : 0u;
    uint32_t nchunks = (uint32_t)((n + kChunkElems - 1) / kChunkElems);
    int sms = 0, per_sm = 0;
    int32_t rc = [&]() -> int32_t {
        NBO_CUDA(nullptr, cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void *)adam_f32_single_kernel, kBlock, 0) !=
                cudaSuccess || per_sm < 1)
            per_sm = 1;
        long long grid = (long long)sms * per_sm;
        if (grid > (long long)nchunks) grid = nchunks;
        adam_f32_single_kernel<<<(int)grid, kBlock, 0, (cudaStream_t)stream>>>(d, nchunks, hp);
        NBO_CUDA(nullptr, cudaGetLastError());
        return NBO_OK;
    }();
    if (prev >= 0 && prev != device) cudaSetDevice(prev);
    return rc;
}

// ---- ZeRO-1 fused with its collectives (fused_nvlink.cuh) ------------------------------------

namespace nbo {

template <int kIn, int kOut>
static int32_t launch_fused_one(nbo_optimizer *h, uint32_t cb, uint32_t nc, const AdamHP &hp, bool with_ctrl,
                                const PeerArgs &pa)
{
    // 2 resident CTAs per SM as for the local update kernel (register-limited)
    int grid = grid_for(h, nc, (const void *)zero1_fused_update_kernel<kIn, kOut>, 2);
    zero1_fused_update_kernel<kIn, kOut><<<grid, kBlock, 0, h->stream>>>(
        h->d_descs, h->d_chunks + cb, nc, hp, with_ctrl ? h->d_ctrl : nullptr, pa);
    return launched(h);
}

// in_transport: 0 local, 1 peer loads, 2 multicast; out_transport: 1 peer stores, 2 multicast stores.
int32_t launch_zero1_fused_update(nbo_optimizer *h, uint32_t cb, uint32_t nc, const AdamHP &hp, bool with_ctrl,
                                  const PeerArgs &pa, int in_transport, int out_transport)
{
    if (nc == 0) return NBO_OK;
    if (out_transport == kMcast) {
        if (in_transport == kLocal) return launch_fused_one<kLocal, kMcast>(h, cb, nc, hp, with_ctrl, pa);
        if (in_transport == kMcast) return launch_fused_one<kMcast, kMcast>(h, cb, nc, hp, with_ctrl, pa);
        return launch_fused_one<kPeer, kMcast>(h, cb, nc, hp, with_ctrl, pa);
    }
    if (in_transport == kLocal) return launch_fused_one<kLocal, kPeer>(h, cb, nc, hp, with_ctrl, pa);
    if (in_transport == kMcast) return launch_fused_one<kMcast, kPeer>(h, cb, nc, hp, with_ctrl, pa);
    return launch_fused_one<kPeer, kPeer>(h, cb, nc, hp, with_ctrl, pa);
}

__global__ void store_int_kernel(int32_t *dst, int32_t value) { *dst = value; }

int32_t launch_store_int(nbo_optimizer *h, int32_t *dst, int32_t value)
{
    store_int_kernel<<<1, 1, 0, h->stream>>>(dst, value);
    return launched(h);
}

int32_t launch_zero1_reduce_norm(nbo_optimizer *h, float inv_scale, const PeerArgs &pa, int in_transport)
{
    NormOut out{h->d_partial_sum, h->d_partial_bad, h->d_ticket, h->d_local, h->d_ctrl};
    if (in_transport == kMcast) {
        int grid = grid_for(h, h->nchunks, (const void *)zero1_reduce_norm_kernel<kMcast>);
        zero1_reduce_norm_kernel<kMcast><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks,
                                                                        inv_scale, out, pa);
    } else {
        int grid = grid_for(h, h->nchunks, (const void *)zero1_reduce_norm_kernel<kPeer>);
        zero1_reduce_norm_kernel<kPeer><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks,
                                                                       inv_scale, out, pa);
    }
    return launched(h);
}

}  // namespace nbo

// ---- gradient norm for callers that cannot allocate --------------------------------------
//
// Some callers of this library run where cudaMalloc is off limits: while some
// thread of the process has a stream capture open in global mode (cudaMalloc is
// then illegal process-wide), under a framework allocator
// that owns all device memory and forbids raw allocations (nabla's own pool,
// nabla-core/src/cuda_hip/common/pool.rs, is one), or in a process that hands
// this library a fixed memory budget.  A handle (nbo_create / nbo_set_tensors)
// allocates its table, state and reduction scratch, so those callers cannot
// use it.  nbo_grad_norm_noalloc gives them the norm / non-finite pass over one
// contiguous gradient buffer with every byte of scratch in the fixed array
// below, which each GPU that loads the library holds until the process exits.
//
// The scratch carries a one-row tensor table, the chunk list (16 bytes per
// 4096 elements, which is what bounds the supported size), the per-CTA
// partials, the ticket and the decision record.  All calls share it and it
// keeps the previous call's contents: the set-up kernel rewrites the table and
// zeroes the ticket on every call, and two calls that overlap on the GPU
// (different streams, no dependency) race on it.

namespace nbo {

constexpr uint32_t kNoAllocMaxChunks = 32768;                                       // 512 KiB of chunk list
constexpr uint64_t kNoAllocMaxElems = (uint64_t)kNoAllocMaxChunks * kChunkElems;    // 134,217,728 elements
constexpr int kNoAllocMaxGrid = 2048;

struct NoAllocScratch {
    TensorDesc desc;
    StepCtrl ctrl;
    uint32_t ticket;
    uint32_t pad;
    double partial_sum[kNoAllocMaxGrid];
    int32_t partial_bad[kNoAllocMaxGrid];
    Chunk chunks[kNoAllocMaxChunks];
};

static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

// Device code may name the array directly; it fills the table for this call.
__global__ void noalloc_setup_kernel(const void *grads, uint64_t n, uint32_t head, uint32_t nchunks)
{
    NoAllocScratch *s = reinterpret_cast<NoAllocScratch *>(g_noalloc_scratch);
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0) {
        TensorDesc d;
        d.p = nullptr; d.g = grads; d.s0 = d.s1 = d.s2 = nullptr;
        d.n = n; d.head = head; d.group = 0;
        s->desc = d;
        s->ticket = 0;  // must start at zero whatever an earlier call left behind
    }
    if (i < nchunks) {
        uint64_t h = head < n ? head : n;
        uint64_t body_items = (n - h) >> 2, i0 = (uint64_t)i * kChunkItems;
        uint64_t ni = i0 >= body_items ? 0 : (body_items - i0 < kChunkItems ? body_items - i0 : kChunkItems);
        bool last = ((uint64_t)i + 1) * kChunkElems >= n;
        s->chunks[i] = Chunk{0u, i, (uint32_t)ni, (i == 0 && h) || (last && ((n - h) & 3)) ? 1u : 0u};
    }
}

}  // namespace nbo

extern "C" int32_t nbo_grad_norm_noalloc(int32_t device, void *stream, const void *grads, uint64_t n,
                                         int32_t precision, float inv_scale, double *out_dev)
{
    using namespace nbo;
    static NoAllocScratch *scratch_of[64] = {nullptr};  // device address of the array, per device
    static int grid_of[64][2] = {{0}};                  // persistent grid per device: [fp32, bf16]
    if (device < 0 || device >= 64)
        return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_grad_norm_noalloc: device index out of range");
    if (!out_dev || (n && !grads))
        return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_grad_norm_noalloc: null pointer");
    if (precision != NBO_F32 && precision != NBO_MIXED_BF16)
        return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_grad_norm_noalloc: unknown precision");
    if (n > kNoAllocMaxElems)
        return fail(nullptr, NBO_ERR_INVALID,
                    "nabla-optim-b200: nbo_grad_norm_noalloc: " + std::to_string(n) +
                        " elements exceed the fixed scratch (max " + std::to_string(kNoAllocMaxElems) +
                        "); use a handle and nbo_grad_norm instead");
    const bool bf16 = precision == NBO_MIXED_BF16;
    const uintptr_t es = bf16 ? 2 : 4;
    if (((uintptr_t)grads & (es - 1)) || ((uintptr_t)out_dev & 7u))
        return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_grad_norm_noalloc: misaligned pointer");
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e == cudaSuccess && prev != device) e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail_cuda(nullptr, e, "cudaSetDevice");
    static std::mutex setup_lock;  // guards the per-device address cache, not the scratch itself
    int32_t rc = [&]() -> int32_t {
        std::lock_guard<std::mutex> guard(setup_lock);
        if (!scratch_of[device]) {
            // The array's name is only a host-side stand-in: ask the runtime for its address on THIS device.
            void *p = nullptr;
            NBO_CUDA(nullptr, cudaGetSymbolAddress(&p, g_noalloc_scratch));
            int sms = 0;
            NBO_CUDA(nullptr, cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
            // Touch every kernel this entry point can launch, for both precisions, so that the driver loads
            // their code now (with lazy module loading a kernel's first use makes the driver set aside device
            // memory for it) and one warm-up call per device covers fp32 and bf16 alike.
            cudaFuncAttributes fa;
            NBO_CUDA(nullptr, cudaFuncGetAttributes(&fa, (const void *)noalloc_setup_kernel));
            const void *ks[2] = {(const void *)norm_kernel<false, true>, (const void *)norm_kernel<true, true>};
            for (int b = 0; b < 2; ++b) {
                NBO_CUDA(nullptr, cudaFuncGetAttributes(&fa, ks[b]));
                int per_sm = 0;
                if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ks[b], kBlock, 0) != cudaSuccess || per_sm < 1)
                    per_sm = 1;
                long long g = (long long)sms * per_sm;
                grid_of[device][b] = (int)(g > kNoAllocMaxGrid ? kNoAllocMaxGrid : g);
            }
            scratch_of[device] = static_cast<NoAllocScratch *>(p);
        }
        NoAllocScratch *s = scratch_of[device];
        cudaStream_t st = (cudaStream_t)stream;
        uint32_t nchunks = (uint32_t)((n + kChunkElems - 1) / kChunkElems);
        // elements before the first 16-byte (fp32) / 8-byte (bf16) boundary are handled one by one
        uint32_t head = (uint32_t)((((bf16 ? 8u : 16u) - ((uintptr_t)grads & (bf16 ? 7u : 15u))) & (bf16 ? 7u : 15u)) / es);
        uint32_t setup_blocks = nchunks / 256 + 1;
        noalloc_setup_kernel<<<setup_blocks, 256, 0, st>>>(grads, n, head, nchunks);
        NBO_CUDA(nullptr, cudaGetLastError());
        long long grid = grid_of[device][bf16 ? 1 : 0];
        long long units = ((long long)nchunks + kNormBatch - 1) / kNormBatch;
        if (grid > units) grid = units;
        if (grid < 1) grid = 1;
        NormOut out{s->partial_sum, s->partial_bad, &s->ticket, out_dev, &s->ctrl};
        if (bf16)
            norm_kernel<true, true><<<(int)grid, kBlock, 0, st>>>(&s->desc, s->chunks, nchunks, inv_scale, 0.0, 1, out,
                                                                  nullptr);
        else
            norm_kernel<false, true><<<(int)grid, kBlock, 0, st>>>(&s->desc, s->chunks, nchunks, inv_scale, 0.0, 1, out,
                                                                   nullptr);
        NBO_CUDA(nullptr, cudaGetLastError());
        return NBO_OK;
    }();
    if (prev >= 0 && prev != device) cudaSetDevice(prev);
    return rc;
}

// ---- plain copy with SM loads and stores ------------------------------------------------------
// The yardstick the NVLink fraction of the fused sharded step is quoted against: the same kind of access
// the fused kernels make (128-bit loads and stores issued by SMs, persistent grid), with nothing else to do.
// Either pointer may be another GPU's memory mapped into this process.

namespace nbo {
__global__ void __launch_bounds__(256) copy_probe_kernel(uint4 *__restrict__ dst, const uint4 *__restrict__ src, uint64_t n16)
{
    const uint64_t stride = (uint64_t)gridDim.x * 256 * 4;
    for (uint64_t i0 = (uint64_t)blockIdx.x * 1024 + threadIdx.x; i0 < n16; i0 += stride) {
        uint4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * 256 < n16) r[u] = src[i0 + u * 256];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * 256 < n16) dst[i0 + u * 256] = r[u];
    }
}
}  // namespace nbo

extern "C" int32_t nbo_copy_probe(int32_t device, void *stream, void *dst, const void *src, uint64_t bytes)
{
    using namespace nbo;
    if (!dst || !src) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_copy_probe: null pointer");
    if ((((uintptr_t)dst | (uintptr_t)src) & 15u) || (bytes & 15u))
        return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_copy_probe: pointers and size must be multiples of 16 bytes");
    if (bytes == 0) return NBO_OK;
    DeviceGuard guard(device);
    int sms = 0;
    cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return fail_cuda(nullptr, e, "cudaDeviceGetAttribute");
    uint64_t n16 = bytes / 16;
    uint64_t want = (n16 + 1023) / 1024;
    int grid = (int)(want < (uint64_t)sms * 8 ? want : (uint64_t)sms * 8);
    copy_probe_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((uint4 *)dst, (const uint4 *)src, n16);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(nullptr, e, "copy_probe_kernel");
    return NBO_OK;
}
