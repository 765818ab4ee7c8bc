// The one translation unit that holds the device code, plus the launchers the
// host code calls.  Grids are persistent: SM count x resident CTAs per SM
// (from the occupancy calculator), capped by the number of chunks.
#include <map>

#include "internal.h"
#include "kernels.cuh"

namespace nbo {

static int grid_for(const nbo_optimizer *h, uint32_t nchunks, const void *kernel)
{
    static std::map<const void *, int> cache;  // resident CTAs per SM, per kernel
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
        int grid = grid_for(h, nc, (const void *)sgd_f32_kernel<true>);
        sgd_f32_kernel<true><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks + cb, nc, hp);
    } else {
        int grid = grid_for(h, nc, (const void *)sgd_f32_kernel<false>);
        sgd_f32_kernel<false><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks + cb, nc, hp);
    }
    return launched(h);
}

int32_t launch_adam_mixed(nbo_optimizer *h, uint32_t cb, uint32_t nc, const AdamHP &hp, bool with_ctrl)
{
    if (nc == 0) return NBO_OK;
    int grid = grid_for(h, nc, (const void *)adam_mixed_kernel);
    adam_mixed_kernel<<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks + cb, nc, hp,
                                                      with_ctrl ? h->d_ctrl : nullptr);
    return launched(h);
}

int32_t launch_norm(nbo_optimizer *h, bool bf16, float inv_scale, double max_norm, int finalize)
{
    NormOut out{h->d_partial_sum, h->d_partial_bad, h->d_ticket, h->d_local, h->d_ctrl};
    if (bf16) {
        int grid = grid_for(h, h->nchunks, (const void *)norm_kernel<true>);
        norm_kernel<true><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks,
                                                          inv_scale, max_norm, finalize, out);
    } else {
        int grid = grid_for(h, h->nchunks, (const void *)norm_kernel<false>);
        norm_kernel<false><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks,
                                                           inv_scale, max_norm, finalize, out);
    }
    return launched(h);
}

int32_t launch_finalize_ranks(nbo_optimizer *h, const double *gathered, int world, double max_norm)
{
    finalize_ranks_kernel<<<1, 32, 0, h->stream>>>(gathered, world, max_norm, h->d_ctrl);
    return launched(h);
}

int32_t launch_scale_grads(nbo_optimizer *h, int mode, float factor)
{
    if (h->nchunks == 0) return NBO_OK;
    int grid = grid_for(h, h->nchunks, (const void *)scale_grads_kernel);
    scale_grads_kernel<<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks, mode, factor,
                                                       h->d_ctrl);
    return launched(h);
}

int32_t launch_zero_grads(nbo_optimizer *h, bool bf16)
{
    if (h->nchunks == 0) return NBO_OK;
    if (bf16) {
        int grid = grid_for(h, h->nchunks, (const void *)zero_grads_kernel<true>);
        zero_grads_kernel<true><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks);
    } else {
        int grid = grid_for(h, h->nchunks, (const void *)zero_grads_kernel<false>);
        zero_grads_kernel<false><<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks);
    }
    return launched(h);
}

int32_t launch_init_master(nbo_optimizer *h)
{
    if (h->nchunks == 0) return NBO_OK;
    int grid = grid_for(h, h->nchunks, (const void *)init_master_kernel);
    init_master_kernel<<<grid, kBlock, 0, h->stream>>>(h->d_descs, h->d_chunks, h->nchunks);
    return launched(h);
}

}  // namespace nbo
