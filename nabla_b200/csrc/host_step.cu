// Host-streamed mixed-precision step: gradients arrive from host memory and the
// updated bf16 parameters return to host memory, slice by slice, while the fp32
// master / m / v state never leaves HBM.
//
// nabla's tensors live in host memory on its CPU backend (nabla-core/src/cpu/mod.rs),
// so a caller that switches only the optimizer step to the GPU holds host buffers on
// both sides of it.  Copying all gradients in, stepping, and copying all parameters
// out serialises the two PCIe directions; the update itself is elementwise, so here the
// chunk list is cut into slices and three streams run as a pipeline:
//
//   copy-in stream : gradients of slice s        host -> device
//   compute stream : update kernel on slice s    (waits for copy-in s)
//   copy-out stream: parameters of slice s       device -> host (waits for update s)
//
// While slice s is copied out, slice s+1 is copied in: both PCIe directions are busy and the
// update (about 1/10 of a slice's copy time) hides behind them.  With loss scaling or
// clipping the skip / clip decision needs every gradient first, so all slices are copied
// in, the norm or flag pass runs once, the decision is read on the host, and only the
// update + copy-out half is pipelined (and left out altogether when the step is skipped).
//
// The arithmetic is the resident step's: the same kernels run over sub-ranges of the same
// chunk list, so the result is bit-identical to nbo_step_mixed on the same data.
#include <new>
#include <vector>

#include "host_plan.h"
#include "internal.h"

namespace nbo {

void host_pipe_destroy(nbo_optimizer *h)
{
    HostPipe *p = h->host_pipe;
    if (!p) return;
    if (p->in) { cudaStreamSynchronize(p->in); cudaStreamDestroy(p->in); }
    if (p->out) { cudaStreamSynchronize(p->out); cudaStreamDestroy(p->out); }
    if (p->start) cudaEventDestroy(p->start);
    for (cudaEvent_t e : p->copied) cudaEventDestroy(e);
    for (cudaEvent_t e : p->updated) cudaEventDestroy(e);
    delete p;
    h->host_pipe = nullptr;
}

int32_t host_pipe_ensure(nbo_optimizer *h, size_t nslices)
{
    if (!h->host_pipe) {
        h->host_pipe = new (std::nothrow) HostPipe();
        if (!h->host_pipe) return fail(h, NBO_ERR_NOMEM, "nabla-optim-b200: out of host memory");
    }
    HostPipe *p = h->host_pipe;
    if (!p->in) NBO_CUDA(h, cudaStreamCreateWithFlags(&p->in, cudaStreamNonBlocking));
    if (!p->out) NBO_CUDA(h, cudaStreamCreateWithFlags(&p->out, cudaStreamNonBlocking));
    if (!p->start) NBO_CUDA(h, cudaEventCreateWithFlags(&p->start, cudaEventDisableTiming));
    while (p->copied.size() < nslices) {
        cudaEvent_t e = nullptr;
        NBO_CUDA(h, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        p->copied.push_back(e);
    }
    while (p->updated.size() < nslices) {
        cudaEvent_t e = nullptr;
        NBO_CUDA(h, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        p->updated.push_back(e);
    }
    return NBO_OK;
}

// Drains the three streams after a failed enqueue so that no copy is still reading or
// writing caller memory when the error is returned.
void host_pipe_drain(nbo_optimizer *h)
{
    HostPipe *p = h->host_pipe;
    if (p && p->in) cudaStreamSynchronize(p->in);
    cudaStreamSynchronize(h->stream);
    if (p && p->out) cudaStreamSynchronize(p->out);
}

static int32_t enqueue(nbo_optimizer *h, const HostPlan &plan, void *const *host_p, const void *const *host_g,
                       bool checked, float inv_scale, double max_norm)
{
    HostPipe *pipe = h->host_pipe;
    const size_t gsz = h->precision == NBO_MIXED_BF16_F32GRAD ? 4 : 2;
    const size_t ns = plan.slices.size();

    std::vector<AdamHP> hp(h->groups.size());
    for (size_t g = 0; g < h->groups.size(); ++g)
        hp[g] = adam_hparams(h->groups[g].cfg, h->groups[g].step_count + 1, inv_scale);

    // work already on the compute stream (an earlier asynchronous step, a table upload) comes first
    NBO_CUDA(h, cudaEventRecord(pipe->start, h->stream));
    NBO_CUDA(h, cudaStreamWaitEvent(pipe->in, pipe->start, 0));
    NBO_CUDA(h, cudaStreamWaitEvent(pipe->out, pipe->start, 0));

    auto copy_in = [&](size_t s) -> int32_t {
        const Slice &sl = plan.slices[s];
        for (uint32_t k = sl.copy_begin; k < sl.copy_end; ++k) {
            const SliceCopy &c = plan.copies[k];
            const Piece &pc = h->pieces[c.row];
            char *dst = (char *)const_cast<void *>(h->h_descs[c.row].g) + c.lo * gsz;
            const char *src = (const char *)host_g[pc.tensor] + (pc.offset + c.lo) * gsz;
            NBO_CUDA(h, cudaMemcpyAsync(dst, src, (c.hi - c.lo) * gsz, cudaMemcpyHostToDevice, pipe->in));
        }
        NBO_CUDA(h, cudaEventRecord(pipe->copied[s], pipe->in));
        return NBO_OK;
    };
    auto update_and_copy_out = [&](size_t s, bool wait_copy) -> int32_t {
        const Slice &sl = plan.slices[s];
        if (wait_copy) NBO_CUDA(h, cudaStreamWaitEvent(h->stream, pipe->copied[s], 0));
        int32_t rc = launch_adam_mixed(h, sl.chunk_begin, sl.chunk_end - sl.chunk_begin, hp[sl.group], checked);
        if (rc != NBO_OK) return rc;
        NBO_CUDA(h, cudaEventRecord(pipe->updated[s], h->stream));
        NBO_CUDA(h, cudaStreamWaitEvent(pipe->out, pipe->updated[s], 0));
        for (uint32_t k = sl.copy_begin; k < sl.copy_end; ++k) {
            const SliceCopy &c = plan.copies[k];
            const Piece &pc = h->pieces[c.row];
            const char *src = (const char *)h->h_descs[c.row].p + c.lo * 2;
            char *dst = (char *)host_p[pc.tensor] + (pc.offset + c.lo) * 2;
            NBO_CUDA(h, cudaMemcpyAsync(dst, src, (c.hi - c.lo) * 2, cudaMemcpyDeviceToHost, pipe->out));
        }
        return NBO_OK;
    };

    if (!checked) {
        for (size_t s = 0; s < ns; ++s) {
            int32_t rc = copy_in(s);
            if (rc != NBO_OK) return rc;
            rc = update_and_copy_out(s, true);
            if (rc != NBO_OK) return rc;
        }
        return NBO_OK;
    }
    for (size_t s = 0; s < ns; ++s) {
        int32_t rc = copy_in(s);
        if (rc != NBO_OK) return rc;
    }
    if (ns) NBO_CUDA(h, cudaStreamWaitEvent(h->stream, pipe->copied[ns - 1], 0));
    // loss scaling without clipping needs the skip decision only (trainer.rs:501-503)
    int32_t rc = max_norm > 0.0 ? launch_norm(h, h->precision == NBO_MIXED_BF16, inv_scale, max_norm, 1)
                                : launch_nonfinite(h, h->precision == NBO_MIXED_BF16);
    if (rc != NBO_OK) return rc;
    // The decision comes to the host here: the copy-in half has to drain before the first update can
    // start anyway, and a skipped step must not copy anything out (the kernel leaves the device
    // parameter buffers untouched on a skip, and they are staging, not the caller's truth).
    rc = read_ctrl(h);
    if (rc != NBO_OK) return rc;
    if (h->h_ctrl->nonfinite) return NBO_OK;
    for (size_t s = 0; s < ns; ++s) {
        rc = update_and_copy_out(s, false);
        if (rc != NBO_OK) return rc;
    }
    return NBO_OK;
}

int32_t host_streamed_step(nbo_optimizer *h, void *const *host_p, const void *const *host_g,
                           uint64_t slice_elems, int32_t use_scaler, double max_norm, nbo_step_result *result)
{
    for (const Piece &pc : h->pieces)
        if (pc.n && (!host_p[pc.tensor] || !host_g[pc.tensor]))
            return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null host pointer for tensor " + std::to_string(pc.tensor));
    if (slice_elems == 0) slice_elems = 32ull << 20;  // 64 MiB of bf16 per slice and direction
    uint64_t slice_chunks = (slice_elems + kChunkElems - 1) / kChunkElems;

    const size_t np = h->pieces.size();
    std::vector<uint64_t> row_n(np);
    std::vector<uint32_t> row_head(np);
    std::vector<int32_t> row_group(np);
    for (size_t i = 0; i < np; ++i) {
        row_n[i] = h->pieces[i].n;
        row_head[i] = h->h_descs[i].head;
        row_group[i] = h->pieces[i].group;
    }
    HostPlan plan = plan_host_slices(row_n, row_head, row_group, (int32_t)h->groups.size(), slice_chunks);
    for (const Slice &sl : plan.slices)  // the planner walks the list the way build_table lays it out
        if (sl.chunk_begin < h->groups[sl.group].chunk_begin || sl.chunk_end > h->groups[sl.group].chunk_end)
            return fail(h, NBO_ERR_STATE, "nabla-optim-b200: slice plan does not match the chunk list");

    int32_t rc = host_pipe_ensure(h, plan.slices.size());
    if (rc != NBO_OK) return rc;

    const bool checked = use_scaler || max_norm > 0.0;
    const float inv_scale = use_scaler ? (float)(1.0 / h->scaler.scale) : 1.0f;
    h->prof_norm_valid = false;
    h->prof_update_valid = false;

    rc = enqueue(h, plan, host_p, host_g, checked, inv_scale, max_norm);
    if (rc != NBO_OK) {
        host_pipe_drain(h);
        return rc;
    }
    NBO_CUDA(h, cudaStreamSynchronize(h->stream));
    NBO_CUDA(h, cudaStreamSynchronize(h->host_pipe->in));
    NBO_CUDA(h, cudaStreamSynchronize(h->host_pipe->out));
    commit_step(h, checked, use_scaler != 0, result);
    return NBO_OK;
}

}  // namespace nbo

using namespace nbo;

extern "C" {

int32_t nbo_step_mixed_host(nbo_optimizer *h, uint64_t n, void *const *params_dev, const void *const *grads_dev,
                            void *const *params_host, const void *const *grads_host, uint64_t slice_elems,
                            int32_t use_scaler, double max_norm, nbo_step_result *result)
{
    NBO_SYNC_STATE(h);
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (!h->configured || h->precision == NBO_F32 || h->zero1)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: nbo_step_mixed_host needs an unsharded mixed-precision handle");
    if (n && (!params_dev || !grads_dev || !params_host || !grads_host))
        return fail(h, NBO_ERR_INVALID, "nabla-train: params/grads length mismatch (null list)");
    DeviceGuard guard(h->device);
    int32_t rc = bind_list(h, n, params_dev, grads_dev, 2, "step");
    if (rc != NBO_OK) return rc;
    return host_streamed_step(h, params_host, grads_host, slice_elems, use_scaler, max_norm, result);
}

}  // extern "C"
