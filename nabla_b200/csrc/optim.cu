// libnabla_optim_b200: handle, device table, and the single-GPU entry points of
// the C ABI declared in include/nabla_optim_b200.h.
#include <math.h>
#include <string.h>

#include <new>

#include "internal.h"

namespace nbo {

static thread_local std::string g_err = "";

int32_t fail(nbo_optimizer *h, int32_t code, const std::string &msg)
{
    if (h) h->err = msg; else g_err = msg;
    return code;
}

int32_t fail_cuda(nbo_optimizer *h, cudaError_t e, const char *what)
{
    std::string m = std::string("CUDA error: ") + cudaGetErrorString(e) + " in " + what;
    int32_t code = (e == cudaErrorMemoryAllocation) ? NBO_ERR_NOMEM : NBO_ERR_CUDA;
    return fail(h, code, m);
}

double powi(double a, int32_t b) { return powi_sqm(a, b); }

AdamHP adam_hparams(const nbo_group_config &c, uint64_t step, float inv_scale)
{
    return adam_hparams_of(c.lr, c.beta1, c.beta2, c.eps, c.weight_decay, c.kind == NBO_ADAMW, step, inv_scale);
}

SgdHP sgd_hparams(const nbo_group_config &c)
{
    SgdHP h;
    float lr_t = (float)c.lr;
    h.nlr = -lr_t;
    h.mu = (float)c.momentum;
    h.wd = (float)c.weight_decay;
    h.use_mu = c.momentum != 0.0;
    h.use_wd = c.weight_decay != 0.0;
    return h;
}

// ---- table ---------------------------------------------------------------------

void free_table(nbo_optimizer *h)
{
    cudaFree(h->d_s0); cudaFree(h->d_s1); cudaFree(h->d_s2);
    h->d_s0 = h->d_s1 = h->d_s2 = nullptr;
    cudaFree(h->d_descs); cudaFree(h->d_chunks);
    h->d_descs = nullptr; h->d_chunks = nullptr;
    if (h->h_descs) cudaFreeHost(h->h_descs);
    h->h_descs = nullptr;
    h->nchunks = 0;
    h->table_bound = false;
}

static uint64_t chunks_of(uint64_t n) { return (n + kChunkElems - 1) / kChunkElems; }

int32_t build_table(nbo_optimizer *h)
{
    const size_t np = h->pieces.size();
    // chunk list, grouped so that every group is one contiguous range
    std::vector<Chunk> chunks;
    uint64_t total_chunks = 0;
    for (const Piece &p : h->pieces) total_chunks += chunks_of(p.n);
    if (total_chunks > 0xfffffff0ull)
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: too many chunks for one table");
    chunks.reserve((size_t)total_chunks);
    for (size_t g = 0; g < h->groups.size(); ++g) {
        h->groups[g].chunk_begin = (uint32_t)chunks.size();
        for (size_t i = 0; i < np; ++i) {
            if (h->pieces[i].group != (int32_t)g) continue;
            const Piece &pc = h->pieces[i];
            uint64_t nc = chunks_of(pc.n);
            // the head an aligned row will have: none for separate tensors, the distance to the next
            // 4-element boundary of the bucket for a piece of a flat bucket
            uint64_t head = h->zero1 ? ((4 - (pc.bucket_off & 3)) & 3) : 0;
            if (head > pc.n) head = pc.n;
            uint64_t body_items = (pc.n - head) >> 2;
            uint64_t tail = (pc.n - head) & 3;
            for (uint64_t c = 0; c < nc; ++c) {
                uint64_t i0 = c * kChunkItems;
                uint64_t ni = i0 >= body_items ? 0 : (body_items - i0 < kChunkItems ? body_items - i0 : kChunkItems);
                bool last = (c + 1) * kChunkElems >= pc.n;
                uint32_t stray = ((c == 0 && head) || (last && tail)) ? 1u : 0u;
                chunks.push_back(Chunk{(uint32_t)i, (uint32_t)c, (uint32_t)ni, stray});
            }
        }
        h->groups[g].chunk_end = (uint32_t)chunks.size();
    }
    h->nchunks = (uint32_t)chunks.size();

    size_t state_bytes = (size_t)(h->state_elems ? h->state_elems : 1) * sizeof(float);
    NBO_CUDA(h, cudaMalloc(&h->d_s0, state_bytes));
    NBO_CUDA(h, cudaMalloc(&h->d_s1, state_bytes));
    NBO_CUDA(h, cudaMemsetAsync(h->d_s0, 0, state_bytes, h->stream));
    NBO_CUDA(h, cudaMemsetAsync(h->d_s1, 0, state_bytes, h->stream));
    if (h->precision != NBO_F32) {
        NBO_CUDA(h, cudaMalloc(&h->d_s2, state_bytes));
        NBO_CUDA(h, cudaMemsetAsync(h->d_s2, 0, state_bytes, h->stream));
    }
    NBO_CUDA(h, cudaMallocHost(&h->h_descs, (np ? np : 1) * sizeof(TensorDesc)));
    NBO_CUDA(h, cudaMalloc(&h->d_descs, (np ? np : 1) * sizeof(TensorDesc)));
    NBO_CUDA(h, cudaMalloc(&h->d_chunks, (chunks.size() ? chunks.size() : 1) * sizeof(Chunk)));
    if (!chunks.empty())
        NBO_CUDA(h, cudaMemcpy(h->d_chunks, chunks.data(), chunks.size() * sizeof(Chunk),
                               cudaMemcpyHostToDevice));
    for (size_t i = 0; i < np; ++i) {
        const Piece &p = h->pieces[i];
        TensorDesc d;
        d.p = nullptr; d.g = nullptr;
        d.s0 = h->d_s0 + p.state_off;
        d.s1 = h->d_s1 + p.state_off;
        d.s2 = h->d_s2 ? h->d_s2 + p.state_off : nullptr;
        d.n = p.n;
        d.head = 0xffffffffu;
        d.group = (uint32_t)p.group;
        h->h_descs[i] = d;
    }
    h->bound_p.assign(np, nullptr);
    h->bound_g.assign(np, nullptr);
    h->table_bound = false;
    h->configured = true;
    return NBO_OK;
}

static int32_t upload_descs(nbo_optimizer *h)
{
    size_t np = h->pieces.size();
    if (np)
        NBO_CUDA(h, cudaMemcpyAsync(h->d_descs, h->h_descs, np * sizeof(TensorDesc),
                                    cudaMemcpyHostToDevice, h->stream));
    NBO_CUDA(h, cudaEventRecord(h->upload_done, h->stream));
    h->uploads += 1;
    h->table_bound = true;
    return NBO_OK;
}

int32_t bind_list(nbo_optimizer *h, uint64_t n, void *const *params, const void *const *grads,
                  int elem_size, const char *who)
{
    // element sizes of the two columns: equal except for bf16 params with fp32 gradients
    const int p_es = elem_size;
    const int g_es = (h->precision == NBO_MIXED_BF16_F32GRAD) ? 4 : elem_size;
    if (!h->configured)
        return fail(h, NBO_ERR_STATE, std::string("nabla-optim-b200: ") + who + " before set_tensors");
    if (h->zero1)
        return fail(h, NBO_ERR_STATE, std::string("nabla-optim-b200: ") + who +
                                          " takes per-tensor pointers; this handle is ZeRO-1 sharded");
    if (n != h->ntensors)
        return fail(h, NBO_ERR_INVALID, std::string("nabla-train: ") + who + " params count mismatch");
    if (n && !params && !grads)
        return fail(h, NBO_ERR_INVALID, std::string("nabla-optim-b200: ") + who + ": null pointer list");
    const uintptr_t p_mask = p_es == 4 ? 15u : 7u, g_mask = g_es == 4 ? 15u : 7u;
    bool changed = !h->table_bound;
    for (uint64_t t = 0; t < n && !changed; ++t) {
        if (params && h->bound_p[t] != params[t]) changed = true;
        if (grads && h->bound_g[t] != grads[t]) changed = true;
    }
    if (!changed) return NBO_OK;
    for (uint64_t t = 0; t < n; ++t) {
        if (h->numel[t] == 0) continue;
        if ((params && !params[t]) || (grads && !grads[t]))
            return fail(h, NBO_ERR_INVALID, std::string("nabla-optim-b200: ") + who +
                                                ": null device pointer for tensor " + std::to_string(t));
        if ((params && ((uintptr_t)params[t] & (uintptr_t)(p_es - 1))) ||
            (grads && ((uintptr_t)grads[t] & (uintptr_t)(g_es - 1))))
            return fail(h, NBO_ERR_INVALID, std::string("nabla-optim-b200: ") + who +
                                                ": pointer not aligned to its element size, tensor " +
                                                std::to_string(t));
    }
    // the staging rows may still be in flight from the previous upload
    NBO_CUDA(h, cudaEventSynchronize(h->upload_done));
    for (uint64_t t = 0; t < n; ++t) {
        TensorDesc &d = h->h_descs[t];
        if (params) { d.p = params[t]; h->bound_p[t] = params[t]; }
        if (grads) { d.g = grads[t]; h->bound_g[t] = grads[t]; }
        bool aligned = (((uintptr_t)d.g & g_mask) == 0) &&
                       (d.p == nullptr || ((uintptr_t)d.p & p_mask) == 0);
        d.head = aligned ? 0u : 0xffffffffu;
    }
    return upload_descs(h);
}

int32_t bind_flat(nbo_optimizer *h, void *params_flat, const void *grads_flat)
{
    if (((uintptr_t)params_flat & 15u) || ((uintptr_t)grads_flat & 15u))
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: flat buckets must be 16-byte aligned");
    size_t np = h->pieces.size();
    bool changed = !h->table_bound || np == 0 || h->bound_p.empty() ||
                   h->bound_p[0] != params_flat || h->bound_g[0] != grads_flat;
    if (!changed) return NBO_OK;
    NBO_CUDA(h, cudaEventSynchronize(h->upload_done));
    for (size_t i = 0; i < np; ++i) {
        const Piece &p = h->pieces[i];
        TensorDesc &d = h->h_descs[i];
        d.p = params_flat ? (void *)((uint16_t *)params_flat + p.bucket_off) : nullptr;
        d.g = grads_flat ? (const void *)((const uint16_t *)grads_flat + p.bucket_off) : nullptr;
        d.head = (uint32_t)((4 - (p.bucket_off & 3)) & 3);
    }
    if (np) { h->bound_p[0] = params_flat; h->bound_g[0] = grads_flat; }
    return upload_descs(h);
}

// ---- step plumbing ---------------------------------------------------------------

int32_t launch_mixed_update(nbo_optimizer *h, float inv_scale, bool with_ctrl)
{
    for (Group &g : h->groups) {
        uint32_t nc = g.chunk_end - g.chunk_begin;
        if (nc == 0) continue;
        AdamHP hp = adam_hparams(g.cfg, g.step_count + 1, inv_scale);
        int32_t rc = launch_adam_mixed(h, g.chunk_begin, nc, hp, with_ctrl);
        if (rc != NBO_OK) return rc;
    }
    return NBO_OK;
}

void commit_step(nbo_optimizer *h, bool checked, bool use_scaler, nbo_step_result *res)
{
    bool bad = checked && h->h_ctrl->nonfinite != 0;
    if (bad) {
        if (use_scaler) {
            h->scaler.scale *= h->scaler.backoff_factor;
            h->scaler.consecutive_ok = 0;
        }
    } else {
        for (Group &g : h->groups)
            if (g.cfg.kind != NBO_SGD) g.step_count += 1;
        if (use_scaler) {
            h->scaler.consecutive_ok += 1;
            if (h->scaler.consecutive_ok >= h->scaler.growth_interval) {
                h->scaler.scale *= h->scaler.growth_factor;
                h->scaler.consecutive_ok = 0;
            }
        }
    }
    if (res) {
        res->applied = bad ? 0 : 1;
        res->nonfinite = bad ? 1 : 0;
        res->grad_norm = (checked && !bad) ? h->h_ctrl->norm : 0.0;
        res->loss_scale = h->scaler.scale;
        res->step_count = h->groups.empty() ? 0 : h->groups[0].step_count;
    }
}

int32_t prof_mark(nbo_optimizer *h, int i)
{
    if (!h->profile) return NBO_OK;
    NBO_CUDA(h, cudaEventRecord(h->prof_ev[i], h->stream));
    if (i == 0) h->prof_norm_valid = false;
    if (i == 1) h->prof_norm_valid = true;
    if (i == 2) h->prof_update_valid = false;
    if (i == 3) h->prof_update_valid = true;
    return NBO_OK;
}

int32_t read_ctrl(nbo_optimizer *h)
{
    NBO_CUDA(h, cudaMemcpyAsync(h->h_ctrl, h->d_ctrl, sizeof(StepCtrl), cudaMemcpyDeviceToHost,
                                h->stream));
    NBO_CUDA(h, cudaStreamSynchronize(h->stream));
    return NBO_OK;
}

int32_t collect_dev_state(nbo_optimizer *h)
{
    if (!h->dev_newer) return NBO_OK;
    if (h->zero1) {  // collectives may be pending on the stream: wait for them with the time limit first
        int32_t rc = zero1_bounded_wait(h, "the asynchronous sharded steps");
        if (rc != NBO_OK) return rc;
    }
    NBO_CUDA(h, cudaMemcpyAsync(h->h_state, h->d_state, sizeof(DevState), cudaMemcpyDeviceToHost, h->stream));
    NBO_CUDA(h, cudaMemcpyAsync(h->h_ctrl, h->d_ctrl, sizeof(StepCtrl), cudaMemcpyDeviceToHost, h->stream));
    NBO_CUDA(h, cudaStreamSynchronize(h->stream));
    const DevState &st = *h->h_state;
    h->scaler.scale = st.scale;
    h->scaler.consecutive_ok = st.consecutive_ok;
    for (size_t g = 0; g < h->groups.size() && g < (size_t)kMaxDevGroups; ++g)
        h->groups[g].step_count = st.g[g].step_count;
    h->dev_newer = false;
    return NBO_OK;
}

// Sends the host-side optimizer / scaler state to its device copy when the host holds the newer one
// (stream-ordered); the asynchronous steps then advance the device copy.
int32_t push_dev_state(nbo_optimizer *h)
{
    if (h->dev_newer) return NBO_OK;
    DevState &st = *h->h_state;
    st.scale = h->scaler.scale; st.growth_factor = h->scaler.growth_factor;
    st.backoff_factor = h->scaler.backoff_factor; st.growth_interval = h->scaler.growth_interval;
    st.consecutive_ok = h->scaler.consecutive_ok; st.ngroups = (int32_t)h->groups.size();
    for (size_t g = 0; g < h->groups.size(); ++g) {
        const nbo_group_config &c = h->groups[g].cfg;
        st.g[g] = DevGroup{c.lr, c.beta1, c.beta2, c.eps, c.weight_decay, c.kind, 0, h->groups[g].step_count};
    }
    NBO_CUDA(h, cudaMemcpyAsync(h->d_state, h->h_state, sizeof(DevState), cudaMemcpyHostToDevice, h->stream));
    return NBO_OK;
}

static bool valid_kind(int32_t k) { return k == NBO_ADAMW || k == NBO_ADAM || k == NBO_SGD; }

}  // namespace nbo

using namespace nbo;

// ---- C ABI ---------------------------------------------------------------------

extern "C" {

int32_t nbo_abi_version(void) { return 2; }

const char *nbo_last_error(const nbo_optimizer *h) { return h ? h->err.c_str() : g_err.c_str(); }

int32_t nbo_create(int32_t device, void *stream, nbo_optimizer **out)
{
    if (!out) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_create: null out pointer");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(nullptr, NBO_ERR_CUDA,
                    std::string("nabla-optim-b200: no CUDA device (there is no CPU fallback): ") +
                        cudaGetErrorString(e));
    if (device < 0 || device >= count)
        return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_create: device index out of range");
    nbo_optimizer *h = new (std::nothrow) nbo_optimizer();
    if (!h) return fail(nullptr, NBO_ERR_NOMEM, "nabla-optim-b200: out of host memory");
    h->device = device;
    h->stream = (cudaStream_t)stream;
    DeviceGuard guard(device);
    int32_t rc = [&]() -> int32_t {
        NBO_CUDA(h, cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, device));
        h->max_grid = h->sm_count * 16;
        NBO_CUDA(h, cudaMalloc(&h->d_partial_sum, h->max_grid * sizeof(double)));
        NBO_CUDA(h, cudaMalloc(&h->d_partial_bad, h->max_grid * sizeof(int32_t)));
        NBO_CUDA(h, cudaMalloc(&h->d_ticket, sizeof(uint32_t)));
        NBO_CUDA(h, cudaMemset(h->d_ticket, 0, sizeof(uint32_t)));
        NBO_CUDA(h, cudaMalloc(&h->d_local, 2 * sizeof(double)));
        NBO_CUDA(h, cudaMalloc(&h->d_ctrl, sizeof(StepCtrl)));
        NBO_CUDA(h, cudaMemset(h->d_ctrl, 0, sizeof(StepCtrl)));
        NBO_CUDA(h, cudaMallocHost(&h->h_ctrl, sizeof(StepCtrl)));
        memset(h->h_ctrl, 0, sizeof(StepCtrl));
        NBO_CUDA(h, cudaEventCreateWithFlags(&h->upload_done, cudaEventDisableTiming));
        NBO_CUDA(h, cudaMalloc(&h->d_state, sizeof(DevState)));
        NBO_CUDA(h, cudaMemset(h->d_state, 0, sizeof(DevState)));
        NBO_CUDA(h, cudaMallocHost(&h->h_state, sizeof(DevState)));
        memset(h->h_state, 0, sizeof(DevState));
        NBO_CUDA(h, cudaMalloc(&h->d_hp, kMaxDevGroups * sizeof(AdamHP)));
        NBO_CUDA(h, cudaMalloc(&h->d_inv_scale, sizeof(float)));
        return NBO_OK;
    }();
    if (rc != NBO_OK) {
        g_err = h->err;
        nbo_destroy(h);
        return rc;
    }
    *out = h;
    return NBO_OK;
}

int32_t nbo_destroy(nbo_optimizer *h)
{
    if (!h) return NBO_OK;
    DeviceGuard guard(h->device);
    cudaStreamSynchronize(h->stream);
    zero1_destroy(h);
    host_pipe_destroy(h);
    free_table(h);
    cudaFree(h->d_partial_sum); cudaFree(h->d_partial_bad); cudaFree(h->d_ticket);
    cudaFree(h->d_local); cudaFree(h->d_ctrl);
    if (h->h_ctrl) cudaFreeHost(h->h_ctrl);
    cudaFree(h->d_state); cudaFree(h->d_hp); cudaFree(h->d_inv_scale);
    if (h->h_state) cudaFreeHost(h->h_state);
    if (h->upload_done) cudaEventDestroy(h->upload_done);
    for (cudaEvent_t e : h->prof_ev)
        if (e) cudaEventDestroy(e);
    delete h;
    return NBO_OK;
}

int32_t nbo_add_group(nbo_optimizer *h, const nbo_group_config *cfg, int32_t *group_id)
{
    if (!h || !cfg) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: nbo_add_group: null argument");
    if (h->configured)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: nbo_add_group after the tensors were declared");
    if (!valid_kind(cfg->kind))
        return fail(h, NBO_ERR_INVALID, "bad optim.kind: " + std::to_string(cfg->kind));
    Group g;
    g.cfg = *cfg;
    g.base_lr = cfg->lr;
    g.step_count = 0;
    g.chunk_begin = g.chunk_end = 0;
    h->groups.push_back(g);
    if (group_id) *group_id = (int32_t)h->groups.size() - 1;
    return NBO_OK;
}

int32_t nbo_set_tensors(nbo_optimizer *h, uint64_t n, const uint64_t *numel, const int32_t *group_ids,
                        int32_t precision)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (h->configured) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: tensors already declared");
    if (h->groups.empty())
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: nbo_set_tensors before any nbo_add_group");
    if (n && !numel) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null numel list");
    if (precision != NBO_F32 && precision != NBO_MIXED_BF16 && precision != NBO_MIXED_BF16_F32GRAD)
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: unknown precision");
    for (uint64_t t = 0; t < n; ++t) {
        int32_t g = group_ids ? group_ids[t] : 0;
        if (g < 0 || (size_t)g >= h->groups.size())
            return fail(h, NBO_ERR_INVALID, "nabla-train: group assignment incomplete");
        if (precision != NBO_F32 && h->groups[g].cfg.kind == NBO_SGD)
            return fail(h, NBO_ERR_INVALID,
                        "nabla-optim-b200: mixed precision supports Adam/AdamW groups only");
    }
    DeviceGuard guard(h->device);
    h->precision = precision;
    h->ntensors = n;
    h->numel.assign(numel, numel + n);
    h->group_of.resize(n);
    h->piece_of.resize(n);
    h->pieces.clear();
    uint64_t off = 0;
    for (uint64_t t = 0; t < n; ++t) {
        h->group_of[t] = group_ids ? group_ids[t] : 0;
        Piece p;
        p.tensor = t; p.offset = 0; p.n = numel[t];
        p.state_off = off; p.bucket_off = 0; p.group = h->group_of[t];
        h->piece_of[t] = (int64_t)h->pieces.size();
        h->pieces.push_back(p);
        off += (numel[t] + 63) & ~63ull;  // every tensor's state starts 256-byte aligned
    }
    h->state_elems = off;
    int32_t rc = build_table(h);
    if (rc != NBO_OK) { free_table(h); h->configured = false; }
    return rc;
}

int32_t nbo_step(nbo_optimizer *h, uint64_t n, void *const *params, const void *const *grads)
{
    NBO_SYNC_STATE(h);
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (h->configured && h->precision != NBO_F32)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: nbo_step needs an fp32 handle; use nbo_step_mixed");
    if (n && (!params || !grads))
        return fail(h, NBO_ERR_INVALID, "nabla-train: params/grads length mismatch (null list)");
    DeviceGuard guard(h->device);
    int32_t rc = bind_list(h, n, params, grads, 4, "step");
    if (rc != NBO_OK) return rc;
    h->prof_norm_valid = false;
    prof_mark(h, 2);
    for (Group &g : h->groups) {
        uint32_t nc = g.chunk_end - g.chunk_begin;
        if (nc == 0) continue;
        if (g.cfg.kind == NBO_SGD)
            rc = launch_sgd_f32(h, g.chunk_begin, nc, sgd_hparams(g.cfg));
        else
            rc = launch_adam_f32(h, g.chunk_begin, nc, adam_hparams(g.cfg, g.step_count + 1, 1.0f));
        if (rc != NBO_OK) return rc;
    }
    // the counters advance only once every group has been launched, so a failed launch leaves them
    // in step with the state; an empty group counts too (alg.rs:120-121)
    for (Group &g : h->groups)
        if (g.cfg.kind != NBO_SGD) g.step_count += 1;
    return prof_mark(h, 3);
}

int32_t nbo_reset(nbo_optimizer *h)
{
    NBO_SYNC_STATE(h);
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    DeviceGuard guard(h->device);
    for (Group &g : h->groups) g.step_count = 0;
    if (h->configured) {
        size_t bytes = (size_t)h->state_elems * sizeof(float);
        if (bytes) {
            NBO_CUDA(h, cudaMemsetAsync(h->d_s0, 0, bytes, h->stream));
            NBO_CUDA(h, cudaMemsetAsync(h->d_s1, 0, bytes, h->stream));
        }
    }
    return NBO_OK;
}

int32_t nbo_set_lr(nbo_optimizer *h, double lr)
{
    NBO_SYNC_STATE(h);
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (h->groups.empty()) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: no group");
    if (h->groups.size() == 1) {
        h->groups[0].cfg.lr = lr;
        return NBO_OK;
    }
    double base = h->groups[0].base_lr;
    if (base <= 0.0) {
        for (Group &g : h->groups) g.cfg.lr = lr;
        return NBO_OK;
    }
    double scale = lr / base;
    for (Group &g : h->groups) g.cfg.lr = g.base_lr * scale;
    return NBO_OK;
}

static int32_t check_group(const nbo_optimizer *h, int32_t gid)
{
    if (!h) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (gid < 0 || (size_t)gid >= h->groups.size())
        return fail(const_cast<nbo_optimizer *>(h), NBO_ERR_INVALID,
                    "nabla-optim-b200: group index out of range");
    return NBO_OK;
}

int32_t nbo_get_lr(const nbo_optimizer *h, int32_t gid, double *lr)
{
    NBO_SYNC_STATE(h);
    int32_t rc = check_group(h, gid);
    if (rc != NBO_OK) return rc;
    if (lr) *lr = h->groups[gid].cfg.lr;
    return NBO_OK;
}

int32_t nbo_step_count(const nbo_optimizer *h, int32_t gid, uint64_t *count)
{
    NBO_SYNC_STATE(h);
    int32_t rc = check_group(h, gid);
    if (rc != NBO_OK) return rc;
    if (count) *count = h->groups[gid].step_count;
    return NBO_OK;
}

int32_t nbo_set_step_count(nbo_optimizer *h, int32_t gid, uint64_t count)
{
    NBO_SYNC_STATE(h);
    int32_t rc = check_group(h, gid);
    if (rc != NBO_OK) return rc;
    h->groups[gid].step_count = count;
    return NBO_OK;
}

int32_t nbo_get_group(const nbo_optimizer *h, int32_t gid, nbo_group_config *cfg)
{
    NBO_SYNC_STATE(h);
    int32_t rc = check_group(h, gid);
    if (rc != NBO_OK) return rc;
    if (cfg) *cfg = h->groups[gid].cfg;
    return NBO_OK;
}

int32_t nbo_set_group(nbo_optimizer *h, int32_t gid, const nbo_group_config *cfg)
{
    NBO_SYNC_STATE(h);
    int32_t rc = check_group(h, gid);
    if (rc != NBO_OK) return rc;
    if (!cfg) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null config");
    if (cfg->kind != h->groups[gid].cfg.kind)
        return fail(h, NBO_ERR_INVALID, "optim kind mismatch");  // load_meta wording, alg.rs:538
    h->groups[gid].cfg = *cfg;
    return NBO_OK;
}

static int32_t state_ptr(nbo_optimizer *h, uint64_t tensor, int32_t which, float **ptr, uint64_t *n)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (!h->configured) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: no tensors declared");
    if (h->zero1)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: sharded handle: use nbo_zero1_state_export");
    if (tensor >= h->ntensors)
        return fail(h, NBO_ERR_INVALID,
                    (which == 0 ? "m index out of range: " : "v index out of range: ") +
                        std::to_string(tensor));
    float *base = which == 0 ? h->d_s0 : which == 1 ? h->d_s1 : which == 2 ? h->d_s2 : nullptr;
    if (!base) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: this handle has no such state tensor");
    const Piece &p = h->pieces[(size_t)h->piece_of[tensor]];
    *ptr = base + p.state_off;
    *n = p.n;
    return NBO_OK;
}

int32_t nbo_state_export(nbo_optimizer *h, uint64_t tensor, int32_t which, float *dst)
{
    float *src; uint64_t n;
    int32_t rc = state_ptr(h, tensor, which, &src, &n);
    if (rc != NBO_OK) return rc;
    if (n && !dst) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null destination");
    DeviceGuard guard(h->device);
    if (n) NBO_CUDA(h, cudaMemcpyAsync(dst, src, n * sizeof(float), cudaMemcpyDeviceToHost, h->stream));
    NBO_CUDA(h, cudaStreamSynchronize(h->stream));
    return NBO_OK;
}

int32_t nbo_state_import(nbo_optimizer *h, uint64_t tensor, int32_t which, const float *srcp)
{
    float *dst; uint64_t n;
    int32_t rc = state_ptr(h, tensor, which, &dst, &n);
    if (rc != NBO_OK) return rc;
    if (n && !srcp) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null source");
    DeviceGuard guard(h->device);
    if (n) NBO_CUDA(h, cudaMemcpyAsync(dst, srcp, n * sizeof(float), cudaMemcpyHostToDevice, h->stream));
    NBO_CUDA(h, cudaStreamSynchronize(h->stream));
    return NBO_OK;
}

int32_t nbo_scaler_get(const nbo_optimizer *h, nbo_scaler_state *out)
{
    NBO_SYNC_STATE(h);
    if (!h || !out) return fail(const_cast<nbo_optimizer *>(h), NBO_ERR_INVALID, "nabla-optim-b200: null argument");
    *out = h->scaler;
    return NBO_OK;
}

int32_t nbo_scaler_set(nbo_optimizer *h, const nbo_scaler_state *in)
{
    NBO_SYNC_STATE(h);
    if (!h || !in) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null argument");
    h->scaler = *in;
    return NBO_OK;
}

int32_t nbo_zero_grad(nbo_optimizer *h, uint64_t n, void *const *grads)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (n && !grads) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null pointer list");
    DeviceGuard guard(h->device);
    bool bf16 = h->precision == NBO_MIXED_BF16;  // the gradient column is bf16 only in this mode
    int32_t rc = bind_list(h, n, nullptr, (const void *const *)grads, bf16 ? 2 : 4, "zero_grad");
    if (rc != NBO_OK) return rc;
    return launch_zero_grads(h, bf16);
}

int32_t nbo_accumulate_grads(nbo_optimizer *h, uint64_t n, void *const *accum, const void *const *grads)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (n && (!accum || !grads)) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null pointer list");
    if (h->configured && h->precision != NBO_F32)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: gradient accumulation is defined for fp32 gradients");
    DeviceGuard guard(h->device);
    int32_t rc = bind_list(h, n, accum, grads, 4, "accumulate_grads");
    if (rc != NBO_OK) return rc;
    return launch_accumulate(h);
}

int32_t nbo_unscale_and_update(nbo_optimizer *h, uint64_t n, void *const *grads, int32_t *ok)
{
    NBO_SYNC_STATE(h);
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (n && !grads) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null pointer list");
    if (h->configured && h->precision != NBO_F32)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: bf16 gradients are unscaled inside nbo_step_mixed");
    DeviceGuard guard(h->device);
    int32_t rc = bind_list(h, n, nullptr, (const void *const *)grads, 4, "unscale_and_update");
    if (rc != NBO_OK) return rc;
    float inv_scale = (float)(1.0 / h->scaler.scale);
    // the flag is taken on the still-scaled values: the norm pass multiplies by 1.0f here
    rc = launch_norm(h, false, 1.0f, 0.0, 1);
    if (rc != NBO_OK) return rc;
    rc = launch_scale_grads(h, 0, inv_scale);
    if (rc != NBO_OK) return rc;
    rc = read_ctrl(h);
    if (rc != NBO_OK) return rc;
    bool bad = h->h_ctrl->nonfinite != 0;
    if (bad) {
        h->scaler.scale *= h->scaler.backoff_factor;
        h->scaler.consecutive_ok = 0;
    } else {
        h->scaler.consecutive_ok += 1;
        if (h->scaler.consecutive_ok >= h->scaler.growth_interval) {
            h->scaler.scale *= h->scaler.growth_factor;
            h->scaler.consecutive_ok = 0;
        }
    }
    if (ok) *ok = bad ? 0 : 1;
    return NBO_OK;
}

int32_t nbo_clip_grad_norm(nbo_optimizer *h, uint64_t n, void *const *grads, double max_norm,
                           double *norm)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (norm) *norm = 0.0;
    if (max_norm <= 0.0) return NBO_OK;  // trainer.rs:501-503
    if (n && !grads) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null pointer list");
    if (h->configured && h->precision != NBO_F32)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: bf16 gradients are clipped inside nbo_step_mixed");
    DeviceGuard guard(h->device);
    int32_t rc = bind_list(h, n, nullptr, (const void *const *)grads, 4, "clip_grad_norm");
    if (rc != NBO_OK) return rc;
    rc = launch_norm(h, false, 1.0f, max_norm, 1);
    if (rc != NBO_OK) return rc;
    rc = launch_scale_grads(h, 1, 1.0f);
    if (rc != NBO_OK) return rc;
    rc = read_ctrl(h);
    if (rc != NBO_OK) return rc;
    if (norm) *norm = h->h_ctrl->norm;
    return NBO_OK;
}

int32_t nbo_grad_norm(nbo_optimizer *h, uint64_t n, const void *const *grads, double *norm,
                      int32_t *nonfinite)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (n && !grads) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null pointer list");
    DeviceGuard guard(h->device);
    bool bf16 = h->precision == NBO_MIXED_BF16;
    int32_t rc = bind_list(h, n, nullptr, grads, bf16 ? 2 : 4, "grad_norm");
    if (rc != NBO_OK) return rc;
    rc = launch_norm(h, bf16, 1.0f, 0.0, 1);
    if (rc != NBO_OK) return rc;
    rc = read_ctrl(h);
    if (rc != NBO_OK) return rc;
    if (norm) *norm = h->h_ctrl->norm;
    if (nonfinite) *nonfinite = h->h_ctrl->nonfinite;
    return NBO_OK;
}

int32_t nbo_init_master_from_params(nbo_optimizer *h, uint64_t n, const void *const *params_bf16)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (!h->configured || h->precision == NBO_F32)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: masters exist only on mixed-precision handles");
    if (n && !params_bf16) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null pointer list");
    DeviceGuard guard(h->device);
    int32_t rc = bind_list(h, n, (void *const *)params_bf16, nullptr, 2, "init_master");
    if (rc != NBO_OK) return rc;
    return launch_init_master(h);
}

int32_t nbo_step_mixed(nbo_optimizer *h, uint64_t n, void *const *params_bf16,
                       const void *const *grads_bf16, int32_t use_scaler, double max_norm,
                       nbo_step_result *result)
{
    NBO_SYNC_STATE(h);
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (h->configured && h->precision == NBO_F32)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: nbo_step_mixed needs a mixed-precision handle");
    if (n && (!params_bf16 || !grads_bf16))
        return fail(h, NBO_ERR_INVALID, "nabla-train: params/grads length mismatch (null list)");
    DeviceGuard guard(h->device);
    int32_t rc = bind_list(h, n, params_bf16, grads_bf16, 2, "step");
    if (rc != NBO_OK) return rc;
    bool checked = use_scaler || max_norm > 0.0;
    float inv_scale = use_scaler ? (float)(1.0 / h->scaler.scale) : 1.0f;
    h->prof_norm_valid = false;
    if (checked) {
        prof_mark(h, 0);
        // loss scaling without clipping needs the skip decision only (clip_grad_norm is then not run and
        // reports 0, trainer.rs:501-503): the flag-only pass is a plain HBM read
        rc = max_norm > 0.0 ? launch_norm(h, h->precision == NBO_MIXED_BF16, inv_scale, max_norm, 1)
                            : launch_nonfinite(h, h->precision == NBO_MIXED_BF16);
        if (rc != NBO_OK) return rc;
        prof_mark(h, 1);
    }
    prof_mark(h, 2);
    rc = launch_mixed_update(h, inv_scale, checked);
    if (rc != NBO_OK) return rc;
    prof_mark(h, 3);
    if (checked) {
        rc = read_ctrl(h);
        if (rc != NBO_OK) return rc;
    } else {
        NBO_CUDA(h, cudaStreamSynchronize(h->stream));
    }
    commit_step(h, checked, use_scaler != 0, result);
    return NBO_OK;
}

int32_t nbo_step_mixed_async(nbo_optimizer *h, uint64_t n, void *const *params_bf16,
                             const void *const *grads_bf16, int32_t use_scaler, double max_norm)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (!h->configured || h->precision == NBO_F32 || h->zero1)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: nbo_step_mixed_async needs an unsharded mixed-precision handle");
    if (h->groups.size() > (size_t)kMaxDevGroups)
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: the asynchronous step supports at most 32 groups");
    if (n && (!params_bf16 || !grads_bf16))
        return fail(h, NBO_ERR_INVALID, "nabla-train: params/grads length mismatch (null list)");
    DeviceGuard guard(h->device);
    int32_t rc = bind_list(h, n, params_bf16, grads_bf16, 2, "step");
    if (rc != NBO_OK) return rc;
    rc = push_dev_state(h);
    if (rc != NBO_OK) return rc;
    bool checked = use_scaler || max_norm > 0.0;
    rc = launch_prepare(h, use_scaler);
    if (rc != NBO_OK) return rc;
    if (checked) {
        rc = max_norm > 0.0 ? launch_norm_dev(h, h->d_inv_scale, max_norm)
                            : launch_nonfinite(h, h->precision == NBO_MIXED_BF16);
        if (rc != NBO_OK) return rc;
    }
    for (size_t g = 0; g < h->groups.size(); ++g) {
        const Group &gr = h->groups[g];
        rc = launch_adam_mixed_dev(h, gr.chunk_begin, gr.chunk_end - gr.chunk_begin, (int)g, checked);
        if (rc != NBO_OK) return rc;
    }
    rc = launch_commit(h, checked, use_scaler);
    if (rc != NBO_OK) return rc;
    h->dev_newer = true;
    h->last_async_checked = checked;
    return NBO_OK;
}

int32_t nbo_step_mixed_collect(nbo_optimizer *h, nbo_step_result *result, uint64_t *steps_enqueued)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (!h->dev_newer && h->h_state->ngroups == 0)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: no asynchronous step has been enqueued");
    DeviceGuard guard(h->device);
    int32_t rc = collect_dev_state(h);
    if (rc != NBO_OK) return rc;
    const DevState &st = *h->h_state;
    if (result) {
        result->applied = st.last_applied;
        result->nonfinite = st.last_nonfinite;
        result->grad_norm = st.last_norm;
        result->loss_scale = st.scale;
        result->step_count = st.ngroups > 0 ? st.g[0].step_count : 0;
    }
    if (steps_enqueued) *steps_enqueued = st.steps_enqueued;
    return NBO_OK;
}

// ---- LR schedules: pure host f64 (nabla-train/src/optim/core.rs:81-173) ---------

static double umax1(uint64_t v) { return (double)(v > 1 ? v : 1); }
static double warmup_lr(double base, uint64_t step, uint64_t warmup) { return base * (double)step / umax1(warmup); }
static double decay_progress(uint64_t step, uint64_t start, uint64_t total)
{
    return (double)(step - start) / umax1(total - start);
}
static double cosine_decay(double high, double low, double progress)
{
    return low + 0.5 * (high - low) * (1.0 + cos(3.14159265358979323846264338327950288 * progress));
}

int32_t nbo_lr_at_step(const nbo_lr_schedule *s, double base_lr, uint64_t step, double *lr)
{
    if (!s || !lr) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: nbo_lr_at_step: null argument");
    switch (s->kind) {
    case NBO_SCHED_COSINE:
        *lr = step < s->warmup_steps
                  ? warmup_lr(base_lr, step, s->warmup_steps)
                  : cosine_decay(base_lr, s->min_lr, decay_progress(step, s->warmup_steps, s->total_steps));
        return NBO_OK;
    case NBO_SCHED_LINEAR:
        if (step < s->warmup_steps) {
            *lr = warmup_lr(base_lr, step, s->warmup_steps);
        } else {
            double pr = 1.0 - decay_progress(step, s->warmup_steps, s->total_steps);
            *lr = base_lr * (pr > 0.0 ? pr : 0.0);
        }
        return NBO_OK;
    case NBO_SCHED_ONECYCLE: {
        uint64_t up = (uint64_t)((double)s->total_steps * s->pct_start);
        *lr = step < up ? base_lr + (s->max_lr - base_lr) * (double)step / umax1(up)
                        : cosine_decay(s->max_lr, base_lr, decay_progress(step, up, s->total_steps));
        return NBO_OK;
    }
    case NBO_SCHED_STEP: {
        uint64_t k = step / (s->step_size > 1 ? s->step_size : 1);
        *lr = base_lr * powi(s->gamma, (int32_t)k);
        return NBO_OK;
    }
    default:
        return fail(nullptr, NBO_ERR_INVALID, "bad schedule.kind: " + std::to_string(s->kind));
    }
}

int32_t nbo_profile(nbo_optimizer *h, int32_t on)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    DeviceGuard guard(h->device);
    if (on && !h->prof_ev[0])
        for (cudaEvent_t &e : h->prof_ev) NBO_CUDA(h, cudaEventCreate(&e));
    h->profile = on != 0;
    h->prof_norm_valid = h->prof_update_valid = false;
    return NBO_OK;
}

int32_t nbo_profile_last(nbo_optimizer *h, float *norm_ms, float *update_ms)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (!h->profile) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: profiling is off (nbo_profile)");
    DeviceGuard guard(h->device);
    NBO_CUDA(h, cudaStreamSynchronize(h->stream));
    float a = 0.f, b = 0.f;
    if (h->prof_norm_valid) NBO_CUDA(h, cudaEventElapsedTime(&a, h->prof_ev[0], h->prof_ev[1]));
    if (h->prof_update_valid) NBO_CUDA(h, cudaEventElapsedTime(&b, h->prof_ev[2], h->prof_ev[3]));
    if (norm_ms) *norm_ms = a;
    if (update_ms) *update_ms = b;
    return NBO_OK;
}

int32_t nbo_launch_count(const nbo_optimizer *h, uint64_t *launches)
{
    if (!h || !launches) return fail(const_cast<nbo_optimizer *>(h), NBO_ERR_INVALID, "nabla-optim-b200: null argument");
    *launches = h->launches;
    return NBO_OK;
}

int32_t nbo_table_info(const nbo_optimizer *h, uint64_t *tensors, uint64_t *chunks, uint64_t *uploads)
{
    if (!h) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (tensors) *tensors = h->pieces.size();
    if (chunks) *chunks = h->nchunks;
    if (uploads) *uploads = h->uploads;
    return NBO_OK;
}

}  // extern "C"
