// ZeRO-1 sharding of the mixed-precision step over NCCL: one process per GPU,
// state (fp32 master, m, v) kept only for this rank's slice of one flat bf16
// bucket.  Replaces the reference's two-rank in-process mean
// (nabla-train/src/dist.rs:7-44) with reduce-scatter -> local fused update ->
// all-gather over NVLink.
//
// NCCL is opened with dlopen on first use, so a single-GPU consumer does not
// need the library at all; world == 1 never touches it.  Two forms of the step
// live here: nbo_zero1_step, whose kernels read local memory only (remote data
// arrives through NCCL collectives first), and nbo_zero1_step_fused, whose
// kernels (fused_nvlink.cuh) load and store the other ranks' buckets directly
// over NVLink with NCCL used only for the stream-ordered barriers around them.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <chrono>
#include <thread>

#include "host_plan.h"
#include "internal.h"

namespace nbo {

struct NcclApi {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                                  cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    std::string why;
};

static NcclApi *nccl_api()
{
    static NcclApi api;
    if (api.lib || !api.why.empty()) return &api;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        api.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (api.lib) break;
    }
    if (!api.lib) {
        api.why = std::string("cannot open libnccl.so.2: ") + dlerror();
        return &api;
    }
#define NBO_SYM(field, name)                                                     \
    do {                                                                         \
        *(void **)(&api.field) = dlsym(api.lib, name);                           \
        if (!api.field) { api.why = std::string("NCCL symbol missing: ") + name; } \
    } while (0)
    NBO_SYM(GetUniqueId, "ncclGetUniqueId");
    NBO_SYM(CommInitRankConfig, "ncclCommInitRankConfig");
    NBO_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    NBO_SYM(CommDestroy, "ncclCommDestroy");
    NBO_SYM(CommAbort, "ncclCommAbort");
    NBO_SYM(ReduceScatter, "ncclReduceScatter");
    NBO_SYM(AllGather, "ncclAllGather");
    NBO_SYM(AllReduce, "ncclAllReduce");
    NBO_SYM(GetErrorString, "ncclGetErrorString");
#undef NBO_SYM
    return &api;
}

struct Zero1 {
    int rank = 0, world = 1;
    uint64_t total = 0, shard = 0, padded = 0, begin = 0, end = 0;
    ncclComm_t comm = nullptr;  // non-blocking communicator: every call is followed by a bounded wait
    double timeout_s = 600.0;   // host-side limit for joining the communicator and for each step's completion
    bool broken = false;        // the communicator was aborted after a timeout or an error
    double *d_gathered = nullptr;  // {sumsq, nonfinite} of every rank, rank order
    // fused path: symmetric-memory buckets
    bool attached = false;
    int transport = 0;             // 1 = plain peer loads/stores, 2 = NVSwitch multicast
    void *g_local = nullptr, *p_local = nullptr;
    PeerArgs pa{};
    int32_t *d_barrier = nullptr;  // [0] the sequence number this rank contributes, [1] the all-reduced (max) result
    int32_t barrier_seq = 0;       // barriers enqueued so far; every rank enqueues the same ones in the same order
    bool keep_reduced = true;      // the fused kernels also leave the reduced gradient in the local slice
};

static int32_t fail_nccl(nbo_optimizer *h, ncclResult_t r, const char *what)
{
    NcclApi *a = nccl_api();
    std::string m = std::string("NCCL error: ") + (a->GetErrorString ? a->GetErrorString(r) : "?") +
                    " in " + what;
    return fail(h, NBO_ERR_NCCL, m);
}

using Clock = std::chrono::steady_clock;

static void abort_comm(Zero1 *z)
{
    if (z->comm) nccl_api()->CommAbort(z->comm);  // also ends an NCCL kernel that waits for a rank that is gone
    z->comm = nullptr;
    z->broken = true;
}

// Failure detection lives on the host: a non-blocking NCCL call is followed until the communicator reports
// success, an error, or the time limit; on the limit the communicator is aborted and the caller gets
// NBO_ERR_TIMEOUT with the CUDA context intact.  No device code waits on another rank.
static int32_t nccl_wait(nbo_optimizer *h, Zero1 *z, ncclResult_t r, const char *what)
{
    NcclApi *a = nccl_api();
    const auto start = Clock::now();
    const auto deadline = start + std::chrono::duration<double>(z->timeout_s);
    while (r == ncclSuccess || r == ncclInProgress) {
        ncclResult_t st = ncclSuccess;
        ncclResult_t q = a->CommGetAsyncError(z->comm, &st);
        if (q != ncclSuccess) { r = q; break; }
        if (st == ncclSuccess) return NBO_OK;
        if (st != ncclInProgress) { r = st; break; }
        if (Clock::now() > deadline) {
            abort_comm(z);
            return fail(h, NBO_ERR_TIMEOUT, std::string("nabla-optim-b200: timed out after ") +
                                                std::to_string(z->timeout_s) + " s in " + what +
                                                " (a rank did not arrive); communicator aborted");
        }
        // an enqueue normally completes within microseconds: spin first, back off only when it drags on
        if (Clock::now() - start < std::chrono::milliseconds(2)) std::this_thread::yield();
        else std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    abort_comm(z);
    return fail_nccl(h, r, what);
}

// Bounded replacement for cudaStreamSynchronize on a stream that carries collectives.
static int32_t stream_wait(nbo_optimizer *h, Zero1 *z, const char *what)
{
    const auto deadline = Clock::now() + std::chrono::duration<double>(z->timeout_s);
    for (;;) {
        cudaError_t e = cudaStreamQuery(h->stream);
        if (e == cudaSuccess) return NBO_OK;
        if (e != cudaErrorNotReady) return fail_cuda(h, e, what);
        if (z->world > 1 && Clock::now() > deadline) {
            abort_comm(z);                       // lets the stuck collective return
            cudaStreamSynchronize(h->stream);    // what follows it on the stream touches local memory only
            return fail(h, NBO_ERR_TIMEOUT, std::string("nabla-optim-b200: timed out after ") +
                                                std::to_string(z->timeout_s) + " s waiting for " + what +
                                                " (a rank stopped taking part); communicator aborted");
        }
        std::this_thread::yield();
    }
}

#define NBO_NCCL(h, call)                                   \
    do {                                                    \
        int32_t rc__ = nccl_wait((h), z, (call), #call);    \
        if (rc__ != NBO_OK) return rc__;                    \
    } while (0)

// Stream-ordered cross-rank barrier: every rank writes the next sequence number and the ranks all-reduce it
// (max).  *expect receives the number the result holds once the barrier has completed; kernels enqueued
// behind it compare (barrier_passed in fused_nvlink.cuh) and leave peer memory alone when it has not.
static int32_t enqueue_barrier(nbo_optimizer *h, Zero1 *z, int32_t *expect)
{
    NcclApi *a = nccl_api();
    z->barrier_seq += 1;
    int32_t rc = launch_store_int(h, z->d_barrier, z->barrier_seq);
    if (rc != NBO_OK) return rc;
    NBO_NCCL(h, a->AllReduce(z->d_barrier, z->d_barrier + 1, 1, ncclInt32, ncclMax, z->comm, h->stream));
    if (expect) *expect = z->barrier_seq;
    return NBO_OK;
}

// The pieces (tensor intersections) of rank `rank`'s shard, in list order: the rows of that rank's table.
static std::vector<Piece> shard_pieces(const std::vector<uint64_t> &numel, const std::vector<int32_t> &group_of,
                                       int rank, uint64_t shard)
{
    std::vector<Piece> out;
    for (const ShardRow &r : shard_rows(numel, group_of, rank, shard)) {
        Piece p;
        p.tensor = r.tensor; p.offset = r.offset; p.n = r.n;
        p.bucket_off = r.bucket_off; p.state_off = r.bucket_off - (uint64_t)rank * shard; p.group = r.group;
        out.push_back(p);
    }
    return out;
}

int32_t zero1_bounded_wait(nbo_optimizer *h, const char *what) { return stream_wait(h, h->zero1, what); }

void zero1_destroy(nbo_optimizer *h)
{
    if (!h->zero1) return;
    Zero1 *z = h->zero1;
    if (z->comm) {
        cudaStreamSynchronize(h->stream);
        nccl_api()->CommDestroy(z->comm);
    }
    cudaFree(z->d_gathered);
    cudaFree(z->d_barrier);
    delete z;
    h->zero1 = nullptr;
}

static void geometry(uint64_t total, int32_t world, uint64_t *shard, uint64_t *padded)
{
    uint64_t per = (total + (uint64_t)world - 1) / (uint64_t)world;
    per = (per + 7) & ~7ull;  // 8 bf16 = 16 bytes
    if (per == 0) per = 8;
    *shard = per;
    *padded = per * (uint64_t)world;
}

}  // namespace nbo

using namespace nbo;

extern "C" {

int32_t nbo_zero1_unique_id(uint8_t id_out[128])
{
    if (!id_out) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: null id buffer");
    NcclApi *a = nccl_api();
    if (!a->why.empty()) return fail(nullptr, NBO_ERR_NCCL, a->why);
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    ncclUniqueId id;
    ncclResult_t r = a->GetUniqueId(&id);
    if (r != ncclSuccess) return fail_nccl(nullptr, r, "ncclGetUniqueId");
    memcpy(id_out, &id, 128);
    return NBO_OK;
}

int32_t nbo_zero1_geometry(uint64_t total, int32_t world, uint64_t *shard_elems, uint64_t *padded_total)
{
    if (world < 1) return fail(nullptr, NBO_ERR_INVALID, "nabla-optim-b200: world must be >= 1");
    uint64_t s, p;
    geometry(total, world, &s, &p);
    if (shard_elems) *shard_elems = s;
    if (padded_total) *padded_total = p;
    return NBO_OK;
}

int32_t nbo_zero1_init(nbo_optimizer *h, uint64_t n, const uint64_t *numel, const int32_t *group_ids,
                       int32_t rank, int32_t world, const uint8_t unique_id[128])
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (h->configured) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: tensors already declared");
    if (h->groups.empty())
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: nbo_zero1_init before any nbo_add_group");
    if (world < 1 || rank < 0 || rank >= world)
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: rank/world out of range");
    if (n && !numel) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null numel list");
    if (world > 1 && !unique_id)
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: world > 1 needs the NCCL unique id");
    for (uint64_t t = 0; t < n; ++t) {
        int32_t g = group_ids ? group_ids[t] : 0;
        if (g < 0 || (size_t)g >= h->groups.size())
            return fail(h, NBO_ERR_INVALID, "nabla-train: group assignment incomplete");
        if (h->groups[g].cfg.kind == NBO_SGD)
            return fail(h, NBO_ERR_INVALID,
                        "nabla-optim-b200: mixed precision supports Adam/AdamW groups only");
    }
    cudaError_t ce = cudaSetDevice(h->device);
    if (ce != cudaSuccess) return fail_cuda(h, ce, "cudaSetDevice");

    Zero1 *z = new Zero1();
    z->rank = rank; z->world = world;
    z->timeout_s = h->zero1_timeout_s;
    uint64_t total = 0;
    for (uint64_t t = 0; t < n; ++t) total += numel[t];
    z->total = total;
    geometry(total, world, &z->shard, &z->padded);
    z->begin = (uint64_t)rank * z->shard;
    z->end = z->begin + z->shard;
    h->zero1 = z;

    h->precision = NBO_MIXED_BF16;
    h->ntensors = n;
    h->numel.assign(numel, numel + n);
    h->group_of.resize(n);
    h->piece_of.assign(n, -1);
    for (uint64_t t = 0; t < n; ++t) h->group_of[t] = group_ids ? group_ids[t] : 0;
    h->pieces = shard_pieces(h->numel, h->group_of, rank, z->shard);
    for (size_t i = 0; i < h->pieces.size(); ++i) h->piece_of[h->pieces[i].tensor] = (int64_t)i;
    h->state_elems = z->shard;
    int32_t rc = build_table(h);
    if (rc != NBO_OK) { free_table(h); h->configured = false; zero1_destroy(h); return rc; }

    if (world > 1) {
        NcclApi *a = nccl_api();
        if (!a->why.empty()) { std::string w = a->why; zero1_destroy(h); return fail(h, NBO_ERR_NCCL, w); }
        NBO_CUDA(h, cudaMalloc(&z->d_gathered, 2 * sizeof(double) * world));
        ncclUniqueId id;
        memcpy(&id, unique_id, 128);
        ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
        config.blocking = 0;  // so that a rank that never arrives ends in a timeout, not in a hang
        NBO_NCCL(h, a->CommInitRankConfig(&z->comm, world, id, rank, &config));
    }
    return NBO_OK;
}

int32_t nbo_zero1_set_timeout(nbo_optimizer *h, double seconds)
{
    if (!h) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null handle");
    if (!(seconds > 0.0)) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: the timeout must be positive");
    h->zero1_timeout_s = seconds;
    if (h->zero1) h->zero1->timeout_s = seconds;
    return NBO_OK;
}

int32_t nbo_zero1_shard(const nbo_optimizer *h, uint64_t *begin, uint64_t *end, uint64_t *pieces)
{
    if (!h || !h->zero1)
        return fail(const_cast<nbo_optimizer *>(h), NBO_ERR_STATE, "nabla-optim-b200: not a ZeRO-1 handle");
    if (begin) *begin = h->zero1->begin;
    if (end) *end = h->zero1->end;
    if (pieces) *pieces = h->pieces.size();
    return NBO_OK;
}

int32_t nbo_zero1_init_master(nbo_optimizer *h, const void *params_flat_bf16)
{
    if (!h || !h->zero1) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: not a ZeRO-1 handle");
    if (!params_flat_bf16) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null bucket");
    cudaError_t ce = cudaSetDevice(h->device);
    if (ce != cudaSuccess) return fail_cuda(h, ce, "cudaSetDevice");
    // bind only the params; the gradient column keeps pointing at the same bucket offsets
    int32_t rc = bind_flat(h, (void *)params_flat_bf16, params_flat_bf16);
    if (rc != NBO_OK) return rc;
    h->table_bound = false;  // the next step must rebind with the real gradient bucket
    return launch_init_master(h);
}

int32_t nbo_zero1_step(nbo_optimizer *h, void *params_flat, void *grads_flat, int32_t average,
                       int32_t use_scaler, double max_norm, nbo_step_result *result)
{
    NBO_SYNC_STATE(h);
    if (!h || !h->zero1) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: not a ZeRO-1 handle");
    if (!params_flat || !grads_flat) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null bucket");
    Zero1 *z = h->zero1;
    if (z->broken) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: the communicator was aborted; create a new handle");
    cudaError_t ce = cudaSetDevice(h->device);
    if (ce != cudaSuccess) return fail_cuda(h, ce, "cudaSetDevice");
    NcclApi *a = z->world > 1 ? nccl_api() : nullptr;
    uint16_t *gflat = (uint16_t *)grads_flat;
    uint16_t *pflat = (uint16_t *)params_flat;

    int32_t rc = bind_flat(h, params_flat, grads_flat);
    if (rc != NBO_OK) return rc;

    if (z->world > 1)  // in place: this rank's reduced slice lands at its own offset
        NBO_NCCL(h, a->ReduceScatter(gflat, gflat + z->begin, z->shard, ncclBfloat16,
                                     average ? ncclAvg : ncclSum, z->comm, h->stream));

    bool checked = use_scaler || max_norm > 0.0;
    float inv_scale = use_scaler ? (float)(1.0 / h->scaler.scale) : 1.0f;
    h->prof_norm_valid = false;
    if (checked) {
        prof_mark(h, 0);
        rc = launch_norm(h, true, inv_scale, max_norm, z->world == 1);
        if (rc != NBO_OK) return rc;
        prof_mark(h, 1);
        if (z->world > 1) {
            NBO_NCCL(h, a->AllGather(h->d_local, z->d_gathered, 2, ncclDouble, z->comm, h->stream));
            rc = launch_finalize_ranks(h, z->d_gathered, z->world, max_norm);
            if (rc != NBO_OK) return rc;
        }
    }
    prof_mark(h, 2);
    rc = launch_mixed_update(h, inv_scale, checked);
    if (rc != NBO_OK) return rc;
    prof_mark(h, 3);

    if (z->world > 1)
        NBO_NCCL(h, a->AllGather(pflat + z->begin, pflat, z->shard, ncclBfloat16, z->comm, h->stream));

    if (checked) {
        NBO_CUDA(h, cudaMemcpyAsync(h->h_ctrl, h->d_ctrl, sizeof(StepCtrl), cudaMemcpyDeviceToHost,
                                    h->stream));
    }
    rc = stream_wait(h, z, "the sharded step");
    if (rc != NBO_OK) return rc;
    commit_step(h, checked, use_scaler != 0, result);
    return NBO_OK;
}

// Enqueues one fused sharded step on the attached buckets, up to and including the closing barrier and the
// copy of the decision record; nothing here waits on the host.
// dev_state: the asynchronous form - hyper-parameters, loss scale and step counters are read from and advanced
// in the handle's device-resident state (prepare_kernel / commit_kernel), nothing is read back.
static int32_t enqueue_fused_step(nbo_optimizer *h, Zero1 *z, int32_t average, int32_t use_scaler, double max_norm,
                                  bool dev_state = false)
{
    NcclApi *a = nccl_api();
    PeerArgs pa = z->pa;
    pa.average = average ? 1 : 0;
    pa.keep_reduced = z->keep_reduced ? 1 : 0;
    pa.barrier_seen = z->d_barrier + 1;
    if (dev_state) {
        int32_t r0 = push_dev_state(h);
        if (r0 != NBO_OK) return r0;
        r0 = launch_prepare(h, use_scaler);
        if (r0 != NBO_OK) return r0;
        pa.inv_scale_dev = h->d_inv_scale;
    }

    // every rank's gradients are final, and nobody still reads the old params, before any peer access
    int32_t rc = enqueue_barrier(h, z, &pa.barrier_expect);
    if (rc != NBO_OK) return rc;

    bool checked = use_scaler || max_norm > 0.0;
    float inv_scale = use_scaler ? (float)(1.0 / h->scaler.scale) : 1.0f;
    h->prof_norm_valid = false;
    int in_transport = z->transport;
    if (checked) {
        prof_mark(h, 0);
        rc = launch_zero1_reduce_norm(h, inv_scale, pa, z->transport);
        if (rc != NBO_OK) return rc;
        prof_mark(h, 1);
        NBO_NCCL(h, a->AllGather(h->d_local, z->d_gathered, 2, ncclDouble, z->comm, h->stream));
        rc = launch_finalize_ranks(h, z->d_gathered, z->world, max_norm);
        if (rc != NBO_OK) return rc;
        in_transport = 0;  // the reduced gradient now sits in the local slice
    }
    prof_mark(h, 2);
    for (Group &g : h->groups) {
        uint32_t nc = g.chunk_end - g.chunk_begin;
        if (nc == 0) continue;
        AdamHP hp = adam_hparams(g.cfg, g.step_count + 1, inv_scale);
        if (dev_state) pa.hp_dev = h->d_hp + (&g - h->groups.data());
        rc = launch_zero1_fused_update(h, g.chunk_begin, nc, hp, checked, pa, in_transport, z->transport);
        if (rc != NBO_OK) return rc;
    }
    prof_mark(h, 3);
    // every rank's parameter stores have landed everywhere before anyone uses the params
    rc = enqueue_barrier(h, z, nullptr);
    if (rc != NBO_OK) return rc;
    if (dev_state) {
        rc = launch_commit(h, checked, use_scaler);
        if (rc != NBO_OK) return rc;
        h->dev_newer = true;
        h->last_async_checked = checked;
        return NBO_OK;
    }
    if (checked)
        NBO_CUDA(h, cudaMemcpyAsync(h->h_ctrl, h->d_ctrl, sizeof(StepCtrl), cudaMemcpyDeviceToHost,
                                    h->stream));
    return NBO_OK;
}



// Host-streamed sharded step, world > 1, on the attached symmetric buckets.
//
// Every rank holds its own gradients for the WHOLE parameter list in host memory (data-parallel replicas)
// and wants the updated parameters of its shard back in host memory.  Rank q's table is cut into slices of
// about `slice_elems` elements; slice s of the step is "slice s of every rank's shard".  Per slice, on every rank:
//   copy-in stream : this rank's host gradients for slice s of ALL ranks' shards -> its device bucket
//   compute stream : barrier (all ranks have slice s on the device) -> fused kernel over this rank's
//                    slice s (reads every rank's bucket, writes every rank's parameter bucket)
//   copy-out stream: this rank's slice s of the parameters -> host
// so the PCIe copies of slice s+1 run while slice s is reduced, updated and published over NVLink.  Every
// rank derives every rank's slice boundaries from the declared sizes alone (same planner, same inputs), so
// no geometry is exchanged.  With loss scaling or clipping the decision needs every gradient first: all
// slices are copied in, the fused checked step runs, and the shard is copied out unless the step was skipped.
static int32_t zero1_host_step_sharded(nbo_optimizer *h, Zero1 *z, void *const *host_p, const void *const *host_g,
                                       uint64_t slice_elems, int32_t average, int32_t use_scaler, double max_norm,
                                       nbo_step_result *result)
{
    for (uint64_t t = 0; t < h->ntensors; ++t)
        if (h->numel[t] && (!host_p[t] || !host_g[t]))
            return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null host pointer for tensor " + std::to_string(t));
    if (slice_elems == 0) {  // 64 MiB of bf16 copied in per slice, but no slice shorter than 1 Mi elements
        slice_elems = (32ull << 20) / (uint64_t)z->world;
        if (slice_elems < (1ull << 20)) slice_elems = 1ull << 20;
    }
    const uint64_t slice_chunks = (slice_elems + kChunkElems - 1) / kChunkElems;

    // every rank's rows and slice plan
    std::vector<std::vector<Piece>> rows(z->world);
    std::vector<HostPlan> plans(z->world);
    size_t ns = 0;
    for (int q = 0; q < z->world; ++q) {
        rows[q] = q == z->rank ? h->pieces : shard_pieces(h->numel, h->group_of, q, z->shard);
        const size_t np = rows[q].size();
        std::vector<uint64_t> row_n(np);
        std::vector<uint32_t> row_head(np);
        std::vector<int32_t> row_group(np);
        for (size_t i = 0; i < np; ++i) {
            row_n[i] = rows[q][i].n;
            row_head[i] = bucket_row_head(rows[q][i].bucket_off);  // as bind_flat sets it
            row_group[i] = rows[q][i].group;
        }
        plans[q] = plan_host_slices(row_n, row_head, row_group, (int32_t)h->groups.size(), slice_chunks);
        if (plans[q].slices.size() > ns) ns = plans[q].slices.size();
    }
    const HostPlan &mine = plans[z->rank];
    for (const Slice &sl : mine.slices)
        if (sl.chunk_begin < h->groups[sl.group].chunk_begin || sl.chunk_end > h->groups[sl.group].chunk_end)
            return fail(h, NBO_ERR_STATE, "nabla-optim-b200: slice plan does not match the chunk list");

    int32_t rc = host_pipe_ensure(h, ns ? ns : 1);
    if (rc != NBO_OK) return rc;
    HostPipe *pipe = h->host_pipe;
    const bool checked = use_scaler || max_norm > 0.0;
    uint16_t *gflat = (uint16_t *)z->g_local;
    const uint16_t *pflat = (const uint16_t *)z->p_local;

    auto copy_in = [&](size_t s) -> int32_t {
        for (int q = 0; q < z->world; ++q) {
            if (s >= plans[q].slices.size()) continue;
            const Slice &sl = plans[q].slices[s];
            for (uint32_t k = sl.copy_begin; k < sl.copy_end; ++k) {
                const SliceCopy &c = plans[q].copies[k];
                const Piece &pc = rows[q][c.row];
                const char *src = (const char *)host_g[pc.tensor] + (pc.offset + c.lo) * 2;
                NBO_CUDA(h, cudaMemcpyAsync(gflat + pc.bucket_off + c.lo, src, (c.hi - c.lo) * 2, cudaMemcpyHostToDevice,
                                            pipe->in));
            }
        }
        NBO_CUDA(h, cudaEventRecord(pipe->copied[s], pipe->in));
        return NBO_OK;
    };
    auto copy_out = [&](size_t s) -> int32_t {
        if (s >= mine.slices.size()) return NBO_OK;
        const Slice &sl = mine.slices[s];
        for (uint32_t k = sl.copy_begin; k < sl.copy_end; ++k) {
            const SliceCopy &c = mine.copies[k];
            const Piece &pc = h->pieces[c.row];
            char *dst = (char *)host_p[pc.tensor] + (pc.offset + c.lo) * 2;
            NBO_CUDA(h, cudaMemcpyAsync(dst, pflat + pc.bucket_off + c.lo, (c.hi - c.lo) * 2, cudaMemcpyDeviceToHost,
                                        pipe->out));
        }
        return NBO_OK;
    };

    rc = [&]() -> int32_t {
        // work already on the compute stream (the previous step's closing barrier above all) comes first
        NBO_CUDA(h, cudaEventRecord(pipe->start, h->stream));
        NBO_CUDA(h, cudaStreamWaitEvent(pipe->in, pipe->start, 0));
        NBO_CUDA(h, cudaStreamWaitEvent(pipe->out, pipe->start, 0));
        if (checked) {
            for (size_t s = 0; s < ns; ++s) {
                int32_t r = copy_in(s);
                if (r != NBO_OK) return r;
            }
            if (ns) NBO_CUDA(h, cudaStreamWaitEvent(h->stream, pipe->copied[ns - 1], 0));
            return enqueue_fused_step(h, z, average, use_scaler, max_norm);
        }
        PeerArgs pa = z->pa;
        pa.average = average ? 1 : 0;
        pa.keep_reduced = z->keep_reduced ? 1 : 0;
        pa.barrier_seen = z->d_barrier + 1;
        std::vector<AdamHP> hp(h->groups.size());
        for (size_t g = 0; g < h->groups.size(); ++g) hp[g] = adam_hparams(h->groups[g].cfg, h->groups[g].step_count + 1, 1.0f);
        h->prof_norm_valid = false;
        for (size_t s = 0; s < ns; ++s) {
            int32_t r = copy_in(s);
            if (r != NBO_OK) return r;
            NBO_CUDA(h, cudaStreamWaitEvent(h->stream, pipe->copied[s], 0));
            r = enqueue_barrier(h, z, &pa.barrier_expect);
            if (r != NBO_OK) return r;
            if (s < mine.slices.size()) {
                const Slice &sl = mine.slices[s];
                r = launch_zero1_fused_update(h, sl.chunk_begin, sl.chunk_end - sl.chunk_begin, hp[sl.group], false, pa,
                                              z->transport, z->transport);
                if (r != NBO_OK) return r;
            }
            NBO_CUDA(h, cudaEventRecord(pipe->updated[s], h->stream));
            NBO_CUDA(h, cudaStreamWaitEvent(pipe->out, pipe->updated[s], 0));
            r = copy_out(s);
            if (r != NBO_OK) return r;
        }
        return enqueue_barrier(h, z, nullptr);  // nobody overwrites gradients a peer may still be reading
    }();
    if (rc != NBO_OK) {
        host_pipe_drain(h);  // an aborted communicator has already let its collectives return
        return rc;
    }
    rc = stream_wait(h, z, "the host-streamed sharded step");  // the one bounded host wait of the step
    if (rc != NBO_OK) return rc;
    if (checked && !h->h_ctrl->nonfinite) {  // copy-out of the shard; a skipped step leaves the host parameters alone
        for (size_t s = 0; s < mine.slices.size(); ++s) {
            rc = copy_out(s);
            if (rc != NBO_OK) { host_pipe_drain(h); return rc; }
        }
    }
    NBO_CUDA(h, cudaStreamSynchronize(pipe->in));
    NBO_CUDA(h, cudaStreamSynchronize(pipe->out));
    commit_step(h, checked, use_scaler != 0, result);
    return NBO_OK;
}

int32_t nbo_zero1_step_host(nbo_optimizer *h, void *params_flat_dev, void *grads_flat_dev, uint64_t n,
                            void *const *params_host, const void *const *grads_host, uint64_t slice_elems,
                            int32_t average, int32_t use_scaler, double max_norm, nbo_step_result *result)
{
    NBO_SYNC_STATE(h);
    if (!h || !h->zero1) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: not a ZeRO-1 handle");
    Zero1 *z = h->zero1;
    if (!params_flat_dev || !grads_flat_dev) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null bucket");
    if (n != h->ntensors || (n && (!params_host || !grads_host)))
        return fail(h, NBO_ERR_INVALID, "nabla-train: params/grads length mismatch: " + std::to_string(n) +
                                            " host tensors for " + std::to_string(h->ntensors));
    DeviceGuard guard(h->device);
    if (z->world > 1) {
        if (!z->attached)
            return fail(h, NBO_ERR_STATE, "nabla-optim-b200: with world > 1 the host-streamed step runs on the buckets "
                                          "given to nbo_zero1_attach_symmetric");
        if (params_flat_dev != z->p_local || grads_flat_dev != z->g_local)
            return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: the device buckets must be the attached symmetric buckets");
        if (z->broken)
            return fail(h, NBO_ERR_STATE, "nabla-optim-b200: the communicator was aborted; create a new handle");
        int32_t rc = bind_flat(h, z->p_local, z->g_local);
        if (rc != NBO_OK) return rc;
        return zero1_host_step_sharded(h, z, params_host, grads_host, slice_elems, average, use_scaler, max_norm, result);
    }
    int32_t rc = bind_flat(h, params_flat_dev, grads_flat_dev);
    if (rc != NBO_OK) return rc;
    return host_streamed_step(h, params_host, grads_host, slice_elems, use_scaler, max_norm, result);
}

int32_t nbo_zero1_attach_symmetric(nbo_optimizer *h, void *grads_local, void *const *grads_peers,
                                   void *grads_mc, void *params_local, void *const *params_peers,
                                   void *params_mc, int32_t transport)
{
    if (!h || !h->zero1) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: not a ZeRO-1 handle");
    Zero1 *z = h->zero1;
    if (z->world < 2)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: the fused path needs world >= 2; use nbo_zero1_step");
    if (z->world > kMaxPeers)
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: fused path supports at most 16 ranks");
    if (!grads_local || !params_local || !grads_peers || !params_peers)
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null bucket or peer list");
    // Measured on the 16 GB buckets: peer 25.4 ms / multicast 50.8 ms at 2 ranks, 37.1 / 39.5 at 4, 48.2 / 33.3 at 8.
    // Peer traffic is 2 (N-1)/N bucket sizes per direction at ~0.65 TB/s, multicast (1 + 1/N) at ~0.52-0.54 TB/s,
    // so multicast pays from 5 ranks on.
    if (transport == 0) transport = (grads_mc && params_mc && z->world >= 5) ? 2 : 1;
    if (transport != 1 && transport != 2) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: unknown transport");
    if (transport == 2 && (!grads_mc || !params_mc))
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: multicast transport needs both multicast mappings");
    uintptr_t all = (uintptr_t)grads_local | (uintptr_t)params_local | (uintptr_t)grads_mc | (uintptr_t)params_mc;
    for (int r = 0; r < z->world; ++r) {
        if (!grads_peers[r] || !params_peers[r])
            return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: null peer mapping for rank " + std::to_string(r));
        all |= (uintptr_t)grads_peers[r] | (uintptr_t)params_peers[r];
    }
    if (all & 15u) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: flat buckets must be 16-byte aligned");
    if (grads_peers[z->rank] != grads_local || params_peers[z->rank] != params_local)
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: peers[rank] must be this rank's own bucket");
    cudaError_t ce = cudaSetDevice(h->device);
    if (ce != cudaSuccess) return fail_cuda(h, ce, "cudaSetDevice");
    PeerArgs pa{};
    pa.world = z->world; pa.rank = z->rank; pa.average = 0; pa.inv_world = 1.0f / (float)z->world;
    pa.g_mc = grads_mc ? (int64_t)((intptr_t)grads_mc - (intptr_t)grads_local) : 0;
    pa.p_mc = params_mc ? (int64_t)((intptr_t)params_mc - (intptr_t)params_local) : 0;
    for (int r = 0; r < z->world; ++r) {
        pa.g_peer[r] = (int64_t)((intptr_t)grads_peers[r] - (intptr_t)grads_local);
        pa.p_peer[r] = (int64_t)((intptr_t)params_peers[r] - (intptr_t)params_local);
    }
    if (!z->d_barrier) {
        NBO_CUDA(h, cudaMalloc(&z->d_barrier, 2 * sizeof(int32_t)));
        NBO_CUDA(h, cudaMemset(z->d_barrier, 0, 2 * sizeof(int32_t)));
    }
    z->pa = pa; z->g_local = grads_local; z->p_local = params_local;
    z->transport = transport; z->attached = true;
    return NBO_OK;
}

int32_t nbo_zero1_step_fused(nbo_optimizer *h, int32_t average, int32_t use_scaler, double max_norm,
                             nbo_step_result *result)
{
    if (!h || !h->zero1) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: not a ZeRO-1 handle");
    Zero1 *z = h->zero1;
    if (!z->attached)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: nbo_zero1_step_fused before nbo_zero1_attach_symmetric");
    if (z->broken) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: the communicator was aborted; create a new handle");
    cudaError_t ce = cudaSetDevice(h->device);
    if (ce != cudaSuccess) return fail_cuda(h, ce, "cudaSetDevice");
    int32_t rc = h->dev_newer ? collect_dev_state(h) : NBO_OK;  // asynchronous steps came before: take their state over
    if (rc != NBO_OK) return rc;
    rc = bind_flat(h, z->p_local, z->g_local);
    if (rc != NBO_OK) return rc;
    // Everything is stream-ordered behind the opening barrier; the kernels that touch other ranks' memory
    // check on the device that the barrier really completed, so the host waits once, at the end.
    rc = enqueue_fused_step(h, z, average, use_scaler, max_norm);
    if (rc != NBO_OK) return rc;
    rc = stream_wait(h, z, "the fused sharded step");
    if (rc != NBO_OK) return rc;
    commit_step(h, use_scaler || max_norm > 0.0, use_scaler != 0, result);
    return NBO_OK;
}

int32_t nbo_zero1_step_fused_async(nbo_optimizer *h, int32_t average, int32_t use_scaler, double max_norm)
{
    if (!h || !h->zero1) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: not a ZeRO-1 handle");
    Zero1 *z = h->zero1;
    if (!z->attached)
        return fail(h, NBO_ERR_STATE, "nabla-optim-b200: nbo_zero1_step_fused_async before nbo_zero1_attach_symmetric");
    if (z->broken) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: the communicator was aborted; create a new handle");
    if (h->groups.size() > (size_t)kMaxDevGroups)
        return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: the asynchronous step supports at most 32 groups");
    cudaError_t ce = cudaSetDevice(h->device);
    if (ce != cudaSuccess) return fail_cuda(h, ce, "cudaSetDevice");
    int32_t rc = bind_flat(h, z->p_local, z->g_local);
    if (rc != NBO_OK) return rc;
    return enqueue_fused_step(h, z, average, use_scaler, max_norm, true);
}

int32_t nbo_zero1_keep_reduced_grads(nbo_optimizer *h, int32_t on)
{
    if (!h || !h->zero1) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: not a ZeRO-1 handle");
    h->zero1->keep_reduced = on != 0;
    return NBO_OK;
}

int32_t nbo_zero1_state_export(nbo_optimizer *h, int32_t which, float *dst)
{
    if (!h || !h->zero1) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: not a ZeRO-1 handle");
    float *base = which == 0 ? h->d_s0 : which == 1 ? h->d_s1 : which == 2 ? h->d_s2 : nullptr;
    if (!base || !dst) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: bad state selector or null buffer");
    cudaError_t ce = cudaSetDevice(h->device);
    if (ce != cudaSuccess) return fail_cuda(h, ce, "cudaSetDevice");
    NBO_CUDA(h, cudaMemcpyAsync(dst, base, h->zero1->shard * sizeof(float), cudaMemcpyDeviceToHost,
                                h->stream));
    NBO_CUDA(h, cudaStreamSynchronize(h->stream));
    return NBO_OK;
}

int32_t nbo_zero1_state_import(nbo_optimizer *h, int32_t which, const float *src)
{
    if (!h || !h->zero1) return fail(h, NBO_ERR_STATE, "nabla-optim-b200: not a ZeRO-1 handle");
    float *base = which == 0 ? h->d_s0 : which == 1 ? h->d_s1 : which == 2 ? h->d_s2 : nullptr;
    if (!base || !src) return fail(h, NBO_ERR_INVALID, "nabla-optim-b200: bad state selector or null buffer");
    cudaError_t ce = cudaSetDevice(h->device);
    if (ce != cudaSuccess) return fail_cuda(h, ce, "cudaSetDevice");
    NBO_CUDA(h, cudaMemcpyAsync(base, src, h->zero1->shard * sizeof(float), cudaMemcpyHostToDevice, h->stream));
    NBO_CUDA(h, cudaStreamSynchronize(h->stream));
    return NBO_OK;
}

}  // extern "C"
