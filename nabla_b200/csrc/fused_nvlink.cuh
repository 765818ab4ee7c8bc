// ZeRO-1 step fused with its collectives over NVLink / NVSwitch peer memory.
//
// Instead of reduce-scatter -> update -> all-gather as three passes with the
// buckets crossing HBM between them, one kernel per rank reads the gradients of
// its shard straight from every rank's bucket, updates its fp32 state, and
// writes the bf16 result straight into every rank's parameter bucket.  The
// buckets live in symmetric memory (every rank's allocation mapped into every
// process; optionally an NVSwitch multicast mapping on top).  Two transports:
//
//   kPeer   plain 64-bit peer loads (one per rank, summed in fp32 in rank
//           order, rounded once to bf16) and plain peer stores.  Per GPU and
//           direction this moves 2 x (N-1)/N x bucket bytes.  Measured faster up to
//           N = 4 (plain accesses run the links at ~0.65 TB/s, multimem at ~0.52).
//   kMcast  multimem.ld_reduce (the switch adds the N copies, fp32 accumulate)
//           and multimem.st (the switch replicates the store).  Per GPU and
//           direction: bucket x (1 + 1/N) bytes.  Fewer bytes from N = 4, faster
//           from N = 5 (measured at 8).
//
// Only plain loads/stores and multimem instructions touch remote memory; no
// tensor-map or bulk-copy engine is involved.  The kernels contain no cross-GPU waits of their own; the
// host orders them with stream-ordered NCCL barriers (see zero1.cu), so nothing
// here can spin.
//
// By default the reduced gradient is also written back into this rank's own
// slice of its gradient bucket (as an in-place reduce-scatter would leave it),
// so the value that was applied can be read back; PeerArgs::keep_reduced = 0
// drops that write for callers that overwrite the gradients anyway.
#pragma once
#include "kernels.cuh"

namespace nbo {

enum Transport { kLocal = 0, kPeer = 1, kMcast = 2 };

__device__ __forceinline__ uint2 mc_ld_reduce_bf16x4(const void *mc_addr)
{
    uint2 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v2.bf16x2 {%0, %1}, [%2];"
                 : "=r"(r.x), "=r"(r.y)
                 : "l"(mc_addr)
                 : "memory");
    return r;
}

__device__ __forceinline__ void mc_st_b64(void *mc_addr, uint2 v)
{
    asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};"
                 :
                 : "l"(mc_addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y))
                 : "memory");
}

__device__ __forceinline__ uint32_t scale_round_bf16(float sum, const PeerArgs &pa)
{
    if (pa.average) sum = __fmul_rn(sum, pa.inv_world);
    return f32_to_bf16(sum);
}

// One item (4 bf16) of this rank's shard, reduced over all ranks.
// Peer accesses carry no cache hint either: plain and .cs measured within 0.5 % at N = 2.
__device__ __forceinline__ uint2 ld_peer(const uint2 *p) { return *p; }
__device__ __forceinline__ void st_peer(uint2 *p, uint2 v) { *p = v; }

template <int kT>
__device__ __forceinline__ uint2 reduce_item(const uint2 *g_local, const PeerArgs &pa)
{
    if (kT == kMcast) {
        uint2 r = mc_ld_reduce_bf16x4((const char *)g_local + pa.g_mc);
        if (pa.average) {
            r.x = scale_round_bf16(bf16_to_f32(r.x & 0xffffu), pa) | (scale_round_bf16(bf16_to_f32(r.x >> 16), pa) << 16);
            r.y = scale_round_bf16(bf16_to_f32(r.y & 0xffffu), pa) | (scale_round_bf16(bf16_to_f32(r.y >> 16), pa) << 16);
        }
        return r;
    }
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    uint2 x[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
        if (r < pa.world) x[r] = ld_peer((const uint2 *)((const char *)g_local + pa.g_peer[r]));
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
        if (r < pa.world) {
            a0 = __fadd_rn(a0, bf16_to_f32(x[r].x & 0xffffu));
            a1 = __fadd_rn(a1, bf16_to_f32(x[r].x >> 16));
            a2 = __fadd_rn(a2, bf16_to_f32(x[r].y & 0xffffu));
            a3 = __fadd_rn(a3, bf16_to_f32(x[r].y >> 16));
        }
    uint2 o;
    o.x = scale_round_bf16(a0, pa) | (scale_round_bf16(a1, pa) << 16);
    o.y = scale_round_bf16(a2, pa) | (scale_round_bf16(a3, pa) << 16);
    return o;
}

// Peer transport with the remote loads of the first kPrefetchRanks ranks issued
// up front (together with the local state loads), so that enough bytes are in
// flight to cover the NVLink round trip; ranks beyond that are fetched when the
// item is reduced.
constexpr int kPrefetchRanks = 4;

struct PeerItem {
    uint2 x[kPrefetchRanks];
};

__device__ __forceinline__ void peer_prefetch(PeerItem &it, const uint2 *g_local, const PeerArgs &pa)
{
#pragma unroll
    for (int r = 0; r < kPrefetchRanks; ++r)
        if (r < pa.world) it.x[r] = ld_peer((const uint2 *)((const char *)g_local + pa.g_peer[r]));
}

__device__ __forceinline__ uint2 peer_reduce(const PeerItem &it, const uint2 *g_local, const PeerArgs &pa)
{
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int r = 0; r < kPrefetchRanks; ++r)
        if (r < pa.world) {
            a0 = __fadd_rn(a0, bf16_to_f32(it.x[r].x & 0xffffu));
            a1 = __fadd_rn(a1, bf16_to_f32(it.x[r].x >> 16));
            a2 = __fadd_rn(a2, bf16_to_f32(it.x[r].y & 0xffffu));
            a3 = __fadd_rn(a3, bf16_to_f32(it.x[r].y >> 16));
        }
    for (int r = kPrefetchRanks; r < pa.world; ++r) {
        uint2 x = ld_peer((const uint2 *)((const char *)g_local + pa.g_peer[r]));
        a0 = __fadd_rn(a0, bf16_to_f32(x.x & 0xffffu));
        a1 = __fadd_rn(a1, bf16_to_f32(x.x >> 16));
        a2 = __fadd_rn(a2, bf16_to_f32(x.y & 0xffffu));
        a3 = __fadd_rn(a3, bf16_to_f32(x.y >> 16));
    }
    uint2 o;
    o.x = scale_round_bf16(a0, pa) | (scale_round_bf16(a1, pa) << 16);
    o.y = scale_round_bf16(a2, pa) | (scale_round_bf16(a3, pa) << 16);
    return o;
}

// One stray element (head / tail of a piece): always plain peer loads, rank order.
__device__ __forceinline__ uint16_t reduce_elem(const uint16_t *g_local, const PeerArgs &pa)
{
    float a = 0.f;
    for (int r = 0; r < pa.world; ++r)
        a = __fadd_rn(a, bf16_to_f32(*(const volatile uint16_t *)((const char *)g_local + pa.g_peer[r])));
    return (uint16_t)scale_round_bf16(a, pa);
}

template <int kT>
__device__ __forceinline__ void publish_item(uint2 *p_local, uint2 v, const PeerArgs &pa)
{
    if (kT == kMcast) {
        mc_st_b64((char *)p_local + pa.p_mc, v);
    } else {
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (r < pa.world) st_peer((uint2 *)((char *)p_local + pa.p_peer[r]), v);
    }
}

__device__ __forceinline__ void publish_elem(uint16_t *p_local, uint16_t v, const PeerArgs &pa)
{
    for (int r = 0; r < pa.world; ++r) *(uint16_t *)((char *)p_local + pa.p_peer[r]) = v;
}

// The cross-rank barrier that precedes a peer-touching kernel is an NCCL all-reduce (max) of a sequence
// number on the same stream.  If a rank has gone away the host's bounded wait aborts the communicator, the
// collective ends without delivering the number, and the kernels queued behind it find a stale value here and
// return without touching any other rank's memory.
__device__ __forceinline__ bool barrier_passed(const PeerArgs &pa)
{
    return pa.barrier_seen == nullptr || *(const volatile int32_t *)pa.barrier_seen == pa.barrier_expect;
}

struct ChunkLoc {
    TensorDesc d;
    ChunkView cv;
};
__device__ __forceinline__ ChunkLoc locate_chunk(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks,
                                                 uint32_t c)
{
    ChunkLoc l;
    const Chunk ck = chunks[c];
    l.d = descs[ck.tensor];
    l.cv = chunk_view(l.d, ck);
    return l;
}

// Fused reduce-scatter + Adam/AdamW + all-gather over this rank's shard.
//   kIn  : where the gradient comes from - kLocal (already reduced into the local slice by an earlier
//          pass), kPeer (plain 64-bit loads from every rank, issued together with the chunk's state loads)
//          or kMcast (multimem.ld_reduce, issued with the chunk's state loads).
//   kOut : how the bf16 params reach the other ranks - kPeer or kMcast.
// Staging the other ranks' gradients several chunks ahead through a shared-memory ring (cp.async, 8 bytes
// per thread and item, 3 to 5 chunks in flight per CTA) was built and measured at world 2 on the 8 G-element
// bucket: 33.1 ms per step against 25.5 ms for the plain loads below - asynchronous copies from peer memory
// through shared memory move fewer bytes per second than register loads, so the ring was dropped.
// Handing the parameter broadcast to the copy engines (the kernel writing its own bucket only, slice by
// slice, DMA copies pushing each finished slice to the peers) was measured as well: a copy-engine push alone
// reaches 770 GB/s per direction against 666 for SM loads and 705 for SM stores, but SM loads and a DMA push
// running together share 677 GB/s per direction, and the step took 30.0 ms against 25.4 ms - also dropped.
// For the multicast transport two more variants were measured on 8 GPUs (18 GB per direction): the next
// chunk's multimem.ld_reduce issued one chunk ahead into registers, 34.4 ms, and 16-byte multimem operations
// shared by lane pairs (halves exchanged by shuffle), 34.4 ms, against 33.3 ms for the form below; at 2 GPUs
// they made no difference either (50.9 / 51.7 / 49.6 ms).  Both were removed.  The same one-chunk-ahead request
// for the single remote rank of the peer transport at 2 GPUs: 27.3 ms against 26.0 ms in the same run - removed.
// Splitting the step into a reduce launch (into the local slice) and a <kLocal, kOut> update launch per slice
// of the shard on two streams, so that inbound and outbound traffic overlap across kernels, was slower too:
// 31.5 against 25.3 ms (peer, 2 GPUs) and 40.6 against 39.5 ms (multicast, 4 GPUs) at the best CTA split.
// In short: with the loads of four items per thread outstanding the links are as busy as this access pattern
// can make them; putting more remote requests in flight only delays the stores that share the direction.
template <int kIn, int kOut>
__global__ void __launch_bounds__(kBlock)
zero1_fused_update_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks,
                          uint32_t nchunks, AdamHP hp, const StepCtrl *__restrict__ ctrl, PeerArgs pa)
{
    if (!barrier_passed(pa))
        return;
    if (pa.hp_dev != nullptr) hp = *pa.hp_dev;
    float clip = 1.0f;
    if (ctrl != nullptr) {
        if (ctrl->skip)
            return;
        clip = ctrl->clip_scale;
    }
    const uint32_t mine = nchunks > blockIdx.x ? (nchunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    for (uint32_t it = 0; it < mine; ++it) {
        const ChunkLoc l = locate_chunk(descs, chunks, blockIdx.x + it * gridDim.x);
        const TensorDesc &d = l.d;
        const ChunkView &cv = l.cv;
        uint16_t *P = (uint16_t *)d.p;
        uint16_t *G = (uint16_t *)d.g;
        uint2 *p2 = (uint2 *)(P + cv.item0);
        uint2 *g2 = (uint2 *)(G + cv.item0);
        float4 *m4 = (float4 *)(d.s0 + cv.item0);
        float4 *v4 = (float4 *)(d.s1 + cv.item0);
        float4 *w4 = (float4 *)(d.s2 + cv.item0);

        uint2 g[kItemsPerThread];
        PeerItem pg[kIn == kPeer ? kItemsPerThread : 1];
        float4 w[kItemsPerThread], m[kItemsPerThread], v[kItemsPerThread];
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (i < cv.nitems) {
                if (kIn == kPeer) peer_prefetch(pg[kIn == kPeer ? u : 0], g2 + i, pa);
                if (kIn == kMcast) g[u] = reduce_item<kMcast>(g2 + i, pa);
                if (kIn == kLocal) g[u] = ld_stream(g2 + i);
                w[u] = ld_stream(w4 + i);
                m[u] = ld_stream(m4 + i);
                v[u] = ld_stream(v4 + i);
            }
        }
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (i < cv.nitems) {
                if (kIn == kPeer) g[u] = peer_reduce(pg[kIn == kPeer ? u : 0], g2 + i, pa);
                if (kIn != kLocal && pa.keep_reduced) st_stream(g2 + i, g[u]);
                mixed_elem<true>(bf16_to_f32(g[u].x & 0xffffu), w[u].x, m[u].x, v[u].x, hp, clip);
                mixed_elem<true>(bf16_to_f32(g[u].x >> 16), w[u].y, m[u].y, v[u].y, hp, clip);
                mixed_elem<true>(bf16_to_f32(g[u].y & 0xffffu), w[u].z, m[u].z, v[u].z, hp, clip);
                mixed_elem<true>(bf16_to_f32(g[u].y >> 16), w[u].w, m[u].w, v[u].w, hp, clip);
                uint2 o;
                o.x = pack_bf16x2(w[u].x, w[u].y);
                o.y = pack_bf16x2(w[u].z, w[u].w);
                st_stream(w4 + i, w[u]);
                st_stream(m4 + i, m[u]);
                st_stream(v4 + i, v[u]);
                publish_item<kOut>(p2 + i, o, pa);
            }
        }
        for (int r = 0; r < 2; ++r) {
            uint64_t b = r ? cv.s_hi0 : cv.s_lo0, e = r ? cv.s_hi1 : cv.s_lo1;
            for (uint64_t i = b + threadIdx.x; i < e; i += kBlock) {
                uint16_t gi = kIn == kLocal ? G[i] : reduce_elem(G + i, pa);
                if (kIn != kLocal && pa.keep_reduced) G[i] = gi;
                mixed_elem<true>(bf16_to_f32(gi), d.s2[i], d.s0[i], d.s1[i], hp, clip);
                publish_elem(P + i, (uint16_t)f32_to_bf16(d.s2[i]), pa);
            }
        }
    }
}

// Reduce-scatter fused with the norm / non-finite pass: the reduced gradient of
// this rank's shard is written into the local slice and its sum of squares and
// non-finite flag are produced in the same sweep (same two-stage reduction as
// norm_kernel).  Used when clipping or loss scaling needs the global norm before
// any element may be updated.
template <int kIn>
__global__ void __launch_bounds__(kBlock)
zero1_reduce_norm_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks,
                         uint32_t nchunks, float inv_scale, NormOut out, PeerArgs pa)
{
    double acc = 0.0;
    int bad = 0;
    if (pa.inv_scale_dev != nullptr) inv_scale = *pa.inv_scale_dev;
    const bool go = barrier_passed(pa);  // a failed barrier leaves every rank's memory alone; the partials still add up
    for (uint32_t c = blockIdx.x; go && c < nchunks; c += gridDim.x) {
        const Chunk ck = chunks[c];
        const TensorDesc d = descs[ck.tensor];
        const ChunkView cv = chunk_view(d, ck);
        uint16_t *G = (uint16_t *)d.g;
        uint2 *g2 = (uint2 *)(G + cv.item0);
        PeerItem pg[kIn == kPeer ? kItemsPerThread : 1];
        uint2 gm[kItemsPerThread];
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (i < cv.nitems) {
                if (kIn == kPeer) peer_prefetch(pg[kIn == kPeer ? u : 0], g2 + i, pa);
                else gm[u] = reduce_item<kMcast>(g2 + i, pa);
            }
        }
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (i < cv.nitems) {
                uint2 g = kIn == kPeer ? peer_reduce(pg[kIn == kPeer ? u : 0], g2 + i, pa) : gm[u];
                st_stream(g2 + i, g);
                sq_acc(bf16_to_f32(g.x & 0xffffu), inv_scale, acc, bad);
                sq_acc(bf16_to_f32(g.x >> 16), inv_scale, acc, bad);
                sq_acc(bf16_to_f32(g.y & 0xffffu), inv_scale, acc, bad);
                sq_acc(bf16_to_f32(g.y >> 16), inv_scale, acc, bad);
            }
        }
        for (int r = 0; r < 2; ++r) {
            uint64_t b = r ? cv.s_hi0 : cv.s_lo0, e = r ? cv.s_hi1 : cv.s_lo1;
            for (uint64_t i = b + threadIdx.x; i < e; i += kBlock) {
                uint16_t gi = reduce_elem(G + i, pa);
                G[i] = gi;
                sq_acc(bf16_to_f32(gi), inv_scale, acc, bad);
            }
        }
    }
    double bsum = block_sum_f64(acc, bad);
    __shared__ bool s_last;
    if (threadIdx.x == 0) {
        out.partial_sum[blockIdx.x] = bsum;
        out.partial_bad[blockIdx.x] = bad;
        __threadfence();
        uint32_t t = atomicInc(out.ticket, gridDim.x - 1);
        s_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last)
        return;
    __threadfence();
    double tot = 0.0;
    int anybad = 0;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += kBlock) {
        tot += __ldcg(out.partial_sum + i);
        anybad |= __ldcg(out.partial_bad + i);
    }
    tot = block_sum_f64(tot, anybad);
    if (threadIdx.x == 0) {
        out.local[0] = tot;
        out.local[1] = anybad ? 1.0 : 0.0;
    }
}

}  // namespace nbo
