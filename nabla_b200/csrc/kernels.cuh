// Device code of libnabla_optim_b200: the multi-tensor-apply (MTA) kernels.
//
// Everything here is HBM-bound streaming work for sm_100a: each element is read
// once and written once per pass, with 128-bit (fp32) / 64-bit (bf16) coalesced
// accesses, a persistent grid sized from the SM count, and no shared-memory
// staging (there is no reuse to stage for).  Tensor cores are not involved.
//
// Arithmetic contract: every fp32 statement is ONE correctly-rounded IEEE
// operation (__fmul_rn / __fadd_rn / __fdiv_rn / __fsqrt_rn) in the order the
// nabla CPU backend applies them (nabla-train/src/optim/alg.rs:136-149 with
// nabla-core/src/cpu/mod.rs:211-223: scale is x*s, axpy is y + (a*x) with the
// product rounded first).  The intrinsics also stop the compiler from
// contracting a multiply and an add into an FMA.  The only deviation is
// powf(x, 0.5f) -> __fsqrt_rn(x): the host libm's powf is not correctly
// rounded, sqrt is, so the two can differ by 1 ulp on a small fraction of
// inputs.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "types.h"

namespace nbo {

// ---- helpers ----------------------------------------------------------------

// Plain (default cache operator) 128-bit / 64-bit accesses.  Measured on B200 against the
// streaming (.cs), .cg and .lu/.wt operators on every array role (state that is read and
// rewritten, gradients read once, bf16 parameters written once): the default operator was the
// fastest or tied in every combination, 2-7 % faster than .cs on both for the update kernels
// (35.3 vs 37.9 ms on 8 G parameters), so no eviction hint is given anywhere.
__device__ __forceinline__ float4 ld_stream(const float4 *p) { return *p; }
__device__ __forceinline__ void st_stream(float4 *p, float4 v) { *p = v; }
__device__ __forceinline__ uint2 ld_stream(const uint2 *p) { return *p; }
__device__ __forceinline__ void st_stream(uint2 *p, uint2 v) { *p = v; }

// bf16 -> f32 is a 16-bit shift (half 2.7.1 bf16::to_f32).
__device__ __forceinline__ float bf16_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

// f32 -> bf16, round-to-nearest-even on the upper half, NaNs quieted with their
// upper payload kept (half 2.7.1 bf16::from_f32; used by Scalar::from_f64 for
// bf16, nabla-core/src/common/scalar/mod.rs:338-340).
__device__ __forceinline__ uint32_t f32_to_bf16(float f)
{
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u)
        return (u >> 16) | 0x0040u;
    uint32_t up = ((u & 0x00008000u) != 0u) && ((u & 0x00017fffu) != 0u);
    return (u >> 16) + up;
}

__device__ __forceinline__ bool is_nonfinite(float f)
{
    return (__float_as_uint(f) & 0x7f800000u) == 0x7f800000u;
}

// One element of Adam (decoupled = 0) or AdamW (decoupled = 1);
// alg.rs:138-148 / 283-290.
__device__ __forceinline__ void adam_elem(float &p, float g, float &m, float &v, const AdamHP &h)
{
    float mm = __fmul_rn(m, h.b1);
    mm = __fadd_rn(mm, __fmul_rn(h.one_minus_b1, g));
    float vv = __fmul_rn(v, h.b2);
    float gs = __fmul_rn(g, g);
    vv = __fadd_rn(vv, __fmul_rn(h.one_minus_b2, gs));
    // Correctly rounded sqrt and divide branch to a slow routine when an operand is zero; a parameter
    // that never received a gradient has g = m = v = 0 on every step, and whole rows of them (unused
    // embedding entries) would run the update a quarter slower.  Both zero cases have exact, trivial
    // answers (sqrt(+0) = +0; 0 / d = 0 for d > 0, sign kept), so they are answered by a select and the
    // routines only ever see non-zero operands.
    float t = __fmul_rn(vv, h.inv_bc2);
    bool tz = t == 0.0f;
    float rt = __fsqrt_rn(tz ? 1.0f : t);
    float den = __fadd_rn(tz ? t : rt, h.eps);
    float a = __fmul_rn(mm, h.ss);
    bool az = a == 0.0f && den > 0.0f;
    float q = __fdiv_rn(az ? den : a, den);
    float u = az ? a : q;
    float pp = p;
    if (h.decoupled)
        pp = __fmul_rn(pp, h.decay);
    pp = __fsub_rn(pp, u);  // p + (-1 * u): the product is an exact negation, so one subtraction rounds the same
    p = pp;
    m = mm;
    v = vv;
}

// One element of Sgd::step (alg.rs:399-413).
__device__ __forceinline__ void sgd_elem(float &p, float g, float &vel, const SgdHP &h)
{
    float ge = g;
    if (h.use_wd)
        ge = __fadd_rn(g, __fmul_rn(p, h.wd));
    if (h.use_mu) {
        vel = __fadd_rn(__fmul_rn(vel, h.mu), ge);
        ge = vel;
    }
    p = __fadd_rn(p, __fmul_rn(h.nlr, ge));
}

// Geometry of one chunk of one tensor.
struct ChunkView {
    uint64_t item0;   // first element of the aligned body this chunk covers
    uint32_t nitems;  // 4-element items in this chunk
    uint64_t s_lo0, s_lo1;  // scalar range A: [s_lo0, s_lo1)  (head, first chunk only)
    uint64_t s_hi0, s_hi1;  // scalar range B: [s_hi0, s_hi1)  (tail, last chunk only)
};

__device__ __forceinline__ ChunkView chunk_view(const TensorDesc &d, uint32_t cidx)
{
    ChunkView c;
    if (d.head == 0xffffffffu) {  // unaligned tensor: plain element loop over the chunk
        uint64_t b = (uint64_t)cidx * kChunkElems;
        uint64_t e = b + kChunkElems < d.n ? b + kChunkElems : d.n;
        c.item0 = 0; c.nitems = 0;
        c.s_lo0 = b; c.s_lo1 = e; c.s_hi0 = c.s_hi1 = 0;
        return c;
    }
    uint64_t head = d.head < d.n ? d.head : d.n;
    uint64_t body_items = (d.n - head) >> 2;
    uint64_t i0 = (uint64_t)cidx * kChunkItems;
    uint64_t i1 = i0 + kChunkItems < body_items ? i0 + kChunkItems : body_items;
    if (i0 > body_items) i0 = body_items;
    c.item0 = head + (i0 << 2);
    c.nitems = (uint32_t)(i1 > i0 ? i1 - i0 : 0);
    c.s_lo0 = 0; c.s_lo1 = cidx == 0 ? head : 0;
    // the tensor owns ceil(n / kChunkElems) chunks whatever its alignment; the final one takes the tail
    bool last = ((uint64_t)cidx + 1) * kChunkElems >= d.n;
    c.s_hi0 = head + (body_items << 2);
    c.s_hi1 = last ? d.n : c.s_hi0;
    return c;
}

// The same geometry from the chunk entry: the host has already counted the
// items of every chunk, so the common case (aligned row, no stray elements)
// costs one multiply-add instead of the 64-bit min/compare chain above.
__device__ __forceinline__ ChunkView chunk_view(const TensorDesc &d, const Chunk &ck)
{
    if (!ck.stray && d.head != 0xffffffffu) {
        ChunkView c;
        c.item0 = d.head + (uint64_t)ck.index * kChunkElems;
        c.nitems = ck.nitems;
        c.s_lo0 = c.s_lo1 = c.s_hi0 = c.s_hi1 = 0;
        return c;
    }
    return chunk_view(d, ck.index);
}

// ---- fp32 Adam / AdamW --------------------------------------------------------

// One chunk of fp32 Adam / AdamW: 16 independent 128-bit loads per thread go out before the first result
// is needed.  Shared by the table-driven kernel and the single-tensor one below.
__device__ __forceinline__ void adam_f32_chunk(const TensorDesc &d, const ChunkView &cv, const AdamHP &hp)
{
    float *P = (float *)d.p;
    const float *G = (const float *)d.g;
    float4 *p4 = (float4 *)(P + cv.item0);
    const float4 *g4 = (const float4 *)(G + cv.item0);
    float4 *m4 = (float4 *)(d.s0 + cv.item0);
    float4 *v4 = (float4 *)(d.s1 + cv.item0);

    float4 p[kItemsPerThread], g[kItemsPerThread], m[kItemsPerThread], v[kItemsPerThread];
#pragma unroll
    for (int u = 0; u < kItemsPerThread; ++u) {
        uint32_t i = threadIdx.x + u * kBlock;
        if (i < cv.nitems) {
            g[u] = ld_stream(g4 + i);
            p[u] = ld_stream(p4 + i);
            m[u] = ld_stream(m4 + i);
            v[u] = ld_stream(v4 + i);
        }
    }
#pragma unroll
    for (int u = 0; u < kItemsPerThread; ++u) {
        uint32_t i = threadIdx.x + u * kBlock;
        if (i < cv.nitems) {
            adam_elem(p[u].x, g[u].x, m[u].x, v[u].x, hp);
            adam_elem(p[u].y, g[u].y, m[u].y, v[u].y, hp);
            adam_elem(p[u].z, g[u].z, m[u].z, v[u].z, hp);
            adam_elem(p[u].w, g[u].w, m[u].w, v[u].w, hp);
            st_stream(p4 + i, p[u]);
            st_stream(m4 + i, m[u]);
            st_stream(v4 + i, v[u]);
        }
    }
    // head / tail / unaligned elements
    for (uint64_t i = cv.s_lo0 + threadIdx.x; i < cv.s_lo1; i += kBlock)
        adam_elem(P[i], G[i], d.s0[i], d.s1[i], hp);
    for (uint64_t i = cv.s_hi0 + threadIdx.x; i < cv.s_hi1; i += kBlock)
        adam_elem(P[i], G[i], d.s0[i], d.s1[i], hp);
}

__global__ void __launch_bounds__(kBlock)
adam_f32_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks,
                uint32_t nchunks, AdamHP hp)
{
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const Chunk ck = chunks[c];
        const TensorDesc d = descs[ck.tensor];
        adam_f32_chunk(d, chunk_view(d, ck), hp);
    }
}

// adamw_step (alg.rs:431-469): one tensor whose m and v belong to the caller.  The table row travels as a
// kernel argument and the chunks are counted off arithmetically, so no handle and no device table exist.
__global__ void __launch_bounds__(kBlock)
adam_f32_single_kernel(TensorDesc d, uint32_t nchunks, AdamHP hp)
{
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x)
        adam_f32_chunk(d, chunk_view(d, c), hp);
}

// ---- fp32 SGD (plain, weight decay, momentum) --------------------------------

template <bool kMomentum>
__global__ void __launch_bounds__(kBlock)
sgd_f32_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks,
               uint32_t nchunks, SgdHP hp)
{
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const Chunk ck = chunks[c];
        const TensorDesc d = descs[ck.tensor];
        const ChunkView cv = chunk_view(d, ck);
        float *P = (float *)d.p;
        const float *G = (const float *)d.g;
        float4 *p4 = (float4 *)(P + cv.item0);
        const float4 *g4 = (const float4 *)(G + cv.item0);
        float4 *s4 = (float4 *)(d.s0 + cv.item0);

        float4 p[kItemsPerThread], g[kItemsPerThread], s[kItemsPerThread];
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (i < cv.nitems) {
                g[u] = ld_stream(g4 + i);
                p[u] = ld_stream(p4 + i);
                if (kMomentum) s[u] = ld_stream(s4 + i);
                else s[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (i < cv.nitems) {
                sgd_elem(p[u].x, g[u].x, s[u].x, hp);
                sgd_elem(p[u].y, g[u].y, s[u].y, hp);
                sgd_elem(p[u].z, g[u].z, s[u].z, hp);
                sgd_elem(p[u].w, g[u].w, s[u].w, hp);
                st_stream(p4 + i, p[u]);
                if (kMomentum) st_stream(s4 + i, s[u]);
            }
        }
        for (int r = 0; r < 2; ++r) {
            uint64_t b = r ? cv.s_hi0 : cv.s_lo0, e = r ? cv.s_hi1 : cv.s_lo1;
            for (uint64_t i = b + threadIdx.x; i < e; i += kBlock) {
                float vel = kMomentum ? d.s0[i] : 0.f;
                sgd_elem(P[i], G[i], vel, hp);
                if (kMomentum) d.s0[i] = vel;
            }
        }
    }
}

// ---- mixed-precision Adam / AdamW ---------------------------------------------
// Per element: g = bf16->f32 (exact); g *= inv_scale (GradScaler unscale,
// core.rs:373-375); g *= clip_scale (clip_grad_norm, trainer.rs:516-520);
// Adam/AdamW on the fp32 master; bf16 param = RNE(master).  Reads 14 B, writes
// 14 B per element.  Returns at once when the norm pass flagged the step as
// skipped.

template <bool kScaled>
__device__ __forceinline__ void mixed_elem(float g, float &w, float &m, float &v, const AdamHP &hp,
                                           float clip)
{
    if (kScaled) {  // x * 1.0f is exact, so the unscaled / unclipped step skips both multiplies
        g = __fmul_rn(g, hp.inv_scale);
        g = __fmul_rn(g, clip);
    }
    adam_elem(w, g, m, v, hp);
}

// Two fp32 -> one bf16x2 word.  The hardware convert is round-to-nearest-even for every non-NaN input
// (infinities, subnormals and the round-up-to-infinity case included) but canonicalises NaNs, so NaNs take
// the integer path that keeps their sign and upper payload as the reference's cast does.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    if (lo != lo || hi != hi) d = f32_to_bf16(lo) | (f32_to_bf16(hi) << 16);
    return d;
}

// kGradF32: the gradients are fp32 (accumulated over micro-batches in fp32) instead of bf16; everything
// else - unscale, clip, Adam on the master, bf16 write-back - is the same.  30 instead of 28 B per element.
template <bool kFull, bool kScaled, bool kGradF32>
__device__ __forceinline__ void mixed_items(uint2 *p2, const void *gbase, float4 *w4, float4 *m4, float4 *v4,
                                            uint32_t nitems, const AdamHP &hp, float clip)
{
    const uint2 *g2 = (const uint2 *)gbase;
    const float4 *g4 = (const float4 *)gbase;
    uint2 g[kGradF32 ? 1 : kItemsPerThread];
    float4 gf[kGradF32 ? kItemsPerThread : 1];
    float4 w[kItemsPerThread], m[kItemsPerThread], v[kItemsPerThread];
#pragma unroll
    for (int u = 0; u < kItemsPerThread; ++u) {
        uint32_t i = threadIdx.x + u * kBlock;
        if (kFull || i < nitems) {
            if (kGradF32) gf[kGradF32 ? u : 0] = ld_stream(g4 + i);
            else g[kGradF32 ? 0 : u] = ld_stream(g2 + i);
            w[u] = ld_stream(w4 + i);
            m[u] = ld_stream(m4 + i);
            v[u] = ld_stream(v4 + i);
        }
    }
#pragma unroll
    for (int u = 0; u < kItemsPerThread; ++u) {
        uint32_t i = threadIdx.x + u * kBlock;
        if (kFull || i < nitems) {
            float g0, g1, g2v, g3;
            if (kGradF32) {
                const float4 t = gf[kGradF32 ? u : 0];
                g0 = t.x; g1 = t.y; g2v = t.z; g3 = t.w;
            } else {
                const uint2 t = g[kGradF32 ? 0 : u];
                g0 = __uint_as_float(t.x << 16); g1 = __uint_as_float(t.x & 0xffff0000u);
                g2v = __uint_as_float(t.y << 16); g3 = __uint_as_float(t.y & 0xffff0000u);
            }
            mixed_elem<kScaled>(g0, w[u].x, m[u].x, v[u].x, hp, clip);
            mixed_elem<kScaled>(g1, w[u].y, m[u].y, v[u].y, hp, clip);
            mixed_elem<kScaled>(g2v, w[u].z, m[u].z, v[u].z, hp, clip);
            mixed_elem<kScaled>(g3, w[u].w, m[u].w, v[u].w, hp, clip);
            uint2 o;
            o.x = pack_bf16x2(w[u].x, w[u].y);
            o.y = pack_bf16x2(w[u].z, w[u].w);
            st_stream(w4 + i, w[u]);
            st_stream(m4 + i, m[u]);
            st_stream(v4 + i, v[u]);
            st_stream(p2 + i, o);
        }
    }
}

// kScaled = false is the plain step (no loss scale, no clipping, no decision record).
// 2 resident CTAs per SM (register-limited).  Forcing 3 (80 registers) was measured slower on the 8 G-element
// case (40.8 vs 36.2 ms): more loads in flight than the memory system absorbs; a tighter register budget at
// the same 2 CTAs made no difference.
template <bool kScaled, bool kGradF32>
__global__ void __launch_bounds__(kBlock)
adam_mixed_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks,
                  uint32_t nchunks, AdamHP hp, const StepCtrl *__restrict__ ctrl,
                  const AdamHP *__restrict__ hp_dev)
{
    if (hp_dev != nullptr) hp = *hp_dev;  // asynchronous step: prepare_kernel wrote this group's scalars
    float clip = 1.0f;
    if (kScaled && ctrl != nullptr) {
        if (ctrl->skip)
            return;
        clip = ctrl->clip_scale;
    }
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const Chunk ck = chunks[c];
        const TensorDesc d = descs[ck.tensor];
        const ChunkView cv = chunk_view(d, ck);
        uint16_t *P = (uint16_t *)d.p;
        uint2 *p2 = (uint2 *)(P + cv.item0);
        const void *gbase = kGradF32 ? (const void *)((const float *)d.g + cv.item0)
                                     : (const void *)((const uint16_t *)d.g + cv.item0);
        float4 *m4 = (float4 *)(d.s0 + cv.item0);
        float4 *v4 = (float4 *)(d.s1 + cv.item0);
        float4 *w4 = (float4 *)(d.s2 + cv.item0);
        mixed_items<false, kScaled, kGradF32>(p2, gbase, w4, m4, v4, cv.nitems, hp, clip);
        for (int r = 0; r < 2; ++r) {
            uint64_t b = r ? cv.s_hi0 : cv.s_lo0, e = r ? cv.s_hi1 : cv.s_lo1;
            for (uint64_t i = b + threadIdx.x; i < e; i += kBlock) {
                float gi = kGradF32 ? ((const float *)d.g)[i] : bf16_to_f32(((const uint16_t *)d.g)[i]);
                mixed_elem<kScaled>(gi, d.s2[i], d.s0[i], d.s1[i], hp, clip);
                P[i] = (uint16_t)f32_to_bf16(d.s2[i]);
            }
        }
    }
}

// fp32 master <- exact widening of the bf16 params.
__global__ void __launch_bounds__(kBlock)
init_master_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks,
                   uint32_t nchunks)
{
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const Chunk ck = chunks[c];
        const TensorDesc d = descs[ck.tensor];
        const uint16_t *P = (const uint16_t *)d.p;
        uint64_t b = (uint64_t)ck.index * kChunkElems;
        uint64_t e = b + kChunkElems < d.n ? b + kChunkElems : d.n;
        for (uint64_t i = b + threadIdx.x; i < e; i += kBlock)
            d.s2[i] = bf16_to_f32(P[i]);
    }
}

// ---- global L2 norm + non-finite flag -------------------------------------------
// Pass 1 (all CTAs): every thread accumulates (g*inv_scale)^2 in f64 - the
// square of an f32 is exact in f64, so this is the reference's `sum += v*v`
// (trainer.rs:505-513) up to summation order - and ORs a non-finite flag taken
// on the still-scaled value (core.rs:356-366).  Warp shuffles, then one shared
// memory step, give one partial per CTA.
// Pass 2 (the last CTA to finish, found with a self-resetting atomicInc
// ticket): adds the partials in index order with a fixed tree, so the result
// does not depend on CTA scheduling, and writes the StepCtrl record.

__device__ __forceinline__ double shfl_down_f64(double x, int off)
{
    int lo = __double2loint(x), hi = __double2hiint(x);
    lo = __shfl_down_sync(0xffffffffu, lo, off);
    hi = __shfl_down_sync(0xffffffffu, hi, off);
    return __hiloint2double(hi, lo);
}

// Sum over the block in a fixed order; valid in thread 0.
__device__ __forceinline__ double block_sum_f64(double x, int &flag)
{
    __shared__ double s_sum[kBlock / 32];
    __shared__ int s_flag[kBlock / 32];
    for (int off = 16; off > 0; off >>= 1) {
        x += shfl_down_f64(x, off);
        flag |= __shfl_down_sync(0xffffffffu, flag, off);
    }
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();  // protect s_* against a previous use
    if (l == 0) { s_sum[w] = x; s_flag[w] = flag; }
    __syncthreads();
    if (w == 0) {
        x = l < kBlock / 32 ? s_sum[l] : 0.0;
        flag = l < kBlock / 32 ? s_flag[l] : 0;
        for (int off = 4; off > 0; off >>= 1) {
            x += shfl_down_f64(x, off);
            flag |= __shfl_down_sync(0xffffffffu, flag, off);
        }
    }
    return x;
}

__device__ __forceinline__ void sq_acc(float g, float inv_scale, double &acc, int &bad)
{
    bad |= is_nonfinite(g) ? 1 : 0;
    double x = (double)__fmul_rn(g, inv_scale);
    acc = fma(x, x, acc);  // x*x is exact in f64, so this equals mul-then-add
}

struct NormOut {
    double *partial_sum;   // [gridDim.x]
    int32_t *partial_bad;  // [gridDim.x]
    uint32_t *ticket;      // zero before the first launch; wraps back to zero by itself
    double *local;         // [2]: {sumsq, nonfinite} of this launch (for the cross-rank exchange)
    StepCtrl *ctrl;        // written when finalize != 0
};

__device__ __forceinline__ void write_ctrl(StepCtrl *ctrl, double sum, int bad, double max_norm)
{
    double norm = sqrt(sum);
    StepCtrl c;
    c.sumsq = sum;
    c.norm = norm;
    c.do_clip = (max_norm > 0.0 && norm > max_norm && norm > 0.0) ? 1 : 0;
    c.clip_scale = c.do_clip ? (float)(max_norm / norm) : 1.0f;
    c.nonfinite = bad;
    c.skip = bad;
    *ctrl = c;
}

// Second half of the norm pass: one partial per CTA, then the last CTA to arrive (self-resetting ticket) adds
// the partials in index order and writes the outputs.
__device__ __forceinline__ void norm_finish(double acc, int bad, const NormOut &out, double max_norm, int finalize)
{
    double bsum = block_sum_f64(acc, bad);
    __shared__ bool s_last;
    if (threadIdx.x == 0) {
        out.partial_sum[blockIdx.x] = bsum;
        out.partial_bad[blockIdx.x] = bad;
        __threadfence();
        uint32_t t = atomicInc(out.ticket, gridDim.x - 1);  // wraps to 0 after the last CTA
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
        if (finalize)
            write_ctrl(out.ctrl, tot, anybad, max_norm);
    }
}

// Sum-of-squares accumulation without a per-element flag: any inf/NaN among the
// inputs makes the f64 sum itself non-finite (squares cannot cancel, and finite
// f32 squares cannot overflow f64), so the flag is read off the total.  That
// equivalence needs |g * inv_scale| <= |g|, i.e. inv_scale <= 1; otherwise a
// finite gradient could overflow in the f32 product and kCheckEach keeps the
// explicit per-element test on the unmultiplied value.
template <bool kCheckEach>
__device__ __forceinline__ void sq_acc_fast(float g, float inv_scale, double &acc, int &bad)
{
    if (kCheckEach) bad |= is_nonfinite(g) ? 1 : 0;
    double x = (double)__fmul_rn(g, inv_scale);
    acc = fma(x, x, acc);
}

// Chunks per loop iteration of the norm pass.  Finding a chunk's data costs two
// dependent loads (chunk entry -> table row) before the gradient loads can go
// out; with 8 KiB of bf16 per chunk that chain, not HBM, bounded the kernel.
// Taking kNormBatch chunks per iteration keeps 4x the bytes in flight per chain.
// Resident CTAs per SM every norm kernel is compiled for and launched with (5 x 256 threads at <= 48
// registers); the power-of-two kernel measured 5.88 / 6.09 / 5.69 TB/s at 4 / 5 / 8 CTAs per SM.
constexpr int kNormCtasPerSm = 5;
constexpr int kNormCtasPerSmF32 = 4;  // fp32 gradients: 16 x 128-bit loads per thread are in flight, 64 registers
constexpr int kNormBatch = 4;  // 2 and 8 measured slower (4.4 / 4.1 vs 5.3 TB/s on 1.5 G bf16 elements)

// kCheckEach = false: flag read off the sum (needs inv_scale <= 1); true: per-element test.
template <bool kBf16, bool kCheckEach>
__global__ void __launch_bounds__(kBlock, kBf16 ? kNormCtasPerSm : kNormCtasPerSmF32)
norm_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks,
            uint32_t nchunks, float inv_scale, double max_norm, int finalize, NormOut out,
            const float *__restrict__ inv_scale_dev)
{
    if (inv_scale_dev != nullptr) inv_scale = *inv_scale_dev;  // asynchronous step: the scale lives on the device
    double acc = 0.0, acc2 = 0.0;  // two chains: halves the DFMA dependency depth
    int bad = 0;
    const uint32_t stride = gridDim.x * kNormBatch;
    for (uint32_t c0 = blockIdx.x * kNormBatch; c0 < nchunks; c0 += stride) {
        const char *base[kNormBatch];
        uint32_t nitems[kNormBatch];
        bool stray = false;  // some chunk of the batch has head / tail / unaligned elements
#pragma unroll
        for (int j = 0; j < kNormBatch; ++j) {
            nitems[j] = 0;
            base[j] = nullptr;
            if (c0 + j < nchunks) {
                const Chunk ck = chunks[c0 + j];
                const TensorDesc d = descs[ck.tensor];
                const ChunkView cv = chunk_view(d, ck);
                base[j] = (const char *)d.g + cv.item0 * (kBf16 ? 2 : 4);
                nitems[j] = cv.nitems;
                stray |= (cv.s_lo1 > cv.s_lo0) | (cv.s_hi1 > cv.s_hi0);
            }
        }
        if (kBf16) {
            uint2 g[kNormBatch][kItemsPerThread];
#pragma unroll
            for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
                for (int u = 0; u < kItemsPerThread; ++u) {
                    uint32_t i = threadIdx.x + u * kBlock;
                    if (i < nitems[j]) g[j][u] = ld_stream((const uint2 *)base[j] + i);
                }
#pragma unroll
            for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
                for (int u = 0; u < kItemsPerThread; ++u) {
                    uint32_t i = threadIdx.x + u * kBlock;
                    if (i < nitems[j]) {
                        sq_acc_fast<kCheckEach>(__uint_as_float(g[j][u].x << 16), inv_scale, acc, bad);
                        sq_acc_fast<kCheckEach>(__uint_as_float(g[j][u].x & 0xffff0000u), inv_scale, acc2, bad);
                        sq_acc_fast<kCheckEach>(__uint_as_float(g[j][u].y << 16), inv_scale, acc, bad);
                        sq_acc_fast<kCheckEach>(__uint_as_float(g[j][u].y & 0xffff0000u), inv_scale, acc2, bad);
                    }
                }
        } else {
            float4 g[kNormBatch][kItemsPerThread];
#pragma unroll
            for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
                for (int u = 0; u < kItemsPerThread; ++u) {
                    uint32_t i = threadIdx.x + u * kBlock;
                    if (i < nitems[j]) g[j][u] = ld_stream((const float4 *)base[j] + i);
                }
#pragma unroll
            for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
                for (int u = 0; u < kItemsPerThread; ++u) {
                    uint32_t i = threadIdx.x + u * kBlock;
                    if (i < nitems[j]) {
                        sq_acc_fast<kCheckEach>(g[j][u].x, inv_scale, acc, bad);
                        sq_acc_fast<kCheckEach>(g[j][u].y, inv_scale, acc2, bad);
                        sq_acc_fast<kCheckEach>(g[j][u].z, inv_scale, acc, bad);
                        sq_acc_fast<kCheckEach>(g[j][u].w, inv_scale, acc2, bad);
                    }
                }
        }
        if (stray) {  // rare: re-derive the views and walk the stray elements one by one
            for (int j = 0; j < kNormBatch && c0 + j < nchunks; ++j) {
                const Chunk ck = chunks[c0 + j];
                const TensorDesc d = descs[ck.tensor];
                const ChunkView cv = chunk_view(d, ck);
                for (int r = 0; r < 2; ++r) {
                    uint64_t b = r ? cv.s_hi0 : cv.s_lo0, e = r ? cv.s_hi1 : cv.s_lo1;
                    for (uint64_t i = b + threadIdx.x; i < e; i += kBlock) {
                        float gi = kBf16 ? bf16_to_f32(((const uint16_t *)d.g)[i]) : ((const float *)d.g)[i];
                        sq_acc_fast<kCheckEach>(gi, inv_scale, acc, bad);
                    }
                }
            }
        }
    }
    acc += acc2;
    if (!kCheckEach) bad = (__double2hiint(acc) & 0x7ff00000) == 0x7ff00000 ? 1 : 0;  // inf or NaN
    norm_finish(acc, bad, out, max_norm, finalize);
}

// ---- bf16 norm pass for power-of-two unscale factors ------------------------------------------------
// The generic kernel above spends a shift or mask, an f32 multiply, an f32 -> f64 convert and an f64 FMA per
// element, and on bf16 input (2 bytes per element) that instruction stream, not HBM, is what bounds it.
// A loss scale is a power of two in practice (it starts at 2^16 and only ever doubles or halves), and
// without a scaler the factor is 1, so here the factor 2^-k never touches an element: the raw values are
// squared and the exact power 2^-2k is applied once per thread at the end.  For k <= 16 the reference's
// f32 product g * 2^-k is exact for every finite bf16 g (the smallest bf16 subnormal, 2^-133, times 2^-16 is
// the smallest f32 subnormal), and scaling by a power of two commutes with every rounding of the f64
// accumulation (nothing under- or overflows: partial sums stay within 2^-300 .. 2^300), so the sum has the
// same bits as the generic kernel's.  Each bf16 half goes to f64 with ONE conversion instruction
// (cvt.f64.bf16, exact for every input; inf / NaN stay inf / NaN and show in the sum), which leaves two
// instructions per element.  Measured on 1.2 G elements: generic 4.81 TB/s; scale folded but shift + f32 ->
// f64 convert kept 5.74; this form 6.09 (5 CTAs per SM).  Building the f64 by integer bit placement
// instead of converting (mask, shift, one FP64 multiply to renormalise, integer max for inf / NaN) was also
// built and measured: 4.9 TB/s for every element, 5.6 for every second one - more issue slots than the
// convert it saves.  Accumulation order (low halves into `acc`, high halves into `acc2`) is the generic
// kernel's.
__device__ __forceinline__ double bf16_half_to_f64(uint16_t h)
{
    double x;
    asm("cvt.f64.bf16 %0, %1;" : "=d"(x) : "h"(h));
    return x;
}

// kGuard (17 <= k <= kPow2MaxK): the f32 product g * 2^-k is exact only while g's lowest set bit is at least
// 2^(k-149), which holds for zero and for every g whose exponent field is at least k - 15.  The batch's words
// are tested for a nonzero magnitude below that threshold T = (k - 15) << 7 with a mask and one two-halfword
// add-and-minimum per word: (magnitude - 1) mod 2^16 is at most T - 2 exactly for 1 <= magnitude < T (zero wraps
// to 0xffff), so the running per-half minimum is compared with T - 1 once per batch.  A thread that finds such
// a value takes the batch the reference's way - f32 product rounded to the f32 subnormal grid, converted,
// brought back by the exact factor 2^k - in the same accumulation order.
// Measured on 1.2 G ordinary elements: 5.95-6.04 TB/s with this guard (5.78 with a mask, two adds and a three-input
// logic operation per word instead of the add-and-minimum), 6.28 without a guard, 4.81 for norm_kernel.
struct Pow2Guard {
    uint32_t limit;     // T - 1
    float inv_scale;    // 2^-k
    double up;          // 2^k
};

template <bool kFull, bool kGuard>
__device__ __forceinline__ void norm_pow2_batch(const char *const (&base)[kNormBatch], const uint32_t (&nitems)[kNormBatch],
                                                double &acc, double &acc2, const Pow2Guard &gd)
{
    uint2 g[kNormBatch][kItemsPerThread];
#pragma unroll
    for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (kFull || i < nitems[j]) g[j][u] = ld_stream((const uint2 *)base[j] + i);
            else g[j][u] = make_uint2(0u, 0u);  // +0: adds nothing to either chain
        }
    if (kGuard) {
        uint32_t mn = 0xffffffffu;  // per half: min over the batch of (magnitude - 1) mod 2^16; zero wraps to 0xffff
#pragma unroll
        for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
            for (int u = 0; u < kItemsPerThread; ++u) {
                mn = __viaddmin_u16x2(g[j][u].x & 0x7fff7fffu, 0xffffffffu, mn);
                mn = __viaddmin_u16x2(g[j][u].y & 0x7fff7fffu, 0xffffffffu, mn);
            }
        const bool tiny = (mn & 0xffffu) < gd.limit || (mn >> 16) < gd.limit;
        if (tiny) {  // rare: element by element, as norm_kernel computes it, times 2^k
#pragma unroll
            for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
                for (int u = 0; u < kItemsPerThread; ++u) {  // unrolled: the words stay in registers
                    const uint32_t w0 = g[j][u].x, w1 = g[j][u].y;
                    double x;
                    x = (double)__fmul_rn(bf16_to_f32(w0 & 0xffffu), gd.inv_scale) * gd.up; acc = fma(x, x, acc);
                    x = (double)__fmul_rn(bf16_to_f32(w0 >> 16), gd.inv_scale) * gd.up; acc2 = fma(x, x, acc2);
                    x = (double)__fmul_rn(bf16_to_f32(w1 & 0xffffu), gd.inv_scale) * gd.up; acc = fma(x, x, acc);
                    x = (double)__fmul_rn(bf16_to_f32(w1 >> 16), gd.inv_scale) * gd.up; acc2 = fma(x, x, acc2);
                }
            return;
        }
    }
#pragma unroll
    for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            const uint32_t w0 = g[j][u].x, w1 = g[j][u].y;
            double x;
            x = bf16_half_to_f64((uint16_t)(w0 & 0xffffu)); acc = fma(x, x, acc);
            x = bf16_half_to_f64((uint16_t)(w0 >> 16)); acc2 = fma(x, x, acc2);
            x = bf16_half_to_f64((uint16_t)(w1 & 0xffffu)); acc = fma(x, x, acc);
            x = bf16_half_to_f64((uint16_t)(w1 >> 16)); acc2 = fma(x, x, acc2);
        }
}

// `scale` = 2^-2k, applied to each thread's sum.
template <bool kGuard>
__global__ void __launch_bounds__(kBlock)
norm_pow2_bf16_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks, uint32_t nchunks,
                      double scale, double max_norm, int finalize, NormOut out, Pow2Guard gd)
{
    double acc = 0.0, acc2 = 0.0;
    const uint32_t stride = gridDim.x * kNormBatch;
    for (uint32_t c0 = blockIdx.x * kNormBatch; c0 < nchunks; c0 += stride) {
        const char *base[kNormBatch];
        uint32_t nitems[kNormBatch];
        bool stray = false, full = true;
#pragma unroll
        for (int j = 0; j < kNormBatch; ++j) {
            nitems[j] = 0;
            base[j] = nullptr;
            if (c0 + j < nchunks) {
                const Chunk ck = chunks[c0 + j];
                const TensorDesc d = descs[ck.tensor];
                const ChunkView cv = chunk_view(d, ck);
                base[j] = (const char *)d.g + cv.item0 * 2;
                nitems[j] = cv.nitems;
                stray |= (cv.s_lo1 > cv.s_lo0) | (cv.s_hi1 > cv.s_hi0);
            }
            full &= nitems[j] == kChunkItems;
        }
        if (full) norm_pow2_batch<true, kGuard>(base, nitems, acc, acc2, gd);  // the common case carries no per-item predicates
        else norm_pow2_batch<false, kGuard>(base, nitems, acc, acc2, gd);
        if (stray) {  // rare: head / tail elements one by one into the first chain, as the generic kernel does
            for (int j = 0; j < kNormBatch && c0 + j < nchunks; ++j) {
                const Chunk ck = chunks[c0 + j];
                const TensorDesc d = descs[ck.tensor];
                const ChunkView cv = chunk_view(d, ck);
                for (int r = 0; r < 2; ++r) {
                    uint64_t b = r ? cv.s_hi0 : cv.s_lo0, e = r ? cv.s_hi1 : cv.s_lo1;
                    for (uint64_t i = b + threadIdx.x; i < e; i += kBlock) {
                        const uint16_t hw = ((const uint16_t *)d.g)[i];
                        double x = kGuard ? (double)__fmul_rn(bf16_to_f32(hw), gd.inv_scale) * gd.up : bf16_half_to_f64(hw);
                        acc = fma(x, x, acc);
                    }
                }
            }
        }
    }
    acc = acc * scale + acc2 * scale;
    int bad = (__double2hiint(acc) & 0x7ff00000) == 0x7ff00000 ? 1 : 0;  // inf or NaN among the inputs
    norm_finish(acc, bad, out, max_norm, finalize);
}

// Non-finite test alone, for steps that use loss scaling but no clipping: no norm is needed then, only the
// all-or-nothing skip decision, and without the f64 squares the pass is a plain HBM read.  The exponent
// field is all ones exactly when adding one to it carries into the (masked-out) sign position, so a whole
// 32-bit word - two bf16 values or one f32 - is tested with an AND, an ADD and an OR.
template <bool kBf16>
__global__ void __launch_bounds__(kBlock)
nonfinite_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks, uint32_t nchunks,
                 NormOut out)
{
    constexpr uint32_t kMask = kBf16 ? 0x7f807f80u : 0x7f800000u;
    constexpr uint32_t kOne = kBf16 ? 0x00800080u : 0x00800000u;
    uint32_t accw = 0;
    const uint32_t stride = gridDim.x * kNormBatch;
    for (uint32_t c0 = blockIdx.x * kNormBatch; c0 < nchunks; c0 += stride) {
        const char *base[kNormBatch];
        uint32_t nitems[kNormBatch];
        bool stray = false;
#pragma unroll
        for (int j = 0; j < kNormBatch; ++j) {
            nitems[j] = 0;
            base[j] = nullptr;
            if (c0 + j < nchunks) {
                const Chunk ck = chunks[c0 + j];
                const TensorDesc d = descs[ck.tensor];
                const ChunkView cv = chunk_view(d, ck);
                base[j] = (const char *)d.g + cv.item0 * (kBf16 ? 2 : 4);
                nitems[j] = cv.nitems;
                stray |= (cv.s_lo1 > cv.s_lo0) | (cv.s_hi1 > cv.s_hi0);
            }
        }
        if (kBf16) {
            uint2 g[kNormBatch][kItemsPerThread];
#pragma unroll
            for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
                for (int u = 0; u < kItemsPerThread; ++u) {
                    uint32_t i = threadIdx.x + u * kBlock;
                    g[j][u] = i < nitems[j] ? ld_stream((const uint2 *)base[j] + i) : make_uint2(0u, 0u);
                }
#pragma unroll
            for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
                for (int u = 0; u < kItemsPerThread; ++u)
                    accw |= ((g[j][u].x & kMask) + kOne) | ((g[j][u].y & kMask) + kOne);
        } else {
            float4 g[kNormBatch][kItemsPerThread];
#pragma unroll
            for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
                for (int u = 0; u < kItemsPerThread; ++u) {
                    uint32_t i = threadIdx.x + u * kBlock;
                    g[j][u] = i < nitems[j] ? ld_stream((const float4 *)base[j] + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
            for (int j = 0; j < kNormBatch; ++j)
#pragma unroll
                for (int u = 0; u < kItemsPerThread; ++u)
                    accw |= ((__float_as_uint(g[j][u].x) & kMask) + kOne) | ((__float_as_uint(g[j][u].y) & kMask) + kOne) |
                            ((__float_as_uint(g[j][u].z) & kMask) + kOne) | ((__float_as_uint(g[j][u].w) & kMask) + kOne);
        }
        if (stray) {
            for (int j = 0; j < kNormBatch && c0 + j < nchunks; ++j) {
                const Chunk ck = chunks[c0 + j];
                const TensorDesc d = descs[ck.tensor];
                const ChunkView cv = chunk_view(d, ck);
                for (int r = 0; r < 2; ++r) {
                    uint64_t b = r ? cv.s_hi0 : cv.s_lo0, e = r ? cv.s_hi1 : cv.s_lo1;
                    for (uint64_t i = b + threadIdx.x; i < e; i += kBlock) {
                        float gi = kBf16 ? bf16_to_f32(((const uint16_t *)d.g)[i]) : ((const float *)d.g)[i];
                        accw |= is_nonfinite(gi) ? 0x80000000u : 0u;
                    }
                }
            }
        }
    }
    int bad = (accw & 0x80008000u) != 0u ? 1 : 0;
    double zero = 0.0;
    block_sum_f64(zero, bad);
    __shared__ bool s_last;
    if (threadIdx.x == 0) {
        out.partial_bad[blockIdx.x] = bad;
        __threadfence();
        uint32_t t = atomicInc(out.ticket, gridDim.x - 1);
        s_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last)
        return;
    __threadfence();
    int anybad = 0;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += kBlock) anybad |= __ldcg(out.partial_bad + i);
    zero = 0.0;
    block_sum_f64(zero, anybad);
    if (threadIdx.x == 0) {
        out.local[0] = 0.0;
        out.local[1] = anybad ? 1.0 : 0.0;
        write_ctrl(out.ctrl, 0.0, anybad, 0.0);
    }
}

// Cross-rank finalize: `gathered` holds {sumsq, nonfinite} of every rank in
// rank order; every rank adds them in that order and so reaches the same
// decision bit for bit.
__global__ void finalize_ranks_kernel(const double *__restrict__ gathered, int world,
                                      double max_norm, StepCtrl *ctrl)
{
    if (threadIdx.x != 0 || blockIdx.x != 0)
        return;
    double tot = 0.0;
    int bad = 0;
    for (int r = 0; r < world; ++r) {
        tot += gathered[2 * r];
        bad |= gathered[2 * r + 1] != 0.0 ? 1 : 0;
    }
    write_ctrl(ctrl, tot, bad, max_norm);
}

// ---- device-resident step state (asynchronous / graph-captured step) ------------------------------
// prepare_kernel: before a step, one thread per group turns the device-held configuration and step
// counter into that group's AdamHP (for step_count + 1, as the host does for the synchronous step) and
// publishes f32(1/scale).  commit_kernel: after the step, one thread applies the outcome to the state -
// GradScaler::unscale_and_update's bookkeeping (core.rs:367-386) and the step counters, which do not
// advance on a skipped step (trainer.rs:230-237).
__global__ void prepare_kernel(const DevState *__restrict__ st, AdamHP *__restrict__ hp_out,
                               float *__restrict__ inv_scale_out, int use_scaler)
{
    float inv_scale = use_scaler ? (float)(1.0 / st->scale) : 1.0f;
    int g = threadIdx.x;
    if (g < st->ngroups) {
        const DevGroup &c = st->g[g];
        hp_out[g] = adam_hparams_of(c.lr, c.beta1, c.beta2, c.eps, c.weight_decay, c.kind == 0 /* AdamW */,
                                    c.step_count + 1, inv_scale);
    }
    if (g == 0) *inv_scale_out = inv_scale;
}

__global__ void commit_kernel(DevState *st, const StepCtrl *__restrict__ ctrl, int use_scaler)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    bool bad = ctrl != nullptr && ctrl->nonfinite != 0;
    if (bad) {
        if (use_scaler) {
            st->scale *= st->backoff_factor;
            st->consecutive_ok = 0;
        }
    } else {
        for (int g = 0; g < st->ngroups; ++g)
            if (st->g[g].kind != 2 /* SGD */) st->g[g].step_count += 1;
        if (use_scaler) {
            st->consecutive_ok += 1;
            if (st->consecutive_ok >= st->growth_interval) {
                st->scale *= st->growth_factor;
                st->consecutive_ok = 0;
            }
        }
    }
    st->last_applied = bad ? 0 : 1;
    st->last_nonfinite = bad ? 1 : 0;
    st->last_norm = (ctrl != nullptr && !bad) ? ctrl->norm : 0.0;
    st->steps_enqueued += 1;
}

// ---- in-place fp32 gradient rewrite ---------------------------------------------
// mode 0: GradScaler::unscale_and_update tail - zero everything when the norm
//         pass saw a non-finite value, else g *= factor (core.rs:367-376).
// mode 1: clip_grad_norm tail - g *= ctrl->clip_scale when ctrl->do_clip, else
//         nothing is touched (trainer.rs:515-521).
__global__ void __launch_bounds__(kBlock)
scale_grads_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks,
                   uint32_t nchunks, int mode, float factor, const StepCtrl *__restrict__ ctrl)
{
    bool zero = false;
    if (mode == 0) {
        zero = ctrl->nonfinite != 0;
    } else {
        if (!ctrl->do_clip)
            return;
        factor = ctrl->clip_scale;
    }
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const Chunk ck = chunks[c];
        const TensorDesc d = descs[ck.tensor];
        const ChunkView cv = chunk_view(d, ck);
        float *G = (float *)d.g;
        float4 *g4 = (float4 *)(G + cv.item0);
        float4 g[kItemsPerThread];
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (i < cv.nitems && !zero) g[u] = ld_stream(g4 + i);
        }
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (i < cv.nitems) {
                float4 o;
                if (zero) {
                    o = make_float4(0.f, 0.f, 0.f, 0.f);
                } else {
                    o.x = __fmul_rn(g[u].x, factor);
                    o.y = __fmul_rn(g[u].y, factor);
                    o.z = __fmul_rn(g[u].z, factor);
                    o.w = __fmul_rn(g[u].w, factor);
                }
                st_stream(g4 + i, o);
            }
        }
        for (int r = 0; r < 2; ++r) {
            uint64_t b = r ? cv.s_hi0 : cv.s_lo0, e = r ? cv.s_hi1 : cv.s_lo1;
            for (uint64_t i = b + threadIdx.x; i < e; i += kBlock)
                G[i] = zero ? 0.f : __fmul_rn(G[i], factor);
        }
    }
}

// Gradient accumulation, buf = buf + g (nabla-train/src/trainer.rs:262-266): the row's `p` column is
// the accumulation buffer, `g` the fresh gradient.  12 B per element.
__global__ void __launch_bounds__(kBlock)
accumulate_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks, uint32_t nchunks)
{
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const Chunk ck = chunks[c];
        const TensorDesc d = descs[ck.tensor];
        const ChunkView cv = chunk_view(d, ck);
        float *A = (float *)d.p;
        const float *G = (const float *)d.g;
        float4 *a4 = (float4 *)(A + cv.item0);
        const float4 *g4 = (const float4 *)(G + cv.item0);
        float4 a[kItemsPerThread], g[kItemsPerThread];
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (i < cv.nitems) { a[u] = ld_stream(a4 + i); g[u] = ld_stream(g4 + i); }
        }
#pragma unroll
        for (int u = 0; u < kItemsPerThread; ++u) {
            uint32_t i = threadIdx.x + u * kBlock;
            if (i < cv.nitems) {
                a[u].x = __fadd_rn(a[u].x, g[u].x); a[u].y = __fadd_rn(a[u].y, g[u].y);
                a[u].z = __fadd_rn(a[u].z, g[u].z); a[u].w = __fadd_rn(a[u].w, g[u].w);
                st_stream(a4 + i, a[u]);
            }
        }
        for (int r = 0; r < 2; ++r) {
            uint64_t b = r ? cv.s_hi0 : cv.s_lo0, e = r ? cv.s_hi1 : cv.s_lo1;
            for (uint64_t i = b + threadIdx.x; i < e; i += kBlock) A[i] = __fadd_rn(A[i], G[i]);
        }
    }
}

// zero_grad: every gradient element becomes +0 (nabla-ml/src/autograd/ops.rs:1668-1673).
template <bool kBf16>
__global__ void __launch_bounds__(kBlock)
zero_grads_kernel(const TensorDesc *__restrict__ descs, const Chunk *__restrict__ chunks,
                  uint32_t nchunks)
{
    for (uint32_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const Chunk ck = chunks[c];
        const TensorDesc d = descs[ck.tensor];
        const ChunkView cv = chunk_view(d, ck);
        if (kBf16) {
            uint16_t *G = (uint16_t *)d.g;
            uint2 *g2 = (uint2 *)(G + cv.item0);
            for (uint32_t i = threadIdx.x; i < cv.nitems; i += kBlock)
                st_stream(g2 + i, make_uint2(0u, 0u));
            for (uint64_t i = cv.s_lo0 + threadIdx.x; i < cv.s_lo1; i += kBlock) G[i] = 0;
            for (uint64_t i = cv.s_hi0 + threadIdx.x; i < cv.s_hi1; i += kBlock) G[i] = 0;
        } else {
            float *G = (float *)d.g;
            float4 *g4 = (float4 *)(G + cv.item0);
            for (uint32_t i = threadIdx.x; i < cv.nitems; i += kBlock)
                st_stream(g4 + i, make_float4(0.f, 0.f, 0.f, 0.f));
            for (uint64_t i = cv.s_lo0 + threadIdx.x; i < cv.s_lo1; i += kBlock) G[i] = 0.f;
            for (uint64_t i = cv.s_hi0 + threadIdx.x; i < cv.s_hi1; i += kBlock) G[i] = 0.f;
        }
    }
}

}  // namespace nbo
