// Plain data shared by host and device code of libnabla_optim_b200.
#pragma once
#include <stdint.h>

namespace nbo {

// Elements per chunk.  A chunk is the unit of work one CTA takes at a time; it
// never crosses a tensor boundary.  4096 fp32 elements = 16 KiB per stream.
constexpr uint32_t kChunkElems = 4096;
constexpr uint32_t kChunkItems = kChunkElems / 4;  // one item = 4 consecutive elements
constexpr int kBlock = 256;
constexpr int kItemsPerThread = kChunkItems / kBlock;  // 4

// One tensor (or, under ZeRO-1, one piece of a tensor) of the device table.
struct TensorDesc {
    void *p;        // parameter (fp32, or bf16 in mixed precision)
    const void *g;  // gradient  (same element type as p)
    float *s0;      // m, or the SGD velocity
    float *s1;      // v
    float *s2;      // fp32 master (mixed precision)
    uint64_t n;     // elements
    uint32_t head;  // leading elements handled one by one so that the rest is 16-byte aligned;
                    // 0xffffffff = no aligned body at all (every element handled one by one)
    uint32_t group;
};
static_assert(sizeof(TensorDesc) == 56, "TensorDesc layout");

struct Chunk {
    uint32_t tensor;
    uint32_t index;   // chunk number inside the tensor
    uint32_t nitems;  // 4-element items of the aligned body in this chunk (valid while the row is aligned)
    uint32_t stray;   // 1 when this chunk also owns head or tail elements that are handled one by one
};
static_assert(sizeof(Chunk) == 16, "Chunk layout");

// Device-resident decision record written by the norm pass and read by the
// update pass of the same step, so a skipped step needs no host round trip.
struct StepCtrl {
    double sumsq;      // sum of squares of the (unscaled) gradients
    double norm;       // sqrt(sumsq)
    float clip_scale;  // f32(max_norm / norm) when clipping applies, else 1.0f
    int32_t do_clip;   // 1 when norm > max_norm && norm > 0
    int32_t nonfinite; // 1 when any still-scaled gradient is inf/NaN
    int32_t skip;      // 1 when the update must not be applied
};

struct AdamHP {
    float b1, one_minus_b1, b2, one_minus_b2, eps, ss, inv_bc2, decay;
    float inv_scale;  // f32(1/loss_scale); 1.0f without a scaler
    int32_t decoupled;
};

struct SgdHP {
    float nlr, mu, wd;
    int32_t use_mu, use_wd;
};

// Optimizer / scaler state kept on the device for the asynchronous step, so that a whole step (and a
// CUDA graph of it) runs without the host: the step counters and the loss scale advance on the device.
constexpr int kMaxDevGroups = 32;
struct DevGroup {
    double lr, beta1, beta2, eps, weight_decay;
    int32_t kind;  // nbo_kind
    int32_t pad;
    uint64_t step_count;
};
struct DevState {
    double scale, growth_factor, backoff_factor;
    uint64_t growth_interval, consecutive_ok;
    int32_t ngroups;
    int32_t last_applied;    // outcome of the most recent asynchronous step
    int32_t last_nonfinite;
    int32_t pad;
    double last_norm;
    uint64_t steps_enqueued;
    DevGroup g[kMaxDevGroups];
};

#ifdef __CUDACC__
#define NBO_HD __host__ __device__
#else
#define NBO_HD
#endif

// f64::powi as the reference's toolchain computes it: square-and-multiply, low bit first.
NBO_HD inline double powi_sqm(double a, int32_t b)
{
    uint32_t e = b < 0 ? (uint32_t)(-(int64_t)b) : (uint32_t)b;
    double r = 1.0;
    for (;;) {
        if (e & 1u) r *= a;
        e >>= 1;
        if (e == 0) break;
        a *= a;
    }
    return b < 0 ? 1.0 / r : r;
}

// Host scalars of one Adam/AdamW step narrowed to f32 once each (alg.rs:120-135).  The same code runs on
// the host (synchronous step) and in prepare_kernel (asynchronous step); IEEE double arithmetic gives
// the same bits in both places.
NBO_HD inline AdamHP adam_hparams_of(double lr, double beta1, double beta2, double eps, double weight_decay,
                                     bool decoupled, uint64_t step, float inv_scale)
{
    AdamHP h;
    double bias_corr1 = 1.0 - powi_sqm(beta1, (int32_t)step);
    double bias_corr2 = 1.0 - powi_sqm(beta2, (int32_t)step);
    double step_size = lr / bias_corr1;
    h.b1 = (float)beta1;
    h.one_minus_b1 = (float)(1.0 - beta1);
    h.b2 = (float)beta2;
    h.one_minus_b2 = (float)(1.0 - beta2);
    float wd_lr = (float)(weight_decay * lr);
    h.eps = (float)eps;
    h.ss = (float)step_size;
    h.inv_bc2 = (float)(1.0 / bias_corr2);
    h.decay = 1.0f - wd_lr;  // subtracted in f32 (alg.rs:135)
    h.inv_scale = inv_scale;
    h.decoupled = decoupled ? 1 : 0;
    return h;
}

// Where the other ranks' copies of the two flat buckets are mapped in this
// process (symmetric memory), as byte offsets from this rank's own bucket so
// that "address of element i on rank r" = local address + delta.
constexpr int kMaxPeers = 16;
struct PeerArgs {
    int32_t world, rank;
    int32_t average;      // divide the reduced gradient by world (mean) instead of summing
    float inv_world;
    int32_t keep_reduced; // also write the reduced gradient into this rank's slice of its own bucket
    int32_t barrier_expect;        // value *barrier_seen must hold for the kernel to touch any peer memory
    const int32_t *barrier_seen;   // output of the stream-ordered cross-rank barrier that precedes the kernel
    const AdamHP *hp_dev;          // asynchronous step: this launch's hyper-parameters, written by prepare_kernel
    const float *inv_scale_dev;    // asynchronous step: f32(1 / loss scale) on the device
    int64_t g_mc, p_mc;   // delta to the NVSwitch multicast mapping of the bucket (0 = none)
    int64_t g_peer[kMaxPeers];
    int64_t p_peer[kMaxPeers];
};

}  // namespace nbo
