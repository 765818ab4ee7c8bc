// Host-side internals shared by the translation units of libnabla_optim_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/nabla_optim_b200.h"
#include "types.h"

namespace nbo {

struct Group {
    nbo_group_config cfg;
    double base_lr;        // lr at creation: set_lr rescales from it (groups.rs:301-312)
    uint64_t step_count;   // Adam/AdamW step counter (alg.rs:120-121)
    uint32_t chunk_begin;  // this group's range in the chunk list
    uint32_t chunk_end;
};

// One table entry on the host: a whole tensor, or under ZeRO-1 the part of a
// tensor that falls into this rank's shard.
struct Piece {
    uint64_t tensor;      // index in the caller's list
    uint64_t offset;      // first element of the piece inside its tensor
    uint64_t n;           // elements
    uint64_t state_off;   // element offset into the flat state arrays
    uint64_t bucket_off;  // element offset into the flat bucket (ZeRO-1 only)
    int32_t group;
};

struct Zero1;     // defined in zero1.cu

// Copy streams and events of the host-streamed steps (host_step.cu, zero1.cu), made on first use.
struct HostPipe {
    cudaStream_t in = nullptr, out = nullptr;
    cudaEvent_t start = nullptr;
    std::vector<cudaEvent_t> copied;   // gradients of slice s are on the device
    std::vector<cudaEvent_t> updated;  // slice s has been updated
};

}  // namespace nbo

struct nbo_optimizer {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::string err;

    std::vector<nbo::Group> groups;

    bool configured = false;
    int precision = NBO_F32;
    uint64_t ntensors = 0;             // length of the caller's list
    std::vector<uint64_t> numel;       // per caller tensor
    std::vector<int32_t> group_of;     // per caller tensor
    std::vector<int64_t> piece_of;     // per caller tensor: its piece (non-ZeRO: identity), -1 if none
    std::vector<nbo::Piece> pieces;    // the table rows

    // flat state (fp32), one allocation each
    uint64_t state_elems = 0;
    float *d_s0 = nullptr, *d_s1 = nullptr, *d_s2 = nullptr;

    // device table
    nbo::TensorDesc *h_descs = nullptr;  // pinned staging, pieces.size() rows
    nbo::TensorDesc *d_descs = nullptr;
    nbo::Chunk *d_chunks = nullptr;
    uint32_t nchunks = 0;
    cudaEvent_t upload_done = nullptr;
    bool table_bound = false;
    uint64_t uploads = 0;
    std::vector<const void *> bound_p, bound_g;  // last bound caller pointers

    // reduction scratch and decision record
    int max_grid = 0;
    int sm_count = 0;
    double *d_partial_sum = nullptr;
    int32_t *d_partial_bad = nullptr;
    uint32_t *d_ticket = nullptr;
    double *d_local = nullptr;       // {sumsq, nonfinite} of the last norm launch
    nbo::StepCtrl *d_ctrl = nullptr;
    nbo::StepCtrl *h_ctrl = nullptr;  // pinned

    // optional device timing (nbo_profile): [0,1] bracket the norm pass, [2,3] the update launches
    bool profile = false;
    bool prof_norm_valid = false, prof_update_valid = false;
    cudaEvent_t prof_ev[4] = {nullptr, nullptr, nullptr, nullptr};

    // device-resident state of the asynchronous step; `dev_newer` = the device copy has advanced past the
    // host mirrors (groups[].step_count, scaler) and must be collected before the host reads or changes them
    nbo::DevState *d_state = nullptr;
    nbo::DevState *h_state = nullptr;  // pinned
    nbo::AdamHP *d_hp = nullptr;       // [kMaxDevGroups]
    float *d_inv_scale = nullptr;
    bool dev_newer = false;
    int last_async_checked = 0;

    nbo_scaler_state scaler{65536.0, 2.0, 0.5, 2000, 0};
    uint64_t launches = 0;

    nbo::Zero1 *zero1 = nullptr;
    double zero1_timeout_s = 600.0;

    nbo::HostPipe *host_pipe = nullptr;  // copy streams + events of the host-streamed step, made on first use
};

namespace nbo {

int32_t fail(nbo_optimizer *h, int32_t code, const std::string &msg);
int32_t fail_cuda(nbo_optimizer *h, cudaError_t e, const char *what);

#define NBO_CUDA(h, call)                                   \
    do {                                                    \
        cudaError_t e__ = (call);                           \
        if (e__ != cudaSuccess)                             \
            return nbo::fail_cuda((h), e__, #call);         \
    } while (0)

// f64::powi as the reference's toolchain computes it (square-and-multiply, low
// bit first); used for the Adam bias corrections and the step LR schedule.
double powi(double a, int32_t b);

// Host scalars of one Adam/AdamW step narrowed to f32 once each (alg.rs:120-135).
AdamHP adam_hparams(const nbo_group_config &c, uint64_t step, float inv_scale);
SgdHP sgd_hparams(const nbo_group_config &c);

// Frees and rebuilds table + state for the pieces already stored in h->pieces.
int32_t build_table(nbo_optimizer *h);
void free_table(nbo_optimizer *h);

// Points the table rows at caller memory.  Either argument may be null (keep
// what is bound).  Re-uploads only when a pointer changed.
int32_t bind_list(nbo_optimizer *h, uint64_t n, void *const *params, const void *const *grads,
                  int elem_size, const char *who);
// ZeRO-1: rows point into the two flat buckets.
int32_t bind_flat(nbo_optimizer *h, void *params_flat, const void *grads_flat);

// Kernel launches (kernels.cu), all on h->stream.  Ranges are in chunk-list
// entries; every launcher counts itself in h->launches.
int32_t launch_adam_f32(nbo_optimizer *h, uint32_t chunk_begin, uint32_t nchunks, const AdamHP &hp);
int32_t launch_sgd_f32(nbo_optimizer *h, uint32_t chunk_begin, uint32_t nchunks, const SgdHP &hp);
int32_t launch_adam_mixed(nbo_optimizer *h, uint32_t chunk_begin, uint32_t nchunks, const AdamHP &hp,
                          bool with_ctrl);
int32_t launch_norm(nbo_optimizer *h, bool bf16, float inv_scale, double max_norm, int finalize);
int32_t launch_finalize_ranks(nbo_optimizer *h, const double *gathered, int world, double max_norm);
int32_t launch_scale_grads(nbo_optimizer *h, int mode, float factor);
int32_t launch_zero_grads(nbo_optimizer *h, bool bf16);
int32_t launch_init_master(nbo_optimizer *h);
int32_t launch_accumulate(nbo_optimizer *h);
int32_t launch_nonfinite(nbo_optimizer *h, bool bf16);  // flag only, no norm (writes the decision record)
int32_t launch_norm_dev(nbo_optimizer *h, const float *inv_scale_dev, double max_norm);
int32_t launch_prepare(nbo_optimizer *h, int use_scaler);
int32_t launch_commit(nbo_optimizer *h, bool checked, int use_scaler);
int32_t launch_adam_mixed_dev(nbo_optimizer *h, uint32_t chunk_begin, uint32_t nchunks, int group, bool with_ctrl);

int32_t push_dev_state(nbo_optimizer *h);
// Sharded handles: waits for the handle's stream with the nbo_zero1_set_timeout limit (zero1.cu).
int32_t zero1_bounded_wait(nbo_optimizer *h, const char *what);

// Brings the host mirrors up to date after asynchronous steps (synchronises the stream); no-op otherwise.
int32_t collect_dev_state(nbo_optimizer *h);

// ZeRO-1 fused with its collectives over peer / multicast mappings (transport: 0 local, 1 peer, 2 multicast)
int32_t launch_zero1_fused_update(nbo_optimizer *h, uint32_t chunk_begin, uint32_t nchunks, const AdamHP &hp,
                                  bool with_ctrl, const PeerArgs &pa, int in_transport, int out_transport);
int32_t launch_zero1_reduce_norm(nbo_optimizer *h, float inv_scale, const PeerArgs &pa, int in_transport);

// One adam_mixed launch per non-empty group, hyper-parameters for step_count + 1.
int32_t launch_mixed_update(nbo_optimizer *h, float inv_scale, bool with_ctrl);
// After the decision record reached the host: advance scaler + step counters.
void commit_step(nbo_optimizer *h, bool checked, bool use_scaler, nbo_step_result *res);

// Records profiling event `i` on the stream when profiling is on.
int32_t prof_mark(nbo_optimizer *h, int i);

void zero1_destroy(nbo_optimizer *h);
void host_pipe_destroy(nbo_optimizer *h);
int32_t host_pipe_ensure(nbo_optimizer *h, size_t nslices);
// Waits for the three streams after a failed enqueue, so that no copy still touches caller memory.
void host_pipe_drain(nbo_optimizer *h);

// One int written on the stream (the input of the cross-rank barrier).
int32_t launch_store_int(nbo_optimizer *h, int32_t *dst, int32_t value);

// Host-streamed mixed-precision step over the table as currently bound (host_step.cu).  `host_p` /
// `host_g` hold one host pointer per caller tensor.
int32_t host_streamed_step(nbo_optimizer *h, void *const *host_p, const void *const *host_g,
                           uint64_t slice_elems, int32_t use_scaler, double max_norm, nbo_step_result *result);

// Brings the decision record to the host (synchronises the stream).
int32_t read_ctrl(nbo_optimizer *h);

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// Every entry point that reads or changes host-side optimizer / scaler state starts with this.
#define NBO_SYNC_STATE(h)                                               \
    do {                                                                \
        if ((h) && (h)->dev_newer) {                                    \
            int32_t rc__ = nbo::collect_dev_state((nbo_optimizer *)(h)); \
            if (rc__ != NBO_OK) return rc__;                            \
        }                                                               \
    } while (0)

}  // namespace nbo
