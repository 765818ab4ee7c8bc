// nabla_optim.hpp - C++ host mirror of nabla-train's optimizer interface over the C ABI.
//
// Header-only.  Same type and method names, argument meaning and failure behaviour as the Rust
// side of the reference (nabla-train/src/optim/core.rs, alg.rs, groups.rs; trainer.rs:500-523):
//   Optimizer::step / step_slices / reset / set_lr, Sgd / Adam / AdamW with their builders,
//   ParamMatch / ParamSelector / ParamGroupConfig / GroupOptimizer, LrSchedule + lr_at_step,
//   GradScaler, clip_grad_norm, zero_grad.
// Where Rust panics (assert_eq! on length mismatches) this throws std::logic_error with the same
// message; where Rust returns Err(String) this throws std::runtime_error with the same text.
// A tensor is what crosses the boundary in the reference too: a device pointer
// (Tensor::device_ptr(), nabla-core/src/common/tensor/mod.rs:132-134) and its shape.
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/nabla_optim_b200.h"

namespace nabla_b200 {

// Borrowed device memory of one 2-D row-major tensor (rows x cols fp32).
struct Tensor {
    void *device_ptr = nullptr;
    size_t rows = 0, cols = 0;
    size_t numel() const { return rows * cols; }
    std::pair<size_t, size_t> shape() const { return {rows, cols}; }
};

using OptimKind = nbo_kind;  // NBO_ADAMW, NBO_ADAM, NBO_SGD (core.rs:46-51)

namespace detail {
inline void check(const nbo_optimizer *h, int32_t rc)
{
    if (rc == NBO_OK) return;
    std::string msg = nbo_last_error(h);
    if (rc == NBO_ERR_INVALID || rc == NBO_ERR_STATE) throw std::logic_error(msg);
    throw std::runtime_error(msg);
}
struct Handle {
    nbo_optimizer *h = nullptr;
    explicit Handle(int device, void *stream)
    {
        int32_t rc = nbo_create(device, stream, &h);
        if (rc != NBO_OK) throw std::runtime_error(nbo_last_error(nullptr));
    }
    ~Handle() { nbo_destroy(h); }
    Handle(const Handle &) = delete;
    Handle &operator=(const Handle &) = delete;
};
}  // namespace detail

// trait Optimizer<f32, Cuda>  (nabla-train/src/optim/core.rs:9-44)
class Optimizer {
public:
    virtual ~Optimizer() = default;

    void step(const std::vector<Tensor *> &params, const std::vector<const Tensor *> &grads)
    {
        if (params.size() != grads.size())
            throw std::logic_error("nabla-train: " + name_ + " params/grads length mismatch");
        if (params.size() != numel_.size())
            throw std::logic_error("nabla-train: " + name_ + " params count mismatch");
        std::vector<void *> p(params.size());
        std::vector<const void *> g(grads.size());
        for (size_t i = 0; i < params.size(); ++i) {
            if (params[i]->numel() != numel_[i] || grads[i]->numel() != numel_[i])
                throw std::logic_error("nabla: axpy_inplace shapes must match");
            p[i] = params[i]->device_ptr;
            g[i] = grads[i]->device_ptr;
        }
        detail::check(h(), nbo_step(h(), p.size(), p.data(), g.data()));
    }

    void step_slices(std::vector<Tensor> &params, const std::vector<Tensor> &grads)
    {
        std::vector<Tensor *> p;
        std::vector<const Tensor *> g;
        for (auto &t : params) p.push_back(&t);
        for (auto &t : grads) g.push_back(&t);
        step(p, g);
    }

    void reset() { detail::check(h(), nbo_reset(h())); }
    void set_lr(double lr) { detail::check(h(), nbo_set_lr(h(), lr)); }

    // nabla-ml/src/autograd/ops.rs:1668-1673
    void zero_grad(const std::vector<Tensor *> &grads)
    {
        if (grads.size() != numel_.size())
            throw std::logic_error("nabla-train: " + name_ + " params count mismatch");
        std::vector<void *> g;
        for (auto *t : grads) g.push_back(t->device_ptr);
        detail::check(h(), nbo_zero_grad(h(), g.size(), g.data()));
    }

    uint64_t step_count(int group = 0) const
    {
        uint64_t c = 0;
        detail::check(h(), nbo_step_count(h(), group, &c));
        return c;
    }

    // OptimState: host copies of m{i} (which = 0) / v{i} (which = 1; the SGD velocity is slot 0)
    std::vector<float> state(size_t tensor, int which) const
    {
        std::vector<float> out(numel_.at(tensor));
        detail::check(h(), nbo_state_export(h(), tensor, which, out.data()));
        return out;
    }
    // (rows, cols) of tensor i's state: the parameter's own shape, which is what the reference writes into a
    // checkpoint for m{i} / v{i} and what its next axpy_inplace expects after a load
    // (nabla-ml/src/module/core.rs:76-78; nabla-core/src/common/tensor/ops.rs:638-646)
    std::pair<size_t, size_t> state_shape(size_t tensor) const { return shapes_.at(tensor); }
    void load_state(size_t tensor, int which, const std::vector<float> &v)
    {
        if (v.size() != numel_.at(tensor)) throw std::runtime_error("nabla: axpy_inplace shapes must match");
        detail::check(h(), nbo_state_import(h(), tensor, which, v.data()));
    }

    nbo_optimizer *raw() const { return h(); }

protected:
    Optimizer(std::string name, int device, void *stream)
        : name_(std::move(name)), handle_(std::make_shared<detail::Handle>(device, stream)) {}
    nbo_optimizer *h() const { return handle_->h; }
    void configure_single(const nbo_group_config &cfg, const std::vector<std::pair<size_t, size_t>> &shapes)
    {
        for (auto &s : shapes) { numel_.push_back((uint64_t)s.first * s.second); shapes_.push_back(s); }
        detail::check(h(), nbo_add_group(h(), &cfg, nullptr));
        detail::check(h(), nbo_set_tensors(h(), numel_.size(), numel_.data(), nullptr, NBO_F32));
    }
    nbo_group_config group(int g = 0) const
    {
        nbo_group_config c;
        detail::check(h(), nbo_get_group(h(), g, &c));
        return c;
    }
    void set_group(const nbo_group_config &c, int g = 0) { detail::check(h(), nbo_set_group(h(), g, &c)); }

    std::string name_;
    std::shared_ptr<detail::Handle> handle_;
    std::vector<uint64_t> numel_;
    std::vector<std::pair<size_t, size_t>> shapes_;
};

using Shapes = std::vector<std::pair<size_t, size_t>>;

// Sgd  (nabla-train/src/optim/alg.rs:310-428)
class Sgd : public Optimizer {
public:
    Sgd(double lr, const Shapes &param_shapes, int device = 0, void *stream = nullptr)
        : Optimizer("SGD", device, stream)
    {
        configure_single(nbo_group_config{NBO_SGD, lr, 0, 0, 0, 0, 0}, param_shapes);
    }
    Sgd &momentum(double m) { auto c = group(); c.momentum = m; set_group(c); return *this; }
    Sgd &weight_decay(double wd) { auto c = group(); c.weight_decay = wd; set_group(c); return *this; }
    double lr() const { return group().lr; }
    double momentum_value() const { return group().momentum; }
    double weight_decay_value() const { return group().weight_decay; }
};

// Adam  (alg.rs:169-308)
class Adam : public Optimizer {
public:
    Adam(double lr, const Shapes &param_shapes, int device = 0, void *stream = nullptr)
        : Optimizer("Adam", device, stream)
    {
        configure_single(nbo_group_config{NBO_ADAM, lr, 0.9, 0.999, 1e-8, 0, 0}, param_shapes);
    }
    Adam &beta1(double v) { auto c = group(); c.beta1 = v; set_group(c); return *this; }
    Adam &beta2(double v) { auto c = group(); c.beta2 = v; set_group(c); return *this; }
    Adam &eps(double v) { auto c = group(); c.eps = v; set_group(c); return *this; }
    double lr() const { return group().lr; }
};

// AdamW  (alg.rs:7-167)
class AdamW : public Optimizer {
public:
    AdamW(double lr, const Shapes &param_shapes, int device = 0, void *stream = nullptr)
        : Optimizer("AdamW", device, stream)
    {
        configure_single(nbo_group_config{NBO_ADAMW, lr, 0.9, 0.999, 1e-8, 0.01, 0}, param_shapes);
    }
    AdamW &beta1(double v) { auto c = group(); c.beta1 = v; set_group(c); return *this; }
    AdamW &beta2(double v) { auto c = group(); c.beta2 = v; set_group(c); return *this; }
    AdamW &eps(double v) { auto c = group(); c.eps = v; set_group(c); return *this; }
    AdamW &weight_decay(double v) { auto c = group(); c.weight_decay = v; set_group(c); return *this; }
    double lr() const { return group().lr; }
};

// ---- parameter groups (nabla-train/src/optim/groups.rs) ------------------------------------

struct ParamMatch {
    enum Kind { Equals, Prefix, Suffix, Contains } kind;
    std::string value;
    bool matches(const std::string &name) const
    {
        switch (kind) {
        case Equals: return name == value;
        case Prefix: return name.rfind(value, 0) == 0;
        case Suffix: return name.size() >= value.size() && name.compare(name.size() - value.size(), value.size(), value) == 0;
        case Contains: return name.find(value) != std::string::npos;
        }
        return false;
    }
};

struct ParamSelector {
    bool all = true;
    std::vector<ParamMatch> any;
    static ParamSelector All() { return {}; }
    static ParamSelector Any(std::vector<ParamMatch> m) { return ParamSelector{false, std::move(m)}; }
    bool matches(const std::string &name) const
    {
        if (all) return true;
        for (auto &m : any) if (m.matches(name)) return true;
        return false;
    }
};

struct ParamGroupConfig {
    std::string name;
    ParamSelector selector;
    nbo_group_config cfg;
    static ParamGroupConfig adamw(std::string n, ParamSelector s, double lr, double wd)
    { return {std::move(n), std::move(s), nbo_group_config{NBO_ADAMW, lr, 0.9, 0.999, 1e-8, wd, 0}}; }
    static ParamGroupConfig adam(std::string n, ParamSelector s, double lr)
    { return {std::move(n), std::move(s), nbo_group_config{NBO_ADAM, lr, 0.9, 0.999, 1e-8, 0, 0}}; }
    static ParamGroupConfig sgd(std::string n, ParamSelector s, double lr, double momentum, double wd)
    { return {std::move(n), std::move(s), nbo_group_config{NBO_SGD, lr, 0, 0, 0, wd, momentum}}; }
};

// GroupOptimizer  (groups.rs:152-313): first matching group wins, unmatched names go to the
// default group, empty groups are dropped, the default group comes last.
class GroupOptimizer : public Optimizer {
public:
    GroupOptimizer(const std::vector<std::pair<std::string, Tensor *>> &named,
                   const std::vector<ParamGroupConfig> &groups, const ParamGroupConfig *default_group,
                   int device = 0, void *stream = nullptr)
        : Optimizer("GroupOptimizer", device, stream)
    {
        std::vector<std::vector<size_t>> buckets(groups.size());
        std::vector<size_t> def;
        for (size_t i = 0; i < named.size(); ++i) {
            bool placed = false;
            for (size_t g = 0; g < groups.size() && !placed; ++g)
                if (groups[g].selector.matches(named[i].first)) { buckets[g].push_back(i); placed = true; }
            if (!placed) {
                if (!default_group) throw std::runtime_error("nabla-train: group assignment incomplete");
                def.push_back(i);
            }
        }
        std::vector<int32_t> gid(named.size(), -1);
        auto add = [&](const ParamGroupConfig &cfg, const std::vector<size_t> &idx) {
            if (idx.empty()) return;
            int32_t id = 0;
            detail::check(h(), nbo_add_group(h(), &cfg.cfg, &id));
            for (size_t i : idx) gid[i] = id;
            ++ngroups_;
        };
        for (size_t g = 0; g < groups.size(); ++g) add(groups[g], buckets[g]);
        if (default_group) add(*default_group, def);
        for (auto &nt : named) { numel_.push_back(nt.second->numel()); shapes_.push_back(nt.second->shape()); }
        detail::check(h(), nbo_set_tensors(h(), numel_.size(), numel_.data(), gid.data(), NBO_F32));
    }
    size_t groups() const { return ngroups_; }

private:
    size_t ngroups_ = 0;
};

// ---- mixed precision -------------------------------------------------------------------------------
// bf16 params and grads owned by the caller, fp32 master / m / v owned by the optimizer.  The reference has
// no such type (its Optimizer has one scalar type); one step is GradScaler::unscale_and_update ->
// clip_grad_norm -> AdamW<f32>::step on the masters -> cast to bf16, in the order of
// Trainer::train_epoch_with_max_steps (trainer.rs:230-283).
class MixedAdamW {
public:
    MixedAdamW(double lr, double weight_decay, const Shapes &shapes, int device = 0, void *stream = nullptr)
        : handle_(std::make_shared<detail::Handle>(device, stream))
    {
        nbo_group_config c{NBO_ADAMW, lr, 0.9, 0.999, 1e-8, weight_decay, 0};
        detail::check(h(), nbo_add_group(h(), &c, nullptr));
        for (auto &s : shapes) numel_.push_back((uint64_t)s.first * s.second);
        detail::check(h(), nbo_set_tensors(h(), numel_.size(), numel_.data(), nullptr, NBO_MIXED_BF16));
    }
    void init_master_from_params(const std::vector<Tensor *> &params_bf16)
    {
        std::vector<const void *> p;
        for (auto *t : params_bf16) p.push_back(t->device_ptr);
        detail::check(h(), nbo_init_master_from_params(h(), p.size(), p.data()));
    }
    // Synchronous step: returns the outcome (applied / skipped, pre-clip norm, next loss scale).
    nbo_step_result step(const std::vector<Tensor *> &params_bf16, const std::vector<const Tensor *> &grads_bf16,
                         bool use_scaler = true, double max_norm = 0.0)
    {
        collect_ptrs(params_bf16, grads_bf16);
        nbo_step_result r{};
        detail::check(h(), nbo_step_mixed(h(), p_.size(), p_.data(), g_.data(), use_scaler, max_norm, &r));
        return r;
    }
    // The same step for bf16 gradients / parameters held in host memory (one pointer per tensor, ideally
    // page-locked): copied in, updated and copied out slice by slice on three streams.  The device
    // tensors are staging.
    nbo_step_result step_host(const std::vector<Tensor *> &params_dev, const std::vector<const Tensor *> &grads_dev,
                              const std::vector<void *> &params_host, const std::vector<const void *> &grads_host,
                              bool use_scaler = true, double max_norm = 0.0, uint64_t slice_elems = 0)
    {
        if (params_host.size() != params_dev.size() || grads_host.size() != grads_dev.size())
            throw std::invalid_argument("nabla-train: AdamW params/grads length mismatch");
        collect_ptrs(params_dev, grads_dev);
        nbo_step_result r{};
        detail::check(h(), nbo_step_mixed_host(h(), p_.size(), p_.data(), g_.data(), params_host.data(),
                                               grads_host.data(), slice_elems, use_scaler, max_norm, &r));
        return r;
    }
    // Enqueue only; optimizer and scaler state advance on the device (graph-capturable).
    void step_async(const std::vector<Tensor *> &params_bf16, const std::vector<const Tensor *> &grads_bf16,
                    bool use_scaler = true, double max_norm = 0.0)
    {
        collect_ptrs(params_bf16, grads_bf16);
        detail::check(h(), nbo_step_mixed_async(h(), p_.size(), p_.data(), g_.data(), use_scaler, max_norm));
    }
    nbo_step_result collect(uint64_t *steps_done = nullptr)
    {
        nbo_step_result r{};
        detail::check(h(), nbo_step_mixed_collect(h(), &r, steps_done));
        return r;
    }
    void set_lr(double lr) { detail::check(h(), nbo_set_lr(h(), lr)); }
    uint64_t step_count() const
    {
        uint64_t c = 0;
        detail::check(h(), nbo_step_count(h(), 0, &c));
        return c;
    }
    std::vector<float> master(size_t tensor) const
    {
        std::vector<float> out(numel_.at(tensor));
        detail::check(h(), nbo_state_export(h(), tensor, 2, out.data()));
        return out;
    }

private:
    nbo_optimizer *h() const { return handle_->h; }
    void collect_ptrs(const std::vector<Tensor *> &p, const std::vector<const Tensor *> &g)
    {
        if (p.size() != g.size()) throw std::logic_error("nabla-train: AdamW params/grads length mismatch");
        if (p.size() != numel_.size()) throw std::logic_error("nabla-train: AdamW params count mismatch");
        p_.clear(); g_.clear();
        for (auto *t : p) p_.push_back(t->device_ptr);
        for (auto *t : g) g_.push_back(t->device_ptr);
    }
    std::shared_ptr<detail::Handle> handle_;
    std::vector<uint64_t> numel_;
    std::vector<void *> p_;
    std::vector<const void *> g_;
};

// ---- schedules (core.rs:81-173) ---------------------------------------------------------------

struct LrSchedule {
    nbo_lr_schedule s{};
    static LrSchedule Cosine(uint64_t warmup, uint64_t total, double min_lr)
    { LrSchedule r; r.s.kind = NBO_SCHED_COSINE; r.s.warmup_steps = warmup; r.s.total_steps = total; r.s.min_lr = min_lr; return r; }
    static LrSchedule Linear(uint64_t warmup, uint64_t total)
    { LrSchedule r; r.s.kind = NBO_SCHED_LINEAR; r.s.warmup_steps = warmup; r.s.total_steps = total; return r; }
    static LrSchedule OneCycle(double max_lr, uint64_t total, double pct_start)
    { LrSchedule r; r.s.kind = NBO_SCHED_ONECYCLE; r.s.max_lr = max_lr; r.s.total_steps = total; r.s.pct_start = pct_start; return r; }
    static LrSchedule Step(uint64_t step_size, double gamma)
    { LrSchedule r; r.s.kind = NBO_SCHED_STEP; r.s.step_size = step_size; r.s.gamma = gamma; return r; }
};

inline double lr_at_step(const LrSchedule &schedule, double base_lr, uint64_t step)
{
    double lr = 0;
    detail::check(nullptr, nbo_lr_at_step(&schedule.s, base_lr, step, &lr));
    return lr;
}

// ---- GradScaler (core.rs:254-260,334-413) and clip_grad_norm (trainer.rs:500-523) --------------

class GradScaler {
public:
    explicit GradScaler(const Shapes &grad_shapes, int device = 0, void *stream = nullptr)
        : handle_(std::make_shared<detail::Handle>(device, stream))
    {
        nbo_group_config c{NBO_SGD, 0, 0, 0, 0, 0, 0};
        detail::check(handle_->h, nbo_add_group(handle_->h, &c, nullptr));
        for (auto &s : grad_shapes) numel_.push_back((uint64_t)s.first * s.second);
        detail::check(handle_->h, nbo_set_tensors(handle_->h, numel_.size(), numel_.data(), nullptr, NBO_F32));
    }
    double scale_factor() const { return state().scale; }
    bool unscale_and_update(std::vector<Tensor> &grads)
    {
        std::vector<void *> g;
        for (auto &t : grads) g.push_back(t.device_ptr);
        int32_t ok = 0;
        detail::check(handle_->h, nbo_unscale_and_update(handle_->h, g.size(), g.data(), &ok));
        return ok != 0;
    }
    double clip_grad_norm(std::vector<Tensor> &grads, double max_norm)
    {
        std::vector<void *> g;
        for (auto &t : grads) g.push_back(t.device_ptr);
        double norm = 0;
        detail::check(handle_->h, nbo_clip_grad_norm(handle_->h, g.size(), g.data(), max_norm, &norm));
        return norm;
    }
    nbo_scaler_state state() const
    {
        nbo_scaler_state s;
        detail::check(handle_->h, nbo_scaler_get(handle_->h, &s));
        return s;
    }
    void load_state(const nbo_scaler_state &s) { detail::check(handle_->h, nbo_scaler_set(handle_->h, &s)); }

private:
    std::shared_ptr<detail::Handle> handle_;
    std::vector<uint64_t> numel_;
};

// clip_grad_norm(&mut grads, max_norm) -> pre-clip norm; max_norm <= 0 returns 0 and changes nothing.
inline double clip_grad_norm(std::vector<Tensor> &grads, double max_norm, int device = 0, void *stream = nullptr)
{
    if (max_norm <= 0.0) return 0.0;
    Shapes shapes;
    for (auto &t : grads) shapes.push_back(t.shape());
    return GradScaler(shapes, device, stream).clip_grad_norm(grads, max_norm);
}

}  // namespace nabla_b200
