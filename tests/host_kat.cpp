// The reference's own optimizer tests (nabla-train/tests/optim.rs:47-165, tests/trainer.rs:171-203),
// written against the C++ host mirror, in f32 on the GPU.  Prints HOST_KAT_OK on success.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <cuda_runtime.h>

#include "../nabla_b200/host/nabla_optim.hpp"

using namespace nabla_b200;

#define REQUIRE(c)                                                        \
    do {                                                                  \
        if (!(c)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #c); std::exit(1); } \
    } while (0)

static Tensor mat(float v)
{
    Tensor t; t.rows = t.cols = 1;
    REQUIRE(cudaMalloc(&t.device_ptr, sizeof(float)) == cudaSuccess);
    REQUIRE(cudaMemcpy(t.device_ptr, &v, sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess);
    return t;
}
static float get(const Tensor &t)
{
    float v;
    REQUIRE(cudaMemcpy(&v, t.device_ptr, sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess);
    return v;
}

int main()
{
    {   // sgd_step_updates_param
        Tensor param = mat(1.0f), grad = mat(1.0f);
        Sgd opt(0.1, {{1, 1}});
        opt.step({&param}, {&grad});
        REQUIRE(std::fabs(get(param) - 0.9f) < 1e-6f);
    }
    {   // adam_step_updates_param / adamw_step_updates_param
        Tensor p1 = mat(1.0f), p2 = mat(1.0f), grad = mat(1.0f);
        Adam a(0.1, {{1, 1}});
        AdamW w(0.1, {{1, 1}});
        a.step({&p1}, {&grad});
        w.step({&p2}, {&grad});
        REQUIRE(get(p1) < 1.0f && get(p2) < 1.0f && get(p2) < get(p1));
        REQUIRE(a.step_count() == 1);
    }
    {   // schedules
        REQUIRE(std::fabs(lr_at_step(LrSchedule::Linear(0, 10), 1.0, 0) - 1.0) < 1e-10);
        REQUIRE(lr_at_step(LrSchedule::Linear(0, 10), 1.0, 10) <= 1e-10);
        auto st = LrSchedule::Step(2, 0.1);
        REQUIRE(std::fabs(lr_at_step(st, 1.0, 0) - 1.0) < 1e-10);
        REQUIRE(std::fabs(lr_at_step(st, 1.0, 2) - 0.1) < 1e-10);
        REQUIRE(std::fabs(lr_at_step(st, 1.0, 4) - 0.01) < 1e-10);
        REQUIRE(lr_at_step(LrSchedule::OneCycle(1.0, 10, 0.5), 0.1, 3) > 0.1);
    }
    {   // grad_scaler_unscale / grad_scaler_detects_inf
        std::vector<Tensor> g{mat(2.0f)};
        GradScaler sc({{1, 1}});
        REQUIRE(sc.unscale_and_update(g));
        REQUIRE(get(g[0]) < 2.0f && get(g[0]) == 2.0f / 65536.0f);
        std::vector<Tensor> bad{mat(INFINITY)};
        GradScaler sc2({{1, 1}});
        REQUIRE(!sc2.unscale_and_update(bad));
        REQUIRE(std::fabs(get(bad[0])) < 1e-12f && sc2.scale_factor() == 32768.0);
    }
    {   // group_optimizer_weight_decay_exclusion
        Tensor weight = mat(2.0f), bias = mat(3.0f), z1 = mat(0.0f), z2 = mat(0.0f);
        auto bias_group = ParamGroupConfig::sgd("no_decay", ParamSelector::Any({{ParamMatch::Suffix, "bias"}}), 1.0, 0.0, 0.0);
        auto decay_group = ParamGroupConfig::sgd("decay", ParamSelector::All(), 1.0, 0.0, 0.1);
        GroupOptimizer opt({{"weight", &weight}, {"bias", &bias}}, {bias_group}, &decay_group);
        REQUIRE(opt.groups() == 2);
        opt.step({&weight, &bias}, {&z1, &z2});
        REQUIRE(std::fabs(get(weight) - 1.8f) < 1e-6f);
        REQUIRE(get(bias) == 3.0f);
    }
    {   // clip_grad_norm_scales
        std::vector<Tensor> grads{mat(3.0f), mat(4.0f)};
        double reported = clip_grad_norm(grads, 2.5);
        double after = std::sqrt((double)get(grads[0]) * get(grads[0]) + (double)get(grads[1]) * get(grads[1]));
        REQUIRE(reported == 5.0 && std::fabs(after - 2.5) < 1e-6);
        REQUIRE(clip_grad_norm(grads, 0.0) == 0.0);
    }
    {   // length mismatches carry the reference's panic text
        Tensor p = mat(1.0f), g = mat(1.0f);
        AdamW opt(0.1, {{1, 1}, {1, 1}});
        bool threw = false;
        try { opt.step({&p}, {&g}); } catch (const std::logic_error &e) {
            threw = std::string(e.what()) == "nabla-train: AdamW params count mismatch";
        }
        REQUIRE(threw);
    }
    {   // mixed precision through the C++ mirror: applied step, overflow skip, asynchronous step
        auto bf16 = [](float f) { uint32_t u; std::memcpy(&u, &f, 4); return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16); };
        auto unbf16 = [](uint16_t hbits) { uint32_t u = (uint32_t)hbits << 16; float f; std::memcpy(&f, &u, 4); return f; };
        const size_t n = 4099;
        std::vector<uint16_t> hp(n, bf16(1.0f)), hg(n, bf16(0.5f * 65536.0f));
        Tensor p, g; p.rows = g.rows = 1; p.cols = g.cols = n;
        REQUIRE(cudaMalloc(&p.device_ptr, n * 2) == cudaSuccess && cudaMalloc(&g.device_ptr, n * 2) == cudaSuccess);
        REQUIRE(cudaMemcpy(p.device_ptr, hp.data(), n * 2, cudaMemcpyHostToDevice) == cudaSuccess);
        REQUIRE(cudaMemcpy(g.device_ptr, hg.data(), n * 2, cudaMemcpyHostToDevice) == cudaSuccess);
        MixedAdamW opt(0.1, 0.0, {{1, n}});
        opt.init_master_from_params({&p});
        nbo_step_result r = opt.step({&p}, {&g}, true, 0.0);
        REQUIRE(r.applied == 1 && r.loss_scale == 65536.0 && r.step_count == 1);
        REQUIRE(cudaMemcpy(hp.data(), p.device_ptr, n * 2, cudaMemcpyDeviceToHost) == cudaSuccess);
        REQUIRE(std::fabs(unbf16(hp[0]) - 0.9f) < 4e-3f && hp[0] == hp[n - 1]);   // first Adam step moves by lr
        hg[n - 1] = 0x7f80;                                                          // +inf: the step must be skipped
        REQUIRE(cudaMemcpy(g.device_ptr, hg.data(), n * 2, cudaMemcpyHostToDevice) == cudaSuccess);
        r = opt.step({&p}, {&g}, true, 0.0);
        REQUIRE(r.applied == 0 && r.nonfinite == 1 && r.loss_scale == 32768.0 && r.step_count == 1);
        opt.step_async({&p}, {&g}, true, 0.0);                                      // still +inf: skipped on the device
        uint64_t done = 0;
        r = opt.collect(&done);
        REQUIRE(done == 1 && r.applied == 0 && r.loss_scale == 16384.0 && opt.step_count() == 1);
        REQUIRE(std::fabs(opt.master(0)[5] - 0.9f) < 1e-6f);
        // host-streamed step from ordinary (pageable) host vectors, 1-chunk slices: a finite gradient moves
        // every parameter by lr again; the result lands in the host vector, not only in the staging tensor
        std::vector<uint16_t> host_g(n, bf16(0.5f * 16384.0f)), host_p(n, 0);
        r = opt.step_host({&p}, {&g}, {host_p.data()}, {host_g.data()}, true, 0.0, 4096);
        REQUIRE(r.applied == 1 && r.step_count == 2 && r.loss_scale == 16384.0);
        REQUIRE(std::fabs(unbf16(host_p[0]) - 0.8f) < 4e-3f && host_p[0] == host_p[n - 1] && host_p[0] == host_p[4096]);
    }
    std::printf("HOST_KAT_OK\n");
    return 0;
}
