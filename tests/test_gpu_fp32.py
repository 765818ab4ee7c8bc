"""GPU: the fp32 path (Sgd / Adam / AdamW / GroupOptimizer / GradScaler / clip_grad_norm) through the
C ABI versus the CPU oracle and the committed vectors.  SGD, m and v involve only mul/add and must be
bit-exact; params of Adam/AdamW go through sqrt where the reference calls powf(x, 0.5) and are held to
1e-5 relative (the stated bar), with the bit-exact fraction reported."""
import json
import math
import os

import numpy as np
import pytest
import torch

from util import assert_close_rel, bits, dev, exact_fraction, host, misaligned

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
KAT = json.load(open(os.path.join(HERE, "golden", "reference_kat.json")))
GOLD = np.load(os.path.join(HERE, "golden", "oracle_vectors.npz"))

SIZES = [1, 3, 4, 5, 255, 256, 257, 1023, 4095, 4096, 4097, 8193, 2 ** 20 - 1, 2 ** 20, 2 ** 20 + 1]


@pytest.fixture(scope="module")
def nb():
    import nabla_b200
    return nabla_b200


def f32(x):
    return np.array([x], dtype=np.float32)


# ---- the reference's own known answers, on the GPU ------------------------------

def test_sgd_step_updates_param(nb):
    k = KAT["sgd_step_updates_param"]
    p, g = dev(f32(k["param"])).reshape(1, 1), dev(f32(k["grad"])).reshape(1, 1)
    opt = nb.Sgd(k["lr"], [(1, 1)])
    opt.step([p], [g])
    v = float(host(p)[0, 0])
    assert abs(v - k["expect"]) < 1e-6            # the reference asserts 1e-10 in f64; f32 here
    assert np.float32(v) == np.float32(1.0) + np.float32(-np.float32(0.1)) * np.float32(1.0)


@pytest.mark.parametrize("cls,name", [("Adam", "adam_step_updates_param"), ("AdamW", "adamw_step_updates_param")])
def test_adam_step_updates_param(nb, oracle, cls, name):
    k = KAT[name]
    p, g = dev(f32(k["param"])).reshape(1, 1), dev(f32(k["grad"])).reshape(1, 1)
    opt = getattr(nb, cls)(k["lr"], [(1, 1)])
    opt.step([p], [g])
    assert float(host(p)[0, 0]) < k["expect_less_than"]
    po, m, v = f32(k["param"]), f32(0), f32(0)
    oracle.adam_step(po, f32(k["grad"]), m, v, k["lr"], weight_decay=0.01 if cls == "AdamW" else 0.0, step=1,
                     decoupled=cls == "AdamW")
    assert_close_rel(p.reshape(-1), po, name)
    assert opt.step_count() == 1


def test_group_optimizer_weight_decay_exclusion(nb):
    k = KAT["group_optimizer_weight_decay_exclusion"]
    w, b = dev(f32(k["params"][0])).reshape(1, 1), dev(f32(k["params"][1])).reshape(1, 1)
    bias_group = nb.ParamGroupConfig.sgd("no_decay", nb.ParamSelector.Any([nb.ParamMatch.Suffix("bias")]), 1.0, 0.0, 0.0)
    decay_group = nb.ParamGroupConfig.sgd("decay", nb.ParamSelector.All(), k["lr"], 0.0, k["decay_wd"])
    opt = nb.GroupOptimizer.from_named_params([("weight", w), ("bias", b)], [bias_group], decay_group)
    assert opt.groups() == 2
    opt.step([w, b], [torch.zeros_like(w), torch.zeros_like(b)])
    assert abs(float(host(w)[0, 0]) - k["expect"][0]) < 1e-6
    assert float(host(b)[0, 0]) == k["expect"][1]


def test_clip_grad_norm_scales(nb):
    k = KAT["clip_grad_norm_scales"]
    g = [dev(f32(k["grads"][0])).reshape(1, 1), dev(f32(k["grads"][1])).reshape(1, 1)]
    reported = nb.clip_grad_norm(g, k["max_norm"])
    after = math.sqrt(sum(float(host(x)[0, 0]) ** 2 for x in g))
    assert reported == k["expect_reported"]
    assert abs(after - k["expect_after"]) < 1e-6
    g2 = [dev(f32(3.0)), dev(f32(4.0))]
    assert nb.clip_grad_norm(g2, 0.0) == 0.0 and float(host(g2[0])[0]) == 3.0   # trainer.rs:501-503
    assert nb.clip_grad_norm(g2, 5.0) == 5.0 and float(host(g2[1])[0]) == 4.0   # norm == max: untouched


def test_grad_scaler_unscale_and_inf(nb):
    g = [dev(f32(KAT["grad_scaler_unscale"]["grad"]))]
    sc = nb.GradScaler(g)
    assert sc.unscale_and_update(g) is True
    assert float(host(g[0])[0]) == 2.0 / 65536.0
    g = [dev(f32(float("inf"))), dev(np.arange(5, dtype=np.float32))]
    sc = nb.GradScaler(g)
    assert sc.unscale_and_update(g) is False
    assert float(host(g[0])[0]) == 0.0 and not host(g[1]).any()
    st = sc.state()
    assert st.scale == 32768.0 and st.consecutive_ok == 0
    g = [dev(f32(float("nan"))), dev(np.ones(5, dtype=np.float32))]
    assert sc.unscale_and_update(g) is False and sc.scale_factor() == 16384.0


def test_grad_scaler_growth_interval(nb):
    g = [dev(np.ones(7, dtype=np.float32))]
    sc = nb.GradScaler(g)
    st = sc.state()
    st.growth_interval = 3
    sc.load_state(st)
    for _ in range(2):
        assert sc.unscale_and_update(g)
    assert sc.scale_factor() == 65536.0
    assert sc.unscale_and_update(g)
    assert sc.scale_factor() == 131072.0 and sc.state().consecutive_ok == 0


# ---- oracle versus kernels ------------------------------------------------------

def run_pair(nb, oracle, kind, sizes, steps, seed, hp, misalign=False):
    rng = np.random.default_rng(seed)
    ps = [rng.normal(0, 0.02, n).astype(np.float32) for n in sizes]
    if misalign:
        dp = [misaligned(n) for n in sizes]
        dg = [misaligned(n, offset_elems=3) for n in sizes]
        for t, a in zip(dp, ps):
            t.copy_(torch.from_numpy(a))
    else:
        dp = [dev(a) for a in ps]
        dg = [torch.empty(n, dtype=torch.float32, device="cuda") for n in sizes]
    shapes = [(n,) for n in sizes]
    if kind == "sgd":
        opt = nb.Sgd(hp["lr"], shapes).momentum(hp.get("momentum", 0.0)).weight_decay(hp.get("weight_decay", 0.0))
    elif kind == "adam":
        opt = nb.Adam(hp["lr"], shapes)
    else:
        opt = nb.AdamW(hp["lr"], shapes).weight_decay(hp.get("weight_decay", 0.01))
    s0 = [np.zeros(n, np.float32) for n in sizes]
    s1 = [np.zeros(n, np.float32) for n in sizes]
    for t in range(1, steps + 1):
        gs = [rng.normal(0, 1e-3, n).astype(np.float32) for n in sizes]
        for d, a in zip(dg, gs):
            d.copy_(torch.from_numpy(a))
        opt.step(dp, dg)
        for i in range(len(sizes)):
            if kind == "sgd":
                oracle.sgd_step(ps[i], gs[i], s0[i], hp["lr"], hp.get("momentum", 0.0), hp.get("weight_decay", 0.0))
            else:
                oracle.adam_step(ps[i], gs[i], s0[i], s1[i], hp["lr"], weight_decay=hp.get("weight_decay", 0.01),
                                 step=t, decoupled=kind == "adamw")
    torch.cuda.synchronize()
    return opt, dp, ps, s0, s1


@pytest.mark.parametrize("hp", [dict(lr=0.01), dict(lr=0.1, momentum=0.9), dict(lr=0.1, weight_decay=0.01),
                                dict(lr=0.1, momentum=0.9, weight_decay=0.01)])
@pytest.mark.parametrize("misalign", [False, True])
def test_sgd_bit_exact(nb, oracle, hp, misalign):
    opt, dp, ps, vel, _ = run_pair(nb, oracle, "sgd", SIZES, 5, 11, hp, misalign)
    gv = opt.velocity()
    for i, n in enumerate(SIZES):
        assert np.array_equal(bits(dp[i]), bits(ps[i])), f"param n={n}"
        if hp.get("momentum"):
            assert np.array_equal(bits(gv[i].numpy()), bits(vel[i])), f"velocity n={n}"


@pytest.mark.parametrize("kind", ["adam", "adamw"])
@pytest.mark.parametrize("misalign", [False, True])
def test_adam_sizes(nb, oracle, kind, misalign):
    opt, dp, ps, m, v = run_pair(nb, oracle, kind, SIZES, 5, 5, dict(lr=1e-3, weight_decay=0.1), misalign)
    gm, gv = opt.moments()
    worst, exact = 0.0, []
    for i, n in enumerate(SIZES):
        assert np.array_equal(bits(gm[i].numpy()), bits(m[i])), f"m n={n}"      # mul/add only: exact
        assert np.array_equal(bits(gv[i].numpy()), bits(v[i])), f"v n={n}"
        worst = max(worst, assert_close_rel(dp[i], ps[i], f"{kind} p n={n}"))
        exact.append(exact_fraction(dp[i], ps[i]))
    print(f"{kind}: worst rel err {worst:.2e}, bit-exact params {100 * np.mean(exact):.3f}%")
    assert opt.step_count() == 5


@pytest.mark.parametrize("kind", ["adam", "adamw"])
def test_adam_100_steps(nb, oracle, kind):
    """fp32 params/m/v within 1e-5 relative after 100 steps."""
    sizes = [50257 * 8, 1024 * 8, 768, 768, 768 * 2304 // 16, 2304, 4097]
    opt, dp, ps, m, v = run_pair(nb, oracle, kind, sizes, 100, 2, dict(lr=1e-3, weight_decay=0.01))
    gm, gv = opt.moments()
    for i, n in enumerate(sizes):
        assert_close_rel(gm[i].numpy(), m[i], "m")
        assert_close_rel(gv[i].numpy(), v[i], "v")
        assert_close_rel(dp[i], ps[i], "p")
        assert exact_fraction(gm[i].numpy(), m[i]) == 1.0 and exact_fraction(gv[i].numpy(), v[i]) == 1.0


def test_committed_vectors(nb):
    p0, grads = GOLD["p0"], GOLD["grads"]
    n = p0.size
    for cls, name in (("Adam", "adam"), ("AdamW", "adamw")):
        p = dev(p0)
        opt = getattr(nb, cls)(1e-3, [(n,)])
        for t in range(10):
            opt.step([p], [dev(grads[t])])
        m, v = opt.moments()
        assert np.array_equal(bits(m[0].numpy()), bits(GOLD[f"{name}_m"]))
        assert np.array_equal(bits(v[0].numpy()), bits(GOLD[f"{name}_v"]))
        assert_close_rel(p, GOLD[f"{name}_p"], name)
    for name, kw in (("sgd", {}), ("sgd_mom", dict(momentum=0.9)), ("sgd_mom_wd", dict(momentum=0.9, weight_decay=0.01))):
        p = dev(p0)
        opt = nb.Sgd(0.1, [(n,)]).momentum(kw.get("momentum", 0.0)).weight_decay(kw.get("weight_decay", 0.0))
        for t in range(10):
            opt.step([p], [dev(grads[t])])
        assert np.array_equal(bits(p), bits(GOLD[f"{name}_p"]))
        assert np.array_equal(bits(opt.velocity()[0].numpy()), bits(GOLD[f"{name}_vel"])) or not kw.get("momentum")


def test_mlp_config_sgd_1000_steps(nb, oracle):
    """MLP 784-256-128-10, SGD lr 0.01, 1000 steps with fresh seeded grads: bit-exact."""
    shapes = [(256, 784), (256,), (128, 256), (128,), (10, 128), (10,)]
    rng = np.random.default_rng(0)
    ps = []
    for s in shapes:
        fan_in = s[1] if len(s) == 2 else {256: 784, 128: 256, 10: 128}[s[0]]
        b = 1.0 / math.sqrt(fan_in)
        ps.append(rng.uniform(-b, b, s).astype(np.float32))
    dp = [dev(a) for a in ps]
    dg = [torch.empty_like(d) for d in dp]
    opt = nb.Sgd.from_params(0.01, dp)
    vel = [np.zeros(a.size, np.float32) for a in ps]
    for _ in range(1000):
        gs = [rng.normal(0, 1e-3, s).astype(np.float32) for s in shapes]
        for d, a in zip(dg, gs):
            d.copy_(torch.from_numpy(a))
        opt.step(dp, dg)
        for p, g, v in zip(ps, gs, vel):
            oracle.sgd_step(p.reshape(-1), g.reshape(-1), v, 0.01)
    for d, a in zip(dp, ps):
        assert np.array_equal(bits(d), bits(a))
    assert opt._h.launch_count() == 1000          # one launch per step for the whole list
    assert opt._h.table_info()[2] == 1            # pointers never changed: one table upload


def test_fragmented_list(nb, oracle):
    """Many tensors, log-uniform sizes incl. zero-length, one SGD-momentum and one AdamW step."""
    rng = np.random.default_rng(5)
    sizes = [int(x) for x in np.exp(rng.uniform(0, math.log(2 ** 16), 600))] + [0, 0, 1, 2, 3]
    for kind, hp in (("sgd", dict(lr=0.1, momentum=0.9)), ("adamw", dict(lr=1e-3, weight_decay=0.01))):
        opt, dp, ps, s0, s1 = run_pair(nb, oracle, kind, sizes, 2, 9, hp)
        for i in range(len(sizes)):
            if kind == "sgd":
                assert np.array_equal(bits(dp[i]), bits(ps[i]))
            else:
                assert_close_rel(dp[i], ps[i], "p")
        tensors, chunks, uploads = opt._h.table_info()
        assert tensors == len(sizes) and chunks == sum((n + 4095) // 4096 for n in sizes) and uploads == 1
        assert opt._h.launch_count() == 2


def test_group_optimizer_mixed_kinds_and_set_lr(nb, oracle):
    rng = np.random.default_rng(21)
    names = ["embed.weight", "l0.weight", "l0.bias", "ln.weight"]
    sizes = [5000, 4096, 77, 300]
    ps = [rng.normal(0, 0.02, n).astype(np.float32) for n in sizes]
    dp = [dev(a) for a in ps]
    P, S, M = nb.ParamGroupConfig, nb.ParamSelector, nb.ParamMatch
    g_sgd = P.sgd("emb", S.Any([M.Prefix("embed")]), 0.5, 0.9, 0.0)
    g_nd = P.adamw("no_decay", S.Any([M.Suffix("bias"), M.Contains("ln")]), 2e-3, 0.0)
    g_dec = P.adamw("decay", S.All(), 1e-3, 0.1)
    opt = nb.GroupOptimizer.from_named_params(list(zip(names, dp)), [g_sgd, g_nd], g_dec)
    cfg = {0: ("sgd", 0.5), 2: ("nd", 2e-3), 3: ("nd", 2e-3), 1: ("dec", 1e-3)}
    s0 = [np.zeros(n, np.float32) for n in sizes]
    s1 = [np.zeros(n, np.float32) for n in sizes]
    lr_scale = 1.0
    for t in range(1, 5):
        if t == 3:                       # GroupOptimizer::set_lr: base_lr[k] * lr / base_lr[0]
            opt.set_lr(0.25)
            lr_scale = 0.25 / 0.5
            assert opt.group_lr(0) == 0.25 and opt.group_lr(1) == 2e-3 * lr_scale and opt.group_lr(2) == 1e-3 * lr_scale
        gs = [rng.normal(0, 1e-3, n).astype(np.float32) for n in sizes]
        opt.step(dp, [dev(g) for g in gs])
        for i in range(4):
            kind, lr = cfg[i]
            if kind == "sgd":
                oracle.sgd_step(ps[i], gs[i], s0[i], lr * lr_scale, 0.9, 0.0)
            else:
                oracle.adam_step(ps[i], gs[i], s0[i], s1[i], lr * lr_scale, weight_decay=0.0 if kind == "nd" else 0.1,
                                 step=t, decoupled=True)
    assert np.array_equal(bits(dp[0]), bits(ps[0]))
    for i in (1, 2, 3):
        assert_close_rel(dp[i], ps[i], names[i])
    assert opt._h.launch_count() == 4 * 3          # one launch per group per step
    names_out = [n for n, _ in opt.state_tensors()]
    assert names_out[:1] == ["g0.v0"] and "g1.m0" in names_out and "g2.v0" in names_out


def test_clip_and_scaler_versus_oracle(nb, oracle):
    rng = np.random.default_rng(4)
    sizes = [1, 5, 4096, 100003]
    gs = [rng.normal(0, 1.0, n).astype(np.float32) for n in sizes]
    dg = [dev(g) for g in gs]
    clipper = nb.GradClipper(dg)
    norm, bad = clipper.grad_norm(dg)
    want = oracle.clip_grad_norm([g.copy() for g in gs], 1e30)
    assert not bad and abs(norm - want) <= 1e-13 * want
    got = clipper.clip_grad_norm(dg, 1.0)
    want = oracle.clip_grad_norm(gs, 1.0)
    assert abs(got - want) <= 1e-13 * want
    for d, g in zip(dg, gs):
        assert np.array_equal(bits(d), bits(g))      # same f32 factor, one multiply: exact
    # scaler: unscale path and zeroing path
    sc_o = oracle.new_scaler()
    sc = nb.GradScaler(dg)
    for inject in (False, True, False):
        gs = [(rng.normal(0, 1.0, n) * 65536).astype(np.float32) for n in sizes]
        if inject:
            gs[3][777] = np.inf
        dg = [dev(g) for g in gs]
        assert sc.unscale_and_update(dg) == oracle.scaler_unscale_and_update(sc_o, gs)
        for d, g in zip(dg, gs):
            assert np.array_equal(bits(d), bits(g))
        st = sc.state()
        assert (st.scale, st.consecutive_ok) == (sc_o.scale, sc_o.consecutive_ok)


def test_norm_is_deterministic_and_detects_every_position(nb):
    n = 3 * 4096 + 5
    g = torch.randn(n, device="cuda")
    clipper = nb.GradClipper([g])
    a = clipper.grad_norm([g])[0]
    for _ in range(3):
        assert clipper.grad_norm([g])[0] == a
    ref = float(torch.linalg.vector_norm(g.double()))
    assert abs(a - ref) < 1e-12 * ref
    for pos in (0, 1, 4095, 4096, n - 6, n - 1):
        for bad in (float("inf"), float("-inf"), float("nan")):
            h = g.clone()
            h[pos] = bad
            assert clipper.grad_norm([h])[1] is True
    assert clipper.grad_norm([g])[1] is False


def test_zero_grad_and_reset(nb):
    sizes = [0, 1, 4097, 70000]
    dp = [torch.randn(n, device="cuda") for n in sizes]
    dg = [torch.randn(n, device="cuda") for n in sizes]
    opt = nb.Adam(1e-3, [(n,) for n in sizes])
    opt.step(dp, dg)
    opt.zero_grad(dg)
    assert all(not host(g).any() for g in dg)
    assert opt.step_count() == 1
    opt.reset()
    assert opt.step_count() == 0
    m, v = opt.moments()
    assert all(not x.numpy().any() for x in m + v)


def test_state_round_trip(nb):
    n = 5000
    p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    a = nb.AdamW(1e-3, [(n,)])
    a.step([p], [g])
    st = a.state_tensors()
    assert [k for k, _ in st] == ["m0", "v0"]
    b = nb.AdamW(1e-3, [(n,)])
    b.load_state_tensors(st)
    b.set_state(a.step_count(), 0.9, 0.999, 1e-8, 0.01, 1e-3)
    p2 = p.clone()
    a.step([p], [g])
    b.step([p2], [g])
    assert torch.equal(p, p2)
    with pytest.raises(ValueError, match="missing v0"):
        nb.AdamW(1e-3, [(n,)]).load_state_tensors(st[:1])


def test_pointer_change_reuploads_table(nb):
    n = 10000
    opt = nb.Sgd(0.1, [(n,)])
    p, g = torch.ones(n, device="cuda"), torch.ones(n, device="cuda")
    opt.step([p], [g]); opt.step([p], [g])
    assert opt._h.table_info()[2] == 1
    g2 = torch.full((n,), 2.0, device="cuda")
    opt.step([p], [g2])
    assert opt._h.table_info()[2] == 2
    assert torch.allclose(p, torch.full((n,), 1.0 - 0.1 - 0.1 - 0.2, device="cuda"))


def test_error_behaviour(nb):
    L = nb._lib
    opt = nb.AdamW(1e-3, [(4,), (4,)])
    p = [torch.zeros(4, device="cuda") for _ in range(2)]
    with pytest.raises(AssertionError, match="nabla-train: AdamW params/grads length mismatch"):
        opt.step(p, p[:1])
    with pytest.raises(AssertionError, match="nabla-train: AdamW params count mismatch"):
        opt.step(p[:1], p[:1])
    # the same mismatch straight at the C ABI
    arr = L.ptr_array([p[0].data_ptr()])
    rc = opt._h.lib.nbo_step(opt._h.h, 1, arr, arr)
    assert rc == L.NBO_ERR_INVALID and b"params count mismatch" in opt._h.lib.nbo_last_error(opt._h.h)
    arr = L.ptr_array([p[0].data_ptr(), 0])
    rc = opt._h.lib.nbo_step(opt._h.h, 2, arr, arr)
    assert rc == L.NBO_ERR_INVALID and b"null device pointer" in opt._h.lib.nbo_last_error(opt._h.h)
    arr = L.ptr_array([p[0].data_ptr(), p[1].data_ptr() + 2])
    rc = opt._h.lib.nbo_step(opt._h.h, 2, arr, arr)
    assert rc == L.NBO_ERR_INVALID and b"not aligned" in opt._h.lib.nbo_last_error(opt._h.h)
    with pytest.raises(TypeError):
        opt.step([x.double() for x in p], p)
    with pytest.raises(nb.optim.NablaDeviceError):
        opt.step([x.cpu() for x in p], p)
    res = L.StepResult()
    rc = opt._h.lib.nbo_step_mixed(opt._h.h, 2, arr, arr, 1, 0.0, None)
    assert rc == L.NBO_ERR_STATE
    # after all those refusals the handle still works
    opt.step(p, [torch.ones(4, device="cuda") for _ in range(2)])
    assert opt.step_count() == 1 and float(p[0][0]) < 0


def test_untouched_parameters_and_zero_eps(nb, oracle):
    """g = m = v = 0 (a parameter that never received a gradient) takes the select path around the sqrt and the
    divide: the result must still be the reference's (decay only), -0 gradients included; with eps = 0 the
    reference's 0/0 = NaN must come out too."""
    n = 5000
    rng = np.random.default_rng(12)
    p = rng.normal(0, 1, n).astype(np.float32)
    g = np.zeros(n, np.float32)
    g[::7] = -0.0
    g[1::3] = rng.normal(0, 1e-3, len(g[1::3])).astype(np.float32)      # a mix of touched and untouched
    for eps in (1e-8, 0.0):
        dp, dg = dev(p), dev(g)
        opt = nb.AdamW(1e-2, [(n,)]).weight_decay(0.1).eps(eps)
        po, m, v = p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
        for t in range(1, 4):
            opt.step([dp], [dg])
            oracle.adam_step(po, g, m, v, 1e-2, eps=eps, weight_decay=0.1, step=t, decoupled=True)
        got = host(dp)
        assert np.array_equal(np.isnan(got), np.isnan(po))
        assert np.isnan(po).any() == (eps == 0.0)
        ok = ~np.isnan(po)
        assert_close_rel(got[ok], po[ok], f"eps={eps}")
        untouched = (g == 0) & ok
        assert np.array_equal(bits(got[untouched]), bits(po[untouched]))      # decay only: exact


@pytest.mark.parametrize("n", [1, 5, 4097, 3 * 4096 + 2, 1 << 20])
def test_adamw_step_free_function(nb, oracle, n):
    """adamw_step (alg.rs:431-469): one tensor, caller-owned m and v, explicit step number; aligned and not."""
    rng = np.random.default_rng(n)
    for off in (0, 1):
        p = rng.normal(0, 0.02, n).astype(np.float32); m = np.zeros(n, np.float32); v = np.zeros(n, np.float32)
        base = [torch.zeros(n + 8, device="cuda") for _ in range(4)]
        dp, dg, dm, dv = [b[off:off + n] for b in base]
        dp.copy_(torch.from_numpy(p))
        for t in range(1, 4):
            g = rng.normal(0, 1e-3, n).astype(np.float32)
            dg.copy_(torch.from_numpy(g))
            nb.adamw_step(dp, dg, dm, dv, 1e-3, 0.9, 0.999, 1e-8, 0.05, t)
            oracle.adam_step(p, g, m, v, 1e-3, weight_decay=0.05, step=t, decoupled=True)
        assert np.array_equal(bits(dm), bits(m)) and np.array_equal(bits(dv), bits(v))
        assert_close_rel(dp, p, f"n={n} off={off}")
        assert not base[0][off + n:].any() and not base[2][:off].any()       # nothing outside the tensor is touched


def test_device_timing_api(nb):
    n = 1 << 22
    p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    opt = nb.AdamW(1e-3, [(n,)])
    with pytest.raises(nb._lib.NablaOptimError, match="profiling is off"):
        opt._h.profile_last()
    opt._h.profile(True)
    opt.step([p], [g])
    norm_ms, upd_ms = opt._h.profile_last()
    assert norm_ms == 0.0 and 0.005 < upd_ms < 5.0
