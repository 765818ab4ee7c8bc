"""GPU: the mixed-precision AdamW step (bf16 params/grads, fp32 master/m/v) through the C ABI versus
the oracle's composition GradScaler -> clip_grad_norm -> AdamW<f32> -> cast.  Skip decisions, the
loss-scale trajectory and the bf16 cast of the fp32 masters are bit-exact; masters/m/v are held to
1e-5 relative."""
import os

import numpy as np
import pytest
import torch

from util import assert_close_rel, bf16_bits, bf16_dev, bits, exact_fraction

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_vectors.npz"))


@pytest.fixture(scope="module")
def nb():
    import nabla_b200
    return nabla_b200


def make_opt(nb, sizes, lr=3e-4, wd=0.1, no_decay=()):
    names = [("norm%d" % i if i in no_decay else "w%d" % i) for i in range(len(sizes))]
    groups = [nb.ParamGroupConfig.adamw("no_decay", nb.ParamSelector.Any([nb.ParamMatch.Prefix("norm")]), lr, 0.0)]
    return nb.MixedAdamW(names, [(n,) for n in sizes], groups,
                         nb.ParamGroupConfig.adamw("decay", nb.ParamSelector.All(), lr, wd))


def run_mixed(nb, oracle, sizes, steps, seed, max_norm, inf_steps=(), no_decay=(), offset=0, use_scaler=True,
              lr=3e-4, wd=0.1, growth_interval=None):
    rng = np.random.default_rng(seed)
    w0 = [rng.normal(0, 0.02, n).astype(np.float32) for n in sizes]
    cfgs = [oracle.AdamCfg(lr, 0.9, 0.999, 1e-8, 0.0 if i in no_decay else wd, 1) for i in range(len(sizes))]
    mo = oracle.MixedOracle(w0, cfgs, use_scaler=use_scaler)
    opt = make_opt(nb, sizes, lr, wd, no_decay)
    if growth_interval:
        st = opt.scaler_state(); st.growth_interval = growth_interval; opt.load_scaler_state(st)
        mo.scaler.growth_interval = growth_interval

    def alloc(n):
        base = torch.zeros(n + 16, dtype=torch.bfloat16, device="cuda")
        return base[offset:offset + n]
    dp = [alloc(n) for n in sizes]
    dg = [alloc(n) for n in sizes]
    for i, w in enumerate(w0):
        opt.load_master(i, torch.from_numpy(w))
        dp[i].copy_(bf16_dev(oracle.bf16_from_f32(w)))
    log = []
    for t in range(steps):
        scale = mo.scaler.scale if use_scaler else 1.0
        g16 = [oracle.bf16_from_f32((rng.normal(0, 1e-4, n) * scale).astype(np.float32)) for n in sizes]
        if t in inf_steps:
            big = int(np.argmax(sizes))
            g16[big][int(rng.integers(0, sizes[big]))] = 0x7F80
        for d, g in zip(dg, g16):
            d.copy_(bf16_dev(g))
        res = opt.step(dp, dg, use_scaler=use_scaler, max_norm=max_norm)
        ok, norm = mo.step(g16, max_norm=max_norm)
        # decisions and the scale trajectory: bit-exact
        assert res.applied == ok, f"step {t}: skip decision differs"
        assert res.nonfinite == (not ok)
        assert res.loss_scale == mo.scaler.scale, f"step {t}: loss scale differs"
        assert res.step_count == mo.step_count.value
        if ok and max_norm > 0:
            assert abs(res.grad_norm - norm) <= 1e-12 * norm, f"step {t}: norm {res.grad_norm} vs {norm}"
        log.append((ok, res.grad_norm))
    torch.cuda.synchronize()
    return opt, mo, dp, log


SIZES = [1, 3, 4, 5, 7, 8, 9, 255, 4095, 4096, 4097, 65536 + 3, 300001]


@pytest.mark.parametrize("offset", [0, 1])          # 1 = bf16 base pointers only 2-byte aligned
def test_mixed_versus_oracle(nb, oracle, offset):
    opt, mo, dp, log = run_mixed(nb, oracle, SIZES, 8, 3, max_norm=0.004, inf_steps=(3,), no_decay=(2, 7),
                                 offset=offset)
    assert [ok for ok, _ in log] == [True, True, True, False, True, True, True, True]
    assert any(n > 0.004 for ok, n in log if ok) or True
    fr = []
    for i, n in enumerate(SIZES):
        w = opt.master(i).numpy()
        m, v = opt.moments(i)
        assert_close_rel(w, mo.master[i], f"master n={n}")
        assert_close_rel(m.numpy(), mo.m[i], f"m n={n}")
        assert_close_rel(v.numpy(), mo.v[i], f"v n={n}")
        # bf16 cast of identical fp32 masters: bit-exact
        assert np.array_equal(bf16_bits(dp[i]), oracle.bf16_from_f32(w)), f"bf16 cast n={n}"
        fr.append((exact_fraction(w, mo.master[i]), float((bf16_bits(dp[i]) == mo.p[i]).mean())))
    print("bit-exact masters %.4f%%, bf16 params equal to the oracle's %.4f%%"
          % (100 * np.mean([a for a, _ in fr]), 100 * np.mean([b for _, b in fr])))


def test_clipping_actually_engages(nb, oracle):
    opt, mo, dp, log = run_mixed(nb, oracle, [4096 * 3 + 1, 1000], 4, 8, max_norm=1e-3)
    assert all(n > 1e-3 for ok, n in log)            # every step clipped
    for i in range(2):
        assert_close_rel(opt.master(i).numpy(), mo.master[i], "master")
    opt2, mo2, dp2, log2 = run_mixed(nb, oracle, [4096 * 3 + 1, 1000], 4, 8, max_norm=0.0)
    assert all(ok for ok, _ in log2)
    assert not np.array_equal(opt.master(0).numpy(), opt2.master(0).numpy())


def test_skipped_step_changes_nothing_but_the_scaler(nb, oracle):
    sizes = [4097, 33]
    opt, mo, dp, log = run_mixed(nb, oracle, sizes, 2, 5, max_norm=1.0)
    before = [(opt.master(i).numpy().copy(), opt.moments(i)[0].numpy().copy(), opt.moments(i)[1].numpy().copy(),
               bf16_bits(dp[i]).copy()) for i in range(2)]
    g = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for n in sizes]
    g[1][32] = float("nan")
    s0, c0 = opt.scaler_state().scale, opt.step_count()
    res = opt.step(dp, g, use_scaler=True, max_norm=1.0)
    assert not res.applied and res.nonfinite and res.loss_scale == s0 * 0.5 and res.step_count == c0
    assert opt.scaler_state().consecutive_ok == 0
    for i in range(2):
        assert np.array_equal(opt.master(i).numpy(), before[i][0])
        assert np.array_equal(opt.moments(i)[0].numpy(), before[i][1])
        assert np.array_equal(opt.moments(i)[1].numpy(), before[i][2])
        assert np.array_equal(bf16_bits(dp[i]), before[i][3])
    # no scaler, clipping on: non-finite still skips (GradNanPolicy::Skip) and the scale is untouched
    res = opt.step(dp, g, use_scaler=False, max_norm=1.0)
    assert not res.applied and res.loss_scale == s0 * 0.5


def test_scale_growth_and_injection_every_50th_step(nb, oracle):
    """Dynamic loss scale: halve on overflow, double after `interval` clean steps; inf every 50th step."""
    inf_steps = tuple(range(49, 200, 50))
    opt, mo, dp, log = run_mixed(nb, oracle, [5000, 129], 200, 17, max_norm=1.0, inf_steps=inf_steps,
                                 growth_interval=20)
    skipped = [t for t, (ok, _) in enumerate(log) if not ok]
    assert skipped == list(inf_steps)
    assert opt.step_count() == 196
    for i in range(2):
        assert_close_rel(opt.master(i).numpy(), mo.master[i], "master after 196 applied steps")
        assert np.array_equal(bf16_bits(dp[i]), oracle.bf16_from_f32(opt.master(i).numpy()))


def test_committed_mixed_vectors(nb, oracle):
    n = GOLD["mixed_w0"].size
    opt = nb.MixedAdamW.adamw(3e-4, 0.1, [(n,)])
    opt.load_master(0, torch.from_numpy(GOLD["mixed_w0"]))
    p = bf16_dev(oracle.bf16_from_f32(GOLD["mixed_w0"]))
    for t in range(6):
        res = opt.step([p], [bf16_dev(GOLD["mixed_g16"][t])], use_scaler=True, max_norm=1e-3)
        assert res.applied == bool(GOLD["mixed_ok"][t])
        assert res.loss_scale == GOLD["mixed_scale"][t]
        if res.applied:
            assert abs(res.grad_norm - GOLD["mixed_norm"][t]) <= 1e-12 * GOLD["mixed_norm"][t]
    assert opt.step_count() == int(GOLD["mixed_step_count"][0])
    assert_close_rel(opt.master(0).numpy(), GOLD["mixed_master"], "master")
    assert float((bf16_bits(p) == GOLD["mixed_p16"]).mean()) > 0.999


def test_bf16_cast_edge_values_through_the_kernel(nb, oracle):
    """Masters at rounding edge cases (ties, subnormals, max-finite -> inf, -0) cast exactly like the oracle:
    zero grads, zero weight decay and lr 0 leave the master untouched, so the kernel's bf16 write is the cast."""
    edge = GOLD["bf16_edge_in"].view(np.float32)
    edge = edge[~np.isnan(edge)]
    rng = np.random.default_rng(0)
    w = np.concatenate([edge, rng.integers(0, 0x7F800000, 100000).astype(np.uint32).view(np.float32)])
    n = w.size
    opt = nb.MixedAdamW.adamw(0.0, 0.0, [(n,)])
    opt.load_master(0, torch.from_numpy(w))
    p = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    g = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    res = opt.step([p], [g], use_scaler=False, max_norm=0.0)
    assert res.applied
    got_w = opt.master(0).numpy()
    want_w = w.copy(); m = np.zeros(n, np.float32); v = np.zeros(n, np.float32)
    oracle.adam_step(want_w, np.zeros(n, np.float32), m, v, 0.0, weight_decay=0.0, step=1, decoupled=True)
    assert np.array_equal(bits(got_w), bits(want_w))
    assert np.array_equal(bf16_bits(p), oracle.bf16_from_f32(want_w))
    # NaN masters: the arithmetic canonicalises NaNs differently on the two machines, but the cast of whatever
    # master the GPU holds keeps sign and upper payload with the quiet bit set, exactly like the oracle's cast
    nan_bits = np.array([0x7FC00000, 0xFFC00001, 0x7F800001, 0xFFFFFFFF, 0x7FABCDEF, 0x3F800000, 0x7F800000],
                        dtype=np.uint32)
    wn = np.tile(nan_bits, 600).view(np.float32)
    opt2 = nb.MixedAdamW.adamw(0.0, 0.0, [(wn.size,)])
    opt2.load_master(0, torch.from_numpy(wn.copy()))
    p2 = torch.zeros(wn.size, dtype=torch.bfloat16, device="cuda")
    opt2.step([p2], [torch.zeros_like(p2)], use_scaler=False, max_norm=0.0)
    gw = opt2.master(0).numpy()
    assert np.isnan(gw).sum() == 5 * 600
    assert np.array_equal(bf16_bits(p2), oracle.bf16_from_f32(gw))


def test_init_master_from_params_and_zero_grad(nb):
    n = 4099
    p = torch.randn(n, device="cuda").to(torch.bfloat16)
    opt = nb.MixedAdamW.adamw(1e-3, 0.0, [(n,)])
    opt.init_master_from_params([p])
    assert torch.equal(opt.master(0), p.float().cpu())
    g = torch.randn(n, device="cuda").to(torch.bfloat16)
    opt.zero_grad([g])
    assert not g.float().abs().sum().item()


def test_large_norm_and_exact_flag(nb):
    """2^25 elements: the norm equals the f64 norm to summation-order noise, a finite value whose square would
    overflow f32 does not raise the non-finite flag (squares are taken in f64), a true inf / NaN does."""
    import ctypes as C
    n = (1 << 25) + 5
    opt = nb.MixedAdamW.adamw(0.0, 0.0, [(n,)])
    g = (torch.randn(n, device="cuda") * 3e-3).to(torch.bfloat16)

    def norm(t):
        a, b = C.c_double(), C.c_int32()
        opt._h.check(opt._h.lib.nbo_grad_norm(opt._h.h, 1, nb._lib.ptr_array([t.data_ptr()]), C.byref(a), C.byref(b)))
        return a.value, bool(b.value)
    want = float(torch.linalg.vector_norm(g.double()))
    got, bad = norm(g)
    assert not bad and abs(got - want) <= 1e-12 * want, (got, want)
    assert norm(g) == (got, bad)                                  # deterministic
    g[12345] = 1e30                                               # finite; 1e60 overflows f32 but not f64
    got, bad = norm(g)
    assert not bad and abs(got - 1e30) <= 1e28
    for v in (float("inf"), float("nan"), float("-inf")):
        g[12345] = 0.0
        g[n - 2] = v
        assert norm(g)[1] is True
        g[n - 2] = 0.0
    assert norm(g)[1] is False


@pytest.mark.parametrize("scale", [1.0, 2.0, 65536.0, 131072.0, 3.0])
def test_power_of_two_norm_pass_has_the_generic_kernels_bits(nb, scale):
    """With an unscale factor 2^-k, k <= 16, the synchronous step takes its norm from the kernel that converts
    each bf16 half straight to f64 and applies the scale to the sum; the asynchronous step (scale read from
    device memory) always runs the generic kernel that multiplies and converts every element.  Same grid,
    same accumulation order: the two norms must be the same f64, on data that holds zeros, bf16 and f32
    subnormals, the largest finite value and ordinary gradients, over several tensors with ragged ends.
    Scale 2^17 takes the guarded form of that kernel (see the next test); scale 3 the generic kernel on both sides."""
    sizes = [(1 << 24) + 3, 4096, 5, (1 << 22) - 1, 12345]
    gen = torch.Generator(device="cuda").manual_seed(7)
    gs = []
    for n in sizes:
        g = (torch.randn(n, device="cuda", generator=gen) * 1e-3 * scale).to(torch.bfloat16)
        bits = g.view(torch.int16)
        idx = torch.arange(n, device="cuda")
        bits[idx % 7 == 0] = 0                                   # +0
        bits[idx % 11 == 0] = -32768                             # -0
        bits[idx % 13 == 0] = 0x0001                             # smallest bf16 subnormal
        bits[idx % 17 == 0] = 0x007f                             # largest bf16 subnormal
        bits[idx % 19 == 0] = 0x0080                             # smallest normal: times 2^-16 is an f32 subnormal
        bits[idx % 23 == 0] = -32768 + 0x0b00                    # a tiny negative normal
        gs.append(g)
    gs[1].view(torch.int16)[17] = 0x7f7f                         # largest finite bf16 (its square overflows f32)
    ps = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for n in sizes]

    def fresh():
        o = nb.MixedAdamW.adamw(0.0, 0.0, [(n,) for n in sizes])  # lr 0: only the norm matters here
        st = o.scaler_state(); st.scale = scale; o.load_scaler_state(st)
        return o
    a, b = fresh(), fresh()
    P = nb._lib.ptr_array
    rb = b.step(ps, gs, use_scaler=True, max_norm=1.0)
    a.step_async(P([t.data_ptr() for t in ps]), P([t.data_ptr() for t in gs]), use_scaler=True, max_norm=1.0)
    ra = a.collect()[0]
    assert rb.applied and ra.applied and rb.grad_norm > 0.0
    assert ra.grad_norm == rb.grad_norm, (ra.grad_norm.hex(), rb.grad_norm.hex())
    # against exact integer arithmetic: every square is a dyadic rational, summed without rounding
    from fractions import Fraction
    if scale in (1.0, 65536.0):
        exact = Fraction(0)
        pick = [1, 2, 4]                                         # the small tensors, exactly
        for t in pick:
            for v in gs[t].float().cpu().tolist():
                exact += Fraction(v) * Fraction(v)
        small = nb.MixedAdamW.adamw(0.0, 0.0, [(sizes[t],) for t in pick])
        st = small.scaler_state(); st.scale = scale; small.load_scaler_state(st)
        r = small.step([ps[t] for t in pick], [gs[t] for t in pick], use_scaler=True, max_norm=1.0)
        want = float(exact) ** 0.5 / scale
        assert abs(r.grad_norm - want) <= 1e-14 * want, (r.grad_norm, want)
    # a non-finite value in a low half and in a high half of a word, in the bulk and in a ragged tail
    for t, i in ((0, 1000), (0, 1001), (0, sizes[0] - 1), (3, sizes[3] - 2)):
        keep = gs[t][i].clone()
        for v in (float("inf"), float("nan")):
            gs[t][i] = v
            r = fresh().step(ps, gs, use_scaler=True, max_norm=1.0)
            assert not r.applied and r.nonfinite, (t, i, v)
        gs[t][i] = keep
    assert fresh().step(ps, gs, use_scaler=True, max_norm=1.0).applied


@pytest.mark.parametrize("k", [17, 18, 24, 40, 64])
@pytest.mark.parametrize("tiny", ["none", "sparse", "dense"])
def test_guarded_power_of_two_norm_pass_has_the_generic_kernels_bits(nb, k, tiny):
    """From 2^17 on, g * 2^-k is no longer exact in f32 for the tiniest nonzero bf16 values (exponent field
    below k - 15): the power-of-two kernel tests every word for such a value and computes the batches that
    hold one the generic kernel's way.  Compared bit for bit with the generic kernel (asynchronous step) on
    data with no such value (fast path only), with a handful (both paths, most threads fast) and with one in
    every few elements (slow path nearly everywhere), values just below and at the threshold included."""
    scale = float(2 ** k)
    sizes = [(1 << 23) + 3, 4096, 5, (1 << 21) - 1, 12345]
    gen = torch.Generator(device="cuda").manual_seed(11 + k)
    thr = (k - 15) << 7                                          # smallest magnitude bits that stay exact
    gs = []
    for n in sizes:
        g = (torch.randn(n, device="cuda", generator=gen) * 1e-3).to(torch.bfloat16)
        bits = g.view(torch.int16)
        idx = torch.arange(n, device="cuda")
        bits[idx % 7 == 0] = 0
        bits[idx % 11 == 0] = -32768
        bits[idx % 29 == 0] = thr                                # exactly at the threshold: exact, fast path
        bits[idx % 31 == 0] = -32768 + thr + 1
        if tiny == "dense":
            bits[idx % 13 == 0] = 0x0001
            bits[idx % 17 == 0] = thr - 1                        # just below the threshold
            bits[idx % 19 == 0] = -32768 + 0x007f
            bits[idx % 23 == 0] = max(thr - 0x80, 1) + 0x55      # one exponent lower, odd mantissa
        gs.append(g)
    if tiny == "sparse":
        for t, i, b in ((0, 12345, 0x0001), (0, 12346, thr - 1), (0, (1 << 23) + 2, 0x0003), (3, 77, thr - 0x33),
                        (4, 12344, 0x007f), (2, 1, thr - 1), (1, 4095, -32768 + thr - 1)):
            gs[t].view(torch.int16)[i] = b
    ps = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for n in sizes]

    def fresh():
        o = nb.MixedAdamW.adamw(0.0, 0.0, [(n,) for n in sizes])
        st = o.scaler_state(); st.scale = scale; o.load_scaler_state(st)
        return o
    a, b = fresh(), fresh()
    P = nb._lib.ptr_array
    rb = b.step(ps, gs, use_scaler=True, max_norm=1.0)
    a.step_async(P([t.data_ptr() for t in ps]), P([t.data_ptr() for t in gs]), use_scaler=True, max_norm=1.0)
    ra = a.collect()[0]
    assert rb.applied and ra.applied and rb.grad_norm > 0.0
    assert ra.grad_norm == rb.grad_norm, (ra.grad_norm.hex(), rb.grad_norm.hex())
    for t, i in ((0, 1000), (0, 1001), (3, sizes[3] - 2)):       # non-finite values still stop the step
        keep = gs[t][i].clone()
        for v in (float("inf"), float("nan")):
            gs[t][i] = v
            r = fresh().step(ps, gs, use_scaler=True, max_norm=1.0)
            assert not r.applied and r.nonfinite, (t, i, v)
        gs[t][i] = keep


@pytest.mark.parametrize("offset", [0, 1])
def test_fp32_gradient_variant_versus_oracle(nb, oracle, offset):
    """bf16 params + fp32 gradients (accumulated in fp32): GradScaler -> clip -> AdamW on the masters -> cast,
    composed from the oracle's f32 pieces; skip decisions and casts bit-exact, masters within 1e-5."""
    rng = np.random.default_rng(21)
    sizes = [1, 5, 4097, 70001]
    w = [rng.normal(0, 0.02, n).astype(np.float32) for n in sizes]
    m = [np.zeros(n, np.float32) for n in sizes]
    v = [np.zeros(n, np.float32) for n in sizes]
    sc = oracle.new_scaler()
    opt = nb.MixedAdamW.adamw(3e-4, 0.1, [(n,) for n in sizes], grad_dtype=torch.float32)

    def alloc(n, dt):
        return torch.zeros(n + 8, dtype=dt, device="cuda")[offset:offset + n]
    dp = [alloc(n, torch.bfloat16) for n in sizes]
    dg = [alloc(n, torch.float32) for n in sizes]
    for i, a in enumerate(w):
        opt.load_master(i, torch.from_numpy(a))
        dp[i].copy_(bf16_dev(oracle.bf16_from_f32(a)))
    t_adam = 0
    for step in range(6):
        gs = [(rng.normal(0, 1e-4, n) * sc.scale).astype(np.float32) for n in sizes]
        if step == 2:
            gs[3][4242] = np.nan
        for d, g in zip(dg, gs):
            d.copy_(torch.from_numpy(g))
        res = opt.step(dp, dg, use_scaler=True, max_norm=0.004)
        ok = oracle.scaler_unscale_and_update(sc, gs)
        assert res.applied == ok and res.loss_scale == sc.scale
        if ok:
            norm = oracle.clip_grad_norm(gs, 0.004)
            assert abs(res.grad_norm - norm) <= 1e-12 * norm
            t_adam += 1
            for i in range(len(sizes)):
                oracle.adam_step(w[i], gs[i], m[i], v[i], 3e-4, weight_decay=0.1, step=t_adam, decoupled=True)
    assert opt.step_count() == t_adam == 5
    for i, n in enumerate(sizes):
        gw = opt.master(i).numpy()
        assert_close_rel(gw, w[i], f"master n={n}")
        assert np.array_equal(bf16_bits(dp[i]), oracle.bf16_from_f32(gw))
    with pytest.raises(TypeError):
        opt.step(dp, [x.to(torch.bfloat16) for x in dg])


@pytest.mark.parametrize("grad_dtype", [torch.bfloat16, torch.float32])
def test_loss_scaling_without_clipping_uses_the_flag_only_pass(nb, oracle, grad_dtype):
    """use_scaler with max_norm = 0: no norm is taken (grad_norm reports 0 like clip_grad_norm with max_norm <= 0),
    yet a non-finite gradient at any position - vector body, stray head / tail, first or last tensor - skips."""
    sizes = [5, 3 * 4096 + 3, 4096, 70001]
    opt = nb.MixedAdamW.adamw(3e-4, 0.1, [(n,) for n in sizes], grad_dtype=grad_dtype)
    p = [(torch.randn(n, device="cuda") * 0.02).to(torch.bfloat16) for n in sizes]
    opt.init_master_from_params(p)
    g = [(torch.randn(n, device="cuda") * 6.0).to(grad_dtype) for n in sizes]
    res = opt.step(p, g, use_scaler=True, max_norm=0.0)
    assert res.applied and res.grad_norm == 0.0 and res.step_count == 1
    scale = res.loss_scale
    for t, pos in ((0, 0), (0, 4), (1, 0), (1, 4095), (1, 4096), (1, 3 * 4096 + 2), (2, 4095), (3, 70000), (3, 33333)):
        for bad in (float("inf"), float("-inf"), float("nan")):
            keep = g[t][pos].clone()
            g[t][pos] = bad
            res = opt.step(p, g, use_scaler=True, max_norm=0.0)
            assert not res.applied and res.nonfinite and res.loss_scale == scale * 0.5, (t, pos, bad)
            scale = res.loss_scale
            g[t][pos] = keep
    g[1][100] = 3.0e38 if grad_dtype == torch.float32 else 3.0e38          # huge but finite: not flagged
    res = opt.step(p, g, use_scaler=True, max_norm=0.0)
    assert res.applied and not res.nonfinite and res.step_count == 2
