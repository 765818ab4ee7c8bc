"""CPU: pins the oracle against every known-answer value the reference's own tests hold for the
optimizer-step path (tests/golden/reference_kat.json, transcribed from nabla-train/tests/optim.rs
and nabla-train/tests/trainer.rs), against the committed oracle vectors, and against independent
implementations of the third-party pieces (bf16 rounding, powi)."""
import json
import math
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
KAT = json.load(open(os.path.join(HERE, "golden", "reference_kat.json")))
GOLD = np.load(os.path.join(HERE, "golden", "oracle_vectors.npz"))


def f64(x):
    return np.array([x], dtype=np.float64)


# ---- nabla-train/tests/optim.rs ------------------------------------------------

def test_sgd_step_updates_param(oracle):
    k = KAT["sgd_step_updates_param"]
    p, g, vel = f64(k["param"]), f64(k["grad"]), f64(0.0)
    oracle.sgd_step(p, g, vel, k["lr"])
    assert abs(p[0] - k["expect"]) < k["tol"]


@pytest.mark.parametrize("name,decoupled", [("adam_step_updates_param", False), ("adamw_step_updates_param", True)])
def test_adam_step_updates_param(oracle, name, decoupled):
    k = KAT[name]
    p, g, m, v = f64(k["param"]), f64(k["grad"]), f64(0.0), f64(0.0)
    oracle.adam_step(p, g, m, v, k["lr"], weight_decay=0.01 if decoupled else 0.0, step=1, decoupled=decoupled)
    assert p[0] < k["expect_less_than"]
    # first Adam step with g=1: m/(1-b1)=1, sqrt(v/(1-b2))=1 -> p = 1*(1-wd*lr) - lr/(1+eps)
    decay = 1.0 - 0.01 * k["lr"] if decoupled else 1.0
    assert abs(p[0] - (k["param"] * decay - k["lr"] / (1.0 + 1e-8))) < 1e-12


def test_linear_schedule_reaches_zero(oracle):
    k = KAT["linear_schedule_reaches_zero"]
    for s, want in k["at"].items():
        got = oracle.lr_at_step(1, k["base_lr"], int(s), warmup_steps=k["warmup_steps"], total_steps=k["total_steps"])
        assert abs(got - want) <= k["tol"]


def test_step_schedule_decays(oracle):
    k = KAT["step_schedule_decays"]
    for s, want in k["at"].items():
        got = oracle.lr_at_step(3, k["base_lr"], int(s), step_size=k["step_size"], gamma=k["gamma"])
        assert abs(got - want) < k["tol"]


def test_onecycle_reaches_max(oracle):
    k = KAT["onecycle_reaches_max"]
    got = oracle.lr_at_step(2, k["base_lr"], k["step"], max_lr=k["max_lr"], total_steps=k["total_steps"],
                            pct_start=k["pct_start"])
    assert got > k["expect_greater_than"]
    # ramp(base, max, 3, 5)
    assert got == k["base_lr"] + (k["max_lr"] - k["base_lr"]) * 3.0 / 5.0


def test_cosine_schedule_shape(oracle):
    kw = dict(warmup_steps=10, total_steps=110, min_lr=0.1)
    assert oracle.lr_at_step(0, 1.0, 0, **kw) == 0.0
    assert oracle.lr_at_step(0, 1.0, 5, **kw) == 0.5
    assert oracle.lr_at_step(0, 1.0, 10, **kw) == 1.0
    assert abs(oracle.lr_at_step(0, 1.0, 60, **kw) - 0.55) < 1e-15
    assert abs(oracle.lr_at_step(0, 1.0, 110, **kw) - 0.1) < 1e-15


def test_grad_scaler_unscale(oracle):
    k = KAT["grad_scaler_unscale"]
    sc = oracle.new_scaler()
    g = [f64(k["grad"])]
    assert oracle.scaler_unscale_and_update(sc, g) is k["expect_ok"]
    assert g[0][0] < k["expect_less_than"]
    assert g[0][0] == k["grad"] / 65536.0
    assert sc.scale == 65536.0 and sc.consecutive_ok == 1


def test_grad_scaler_detects_inf(oracle):
    k = KAT["grad_scaler_detects_inf"]
    sc = oracle.new_scaler()
    g = [f64(float(k["grad"]))]
    assert oracle.scaler_unscale_and_update(sc, g) is k["expect_ok"]
    assert abs(g[0][0]) < k["expect_abs_below"]
    assert sc.scale == 32768.0 and sc.consecutive_ok == 0


def test_grad_scaler_growth(oracle):
    sc = oracle.new_scaler()
    g = [np.ones(3, np.float32)]
    for i in range(1999):
        assert oracle.scaler_unscale_and_update(sc, g)
    assert sc.scale == 65536.0 and sc.consecutive_ok == 1999
    assert oracle.scaler_unscale_and_update(sc, g)
    assert sc.scale == 131072.0 and sc.consecutive_ok == 0


def test_group_optimizer_weight_decay_exclusion(oracle):
    k = KAT["group_optimizer_weight_decay_exclusion"]
    w, b = f64(k["params"][0]), f64(k["params"][1])
    oracle.sgd_step(w, f64(0.0), f64(0.0), k["lr"], 0.0, k["decay_wd"])  # "decay" group
    oracle.sgd_step(b, f64(0.0), f64(0.0), k["lr"], 0.0, 0.0)            # "no_decay" group
    assert abs(w[0] - k["expect"][0]) < k["tol"]
    assert abs(b[0] - k["expect"][1]) < k["tol"]


# ---- nabla-train/tests/trainer.rs ----------------------------------------------

def test_clip_grad_norm_scales(oracle):
    k = KAT["clip_grad_norm_scales"]
    g = [f64(k["grads"][0]), f64(k["grads"][1])]
    reported = oracle.clip_grad_norm(g, k["max_norm"])
    after = math.sqrt(sum(float(x[0]) ** 2 for x in g))
    assert abs(reported - k["expect_reported"]) < k["tol"]
    assert abs(after - k["expect_after"]) < k["tol"]


def test_clip_grad_norm_disabled_and_below(oracle):
    g = [f64(3.0), f64(4.0)]
    assert oracle.clip_grad_norm(g, 0.0) == 0.0 and g[0][0] == 3.0   # trainer.rs:501-503
    assert oracle.clip_grad_norm(g, -1.0) == 0.0
    assert oracle.clip_grad_norm(g, 5.0) == 5.0 and g[1][0] == 4.0    # norm == max: untouched
    z = [f64(0.0)]
    assert oracle.clip_grad_norm(z, 1.0) == 0.0 and z[0][0] == 0.0


def test_nan_policy_skip_drops_step(oracle):
    g = [f64(float("nan"))]
    assert oracle.has_non_finite(g)
    assert not oracle.has_non_finite([f64(1.0)])
    w0 = np.array([1.0], np.float32)
    mo = oracle.MixedOracle([w0], [oracle.AdamCfg(0.1, 0.9, 0.999, 1e-8, 0.0, 1)], use_scaler=False)
    ok, _ = mo.step([np.array([0x7FC0], np.uint16)])
    assert not ok and mo.step_count.value == KAT["nan_policy_skip_drops_step"]["expect_steps"]
    assert mo.master[0][0] == 1.0


# ---- oracle self-consistency ---------------------------------------------------

def test_oracle_matches_committed_vectors(oracle):
    """A change of compiler, libm or oracle source that moves one bit shows up here."""
    p0, grads = GOLD["p0"], GOLD["grads"]
    n = p0.size
    for name, kw in (("adam", dict(decoupled=False)), ("adamw", dict(decoupled=True, weight_decay=0.01))):
        p, m, v = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
        for t in range(10):
            oracle.adam_step(p, grads[t], m, v, 1e-3, step=t + 1, **kw)
        for a, key in ((p, "p"), (m, "m"), (v, "v")):
            assert np.array_equal(a.view(np.uint32), GOLD[f"{name}_{key}"].view(np.uint32)), (name, key)
    for name, kw in (("sgd", {}), ("sgd_mom", dict(momentum=0.9)), ("sgd_mom_wd", dict(momentum=0.9, weight_decay=0.01))):
        p, vel = p0.copy(), np.zeros(n, np.float32)
        for t in range(10):
            oracle.sgd_step(p, grads[t], vel, 0.1, **kw)
        assert np.array_equal(p.view(np.uint32), GOLD[f"{name}_p"].view(np.uint32))
        assert np.array_equal(vel.view(np.uint32), GOLD[f"{name}_vel"].view(np.uint32))


def test_mixed_oracle_matches_committed_vectors(oracle):
    mo = oracle.MixedOracle([GOLD["mixed_w0"]], [oracle.AdamCfg(3e-4, 0.9, 0.999, 1e-8, 0.1, 1)])
    for t in range(6):
        ok, norm = mo.step([GOLD["mixed_g16"][t].copy()], max_norm=1e-3)
        assert ok == bool(GOLD["mixed_ok"][t])
        assert norm == GOLD["mixed_norm"][t]
        assert mo.scaler.scale == GOLD["mixed_scale"][t]
    assert list(GOLD["mixed_ok"]) == [True, True, True, False, True, True]
    assert mo.step_count.value == 5 == GOLD["mixed_step_count"][0]
    assert np.array_equal(mo.p[0], GOLD["mixed_p16"])
    assert np.array_equal(mo.master[0].view(np.uint32), GOLD["mixed_master"].view(np.uint32))


def test_passes_shape_is_bit_identical_to_fused(oracle):
    """The reference-shaped 12-pass AdamW (timed as the CPU baseline) and the fused loop agree bit for bit."""
    rng = np.random.default_rng(1)
    n = 4099
    p1 = rng.normal(0, 1, n).astype(np.float32); p2 = p1.copy()
    m1 = np.zeros(n, np.float32); m2 = m1.copy(); v1 = m1.copy(); v2 = m1.copy()
    for t in range(1, 6):
        g = rng.normal(0, 1e-2, n).astype(np.float32)
        oracle.adam_step(p1, g, m1, v1, 1e-3, weight_decay=0.05, step=t, decoupled=True)
        oracle.adam_step(p2, g, m2, v2, 1e-3, weight_decay=0.05, step=t, decoupled=True, passes=True)
    for a, b in ((p1, p2), (m1, m2), (v1, v2)):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_no_fma_contraction(oracle):
    """y + a*x must round the product first (nabla-core/src/cpu/mod.rs:216-223)."""
    a = np.float32(1.0 + 2.0 ** -12)
    x = np.float32(1.0 + 2.0 ** -12)
    y = np.float32(-1.0)
    p = np.array([y], np.float32)
    oracle.sgd_step(p, np.array([x], np.float32), np.zeros(1, np.float32), float(-a))  # p + (-(-a))*x
    want = np.float32(y + np.float32(a * x))
    fused = np.float32(float(y) + float(a) * float(x))
    assert want != fused
    assert p[0] == want


def test_powi_is_square_and_multiply(oracle):
    def ref(a, b):
        r, e = 1.0, abs(b)
        while True:
            if e & 1:
                r *= a
            e >>= 1
            if e == 0:
                break
            a *= a
        return 1.0 / r if b < 0 else r
    for a in (0.9, 0.999, 0.1, 1.5):
        for b in (0, 1, 2, 3, 7, 100, 1000, 12345, -3):
            assert oracle.powi(a, b) == ref(a, b)
    assert oracle.powi(0.999, 1000) != 0.999 ** 1000 or True  # libm pow may differ; powi is what is pinned


def test_bf16_rounding_matches_independent_implementations(oracle):
    import ml_dtypes
    import torch
    rng = np.random.default_rng(7)
    bits = rng.integers(0, 2 ** 32, 200000, dtype=np.uint64).astype(np.uint32)
    bits = np.concatenate([bits, GOLD["bf16_edge_in"]])
    x = bits.view(np.float32)
    got = oracle.bf16_from_f32(x)
    finite_or_inf = ~np.isnan(x)
    ml = x.astype(ml_dtypes.bfloat16).view(np.uint16)
    th = torch.from_numpy(x.copy()).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got[finite_or_inf], ml[finite_or_inf])
    assert np.array_equal(got[finite_or_inf], th[finite_or_inf])
    # NaNs stay NaNs with the sign and upper payload kept and the quiet bit set (half 2.7.1)
    nan = np.isnan(x)
    assert np.all((got[nan] & 0x7F80) == 0x7F80) and np.all((got[nan] & 0x007F) != 0)
    assert np.array_equal(got[nan], ((bits[nan] >> 16) | 0x40).astype(np.uint16))
    assert np.array_equal(oracle.bf16_from_f32(GOLD["bf16_edge_in"].view(np.float32)), GOLD["bf16_edge_out"])
    # widening is exact
    h = rng.integers(0, 2 ** 16, 10000).astype(np.uint16)
    assert np.array_equal(oracle.bf16_to_f32(h).view(np.uint32), h.astype(np.uint32) << 16)


def test_powf_half_versus_sqrt_rate(oracle):
    """The kernels use a correctly rounded sqrt where the reference calls powf(x, 0.5); measure how often
    and by how much the host libm's powf differs so the 1e-5 budget is known to cover it."""
    import ctypes
    libm = ctypes.CDLL("libm.so.6")
    libm.powf.restype = ctypes.c_float
    libm.powf.argtypes = [ctypes.c_float, ctypes.c_float]
    rng = np.random.default_rng(3)
    x = np.exp(rng.uniform(-40, 10, 20000)).astype(np.float32)
    pw = np.array([libm.powf(float(v), 0.5) for v in x], dtype=np.float32)
    sq = np.sqrt(x)
    ulp = np.abs(pw.view(np.int32).astype(np.int64) - sq.view(np.int32).astype(np.int64))
    assert ulp.max() <= 1
    assert (ulp != 0).mean() < 0.05


def test_adam_and_adamw_against_an_independent_implementation(oracle):
    """The reference's tests do not pin Adam/AdamW values, so the restatement is cross-checked against a second,
    independently written implementation of the same published update (torch.optim, float64): the f64 oracle
    must agree to rounding noise and the f32 oracle to f32 precision, over 50 steps."""
    import torch
    rng = np.random.default_rng(42)
    n = 2000
    p0 = rng.normal(0, 0.5, n)
    grads = rng.normal(0, 1e-2, (50, n))
    for decoupled, cls, kw in ((False, torch.optim.Adam, {}), (True, torch.optim.AdamW, dict(weight_decay=0.05))):
        tp = torch.nn.Parameter(torch.tensor(p0, dtype=torch.float64))
        topt = cls([tp], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, **kw)
        p64, m64, v64 = p0.copy(), np.zeros(n), np.zeros(n)
        p32, m32, v32 = p0.astype(np.float32), np.zeros(n, np.float32), np.zeros(n, np.float32)
        for t in range(50):
            tp.grad = torch.tensor(grads[t])
            topt.step()
            oracle.adam_step(p64, grads[t].copy(), m64, v64, 1e-3, weight_decay=kw.get("weight_decay", 0.0), step=t + 1,
                             decoupled=decoupled)
            oracle.adam_step(p32, grads[t].astype(np.float32), m32, v32, 1e-3,
                             weight_decay=kw.get("weight_decay", 0.0), step=t + 1, decoupled=decoupled)
        want = tp.detach().numpy()
        assert np.max(np.abs(p64 - want)) < 1e-12
        assert np.max(np.abs(p32.astype(np.float64) - want)) < 5e-6


def test_sgd_momentum_against_an_independent_implementation(oracle):
    import torch
    rng = np.random.default_rng(43)
    n = 1000
    p0 = rng.normal(0, 0.5, n)
    grads = rng.normal(0, 1e-2, (30, n))
    tp = torch.nn.Parameter(torch.tensor(p0, dtype=torch.float64))
    topt = torch.optim.SGD([tp], lr=0.1, momentum=0.9, weight_decay=0.01)      # no dampening, no Nesterov
    p, vel = p0.copy(), np.zeros(n)
    for t in range(30):
        tp.grad = torch.tensor(grads[t])
        topt.step()
        oracle.sgd_step(p, grads[t].copy(), vel, 0.1, 0.9, 0.01)
    assert np.max(np.abs(p - tp.detach().numpy())) < 1e-12


def _powf_half(x32: np.ndarray) -> np.ndarray:
    """Elementwise libm powf(x, 0.5f) (what `Tensor::powf` reaches on the reference's CPU backend,
    nabla-core/src/cpu/mod.rs:264-272); numpy's own power() short-cuts an exponent of 0.5 to sqrt."""
    import ctypes
    libm = ctypes.CDLL("libm.so.6")
    libm.powf.restype = ctypes.c_float
    libm.powf.argtypes = [ctypes.c_float, ctypes.c_float]
    return np.array([libm.powf(float(v), 0.5) for v in x32], dtype=np.float32)


def test_f32_adamw_sgd_bit_for_bit_against_a_second_restatement(oracle):
    """A second restatement of AdamW / Adam / Sgd::step, written tensor op by tensor op from
    nabla-train/src/optim/alg.rs:120-149, 283-290, 393-413 in numpy float32 (every numpy f32 operation is one
    IEEE rounding, as every reference tensor op is; scale is x*s and axpy is y + (a*x) with the product rounded
    first, nabla-core/src/cpu/mod.rs:211-223).  It shares no code with the C oracle; the two must agree bit for
    bit, parameters and moments, over 40 steps including the f64 -> f32 narrowing of the step scalars."""
    f32 = np.float32
    rng = np.random.default_rng(7)
    n = 3000
    p0 = rng.normal(0, 0.5, n).astype(f32)
    p0[::97] = 0.0                                             # parameters that sit at zero
    grads = (rng.normal(0, 1e-2, (40, n)) * np.exp(rng.uniform(-8, 2, (40, n)))).astype(f32)
    grads[:, ::53] = 0.0                                       # elements that never receive a gradient
    lr, b1, b2, eps, wd = 3e-4, 0.9, 0.999, 1e-8, 0.1
    for decoupled in (True, False):
        p, m, v = p0.copy(), np.zeros(n, f32), np.zeros(n, f32)
        po, mo, vo = p0.copy(), np.zeros(n, f32), np.zeros(n, f32)
        for t in range(1, 41):
            g = grads[t - 1]
            # host scalars in f64, narrowed once each (alg.rs:120-135); powi is square-and-multiply
            bc1 = 1.0 - oracle.powi(b1, t)
            bc2 = 1.0 - oracle.powi(b2, t)
            ss, ibc2 = f32(lr / bc1), f32(1.0 / bc2)
            decay = f32(1.0) - f32(wd * lr)
            m = m * f32(b1)
            m = m + f32(1.0 - b1) * g
            v = v * f32(b2)
            gs = g * g
            v = v + f32(1.0 - b2) * gs
            d = _powf_half(v * ibc2) + f32(eps)
            u = (m * ss) / d
            if decoupled:
                p = p * decay
            p = p + f32(-1.0) * u
            assert p.dtype == m.dtype == v.dtype == f32
            oracle.adam_step(po, g.copy(), mo, vo, lr, b1, b2, eps, wd, step=t, decoupled=decoupled)
            assert np.array_equal(m.view(np.uint32), mo.view(np.uint32)), (decoupled, t, "m")
            assert np.array_equal(v.view(np.uint32), vo.view(np.uint32)), (decoupled, t, "v")
            assert np.array_equal(p.view(np.uint32), po.view(np.uint32)), (decoupled, t, "p")
    # Sgd::step with weight decay and momentum (alg.rs:393-413)
    p, vel = p0.copy(), np.zeros(n, f32)
    po, velo = p0.copy(), np.zeros(n, f32)
    for t in range(20):
        g = grads[t]
        ge = g + p * f32(0.01)
        vel = vel * f32(0.9) + ge
        p = p + (-f32(0.1)) * vel
        oracle.sgd_step(po, g.copy(), velo, 0.1, 0.9, 0.01)
        assert np.array_equal(p.view(np.uint32), po.view(np.uint32)) and np.array_equal(vel.view(np.uint32), velo.view(np.uint32))
