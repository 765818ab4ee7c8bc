"""GPU: the trainer tail (scaler -> nan policy -> accumulate -> set_lr -> clip -> step -> zero) versus the same
sequence composed from the oracle's pieces (nabla-train/src/trainer.rs:230-292)."""
import numpy as np
import pytest
import torch

from util import assert_close_rel, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nb():
    import nabla_b200
    return nabla_b200


def test_tail_matches_oracle_sequence(nb, oracle):
    rng = np.random.default_rng(3)
    sizes = [4097, 33, 1000]
    shapes = [(n,) for n in sizes]
    ps = [rng.normal(0, 0.02, n).astype(np.float32) for n in sizes]
    dp = [dev(a) for a in ps]
    opt = nb.AdamW(1e-3, shapes).weight_decay(0.05)
    sched = nb.LrSchedule.Cosine(2, 20, 1e-5)
    tail = nb.TrainerTail(opt, shapes, scaler=True, nan_policy=nb.GradNanPolicy.Skip, schedule=(sched, 1e-3),
                          grad_clip=0.05, grad_accum=2)
    # oracle side
    sc = oracle.new_scaler()
    m = [np.zeros(n, np.float32) for n in sizes]
    v = [np.zeros(n, np.float32) for n in sizes]
    buf, count, step, adam_t = None, 0, 0, 0
    applied = []
    for it in range(11):
        gs = [(rng.normal(0, 1e-2, n) * sc.scale).astype(np.float32) for n in sizes]
        if it == 4:
            gs[0][17] = np.inf
        dg = [dev(g) for g in gs]
        did = tail.on_backward(dp, dg)
        ok = oracle.scaler_unscale_and_update(sc, gs)
        o_did = False
        if not ok:
            buf, count = None, 0
        else:
            if buf is None:
                buf = [np.zeros(n, np.float32) for n in sizes]
            buf = [(b + g).astype(np.float32) for b, g in zip(buf, gs)]
            count += 1
            if count >= 2:
                lr = oracle.lr_at_step(0, 1e-3, step, warmup_steps=2, total_steps=20, min_lr=1e-5)
                norm = oracle.clip_grad_norm(buf, 0.05)
                adam_t += 1
                for i in range(3):
                    oracle.adam_step(ps[i], buf[i], m[i], v[i], lr, weight_decay=0.05, step=adam_t, decoupled=True)
                count, buf, step, o_did = 0, [np.zeros(n, np.float32) for n in sizes], step + 1, True
                assert abs(tail.last_grad_norm - norm) <= 1e-12 * norm
        assert did == o_did, it
        applied.append(did)
        assert tail.scaler.scale_factor() == sc.scale
    assert applied == [False, True, False, True, False, False, True, False, True, False, True]
    assert tail.state.step == step == 5 and opt.step_count() == 5
    gm, gv = opt.moments()
    for i in range(3):
        assert_close_rel(gm[i].numpy(), m[i], "m")
        assert_close_rel(gv[i].numpy(), v[i], "v")
        assert_close_rel(dp[i], ps[i], "p")


def test_nan_policy_skip_and_stop(nb):
    """nan_policy_skip_drops_step (nabla-train/tests/trainer.rs:148-169): NaN grads + Skip -> 0 steps."""
    p = [torch.ones(4, device="cuda")]
    g = [torch.full((4,), float("nan"), device="cuda")]
    tail = nb.TrainerTail(nb.Sgd(0.1, [(4,)]), [(4,)], nan_policy=nb.GradNanPolicy.Skip)
    assert tail.on_backward(p, g) is False and tail.state.step == 0 and float(p[0][0]) == 1.0
    tail = nb.TrainerTail(nb.Sgd(0.1, [(4,)]), [(4,)], nan_policy=nb.GradNanPolicy.Stop)
    with pytest.raises(nb.NonFiniteGradient, match="non-finite gradient"):
        tail.on_backward(p, g)
    tail = nb.TrainerTail(nb.Sgd(0.1, [(4,)]), [(4,)])            # no policy: the NaN goes through
    assert tail.on_backward(p, g) is True and torch.isnan(p[0]).all()


def test_accumulator_is_exact(nb):
    n = 3 * 4096 + 3
    a = torch.randn(n, device="cuda"); g = torch.randn(n, device="cuda")
    want = a + g
    acc = nb.GradAccumulator([(n,)])
    acc.add([a], [g])
    assert torch.equal(a, want)
    acc.zero([a])
    assert not a.any()
