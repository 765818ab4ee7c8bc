"""GPU: checkpoint / resume in the reference's directory format: a resumed optimizer continues bit for bit."""
import numpy as np
import pytest
import torch

from util import bf16_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nb():
    import nabla_b200
    return nabla_b200


def test_adamw_resume_is_bit_exact_and_meta_matches_reference_layout(nb, tmp_path):
    ck = nb.checkpoint
    shapes = [(64, 33), (129,)]
    torch.manual_seed(0)
    p = [torch.randn(s, device="cuda") for s in shapes]
    grads = [[torch.randn(s, device="cuda") * 1e-2 for s in shapes] for _ in range(5)]
    a = nb.AdamW(1e-3, shapes).weight_decay(0.1)
    for t in range(3):
        a.step(p, grads[t])
    sched = ck.ScheduleState(1e-3, nb.LrSchedule.Cosine(10, 1000, 1e-5))
    ck.save_checkpoint(str(tmp_path), a, None, sched, ck.TrainState(2, 3, 1, 42),
                       named_params=[("w", p[0]), ("b", p[1])])
    meta = open(tmp_path / "meta.txt").read().splitlines()
    assert meta == ["version=1", "epoch=2", "step=3", "grad_accum=1", "rng.state=42", "optim.kind=adamw",
                    "optim.lr=0.001", "optim.beta1=0.9", "optim.beta2=0.999", "optim.eps=0.00000001",
                    "optim.weight_decay=0.1", "optim.momentum=0", "optim.step_count=3", "schedule.enabled=1",
                    "schedule.base_lr=0.001", "schedule.kind=cosine", "schedule.warmup_steps=10",
                    "schedule.total_steps=1000", "schedule.min_lr=0.00001", "scaler.enabled=0"]
    names = [n for n, _ in ck.load_tensors(str(tmp_path / "optim.nbla"))]
    assert names == ["m0", "m1", "v0", "v1"]
    # state tensors carry their parameter's (rows, cols): the reference installs a loaded tensor unchecked
    # and its next axpy_inplace asserts equal shapes (nabla-core/src/common/tensor/ops.rs:638-646)
    assert [t.shape for _, t in ck.load_tensors(str(tmp_path / "optim.nbla"))] == [(64, 33), (1, 129)] * 2
    assert [n for n, _ in ck.load_tensors(str(tmp_path / "params.nbla"))] == ["w", "b"]

    b = nb.AdamW(5.0, shapes)                       # wrong hyper-parameters on purpose: the checkpoint wins
    st, sc = ck.load_checkpoint(str(tmp_path), b)
    assert (st.epoch, st.step, st.grad_accum, st.rng_state) == (2, 3, 1, 42) and sc == sched
    assert b.step_count() == 3 and b.lr() == 1e-3
    q = [x.clone() for x in p]
    for t in range(3, 5):
        a.step(p, grads[t])
        b.step(q, grads[t])
    assert all(torch.equal(x, y) for x, y in zip(p, q))
    with pytest.raises(ValueError, match="optim kind mismatch"):
        ck.load_checkpoint(str(tmp_path), nb.Adam(1e-3, shapes))


def test_group_optimizer_and_sgd_velocity_names(nb, tmp_path):
    ck = nb.checkpoint
    names, sizes = ["embed.w", "l.w", "l.bias"], [300, 4097, 5]
    P, S, M = nb.ParamGroupConfig, nb.ParamSelector, nb.ParamMatch
    groups = [P.sgd("emb", S.Any([M.Prefix("embed")]), 0.5, 0.9, 0.0)]
    dflt = P.adamw("rest", S.All(), 1e-3, 0.01)
    p = [torch.randn(n, device="cuda") for n in sizes]
    g = [torch.randn(n, device="cuda") for n in sizes]
    a = nb.GroupOptimizer.from_named_params(list(zip(names, p)), groups, dflt)
    a.step(p, g); a.step(p, g)
    ck.save_checkpoint(str(tmp_path), a)
    assert [n for n, _ in ck.load_tensors(str(tmp_path / "optim.nbla"))] == ["g0.v0", "g1.m0", "g1.m1", "g1.v0", "g1.v1"]
    meta = ck.read_meta(str(tmp_path / "meta.txt"))
    assert meta["optim.group.count"] == "2" and meta["optim.group.0.kind"] == "sgd" and meta["optim.group.1.step_count"] == "2"
    assert meta["optim.group.0.momentum"] == "0.9" and meta["optim.group.0.name"] == "emb"
    b = nb.GroupOptimizer.from_named_params(list(zip(names, p)), groups, dflt)
    ck.load_checkpoint(str(tmp_path), b)
    q = [x.clone() for x in p]
    a.step(p, g); b.step(q, g)
    assert all(torch.equal(x, y) for x, y in zip(p, q))


def test_mixed_and_zero1_resume(nb, tmp_path):
    ck = nb.checkpoint
    sizes = [4099, 130, 7]
    shapes = [(n,) for n in sizes]
    torch.manual_seed(1)
    p = [(torch.randn(n, device="cuda") * 0.02).to(torch.bfloat16) for n in sizes]
    gs = [[(torch.randn(n, device="cuda") * 1e-4 * 65536).to(torch.bfloat16) for n in sizes] for _ in range(4)]
    a = nb.MixedAdamW.adamw(3e-4, 0.1, shapes)
    a.init_master_from_params(p)
    gs[1][0][5] = float("inf")
    for t in range(2):
        a.step(p, gs[t], use_scaler=True, max_norm=1.0)
    ck.save_checkpoint(str(tmp_path / "m"), a, scaler=a)
    meta = ck.read_meta(str(tmp_path / "m" / "meta.txt"))
    assert meta["scaler.enabled"] == "1" and meta["scaler.scale"] == "32768" and meta["optim.group.0.step_count"] == "1"
    b = nb.MixedAdamW.adamw(3e-4, 0.1, shapes)
    ck.load_checkpoint(str(tmp_path / "m"), b, scaler=b)
    assert b.scaler_state().scale == 32768.0 and b.step_count() == 1
    q = [x.clone() for x in p]
    for t in range(2, 4):
        ra = a.step(p, gs[t], use_scaler=True, max_norm=1.0)
        rb = b.step(q, gs[t], use_scaler=True, max_norm=1.0)
        assert (ra.applied, ra.loss_scale, ra.grad_norm) == (rb.applied, rb.loss_scale, rb.grad_norm)
    assert all(np.array_equal(bf16_bits(x), bf16_bits(y)) for x, y in zip(p, q))
    # the same file resumes a ZeRO-1 (world 1) optimizer: shards are cut from the per-tensor state
    z = nb.Zero1AdamW.adamw(3e-4, 0.1, shapes, 0, 1)
    ck.load_checkpoint(str(tmp_path / "m"), z, scaler=z)
    total = sum(sizes)
    pflat = torch.zeros(z.padded, dtype=torch.bfloat16, device="cuda")
    pflat[:total] = torch.cat([x.reshape(-1) for x in q])
    c = nb.MixedAdamW.adamw(3e-4, 0.1, shapes)
    ck.load_checkpoint(str(tmp_path / "m"), c, scaler=c)
    # both continue from the checkpoint with the same gradients
    q2 = [x.clone() for x in torch.split(pflat[:total].clone(), sizes)]
    gflat = torch.zeros(z.padded, dtype=torch.bfloat16, device="cuda")
    gflat[:total] = torch.cat([x.reshape(-1) for x in gs[2]])
    rz = z.step(pflat, gflat, use_scaler=True, max_norm=1.0)
    rc = c.step(q2, gs[2], use_scaler=True, max_norm=1.0)
    assert rz.applied == rc.applied and rz.loss_scale == rc.loss_scale
    assert np.array_equal(bf16_bits(pflat[:total]), bf16_bits(torch.cat(q2)))
    ck.save_checkpoint(str(tmp_path / "z"), z, scaler=z)
    assert [n for n, _ in ck.load_tensors(str(tmp_path / "z" / "optim.nbla"))][:4] == ["g0.m0", "g0.m1", "g0.m2", "g0.v0"]
