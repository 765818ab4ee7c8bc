"""GPU: the asynchronous mixed step (state advanced on the device, no host round trip) is bit-identical to the
synchronous one, hands its state back and forth with the host correctly, and replays from a CUDA graph."""
import numpy as np
import pytest
import torch

from util import bf16_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nb():
    import nabla_b200
    return nabla_b200


SIZES = [4097, 130, 7, 20000]


def make(nb, growth_interval=4):
    names = ["w0", "norm1", "w2", "w3"]
    groups = [nb.ParamGroupConfig.adamw("no_decay", nb.ParamSelector.Any([nb.ParamMatch.Prefix("norm")]), 3e-4, 0.0)]
    opt = nb.MixedAdamW(names, [(n,) for n in SIZES], groups,
                        nb.ParamGroupConfig.adamw("decay", nb.ParamSelector.All(), 3e-4, 0.1))
    st = opt.scaler_state()
    st.growth_interval = growth_interval
    opt.load_scaler_state(st)
    return opt


def grads_for(step, scale, inject=False):
    g = torch.Generator(device="cuda").manual_seed(1000 + step)
    out = [(torch.randn(n, device="cuda", generator=g) * 1e-4 * scale).to(torch.bfloat16) for n in SIZES]
    if inject:
        out[3][777] = float("inf")
    return out


def same_state(a, b, pa, pb):
    for i in range(len(SIZES)):
        assert np.array_equal(bf16_bits(pa[i]), bf16_bits(pb[i])), f"params {i}"
        assert torch.equal(a.master(i), b.master(i))
        ma, va = a.moments(i); mb, vb = b.moments(i)
        assert torch.equal(ma, mb) and torch.equal(va, vb)
    sa, sb = a.scaler_state(), b.scaler_state()
    assert (sa.scale, sa.consecutive_ok) == (sb.scale, sb.consecutive_ok)
    assert a.step_count(0) == b.step_count(0) and a.step_count(1) == b.step_count(1)


def test_async_equals_sync_including_skips_growth_and_host_changes(nb):
    torch.manual_seed(0)
    p0 = [(torch.randn(n, device="cuda") * 0.02).to(torch.bfloat16) for n in SIZES]
    a, b = make(nb), make(nb)
    pa, pb = [x.clone() for x in p0], [x.clone() for x in p0]
    a.init_master_from_params(pa); b.init_master_from_params(pb)
    P = nb._lib.ptr_array
    scale = 65536.0
    for step in range(14):
        g = grads_for(step, scale, inject=step in (5, 6))
        if step == 9:                                   # a host-side change in the middle of asynchronous steps
            a.set_lr(1e-4); b.set_lr(1e-4)
        rb = b.step(pb, g, use_scaler=True, max_norm=5e-3)
        a.step_async(P([t.data_ptr() for t in pa]), P([t.data_ptr() for t in g]), use_scaler=True, max_norm=5e-3)
        scale = rb.loss_scale
        if step in (3, 6, 13):                          # hand the state back only now and then
            ra, done = a.collect()
            assert (ra.applied, ra.nonfinite, ra.loss_scale, ra.step_count) == (rb.applied, rb.nonfinite, rb.loss_scale, rb.step_count)
            assert ra.grad_norm == rb.grad_norm
            same_state(a, b, pa, pb)
    assert a.collect()[1] == 14 and b.step_count() == 12
    # back to the synchronous entry point on the same handle
    g = grads_for(99, scale)
    ra, rb = a.step(pa, g, use_scaler=True, max_norm=5e-3), b.step(pb, g, use_scaler=True, max_norm=5e-3)
    assert (ra.applied, ra.loss_scale, ra.grad_norm) == (rb.applied, rb.loss_scale, rb.grad_norm)
    same_state(a, b, pa, pb)


def test_async_step_replays_from_a_cuda_graph(nb):
    """One captured step, replayed: the step counter and loss scale advance on the device between replays."""
    torch.manual_seed(1)
    p0 = [(torch.randn(n, device="cuda") * 0.02).to(torch.bfloat16) for n in SIZES]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        a = make(nb, growth_interval=3)                  # the handle enqueues on `stream`
    b = make(nb, growth_interval=3)
    pa, pb = [x.clone() for x in p0], [x.clone() for x in p0]
    a.init_master_from_params(pa); b.init_master_from_params(pb)
    gbuf = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for n in SIZES]
    P = nb._lib.ptr_array
    parr, garr = P([t.data_ptr() for t in pa]), P([t.data_ptr() for t in gbuf])
    scale, step = 65536.0, 0

    def load(step, inject=False):
        for dst, src in zip(gbuf, grads_for(step, scale, inject)):
            dst.copy_(src)
        torch.cuda.synchronize()
    # one eager step first: it uploads the table and the state, so the captured step contains kernels only
    load(step)
    with torch.cuda.stream(stream):
        a.step_async(parr, garr, use_scaler=True, max_norm=5e-3)
    scale = b.step(pb, [x.clone() for x in gbuf], use_scaler=True, max_norm=5e-3).loss_scale
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    load(1)
    with torch.cuda.graph(graph, stream=stream):
        a.step_async(parr, garr, use_scaler=True, max_norm=5e-3)
    for step in range(1, 8):
        load(step, inject=step == 4)
        graph.replay()
        torch.cuda.synchronize()
        scale = b.step(pb, [x.clone() for x in gbuf], use_scaler=True, max_norm=5e-3).loss_scale
    ra, done = a.collect()
    assert done == 8 and ra.loss_scale == scale
    same_state(a, b, pa, pb)
    assert a.step_count() == 7                           # 8 steps, one skipped
