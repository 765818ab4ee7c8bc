"""GPU: the host-streamed mixed-precision step (nbo_step_mixed_host / nbo_zero1_step_host) against the
resident step (nbo_step_mixed) on the same seeded data.  The two run the same kernels over the same
chunk list, so parameters, masters, m, v, skip decisions and the loss scale must be bit-identical;
what is under test is the slicing (every element copied in before its update and copied out after it,
nothing copied twice or left behind) and the skip path (a skipped step writes nothing to the host)."""
import numpy as np
import pytest
import torch

from util import bf16_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nb():
    import nabla_b200
    return nabla_b200


SIZES = [1, 5, 4096, 4097, 3, 8191, 12289, 100003, 2, 40960]


def two_group_opt(nb, sizes, grad_dtype=torch.bfloat16):
    names = [("norm%d" % i if i % 3 == 0 else "w%d" % i) for i in range(len(sizes))]
    groups = [nb.ParamGroupConfig.adamw("no_decay", nb.ParamSelector.Any([nb.ParamMatch.Prefix("norm")]), 3e-4, 0.0)]
    return nb.MixedAdamW(names, [(n,) for n in sizes], groups,
                         nb.ParamGroupConfig.adamw("decay", nb.ParamSelector.All(), 3e-4, 0.1),
                         grad_dtype=grad_dtype)


def carve(sizes, dtype, offset):
    """Device tensors cut from one allocation; `offset` = 1 leaves every tensor without 8/16-byte alignment."""
    out = []
    for n in sizes:
        base = torch.zeros(n + 16, dtype=dtype, device="cuda")
        out.append(base[offset:offset + n])
    return out


@pytest.mark.parametrize("offset,slice_elems,max_norm,use_scaler,grad_dtype", [
    (0, 8192, 0.0, False, torch.bfloat16),       # pipelined path, many 2-chunk slices
    (1, 4096, 0.0, False, torch.bfloat16),       # rows without an aligned body, 1-chunk slices
    (0, 20000, 0.01, True, torch.bfloat16),      # decision first, then update + copy-out
    (0, 0, 0.0, True, torch.bfloat16),           # default slice (one slice per group), flag-only pass
    (0, 12288, 0.01, False, torch.float32),      # fp32 gradients
])
def test_host_streamed_step_equals_resident_step(nb, offset, slice_elems, max_norm, use_scaler, grad_dtype):
    torch.manual_seed(3)
    a, b = two_group_opt(nb, SIZES, grad_dtype), two_group_opt(nb, SIZES, grad_dtype)
    p_res = carve(SIZES, torch.bfloat16, offset)
    g_res = carve(SIZES, grad_dtype, offset)
    p_dev = carve(SIZES, torch.bfloat16, offset)
    g_dev = carve(SIZES, grad_dtype, offset)
    for p in p_res:
        p.copy_((torch.randn(p.numel(), device="cuda") * 0.02).to(torch.bfloat16))
    a.init_master_from_params(p_res)
    b.init_master_from_params(p_res)
    p_host = [torch.full((n,), 7.0, dtype=torch.bfloat16).pin_memory() for n in SIZES]   # sentinel
    g_host = [torch.zeros(n, dtype=grad_dtype).pin_memory() for n in SIZES]
    for t in range(4):
        scale = 65536.0 if use_scaler else 1.0
        for i, n in enumerate(SIZES):
            g = (torch.randn(n, device="cuda") * 1e-4 * scale).to(grad_dtype)
            if t == 0 and use_scaler and i == 7:
                g[n // 2] = float("inf")
            g_res[i].copy_(g)
            g_host[i].copy_(g)
            g_dev[i].fill_(123.0)                    # staging holds rubbish before the call
        torch.cuda.synchronize()
        r1 = a.step(p_res, g_res, use_scaler=use_scaler, max_norm=max_norm)
        r2 = b.step_host(p_dev, g_dev, p_host, g_host, use_scaler=use_scaler, max_norm=max_norm,
                         slice_elems=slice_elems)
        assert (r1.applied, r1.nonfinite, r1.loss_scale, r1.step_count) == \
               (r2.applied, r2.nonfinite, r2.loss_scale, r2.step_count)
        assert r1.grad_norm == r2.grad_norm
        if t == 0 and use_scaler:
            assert not r2.applied
            for ph in p_host:                        # a skipped step copies nothing out
                assert bool((ph.float() == 7.0).all())
            continue
        for i in range(len(SIZES)):
            assert np.array_equal(bf16_bits(p_host[i]), bf16_bits(p_res[i])), f"step {t} tensor {i}"
    for i in range(len(SIZES)):
        assert torch.equal(a.master(i), b.master(i))
        for which in (0, 1):
            assert torch.equal(a._h.state_export(i, which, SIZES[i]), b._h.state_export(i, which, SIZES[i]))


def test_host_streamed_step_on_a_world1_zero1_handle(nb):
    sizes = [5, 4096, 3, 70001, 1, 8192, 2]
    total = sum(sizes)
    shard, padded = nb.geometry(total, 1)
    torch.manual_seed(0)
    offs = np.cumsum([0] + sizes)
    init = (torch.randn(total, device="cuda") * 0.02).to(torch.bfloat16)
    p1 = torch.zeros(padded, dtype=torch.bfloat16, device="cuda"); p1[:total] = init
    p2 = p1.clone()
    g1 = torch.zeros(padded, dtype=torch.bfloat16, device="cuda")
    g2 = torch.zeros(padded, dtype=torch.bfloat16, device="cuda")
    z1 = nb.Zero1AdamW.adamw(3e-4, 0.1, [(n,) for n in sizes], 0, 1)
    z2 = nb.Zero1AdamW.adamw(3e-4, 0.1, [(n,) for n in sizes], 0, 1)
    z1.init_master(p1)
    z2.init_master(p2)
    p_host = [torch.zeros(n, dtype=torch.bfloat16).pin_memory() for n in sizes]
    g_host = [torch.zeros(n, dtype=torch.bfloat16).pin_memory() for n in sizes]
    pa = nb._lib.ptr_array([t.data_ptr() for t in p_host])
    ga = nb._lib.ptr_array([t.data_ptr() for t in g_host])
    for t in range(3):
        g = (torch.randn(total, device="cuda") * 1e-4).to(torch.bfloat16)
        g1[:total] = g
        for i in range(len(sizes)):
            g_host[i].copy_(g[offs[i]:offs[i + 1]])
        g2.fill_(55.0)
        torch.cuda.synchronize()
        r1 = z1.step(p1, g1, max_norm=0.01 if t == 1 else 0.0)
        r2 = z2.step_host_ptrs(p2.data_ptr(), g2.data_ptr(), pa, ga, max_norm=0.01 if t == 1 else 0.0,
                               slice_elems=8192)
        assert (r1.applied, r1.step_count, r1.grad_norm) == (r2.applied, r2.step_count, r2.grad_norm)
        for i in range(len(sizes)):
            assert np.array_equal(bf16_bits(p_host[i]), bf16_bits(p1[offs[i]:offs[i + 1]])), f"step {t} tensor {i}"
    assert torch.equal(z1.state_shard(2), z2.state_shard(2))
    assert torch.equal(z1.state_shard(0), z2.state_shard(0))


def test_host_step_argument_errors(nb):
    opt = nb.MixedAdamW.adamw(1e-3, 0.0, [(64,)])
    p = [torch.zeros(64, dtype=torch.bfloat16, device="cuda")]
    g = [torch.zeros(64, dtype=torch.bfloat16, device="cuda")]
    opt.init_master_from_params(p)
    with pytest.raises(ValueError):
        opt.step_host(p, g, [torch.zeros(63, dtype=torch.bfloat16)], [torch.zeros(64, dtype=torch.bfloat16)])
    null = nb._lib.ptr_array([0])
    with pytest.raises(nb._lib.NablaOptimError):
        opt.step_host_ptrs(nb._lib.ptr_array([p[0].data_ptr()]), nb._lib.ptr_array([g[0].data_ptr()]), null, null)
    f32 = nb.AdamW(1e-3, [(64,)])
    with pytest.raises(nb._lib.NablaOptimError):
        f32._h.check(f32._h.lib.nbo_step_mixed_host(f32._h.h, 1, null, null, null, null, 0, 0, 0.0, None))
    # the handle stays usable
    ph = [torch.zeros(64, dtype=torch.bfloat16).pin_memory()]
    gh = [torch.ones(64, dtype=torch.bfloat16).pin_memory()]
    r = opt.step_host(p, g, ph, gh, use_scaler=False)
    assert r.applied and r.step_count == 1
    assert float(ph[0].float().abs().sum()) > 0
