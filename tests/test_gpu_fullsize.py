"""GPU: the benchmark configurations at their full sizes, checked through properties that do not need a CPU run
of the whole thing: independence of the tensor partition (elementwise work must not care how a buffer is cut
into tensors), cast exactness over every element, all-or-nothing skip, and the oracle on seeded slices."""
import math

import numpy as np
import pytest
import torch

from util import assert_close_rel, bf16_bits, bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nb():
    import nabla_b200
    return nabla_b200


def carve(flat, sizes, align):
    out, off = [], 0
    for n in sizes:
        out.append(flat[off:off + n])
        off += (n + align - 1) // align * align
    return out


def test_fragmentation_10000_tensors_equals_one_big_tensor(nb, oracle):
    """10,000 fp32 tensors, sizes log-uniform in [1, 2^20]: one SGD-momentum and one AdamW step give, element for
    element, the bits of the same step over the same memory bound as ONE tensor; a sample of tensors is also
    checked against the oracle."""
    rng = np.random.default_rng(0)
    sizes = [int(x) for x in np.floor(np.exp(rng.uniform(0.0, math.log(2 ** 20), 10000)))]
    total = sum((n + 3) // 4 * 4 for n in sizes)
    gen = torch.Generator(device="cuda").manual_seed(5)
    for kind in ("sgdm", "adamw"):
        p1 = torch.empty(total, device="cuda").normal_(0, 1, generator=gen)
        g = torch.empty(total, device="cuda").normal_(0, 1e-3, generator=gen)
        p2 = p1.clone()
        shapes = [(n,) for n in sizes]
        if kind == "sgdm":
            many, one = nb.Sgd(0.1, shapes).momentum(0.9), nb.Sgd(0.1, [(total,)]).momentum(0.9)
        else:
            many, one = nb.AdamW(1e-3, shapes).weight_decay(0.01), nb.AdamW(1e-3, [(total,)]).weight_decay(0.01)
        ps, gs = carve(p1, sizes, 4), carve(g, sizes, 4)
        sample = [0, 1, 17, 4242, 9999] + [int(i) for i in rng.integers(0, 10000, 10)]
        before = {i: (ps[i].cpu().numpy().copy(), gs[i].cpu().numpy().copy()) for i in sample}
        many.step(ps, gs)
        one.step([p2], [g])
        # the padding between tensors is untouched by `many` and updated by `one`: compare tensor by tensor
        mism = 0
        for a, b in zip(ps, carve(p2, sizes, 4)):
            mism += int((a.view(torch.int32) != b.view(torch.int32)).sum())
        assert mism == 0
        tensors, chunks, uploads = many._h.table_info()
        assert tensors == 10000 and uploads == 1 and many._h.launch_count() == 1
        for i in sample:
            p, gg = before[i]
            s0, s1 = np.zeros_like(p), np.zeros_like(p)
            if kind == "sgdm":
                oracle.sgd_step(p, gg, s0, 0.1, 0.9, 0.0)
                assert np.array_equal(bits(ps[i]), bits(p))
            else:
                oracle.adam_step(p, gg, s0, s1, 1e-3, weight_decay=0.01, step=1, decoupled=True)
                assert_close_rel(ps[i], p, f"tensor {i}")
        del p1, p2, g, ps, gs, many, one
        torch.cuda.empty_cache()


def gpt2_shapes():
    s = [(50257, 768), (1024, 768)]
    for _ in range(12):
        s += [(768,), (768,), (768,), (768,), (768, 2304), (2304,), (768, 768), (768,), (768, 3072), (3072,),
              (3072, 768), (768,)]
    return s + [(768,), (768,)]


def test_gpt2_adam_full_size_against_oracle(nb, oracle):
    """All 148 tensors / 124,439,808 params of the GPT-2-small list, 3 Adam steps, against the oracle in full."""
    shapes = gpt2_shapes()
    assert len(shapes) == 148 and sum(a * (b[0] if b else 1) for a, *b in shapes) == 124439808
    rng = np.random.default_rng(1)
    ps = [(rng.standard_normal(s, dtype=np.float32) * np.float32(0.02)) for s in shapes]
    dp = [torch.from_numpy(a).cuda() for a in ps]
    opt = nb.Adam(1e-3, shapes)
    ms = [np.zeros(a.size, np.float32) for a in ps]
    vs = [np.zeros(a.size, np.float32) for a in ps]
    for t in range(1, 4):
        gs = [(rng.standard_normal(s, dtype=np.float32) * np.float32(1e-4)) for s in shapes]
        opt.step(dp, [torch.from_numpy(g).cuda() for g in gs])
        for p, g, m, v in zip(ps, gs, ms, vs):
            oracle.adam_step(p.reshape(-1), g.reshape(-1), m, v, 1e-3, step=t, decoupled=False)
    gm, gv = opt.moments()
    exact = 0
    for i in range(len(shapes)):
        assert np.array_equal(bits(gm[i].numpy()), bits(ms[i])) and np.array_equal(bits(gv[i].numpy()), bits(vs[i]))
        assert_close_rel(dp[i].reshape(-1), ps[i].reshape(-1), f"tensor {i}")
        exact += int((bits(dp[i]).ravel() == bits(ps[i]).ravel()).sum())
    print(f"gpt2 full size: {100.0 * exact / 124439808:.4f}% of params bit-exact after 3 steps")


def llama_shapes(d, layers, ffn, vocab, kv):
    s = [(vocab, d)]
    for _ in range(layers):
        s += [(d, d), (d, kv), (d, kv), (d, d), (d, ffn), (d, ffn), (ffn, d), (d,), (d,)]
    return s + [(d,), (vocab, d)]


def test_llama1b_mixed_full_size_properties(nb, oracle):
    """1,204,881,408 params, bf16 p/g + fp32 master/m/v, loss scale 2^16, clip 1.0: an injected +inf skips the
    whole step and changes no byte; after applied steps every bf16 param is the RNE cast of its master; a slice
    of one tensor follows the oracle."""
    shapes = llama_shapes(2048, 16, 8192, 32000, 2048)
    sizes = [int(np.prod(s)) for s in shapes]
    total = sum(sizes)
    assert total == 1204881408 and len(shapes) == 147
    gen = torch.Generator(device="cuda").manual_seed(3)
    pflat = torch.empty(total, dtype=torch.bfloat16, device="cuda")
    gflat = torch.empty(total, dtype=torch.bfloat16, device="cuda")
    for off in range(0, total, 1 << 27):
        m = min(1 << 27, total - off)
        pflat[off:off + m] = torch.randn(m, device="cuda", generator=gen) * 0.02
        gflat[off:off + m] = torch.randn(m, device="cuda", generator=gen) * (1e-4 * 65536)
    ps, gs = carve(pflat, sizes, 1), carve(gflat, sizes, 1)
    opt = nb.MixedAdamW.adamw(3e-4, 0.1, shapes)
    opt.init_master_from_params(ps)
    pa, ga = nb._lib.ptr_array([t.data_ptr() for t in ps]), nb._lib.ptr_array([t.data_ptr() for t in gs])
    # oracle twin for a slice of tensor 5 (a 2048 x 8192 matrix)
    T, LO, N = 5, 1234567, 200000
    w0 = ps[T].reshape(-1)[LO:LO + N].float().cpu().numpy()
    g16 = bf16_bits(gs[T].reshape(-1)[LO:LO + N])
    m_o, v_o = np.zeros(N, np.float32), np.zeros(N, np.float32)

    r1 = opt.step_ptrs(pa, ga, use_scaler=True, max_norm=1.0)
    assert r1.applied and r1.loss_scale == 65536.0 and r1.step_count == 1
    want_norm = float(torch.linalg.vector_norm(gflat.float() / 65536.0, dtype=torch.float64))
    assert abs(r1.grad_norm - want_norm) <= 1e-9 * want_norm
    clip = np.float32(1.0 / r1.grad_norm) if r1.grad_norm > 1.0 else np.float32(1.0)
    g_o = (oracle.bf16_to_f32(g16) * np.float32(1.0 / 65536.0)).astype(np.float32)
    g_o = (g_o * clip).astype(np.float32) if r1.grad_norm > 1.0 else g_o
    oracle.adam_step(w0, g_o, m_o, v_o, 3e-4, weight_decay=0.1, step=1, decoupled=True)
    got_w = opt.master(T).numpy()[LO:LO + N]
    assert_close_rel(got_w, w0, "master slice")
    assert np.array_equal(bf16_bits(ps[T].reshape(-1)[LO:LO + N]), oracle.bf16_from_f32(got_w))

    # every bf16 param is the round-to-nearest-even cast of its fp32 master (torch's cast is RNE for finite values)
    for i in (0, 5, 9, 146):
        master = opt._h.state_export(i, 2, sizes[i]).cuda()
        assert torch.equal(master.to(torch.bfloat16).view(torch.int16), ps[i].reshape(-1).view(torch.int16))
        del master
    # all-or-nothing skip: one +inf anywhere -> nothing but the scaler changes
    digest_p = pflat.view(torch.int16).to(torch.int64).sum().item()
    m_before = opt._h.state_export(146, 0, sizes[146]).clone()
    gs[100].view(-1)[12345] = float("inf")
    r2 = opt.step_ptrs(pa, ga, use_scaler=True, max_norm=1.0)
    assert not r2.applied and r2.nonfinite and r2.loss_scale == 32768.0 and r2.step_count == 1
    assert pflat.view(torch.int16).to(torch.int64).sum().item() == digest_p
    assert torch.equal(opt._h.state_export(146, 0, sizes[146]), m_before)


def test_single_tensor_beyond_2_to_32_elements(nb, oracle):
    """One bf16 tensor of 2^32 + 4101 elements (69 GB with its state): offsets need 64 bits, the chunk list has
    more than a million entries and ends in a partial chunk with a tail.  Slices around 0, 2^31, 2^32 and the
    end follow the oracle; untouched guard elements past the end stay untouched."""
    n = (1 << 32) + 4101
    free, _ = torch.cuda.mem_get_info()
    if free < 80 * (1 << 30):
        pytest.skip("needs 80 GB of free device memory")
    guard = 64
    p = torch.empty(n + guard, dtype=torch.bfloat16, device="cuda")
    g = torch.empty(n + guard, dtype=torch.bfloat16, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(9)
    for off in range(0, n + guard, 1 << 28):
        m = min(1 << 28, n + guard - off)
        p[off:off + m] = torch.randn(m, device="cuda", generator=gen) * 0.02
        g[off:off + m] = torch.randn(m, device="cuda", generator=gen) * 1e-3
    p_guard = p[n:].clone()
    opt = nb.MixedAdamW.adamw(1e-3, 0.1, [(n,)])
    pv, gv = p[:n], g[:n]
    opt.init_master_from_params([pv])
    windows = [(0, 3000), ((1 << 31) - 1500, 3000), ((1 << 32) - 2000, 4000), (n - 3000, 3000)]
    before = [(pv[a:a + k].float().cpu().numpy(), gv[a:a + k].float().cpu().numpy()) for a, k in windows]
    res = opt.step([pv], [gv], use_scaler=False, max_norm=0.0)
    assert res.applied and opt.step_count() == 1
    assert opt._h.table_info()[1] == (n + 4095) // 4096
    for (a, k), (w0, g0) in zip(windows, before):
        w, m, v = w0.copy(), np.zeros(k, np.float32), np.zeros(k, np.float32)
        oracle.adam_step(w, g0, m, v, 1e-3, weight_decay=0.1, step=1, decoupled=True)
        got = bf16_bits(pv[a:a + k])
        want = oracle.bf16_from_f32(w)
        assert float((got == want).mean()) > 0.999, f"window at {a}"
        assert np.abs(oracle.bf16_to_f32(got) - oracle.bf16_to_f32(want)).max() <= np.abs(w).max() * 2 ** -7
    assert torch.equal(p[n:].view(torch.int16), p_guard.view(torch.int16))
    # the norm pass over the same tensor: 64-bit offsets there too
    import ctypes as C
    a_, b_ = C.c_double(), C.c_int32()
    opt._h.check(opt._h.lib.nbo_grad_norm(opt._h.h, 1, nb._lib.ptr_array([gv.data_ptr()]), C.byref(a_), C.byref(b_)))
    want = 0.0
    for off in range(0, n, 1 << 28):
        m = min(1 << 28, n - off)
        want += float((gv[off:off + m].double() ** 2).sum())
    assert not b_.value and abs(a_.value - want ** 0.5) <= 1e-11 * want ** 0.5


def test_mixed_64m_element_slice_20_steps_against_oracle(nb, oracle):
    """A 64 Mi-element tensor (the size class of the large matrices of the 8 G-parameter list) through 20
    mixed-precision steps with loss scaling, an injected overflow and clipping, against the oracle element
    for element: decisions and loss scale exact, masters / m / v within 1e-5, bf16 params = cast of masters."""
    n = (1 << 26) + 3
    gen = torch.Generator(device="cuda").manual_seed(11)
    w0 = (torch.randn(n, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    p = w0.clone()
    opt = nb.MixedAdamW.adamw(3e-4, 0.1, [(n,)])
    opt.init_master_from_params([p])
    mo = oracle.MixedOracle([w0.float().cpu().numpy()], [oracle.AdamCfg(3e-4, 0.9, 0.999, 1e-8, 0.1, 1)])
    for step in range(20):
        g = (torch.randn(n, device="cuda", generator=gen) * (1e-4 * mo.scaler.scale)).to(torch.bfloat16)
        if step == 7:
            g[n - 2] = float("-inf")
        res = opt.step([p], [g], use_scaler=True, max_norm=0.5)
        ok, norm = mo.step([bf16_bits(g)], max_norm=0.5)
        assert res.applied == ok and res.loss_scale == mo.scaler.scale and res.step_count == mo.step_count.value
        if ok:   # the reference's serial f64 sum over 6.7e7 squares carries ~1e-12 of rounding itself
            assert abs(res.grad_norm - norm) <= 1e-10 * norm
    assert opt.step_count() == 19
    gw = opt.master(0).numpy()
    gm, gv = opt.moments(0)
    assert_close_rel(gw, mo.master[0], "master")
    assert_close_rel(gm.numpy(), mo.m[0], "m")
    assert_close_rel(gv.numpy(), mo.v[0], "v")
    assert np.array_equal(bf16_bits(p), oracle.bf16_from_f32(gw))
    same = float((bf16_bits(p) == mo.p[0]).mean())
    print(f"64 Mi slice, 19 applied steps: {100 * same:.4f}% of bf16 params equal the oracle's")
    assert same > 0.999
