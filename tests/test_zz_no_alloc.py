"""GPU: nbo_grad_norm_noalloc - the gradient norm / non-finite pass for callers that may not allocate
device memory (a stream capture open elsewhere in the process, an allocator that owns the whole device, a fixed memory
budget).  It must agree with the handle-based nbo_grad_norm, which allocates its own scratch, on two
calls in a row: the second call reuses the one fixed scratch array and sees whatever the first left there.

This file sorts after every other test file on purpose: a run that stops at the first failure has then
already run the rest of the suite."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ELEMS = 1 << 27


@pytest.fixture(scope="module")
def nb():
    import nabla_b200
    return nabla_b200


def noalloc_norm(nb, g: torch.Tensor, inv_scale: float = 1.0):
    """(norm, nonfinite) through the C ABI; only the two-double output buffer is caller memory."""
    lib = nb._lib.load()
    out = torch.full((2,), -1.0, dtype=torch.float64, device=g.device)
    prec = nb._lib.NBO_MIXED_BF16 if g.dtype == torch.bfloat16 else nb._lib.NBO_F32
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.nbo_grad_norm_noalloc(g.device.index, C.c_void_p(stream), C.c_void_p(g.data_ptr()), g.numel(), prec,
                                   C.c_float(inv_scale), C.c_void_p(out.data_ptr()))
    nb._lib.check(None, rc)
    sumsq, bad = out.cpu().tolist()
    return sumsq ** 0.5, bool(bad)


def handle_norm(nb, g: torch.Tensor):
    if g.dtype == torch.bfloat16:
        opt = nb.MixedAdamW.adamw(0.0, 0.0, [(g.numel(),)])
        h = opt._h
        norm, bad = C.c_double(), C.c_int32()
        h.check(h.lib.nbo_grad_norm(h.h, 1, nb._lib.ptr_array([g.data_ptr()]), C.byref(norm), C.byref(bad)))
        return norm.value, bool(bad.value)
    return nb.GradClipper([g]).grad_norm([g])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 5, 4096, 4097, 3 * 4096 + 7, 1 << 22])
def test_two_calls_in_a_row_match_the_allocating_entry_point(nb, dtype, n):
    torch.manual_seed(n)
    first = torch.randn(n, device="cuda").to(dtype)
    second = (torch.randn(n, device="cuda") * 3).to(dtype)
    for g in (first, second):                        # second call: scratch still holds the first call's data
        want, want_bad = handle_norm(nb, g)
        got, got_bad = noalloc_norm(nb, g)
        assert got_bad is False and want_bad is False
        assert abs(got - want) <= 1e-12 * want, (got, want)
    # and the same buffer twice gives the same bits
    assert noalloc_norm(nb, second) == noalloc_norm(nb, second)


def test_non_finite_flag_and_scale(nb):
    g = torch.randn(100000, device="cuda")
    assert noalloc_norm(nb, g)[1] is False
    g[77777] = float("inf")
    assert noalloc_norm(nb, g)[1] is True and handle_norm(nb, g)[1] is True
    g[77777] = 0.0
    assert noalloc_norm(nb, g)[1] is False           # the flag does not stick from the previous call
    a, _ = noalloc_norm(nb, g)
    b, _ = noalloc_norm(nb, g, inv_scale=0.5)
    assert abs(b - 0.5 * a) <= 1e-12 * a


def test_device_free_memory_is_unchanged_across_calls(nb):
    """The property in the name: after one warm-up call on the device (which looks up the scratch address and
    has the driver load the kernels of both precisions), calls in either precision leave the amount of
    free device memory exactly as it was - nothing is allocated, by the library or by the driver for it."""
    lib = nb._lib.load()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    g32 = torch.randn(1 << 20, device="cuda")
    g16 = torch.randn(1 << 20, device="cuda").to(torch.bfloat16)
    out = torch.zeros(2, dtype=torch.float64, device="cuda")
    dev = g32.device.index

    def call(g, prec):
        rc = lib.nbo_grad_norm_noalloc(dev, stream, C.c_void_p(g.data_ptr()), g.numel(), prec, C.c_float(1.0),
                                       C.c_void_p(out.data_ptr()))
        nb._lib.check(None, rc)

    call(g32, nb._lib.NBO_F32)                       # the one warm-up call, fp32 only
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(2):
        call(g16, nb._lib.NBO_MIXED_BF16)            # first bf16 call comes after the measurement started
        call(g32, nb._lib.NBO_F32)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    want = float(torch.linalg.vector_norm(g32.double()))
    assert abs(float(out[0]) ** 0.5 - want) <= 1e-12 * want


def test_unaligned_buffer(nb):
    for dtype, off in ((torch.float32, 1), (torch.float32, 3), (torch.bfloat16, 1), (torch.bfloat16, 3)):
        base = torch.randn(20000, device="cuda").to(dtype)
        g = base[off:off + 12345]
        want = float(torch.linalg.vector_norm(g.double()))
        got, bad = noalloc_norm(nb, g)
        assert not bad and abs(got - want) <= 1e-12 * want


def test_sizes_beyond_the_fixed_scratch_are_refused(nb):
    lib = nb._lib.load()
    g = torch.zeros(16, device="cuda")
    out = torch.zeros(2, dtype=torch.float64, device="cuda")
    rc = lib.nbo_grad_norm_noalloc(0, None, C.c_void_p(g.data_ptr()), MAX_ELEMS + 1, nb._lib.NBO_F32, C.c_float(1.0),
                                   C.c_void_p(out.data_ptr()))
    assert rc == nb._lib.NBO_ERR_INVALID
    msg = lib.nbo_last_error(None).decode()
    assert "exceed the fixed scratch" in msg and str(MAX_ELEMS) in msg
    rc = lib.nbo_grad_norm_noalloc(0, None, C.c_void_p(g.data_ptr()), 16, nb._lib.NBO_F32, C.c_float(1.0), None)
    assert rc == nb._lib.NBO_ERR_INVALID
    # the largest supported size works
    big = torch.ones(MAX_ELEMS, dtype=torch.bfloat16, device="cuda")
    got, bad = noalloc_norm(nb, big)
    assert not bad and got == float(MAX_ELEMS) ** 0.5
