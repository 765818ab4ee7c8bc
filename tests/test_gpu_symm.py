"""GPU (one device): the library's own symmetric allocator at world size 1 (CUDA virtual-memory allocation,
mapped and usable like any device buffer, released cleanly) and the plain SM copy used as the NVLink
yardstick.  The multi-rank set-up (descriptors over unix sockets, peer mappings, multicast binding) is
exercised by tests/zero1_worker.py native-peer / native-mcast under torch.distributed.run."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nb():
    import nabla_b200
    return nabla_b200


def test_world1_allocation_is_ordinary_device_memory(nb):
    from nabla_b200.zero1 import _device_view
    lib = nb._lib.load()
    n = (1 << 20) + 24                                      # not a multiple of the allocation granularity
    sh = C.c_void_p()
    nb._lib.check(None, lib.nbo_symm_alloc(0, 0, 1, 2 * n, None, 0, 1, 5.0, C.byref(sh)))
    local, mc = C.c_void_p(), C.c_void_p()
    peers = (C.c_void_p * 1)()
    nb._lib.check(None, lib.nbo_symm_pointers(sh, C.byref(local), peers, C.byref(mc)))
    assert local.value and peers[0] == local.value and not mc.value      # one rank: nothing to multicast to
    assert local.value % 16 == 0
    t = _device_view(local.value, n, 0)
    src = torch.randn(n, device="cuda").to(torch.bfloat16)
    t.copy_(src)
    assert torch.equal(t.view(torch.int16), src.view(torch.int16))
    # a sharded optimizer of world 1 steps on it like on any bucket
    z = nb.Zero1AdamW.adamw(1e-3, 0.0, [(n - 24,)], 0, 1)
    assert z.padded <= n
    pflat = t[:z.padded]
    before = pflat.clone()
    gflat = torch.full((z.padded,), 0.5, dtype=torch.bfloat16, device="cuda")
    z.init_master(pflat)
    assert z.step(pflat, gflat).applied
    assert not torch.equal(pflat[:n - 24].view(torch.int16), before[:n - 24].view(torch.int16))
    del z, pflat, t
    torch.cuda.synchronize()
    nb._lib.check(None, lib.nbo_symm_free(sh))


def test_allocator_argument_errors(nb):
    lib = nb._lib.load()
    sh = C.c_void_p()
    tok = (C.c_uint8 * 16)()
    nb._lib.check(None, lib.nbo_symm_token(tok))
    assert any(tok)                                                       # not all zero
    assert lib.nbo_symm_alloc(0, 2, 2, 4096, tok, 0, 1, 1.0, C.byref(sh)) == nb._lib.NBO_ERR_INVALID
    assert b"rank/world" in lib.nbo_last_error(None)
    assert lib.nbo_symm_alloc(0, 0, 1, 0, None, 0, 1, 1.0, C.byref(sh)) == nb._lib.NBO_ERR_INVALID
    assert lib.nbo_symm_alloc(0, 0, 2, 4096, None, 0, 1, 1.0, C.byref(sh)) == nb._lib.NBO_ERR_INVALID
    assert b"token" in lib.nbo_last_error(None)
    assert lib.nbo_symm_free(None) == nb._lib.NBO_OK


def test_a_rank_that_never_calls_in_ends_in_a_timeout(nb):
    """World 2 with nobody on the other side: the set-up gives up after the limit, releases what it made and
    leaves the device usable."""
    import time
    lib = nb._lib.load()
    tok = (C.c_uint8 * 16)()
    nb._lib.check(None, lib.nbo_symm_token(tok))
    sh = C.c_void_p()
    free0 = torch.cuda.mem_get_info()[0]
    t0 = time.time()
    rc = lib.nbo_symm_alloc(0, 0, 2, 1 << 22, tok, 7, 1, 1.5, C.byref(sh))
    assert rc == nb._lib.NBO_ERR_TIMEOUT and 1.0 < time.time() - t0 < 20.0
    assert b"timed out" in lib.nbo_last_error(None) and not sh.value
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free0 - (1 << 20)              # the 4 MiB allocation was given back
    assert float(torch.ones(8, device="cuda").sum()) == 8.0


def test_copy_probe_copies(nb):
    lib = nb._lib.load()
    n = (1 << 22) + 16                                                    # bytes, a multiple of 16
    src = torch.randint(-128, 127, (n,), dtype=torch.int8, device="cuda")
    dst = torch.zeros_like(src)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    nb._lib.check(None, lib.nbo_copy_probe(0, stream, C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()), n))
    torch.cuda.synchronize()
    assert torch.equal(dst, src)
    rc = lib.nbo_copy_probe(0, stream, C.c_void_p(dst.data_ptr() + 1), C.c_void_p(src.data_ptr()), 16)
    assert rc == nb._lib.NBO_ERR_INVALID and b"multiples of 16" in lib.nbo_last_error(None)
