"""GPU: ZeRO-1.  world = 1 runs in-process and must reproduce the per-tensor mixed step bit for bit;
world >= 2 runs tests/zero1_worker.py under torch.distributed.run when the box has the GPUs."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from util import bf16_bits

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def nb():
    import nabla_b200
    return nabla_b200


@pytest.mark.parametrize("max_norm,use_scaler", [(0.0, False), (0.01, True)])
def test_world1_flat_bucket_equals_per_tensor_step(nb, max_norm, use_scaler):
    sizes = [5, 4096, 3, 70001, 1, 8192, 2]          # odd sizes: tensors start at every alignment in the bucket
    total = sum(sizes)
    shard, padded = nb.geometry(total, 1)
    torch.manual_seed(0)
    pflat = torch.zeros(padded, dtype=torch.bfloat16, device="cuda")
    pflat[:total] = (torch.randn(total, device="cuda") * 0.02).to(torch.bfloat16)
    gflat = torch.zeros(padded, dtype=torch.bfloat16, device="cuda")
    z = nb.Zero1AdamW.adamw(3e-4, 0.1, [(n,) for n in sizes], 0, 1)
    assert z.shard_range() == (0, padded, len(sizes))
    z.init_master(pflat)
    # the same thing with one pointer per tensor
    offs = np.cumsum([0] + sizes)
    ps = [pflat[offs[i]:offs[i + 1]].clone() for i in range(len(sizes))]
    m = nb.MixedAdamW.adamw(3e-4, 0.1, [(n,) for n in sizes])
    m.init_master_from_params(ps)
    for t in range(4):
        scale = 65536.0 if use_scaler else 1.0
        gflat[:total] = (torch.randn(total, device="cuda") * 1e-4 * scale).to(torch.bfloat16)
        if t == 2 and use_scaler:
            gflat[4100] = float("inf")
        gs = [gflat[offs[i]:offs[i + 1]].clone() for i in range(len(sizes))]
        r1 = z.step(pflat, gflat, use_scaler=use_scaler, max_norm=max_norm)
        r2 = m.step(ps, gs, use_scaler=use_scaler, max_norm=max_norm)
        assert (r1.applied, r1.loss_scale, r1.step_count) == (r2.applied, r2.loss_scale, r2.step_count)
        if max_norm > 0 and r1.applied:
            assert abs(r1.grad_norm - r2.grad_norm) <= 1e-13 * r2.grad_norm
    master = z.state_shard(2)
    for i in range(len(sizes)):
        assert np.array_equal(bf16_bits(pflat[offs[i]:offs[i + 1]]), bf16_bits(ps[i])), f"tensor {i}"
        assert torch.equal(master[offs[i]:offs[i + 1]], m.master(i))
    assert not pflat[total:].float().abs().sum().item()      # padding is never written


def test_bucket_validation(nb):
    z = nb.Zero1AdamW.adamw(1e-3, 0.0, [(100,)], 0, 1)
    good = torch.zeros(z.padded, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        z.step(good[:-8], good)
    L = nb._lib
    res = L.StepResult()
    import ctypes as C
    rc = z._h.lib.nbo_zero1_step(z._h.h, C.c_void_p(good.data_ptr() + 2), C.c_void_p(good.data_ptr()), 0, 0, 0.0,
                                 C.byref(res))
    assert rc == L.NBO_ERR_INVALID and b"16-byte aligned" in z._h.lib.nbo_last_error(z._h.h)
    with pytest.raises(L.NablaOptimError, match="rank/world"):
        nb.Zero1AdamW.adamw(1e-3, 0.0, [(100,)], 2, 2)


@pytest.mark.parametrize("mode", ["nccl", "peer", "mcast", "native-peer", "native-mcast"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_gpu_matches_single_gpu(world, mode):
    """nccl: collectives around the update; peer / mcast: collectives fused into the kernels; native-*: the same
    on buckets the library allocates itself (no framework symmetric memory)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = 29500 + world + {"nccl": 0, "peer": 20, "mcast": 40, "native-peer": 60, "native-mcast": 80}[mode]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "zero1_worker.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    if "ZERO1_WORKER_SKIP" in r.stdout:
        pytest.skip(r.stdout.strip().splitlines()[-1])
    assert "ZERO1_WORKER_OK" in r.stdout


@pytest.mark.parametrize("mode", ["peer", "mcast"])
@pytest.mark.parametrize("world", [2, 4])
def test_host_streamed_sharded_step_equals_the_fused_step(world, mode):
    """nbo_zero1_step_host at world > 1: sliced copy-in / barrier / fused kernel / copy-out pipeline, bit for bit
    the result of nbo_zero1_step_fused (tests/zero1_host_worker.py)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = 29600 + world + (20 if mode == "mcast" else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "zero1_host_worker.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    if "ZERO1_HOST_SKIP" in r.stdout:
        pytest.skip(r.stdout.strip().splitlines()[-1])
    assert "ZERO1_HOST_OK" in r.stdout


def test_rank_that_never_arrives_times_out(nb):
    """Communicator set-up with a peer that never calls in: NBO_ERR_TIMEOUT after the limit, context intact."""
    import ctypes as C
    import time
    L = nb._lib
    uid = (C.c_uint8 * 128)()
    L.check(None, L.load().nbo_zero1_unique_id(uid))
    t0 = time.time()
    with pytest.raises(L.NablaOptimError) as ei:
        nb.Zero1AdamW.adamw(1e-3, 0.0, [(1000,)], 0, 2, bytes(uid), timeout_s=2.0)
    assert ei.value.code == L.NBO_ERR_TIMEOUT and "did not arrive" in ei.value.message
    assert 1.5 < time.time() - t0 < 30.0
    p = torch.ones(100, device="cuda")
    nb.Sgd(0.1, [(100,)]).step([p], [torch.ones(100, device="cuda")])
    assert abs(float(p[0]) - 0.9) < 1e-6


def test_rank_leaving_between_steps_ends_in_a_timeout():
    """Only the NCCL path is exercised: its buckets are ordinary device memory and NVLS is off, so the
    rank that leaves holds no NVLink multicast binding.  Symmetric-memory buckets (the fused path) are
    always bound to a multicast object where the fabric offers one, and a rank must not end in that state."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29580",
           os.path.join(ROOT, "tests", "zero1_leave_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert "ZERO1_LEAVE_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
