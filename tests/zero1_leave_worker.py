"""Failure detection of the sharded step, made on the host: after two good steps rank 1 leaves between steps
(nothing of its own in flight); rank 0's next step must end with NBO_ERR_TIMEOUT within the configured limit,
leave the CUDA context usable, and refuse further sharded steps.  Launched by tests/test_gpu_zero1.py on two
GPUs with NVLS off.  The buckets are ordinary device memory and the collectives go through NCCL, so no
NVLink multicast object is bound anywhere when the rank leaves (symmetric-memory buckets would be).
"""
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import nabla_b200 as nb  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    sizes = [4096, 70001, 5]
    total = sum(sizes)
    z = nb.Zero1AdamW.adamw(3e-4, 0.1, [(n,) for n in sizes], rank, world, nb.exchange_unique_id(rank, world),
                            timeout_s=4.0)
    assert os.environ.get("NCCL_NVLS_ENABLE") == "0", "run this worker with NCCL_NVLS_ENABLE=0"
    pflat = torch.zeros(z.padded, dtype=torch.bfloat16, device="cuda")
    gflat = torch.zeros(z.padded, dtype=torch.bfloat16, device="cuda")
    step = lambda: z.step(pflat, gflat, average=True)
    pflat[:total] = 0.01
    gflat[:total] = 1e-4
    z.init_master(pflat)
    for _ in range(2):
        assert step().applied
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    if rank != 0:
        os._exit(0)                       # leaves between steps, nothing in flight
    time.sleep(1.0)
    t0 = time.time()
    try:
        step()
        print("ZERO1_LEAVE_FAIL step returned although a rank is gone")
        os._exit(1)
    except nb._lib.NablaOptimError as e:
        dt = time.time() - t0
        assert e.code == nb._lib.NBO_ERR_TIMEOUT, (e.code, e.message)
        assert "timed out" in e.message and dt < 30.0, (e.message, dt)
    try:
        step()
        os._exit(1)
    except nb._lib.NablaOptimError as e:
        assert e.code == nb._lib.NBO_ERR_STATE and "aborted" in e.message
    # the context is intact: a fresh single-GPU optimizer on the same device works
    p = torch.ones(1000, device="cuda")
    nb.Sgd(0.1, [(1000,)]).step([p], [torch.ones(1000, device="cuda")])
    torch.cuda.synchronize()
    assert abs(float(p[0]) - 0.9) < 1e-6
    print("ZERO1_LEAVE_OK", f"{dt:.1f}s", flush=True)
    os._exit(0)                           # the torch process group cannot be torn down without its peer


if __name__ == "__main__":
    main()
