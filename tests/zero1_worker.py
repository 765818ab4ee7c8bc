"""One rank of the multi-GPU ZeRO-1 check (launched by tests/test_gpu_zero1.py under torch.distributed.run).

    zero1_worker.py [nccl|peer|mcast|native-peer|native-mcast]

nccl  : reduce-scatter / all-gather issued as NCCL collectives around the local update (nbo_zero1_step)
peer  : collectives fused into the kernels with plain peer loads/stores (nbo_zero1_step_fused, transport 1)
mcast : the same through NVSwitch multimem ld_reduce / st (transport 2)
native-peer / native-mcast : as peer / mcast, with the symmetric buckets made by the library itself
        (nbo_symm_alloc: CUDA virtual memory + multicast object) instead of torch's symmetric-memory module

Every rank holds its own bf16 gradients.  Each sharded step is checked three ways:
  (0) the cross-rank reduction against an independent reference: every rank's INPUT gradients are
      all-gathered before the step, this rank's shard is summed in fp32 in rank order with torch on local
      memory, multiplied by f32(1/world) when averaging (the mean of the replicas,
      nabla-train/src/dist.rs:36-43) and rounded once to bf16.  The reduced gradients the step leaves in
      place must equal that bit for bit on the `peer` transport (same order, one rounding) and stay within
      the rounding bounds of the other summation orders for `mcast` (the switch rounds to bf16 once, the
      averaging rounds again: 1 ulp) and `nccl` (bf16 roundings between the ring's hops);
  (1) the parameter bucket is identical on all ranks, and
  (2) a world = 1 optimizer on the same GPU, fed the reduced gradients the sharded step actually used
      (gathered from the in-place reduce-scatter output), produces bit-identical parameters - i.e.
      sharding changes where an element is updated, never its value.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import nabla_b200 as nb  # noqa: E402


def ordered(bits16: torch.Tensor) -> torch.Tensor:
    """bf16 bit patterns as integers that increase with the value (one step = one ulp)."""
    i = bits16.view(torch.int16).to(torch.int32) & 0xffff
    return torch.where(i >= 0x8000, 0x8000 - i, i)


def check_reduction(mode, world, rank, raw, reduced, b, e, average, total):
    """`raw`: every rank's input bucket; `reduced`: this rank's slice after the step."""
    hi = min(e, total)
    if hi <= b:
        return
    acc = torch.zeros(hi - b, dtype=torch.float32, device="cuda")
    mag = torch.zeros_like(acc)
    for r in range(world):                                   # rank order, one fp32 rounding per addition
        x = raw[r][b:hi].float()
        acc += x
        mag += x.abs()
    if average:
        acc *= torch.tensor(1.0, dtype=torch.float32, device="cuda") / torch.tensor(float(world), dtype=torch.float32,
                                                                                     device="cuda")
    want = acc.to(torch.bfloat16)
    got = reduced[:hi - b]
    if mode == "peer":
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), \
            f"rank {rank}: peer reduction differs from the fp32 rank-order sum"
        return
    ulps = (ordered(got) - ordered(want)).abs()
    err = (got.float() - want.float()).abs()
    if mode == "mcast":
        ok = (ulps <= 1) | (err <= mag * 2.0 ** -20)
    else:                                                    # nccl: a bf16 rounding per hop, each on a partial sum <= mag
        ok = err <= mag * (world * 2.0 ** -8) * (1.0 / world if average else 1.0) + 1e-30
    assert bool(ok.all()), (f"rank {rank} {mode}: reduced gradient off: worst {int(ulps.max())} ulp, "
                            f"{int((~ok).sum())} elements outside the bound")
    if rank == 0:
        print(f"ZERO1_REDUCTION {mode} world {world} average {average}: worst {int(ulps.max())} ulp, "
              f"{float((ulps > 0).float().mean()):.4f} of elements differ", flush=True)


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "nccl"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    sizes = [5, 4096, 3, 70001, 1, 8192, 2, 100000]
    total = sum(sizes)
    uid = nb.exchange_unique_id(rank, world)
    # two parameter groups (no weight decay on the "norm" tensors): group ranges must survive sharding
    names = ["w0", "w1", "norm2", "w3", "norm4", "w5", "norm6", "w7"]
    shapes = [(n,) for n in sizes]
    nd = [nb.ParamGroupConfig.adamw("no_decay", nb.ParamSelector.Any([nb.ParamMatch.Prefix("norm")]), 3e-4, 0.0)]
    dec = nb.ParamGroupConfig.adamw("decay", nb.ParamSelector.All(), 3e-4, 0.1)
    z = nb.Zero1AdamW(names, shapes, nd, dec, rank, world, uid)
    ref = nb.Zero1AdamW(names, shapes, nd, dec, 0, 1)                      # single-GPU twin, full bucket
    padded = z.padded
    assert ref.padded <= padded
    g0 = torch.Generator(device="cuda").manual_seed(1234)
    if mode == "nccl":
        pflat = torch.zeros(padded, dtype=torch.bfloat16, device="cuda")
        gbuf = None
    else:
        native = mode.startswith("native-")               # buckets made by the library's own nbo_symm_alloc
        if native:
            mode = mode[len("native-"):]
            pflat, gbuf = z.attach_symmetric_native(transport=1 if mode == "peer" else 2)
        else:
            pflat, gbuf = z.attach_symmetric(transport=1 if mode == "peer" else 2)
        if mode == "mcast" and not z.has_multicast:
            if native:
                z.release_symmetric()
            if rank == 0:
                print("ZERO1_WORKER_SKIP no multicast mapping on this fabric")
            dist.destroy_process_group()
            return

    def do_step(gflat, **kw):
        if mode == "nccl":
            return z.step(pflat, gflat, **kw), gflat
        gbuf.copy_(gflat)
        torch.cuda.synchronize()
        return z.step_fused(**kw), gbuf

    pflat[:total] = (torch.randn(total, device="cuda", generator=g0) * 0.02).to(torch.bfloat16)
    pref = pflat[:ref.padded].clone()
    z.init_master(pflat)
    ref.init_master(pref)
    gr = torch.Generator(device="cuda").manual_seed(99 + rank)
    for step in range(3):
        for use_scaler, max_norm in ((False, 0.0),):
            gflat = torch.zeros(padded, dtype=torch.bfloat16, device="cuda")
            gflat[:total] = (torch.randn(total, device="cuda", generator=gr) * 1e-4).to(torch.bfloat16)
            raw = [torch.empty_like(gflat) for _ in range(world)]
            dist.all_gather(raw, gflat)                          # every rank's input, before anything is reduced
            res, gflat = do_step(gflat, average=(step != 1), use_scaler=use_scaler, max_norm=max_norm)
            assert res.applied
            # the reduced gradients each rank used sit in its slice of gflat
            b, e, _ = z.shard_range()
            check_reduction(mode, world, rank, raw, gflat[b:e], b, e, step != 1, total)
            parts = [torch.empty(z.shard, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
            dist.all_gather(parts, gflat[b:e].contiguous())
            gfull = torch.cat(parts)[:ref.padded].contiguous()
            r2 = ref.step(pref, gfull, use_scaler=use_scaler, max_norm=max_norm)
            assert r2.applied
            assert torch.equal(pflat[:total].view(torch.int16), pref[:total].view(torch.int16)), \
                f"rank {rank} step {step}: sharded params differ from the single-GPU twin"
    # clipping + scaler on: the decision is taken from all-gathered per-rank sums, identical everywhere
    gflat = torch.zeros(padded, dtype=torch.bfloat16, device="cuda")
    gflat[:total] = (torch.randn(total, device="cuda", generator=gr) * 1e-4 * 65536).to(torch.bfloat16)
    if rank == world - 1:
        gflat[7] = float("inf")              # lands in rank 0's shard after the reduce-scatter
    before = pflat.clone()
    res, gflat = do_step(gflat, average=False, use_scaler=True, max_norm=1.0)
    assert not res.applied and res.nonfinite and res.loss_scale == 32768.0, (rank, res)
    assert torch.equal(before.view(torch.int16), pflat.view(torch.int16))
    gflat = torch.zeros(padded, dtype=torch.bfloat16, device="cuda")
    gflat[:total] = (torch.randn(total, device="cuda", generator=gr) * 1e-4 * 32768).to(torch.bfloat16)
    raw = [torch.empty_like(gflat) for _ in range(world)]
    dist.all_gather(raw, gflat)
    res, gflat = do_step(gflat, average=True, use_scaler=True, max_norm=1e-3)
    assert res.applied and res.grad_norm > 1e-3
    b, e, _ = z.shard_range()
    check_reduction(mode, world, rank, raw, gflat[b:e], b, e, True, total)   # the reduce + norm kernel's output
    # the clipped, unscaled step against the single-GPU twin fed the same reduced gradients
    b, e, _ = z.shard_range()
    parts = [torch.empty(z.shard, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    dist.all_gather(parts, gflat[b:e].contiguous())
    gfull = torch.cat(parts)[:ref.padded].contiguous()
    st = ref._h.lib.nbo_scaler_set  # twin scaler: same scale as the sharded optimizer had for this step
    import ctypes as C
    sc = nb._lib.ScalerState(32768.0, 2.0, 0.5, 2000, 0)
    ref._h.check(st(ref._h.h, C.byref(sc)))
    r2 = ref.step(pref, gfull, use_scaler=True, max_norm=1e-3)
    assert r2.applied and abs(r2.grad_norm - res.grad_norm) <= 1e-12 * res.grad_norm, (r2.grad_norm, res.grad_norm)
    same = (pflat[:total].view(torch.int16) == pref[:total].view(torch.int16)).float().mean().item()
    assert same > 0.9999, f"clipped step: only {same:.6f} of the params match the single-GPU twin"
    norms = [torch.zeros(1, dtype=torch.float64, device="cuda") for _ in range(world)]
    dist.all_gather(norms, torch.tensor([res.grad_norm], dtype=torch.float64, device="cuda"))
    assert all(float(n) == res.grad_norm for n in norms), "grad norm differs between ranks"
    # identical parameters on every rank
    digest = pflat.view(torch.int16).to(torch.int64).sum().reshape(1)
    digests = [torch.zeros_like(digest) for _ in range(world)]
    dist.all_gather(digests, digest)
    assert all(int(d) == int(digest) for d in digests)
    dist.barrier()
    if sys.argv[1:] and sys.argv[1].startswith("native-"):
        assert "torch.distributed._symmetric_memory" not in sys.modules     # the framework module was never needed
        del pflat, gbuf, gflat, before
        z.release_symmetric()                               # unbind / unmap on every rank before anyone exits
    if rank == 0:
        print("ZERO1_WORKER_OK", world, sys.argv[1] if sys.argv[1:] else mode)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
