"""One rank of the host-streamed sharded step check (launched by tests/test_gpu_zero1.py under
torch.distributed.run):  zero1_host_worker.py [peer|mcast]

Two sharded optimizers with the same initial state take the same gradients.  One has them in its symmetric
device bucket and runs nbo_zero1_step_fused; the other gets them from pinned HOST tensors (one per
parameter tensor, as nabla's CPU-backend tensors are) through nbo_zero1_step_host, which slices the shard
and pipelines copy-in, barrier, fused kernel and copy-out.  After every step the host parameters of this
rank's shard must equal the fused step's device parameters bit for bit, the host elements outside the
shard must be untouched, and at the end the fp32 state shards must be equal.  Unchecked steps are cut
into many slices (ragged: the ranks have different slice counts); steps with loss scaling and clipping,
including a skipped one, go through the copy-everything-first path.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import nabla_b200 as nb  # noqa: E402


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "peer"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    sizes = [5, 4096, 3, 70001, 1, 8192, 2, 100000, 12289]
    names = ["w0", "w1", "norm2", "w3", "norm4", "w5", "norm6", "w7", "w8"]
    total = sum(sizes)
    shapes = [(n,) for n in sizes]
    nd = [nb.ParamGroupConfig.adamw("no_decay", nb.ParamSelector.Any([nb.ParamMatch.Prefix("norm")]), 3e-4, 0.0)]
    dec = nb.ParamGroupConfig.adamw("decay", nb.ParamSelector.All(), 3e-4, 0.1)
    tr = 1 if mode == "peer" else 2
    zf = nb.Zero1AdamW(names, shapes, nd, dec, rank, world, nb.exchange_unique_id(rank, world))
    zh = nb.Zero1AdamW(names, shapes, nd, dec, rank, world, nb.exchange_unique_id(rank, world))
    pf, gf = zf.attach_symmetric(transport=tr)
    ph, gh = zh.attach_symmetric(transport=tr)
    if mode == "mcast" and not (zf.has_multicast and zh.has_multicast):
        if rank == 0:
            print("ZERO1_HOST_SKIP no multicast mapping on this fabric")
        dist.destroy_process_group()
        return
    g0 = torch.Generator(device="cuda").manual_seed(4321)
    pf[:total] = (torch.randn(total, device="cuda", generator=g0) * 0.02).to(torch.bfloat16)
    ph.copy_(pf)
    zf.init_master(pf)
    zh.init_master(ph)
    torch.cuda.synchronize()
    dist.barrier()

    offs = [0]
    for n in sizes:
        offs.append(offs[-1] + n)
    host_g = [torch.empty(n, dtype=torch.bfloat16).pin_memory() for n in sizes]
    host_p = [torch.empty(n, dtype=torch.bfloat16).pin_memory() for n in sizes]
    hga = nb._lib.ptr_array([t.data_ptr() for t in host_g])
    hpa = nb._lib.ptr_array([t.data_ptr() for t in host_p])
    b, e, _ = zf.shard_range()
    gr = torch.Generator(device="cuda").manual_seed(99 + rank)
    SENTINEL = -7.0

    plan = [dict(average=True, use_scaler=False, max_norm=0.0, slice_elems=8192),
            dict(average=False, use_scaler=False, max_norm=0.0, slice_elems=4096),
            dict(average=True, use_scaler=False, max_norm=0.0, slice_elems=0),
            dict(average=True, use_scaler=True, max_norm=1e-3, slice_elems=8192, scale=65536.0),
            dict(average=True, use_scaler=True, max_norm=1e-3, slice_elems=8192, scale=65536.0, inf=True),
            dict(average=True, use_scaler=True, max_norm=0.0, slice_elems=16384, scale=32768.0),
            dict(average=True, use_scaler=False, max_norm=0.0, slice_elems=8192)]
    for step, cfg in enumerate(plan):
        cfg = dict(cfg)
        scale, inf, se = cfg.pop("scale", 1.0), cfg.pop("inf", False), cfg.pop("slice_elems")
        g = torch.zeros(zf.padded, dtype=torch.bfloat16, device="cuda")
        g[:total] = (torch.randn(total, device="cuda", generator=gr) * 1e-4 * scale).to(torch.bfloat16)
        if inf and rank == world - 1:
            g[7] = float("inf")
        gf.copy_(g)
        for i, t in enumerate(host_g):
            t.copy_(g[offs[i]:offs[i + 1]])
        for t in host_p:
            t.fill_(SENTINEL)
        torch.cuda.synchronize()
        dist.barrier()
        rf = zf.step_fused(**cfg)
        rh = zh.step_host_ptrs(ph.data_ptr(), gh.data_ptr(), hpa, hga, slice_elems=se, **cfg)
        assert (rf.applied, rf.nonfinite, rf.loss_scale, rf.step_count) == \
               (rh.applied, rh.nonfinite, rh.loss_scale, rh.step_count), (step, rf, rh)
        assert rf.grad_norm == rh.grad_norm, (step, rf.grad_norm, rh.grad_norm)
        assert bool(rf.applied) == (not inf)
        flat_host = torch.cat(host_p)
        lo, hi = b, min(e, total)
        if rf.applied:
            assert torch.equal(flat_host[lo:hi].view(torch.int16), pf[lo:hi].cpu().view(torch.int16)), \
                f"rank {rank} step {step}: host parameters of the shard differ from the fused step's"
            outside = torch.cat([flat_host[:lo], flat_host[hi:]])
        else:
            outside = flat_host                                   # a skipped step copies nothing out
        assert bool((outside.float() == SENTINEL).all()), f"rank {rank} step {step}: wrote outside its shard"
        # both device parameter buckets agree everywhere (every rank published its slice to every rank)
        assert torch.equal(ph[:total].view(torch.int16), pf[:total].view(torch.int16)), (rank, step)
    for which in (0, 1, 2):
        assert torch.equal(zf.state_shard(which), zh.state_shard(which)), f"state {which} differs"

    # the asynchronous fused step (state advanced on the device, no host wait) against the synchronous one:
    # four steps enqueued back to back, the second of them skipped because of an inf, then one collect
    scale = zf.scaler_state().scale
    assert scale == zh.scaler_state().scale
    seq = []
    for k in range(4):
        g = torch.zeros(zf.padded, dtype=torch.bfloat16, device="cuda")
        g[:total] = (torch.randn(total, device="cuda", generator=gr) * 1e-4 * scale).to(torch.bfloat16)
        if k == 1 and rank == 0:
            g[total - 3] = float("nan")
        seq.append(g)
    outcomes = []
    for g in seq:
        gf.copy_(g)
        torch.cuda.synchronize(); dist.barrier()
        outcomes.append(zf.step_fused(average=True, use_scaler=True, max_norm=1e-3))
    stage = [torch.empty_like(gh) for _ in seq]                 # the asynchronous side must not wait between steps:
    for s_, g in zip(stage, seq):                               # every step's gradients are staged up front
        s_.copy_(g)
    torch.cuda.synchronize(); dist.barrier()
    for s_ in stage:
        gh.copy_(s_, non_blocking=True)                          # stream-ordered before the step that reads it
        zh.step_fused_async(average=True, use_scaler=True, max_norm=1e-3)
    last, done = zh.collect()
    assert done == len(seq)
    assert [o.applied for o in outcomes] == [True, False, True, True]
    assert (last.applied, last.loss_scale, last.step_count, last.grad_norm) == \
           (outcomes[-1].applied, outcomes[-1].loss_scale, outcomes[-1].step_count, outcomes[-1].grad_norm)
    assert torch.equal(ph[:total].view(torch.int16), pf[:total].view(torch.int16)), "async params differ"
    for which in (0, 1, 2):
        assert torch.equal(zf.state_shard(which), zh.state_shard(which)), f"async state {which} differs"
    sa, sb = zf.scaler_state(), zh.scaler_state()
    assert (sa.scale, sa.consecutive_ok) == (sb.scale, sb.consecutive_ok)
    assert zf.step_count(0) == zh.step_count(0) and zf.step_count(1) == zh.step_count(1)
    dist.barrier()
    if rank == 0:
        print("ZERO1_HOST_OK", world, mode)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
