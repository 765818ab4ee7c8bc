"""CPU, world_size 2 over gloo: the host-side logic of the sharded step.

Each rank takes the shard plan from the library's pure-host entry points (nbo_zero1_geometry and the
piece intersection mirrored by nabla_b200.shard_pieces), averages the two ranks' gradients over gloo,
runs the ORACLE's mixed-precision composition on its own pieces only (per-piece hyper-parameters from the
group routing), gathers the bf16 params, and the result must equal the unsharded oracle bit for bit -
sharding may change where an element is updated, never its value.  The global grad norm is combined in rank
order from per-rank partial sums, as the device code does."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SIZES = [5, 4096, 3, 7001, 1, 8192, 2, 1000]
NAMES = ["embed.weight", "l0.w", "l0.bias", "l1.w", "ln.weight", "l2.w", "l2.bias", "head.w"]


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import nabla_b200 as nb
    from oracle import binding as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        P, S, M = nb.ParamGroupConfig, nb.ParamSelector, nb.ParamMatch
        nd = P.adamw("no_decay", S.Any([M.Suffix("bias"), M.Contains("ln")]), 3e-4, 0.0)
        dec = P.adamw("decay", S.All(), 3e-4, 0.1)
        kept, gid = nb.assign_groups(NAMES, [nd], dec)
        cfg_of = lambda t: orc.AdamCfg(kept[gid[t]].lr, 0.9, 0.999, 1e-8, kept[gid[t]].weight_decay, 1)
        total = sum(SIZES)
        shard, padded = nb.geometry(total, world)
        pieces = nb.shard_pieces(SIZES, rank, world)
        offs = np.cumsum([0] + SIZES)

        rng = np.random.default_rng(11)                       # same masters everywhere
        w_full = rng.normal(0, 0.02, total).astype(np.float32)
        # unsharded reference on every rank
        ref = orc.MixedOracle([w_full[offs[t]:offs[t + 1]] for t in range(len(SIZES))],
                              [cfg_of(t) for t in range(len(SIZES))], use_scaler=False)
        # sharded: state only for this rank's pieces
        mine = orc.MixedOracle([w_full[offs[t] + o:offs[t] + o + n] for t, o, n in pieces],
                               [cfg_of(t) for t, _, _ in pieces], use_scaler=False)
        p_flat = np.zeros(padded, np.uint16)
        p_flat[:total] = orc.bf16_from_f32(w_full)
        for step in range(3):
            g_rank = np.random.default_rng(100 * step + rank).normal(0, 1e-4, total).astype(np.float32)
            g16_rank = orc.bf16_to_f32(orc.bf16_from_f32(g_rank))          # each rank's bf16 grads, widened
            t = torch.from_numpy(g16_rank.copy())
            dist.all_reduce(t)                                            # the reduce half of reduce-scatter
            g_avg16 = orc.bf16_from_f32((t.numpy() / world).astype(np.float32))
            max_norm = 1e-3
            # per-rank partial sum of squares, combined in rank order (finalize_ranks_kernel)
            part = 0.0
            for tt, o, n in pieces:
                v = orc.bf16_to_f32(g_avg16[offs[tt] + o:offs[tt] + o + n]).astype(np.float64)
                for x in v:
                    part += x * x
            parts = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
            dist.all_gather(parts, torch.tensor([part], dtype=torch.float64))
            norm = float(np.sqrt(sum(float(x) for x in parts)))
            ok_ref, norm_ref = ref.step([g_avg16[offs[t]:offs[t + 1]].copy() for t in range(len(SIZES))],
                                        max_norm=max_norm)
            assert ok_ref and abs(norm - norm_ref) <= 1e-13 * norm_ref
            # local update with the globally decided clip factor: clip on the piece grads by hand
            gs = [orc.bf16_to_f32(g_avg16[offs[tt] + o:offs[tt] + o + n]) for tt, o, n in pieces]
            if norm > max_norm and norm > 0:
                f = np.float32(max_norm / norm)
                gs = [(g * f).astype(np.float32) for g in gs]
            mine.step_count.value += 1
            for i, (tt, o, n) in enumerate(pieces):
                c = mine.cfgs[i]
                orc.adam_step(mine.master[i], gs[i], mine.m[i], mine.v[i], c.lr, c.beta1, c.beta2, c.eps,
                              c.weight_decay, mine.step_count.value, decoupled=True)
                p_flat[offs[tt] + o:offs[tt] + o + n] = orc.bf16_from_f32(mine.master[i])
            # all-gather of the shards
            b, e = rank * shard, (rank + 1) * shard
            got = [torch.zeros(shard, dtype=torch.int32) for _ in range(world)]     # gloo has no 16-bit types
            dist.all_gather(got, torch.from_numpy(p_flat[b:e].astype(np.int32)))
            p_flat = np.concatenate([x.numpy().astype(np.uint16) for x in got])
            want = np.concatenate(ref.p)
            assert np.array_equal(p_flat[:total], want), f"rank {rank} step {step}: sharded != unsharded"
        out[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_sharded_oracle_equals_unsharded_world2():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        out = mgr.dict()
        port = 29650 + os.getpid() % 200
        procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=300)
        for p in procs:
            if p.is_alive():
                p.kill()
                pytest.fail("gloo worker timed out")
        assert dict(out) == {0: "ok", 1: "ok"}, dict(out)
        assert all(p.exitcode == 0 for p in procs)
