"""CPU: the C-ABI library loads, exports every symbol the header declares, runs its pure-host
entry points (schedules, shard geometry) identically to the oracle, and refuses to work
without a CUDA device instead of falling back to anything."""
import ctypes as C
import os
import re
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "nabla_optim_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"NBO_API\s+[\w\s\*]+?\b(nbo_\w+)\s*\(", text)))


def test_header_compiles_as_c99():
    r = subprocess.run(["/usr/bin/gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-fsyntax-only",
                        "-x", "c", HEADER], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_library_exports_every_declared_symbol(nbo_lib):
    from nabla_b200 import _lib
    syms = declared_symbols()
    assert len(syms) >= 30
    for s in syms:
        assert hasattr(nbo_lib, s), f"{s} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == syms, "Python binding and header disagree"
    assert nbo_lib.nbo_abi_version() == 2


def test_library_has_no_link_dependency_on_nccl_or_oracle():
    from nabla_b200 import _lib
    out = subprocess.run(["ldd", _lib.LIB_PATH], capture_output=True, text=True).stdout
    assert "nccl" not in out and "oracle" not in out


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_create_fails_loudly_without_gpu(nbo_lib):
    h = C.c_void_p()
    rc = nbo_lib.nbo_create(0, None, C.byref(h))
    assert rc != 0 and not h
    assert b"no CPU fallback" in nbo_lib.nbo_last_error(None)
    import nabla_b200 as nb
    with pytest.raises(nb.optim.NablaDeviceError):
        nb.Sgd(0.1, [(1, 1)])


def test_lr_at_step_matches_oracle(nbo_lib, oracle):
    import nabla_b200 as nb
    cases = [
        (nb.LrSchedule.Cosine(10, 110, 0.1), dict(kind=0, warmup_steps=10, total_steps=110, min_lr=0.1)),
        (nb.LrSchedule.Cosine(0, 1, 0.0), dict(kind=0, warmup_steps=0, total_steps=1, min_lr=0.0)),
        (nb.LrSchedule.Linear(5, 50), dict(kind=1, warmup_steps=5, total_steps=50)),
        (nb.LrSchedule.OneCycle(1.0, 100, 0.3), dict(kind=2, max_lr=1.0, total_steps=100, pct_start=0.3)),
        (nb.LrSchedule.OneCycle(1.0, 10, 0.0), dict(kind=2, max_lr=1.0, total_steps=10, pct_start=0.0)),
        (nb.LrSchedule.Step(7, 0.5), dict(kind=3, step_size=7, gamma=0.5)),
        (nb.LrSchedule.Step(0, 0.9), dict(kind=3, step_size=0, gamma=0.9)),
    ]
    for sched, okw in cases:
        kind = okw.pop("kind")
        for base in (1.0, 3e-4):
            for step in list(range(0, 60)) + [99, 100, 110, 1000]:
                if kind in (0, 1) and step > okw["total_steps"] and kind == 0:
                    pass
                got = nb.lr_at_step(sched, base, step)
                want = oracle.lr_at_step(kind, base, step, **okw)
                assert got == want, (kind, base, step)


def test_reference_schedule_kats_through_the_abi(nbo_lib):
    import nabla_b200 as nb
    lin = nb.LrSchedule.Linear(0, 10)
    assert abs(nb.lr_at_step(lin, 1.0, 0) - 1.0) < 1e-10 and nb.lr_at_step(lin, 1.0, 10) <= 1e-10
    st = nb.LrSchedule.Step(2, 0.1)
    for s, want in ((0, 1.0), (2, 0.1), (4, 0.01)):
        assert abs(nb.lr_at_step(st, 1.0, s) - want) < 1e-10
    assert nb.lr_at_step(nb.LrSchedule.OneCycle(1.0, 10, 0.5), 0.1, 3) > 0.1
    bad = nb.LrSchedule(kind=9)
    with pytest.raises(nb._lib.NablaOptimError, match="bad schedule.kind"):
        nb.lr_at_step(bad, 1.0, 0)


def test_zero1_geometry(nbo_lib):
    import nabla_b200 as nb
    for total in (0, 1, 7, 8, 9, 1001, 8030261248):
        for world in (1, 2, 3, 4, 8):
            shard, padded = nb.geometry(total, world)
            assert shard % 8 == 0 and shard >= 8
            assert padded == shard * world >= total
            assert padded - total < world * 8 + world or total == 0
    with pytest.raises(nb._lib.NablaOptimError):
        nb.geometry(10, 0)


def test_shard_pieces_cover_every_element_once(nbo_lib):
    import nabla_b200 as nb
    numel = [10, 0, 5, 4099, 1, 30]
    for world in (1, 2, 3, 8):
        seen = [0] * len(numel)
        for r in range(world):
            for t, off, n in nb.shard_pieces(numel, r, world):
                assert 0 <= off and off + n <= numel[t] and n > 0
                seen[t] += n
        assert seen == numel


def test_group_assignment_follows_reference_rules():
    import nabla_b200 as nb
    P, S = nb.ParamGroupConfig, nb.ParamSelector
    names = ["embed.weight", "l0.attn.weight", "l0.attn.bias", "l0.ln1.weight", "head.weight"]
    nd = P.adamw("no_decay", S.Any([nb.ParamMatch.Suffix("bias"), nb.ParamMatch.Contains("ln")]), 1e-3, 0.0)
    unused = P.adamw("unused", S.Any([nb.ParamMatch.Equals("nope")]), 1e-3, 0.0)
    dec = P.adamw("decay", S.All(), 1e-3, 0.1)
    kept, gid = nb.assign_groups(names, [unused, nd], dec)
    assert [k.name for k in kept] == ["no_decay", "decay"]      # empty groups dropped, default last
    assert gid == [1, 1, 0, 0, 1]
    with pytest.raises(ValueError, match="group assignment incomplete"):
        nb.assign_groups(names, [nd], None)
    # first matching group wins
    a = P.sgd("a", S.Any([nb.ParamMatch.Prefix("l0")]), 1.0, 0.0, 0.0)
    b = P.sgd("b", S.Any([nb.ParamMatch.Contains("attn")]), 1.0, 0.0, 0.0)
    _, gid = nb.assign_groups(names, [a, b], dec)
    assert gid == [2, 0, 0, 0, 2][:len(gid)] or gid == [1, 0, 0, 0, 1]
