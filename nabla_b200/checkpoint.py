"""Checkpoint / resume of optimizer, scaler and schedule state in the reference's on-disk format.

Directory layout and encodings follow nabla-train/src/checkpoint.rs:34-150 and
nabla-ml/src/module/core.rs:66-133:

    meta.txt      key=value lines: version, epoch, step, grad_accum, [rng.state], optim.* (or
                  optim.group.*), [schedule.*], scaler.*
    optim.nbla    b"NBLA", u32 count, then per tensor: u32 name length, UTF-8 name, u32 rows, u32 cols,
                  rows*cols f64 little-endian (every element is widened to f64 on disk)
    params.nbla   same container (written only when named params are passed)

State tensors keep the reference's names: m{i} / v{i} (Adam, AdamW), v{i} (the SGD velocity), prefixed
g{k}. inside a GroupOptimizer (alg.rs:476-485,620-640; groups.rs:320-328), and the reference's shapes:
every m / v / w tensor is written with its parameter's (rows, cols), because the reference installs a loaded
tensor as it is (alg.rs:487-518) and its next axpy_inplace insists on equal shapes
(nabla-core/src/common/tensor/ops.rs:638-646).  On load either layout of the right element count is taken.
The mixed-precision and ZeRO-1 optimizers additionally store their fp32 masters as w{i}; the reference's
loaders skip names that start with neither m nor v, so such a file still loads there.
Numbers in meta.txt are written the way Rust's `{}` prints an f64 (shortest round-trip digits, positional,
no exponent, no trailing ".0") so files are byte-compatible, and parsed leniently like `str::parse::<f64>`.
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass
from decimal import Decimal
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib as L
from .optim import GroupOptimizer, LrSchedule, MixedAdamW, _as_state, _flat_state

NBLA_MAGIC = b"NBLA"
META_FILE, PARAMS_FILE, OPTIM_FILE = "meta.txt", "params.nbla", "optim.nbla"
KIND_STR = {L.NBO_ADAMW: "adamw", L.NBO_ADAM: "adam", L.NBO_SGD: "sgd"}
STR_KIND = {v: k for k, v in KIND_STR.items()}


def rust_f64(x: float) -> str:
    """`format!("{}", x)` for an f64."""
    if x != x:
        return "NaN"
    if x in (float("inf"), float("-inf")):
        return "inf" if x > 0 else "-inf"
    if x == 0:
        return "-0" if str(x).startswith("-") else "0"
    s = format(Decimal(repr(float(x))), "f")
    if "." in s:
        s = s.rstrip("0").rstrip(".")
    return s


@dataclass
class TrainState:
    """`struct TrainState` (nabla-train/src/trainer.rs:12-17)."""
    epoch: int = 0
    step: int = 0
    grad_accum: int = 1
    rng_state: Optional[int] = None


@dataclass
class ScheduleState:
    """`struct ScheduleState` (optim/core.rs:123-127)."""
    base_lr: float
    schedule: LrSchedule


# ----------------------------------------------------------------------------- .nbla container

def save_tensors(tensors: Sequence[Tuple[str, np.ndarray]], path: str) -> None:
    with open(path, "wb") as f:
        f.write(NBLA_MAGIC)
        f.write(struct.pack("<I", len(tensors)))
        for name, t in tensors:
            a = np.asarray(t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else t)
            if a.ndim == 1:
                a = a.reshape(1, -1) if a.size else a.reshape(0, 0)
            if a.ndim != 2:
                a = a.reshape(a.shape[0], -1)
            if a.shape[0] > 0xFFFFFFFF or a.shape[1] > 0xFFFFFFFF:
                # the reference writes `rows as u32`, `cols as u32` (module/core.rs:76-78): a larger extent
                # would wrap silently and the file could not be read back, so it is refused instead
                raise ValueError(f"tensor {name}: shape {a.shape} does not fit the u32 rows/cols of the nabla format")
            nb = name.encode("utf-8")
            f.write(struct.pack("<I", len(nb)))
            f.write(nb)
            f.write(struct.pack("<II", a.shape[0], a.shape[1]))
            f.write(np.ascontiguousarray(a, dtype="<f8").tobytes())


def load_tensors(path: str) -> List[Tuple[str, np.ndarray]]:
    out = []
    with open(path, "rb") as f:
        if f.read(4) != NBLA_MAGIC:
            raise ValueError("not a nabla tensor file")
        (count,) = struct.unpack("<I", f.read(4))
        for _ in range(count):
            (nlen,) = struct.unpack("<I", f.read(4))
            name = f.read(nlen).decode("utf-8")
            rows, cols = struct.unpack("<II", f.read(8))
            raw = f.read(8 * rows * cols)
            if len(raw) != 8 * rows * cols:
                raise ValueError("truncated nabla tensor file")
            out.append((name, np.frombuffer(raw, dtype="<f8").reshape(rows, cols).copy()))
    return out


# ----------------------------------------------------------------------------- meta pairs

def _meta_of_group(opt, gid: int) -> Dict[str, str]:
    cfg = opt._h.get_group(gid)
    kind = cfg.kind
    adamish = kind != L.NBO_SGD
    return {
        "kind": KIND_STR[kind], "lr": rust_f64(cfg.lr),
        "beta1": rust_f64(cfg.beta1 if adamish else 0.0), "beta2": rust_f64(cfg.beta2 if adamish else 0.0),
        "eps": rust_f64(cfg.eps if adamish else 0.0),
        "weight_decay": rust_f64(0.0 if kind == L.NBO_ADAM else cfg.weight_decay),
        "momentum": rust_f64(cfg.momentum if kind == L.NBO_SGD else 0.0),
        "step_count": str(opt._h.step_count(gid) if adamish else 0),
    }


def optim_meta_pairs(opt) -> List[Tuple[str, str]]:
    """OptimState::meta_pairs (optim/core.rs:262-277; groups.rs:367-398)."""
    if hasattr(opt, "_configs"):          # grouped (GroupOptimizer, MixedAdamW, Zero1AdamW)
        out = [("optim.group.count", str(len(opt._configs)))]
        for gi, cfg in enumerate(opt._configs):
            out.append((f"optim.group.{gi}.name", cfg.name))
            m = _meta_of_group(opt, gi)
            for k in ("kind", "lr", "beta1", "beta2", "eps", "weight_decay", "momentum", "step_count"):
                out.append((f"optim.group.{gi}.{k}", m[k]))
        return out
    m = _meta_of_group(opt, 0)
    return [(f"optim.{k}", m[k]) for k in ("kind", "lr", "beta1", "beta2", "eps", "weight_decay", "momentum",
                                           "step_count")]


def _need(mp: Dict[str, str], key: str) -> str:
    if key not in mp:
        raise ValueError(f"missing {key}")
    return mp[key]


def _f64(mp, key) -> float:
    v = _need(mp, key)
    try:
        return float(v)
    except ValueError:
        raise ValueError(f"bad {key}: {v}")


def _usize(mp, key) -> int:
    v = _need(mp, key)
    if not v.isdigit():
        raise ValueError(f"bad {key}: {v}")
    return int(v)


def load_optim_meta_pairs(opt, mp: Dict[str, str]) -> None:
    """OptimState::load_meta_pairs: same checks and error texts as the reference."""
    def apply(gid: int, prefix: str):
        kind_s = _need(mp, prefix + "kind")
        if kind_s not in STR_KIND:
            raise ValueError(f"bad optim.kind: {kind_s}")
        cfg = opt._h.get_group(gid)
        if STR_KIND[kind_s] != cfg.kind:
            raise ValueError("optim kind mismatch")
        cfg.lr = _f64(mp, prefix + "lr")
        if cfg.kind == L.NBO_SGD:
            cfg.momentum = _f64(mp, prefix + "momentum")
            cfg.weight_decay = _f64(mp, prefix + "weight_decay")
        else:
            cfg.beta1, cfg.beta2, cfg.eps = _f64(mp, prefix + "beta1"), _f64(mp, prefix + "beta2"), _f64(mp, prefix + "eps")
            if cfg.kind == L.NBO_ADAMW:
                cfg.weight_decay = _f64(mp, prefix + "weight_decay")
        step = _usize(mp, prefix + "step_count")
        _f64(mp, prefix + "momentum"); _f64(mp, prefix + "weight_decay")
        opt._h.set_group(gid, cfg)
        if cfg.kind != L.NBO_SGD:
            opt._h.check(opt._h.lib.nbo_set_step_count(opt._h.h, gid, step))

    if hasattr(opt, "_configs"):
        if _usize(mp, "optim.group.count") != len(opt._configs):
            raise ValueError("optim.group.count mismatch")
        for gi, cfg in enumerate(opt._configs):
            if _need(mp, f"optim.group.{gi}.name") != cfg.name:
                raise ValueError(f"optim.group.{gi}.name mismatch")
            apply(gi, f"optim.group.{gi}.")
    else:
        apply(0, "optim.")


def schedule_pairs(st: ScheduleState) -> List[Tuple[str, str]]:
    s = st.schedule
    out = [("schedule.enabled", "1"), ("schedule.base_lr", rust_f64(st.base_lr))]
    if s.kind == L.NBO_SCHED_COSINE:
        out += [("schedule.kind", "cosine"), ("schedule.warmup_steps", str(s.warmup_steps)),
                ("schedule.total_steps", str(s.total_steps)), ("schedule.min_lr", rust_f64(s.min_lr))]
    elif s.kind == L.NBO_SCHED_LINEAR:
        out += [("schedule.kind", "linear"), ("schedule.warmup_steps", str(s.warmup_steps)),
                ("schedule.total_steps", str(s.total_steps))]
    elif s.kind == L.NBO_SCHED_ONECYCLE:
        out += [("schedule.kind", "onecycle"), ("schedule.max_lr", rust_f64(s.max_lr)),
                ("schedule.total_steps", str(s.total_steps)), ("schedule.pct_start", rust_f64(s.pct_start))]
    else:
        out += [("schedule.kind", "step"), ("schedule.step_size", str(s.step_size)),
                ("schedule.gamma", rust_f64(s.gamma))]
    return out


def parse_schedule_state(mp: Dict[str, str]) -> Optional[ScheduleState]:
    if mp.get("schedule.enabled", "0") != "1":
        return None
    base = _f64(mp, "schedule.base_lr")
    kind = _need(mp, "schedule.kind")
    if kind == "cosine":
        s = LrSchedule.Cosine(_usize(mp, "schedule.warmup_steps"), _usize(mp, "schedule.total_steps"),
                              _f64(mp, "schedule.min_lr"))
    elif kind == "linear":
        s = LrSchedule.Linear(_usize(mp, "schedule.warmup_steps"), _usize(mp, "schedule.total_steps"))
    elif kind == "onecycle":
        s = LrSchedule.OneCycle(_f64(mp, "schedule.max_lr"), _usize(mp, "schedule.total_steps"),
                                _f64(mp, "schedule.pct_start"))
    elif kind == "step":
        s = LrSchedule.Step(_usize(mp, "schedule.step_size"), _f64(mp, "schedule.gamma"))
    else:
        raise ValueError(f"bad schedule.kind: {kind}")
    return ScheduleState(base, s)


# ----------------------------------------------------------------------------- state tensors

def state_tensors(opt) -> List[Tuple[str, torch.Tensor]]:
    from .zero1 import Zero1AdamW
    if isinstance(opt, Zero1AdamW):
        return opt.state_tensors()
    if isinstance(opt, MixedAdamW):
        out = []
        for gi in range(len(opt._configs)):
            idx = [i for i, g in enumerate(opt._gid_of) if g == gi]
            for which, p in ((0, "m"), (1, "v"), (2, "w")):
                for li, i in enumerate(idx):
                    out.append((f"g{gi}.{p}{li}", _as_state(opt._h.state_export(i, which, opt._numel[i]),
                                                            opt._shapes[i])))
        return out
    return opt.state_tensors()


def load_state_tensors(opt, tensors: Sequence[Tuple[str, np.ndarray]]) -> None:
    from .zero1 import Zero1AdamW
    tens = [(n, torch.from_numpy(np.asarray(a, dtype=np.float32))) for n, a in tensors]
    if isinstance(opt, Zero1AdamW):
        opt.load_state_tensors(tens)
        return
    if isinstance(opt, (GroupOptimizer, MixedAdamW)):
        ngroups = len(opt._configs)
        slots: Dict[Tuple[int, str, int], torch.Tensor] = {}
        for name, t in tens:
            if "." not in name:
                raise ValueError(f"bad group tensor key: {name}")
            g, rest = name.split(".", 1)
            if not g.startswith("g"):
                raise ValueError(f"bad group tensor key: {name}")
            if not g[1:].isdigit():
                raise ValueError(f"bad group index: {g[1:]}")
            gi = int(g[1:])
            if gi >= ngroups:
                raise ValueError(f"group index out of range: {gi}")
            if rest[:1] in ("m", "v", "w"):
                if not rest[1:].isdigit():
                    raise ValueError(f"bad tensor key: {rest}")
                slots[(gi, rest[0], int(rest[1:]))] = t
        for gi, cfg in enumerate(opt._configs):
            idx = [i for i, g in enumerate(opt._gid_of) if g == gi]
            want = [("v", 0)] if cfg.kind == L.NBO_SGD else [("m", 0), ("v", 1)]
            if isinstance(opt, MixedAdamW):
                want.append(("w", 2))
            for p, which in want:
                for li, i in enumerate(idx):
                    if (gi, p, li) not in slots:
                        raise ValueError(f"missing {p}{li}")
                    opt._h.state_import(i, which, _flat_state(slots[(gi, p, li)], opt._numel[i], f"g{gi}.{p}{li}"))
        return
    opt.load_state_tensors(tens)


# ----------------------------------------------------------------------------- checkpoint dir

def save_checkpoint(directory: str, optimizer, scaler=None, schedule: Optional[ScheduleState] = None,
                    state: Optional[TrainState] = None, named_params=None) -> None:
    """save_checkpoint (nabla-train/src/checkpoint.rs:34-63).  `scaler` is a GradScaler, or the mixed
    optimizer itself (its loss scaler lives in the handle)."""
    state = state or TrainState()
    tensors = state_tensors(optimizer)
    if tensors is None:        # a ZeRO-1 rank other than 0: it only contributed its shard
        return
    os.makedirs(directory, exist_ok=True)
    if named_params is not None:
        save_tensors([(n, t.detach().float().cpu().numpy()) for n, t in named_params],
                     os.path.join(directory, PARAMS_FILE))
    save_tensors([(n, t.numpy()) for n, t in tensors], os.path.join(directory, OPTIM_FILE))
    lines = ["version=1", f"epoch={state.epoch}", f"step={state.step}", f"grad_accum={state.grad_accum}"]
    if state.rng_state is not None:
        lines.append(f"rng.state={state.rng_state}")
    lines += [f"{k}={v}" for k, v in optim_meta_pairs(optimizer)]
    if schedule is not None:
        lines += [f"{k}={v}" for k, v in schedule_pairs(schedule)]
    if scaler is not None:
        st = scaler.scaler_state() if hasattr(scaler, "scaler_state") else scaler.state()
        lines += ["scaler.enabled=1", f"scaler.scale={rust_f64(st.scale)}",
                  f"scaler.growth_factor={rust_f64(st.growth_factor)}",
                  f"scaler.backoff_factor={rust_f64(st.backoff_factor)}",
                  f"scaler.growth_interval={st.growth_interval}", f"scaler.consecutive_ok={st.consecutive_ok}"]
    else:
        lines.append("scaler.enabled=0")
    with open(os.path.join(directory, META_FILE), "w") as f:
        f.write("\n".join(lines) + "\n")


def read_meta(path: str) -> Dict[str, str]:
    mp: Dict[str, str] = {}
    for line in open(path).read().splitlines():
        if not line.strip():
            continue
        if "=" not in line:
            raise ValueError(line)
        k, v = line.split("=", 1)
        mp[k] = v
    return mp


def load_checkpoint(directory: str, optimizer, scaler=None):
    """load_checkpoint (checkpoint.rs:65-104): returns (TrainState, Optional[ScheduleState])."""
    load_state_tensors(optimizer, load_tensors(os.path.join(directory, OPTIM_FILE)))
    mp = read_meta(os.path.join(directory, META_FILE))
    epoch, step, accum = _usize(mp, "epoch"), _usize(mp, "step"), _usize(mp, "grad_accum")
    load_optim_meta_pairs(optimizer, mp)
    if scaler is not None and mp.get("scaler.enabled", "0") == "1":
        st = L.ScalerState(_f64(mp, "scaler.scale"), _f64(mp, "scaler.growth_factor"),
                           _f64(mp, "scaler.backoff_factor"), _usize(mp, "scaler.growth_interval"),
                           _usize(mp, "scaler.consecutive_ok"))
        (scaler.load_scaler_state if hasattr(scaler, "load_scaler_state") else scaler.load_state)(st)
    rng = int(mp["rng.state"]) if mp.get("rng.state", "").isdigit() else None
    return TrainState(epoch, step, accum, rng), parse_schedule_state(mp)
