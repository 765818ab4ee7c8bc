"""Host-side mirror of nabla-train's optimizer interface over the C ABI.

Same names, argument meaning and error behaviour as the Rust types in
nabla-train/src/optim/{core,alg,groups}.rs and trainer.rs, so code and tests
written against the reference read the same here:

    Optimizer.step / step_slices / reset / set_lr      optim/core.rs:9-44
    Sgd, Adam, AdamW (+ builders)                       optim/alg.rs
    ParamMatch, ParamSelector, ParamGroupConfig,
    ParamExclusionPreset, GroupOptimizer                optim/groups.rs
    LrSchedule, lr_at_step, GradScaler                  optim/core.rs:81-173,334-413
    clip_grad_norm, zero_grad                           trainer.rs:500-523, autograd/ops.rs:1668

Tensors are torch CUDA tensors used purely as device buffers (pointer + numel);
all arithmetic happens in libnabla_optim_b200.so.  Where Rust panics with
``assert_eq!`` this raises AssertionError with the same message; where Rust
returns ``Err(String)`` this raises ValueError with the same text.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib as L


def _numel_of(shape) -> int:
    if isinstance(shape, int):
        return shape
    n = 1
    for d in shape:
        n *= int(d)
    return n


def _shape2d_of(shape) -> Tuple[int, int]:
    """The (rows, cols) a nabla tensor of this shape has: every reference tensor is 2-D row-major
    (`param_shapes: &[(usize, usize)]`, alg.rs:20-27).  A bare count or a 1-D shape is one row;
    more than two dimensions keep the first as rows."""
    if isinstance(shape, int):
        return (1, shape)
    dims = [int(d) for d in shape]
    if len(dims) == 0:
        return (1, 1)
    if len(dims) == 1:
        return (1, dims[0])
    cols = 1
    for d in dims[1:]:
        cols *= d
    return (dims[0], cols)


def _as_state(flat: torch.Tensor, shape2d: Tuple[int, int]) -> torch.Tensor:
    """A state tensor as the reference holds it: the parameter's own (rows, cols)."""
    return flat.reshape(shape2d)


def _flat_state(t, numel: int, key: str) -> torch.Tensor:
    """A loaded state tensor as the flat fp32 run the library stores.  Either layout of the same elements
    is accepted ((rows, cols) as the reference writes it, or one row); a different element count is what
    the reference would trip over on its next step (`axpy_inplace ... shapes must match`,
    nabla-core/src/common/tensor/ops.rs:638-646) and is refused here, before anything is copied."""
    t = torch.as_tensor(t)
    if t.numel() != numel:
        raise ValueError(f"nabla: axpy_inplace shapes must match ({key}: {tuple(t.shape)} holds {t.numel()} "
                         f"elements, the parameter has {numel})")
    return t.reshape(-1)


def _check_tensors(ts: Sequence[torch.Tensor], dtype, what: str):
    for i, t in enumerate(ts):
        if not t.is_cuda:
            raise NablaDeviceError(f"{what}[{i}] is not a CUDA tensor (no CPU fallback exists)")
        if t.dtype != dtype:
            raise TypeError(f"{what}[{i}] has dtype {t.dtype}, expected {dtype}")
        if not t.is_contiguous():
            raise ValueError(f"{what}[{i}] is not contiguous")


class NablaDeviceError(RuntimeError):
    pass


def _ptrs(ts: Sequence[torch.Tensor]):
    return L.ptr_array([t.data_ptr() for t in ts])


# --------------------------------------------------------------------------- handle

class _Handle:
    """Owns one nbo_optimizer."""

    def __init__(self, device: Optional[int] = None, stream: Optional[int] = None):
        self.lib = L.load()
        if device is None:
            if not torch.cuda.is_available():
                raise NablaDeviceError("no CUDA device: the optimizer kernels have no CPU fallback")
            device = torch.cuda.current_device()
        if stream is None:
            stream = torch.cuda.current_stream(device).cuda_stream
        self.device = device
        self.h = L._H()
        L.check(None, self.lib.nbo_create(device, C.c_void_p(stream), C.byref(self.h)))

    def check(self, status: int):
        L.check(self.h, status)

    def close(self):
        if getattr(self, "h", None) is not None and self.h:
            self.lib.nbo_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # group access
    def add_group(self, cfg: L.GroupConfig) -> int:
        gid = C.c_int32()
        self.check(self.lib.nbo_add_group(self.h, C.byref(cfg), C.byref(gid)))
        return gid.value

    def get_group(self, gid: int) -> L.GroupConfig:
        cfg = L.GroupConfig()
        self.check(self.lib.nbo_get_group(self.h, gid, C.byref(cfg)))
        return cfg

    def set_group(self, gid: int, cfg: L.GroupConfig):
        self.check(self.lib.nbo_set_group(self.h, gid, C.byref(cfg)))

    def set_tensors(self, numel: Sequence[int], group_ids: Optional[Sequence[int]], precision: int):
        n = len(numel)
        arr = (C.c_uint64 * n)(*numel)
        gids = (C.c_int32 * n)(*group_ids) if group_ids is not None else None
        self.check(self.lib.nbo_set_tensors(self.h, n, arr, gids, precision))

    def step_count(self, gid: int = 0) -> int:
        c = C.c_uint64()
        self.check(self.lib.nbo_step_count(self.h, gid, C.byref(c)))
        return c.value

    def launch_count(self) -> int:
        c = C.c_uint64()
        self.check(self.lib.nbo_launch_count(self.h, C.byref(c)))
        return c.value

    def profile(self, on: bool = True):
        self.check(self.lib.nbo_profile(self.h, 1 if on else 0))

    def profile_last(self) -> Tuple[float, float]:
        """(norm pass ms, update launches ms) of the most recent step, from CUDA events on the stream."""
        a, b = C.c_float(), C.c_float()
        self.check(self.lib.nbo_profile_last(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def table_info(self) -> Tuple[int, int, int]:
        a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint64()
        self.check(self.lib.nbo_table_info(self.h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    def state_export(self, tensor: int, which: int, numel: int) -> torch.Tensor:
        out = torch.empty(numel, dtype=torch.float32)
        self.check(self.lib.nbo_state_export(self.h, tensor, which, C.c_void_p(out.data_ptr())))
        return out

    def state_import(self, tensor: int, which: int, src: torch.Tensor):
        src = src.detach().to("cpu", torch.float32).contiguous()
        self.check(self.lib.nbo_state_import(self.h, tensor, which, C.c_void_p(src.data_ptr())))


# --------------------------------------------------------------------------- Optimizer trait

class Optimizer:
    """``trait Optimizer<T, B>`` (nabla-train/src/optim/core.rs:9-44), T = f32, B = Cuda."""

    _NAME = "Optimizer"
    _h: _Handle
    _numel: List[int]

    def step(self, params: Sequence[torch.Tensor], grads: Sequence[torch.Tensor]) -> None:
        assert len(params) == len(grads), f"nabla-train: {self._NAME} params/grads length mismatch"
        assert len(params) == len(self._numel), f"nabla-train: {self._NAME} params count mismatch"
        _check_tensors(params, torch.float32, "params")
        _check_tensors(grads, torch.float32, "grads")
        for i, (p, g) in enumerate(zip(params, grads)):
            if p.numel() != self._numel[i] or g.numel() != self._numel[i]:
                raise AssertionError(
                    f"nabla: axpy_inplace shapes must match (tensor {i}: expected {self._numel[i]} elements)")
        self.step_ptrs(_ptrs(params), _ptrs(grads))

    def step_ptrs(self, params_arr, grads_arr) -> None:
        """`step` on prebuilt ``c_void_p`` arrays of device pointers (no per-call list walk)."""
        self._h.check(self._h.lib.nbo_step(self._h.h, len(self._numel), params_arr, grads_arr))

    def step_slices(self, params: Sequence[torch.Tensor], grads: Sequence[torch.Tensor]) -> None:
        self.step(list(params), list(grads))

    def reset(self) -> None:
        self._h.check(self._h.lib.nbo_reset(self._h.h))

    def set_lr(self, lr: float) -> None:
        self._h.check(self._h.lib.nbo_set_lr(self._h.h, float(lr)))

    def zero_grad(self, grads: Sequence[torch.Tensor]) -> None:
        """Every gradient becomes zeros (nabla-ml/src/autograd/ops.rs:1668-1673)."""
        assert len(grads) == len(self._numel), f"nabla-train: {self._NAME} params count mismatch"
        self._h.check(self._h.lib.nbo_zero_grad(self._h.h, len(grads), _ptrs(grads)))

    # OptimState (core.rs:64-79): state tensors are named m{i} / v{i}
    def _state(self, i: int, which: int) -> torch.Tensor:
        return _as_state(self._h.state_export(i, which, self._numel[i]), self._shapes[i])

    def state_tensors(self) -> List[Tuple[str, torch.Tensor]]:
        """Named m{i} / v{i}, each with its parameter's (rows, cols) as in the reference (alg.rs:476-485)."""
        out = []
        for i in range(len(self._numel)):
            out.append((f"m{i}", self._state(i, 0)))
        for i in range(len(self._numel)):
            out.append((f"v{i}", self._state(i, 1)))
        return out

    def load_state_tensors(self, tensors: Sequence[Tuple[str, torch.Tensor]]) -> None:
        m = [None] * len(self._numel)
        v = [None] * len(self._numel)
        for name, t in tensors:
            for prefix, dst in (("m", m), ("v", v)):
                if name.startswith(prefix):
                    try:
                        i = int(name[1:])
                    except ValueError:
                        raise ValueError(f"bad tensor key: {name}")
                    if i >= len(dst):
                        raise ValueError(f"{prefix} index out of range: {i}")
                    dst[i] = t
                    break
        for i, t in enumerate(m):
            if t is None:
                raise ValueError(f"missing m{i}")
        for i, t in enumerate(v):
            if t is None:
                raise ValueError(f"missing v{i}")
        flat = [(_flat_state(m[i], n, f"m{i}"), _flat_state(v[i], n, f"v{i}")) for i, n in enumerate(self._numel)]
        for i, (mi, vi) in enumerate(flat):
            self._h.state_import(i, 0, mi)
            self._h.state_import(i, 1, vi)


class _Single(Optimizer):
    _KIND = L.NBO_ADAMW

    def __init__(self, lr: float, param_shapes: Sequence, *, device=None, stream=None, **defaults):
        self._numel = [_numel_of(s) for s in param_shapes]
        self._shapes = [_shape2d_of(s) for s in param_shapes]
        self._h = _Handle(device, stream)
        cfg = L.GroupConfig(kind=self._KIND, lr=float(lr), beta1=defaults.get("beta1", 0.0),
                            beta2=defaults.get("beta2", 0.0), eps=defaults.get("eps", 0.0),
                            weight_decay=defaults.get("weight_decay", 0.0),
                            momentum=defaults.get("momentum", 0.0))
        self._h.add_group(cfg)
        self._h.set_tensors(self._numel, None, L.NBO_F32)

    @classmethod
    def from_params(cls, lr: float, params: Sequence[torch.Tensor], **kw):
        dev = params[0].device.index if params and params[0].is_cuda else None
        return cls(lr, [tuple(p.shape) for p in params], device=dev, **kw)

    def _update(self, **kw):
        cfg = self._h.get_group(0)
        for k, v in kw.items():
            setattr(cfg, k, float(v))
        self._h.set_group(0, cfg)
        return self

    def lr(self) -> float:
        return self._h.get_group(0).lr

    def step_count(self) -> int:
        return self._h.step_count(0)


class AdamW(_Single):
    """``AdamW<f32, Cuda>`` (nabla-train/src/optim/alg.rs:7-167)."""
    _NAME, _KIND = "AdamW", L.NBO_ADAMW

    def __init__(self, lr, param_shapes, **kw):
        super().__init__(lr, param_shapes, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, **kw)

    def beta1(self, v): return self._update(beta1=v)
    def beta2(self, v): return self._update(beta2=v)
    def eps(self, v): return self._update(eps=v)
    def weight_decay(self, v): return self._update(weight_decay=v)

    def moments(self):
        n = len(self._numel)
        return ([self._h.state_export(i, 0, self._numel[i]) for i in range(n)],
                [self._h.state_export(i, 1, self._numel[i]) for i in range(n)])

    def set_state(self, step_count, beta1, beta2, eps, weight_decay, lr):
        self._update(beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, lr=lr)
        self._h.check(self._h.lib.nbo_set_step_count(self._h.h, 0, int(step_count)))


class Adam(_Single):
    """``Adam<f32, Cuda>`` (nabla-train/src/optim/alg.rs:169-308)."""
    _NAME, _KIND = "Adam", L.NBO_ADAM

    def __init__(self, lr, param_shapes, **kw):
        super().__init__(lr, param_shapes, beta1=0.9, beta2=0.999, eps=1e-8, **kw)

    def beta1(self, v): return self._update(beta1=v)
    def beta2(self, v): return self._update(beta2=v)
    def eps(self, v): return self._update(eps=v)
    moments = AdamW.moments

    def set_state(self, step_count, beta1, beta2, eps, lr):
        self._update(beta1=beta1, beta2=beta2, eps=eps, lr=lr)
        self._h.check(self._h.lib.nbo_set_step_count(self._h.h, 0, int(step_count)))


class Sgd(_Single):
    """``Sgd<f32, Cuda>`` (nabla-train/src/optim/alg.rs:310-428)."""
    _NAME, _KIND = "SGD", L.NBO_SGD

    def __init__(self, lr, param_shapes, **kw):
        super().__init__(lr, param_shapes, **kw)

    def momentum(self, v): return self._update(momentum=v)
    def weight_decay(self, v): return self._update(weight_decay=v)
    def momentum_value(self): return self._h.get_group(0).momentum
    def weight_decay_value(self): return self._h.get_group(0).weight_decay

    def velocity(self):
        return [self._h.state_export(i, 0, n) for i, n in enumerate(self._numel)]

    def set_state(self, lr, momentum, weight_decay):
        self._update(lr=lr, momentum=momentum, weight_decay=weight_decay)

    # Sgd names its velocity v{i} (alg.rs:620-640); it lives in state slot 0 here
    def state_tensors(self):
        return [(f"v{i}", self._state(i, 0)) for i in range(len(self._numel))]

    def load_state_tensors(self, tensors):
        v = [None] * len(self._numel)
        for name, t in tensors:
            if name.startswith("v"):
                try:
                    i = int(name[1:])
                except ValueError:
                    raise ValueError(f"bad tensor key: {name}")
                if i >= len(v):
                    raise ValueError(f"v index out of range: {i}")
                v[i] = t
        for i, t in enumerate(v):
            if t is None:
                raise ValueError(f"missing v{i}")
        flat = [_flat_state(t, self._numel[i], f"v{i}") for i, t in enumerate(v)]
        for i, t in enumerate(flat):
            self._h.state_import(i, 0, t)


def adamw_step(param: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor, lr: float, beta1: float,
               beta2: float, eps: float, weight_decay: float, step: int) -> None:
    """``adamw_step`` (nabla-train/src/optim/alg.rs:431-469): AdamW on one tensor with caller-owned m and v."""
    _check_tensors([param, grad, m, v], torch.float32, "adamw_step")
    n = param.numel()
    if not (grad.numel() == m.numel() == v.numel() == n):
        raise AssertionError("nabla: axpy_inplace shapes must match")
    stream = torch.cuda.current_stream(param.device).cuda_stream
    L.check(None, L.load().nbo_adamw_step(param.device.index, C.c_void_p(stream), C.c_void_p(param.data_ptr()),
                                          C.c_void_p(grad.data_ptr()), C.c_void_p(m.data_ptr()),
                                          C.c_void_p(v.data_ptr()), n, lr, beta1, beta2, eps, weight_decay, step))


# --------------------------------------------------------------------------- param groups

@dataclass
class ParamMatch:
    """``enum ParamMatch`` (groups.rs:11-17): kind is Equals / Prefix / Suffix / Contains."""
    kind: str
    value: str

    @staticmethod
    def Equals(v): return ParamMatch("Equals", v)
    @staticmethod
    def Prefix(v): return ParamMatch("Prefix", v)
    @staticmethod
    def Suffix(v): return ParamMatch("Suffix", v)
    @staticmethod
    def Contains(v): return ParamMatch("Contains", v)

    def matches(self, name: str) -> bool:
        return {"Equals": name == self.value, "Prefix": name.startswith(self.value),
                "Suffix": name.endswith(self.value), "Contains": self.value in name}[self.kind]


@dataclass
class ParamSelector:
    """``enum ParamSelector`` (groups.rs:19-38): All, or Any(list of ParamMatch)."""
    any_of: Optional[List[ParamMatch]] = None

    @staticmethod
    def All(): return ParamSelector(None)
    @staticmethod
    def Any(matches): return ParamSelector(list(matches))

    def matches(self, name: str) -> bool:
        return True if self.any_of is None else any(m.matches(name) for m in self.any_of)


@dataclass
class ParamGroupConfig:
    """``struct ParamGroupConfig`` with its constructors (groups.rs:40-127)."""
    name: str
    selector: ParamSelector
    kind: int
    lr: float
    weight_decay: float = 0.0
    momentum: float = 0.0
    beta1: float = 0.0
    beta2: float = 0.0
    eps: float = 0.0

    @staticmethod
    def adamw(name, selector, lr, weight_decay):
        return ParamGroupConfig(name, selector, L.NBO_ADAMW, lr, weight_decay, 0.0, 0.9, 0.999, 1e-8)

    @staticmethod
    def adam(name, selector, lr):
        return ParamGroupConfig(name, selector, L.NBO_ADAM, lr, 0.0, 0.0, 0.9, 0.999, 1e-8)

    @staticmethod
    def sgd(name, selector, lr, momentum, weight_decay):
        return ParamGroupConfig(name, selector, L.NBO_SGD, lr, weight_decay, momentum, 0.0, 0.0, 0.0)

    def betas(self, b1, b2):
        self.beta1, self.beta2 = b1, b2
        return self

    def to_c(self) -> L.GroupConfig:
        return L.GroupConfig(kind=self.kind, lr=self.lr, beta1=self.beta1, beta2=self.beta2, eps=self.eps,
                             weight_decay=self.weight_decay, momentum=self.momentum)


class ParamExclusionPreset:
    """``enum ParamExclusionPreset`` patterns (groups.rs:136-150)."""
    Bias = ("bias",)
    Norm = ("norm", "bn", "ln")
    Embedding = ("embed", "embedding")


def assign_groups(names: Sequence[str], groups: Sequence[ParamGroupConfig],
                  default_group: Optional[ParamGroupConfig]):
    """Routing of GroupOptimizer::from_named_params (groups.rs:168-218): first matching group wins,
    unmatched names go to the default group, empty groups are dropped, default group comes last.
    Returns (kept configs, group index per tensor)."""
    buckets = [[] for _ in groups]
    default_bucket: List[int] = []
    for i, name in enumerate(names):
        placed = False
        for gi, cfg in enumerate(groups):
            if cfg.selector.matches(name):
                buckets[gi].append(i)
                placed = True
                break
        if not placed:
            if default_group is None:
                raise ValueError("nabla-train: group assignment incomplete")
            default_bucket.append(i)
    kept: List[ParamGroupConfig] = []
    gid_of = [-1] * len(names)
    for cfg, idxs in list(zip(groups, buckets)) + ([(default_group, default_bucket)] if default_group else []):
        if not idxs:
            continue
        for i in idxs:
            gid_of[i] = len(kept)
        kept.append(cfg)
    return kept, gid_of


class GroupOptimizer(Optimizer):
    """``GroupOptimizer<f32, Cuda>`` (nabla-train/src/optim/groups.rs:152-313).

    The reference clones every member tensor into a per-group optimizer and back
    on each step; here a group is a hyper-parameter set plus a range of the
    device chunk list, and the step is one kernel launch per group."""
    _NAME = "GroupOptimizer"

    def __init__(self, names, shapes, groups, default_group=None, *, precision=L.NBO_F32, device=None,
                 stream=None):
        kept, gid_of = assign_groups(names, groups, default_group)
        self._numel = [_numel_of(s) for s in shapes]
        self._shapes = [_shape2d_of(s) for s in shapes]
        self._configs = kept
        self._gid_of = gid_of
        self._h = _Handle(device, stream)
        for cfg in kept:
            self._h.add_group(cfg.to_c())
        self._h.set_tensors(self._numel, gid_of, precision)

    @classmethod
    def from_named_params(cls, named: Sequence[Tuple[str, torch.Tensor]], groups, default_group=None, **kw):
        dev = named[0][1].device.index if named and named[0][1].is_cuda else None
        return cls([n for n, _ in named], [tuple(t.shape) for _, t in named], groups, default_group,
                   device=dev, **kw)

    @classmethod
    def adamw_with_decay_exclusions(cls, named, lr, weight_decay, exclude: Sequence[str], **kw):
        matches = []
        for s in exclude:
            matches += [ParamMatch.Suffix(s), ParamMatch.Contains(s)]
        no_decay = ParamGroupConfig.adamw("no_decay", ParamSelector.Any(matches), lr, 0.0)
        decay = ParamGroupConfig.adamw("decay", ParamSelector.All(), lr, weight_decay)
        return cls.from_named_params(named, [no_decay], decay, **kw)

    @classmethod
    def adamw_with_decay_presets(cls, named, lr, weight_decay, presets, **kw):
        pats = [p for preset in presets for p in preset]
        return cls.adamw_with_decay_exclusions(named, lr, weight_decay, pats, **kw)

    def groups(self) -> int:
        return len(self._configs)

    def group_lr(self, gid: int) -> float:
        return self._h.get_group(gid).lr

    def step_count(self, gid: int = 0) -> int:
        return self._h.step_count(gid)

    def state_tensors(self):
        out = []
        for gi, cfg in enumerate(self._configs):
            idxs = [i for i, g in enumerate(self._gid_of) if g == gi]
            if cfg.kind == L.NBO_SGD:
                for li, i in enumerate(idxs):
                    out.append((f"g{gi}.v{li}", self._state(i, 0)))
            else:
                for li, i in enumerate(idxs):
                    out.append((f"g{gi}.m{li}", self._state(i, 0)))
                for li, i in enumerate(idxs):
                    out.append((f"g{gi}.v{li}", self._state(i, 1)))
        return out


# --------------------------------------------------------------------------- schedules

@dataclass
class LrSchedule:
    """``enum LrSchedule`` (nabla-train/src/optim/core.rs:101-121)."""
    kind: int
    warmup_steps: int = 0
    total_steps: int = 0
    min_lr: float = 0.0
    max_lr: float = 0.0
    pct_start: float = 0.0
    step_size: int = 0
    gamma: float = 0.0

    @staticmethod
    def Cosine(warmup_steps, total_steps, min_lr):
        return LrSchedule(L.NBO_SCHED_COSINE, warmup_steps=warmup_steps, total_steps=total_steps, min_lr=min_lr)

    @staticmethod
    def Linear(warmup_steps, total_steps):
        return LrSchedule(L.NBO_SCHED_LINEAR, warmup_steps=warmup_steps, total_steps=total_steps)

    @staticmethod
    def OneCycle(max_lr, total_steps, pct_start):
        return LrSchedule(L.NBO_SCHED_ONECYCLE, max_lr=max_lr, total_steps=total_steps, pct_start=pct_start)

    @staticmethod
    def Step(step_size, gamma):
        return LrSchedule(L.NBO_SCHED_STEP, step_size=step_size, gamma=gamma)

    def to_c(self) -> L.LrScheduleC:
        return L.LrScheduleC(self.kind, self.warmup_steps, self.total_steps, self.min_lr, self.max_lr,
                             self.pct_start, self.step_size, self.gamma)


def lr_at_step(schedule: LrSchedule, base_lr: float, step: int) -> float:
    """``lr_at_step`` (nabla-train/src/optim/core.rs:130-173); pure host f64 math in the library."""
    out = C.c_double()
    sc = schedule.to_c()
    L.check(None, L.load().nbo_lr_at_step(C.byref(sc), float(base_lr), int(step), C.byref(out)))
    return out.value


# --------------------------------------------------------------------------- scaler / clip

class GradScaler:
    """``GradScaler`` (nabla-train/src/optim/core.rs:254-260,334-413) for fp32 device gradients."""

    def __init__(self, numel_or_grads: Sequence, *, device=None, stream=None):
        numel = [g.numel() if isinstance(g, torch.Tensor) else _numel_of(g) for g in numel_or_grads]
        if device is None and numel_or_grads and isinstance(numel_or_grads[0], torch.Tensor):
            device = numel_or_grads[0].device.index
        self._numel = numel
        self._h = _Handle(device, stream)
        self._h.add_group(L.GroupConfig(kind=L.NBO_SGD, lr=0.0))
        self._h.set_tensors(numel, None, L.NBO_F32)

    def scale_factor(self) -> float:
        return self.state().scale

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * torch.tensor(self.scale_factor(), dtype=loss.dtype, device=loss.device)

    def unscale_and_update(self, grads: Sequence[torch.Tensor]) -> bool:
        _check_tensors(grads, torch.float32, "grads")
        ok = C.c_int32()
        self._h.check(self._h.lib.nbo_unscale_and_update(self._h.h, len(grads), _ptrs(grads), C.byref(ok)))
        return bool(ok.value)

    def state(self) -> L.ScalerState:
        st = L.ScalerState()
        self._h.check(self._h.lib.nbo_scaler_get(self._h.h, C.byref(st)))
        return st

    def load_state(self, st: L.ScalerState) -> None:
        self._h.check(self._h.lib.nbo_scaler_set(self._h.h, C.byref(st)))


class GradClipper:
    """Holds the device table for repeated ``clip_grad_norm`` calls on one gradient list."""

    def __init__(self, numel_or_grads: Sequence, *, device=None, stream=None):
        self._sc = GradScaler(numel_or_grads, device=device, stream=stream)

    def clip_grad_norm(self, grads: Sequence[torch.Tensor], max_norm: float) -> float:
        _check_tensors(grads, torch.float32, "grads")
        h = self._sc._h
        norm = C.c_double()
        h.check(h.lib.nbo_clip_grad_norm(h.h, len(grads), _ptrs(grads), float(max_norm), C.byref(norm)))
        return norm.value

    def grad_norm(self, grads: Sequence[torch.Tensor]) -> Tuple[float, bool]:
        h = self._sc._h
        norm, bad = C.c_double(), C.c_int32()
        h.check(h.lib.nbo_grad_norm(h.h, len(grads), _ptrs(grads), C.byref(norm), C.byref(bad)))
        return norm.value, bool(bad.value)


def clip_grad_norm(grads: Sequence[torch.Tensor], max_norm: float) -> float:
    """``clip_grad_norm`` (nabla-train/src/trainer.rs:500-523): returns the pre-clip norm."""
    if max_norm <= 0.0:
        return 0.0
    return GradClipper(grads).clip_grad_norm(grads, max_norm)


# --------------------------------------------------------------------------- mixed precision

@dataclass
class StepOutcome:
    applied: bool
    nonfinite: bool
    grad_norm: float
    loss_scale: float
    step_count: int

    @staticmethod
    def from_c(r: L.StepResult) -> "StepOutcome":
        return StepOutcome(bool(r.applied), bool(r.nonfinite), r.grad_norm, r.loss_scale, r.step_count)


class MixedAdamW:
    """Mixed-precision Adam/AdamW: bf16 params and grads owned by the caller, fp32 master/m/v owned by
    the optimizer.  The reference has no such type (its Optimizer has one scalar type); one step is the
    composition GradScaler::unscale_and_update -> clip_grad_norm -> AdamW<f32>::step on the masters ->
    cast to bf16, in the order of Trainer::train_epoch_with_max_steps (trainer.rs:230-283)."""

    def __init__(self, names, shapes, groups: Sequence[ParamGroupConfig],
                 default_group: Optional[ParamGroupConfig] = None, *, device=None, stream=None,
                 grad_dtype: torch.dtype = torch.bfloat16):
        """`grad_dtype=torch.float32` takes fp32 gradients (e.g. accumulated over micro-batches in fp32)
        for the same bf16 params / fp32 master step."""
        kept, gid_of = assign_groups(names, groups, default_group)
        self._numel = [_numel_of(s) for s in shapes]
        self._shapes = [_shape2d_of(s) for s in shapes]
        self._configs, self._gid_of = kept, gid_of
        self._grad_dtype = grad_dtype
        self._h = _Handle(device, stream)
        for cfg in kept:
            self._h.add_group(cfg.to_c())
        self._h.set_tensors(self._numel, gid_of,
                            L.NBO_MIXED_BF16 if grad_dtype == torch.bfloat16 else L.NBO_MIXED_BF16_F32GRAD)

    @classmethod
    def adamw(cls, lr, weight_decay, shapes, **kw):
        names = [f"p{i}" for i in range(len(shapes))]
        return cls(names, shapes, [], ParamGroupConfig.adamw("all", ParamSelector.All(), lr, weight_decay), **kw)

    def init_master_from_params(self, params: Sequence[torch.Tensor]) -> None:
        _check_tensors(params, torch.bfloat16, "params")
        self._h.check(self._h.lib.nbo_init_master_from_params(self._h.h, len(params), _ptrs(params)))

    def load_master(self, i: int, values: torch.Tensor) -> None:
        self._h.state_import(i, 2, values.reshape(-1))

    def master(self, i: int) -> torch.Tensor:
        return self._h.state_export(i, 2, self._numel[i])

    def moments(self, i: int):
        return self._h.state_export(i, 0, self._numel[i]), self._h.state_export(i, 1, self._numel[i])

    def step(self, params, grads, *, use_scaler: bool = True, max_norm: float = 0.0) -> StepOutcome:
        assert len(params) == len(grads), "nabla-train: AdamW params/grads length mismatch"
        assert len(params) == len(self._numel), "nabla-train: AdamW params count mismatch"
        _check_tensors(params, torch.bfloat16, "params")
        _check_tensors(grads, self._grad_dtype, "grads")
        return self.step_ptrs(_ptrs(params), _ptrs(grads), use_scaler=use_scaler, max_norm=max_norm)

    def step_ptrs(self, params_arr, grads_arr, *, use_scaler=True, max_norm=0.0) -> StepOutcome:
        res = L.StepResult()
        self._h.check(self._h.lib.nbo_step_mixed(self._h.h, len(self._numel), params_arr, grads_arr,
                                                 1 if use_scaler else 0, float(max_norm), C.byref(res)))
        return StepOutcome.from_c(res)

    def step_host(self, params_dev, grads_dev, params_host, grads_host, *, use_scaler: bool = True,
                  max_norm: float = 0.0, slice_elems: int = 0) -> StepOutcome:
        """The same step for gradients and parameters that live in HOST memory (pinned, for overlap):
        gradients are copied in, updated and the bf16 parameters copied out slice by slice on three
        streams, so both PCIe directions run at once; `params_dev` / `grads_dev` are device staging
        tensors of the same shapes.  Returns when `params_host` is complete."""
        n = len(self._numel)
        assert len(params_dev) == len(grads_dev) == len(params_host) == len(grads_host) == n, \
            "nabla-train: AdamW params/grads length mismatch"
        _check_tensors(params_dev, torch.bfloat16, "params")
        _check_tensors(grads_dev, self._grad_dtype, "grads")
        for i, (p, g) in enumerate(zip(params_host, grads_host)):
            if p.is_cuda or g.is_cuda or p.dtype != torch.bfloat16 or g.dtype != self._grad_dtype \
                    or not p.is_contiguous() or not g.is_contiguous() \
                    or p.numel() != self._numel[i] or g.numel() != self._numel[i]:
                raise ValueError(f"host tensor {i}: expected contiguous CPU tensors of {self._numel[i]} elements")
        return self.step_host_ptrs(_ptrs(params_dev), _ptrs(grads_dev), _ptrs(params_host), _ptrs(grads_host),
                                   use_scaler=use_scaler, max_norm=max_norm, slice_elems=slice_elems)

    def step_host_ptrs(self, params_dev_arr, grads_dev_arr, params_host_arr, grads_host_arr, *,
                       use_scaler=True, max_norm=0.0, slice_elems=0) -> StepOutcome:
        res = L.StepResult()
        self._h.check(self._h.lib.nbo_step_mixed_host(
            self._h.h, len(self._numel), params_dev_arr, grads_dev_arr, params_host_arr, grads_host_arr,
            int(slice_elems), 1 if use_scaler else 0, float(max_norm), C.byref(res)))
        return StepOutcome.from_c(res)

    def step_async(self, params_arr, grads_arr, *, use_scaler=True, max_norm=0.0) -> None:
        """Enqueues one step and returns without waiting; the step counter, bias corrections and loss-scale
        bookkeeping advance on the device.  Every launch has constant arguments, so the call can be captured
        into a CUDA graph and replayed.  `collect()` (or any state accessor) hands the state back."""
        self._h.check(self._h.lib.nbo_step_mixed_async(self._h.h, len(self._numel), params_arr, grads_arr,
                                                       1 if use_scaler else 0, float(max_norm)))

    def collect(self):
        """(outcome of the most recent asynchronous step, asynchronous steps completed on the device)."""
        res, k = L.StepResult(), C.c_uint64()
        self._h.check(self._h.lib.nbo_step_mixed_collect(self._h.h, C.byref(res), C.byref(k)))
        return StepOutcome.from_c(res), k.value

    def set_lr(self, lr: float) -> None:
        self._h.check(self._h.lib.nbo_set_lr(self._h.h, float(lr)))

    def reset(self) -> None:
        self._h.check(self._h.lib.nbo_reset(self._h.h))

    def zero_grad(self, grads) -> None:
        self._h.check(self._h.lib.nbo_zero_grad(self._h.h, len(grads), _ptrs(grads)))

    def scaler_state(self) -> L.ScalerState:
        st = L.ScalerState()
        self._h.check(self._h.lib.nbo_scaler_get(self._h.h, C.byref(st)))
        return st

    def load_scaler_state(self, st: L.ScalerState) -> None:
        self._h.check(self._h.lib.nbo_scaler_set(self._h.h, C.byref(st)))

    def step_count(self, gid: int = 0) -> int:
        return self._h.step_count(gid)
