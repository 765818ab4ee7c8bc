"""ctypes binding of the CPU oracle (oracle/nabla_oracle.c) - TEST INFRASTRUCTURE.

Only tests/, the smoke check and the benchmark's CPU-baseline leg import this.
Arrays are numpy; float32/float64 pick the _f32/_f64 variant of each function.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnabla_oracle.so")


def build(force: bool = False) -> str:
    src = [os.path.join(_HERE, f) for f in ("nabla_oracle.c", "oracle_body.inc", "Makefile")]
    stale = force or not os.path.exists(LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(LIB_PATH) for s in src)
    if stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return LIB_PATH


class Scaler(C.Structure):
    _fields_ = [("scale", C.c_double), ("growth_factor", C.c_double), ("backoff_factor", C.c_double),
                ("growth_interval", C.c_uint64), ("consecutive_ok", C.c_uint64)]


class Schedule(C.Structure):
    _fields_ = [("kind", C.c_int32), ("warmup_steps", C.c_uint64), ("total_steps", C.c_uint64),
                ("min_lr", C.c_double), ("max_lr", C.c_double), ("pct_start", C.c_double),
                ("step_size", C.c_uint64), ("gamma", C.c_double)]


class AdamCfg(C.Structure):
    _fields_ = [("lr", C.c_double), ("beta1", C.c_double), ("beta2", C.c_double), ("eps", C.c_double),
                ("weight_decay", C.c_double), ("decoupled", C.c_int32)]


_lib = None
_VP = C.c_void_p


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        l = C.CDLL(LIB_PATH)
        l.orc_powi.restype = C.c_double
        l.orc_powi.argtypes = [C.c_double, C.c_int32]
        l.orc_bf16_from_f32.restype = C.c_uint16
        l.orc_bf16_from_f32.argtypes = [C.c_float]
        l.orc_bf16_to_f32.restype = C.c_float
        l.orc_bf16_to_f32.argtypes = [C.c_uint16]
        l.orc_bf16_from_f32_array.argtypes = [_VP, _VP, C.c_uint64]
        l.orc_bf16_to_f32_array.argtypes = [_VP, _VP, C.c_uint64]
        l.orc_scaler_init.argtypes = [C.POINTER(Scaler)]
        l.orc_lr_at_step.restype = C.c_double
        l.orc_lr_at_step.argtypes = [C.POINTER(Schedule), C.c_double, C.c_uint64]
        for suf in ("f32", "f64"):
            f = getattr(l, f"orc_adam_step_{suf}")
            f.argtypes = [_VP, _VP, _VP, _VP, C.c_uint64, C.c_double, C.c_double, C.c_double, C.c_double,
                          C.c_double, C.c_uint64, C.c_int]
            f.restype = None
            f = getattr(l, f"orc_sgd_step_{suf}")
            f.argtypes = [_VP, _VP, _VP, C.c_uint64, C.c_double, C.c_double, C.c_double]
            f.restype = None
            f = getattr(l, f"orc_scaler_unscale_and_update_{suf}")
            f.argtypes = [C.POINTER(Scaler), _VP, _VP, C.c_uint64]
            f.restype = C.c_int
            f = getattr(l, f"orc_clip_grad_norm_{suf}")
            f.argtypes = [_VP, _VP, C.c_uint64, C.c_double]
            f.restype = C.c_double
            f = getattr(l, f"orc_has_non_finite_{suf}")
            f.argtypes = [_VP, _VP, C.c_uint64]
            f.restype = C.c_int
        l.orc_adam_step_passes_f32.argtypes = l.orc_adam_step_f32.argtypes
        l.orc_adam_step_passes_f32.restype = None
        l.orc_mixed_adamw_step.argtypes = [_VP, _VP, _VP, _VP, _VP, _VP, C.c_uint64, C.POINTER(AdamCfg),
                                           C.POINTER(C.c_uint64), C.POINTER(Scaler), C.c_int, C.c_double,
                                           C.POINTER(C.c_double), C.c_int]
        l.orc_mixed_adamw_step.restype = C.c_int
        _lib = l
    return _lib


def _suf(a: np.ndarray) -> str:
    if a.dtype == np.float32:
        return "f32"
    if a.dtype == np.float64:
        return "f64"
    raise TypeError(a.dtype)


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_VP)


def _plist(arrs):
    return (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])


def _nlist(arrs):
    return (C.c_uint64 * len(arrs))(*[a.size for a in arrs])


def powi(a: float, b: int) -> float:
    return lib().orc_powi(a, b)


def adam_step(p, g, m, v, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, decoupled=False,
              passes=False):
    """One Adam (decoupled=False) / AdamW (True) update of one tensor, in place."""
    s = _suf(p)
    fn = lib().orc_adam_step_passes_f32 if passes else getattr(lib(), f"orc_adam_step_{s}")
    fn(_p(p), _p(g), _p(m), _p(v), p.size, lr, beta1, beta2, eps, weight_decay, step, int(decoupled))


def sgd_step(p, g, vel, lr, momentum=0.0, weight_decay=0.0):
    getattr(lib(), f"orc_sgd_step_{_suf(p)}")(_p(p), _p(g), _p(vel), p.size, lr, momentum, weight_decay)


def new_scaler() -> Scaler:
    s = Scaler()
    lib().orc_scaler_init(C.byref(s))
    return s


def scaler_unscale_and_update(sc: Scaler, grads) -> bool:
    fn = getattr(lib(), f"orc_scaler_unscale_and_update_{_suf(grads[0])}")
    return bool(fn(C.byref(sc), _plist(grads), _nlist(grads), len(grads)))


def clip_grad_norm(grads, max_norm: float) -> float:
    fn = getattr(lib(), f"orc_clip_grad_norm_{_suf(grads[0])}")
    return fn(_plist(grads), _nlist(grads), len(grads), max_norm)


def has_non_finite(grads) -> bool:
    fn = getattr(lib(), f"orc_has_non_finite_{_suf(grads[0])}")
    return bool(fn(_plist(grads), _nlist(grads), len(grads)))


def lr_at_step(kind, base_lr, step, warmup_steps=0, total_steps=0, min_lr=0.0, max_lr=0.0, pct_start=0.0,
               step_size=0, gamma=0.0) -> float:
    sc = Schedule(kind, warmup_steps, total_steps, min_lr, max_lr, pct_start, step_size, gamma)
    return lib().orc_lr_at_step(C.byref(sc), base_lr, step)


def bf16_from_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_bf16_from_f32_array(_p(out), _p(a), a.size)
    return out


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().orc_bf16_to_f32_array(_p(out), _p(a), a.size)
    return out


class MixedOracle:
    """State holder for the mixed-precision composition (see orc_mixed_adamw_step)."""

    def __init__(self, masters, cfgs, use_scaler=True):
        self.master = [np.ascontiguousarray(w, dtype=np.float32).copy() for w in masters]
        self.m = [np.zeros_like(w) for w in self.master]
        self.v = [np.zeros_like(w) for w in self.master]
        self.p = [bf16_from_f32(w) for w in self.master]
        self.cfgs = (AdamCfg * len(cfgs))(*cfgs)
        self.step_count = C.c_uint64(0)
        self.scaler = new_scaler()
        self.use_scaler = use_scaler

    def step(self, grads_bf16, max_norm=0.0, passes=False):
        norm = C.c_double()
        ok = lib().orc_mixed_adamw_step(_plist(self.p), _plist(grads_bf16), _plist(self.master),
                                        _plist(self.m), _plist(self.v), _nlist(self.master),
                                        len(self.master), self.cfgs, C.byref(self.step_count),
                                        C.byref(self.scaler), int(self.use_scaler), max_norm,
                                        C.byref(norm), int(passes))
        return bool(ok), norm.value
