"""ctypes binding of libnabla_optim_b200.so (the C ABI in include/nabla_optim_b200.h).

The shared library is built ahead of time by ``nabla_b200/csrc/Makefile`` (nvcc,
sm_100a).  There is no Python or CPU fallback: if the library is missing, or no
CUDA device is present when an optimizer is created, an error is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# NABLA_OPTIM_B200_LIB names another build of the library (same ABI), e.g. one kept outside the package.
LIB_PATH = os.environ.get("NABLA_OPTIM_B200_LIB") or os.path.join(_HERE, "libnabla_optim_b200.so")

NBO_OK = 0
NBO_ERR_INVALID, NBO_ERR_CUDA, NBO_ERR_NCCL, NBO_ERR_TIMEOUT, NBO_ERR_STATE, NBO_ERR_NOMEM = 1, 2, 3, 4, 5, 6
NBO_ADAMW, NBO_ADAM, NBO_SGD = 0, 1, 2
NBO_F32, NBO_MIXED_BF16, NBO_MIXED_BF16_F32GRAD = 0, 1, 2
NBO_SCHED_COSINE, NBO_SCHED_LINEAR, NBO_SCHED_ONECYCLE, NBO_SCHED_STEP = 0, 1, 2, 3


class GroupConfig(C.Structure):
    _fields_ = [("kind", C.c_int32), ("lr", C.c_double), ("beta1", C.c_double), ("beta2", C.c_double),
                ("eps", C.c_double), ("weight_decay", C.c_double), ("momentum", C.c_double)]


class ScalerState(C.Structure):
    _fields_ = [("scale", C.c_double), ("growth_factor", C.c_double), ("backoff_factor", C.c_double),
                ("growth_interval", C.c_uint64), ("consecutive_ok", C.c_uint64)]


class LrScheduleC(C.Structure):
    _fields_ = [("kind", C.c_int32), ("warmup_steps", C.c_uint64), ("total_steps", C.c_uint64),
                ("min_lr", C.c_double), ("max_lr", C.c_double), ("pct_start", C.c_double),
                ("step_size", C.c_uint64), ("gamma", C.c_double)]


class StepResult(C.Structure):
    _fields_ = [("applied", C.c_int32), ("nonfinite", C.c_int32), ("grad_norm", C.c_double),
                ("loss_scale", C.c_double), ("step_count", C.c_uint64)]


class NablaOptimError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[nbo status {code}] {message}")
        self.code = code
        self.message = message


_H = C.c_void_p
_PP = C.POINTER(C.c_void_p)
_U64P = C.POINTER(C.c_uint64)
_I32P = C.POINTER(C.c_int32)
_F32P = C.POINTER(C.c_float)
_F64P = C.POINTER(C.c_double)

# name -> (restype, argtypes); every symbol include/nabla_optim_b200.h declares
SIGNATURES = {
    "nbo_abi_version": (C.c_int32, []),
    "nbo_last_error": (C.c_char_p, [_H]),
    "nbo_create": (C.c_int32, [C.c_int32, C.c_void_p, C.POINTER(_H)]),
    "nbo_destroy": (C.c_int32, [_H]),
    "nbo_add_group": (C.c_int32, [_H, C.POINTER(GroupConfig), _I32P]),
    "nbo_set_tensors": (C.c_int32, [_H, C.c_uint64, _U64P, _I32P, C.c_int32]),
    "nbo_step": (C.c_int32, [_H, C.c_uint64, _PP, _PP]),
    "nbo_adamw_step": (C.c_int32, [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64,
                                   C.c_double, C.c_double, C.c_double, C.c_double, C.c_double, C.c_uint64]),
    "nbo_reset": (C.c_int32, [_H]),
    "nbo_set_lr": (C.c_int32, [_H, C.c_double]),
    "nbo_get_lr": (C.c_int32, [_H, C.c_int32, _F64P]),
    "nbo_zero_grad": (C.c_int32, [_H, C.c_uint64, _PP]),
    "nbo_accumulate_grads": (C.c_int32, [_H, C.c_uint64, _PP, _PP]),
    "nbo_step_count": (C.c_int32, [_H, C.c_int32, _U64P]),
    "nbo_set_step_count": (C.c_int32, [_H, C.c_int32, C.c_uint64]),
    "nbo_get_group": (C.c_int32, [_H, C.c_int32, C.POINTER(GroupConfig)]),
    "nbo_set_group": (C.c_int32, [_H, C.c_int32, C.POINTER(GroupConfig)]),
    "nbo_state_export": (C.c_int32, [_H, C.c_uint64, C.c_int32, C.c_void_p]),
    "nbo_state_import": (C.c_int32, [_H, C.c_uint64, C.c_int32, C.c_void_p]),
    "nbo_scaler_get": (C.c_int32, [_H, C.POINTER(ScalerState)]),
    "nbo_scaler_set": (C.c_int32, [_H, C.POINTER(ScalerState)]),
    "nbo_unscale_and_update": (C.c_int32, [_H, C.c_uint64, _PP, _I32P]),
    "nbo_clip_grad_norm": (C.c_int32, [_H, C.c_uint64, _PP, C.c_double, _F64P]),
    "nbo_grad_norm": (C.c_int32, [_H, C.c_uint64, _PP, _F64P, _I32P]),
    "nbo_grad_norm_noalloc": (C.c_int32, [C.c_int32, C.c_void_p, C.c_void_p, C.c_uint64, C.c_int32, C.c_float,
                                          C.c_void_p]),
    "nbo_init_master_from_params": (C.c_int32, [_H, C.c_uint64, _PP]),
    "nbo_step_mixed": (C.c_int32, [_H, C.c_uint64, _PP, _PP, C.c_int32, C.c_double, C.POINTER(StepResult)]),
    "nbo_step_mixed_async": (C.c_int32, [_H, C.c_uint64, _PP, _PP, C.c_int32, C.c_double]),
    "nbo_step_mixed_collect": (C.c_int32, [_H, C.POINTER(StepResult), _U64P]),
    "nbo_step_mixed_host": (C.c_int32, [_H, C.c_uint64, _PP, _PP, _PP, _PP, C.c_uint64, C.c_int32, C.c_double,
                                        C.POINTER(StepResult)]),
    "nbo_lr_at_step": (C.c_int32, [C.POINTER(LrScheduleC), C.c_double, C.c_uint64, _F64P]),
    "nbo_zero1_unique_id": (C.c_int32, [C.c_void_p]),
    "nbo_zero1_geometry": (C.c_int32, [C.c_uint64, C.c_int32, _U64P, _U64P]),
    "nbo_zero1_init": (C.c_int32, [_H, C.c_uint64, _U64P, _I32P, C.c_int32, C.c_int32, C.c_void_p]),
    "nbo_zero1_set_timeout": (C.c_int32, [_H, C.c_double]),
    "nbo_zero1_init_master": (C.c_int32, [_H, C.c_void_p]),
    "nbo_zero1_step": (C.c_int32, [_H, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_double,
                                   C.POINTER(StepResult)]),
    "nbo_zero1_step_host": (C.c_int32, [_H, C.c_void_p, C.c_void_p, C.c_uint64, _PP, _PP, C.c_uint64, C.c_int32,
                                        C.c_int32, C.c_double, C.POINTER(StepResult)]),
    "nbo_zero1_step_fused_async": (C.c_int32, [_H, C.c_int32, C.c_int32, C.c_double]),
    "nbo_zero1_keep_reduced_grads": (C.c_int32, [_H, C.c_int32]),
    "nbo_symm_token": (C.c_int32, [C.c_void_p]),
    "nbo_symm_alloc": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_uint64, C.c_void_p, C.c_int32, C.c_int32,
                                   C.c_double, C.POINTER(C.c_void_p)]),
    "nbo_symm_pointers": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), _PP, C.POINTER(C.c_void_p)]),
    "nbo_symm_free": (C.c_int32, [C.c_void_p]),
    "nbo_copy_probe": (C.c_int32, [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64]),
    "nbo_zero1_attach_symmetric": (C.c_int32, [_H, C.c_void_p, _PP, C.c_void_p, C.c_void_p, _PP, C.c_void_p,
                                               C.c_int32]),
    "nbo_zero1_step_fused": (C.c_int32, [_H, C.c_int32, C.c_int32, C.c_double, C.POINTER(StepResult)]),
    "nbo_zero1_shard": (C.c_int32, [_H, _U64P, _U64P, _U64P]),
    "nbo_zero1_state_export": (C.c_int32, [_H, C.c_int32, C.c_void_p]),
    "nbo_zero1_state_import": (C.c_int32, [_H, C.c_int32, C.c_void_p]),
    "nbo_profile": (C.c_int32, [_H, C.c_int32]),
    "nbo_profile_last": (C.c_int32, [_H, _F32P, _F32P]),
    "nbo_launch_count": (C.c_int32, [_H, _U64P]),
    "nbo_table_info": (C.c_int32, [_H, _U64P, _U64P, _U64P]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library (once) and types every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C nabla_b200/csrc` "
            "(there is no CPU or Python fallback for the optimizer kernels)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(handle, status: int) -> None:
    if status != NBO_OK:
        msg = load().nbo_last_error(handle)
        raise NablaOptimError(status, msg.decode() if msg else "")


def ptr_array(ptrs) -> C.Array:
    return (C.c_void_p * len(ptrs))(*ptrs)
