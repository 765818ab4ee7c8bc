"""ZeRO-1 sharded mixed-precision AdamW over NCCL, one process per GPU.

Replaces the reference's whole distributed layer (a two-rank in-process mean,
nabla-train/src/dist.rs:7-44).  The parameters and gradients live in two flat
bf16 buckets owned by the caller; each rank keeps fp32 master/m/v only for its
slice and a step is reduce-scatter(grads) -> fused local update -> all-gather(params).
The collectives are issued by the C library on its own NCCL communicator;
torch.distributed is only used to hand the NCCL unique id to the other ranks.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence, Tuple

import torch

from . import _lib as L
from .optim import (ParamGroupConfig, ParamSelector, StepOutcome, _flat_state, _Handle, _numel_of, _shape2d_of,
                    assign_groups)


def geometry(total: int, world: int) -> Tuple[int, int]:
    """(elements per rank, padded bucket length); pure host arithmetic in the library."""
    s, p = C.c_uint64(), C.c_uint64()
    L.check(None, L.load().nbo_zero1_geometry(int(total), int(world), C.byref(s), C.byref(p)))
    return s.value, p.value


def shard_pieces(numel: Sequence[int], rank: int, world: int):
    """The (tensor, offset-in-tensor, length) pieces of rank `rank`'s shard - the same intersection
    the library builds its table from.  Host-only helper, used by tests and tools."""
    total = sum(numel)
    shard, _ = geometry(total, world)
    begin, end = rank * shard, (rank + 1) * shard
    out, off = [], 0
    for t, n in enumerate(numel):
        lo, hi = max(off, begin), min(off + n, end)
        if hi > lo:
            out.append((t, lo - off, hi - lo))
        off += n
    return out


def exchange_unique_id(rank: int, world: int, group=None) -> Optional[bytes]:
    """Rank 0 creates the NCCL unique id; the others receive it through torch.distributed."""
    if world == 1:
        return None
    import torch.distributed as dist
    buf = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        raw = (C.c_uint8 * 128)()
        L.check(None, L.load().nbo_zero1_unique_id(raw))
        buf = torch.tensor(list(raw), dtype=torch.uint8)
    if dist.get_backend(group) == "nccl":
        dev = torch.device("cuda", torch.cuda.current_device())
        t = buf.to(dev)
        dist.broadcast(t, src=0, group=group)
        buf = t.cpu()
    else:
        dist.broadcast(buf, src=0, group=group)
    return bytes(buf.tolist())


class _RawDeviceMemory:
    """Zero-copy handle on device memory the library allocated, for torch.as_tensor."""

    def __init__(self, ptr: int, n_int16: int):
        self.__cuda_array_interface__ = {"shape": (n_int16,), "typestr": "<i2", "data": (ptr, False), "version": 2}


def _device_view(ptr: int, elems: int, device: int) -> torch.Tensor:
    """A bf16 torch view of `elems` elements at device address `ptr` (memory owned by the library)."""
    t = torch.as_tensor(_RawDeviceMemory(ptr, elems), device=torch.device("cuda", device))
    assert t.data_ptr() == ptr
    return t.view(torch.bfloat16)


class Zero1AdamW:
    """Sharded mixed-precision Adam/AdamW on flat bf16 buckets."""

    def __init__(self, names, shapes, groups: Sequence[ParamGroupConfig],
                 default_group: Optional[ParamGroupConfig], rank: int, world: int,
                 unique_id: Optional[bytes] = None, *, device=None, stream=None, timeout_s: Optional[float] = None):
        kept, gid_of = assign_groups(names, groups, default_group)
        self._numel = [_numel_of(s) for s in shapes]
        self._shapes = [_shape2d_of(s) for s in shapes]
        self._configs, self._gid_of = kept, gid_of
        self.total = sum(self._numel)
        self.rank, self.world = rank, world
        self.shard, self.padded = geometry(self.total, world)
        self._h = _Handle(device, stream)
        for cfg in kept:
            self._h.add_group(cfg.to_c())
        n = len(self._numel)
        arr = (C.c_uint64 * n)(*self._numel)
        gids = (C.c_int32 * n)(*gid_of)
        uid = (C.c_uint8 * 128)(*unique_id) if unique_id is not None else None
        if timeout_s is not None:
            self._h.check(self._h.lib.nbo_zero1_set_timeout(self._h.h, float(timeout_s)))
        self._h.check(self._h.lib.nbo_zero1_init(self._h.h, n, arr, gids, rank, world, uid))

    @classmethod
    def adamw(cls, lr, weight_decay, shapes, rank, world, unique_id=None, **kw):
        names = [f"p{i}" for i in range(len(shapes))]
        return cls(names, shapes, [], ParamGroupConfig.adamw("all", ParamSelector.All(), lr, weight_decay),
                   rank, world, unique_id, **kw)

    def set_timeout(self, seconds: float) -> None:
        """Host-side limit for each sharded step; on expiry the step raises with status NBO_ERR_TIMEOUT."""
        self._h.check(self._h.lib.nbo_zero1_set_timeout(self._h.h, float(seconds)))

    def shard_range(self) -> Tuple[int, int, int]:
        b, e, p = C.c_uint64(), C.c_uint64(), C.c_uint64()
        self._h.check(self._h.lib.nbo_zero1_shard(self._h.h, C.byref(b), C.byref(e), C.byref(p)))
        return b.value, e.value, p.value

    def _check_bucket(self, t: torch.Tensor, what: str):
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous() and t.numel() == self.padded):
            raise ValueError(f"{what} must be a contiguous CUDA bf16 tensor of {self.padded} elements")

    def init_master(self, params_flat: torch.Tensor) -> None:
        self._check_bucket(params_flat, "params_flat")
        self._h.check(self._h.lib.nbo_zero1_init_master(self._h.h, C.c_void_p(params_flat.data_ptr())))

    def step(self, params_flat: torch.Tensor, grads_flat: torch.Tensor, *, average: bool = False,
             use_scaler: bool = False, max_norm: float = 0.0) -> StepOutcome:
        self._check_bucket(params_flat, "params_flat")
        self._check_bucket(grads_flat, "grads_flat")
        return self.step_ptrs(params_flat.data_ptr(), grads_flat.data_ptr(), average=average,
                              use_scaler=use_scaler, max_norm=max_norm)

    def step_ptrs(self, params_ptr: int, grads_ptr: int, *, average=False, use_scaler=False,
                  max_norm=0.0) -> StepOutcome:
        res = L.StepResult()
        self._h.check(self._h.lib.nbo_zero1_step(self._h.h, C.c_void_p(params_ptr), C.c_void_p(grads_ptr),
                                                 1 if average else 0, 1 if use_scaler else 0,
                                                 float(max_norm), C.byref(res)))
        return StepOutcome.from_c(res)

    def step_host_ptrs(self, params_ptr: int, grads_ptr: int, params_host_arr, grads_host_arr, *,
                       average=False, use_scaler=False, max_norm=0.0, slice_elems=0) -> StepOutcome:
        """Gradients come from, and parameters return to, HOST tensors (one pointer per declared tensor,
        `_lib.ptr_array`), pipelined slice by slice through the two flat device buckets.  With world > 1 the
        buckets are the attached symmetric ones, every rank passes its own gradients for the whole list and
        gets the parameters of its own shard back."""
        res = L.StepResult()
        self._h.check(self._h.lib.nbo_zero1_step_host(
            self._h.h, C.c_void_p(params_ptr), C.c_void_p(grads_ptr), len(params_host_arr), params_host_arr,
            grads_host_arr, int(slice_elems), 1 if average else 0, 1 if use_scaler else 0, float(max_norm),
            C.byref(res)))
        return StepOutcome.from_c(res)

    def keep_reduced_grads(self, on: bool) -> None:
        """Fused step: whether the reduced gradient is also written into this rank's slice of its bucket."""
        self._h.check(self._h.lib.nbo_zero1_keep_reduced_grads(self._h.h, 1 if on else 0))

    # ---- fused path over NVLink / NVSwitch peer memory -------------------------------------------
    def attach_symmetric(self, group=None, transport: int = 0):
        """Allocates the two flat bf16 buckets in symmetric memory (torch.distributed._symmetric_memory:
        every rank's buffer mapped into every process, plus an NVSwitch multicast mapping when the fabric
        offers one) and registers them for `step_fused`.  Returns (params_flat, grads_flat); the caller
        fills them like ordinary tensors.  transport: 0 = choose, 1 = peer loads/stores, 2 = multicast."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        dev = torch.device("cuda", self._h.device)
        bufs, handles = [], []
        for _ in range(2):
            t = symm.empty(self.padded, dtype=torch.bfloat16, device=dev)
            hd = symm.rendezvous(t, group.group_name)
            t.zero_()
            bufs.append(t)
            handles.append(hd)
        (pflat, gflat), (ph, gh) = bufs, handles
        if gh.buffer_ptrs[self.rank] != gflat.data_ptr() or ph.buffer_ptrs[self.rank] != pflat.data_ptr():
            raise RuntimeError("symmetric memory: buffer_ptrs[rank] is not the local allocation")
        gp = L.ptr_array(list(gh.buffer_ptrs))
        pp = L.ptr_array(list(ph.buffer_ptrs))
        gmc = C.c_void_p(gh.multicast_ptr) if gh.multicast_ptr else None
        pmc = C.c_void_p(ph.multicast_ptr) if ph.multicast_ptr else None
        self._h.check(self._h.lib.nbo_zero1_attach_symmetric(
            self._h.h, C.c_void_p(gflat.data_ptr()), gp, gmc, C.c_void_p(pflat.data_ptr()), pp, pmc, transport))
        self._symm = (pflat, gflat, ph, gh)          # keep the mappings alive
        self.peer_grad_ptrs = list(gh.buffer_ptrs)
        self.has_multicast = bool(gh.multicast_ptr and ph.multicast_ptr)
        torch.cuda.synchronize()
        dist.barrier(group)
        return pflat, gflat

    def attach_symmetric_native(self, group=None, transport: int = 0, want_multicast: bool = True,
                                timeout_s: float = 60.0):
        """`attach_symmetric` without torch's symmetric-memory module: the two buckets are made by the
        library itself (nbo_symm_alloc: CUDA virtual-memory allocations mapped into every rank, bound to an
        NVSwitch multicast object where the fabric has one).  torch.distributed only carries the 16-byte
        token from rank 0 to the others.  Returns (params_flat, grads_flat) as torch views of that memory;
        call `release_symmetric()` on every rank before the process ends."""
        import torch.distributed as dist
        lib = self._h.lib
        tok = torch.zeros(16, dtype=torch.uint8)
        if self.rank == 0:
            raw = (C.c_uint8 * 16)()
            L.check(None, lib.nbo_symm_token(raw))
            tok = torch.tensor(list(raw), dtype=torch.uint8)
        if self.world > 1:
            if dist.get_backend(group) == "nccl":
                t = tok.to(torch.device("cuda", self._h.device))
                dist.broadcast(t, src=0, group=group)
                tok = t.cpu()
            else:
                dist.broadcast(tok, src=0, group=group)
        token = (C.c_uint8 * 16)(*tok.tolist())
        self._native_tag = getattr(Zero1AdamW, "_next_symm_tag", 0)
        Zero1AdamW._next_symm_tag = self._native_tag + 2
        handles, views, peers, mcs = [], [], [], []
        for k in range(2):                                   # 0: params, 1: grads
            sh = C.c_void_p()
            L.check(None, lib.nbo_symm_alloc(self._h.device, self.rank, self.world, 2 * self.padded, token,
                                             self._native_tag + k, 1 if want_multicast else 0, float(timeout_s),
                                             C.byref(sh)))
            handles.append(sh)
            local, mc = C.c_void_p(), C.c_void_p()
            pp = (C.c_void_p * self.world)()
            L.check(None, lib.nbo_symm_pointers(sh, C.byref(local), pp, C.byref(mc)))
            views.append(_device_view(local.value, self.padded, self._h.device))
            peers.append(pp)
            mcs.append(mc)
        self._native = handles
        (pflat, gflat), (pp, gp), (pmc, gmc) = views, peers, mcs
        pflat.zero_(); gflat.zero_()
        self._h.check(lib.nbo_zero1_attach_symmetric(
            self._h.h, C.c_void_p(gflat.data_ptr()), gp, gmc if gmc.value else None,
            C.c_void_p(pflat.data_ptr()), pp, pmc if pmc.value else None, transport))
        self.has_multicast = bool(gmc.value and pmc.value)
        self.peer_grad_ptrs = [gp[r] for r in range(self.world)]
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group)
        return pflat, gflat

    def release_symmetric(self, group=None) -> None:
        """Frees the buckets made by `attach_symmetric_native` (unbinds them from the multicast object first).
        Collective in effect: every rank calls it once no rank uses the buckets any more."""
        handles = getattr(self, "_native", None)
        if not handles:
            return
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group)
        self._h.close()                                      # the handle's tables point into the buckets
        for sh in handles:
            L.check(None, self._h.lib.nbo_symm_free(sh))
        self._native = None

    def step_fused(self, *, average: bool = False, use_scaler: bool = False, max_norm: float = 0.0) -> StepOutcome:
        """One step on the attached buckets with reduce-scatter and all-gather fused into the kernels."""
        res = L.StepResult()
        self._h.check(self._h.lib.nbo_zero1_step_fused(self._h.h, 1 if average else 0, 1 if use_scaler else 0,
                                                       float(max_norm), C.byref(res)))
        return StepOutcome.from_c(res)

    def step_fused_async(self, *, average: bool = False, use_scaler: bool = False, max_norm: float = 0.0) -> None:
        """Enqueues one fused sharded step and returns without waiting; `collect()` hands the state back."""
        self._h.check(self._h.lib.nbo_zero1_step_fused_async(self._h.h, 1 if average else 0, 1 if use_scaler else 0,
                                                             float(max_norm)))

    def collect(self):
        """(outcome of the most recent asynchronous step, asynchronous steps completed on the device)."""
        res, k = L.StepResult(), C.c_uint64()
        self._h.check(self._h.lib.nbo_step_mixed_collect(self._h.h, C.byref(res), C.byref(k)))
        return StepOutcome.from_c(res), k.value

    def state_shard(self, which: int) -> torch.Tensor:
        """fp32 state of this rank's shard on the host: 0 = m, 1 = v, 2 = master."""
        out = torch.empty(self.shard, dtype=torch.float32)
        self._h.check(self._h.lib.nbo_zero1_state_export(self._h.h, which, C.c_void_p(out.data_ptr())))
        return out

    def load_state_shard(self, which: int, values: torch.Tensor) -> None:
        v = values.detach().to("cpu", torch.float32).contiguous()
        if v.numel() != self.shard:
            raise ValueError(f"expected {self.shard} floats for this rank's shard")
        self._h.check(self._h.lib.nbo_zero1_state_import(self._h.h, which, C.c_void_p(v.data_ptr())))

    # ---- checkpoint: stitch the shards back into the reference's per-tensor state names ----------
    def state_tensors(self, group=None):
        """On rank 0: [(name, tensor)] with the names a GroupOptimizer uses (g{k}.m{i} / g{k}.v{i}) plus the
        fp32 masters as g{k}.w{i}, each with its parameter's (rows, cols); None on the other ranks.  The
        shards travel through the host."""
        full = []
        for which in (0, 1, 2):
            shard = self.state_shard(which)
            if self.world == 1:
                full.append(shard[:self.total])
                continue
            import torch.distributed as dist
            parts = [None] * self.world if self.rank == 0 else None
            dist.gather_object(shard, parts, dst=0, group=group)
            full.append(torch.cat(parts)[:self.total] if self.rank == 0 else None)
        if self.rank != 0:
            return None
        offs, out = [0], []
        for n in self._numel:
            offs.append(offs[-1] + n)
        for gi in range(len(self._configs)):
            idx = [i for i, g in enumerate(self._gid_of) if g == gi]
            for which, p in ((0, "m"), (1, "v"), (2, "w")):
                for li, i in enumerate(idx):
                    out.append((f"g{gi}.{p}{li}", full[which][offs[i]:offs[i + 1]].clone().reshape(self._shapes[i])))
        return out

    def load_state_tensors(self, tensors) -> None:
        """Every rank passes the full per-tensor list (as loaded from optim.nbla) and keeps its own slice."""
        offs = [0]
        for n in self._numel:
            offs.append(offs[-1] + n)
        byname = {n: torch.as_tensor(t, dtype=torch.float32) for n, t in tensors}
        b = self.rank * self.shard
        for which, p in ((0, "m"), (1, "v"), (2, "w")):
            flat = torch.zeros(self.padded, dtype=torch.float32)
            for gi in range(len(self._configs)):
                idx = [i for i, g in enumerate(self._gid_of) if g == gi]
                for li, i in enumerate(idx):
                    key = f"g{gi}.{p}{li}"
                    if key not in byname:
                        raise ValueError(f"missing {p}{li}")
                    flat[offs[i]:offs[i + 1]] = _flat_state(byname[key], self._numel[i], key)
            self.load_state_shard(which, flat[b:b + self.shard])

    def scaler_state(self) -> L.ScalerState:
        st = L.ScalerState()
        self._h.check(self._h.lib.nbo_scaler_get(self._h.h, C.byref(st)))
        return st

    def load_scaler_state(self, st: L.ScalerState) -> None:
        self._h.check(self._h.lib.nbo_scaler_set(self._h.h, C.byref(st)))

    def set_lr(self, lr: float) -> None:
        self._h.check(self._h.lib.nbo_set_lr(self._h.h, float(lr)))

    def step_count(self, gid: int = 0) -> int:
        return self._h.step_count(gid)

    def launch_count(self) -> int:
        return self._h.launch_count()
