#!/usr/bin/env python
"""Benchmark of the optimizer-step hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (`llama8b_zero1`): the Llama-3-8B-shaped mixed-precision AdamW step, ZeRO-1 sharded over
N GPUs - per step a bf16 grad reduce-scatter, the fused local update of this rank's shard and a bf16 param
all-gather (the collectives vanish at N = 1).  One JSON line is printed by rank 0.

  value     whole-job params updated per second, inputs resident in HBM, CUDA events on the launch stream,
            max over ranks, K steps after W warm-up steps.
  roofline  the fused update kernel: 28 algorithmic bytes per element over its own launch duration (CUDA
            events recorded by the library around the launch), against the measured copy bandwidth.
  e2e       the same step through the public API with HOST buffers, copies inside the timed region: at
            N = 1 the host-streamed step (gradients in from pinned host memory, update, bf16 params back
            out, pipelined slice by slice so both PCIe directions run at once); at N > 1 the gradients
            copied in, the sharded step, and the updated params of this rank's shard copied back.
  cpu_baseline (N = 1, rank 0)  the CPU oracle in the reference's own 12-pass shape on a bounded sample.

`--impl reference` times that CPU port on the host cores alone (rank 0 only).
Other workloads (`llama1b_mixed`, `gpt2_adam`, `frag_adamw`, `frag_sgdm`, `mlp_sgd`) are the remaining
configurations; they run on one GPU and are used for profiling and for the per-config table.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
# stdout must carry the one JSON line only, but libraries write there too (NCCL prints its version banner and,
# at higher NCCL_DEBUG levels, its communicator log).  Nothing is muted or re-levelled: file descriptor 1 is
# pointed at stderr for the whole run, so whatever a library prints still reaches the run's log, and the JSON
# line is written to the saved original stdout at the end.
sys.stdout.flush()
_REAL_STDOUT = os.fdopen(os.dup(1), "w")
os.dup2(2, 1)


def emit(line: dict) -> None:
    _REAL_STDOUT.write(json.dumps(line) + "\n")
    _REAL_STDOUT.flush()


# dram__bytes_read.sum + dram__bytes_write.sum per element, from the ncu captures summarised under profiles/
# (small cases of the same kernels: 5.535 GB / 199,757,824 elements and 3.430 GB / 124,439,808 elements).
# DRAM traffic of these streaming kernels grows in proportion to the element count, so a launch's traffic is
# this figure times the elements it covers.
NCU_TRAFFIC_BYTES_PER_ELEM = {"adam_mixed_kernel": 27.71, "adam_f32_kernel": 27.56}
NOMINAL_HBM_GBS = 8000.0
# the arithmetic type of the path; the mixed step reads bf16 gradients and writes bf16 parameters around it
DTYPE_OF_KIND = {"zero1": "f32 (bf16 params/grads, f32 master/m/v)", "mixed": "f32 (bf16 params/grads, f32 master/m/v)",
                 "f32": "f32"}
FALLBACK_HBM_GBS = 6650.0


# ----------------------------------------------------------------------------- workloads

def llama_shapes(d, layers, ffn, vocab, kv_dim):
    s = [(vocab, d)]
    for _ in range(layers):
        s += [(d, d), (d, kv_dim), (d, kv_dim), (d, d), (d, ffn), (d, ffn), (ffn, d), (d,), (d,)]
    s += [(d,), (vocab, d)]
    return s


def gpt2_shapes():
    s = [(50257, 768), (1024, 768)]
    for _ in range(12):
        s += [(768,), (768,), (768,), (768,), (768, 2304), (2304,), (768, 768), (768,), (768, 3072), (3072,),
              (3072, 768), (768,)]
    s += [(768,), (768,)]
    return s


def frag_sizes(seed=0, n=10000):
    import numpy as np
    rng = np.random.default_rng(seed)
    return [(int(x),) for x in np.floor(np.exp(rng.uniform(0.0, math.log(2 ** 20), n))).astype(np.int64)]


WORKLOADS = {
    "llama8b_zero1": dict(kind="zero1", shapes=lambda: llama_shapes(4096, 32, 14336, 128256, 1024),
                          lr=3e-4, wd=0.1, bytes_per_elem=28,
                          desc="Llama-3-8B-shaped mixed-precision AdamW, ZeRO-1 (bf16 p/g, f32 master/m/v)"),
    "llama1b_mixed": dict(kind="mixed", shapes=lambda: llama_shapes(2048, 16, 8192, 32000, 2048),
                          lr=3e-4, wd=0.1, bytes_per_elem=30, use_scaler=True, max_norm=1.0,
                          desc="Llama-1B-shaped mixed AdamW with dynamic loss scale and clip 1.0"),
    "llama1b_scaler": dict(kind="mixed", shapes=lambda: llama_shapes(2048, 16, 8192, 32000, 2048),
                           lr=3e-4, wd=0.1, bytes_per_elem=30, use_scaler=True, max_norm=0.0,
                           desc="Llama-1B-shaped mixed AdamW with dynamic loss scale, no clipping (flag-only pre-pass)"),
    "mixed_small": dict(kind="mixed", shapes=lambda: llama_shapes(2048, 2, 8192, 16000, 2048),
                        lr=3e-4, wd=0.1, bytes_per_elem=30, use_scaler=True, max_norm=1.0,
                        desc="2-layer slice of the Llama-1B shapes (0.2 G params, 3.2 GB): the small case for ncu"),
    "mixed_small_scaler": dict(kind="mixed", shapes=lambda: llama_shapes(2048, 2, 8192, 16000, 2048),
                               lr=3e-4, wd=0.1, bytes_per_elem=30, use_scaler=True, max_norm=0.0,
                               desc="mixed_small with loss scaling only (flag-only pre-pass): small case for ncu"),
    "gpt2_adam": dict(kind="f32", opt="adam", shapes=gpt2_shapes, lr=1e-3, bytes_per_elem=28,
                      desc="GPT-2-small-shaped fp32 Adam"),
    "frag_adamw": dict(kind="f32", opt="adamw", shapes=frag_sizes, lr=1e-3, wd=0.01, bytes_per_elem=28,
                       desc="10,000 fp32 tensors log-uniform in [1, 2^20], AdamW"),
    "frag_sgdm": dict(kind="f32", opt="sgdm", shapes=frag_sizes, lr=0.1, bytes_per_elem=20,
                      desc="10,000 fp32 tensors log-uniform in [1, 2^20], SGD momentum 0.9"),
    "one_adamw": dict(kind="f32", opt="adamw", shapes=lambda: [(sum(n for (n,) in frag_sizes()),)], lr=1e-3, wd=0.01,
                      bytes_per_elem=28, desc="the frag list's elements as ONE fp32 tensor, AdamW (roofline reference)"),
    "one_sgdm": dict(kind="f32", opt="sgdm", shapes=lambda: [(sum(n for (n,) in frag_sizes()),)], lr=0.1,
                     bytes_per_elem=20, desc="the frag list's elements as ONE fp32 tensor, SGD momentum 0.9"),
    "mlp_sgd": dict(kind="f32", opt="sgd", shapes=lambda: [(256, 784), (256,), (128, 256), (128,), (10, 128), (10,)],
                    lr=0.01, bytes_per_elem=12, desc="MLP 784-256-128-10 fp32 SGD"),
}


def numel(shape):
    n = 1
    for d in shape:
        n *= d
    return n


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------------------- clocks

class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark(self):
        """The timed region starts now: only samples written from here on are reported.  (The sampler itself
        is started earlier, before the warm-up steps, because nvidia-smi takes up to a second to deliver its
        first sample - longer than a short timed region on an 8-GPU box.)"""
        try:
            self.offset = os.path.getsize(self.path)
        except (OSError, TypeError):
            self.offset = 0

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as fh:
                fh.seek(getattr(self, "offset", 0))
                lines = fh.read().splitlines()
            for line in lines:
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


# ----------------------------------------------------------------------------- CPU arm (oracle port)

def omp_use_all_cores():
    """Gives the oracle's OpenMP runtime every core this process may run on and returns the thread count
    the runtime then reports (what is actually used, not what the affinity mask promises).  Launchers such
    as torch.distributed.run export OMP_NUM_THREADS=1 to their workers, which would otherwise make the CPU
    arm single-threaded."""
    import ctypes
    want = len(os.sched_getaffinity(0))
    try:
        gomp = ctypes.CDLL("libgomp.so.1")
        gomp.omp_set_num_threads(ctypes.c_int(want))
        gomp.omp_get_max_threads.restype = ctypes.c_int
        return int(gomp.omp_get_max_threads())
    except OSError:
        return int(os.environ.get("OMP_NUM_THREADS", "1"))


def cpu_reference_step_time(sample_elems, steps, warmup, mixed=True, passes=True):
    """Times the reference-shaped CPU port (12-pass AdamW incl. the serial `map`, plus - for the mixed step -
    the serial cast / scaler / clip walks) on `sample_elems` elements.  `passes=False` times the port's
    single fused pass over the same data instead (context only: nabla's CPU backend does not run that).
    Returns (seconds per step, cores)."""
    import numpy as np
    from oracle import binding as orc
    orc.build()
    orc.lib()
    rng = np.random.default_rng(0)
    n = int(sample_elems)
    w = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02))
    g = (rng.standard_normal(n, dtype=np.float32) * np.float32(1e-4))
    cores = omp_use_all_cores()
    if mixed:
        mo = orc.MixedOracle([w], [orc.AdamCfg(3e-4, 0.9, 0.999, 1e-8, 0.1, 1)], use_scaler=False)
        g16 = orc.bf16_from_f32(g)
        fn = lambda: mo.step([g16], max_norm=0.0, passes=passes)
    else:
        m = np.zeros(n, np.float32); v = np.zeros(n, np.float32)
        st = [0]

        def fn():
            st[0] += 1
            orc.adam_step(w, g, m, v, 1e-3, step=st[0], decoupled=False, passes=passes)
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    return (time.perf_counter() - t0) / max(steps, 1), cores


def calibrated_cpu_sample(target_seconds, mixed=True, cap=1 << 29):
    probe = 1 << 23
    t, _ = cpu_reference_step_time(probe, 1, 1, mixed)
    n = int(probe * target_seconds / max(t, 1e-6))
    return max(probe, min(n, cap))


def run_reference_arm(args, wl_name, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))   # before any OpenMP runtime starts
    mixed = wl["kind"] in ("zero1", "mixed")
    total = sum(numel(s) for s in wl["shapes"]())
    budget = 150.0 / max(args.steps + args.warmup, 1)          # whole run within a few minutes
    sample = calibrated_cpu_sample(min(budget, 6.0), mixed)
    sample = min(sample, total)
    sec, cores = cpu_reference_step_time(sample, args.steps, args.warmup, mixed)
    value = sample / sec
    line = {
        "impl": "reference", "metric": "params_updated_per_s", "value": value, "unit": "params/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE_OF_KIND[wl["kind"]],
        "data": "synthetic",
        "config": {"workload": wl_name, "description": wl["desc"], "params": total,
                   "tensors": len(wl["shapes"]()),
                   "parallelism": f"zero1-dp{args.gpus}" if wl["kind"] == "zero1" else "single-gpu",
                   "note": "CPU port of nabla's CPU-backend optimizer path (the Rust reference cannot be built: "
                           "no Rust toolchain); each step runs on a bounded sample of the workload"},
        "cpu_baseline": {"value": value, "unit": "params/s", "cores": cores, "omp_threads": cores, "kind": "port",
                         "sample": f"{sample} elements per step, reference-shaped 12-pass AdamW incl. serial map"},
        "e2e": {"value": value, "unit": "params/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ----------------------------------------------------------------------------- GPU arm

def fill_randn_bf16(t, std, gen, chunk=1 << 28):
    import torch
    n = t.numel()
    for off in range(0, n, chunk):
        m = min(chunk, n - off)
        t[off:off + m].copy_(torch.randn(m, device=t.device, generator=gen, dtype=torch.float32).mul_(std))


def bf16_ordered(t):
    """bf16 bit patterns as integers that increase with the value (one step = one ulp)."""
    import torch
    i = t.view(torch.int16).to(torch.int32) & 0xffff
    return torch.where(i >= 0x8000, 0x8000 - i, i)


def zero1_self_check(opt, step, pflat, gflat, total, rank, world, dev, transport):
    """Outside the timed region: one more sharded step whose cross-rank reduction is compared with an
    independent fp32 rank-order sum (mean of the replicas, nabla-train/src/dist.rs:36-43) on a slice of
    every rank's shard (64 Mi elements in all), and whose parameters must be identical on all ranks."""
    import torch
    import torch.distributed as dist
    b, e, _ = opt.shard_range()
    shard = e - b
    m = min(shard, (64 << 20) // world) // 8 * 8
    send = torch.cat([gflat[r * shard:r * shard + m] for r in range(world)])      # my inputs at every rank's slice
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send)                                             # every rank's inputs at my slice
    acc = torch.zeros(m, dtype=torch.float32, device=dev)
    mag = torch.zeros_like(acc)
    for r in range(world):
        x = recv[r * m:(r + 1) * m].float()
        acc += x
        mag += x.abs()
    acc *= torch.tensor(1.0, dtype=torch.float32, device=dev) / torch.tensor(float(world), dtype=torch.float32, device=dev)
    want = acc.to(torch.bfloat16)
    del send, recv, acc
    step()                                                                         # average=True, reduced grads kept
    got = gflat[b:b + m]
    ulps = (bf16_ordered(got) - bf16_ordered(want)).abs()
    err = (got.float() - want.float()).abs()
    if transport == "peer":
        ok = ulps == 0
        bound = "bit-exact (fp32 sum in rank order, one rounding)"
    elif transport == "mcast":
        ok = (ulps <= 1) | (err <= mag * 2.0 ** -20)
        bound = "<= 1 bf16 ulp (the switch rounds the sum to bf16, the averaging rounds again)"
    else:
        ok = err <= mag * (world * 2.0 ** -8) / world + 1e-30
        bound = "within the bf16 roundings between the hops of NCCL's reduction"
    digest = torch.zeros(1, dtype=torch.int64, device=dev)
    bits = pflat.view(torch.int16)
    for off in range(0, bits.numel(), 1 << 28):                # position-weighted, in pieces: no 8 G-element temporary
        piece = bits[off:off + (1 << 28)].to(torch.int64)
        digest += (piece * (1 + (off >> 28))).sum()
        del piece
    digests = [torch.zeros_like(digest) for _ in range(world)]
    dist.all_gather(digests, digest)
    same_params = all(int(d) == int(digest) for d in digests)
    stats = torch.tensor([float(ok.all()), float(ulps.max()), float((ulps > 0).float().mean()), float(same_params)],
                         dtype=torch.float64, device=dev)
    worst = stats.clone()
    dist.all_reduce(stats, op=dist.ReduceOp.MIN)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    rel = torch.tensor([float((err / mag.clamp_min(1e-30)).max())], dtype=torch.float64, device=dev)
    dist.all_reduce(rel, op=dist.ReduceOp.MAX)
    return {"ok": bool(stats[0] > 0 and stats[3] > 0), "reduction_within_bound": bool(stats[0] > 0),
            "reduced_grad_max_err_over_sum_of_magnitudes": float(rel),
            "params_identical_on_all_ranks": bool(stats[3] > 0), "reduced_grad_max_ulp": int(worst[1]),
            "reduced_grad_frac_differing": float(worst[2]), "elements_per_rank": m, "bound": bound,
            "reference": "every rank's input gradients for the slice, summed in fp32 in rank order with torch, "
                         "times f32(1/world), rounded once to bf16"}


def pcie_rates(torch, dev, world, host_buf, dev_buf, barrier, max_over_ranks):
    """Host<->device copy rates with every rank copying at the same time (GB/s per GPU, the slowest rank):
    the floor under the end-to-end step, which has to bring every rank's whole gradient bucket in.
    Returns (h2d alone, d2h alone, h2d while d2h runs, d2h while h2d runs)."""
    n = min(host_buf.numel(), dev_buf.numel(), 1 << 29)
    other = torch.empty(n, dtype=host_buf.dtype).pin_memory()
    side = torch.cuda.Stream()
    nbytes = n * host_buf.element_size()

    def timed(fn_main, fn_side=None, reps=3):
        best = [0.0, 0.0]
        for _ in range(reps):
            barrier()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            e[0].record()
            fn_main()
            e[1].record()
            if fn_side is not None:
                with torch.cuda.stream(side):
                    e[2].record()
                    fn_side()
                    e[3].record()
            torch.cuda.synchronize()
            best[0] = max(best[0], nbytes / (e[0].elapsed_time(e[1]) * 1e-3) / 1e9)
            if fn_side is not None:
                best[1] = max(best[1], nbytes / (e[2].elapsed_time(e[3]) * 1e-3) / 1e9)
        return [-max_over_ranks(-b) for b in best]                 # the slowest rank's best

    h2d = lambda: dev_buf[:n].copy_(host_buf[:n], non_blocking=True)
    d2h = lambda: other.copy_(dev_buf[n:2 * n] if dev_buf.numel() >= 2 * n else dev_buf[:n], non_blocking=True)
    a = timed(h2d)[0]
    b = timed(d2h)[0]
    c = timed(h2d, d2h)
    return a, b, c[0], c[1]


def peer_copy_peak(nb, opt, rank, world, dev, nbytes=1 << 30, reps=5, write=False):
    """GB/s per GPU and direction of a plain SM copy between this rank and the next rank's gradient bucket,
    all ranks at once (ring pattern: every GPU reads from / writes to one peer and is read / written by one).
    write=False: 128-bit loads from the peer, stores to local memory; write=True: the reverse."""
    import ctypes as C

    import torch
    import torch.distributed as dist
    nbytes = min(nbytes, opt.padded * 2) // 16 * 16
    src = opt.peer_grad_ptrs[(rank + 1) % world]
    dst = torch.empty(nbytes // 2, dtype=torch.bfloat16, device=dev)
    if write:
        src, dst_ptr = dst.data_ptr(), src
    else:
        dst_ptr = dst.data_ptr()
    lib = nb._lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    best = 0.0
    for it in range(reps + 1):
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        nb._lib.check(None, lib.nbo_copy_probe(dev.index, C.c_void_p(stream), C.c_void_p(dst_ptr), C.c_void_p(src),
                                              nbytes))
        e1.record()
        torch.cuda.synchronize()
        if it:
            best = max(best, nbytes / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    t = torch.tensor([best], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return float(t.item())


def quick_config(nb, torch, dev, name, steps=10, warmup=3):
    """One short entry of the per-configuration table: the workload `name` on one GPU, device-timed."""
    wl = WORKLOADS[name]
    shapes = wl["shapes"]()
    sizes = [numel(s) for s in shapes]
    total = sum(sizes)
    mixed = wl["kind"] == "mixed"
    dt = torch.bfloat16 if mixed else torch.float32
    es = 2 if mixed else 4
    al = 16 // es
    gen = torch.Generator(device=dev).manual_seed(99)
    flat_p = torch.empty(sum((n + al - 1) // al * al for n in sizes) + al, dtype=dt, device=dev)
    flat_g = torch.empty_like(flat_p)
    if mixed:
        fill_randn_bf16(flat_p, 0.02, gen); fill_randn_bf16(flat_g, 1e-4 * 65536.0, gen)
    else:
        flat_p.normal_(0, 0.02, generator=gen); flat_g.normal_(0, 1e-4, generator=gen)
    ps, gs, off = [], [], 0
    for n in sizes:
        ps.append(flat_p[off:off + n]); gs.append(flat_g[off:off + n])
        off += (n + al - 1) // al * al
    pa, ga = nb._lib.ptr_array([t.data_ptr() for t in ps]), nb._lib.ptr_array([t.data_ptr() for t in gs])
    if mixed:
        opt = nb.MixedAdamW.adamw(wl["lr"], wl["wd"], shapes)
        opt.init_master_from_params(ps)
        step = lambda: opt.step_ptrs(pa, ga, use_scaler=wl["use_scaler"], max_norm=wl["max_norm"])
    else:
        o = wl["opt"]
        opt = (nb.Adam(wl["lr"], shapes) if o == "adam" else nb.AdamW(wl["lr"], shapes).weight_decay(wl["wd"]) if o == "adamw"
               else nb.Sgd(wl["lr"], shapes).momentum(0.9) if o == "sgdm" else nb.Sgd(wl["lr"], shapes))
        step = lambda: opt.step_ptrs(pa, ga)
    h = opt._h
    h.profile(True)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    l0 = h.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    norm_ms = upd_ms = 0.0
    e0.record()
    for _ in range(steps):
        step()
        if mixed:
            a, u = h.profile_last()
            norm_ms += a; upd_ms += u
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    peak, _ = measured_peak()
    out = {"params": total, "tensors": len(sizes), "ms_per_step": ms, "launches_per_step": (h.launch_count() - l0) / steps}
    if name == "mlp_sgd":
        out["us_per_step"] = ms * 1e3
    elif mixed:
        upd_ms /= steps; norm_ms /= steps
        out.update(update_ms=upd_ms, norm_ms=norm_ms, update_gbs=28 * total / upd_ms / 1e6,
                   update_frac=28 * total / upd_ms / 1e6 / peak, norm_gbs=2 * total / norm_ms / 1e6 if norm_ms else None,
                   norm_frac=2 * total / norm_ms / 1e6 / peak if norm_ms else None,
                   step_gbs=30 * total / (upd_ms + norm_ms) / 1e6, step_frac=30 * total / (upd_ms + norm_ms) / 1e6 / peak)
    else:
        gbs = wl["bytes_per_elem"] * total / ms / 1e6
        out.update(gbs=gbs, frac=gbs / peak, frac_of_nominal_8TBs=gbs / NOMINAL_HBM_GBS)
    del opt, flat_p, flat_g, ps, gs
    torch.cuda.empty_cache()
    return out


def run_ours(args, wl_name, wl):
    import torch
    import torch.distributed as dist

    import nabla_b200 as nb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    shapes = wl["shapes"]()
    sizes = [numel(s) for s in shapes]
    total = sum(sizes)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    peak, peak_kind = measured_peak()
    h2d = d2h = 0
    extra = {}

    if wl["kind"] == "zero1":
        uid = nb.exchange_unique_id(rank, world)
        opt = nb.Zero1AdamW.adamw(wl["lr"], wl["wd"], shapes, rank, world, uid)
        padded, shard = opt.padded, opt.shard
        fused = world > 1 and args.zero1_path != "nccl"
        if fused:
            # buckets in symmetric memory; the collectives are fused into the update kernels.  If the fabric
            # or the runtime cannot provide symmetric memory on some rank, every rank falls back to the
            # NCCL-around-the-update path together and the line says so.
            tr = {"auto": 0, "peer": 1, "mcast": 2}[args.zero1_path]
            # the buckets come from the library's own allocator (nbo_symm_alloc); torch's symmetric-memory module is
            # the second choice
            for how in (["native", "torch"] if args.symm == "auto" else [args.symm]):
                ok = 1
                try:
                    pflat, gflat = (opt.attach_symmetric_native(transport=tr) if how == "native"
                                    else opt.attach_symmetric(transport=tr))
                except Exception as exc:                   # noqa: BLE001 - any failure means "not available"
                    ok = 0
                    extra[f"symm_{how}_unavailable"] = f"{type(exc).__name__}: {exc}"[:200]
                agree = torch.tensor([ok], device=dev)
                dist.all_reduce(agree, op=dist.ReduceOp.MIN)
                if int(agree.item()) == 1:
                    extra["symmetric_memory"] = ("nbo_symm_alloc (CUDA virtual memory + multicast, this library)"
                                                 if how == "native" else "torch.distributed._symmetric_memory")
                    break
                if ok and how == "native":
                    opt.release_symmetric()                # another rank failed: give the buckets back, all together
                    raise SystemExit("symmetric allocation succeeded on some ranks only")
            if int(agree.item()) == 0:
                fused = False
                del opt
                torch.cuda.empty_cache()
                uid = nb.exchange_unique_id(rank, world)
                opt = nb.Zero1AdamW.adamw(wl["lr"], wl["wd"], shapes, rank, world, uid)
        if not fused:
            pflat = torch.zeros(padded, dtype=torch.bfloat16, device=dev)
            gflat = torch.zeros(padded, dtype=torch.bfloat16, device=dev)
        fill_randn_bf16(pflat[:total], 0.02, torch.Generator(device=dev).manual_seed(7))
        fill_randn_bf16(gflat[:total], 1e-4, gen)
        opt.init_master(pflat)
        pp, gp = pflat.data_ptr(), gflat.data_ptr()
        if fused:
            # the reduced gradient is consumed in registers; it is not also written back into the gradient
            # bucket during the timed steps (the self-check below runs with the write-back on)
            opt.keep_reduced_grads(False)
            step = lambda: opt.step_fused(average=True, use_scaler=False, max_norm=0.0)
        else:
            step = lambda: opt.step_ptrs(pp, gp, average=True, use_scaler=False, max_norm=0.0)
        extra["zero1_path"] = ("fused-" + args.zero1_path) if fused else ("nccl" if world > 1 else "local")
        if fused:
            extra["zero1_transport"] = "mcast" if (tr == 2 or (tr == 0 and world >= 5 and opt.has_multicast)) else "peer"
        handle = opt._h
        b, e, _ = opt.shard_range()
        local_elems = max(0, min(e, total) - b)
        ring_elems = min(1 << 29, padded)                      # 1 GiB of bf16 in pinned host memory
        ring_in = torch.empty(ring_elems, dtype=torch.bfloat16).pin_memory()
        ring_in.copy_(gflat[:ring_elems])
        ring_out = torch.empty(min(ring_elems, shard), dtype=torch.bfloat16).pin_memory()

        if world == 1 or fused:
            # host tensors (one per parameter tensor, as the reference's CPU tensors are) aliased onto the
            # two pinned rings; the step streams them through the device buckets slice by slice
            ring_out = torch.empty(ring_elems, dtype=torch.bfloat16).pin_memory()
            hp_ptrs, hg_ptrs, off = [], [], 0
            for n in sizes:
                if off + n > ring_elems:
                    off = 0
                hg_ptrs.append(ring_in.data_ptr() + 2 * off)
                hp_ptrs.append(ring_out.data_ptr() + 2 * off)
                off += n
            hpa, hga = nb._lib.ptr_array(hp_ptrs), nb._lib.ptr_array(hg_ptrs)

            def e2e_step():
                opt.step_host_ptrs(pp, gp, hpa, hga, average=True, use_scaler=False, max_norm=0.0)
            e2e_path = ("nbo_zero1_step_host: copy-in / update / copy-out pipelined over 3 streams, 32 Mi-element slices"
                        if world == 1 else
                        "nbo_zero1_step_host: per slice of every rank's shard, copy-in of this rank's gradients, "
                        "stream-ordered barrier, fused reduce/update/publish kernel, copy-out of this rank's "
                        f"parameters; {(32 << 20) // world} elements per rank and slice")
            e2e_path += ("; every host tensor aliases one of two 1 GiB pinned rings, so the bytes cross PCIe but "
                         "the host side re-reads / overwrites the same 1 GiB")
        else:
            def e2e_step():
                for off in range(0, padded, ring_elems):
                    m = min(ring_elems, padded - off)
                    gflat[off:off + m].copy_(ring_in[:m], non_blocking=True)
                step()
                ro = ring_out.numel()
                for off in range(b, e, ro):
                    m = min(ro, e - off)
                    ring_out[:m].copy_(pflat[off:off + m], non_blocking=True)
                torch.cuda.synchronize()
            e2e_path = "copy-in, sharded step, copy-out of the shard, in stream order"
        h2d, d2h = 2 * padded * world, 2 * shard * world
        parallelism = f"zero1-dp{world}"
        staging = "two 1 GiB pinned rings (gradients in, params out); the host tensors / chunks alias them"
    else:
        mixed = wl["kind"] == "mixed"
        dt = torch.bfloat16 if mixed else torch.float32
        es = 2 if mixed else 4
        # tensors are carved from one allocation, each starting 16-byte aligned like separate allocations
        ps, gs, off = [], [], 0
        al = 16 // es
        flat_p = torch.empty(sum((n + al - 1) // al * al for n in sizes) + al, dtype=dt, device=dev)
        flat_g = torch.empty_like(flat_p)
        if mixed:
            fill_randn_bf16(flat_p, 0.02, gen); fill_randn_bf16(flat_g, 1e-4 * 65536.0, gen)
        else:
            flat_p.normal_(0, 0.02, generator=gen); flat_g.normal_(0, 1e-4, generator=gen)
        for n in sizes:
            ps.append(flat_p[off:off + n]); gs.append(flat_g[off:off + n])
            off += (n + al - 1) // al * al
        if mixed:
            opt = nb.MixedAdamW.adamw(wl["lr"], wl["wd"], shapes)
            opt.init_master_from_params(ps)
            if args.loss_scale:
                st = opt.scaler_state(); st.scale = float(args.loss_scale); opt.load_scaler_state(st)
            pa, ga = nb._lib.ptr_array([t.data_ptr() for t in ps]), nb._lib.ptr_array([t.data_ptr() for t in gs])
            step = lambda: opt.step_ptrs(pa, ga, use_scaler=wl["use_scaler"], max_norm=wl["max_norm"])
        else:
            o = wl["opt"]
            if o == "adam":
                opt = nb.Adam(wl["lr"], shapes)
            elif o == "adamw":
                opt = nb.AdamW(wl["lr"], shapes).weight_decay(wl["wd"])
            elif o == "sgdm":
                opt = nb.Sgd(wl["lr"], shapes).momentum(0.9)
            else:
                opt = nb.Sgd(wl["lr"], shapes)
            pa, ga = nb._lib.ptr_array([t.data_ptr() for t in ps]), nb._lib.ptr_array([t.data_ptr() for t in gs])
            step = lambda: opt.step_ptrs(pa, ga)
        handle = opt._h
        local_elems = total
        host_g = torch.empty(flat_g.numel(), dtype=dt).pin_memory()
        host_g.copy_(flat_g)
        host_p = torch.empty(flat_p.numel(), dtype=dt).pin_memory()

        if mixed:
            hp_ptrs, hg_ptrs = [], []
            for t_p, t_g in zip(ps, gs):
                hp_ptrs.append(host_p.data_ptr() + (t_p.data_ptr() - flat_p.data_ptr()))
                hg_ptrs.append(host_g.data_ptr() + (t_g.data_ptr() - flat_g.data_ptr()))
            hpa, hga = nb._lib.ptr_array(hp_ptrs), nb._lib.ptr_array(hg_ptrs)

            def e2e_step():
                opt.step_host_ptrs(pa, ga, hpa, hga, use_scaler=wl["use_scaler"], max_norm=wl["max_norm"])
            e2e_path = "nbo_step_mixed_host: copy-in / update / copy-out pipelined over 3 streams, 32 Mi-element slices"
        else:
            def e2e_step():
                flat_g.copy_(host_g, non_blocking=True)
                step()
                host_p.copy_(flat_p, non_blocking=True)
                torch.cuda.synchronize()
            e2e_path = "copy-in, step, copy-out, in stream order"
        h2d = d2h = flat_g.numel() * es
        parallelism = "single-gpu"
        staging = "whole gradient / param buffers in pinned host memory"

    handle.profile(True)
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    launches0 = handle.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    upd_ms = norm_ms = 0.0
    barrier()
    sampler.mark()
    ev0.record()
    t0 = time.perf_counter()
    sync_steps = wl["kind"] != "f32"      # mixed / sharded steps end with a stream sync of their own
    for _ in range(args.steps):
        step()
        if sync_steps:                    # reading the library's events costs no extra sync there
            a, u = handle.profile_last()
            norm_ms += a; upd_ms += u
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    dev_s = max_over_ranks(ev0.elapsed_time(ev1) / 1e3)
    launches = handle.launch_count() - launches0
    if not sync_steps:                    # fp32 steps are asynchronous launches back to back on one stream:
        upd_ms = dev_s * 1e3              # the region is the sum of the kernel durations
    upd_ms = max_over_ranks(upd_ms / args.steps)
    norm_ms = max_over_ranks(norm_ms / args.steps)
    value = total * args.steps / dev_s

    # context for the roofline fraction: the same copy the peak was measured with (torch copy_, 2 x 2 GiB),
    # but run back to back for as long as the timed region lasted, i.e. under the same power cap
    copy_sustained = None
    if world == 1 and not args.no_copy_probe:
        try:
            src = torch.empty(1 << 30, dtype=torch.bfloat16, device=dev).normal_()
            dst = torch.empty_like(src)
            reps = max(8, int(max(dev_s, 0.2) / 0.00066))
            for _ in range(3):
                dst.copy_(src)
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(reps // 2):
                dst.copy_(src)
            c0.record()
            for _ in range(reps - reps // 2):
                dst.copy_(src)
            c1.record()
            torch.cuda.synchronize()
            copy_sustained = (reps - reps // 2) * 2 * src.numel() * 2 / (c0.elapsed_time(c1) * 1e-3) / 1e9
            del src, dst
        except RuntimeError:
            copy_sustained = None

    # SGD has step-independent launch arguments, so a run of steps can be captured once and replayed
    # (Adam/AdamW bias corrections change every step; their graph-capturable form is the asynchronous mixed step)
    if wl["kind"] == "f32" and wl.get("opt") in ("sgd", "sgdm"):
        cap_stream = torch.cuda.Stream()
        with torch.cuda.stream(cap_stream):
            opt_g = nb.Sgd(wl["lr"], shapes).momentum(0.9 if wl["opt"] == "sgdm" else 0.0)
            opt_g.step_ptrs(pa, ga)                      # uploads the table outside the capture
        cap_stream.synchronize()
        per_graph = 20
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=cap_stream):
            for _ in range(per_graph):
                opt_g.step_ptrs(pa, ga)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(1, args.steps // per_graph)
        g0.record()
        for _ in range(reps):
            graph.replay()
        g1.record()
        torch.cuda.synchronize()
        extra["cuda_graph_us_per_step"] = g0.elapsed_time(g1) * 1e3 / (reps * per_graph)

    # end to end with host buffers
    e2e_steps = max(1, min(args.steps, 10))
    if args.no_e2e:                                               # kernel experiments only: the line then has no e2e number
        e2e_steps, e2e_s = 0, float("inf")
    else:
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_s = max_over_ranks((time.perf_counter() - t0)) / e2e_steps

    # the 8 G-parameter step with dynamic loss scaling and clipping on (norm / non-finite pass + scaled update)
    scaled = None
    if wl["kind"] == "zero1" and world == 1 and not args.no_configs:
        for off in range(0, total, 1 << 28):                      # the same gradients times the loss scale 2^16
            gflat[off:min(off + (1 << 28), total)].mul_(65536.0)
        sstep = lambda: opt.step_ptrs(pp, gp, average=True, use_scaler=True, max_norm=1.0)
        for _ in range(3):
            sstep()
        sn = su = 0.0
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(5):
            r = sstep()
            a, u = handle.profile_last()
            sn += a; su += u
        s1.record()
        torch.cuda.synchronize()
        sn /= 5; su /= 5
        scaled = {"params": total, "use_scaler": True, "max_norm": 1.0, "applied": bool(r.applied),
                  "ms_per_step": s0.elapsed_time(s1) / 5, "update_ms": su, "norm_ms": sn,
                  "update_gbs": 28 * total / su / 1e6, "norm_gbs": 2 * total / sn / 1e6,
                  "step_gbs_30B_per_elem": 30 * total / (su + sn) / 1e6,
                  "step_frac": 30 * total / (su + sn) / 1e6 / peak,
                  "step_frac_of_nominal_8TBs": 30 * total / (su + sn) / 1e6 / NOMINAL_HBM_GBS}

    pcie = None
    if wl["kind"] == "zero1" and not args.no_e2e:
        pcie = pcie_rates(torch, dev, world, ring_in, gflat, barrier, max_over_ranks)

    zero1_check = nvlink_peak = nvlink_peak_write = None
    if wl["kind"] == "zero1" and world > 1:
        if fused:
            opt.keep_reduced_grads(True)
        tr_name = extra.get("zero1_transport", "nccl")
        fill_randn_bf16(gflat[:total], 1e-4, gen)                 # fresh inputs (the NCCL path reduces in place)
        zero1_check = zero1_self_check(opt, step, pflat, gflat, total, rank, world, dev, tr_name)
        if fused:
            nvlink_peak = peer_copy_peak(nb, opt, rank, world, dev)
            nvlink_peak_write = peer_copy_peak(nb, opt, rank, world, dev, write=True)   # overwrites gradients: last use

    configs = None
    if wl["kind"] == "zero1" and world == 1 and rank == 0 and not args.no_configs:
        handle.close()                                            # frees the 96 GB of fp32 state
        del pflat, gflat, ring_in, ring_out
        torch.cuda.empty_cache()
        configs = {"scaled_8b": scaled}
        for name in ("mlp_sgd", "gpt2_adam", "llama1b_mixed", "frag_adamw", "frag_sgdm", "one_adamw", "one_sgdm"):
            try:
                configs[name] = quick_config(nb, torch, dev, name)
            except Exception as exc:                              # noqa: BLE001 - one entry failing must not lose the line
                configs[name] = {"error": f"{type(exc).__name__}: {exc}"[:200]}

    alg_bytes = 28 * local_elems if wl["kind"] != "f32" else wl["bytes_per_elem"] * local_elems
    achieved = alg_bytes / (upd_ms * 1e-3) / 1e9 if upd_ms > 0 else 0.0
    step_bytes = wl["bytes_per_elem"] * local_elems
    kname = "adam_mixed_kernel" if wl["kind"] != "f32" else (
        "adam_f32_kernel" if wl.get("opt") in ("adam", "adamw") else "sgd_f32_kernel")
    per_elem = NCU_TRAFFIC_BYTES_PER_ELEM.get(kname)
    traffic = per_elem * local_elems if per_elem else None
    line = {
        "metric": "params_updated_per_s", "value": value, "unit": "params/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_s * 1e3 / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE_OF_KIND[wl["kind"]],
        "data": "synthetic",
        "config": {"workload": wl_name, "description": wl["desc"], "params": total, "tensors": len(sizes),
                   "parallelism": parallelism, "storage": "bf16 params+grads, f32 master/m/v" if wl["kind"] != "f32" else "f32",
                   "l2": "inputs (>= 100x the 126 MB L2) are streamed once per step; no flush needed",
                   "host_staging": staging},
        "roofline": {"bound": "hbm", "kernel": kname,
                     "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": achieved / peak, "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                     "algorithmic_bytes_per_launch": alg_bytes, "kernel_ms": upd_ms, "traffic": traffic,
                     "copy_sustained_gbs": copy_sustained,
                     "traffic_note": "ncu dram bytes of a small case of this kernel, scaled by elements per launch"},
        "kernel_ms": {"update": upd_ms, "norm_nonfinite": norm_ms},
        "step_hbm_gbs_per_gpu": step_bytes / (dev_s / args.steps) / 1e9,
        "e2e": {"value": total / e2e_s, "unit": "params/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s * 1e3, "steps": e2e_steps, "path": e2e_path},
        "gpu_launches": launches,
        "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                   "samples": clocks["samples"]},
        "wall_ms_per_step": wall * 1e3 / args.steps,
    }
    line["config"].update(extra)
    if pcie is not None:
        # every rank must bring its whole gradient bucket in: h2d bytes per rank / the rate all ranks reach together
        floor_s = (h2d / world) / (pcie[0] * 1e9) if pcie[0] else None
        line["e2e"].update(h2d_gbs_all_ranks_at_once=pcie[0], d2h_gbs_all_ranks_at_once=pcie[1],
                           h2d_gbs_while_d2h=pcie[2], d2h_gbs_while_h2d=pcie[3],
                           h2d_gbs_achieved=(h2d / world) / e2e_s / 1e9,
                           floor_ms=floor_s * 1e3 if floor_s else None,
                           floor_note="per-rank gradient bytes over the host-to-device rate every rank reaches when all "
                                      "ranks copy in at once and nothing is copied out (1 GiB pinned buffers, "
                                      "cudaMemcpyAsync); with copy-out running the in-rate drops to h2d_gbs_while_d2h")
    if configs is not None:
        line["configs"] = configs
    if wl["kind"] == "zero1" and world > 1:
        # bytes that must cross NVLink per GPU and direction for one step, against the plain SM copy from a
        # peer's bucket measured in this run (nbo_copy_probe, all ranks at once)
        bucket = 2.0 * padded
        tr = extra.get("zero1_transport", "nccl")
        per_dir = bucket * (1.0 + 1.0 / world) if tr == "mcast" else 2.0 * bucket * (world - 1) / world
        step_s = dev_s / args.steps
        line["nvlink"] = {"transport": tr, "bytes_per_gpu_per_direction": per_dir, "peak_measured": nvlink_peak,
                          "peak_measured_stores": nvlink_peak_write,
                          "unit": "GB/s", "achieved": per_dir / step_s / 1e9,
                          "frac": per_dir / step_s / 1e9 / nvlink_peak if nvlink_peak else None,
                          "target_ms": per_dir / (nvlink_peak * 1e9) * 1e3 if nvlink_peak else None,
                          "peak_how": "1 GiB read from the next rank's bucket with 128-bit SM loads into local memory, "
                                      "every rank at once, best of 5 (GB/s per GPU and direction, min over ranks)",
                          "note": "the sharded step is NVLink-bound for N >= 2; roofline.frac is the local HBM share only"}
        line["zero1_check"] = zero1_check
        line["config"]["reduced_grads_written_back_in_timed_steps"] = not fused
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        mixed = wl["kind"] != "f32"
        sample = min(calibrated_cpu_sample(12.0, mixed), total)
        sec, cores = cpu_reference_step_time(sample, 1, 0, mixed)
        fused_sec, _ = cpu_reference_step_time(sample, 1, 0, mixed, passes=False)
        line["vs_cpu_port"] = {"value": value / (sample / sec), "e2e": (total / e2e_s) / (sample / sec),
                               "note": "this line's value and e2e.value over cpu_baseline.value (the CPU port, not a "
                                       "published number: vs_baseline stays null)"}
        line["cpu_baseline"] = {"value": sample / sec, "unit": "params/s", "cores": cores, "omp_threads": cores,
                                "kind": "port",
                                "sample": f"1 step on {sample} elements ({sec:.1f} s), reference-shaped 12-pass "
                                          "AdamW incl. the serial map / cast walks",
                                "fused_single_pass_value": sample / fused_sec,
                                "fused_note": "the same port as one fused pass (context; not what the reference runs)"}
    if rank == 0:
        emit(line)
    if world > 1:
        if wl["kind"] == "zero1" and getattr(opt, "_native", None):
            del pflat, gflat                               # views of memory the library is about to unmap
            opt.release_symmetric()                        # unbind from the multicast object before any rank exits
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="llama8b_zero1")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-copy-probe", action="store_true")
    ap.add_argument("--symm", choices=["auto", "native", "torch"], default="auto",
                    help="N > 1, fused path: who allocates the symmetric buckets (auto = the library, then torch)")
    ap.add_argument("--loss-scale", type=float, default=0.0,
                    help="initial loss scale of a single-GPU mixed workload (default: the scaler's own 65536); "
                         "from 2^17 on the norm pass runs its guarded form")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (kernel experiments)")
    ap.add_argument("--no-configs", action="store_true", help="skip the per-configuration table of the default line")
    ap.add_argument("--zero1-path", choices=["auto", "peer", "mcast", "nccl"], default="auto",
                    help="N > 1: collectives fused into the kernels (auto/peer/mcast) or issued through NCCL")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, args.workload, wl)
    else:
        run_ours(args, args.workload, wl)


if __name__ == "__main__":
    main()
