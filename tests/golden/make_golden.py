"""Writes tests/golden/oracle_vectors.npz: seeded input/output vectors of the CPU oracle.

The reference is Rust and cannot be built or imported where this runs, so these vectors do not come
from the reference itself; they freeze the oracle's restatement (oracle/nabla_oracle.c) so that a
later change of the oracle, the compiler or libm that alters a single bit is caught, and they give
the GPU tests a fixture that does not depend on the oracle being rebuilt.  Re-run from the repo root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import binding as o  # noqa: E402

N = 1031  # odd on purpose: exercises vector body + scalar tail


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    p0 = rng.normal(0, 0.02, N).astype(np.float32)
    grads = (rng.normal(0, 1e-4, (10, N))).astype(np.float32)
    out["p0"], out["grads"] = p0, grads

    for name, kw in (("adam", dict(decoupled=False)), ("adamw", dict(decoupled=True, weight_decay=0.01))):
        p, m, v = p0.copy(), np.zeros(N, np.float32), np.zeros(N, np.float32)
        for t in range(10):
            o.adam_step(p, grads[t], m, v, 1e-3, step=t + 1, **kw)
        out[f"{name}_p"], out[f"{name}_m"], out[f"{name}_v"] = p, m, v

    for name, kw in (("sgd", {}), ("sgd_mom", dict(momentum=0.9)), ("sgd_mom_wd", dict(momentum=0.9, weight_decay=0.01))):
        p, vel = p0.copy(), np.zeros(N, np.float32)
        for t in range(10):
            o.sgd_step(p, grads[t], vel, 0.1, **kw)
        out[f"{name}_p"], out[f"{name}_vel"] = p, vel

    # mixed precision: bf16 grads scaled by 2^16, an inf at step 3, clip at 1e-3
    w0 = rng.normal(0, 0.02, N).astype(np.float32)
    g16 = np.stack([o.bf16_from_f32((grads[t] * 65536.0).astype(np.float32)) for t in range(6)])
    g16[3, 77] = 0x7F80  # +inf
    cfg = o.AdamCfg(3e-4, 0.9, 0.999, 1e-8, 0.1, 1)
    mo = o.MixedOracle([w0], [cfg])
    oks, norms, scales = [], [], []
    for t in range(6):
        ok, norm = mo.step([g16[t]], max_norm=1e-3)
        oks.append(ok); norms.append(norm); scales.append(mo.scaler.scale)
    out["mixed_w0"], out["mixed_g16"] = w0, g16
    out["mixed_master"], out["mixed_m"], out["mixed_v"], out["mixed_p16"] = mo.master[0], mo.m[0], mo.v[0], mo.p[0]
    out["mixed_ok"] = np.array(oks); out["mixed_norm"] = np.array(norms); out["mixed_scale"] = np.array(scales)
    out["mixed_step_count"] = np.array([mo.step_count.value])

    # bf16 cast edge cases
    edge = np.array([0x00000000, 0x80000000, 0x00000001, 0x00008000, 0x00008001, 0x00018000, 0x3F808000,
                     0x3F818000, 0x3F80FFFF, 0x7F7FFFFF, 0x7F800000, 0xFF800000, 0x7FC00000, 0x7F800001,
                     0xFFFFFFFF, 0x7F7F8000, 0x00400000, 0x807FFFFF], dtype=np.uint32)
    out["bf16_edge_in"] = edge
    out["bf16_edge_out"] = o.bf16_from_f32(edge.view(np.float32))
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_vectors.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
