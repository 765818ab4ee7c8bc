"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

REL_TOL = 1e-5  # fp32 params / m / v versus the oracle, elementwise relative (the stated bar)


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def bits(a) -> np.ndarray:
    a = host(a) if isinstance(a, torch.Tensor) else a
    return np.ascontiguousarray(a).view(np.uint32 if a.dtype == np.float32 else np.uint16)


def bf16_dev(u16: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).cuda().view(torch.bfloat16)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


LAST_WORST = {}  # the most recent assert_close_rel call: {what, floored, unfloored} worst relative errors


def assert_close_rel(got, want, what="", rel=REL_TOL, floor=0.1, unfloored_from=1e-3):
    """Elementwise |got - want| <= rel * max(|want|, floor * rms(want)).

    The bar is 1e-5 relative.  A purely elementwise relative test is undefined for the handful of
    elements that happen to sit next to zero (a parameter crossing zero has |want| ~ 1e-7 while its
    rounding noise is a few ulp of the update, ~1e-9), so below a tenth of the tensor's RMS the error is
    measured against that floor instead of against |want|.  In addition the plain, un-floored
    |got - want| / |want| is asserted on every element with |want| >= unfloored_from * rms.  Returns the
    worst (floored) relative error seen; LAST_WORST keeps both figures."""
    got = host(got) if isinstance(got, torch.Tensor) else got
    g, w = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
    assert g.shape == w.shape, what
    if g.size == 0:
        return 0.0
    assert np.array_equal(np.isnan(g), np.isnan(w)), f"{what}: NaN pattern differs"
    ok = ~np.isnan(w)
    g, w = g[ok], w[ok]
    if g.size == 0:
        return 0.0
    err = np.abs(g - w)
    scale = np.maximum(np.abs(w), floor * np.sqrt(np.mean(w * w)))
    same = g == w
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.where(same, 0.0, err / scale)
    bad = r > rel
    assert not bad.any(), (f"{what}: {bad.sum()} of {g.size} elements off by more than {rel} relative; "
                           f"worst {r.max():.3e} (abs {err[r.argmax()]:.3e} at value {w[r.argmax()]:.6e})")
    # The bar as literally worded - |got - want| / |want| with no floor - on every element that is not
    # vanishingly small next to its tensor (|want| >= 1e-3 * rms): asserted too, and kept for reporting.
    rms = np.sqrt(np.mean(w * w))
    sel = np.abs(w) >= unfloored_from * rms
    worst_plain = 0.0
    if sel.any() and rms > 0.0:
        plain = np.where(same[sel], 0.0, err[sel] / np.abs(w[sel]))
        worst_plain = float(plain.max())
        assert worst_plain <= rel, (f"{what}: un-floored relative error {worst_plain:.3e} > {rel} on an element "
                                    f"with |want| >= {unfloored_from} * rms")
    LAST_WORST.update(what=what, floored=float(r.max()), unfloored=worst_plain)
    return float(r.max())


def exact_fraction(got, want) -> float:
    gb, wb = bits(got).ravel(), bits(want).ravel()
    return float((gb == wb).mean()) if gb.size else 1.0


def misaligned(n: int, dtype=torch.float32, offset_elems: int = 1) -> torch.Tensor:
    """A contiguous CUDA tensor whose base pointer is NOT 16-byte aligned."""
    base = torch.zeros(n + 64, dtype=dtype, device="cuda")
    view = base[offset_elems:offset_elems + n]
    assert view.data_ptr() % 16 != 0
    return view
