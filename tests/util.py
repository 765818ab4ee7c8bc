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


def assert_close_rel(got, want, what="", rel=REL_TOL):
    got = host(got) if isinstance(got, torch.Tensor) else got
    g, w = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
    assert g.shape == w.shape, what
    if g.size == 0:
        return 0.0
    err = np.abs(g - w)
    bound = rel * np.abs(w)
    bad = err > bound
    assert not bad.any(), (f"{what}: {bad.sum()} of {g.size} elements off by more than {rel} relative; "
                           f"worst {err.max():.3e} at value {w[err.argmax()]:.6e}")
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.where(w != 0, err / np.abs(w), 0.0)
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
