"""CPU: the on-disk checkpoint format (nabla-ml/src/module/core.rs:66-133, nabla-train/src/checkpoint.rs:107-150)."""
import struct

import numpy as np
import pytest

from nabla_b200 import LrSchedule
from nabla_b200 import checkpoint as ck


def test_nbla_container_is_byte_exact(tmp_path):
    a = np.array([[1.5, -2.0], [0.25, 3.0]], dtype=np.float32)
    b = np.array([7.0], dtype=np.float32)
    path = str(tmp_path / "optim.nbla")
    ck.save_tensors([("m0", a), ("v0", b)], path)
    want = b"NBLA" + struct.pack("<I", 2)
    want += struct.pack("<I", 2) + b"m0" + struct.pack("<II", 2, 2) + struct.pack("<4d", 1.5, -2.0, 0.25, 3.0)
    want += struct.pack("<I", 2) + b"v0" + struct.pack("<II", 1, 1) + struct.pack("<d", 7.0)
    assert open(path, "rb").read() == want
    back = ck.load_tensors(path)
    assert [n for n, _ in back] == ["m0", "v0"]
    assert np.array_equal(back[0][1], a.astype(np.float64)) and back[1][1].shape == (1, 1)
    open(path, "wb").write(b"NOPE" + want[4:])
    with pytest.raises(ValueError, match="not a nabla tensor file"):
        ck.load_tensors(path)


def test_state_tensor_bytes_of_a_2x3_moment(tmp_path):
    """The bytes the reference's save_tensors writes for one 2x3 tensor named m0, built by hand from
    nabla-ml/src/module/core.rs:66-85: magic, u32 count, u32 name length, name, u32 rows, u32 cols, then
    the elements row-major as little-endian f64."""
    from nabla_b200.optim import _as_state, _flat_state, _shape2d_of
    import torch
    flat = torch.tensor([0.5, -1.0, 2.0, 4.0, -8.0, 0.125])               # what the library exports
    m0 = _as_state(flat, _shape2d_of((2, 3)))
    assert tuple(m0.shape) == (2, 3)
    path = str(tmp_path / "optim.nbla")
    ck.save_tensors([("m0", m0.numpy())], path)
    want = (b"NBLA" + struct.pack("<I", 1) + struct.pack("<I", 2) + b"m0" + struct.pack("<II", 2, 3)
            + struct.pack("<6d", 0.5, -1.0, 2.0, 4.0, -8.0, 0.125))
    assert open(path, "rb").read() == want
    (name, back), = ck.load_tensors(path)
    assert name == "m0" and back.shape == (2, 3)
    # both layouts of the same elements are taken on load; another element count is refused
    assert torch.equal(_flat_state(torch.from_numpy(back).float(), 6, "m0"), flat)
    assert torch.equal(_flat_state(flat.reshape(1, 6), 6, "m0"), flat)
    with pytest.raises(ValueError, match="shapes must match"):
        _flat_state(flat[:5], 6, "m0")
    # the shapes a parameter list declares
    assert [_shape2d_of(s) for s in (7, (7,), (64, 33), (2, 3, 4), ())] == [(1, 7), (1, 7), (64, 33), (2, 12), (1, 1)]


def test_extents_beyond_u32_are_refused(tmp_path):
    class Huge:                                     # stands in for an array with 2^32 columns
        ndim, size = 2, 1 << 32
        shape = (1, 1 << 32)
    import numpy as _np
    orig = _np.asarray
    try:
        ck.np.asarray = lambda a, *k, **kw: a if isinstance(a, Huge) else orig(a, *k, **kw)
        with pytest.raises(ValueError, match="does not fit the u32"):
            ck.save_tensors([("m0", Huge())], str(tmp_path / "x.nbla"))
    finally:
        ck.np.asarray = orig


def test_numbers_print_like_rust_display():
    cases = {0.001: "0.001", 1e-8: "0.00000001", 65536.0: "65536", 0.9: "0.9", 0.999: "0.999", 3e-4: "0.0003",
             1.0: "1", 0.01: "0.01", 2.0: "2", 0.5: "0.5", 0.0: "0", 32768.0: "32768", 1e21: "1000000000000000000000",
             float("inf"): "inf", 0.1 + 0.2: "0.30000000000000004"}
    for x, want in cases.items():
        assert ck.rust_f64(x) == want
        assert float(ck.rust_f64(x)) == x
    assert ck.rust_f64(float("nan")) == "NaN"


def test_schedule_pairs_round_trip():
    for s in (LrSchedule.Cosine(10, 100, 1e-5), LrSchedule.Linear(5, 50), LrSchedule.OneCycle(1.0, 100, 0.3),
              LrSchedule.Step(7, 0.5)):
        st = ck.ScheduleState(3e-4, s)
        pairs = ck.schedule_pairs(st)
        assert pairs[0] == ("schedule.enabled", "1") and pairs[1] == ("schedule.base_lr", "0.0003")
        back = ck.parse_schedule_state(dict(pairs))
        assert back == st
    assert ck.parse_schedule_state({}) is None
    with pytest.raises(ValueError, match="bad schedule.kind: nope"):
        ck.parse_schedule_state({"schedule.enabled": "1", "schedule.base_lr": "1", "schedule.kind": "nope"})
    with pytest.raises(ValueError, match="missing schedule.base_lr"):
        ck.parse_schedule_state({"schedule.enabled": "1"})


def test_meta_reader(tmp_path):
    p = tmp_path / "meta.txt"
    p.write_text("version=1\nepoch=3\n\nstep=17\nkey=a=b\n")
    assert ck.read_meta(str(p)) == {"version": "1", "epoch": "3", "step": "17", "key": "a=b"}
    p.write_text("novalue\n")
    with pytest.raises(ValueError):
        ck.read_meta(str(p))
