"""CPU tests of the boundary: the shared library loads and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cudarl.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cudarl_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(pkg):
    lib = pkg.load()
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), "libcudarl.so does not export " + n


def test_python_binding_covers_header(pkg):
    assert sorted(pkg.ABI) == declared_symbols()


def test_config_struct_layout(pkg):
    c = pkg.default_config()          # filled by the C side: sizes must agree or struct_size is off
    assert c.struct_size == ctypes.sizeof(pkg.Config)
    assert (c.width, c.height, c.num_envs) == (10, 10, 1)
    assert abs(c.lr - 0.1) < 1e-7 and abs(c.gamma - 0.99) < 1e-7
    assert c.eps0 == 1.0 and c.eps_decay == 0.995


def test_version(pkg):
    assert pkg.load().cudarl_version() == b"0.1.0"


def test_create_rejects_bad_arguments(pkg):
    lib = pkg.load()
    h = ctypes.c_void_p()
    c = pkg.default_config()
    c.struct_size = 12
    assert lib.cudarl_create(ctypes.byref(c), ctypes.byref(h)) < 0
    assert b"struct_size" in lib.cudarl_last_global_error()
    c = pkg.default_config()
    c.width = 0
    assert lib.cudarl_create(ctypes.byref(c), ctypes.byref(h)) < 0
    assert not h.value


def test_reference_checkpoint_layout_roundtrip(pkg, tmp_path):
    """.npy interop with QTableAgent.save/load of the reference (src/train.py:150-168): float64 (W,H,A) [x,y,a]."""
    import numpy as np
    w, h = 7, 5
    native = np.arange(w * h * 4, dtype=np.float32) * 0.25
    ref = pkg.q_to_reference_layout(native, w, h)
    assert ref.shape == (w, h, 4) and ref.dtype == np.float64
    for x, y, a in [(0, 0, 0), (6, 4, 3), (3, 2, 1)]:
        assert ref[x, y, a] == native[(y * w + x) * 4 + a]
    assert np.array_equal(pkg.q_from_reference_layout(ref), native)

    class FakeWorld:
        W, H = w, h
        def get_q(self): return native
        def set_q(self, q): self.got = q
    fw = FakeWorld()
    path = str(tmp_path / "qtable_agent.npy")
    pkg.save_q_npy(path, fw)
    pkg.load_q_npy(path, fw)
    assert np.array_equal(fw.got, native)
