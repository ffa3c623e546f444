"""cudarl_update_batch_static: the TD update for callers that must not allocate device memory
(real-time loops, plug-ins under a framework that owns the device heap, processes at their memory cap).

The entry point takes caller-owned DEVICE buffers and keeps its working memory in a fixed static array
inside the library.  This test drives it through the C ABI and compares the resulting table with what the
allocating entry point (cudarl_update_batch on a context) produces for the same batch -- bit for bit,
which is the tolerance every other Q-table check here uses -- twice in a row, so that whatever the first
call left behind in the shared array is seen by the second.  The file name sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


class DeviceBuffers:
    """Device memory for the test itself, straight from the CUDA runtime (the entry point under test
    allocates nothing; its caller -- here the test -- owns every buffer)."""

    def __init__(self):
        self.rt = None
        for name in ("libcudart.so.12", "libcudart.so", "/usr/local/cuda/lib64/libcudart.so.12"):
            try:
                self.rt = C.CDLL(name)
                break
            except OSError:
                continue
        assert self.rt is not None, "CUDA runtime library not found"
        self.rt.cudaMalloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t]
        self.rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        self.rt.cudaFree.argtypes = [C.c_void_p]
        self.ptrs = []

    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        p = C.c_void_p()
        assert self.rt.cudaMalloc(C.byref(p), max(arr.nbytes, 16)) == 0
        assert self.rt.cudaMemcpy(p, arr.ctypes.data_as(C.c_void_p), arr.nbytes, 1) == 0
        self.ptrs.append(p)
        return p

    def download(self, p, like):
        out = np.empty_like(like)
        assert self.rt.cudaDeviceSynchronize() == 0
        assert self.rt.cudaMemcpy(out.ctypes.data_as(C.c_void_p), p, out.nbytes, 2) == 0
        return out

    def close(self):
        for p in self.ptrs:
            self.rt.cudaFree(p)
        self.ptrs = []


def make_batch(rng, w, h, n):
    return dict(sx=rng.randint(0, w, n).astype(np.int32), sy=rng.randint(0, h, n).astype(np.int32),
                a=rng.randint(0, 4, n).astype(np.int32), r=rng.choice([-0.01, 1.0, 0.25], n).astype(np.float32),
                nx=rng.randint(0, w, n).astype(np.int32), ny=rng.randint(0, h, n).astype(np.int32),
                dn=(rng.rand(n) < 0.2).astype(np.uint8))


@pytest.mark.parametrize("w,h,sizes", [(9, 7, (3000, 50000)), (300, 200, (65536, 1)), (2, 1, (4000, 4000))])
def test_static_entry_point_matches_allocating_one(pkg, w, h, sizes):
    lib = pkg.load()
    rng = np.random.RandomState(w * 1000 + h)
    lr, gamma = 0.3, 0.95
    ref = pkg.VecGridWorld(pkg.make_config(w, h, 1, lr=lr, gamma=gamma))      # existing, allocating path
    q0 = rng.uniform(-1, 1, w * h * 4).astype(np.float32)
    ref.set_q(q0)
    dev = DeviceBuffers()
    d_q = dev.upload(q0)
    try:
        for n in sizes:                                  # two calls in a row on the same static scratch
            b = make_batch(rng, w, h, n)
            ref.update_batch(**b)
            d = {k: dev.upload(v) for k, v in b.items()}
            rc = lib.cudarl_update_batch_static(d_q, w, h, n, d["sx"], d["sy"], d["a"], d["r"], d["nx"], d["ny"], d["dn"],
                                                C.c_float(lr), C.c_float(gamma), 0, None)
            assert rc == 0
            got = dev.download(d_q, q0)
            assert np.array_equal(got, ref.get_q()), "table differs after a batch of %d" % n
    finally:
        dev.close()
        ref.close()


def test_static_entry_point_rejects_oversized_batches(pkg):
    lib = pkg.load()
    dev = DeviceBuffers()
    q = np.zeros(16, np.float32)
    d_q = dev.upload(q)
    z = dev.upload(np.zeros(4, np.int32))
    try:
        rc = lib.cudarl_update_batch_static(d_q, 2, 2, pkg.STATIC_MAX_BATCH + 1, z, z, z, z, z, z, z, C.c_float(0.1), C.c_float(0.9), 0, None)
        assert rc == -5
        assert np.array_equal(dev.download(d_q, q), q)    # nothing was launched
    finally:
        dev.close()
