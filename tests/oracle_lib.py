"""ctypes binding of oracle/liboracle.so -- the CPU checker.  Test infrastructure only."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from conftest import load_package  # noqa: E402

pkg = load_package()
LIB_PATH = os.path.join(ROOT, "oracle", "liboracle.so")
_lib = None


def lib():
    global _lib
    if _lib is None:
        src = os.path.join(ROOT, "oracle", "oracle.cpp")
        if (not os.path.exists(LIB_PATH)) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
            subprocess.check_call(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fPIC", "-shared", "-pthread",
                                   "-o", LIB_PATH, src])
        L = C.CDLL(LIB_PATH)
        L.orc_create.restype = C.c_void_p
        L.orc_create.argtypes = [C.POINTER(pkg.Config)]
        L.orc_error.restype = C.c_char_p
        L.orc_error.argtypes = [C.c_void_p]
        for name in ("orc_destroy", "orc_reset_all"):
            getattr(L, name).argtypes = [C.c_void_p]
            getattr(L, name).restype = None
        L.orc_set_threads.argtypes = [C.c_void_p, C.c_int]
        L.orc_count_conflicts.argtypes = [C.c_void_p, C.c_int]
        L.orc_step_actions.argtypes = [C.c_void_p] * 4
        L.orc_train_steps.argtypes = [C.c_void_p, C.c_int64]
        L.orc_train_steps_eps.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        L.orc_get_trace.argtypes = [C.c_void_p] * 4
        L.orc_eval_rollout.argtypes = [C.c_void_p, C.c_int32, C.POINTER(pkg.EvalStats)]
        L.orc_update_batch.argtypes = [C.c_void_p, C.c_int64] + [C.c_void_p] * 7
        L.orc_update_batch.restype = C.c_int
        L.orc_get_state.argtypes = [C.c_void_p] * 4
        L.orc_set_state.argtypes = [C.c_void_p] * 4
        L.orc_get_q.argtypes = [C.c_void_p] * 2
        L.orc_set_q.argtypes = [C.c_void_p] * 2
        L.orc_get_cells.argtypes = [C.c_void_p] * 2
        L.orc_add_obstacle.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.orc_set_goal.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.orc_add_trap.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float]
        L.orc_get_stats.argtypes = [C.c_void_p, C.POINTER(pkg.Stats)]
        L.orc_average_replicas.argtypes = [C.POINTER(C.c_void_p), C.c_int]
        L.orc_philox.argtypes = [C.c_void_p] * 3
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def philox(ctr, key):
    c = np.asarray(ctr, np.uint32)
    k = np.asarray(key, np.uint32)
    o = np.zeros(4, np.uint32)
    lib().orc_philox(_p(c), _p(k), _p(o))
    return o


class Oracle:
    """Same method names as the package's VecGridWorld, computed on the CPU."""

    def __init__(self, cfg, threads=1):
        self.L = lib()
        self.cfg = cfg.copy()
        self.cfg.struct_size = C.sizeof(pkg.Config)
        self.h = C.c_void_p(self.L.orc_create(C.byref(self.cfg)))
        err = self.L.orc_error(self.h).decode()
        if err:
            self.L.orc_destroy(self.h)
            self.h = None
            raise RuntimeError("oracle: " + err)
        self.N, self.W, self.H = int(cfg.num_envs), int(cfg.width), int(cfg.height)
        if threads > 1:
            self.L.orc_set_threads(self.h, threads)

    def close(self):
        if self.h:
            self.L.orc_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def count_conflicts(self, on):
        self.L.orc_count_conflicts(self.h, 1 if on else 0)

    def reset_all(self):
        self.L.orc_reset_all(self.h)

    def step_actions(self, actions):
        a = np.ascontiguousarray(actions, dtype=np.int32)
        r, d = np.empty(self.N, np.float32), np.empty(self.N, np.uint8)
        self.L.orc_step_actions(self.h, _p(a), _p(r), _p(d))
        return r, d

    def train_steps(self, n):
        self.L.orc_train_steps(self.h, n)

    def train_steps_eps(self, eps):
        e = np.ascontiguousarray(eps, dtype=np.float32)
        self.L.orc_train_steps_eps(self.h, len(e), _p(e))

    def get_trace(self):
        a, r, d = np.empty(self.N, np.int32), np.empty(self.N, np.float32), np.empty(self.N, np.uint8)
        self.L.orc_get_trace(self.h, _p(a), _p(r), _p(d))
        return a, r, d

    def eval_rollout(self, max_steps):
        s = pkg.EvalStats()
        self.L.orc_eval_rollout(self.h, max_steps, C.byref(s))
        return s

    def update_batch(self, sx, sy, a, r, nx, ny, dn):
        arrs = [np.ascontiguousarray(v, dtype=t) for v, t in
                ((sx, np.int32), (sy, np.int32), (a, np.int32), (r, np.float32), (nx, np.int32), (ny, np.int32), (dn, np.uint8))]
        return self.L.orc_update_batch(self.h, len(arrs[0]), *[_p(v) for v in arrs])

    def get_state(self):
        x, y, t = (np.empty(self.N, np.int32) for _ in range(3))
        self.L.orc_get_state(self.h, _p(x), _p(y), _p(t))
        return x, y, t

    def set_state(self, x=None, y=None, t=None):
        x, y, t = (None if v is None else np.ascontiguousarray(v, dtype=np.int32) for v in (x, y, t))
        self.L.orc_set_state(self.h, _p(x), _p(y), _p(t))

    def get_q(self):
        q = np.empty(self.W * self.H * 4, np.float32)
        self.L.orc_get_q(self.h, _p(q))
        return q

    def set_q(self, q):
        q = np.ascontiguousarray(q, dtype=np.float32).ravel()
        self.L.orc_set_q(self.h, _p(q))

    def get_cells(self):
        c = np.empty(self.W * self.H, np.uint8)
        self.L.orc_get_cells(self.h, _p(c))
        return c

    def add_obstacle(self, x, y):
        return self.L.orc_add_obstacle(self.h, x, y)

    def set_goal(self, x, y):
        return self.L.orc_set_goal(self.h, x, y)

    def add_trap(self, x, y, penalty=-0.5):
        return self.L.orc_add_trap(self.h, x, y, penalty)

    def get_stats(self):
        s = pkg.Stats()
        self.L.orc_get_stats(self.h, C.byref(s))
        return s


def average_replicas(oracles):
    arr = (C.c_void_p * len(oracles))(*[o.h for o in oracles])
    lib().orc_average_replicas(arr, len(oracles))
