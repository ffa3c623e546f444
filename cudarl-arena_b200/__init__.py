"""cudarl-arena_b200 -- host-side mirror of the C ABI in include/cudarl.h.

The product is `libcudarl.so` (hand-written sm_100a CUDA behind a C ABI) plus the `cudarl_core`
pybind11 module with the reference's surface.  This Python file only binds the C ABI with ctypes
for tests, the benchmark and scripted use; it contains no arithmetic of its own and has no
fallback: if the shared library is missing, loading raises.

The directory name contains a hyphen, so import it by path, e.g.

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location("cudarl_arena_b200", ".../cudarl-arena_b200/__init__.py")
    m = importlib.util.module_from_spec(spec); sys.modules[spec.name] = m; spec.loader.exec_module(m)
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcudarl.so")
MAX_GOALS = 64
STATIC_MAX_BATCH = 65536
COMM_ID_BYTES = 128

OBST_NONE, OBST_BERNOULLI, OBST_WALLS = 0, 1, 2
GOAL_TOP_RIGHT, GOAL_LIST, GOAL_SEEDED = 0, 1, 2
START_CENTRE, START_FIXED, START_RANDOM = 0, 1, 2
EPS_FIXED, EPS_MULT_PER_STEP, EPS_MULT_PER_EPISODE, EPS_LINEAR = 0, 1, 2, 3
QINIT_ZERO, QINIT_UNIFORM = 0, 1


class Config(C.Structure):
    """cudarl_config of include/cudarl.h, field for field."""
    _fields_ = [
        ("struct_size", C.c_uint32), ("device", C.c_int32),
        ("width", C.c_int32), ("height", C.c_int32),
        ("num_envs", C.c_int64), ("env_offset", C.c_int64), ("seed", C.c_uint64),
        ("obstacle_kind", C.c_int32), ("obstacle_p", C.c_float),
        ("goal_mode", C.c_int32), ("num_goals", C.c_int32), ("goal_xy", C.c_int32 * (2 * MAX_GOALS)),
        ("start_mode", C.c_int32), ("start_x", C.c_int32), ("start_y", C.c_int32),
        ("max_steps", C.c_int32), ("lr", C.c_float), ("gamma", C.c_float),
        ("eps_kind", C.c_int32), ("reserved0", C.c_int32),
        ("eps0", C.c_double), ("eps_decay", C.c_double), ("eps_end", C.c_double),
        ("eps_steps", C.c_int64),
        ("q_init_kind", C.c_int32), ("q_init_scale", C.c_float),
        ("legacy_clamp", C.c_int32), ("sync_every", C.c_int32),
        ("rebucket_every", C.c_int32), ("tile_edge", C.c_int32), ("avg_over_nccl", C.c_int32), ("reserved", C.c_int32 * 1),
    ]

    def copy(self):
        c = Config()
        C.memmove(C.byref(c), C.byref(self), C.sizeof(Config))
        return c


class Stats(C.Structure):
    _fields_ = [("steps", C.c_int64), ("env_steps", C.c_int64), ("episodes", C.c_int64), ("goals", C.c_int64),
                ("timeouts", C.c_int64), ("conflicts", C.c_int64), ("long_chains", C.c_int64), ("chained", C.c_int64),
                ("reward_sum", C.c_double), ("epsilon", C.c_float), ("device_error", C.c_int32)]


class EvalStats(C.Structure):
    _fields_ = [("envs", C.c_int64), ("reached", C.c_int64), ("total_steps", C.c_int64), ("reward_sum", C.c_double)]


# every exported symbol of include/cudarl.h with (restype, argtypes)
_P = C.c_void_p
_I32P, _F32P, _U8P = C.POINTER(C.c_int32), C.POINTER(C.c_float), C.POINTER(C.c_uint8)
ABI = {
    "cudarl_default_config": (None, [C.POINTER(Config)]),
    "cudarl_create": (C.c_int, [C.POINTER(Config), C.POINTER(_P)]),
    "cudarl_destroy": (None, [_P]),
    "cudarl_last_error": (C.c_char_p, [_P]),
    "cudarl_last_global_error": (C.c_char_p, []),
    "cudarl_reset_all": (C.c_int, [_P]),
    "cudarl_step_actions": (C.c_int, [_P, _P, _P, _P]),
    "cudarl_step_actions_device": (C.c_int, [_P, _P, _P, _P]),
    "cudarl_train_steps": (C.c_int, [_P, C.c_int64]),
    "cudarl_train_steps_eps": (C.c_int, [_P, C.c_int64, _P]),
    "cudarl_synchronize": (C.c_int, [_P]),
    "cudarl_set_trace": (C.c_int, [_P, C.c_int]),
    "cudarl_get_trace": (C.c_int, [_P, _P, _P, _P]),
    "cudarl_eval_rollout": (C.c_int, [_P, C.c_int32, C.POINTER(EvalStats)]),
    "cudarl_update_batch": (C.c_int, [_P, C.c_int64, _P, _P, _P, _P, _P, _P, _P]),
    "cudarl_update_batch_static": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int64, _P, _P, _P, _P, _P, _P, _P,
                                            C.c_float, C.c_float, C.c_int32, _P]),
    "cudarl_get_state": (C.c_int, [_P, _P, _P, _P]),
    "cudarl_set_state": (C.c_int, [_P, _P, _P, _P]),
    "cudarl_get_reward_done": (C.c_int, [_P, _P, _P]),
    "cudarl_get_q": (C.c_int, [_P, _P]),
    "cudarl_set_q": (C.c_int, [_P, _P]),
    "cudarl_get_cells": (C.c_int, [_P, _P]),
    "cudarl_add_obstacle": (C.c_int, [_P, C.c_int32, C.c_int32]),
    "cudarl_set_goal": (C.c_int, [_P, C.c_int32, C.c_int32]),
    "cudarl_add_trap": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_float]),
    "cudarl_get_traps": (C.c_int, [_P, C.c_int32, _P, _P, C.POINTER(C.c_int32)]),
    "cudarl_set_legacy_clamp": (C.c_int, [_P, C.c_int]),
    "cudarl_get_stats": (C.c_int, [_P, C.POINTER(Stats)]),
    "cudarl_get_config": (C.c_int, [_P, C.POINTER(Config)]),
    "cudarl_comm_unique_id": (C.c_int, [_P]),
    "cudarl_comm_init": (C.c_int, [_P, _P, C.c_int32, C.c_int32]),
    "cudarl_average_replicas": (C.c_int, [_P]),
    "cudarl_comm_peer_memory": (C.c_int, [_P]),
    "cudarl_timer_start": (C.c_int, [_P]),
    "cudarl_timer_stop_ms": (C.c_int, [_P, C.POINTER(C.c_float)]),
    "cudarl_kernel_timing": (C.c_int, [_P, C.c_int]),
    "cudarl_kernel_time_ms": (C.c_int, [_P, C.POINTER(C.c_float), C.POINTER(C.c_int64)]),
    "cudarl_debug_set_copy_wait_polls": (C.c_int, [_P, C.c_int32]),
    "cudarl_version": (C.c_char_p, []),
}

_lib = None


def load():
    """dlopen libcudarl.so and type every entry point.  Raises if the library is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("libcudarl.so is not built (run `python cudarl-arena_b200/build.py`); "
                               "there is no CPU fallback")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in ABI.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def default_config():
    c = Config()
    load().cudarl_default_config(C.byref(c))
    return c


def make_config(width, height, num_envs, seed=0xC0DA2025, **kw):
    """Config with the reference defaults, then keyword overrides (goals=[(x,y),...] for a goal list)."""
    c = Config()
    c.struct_size = C.sizeof(Config)
    c.width, c.height, c.num_envs, c.seed = width, height, num_envs, seed
    c.goal_mode, c.start_mode = GOAL_TOP_RIGHT, START_CENTRE
    c.lr, c.gamma = 0.1, 0.99
    c.eps_kind, c.eps0, c.eps_decay, c.eps_end = EPS_MULT_PER_STEP, 1.0, 0.995, 0.0
    c.q_init_scale = 0.01
    goals = kw.pop("goals", None)
    if goals is not None:
        c.goal_mode, c.num_goals = GOAL_LIST, len(goals)
        for i, (gx, gy) in enumerate(goals):
            c.goal_xy[2 * i], c.goal_xy[2 * i + 1] = gx, gy
    for k, v in kw.items():
        if not hasattr(c, k):
            raise AttributeError("cudarl_config has no field %r" % k)
        setattr(c, k, v)
    return c


def preset(name, num_envs=None, env_offset=0, device=0, seed=0xC0DA2025):
    """The five workload configurations (grid, environments, hyper-parameters)."""
    if name == "C1":   # 10x10, one env, start (0,0), goal (9,9), Bernoulli(0.1), eps 1.0 x0.995 per episode
        c = make_config(10, 10, num_envs or 1, seed, obstacle_kind=OBST_BERNOULLI, obstacle_p=0.1, goals=[(9, 9)],
                        start_mode=START_FIXED, start_x=0, start_y=0, max_steps=500, lr=0.1, gamma=0.99,
                        eps_kind=EPS_MULT_PER_EPISODE, eps0=1.0, eps_decay=0.995)
    elif name == "C2":  # 64x64, 4096 envs, Bernoulli(0.15), one seeded goal, cap 1024, eps 0.1
        c = make_config(64, 64, num_envs or 4096, seed, obstacle_kind=OBST_BERNOULLI, obstacle_p=0.15,
                        goal_mode=GOAL_SEEDED, num_goals=1, start_mode=START_RANDOM, max_steps=1024,
                        lr=0.1, gamma=0.99, eps_kind=EPS_FIXED, eps0=0.1)
    elif name == "C3":  # 256x256, 65536 envs, Bernoulli(0.2), 8 goals, cap 4096, Q~U[0,0.01), eps 1.0->0.05 over 1e5
        c = make_config(256, 256, num_envs or 65536, seed, obstacle_kind=OBST_BERNOULLI, obstacle_p=0.2,
                        goal_mode=GOAL_SEEDED, num_goals=8, start_mode=START_RANDOM, max_steps=4096,
                        lr=0.05, gamma=0.99, eps_kind=EPS_LINEAR, eps0=1.0, eps_end=0.05, eps_steps=100000,
                        q_init_kind=QINIT_UNIFORM, q_init_scale=0.01)
    elif name == "C4":  # 1024x1024, 2^20 envs/GPU, walls 0.25, one goal, average every 64, gamma 0.995
        c = make_config(1024, 1024, num_envs or (1 << 20), seed, obstacle_kind=OBST_WALLS, obstacle_p=0.25,
                        goal_mode=GOAL_SEEDED, num_goals=1, start_mode=START_RANDOM, max_steps=4096,
                        lr=0.1, gamma=0.995, eps_kind=EPS_FIXED, eps0=0.1, sync_every=64)
    elif name == "C5":  # 4096x4096, 2^22 envs/GPU, Bernoulli(0.3), 64 goals, cap 16384, average every 256, eps 0.05
        c = make_config(4096, 4096, num_envs or (1 << 22), seed, obstacle_kind=OBST_BERNOULLI, obstacle_p=0.3,
                        goal_mode=GOAL_SEEDED, num_goals=64, start_mode=START_RANDOM, max_steps=16384,
                        lr=0.1, gamma=0.99, eps_kind=EPS_FIXED, eps0=0.05, sync_every=256)
    else:
        raise ValueError("unknown preset %r" % name)
    c.env_offset, c.device = env_offset, device
    return c


def q_to_reference_layout(q, width, height):
    """Table as the reference's Python agent stores and saves it (src/train.py:63,150-168): float64, shape
    (width, height, 4), indexed [x, y, a].  Input: the native fp32 layout (y*width + x)*4 + a."""
    return np.ascontiguousarray(np.asarray(q, np.float32).reshape(height, width, 4).transpose(1, 0, 2)).astype(np.float64)


def q_from_reference_layout(q_xya):
    """Inverse of q_to_reference_layout: (width, height, 4) indexed [x, y, a] -> native fp32 vector."""
    q = np.asarray(q_xya)
    assert q.ndim == 3 and q.shape[2] == 4
    return np.ascontiguousarray(q.transpose(1, 0, 2)).astype(np.float32).reshape(-1)


def save_q_npy(path, world):
    """Write the table of a VecGridWorld as the .npy file QTableAgent.save of the reference produces."""
    np.save(path, q_to_reference_layout(world.get_q(), world.W, world.H))


def load_q_npy(path, world):
    """Load a .npy written by the reference's QTableAgent.save (or save_q_npy) into a VecGridWorld."""
    q = np.load(path)
    if q.shape != (world.W, world.H, 4):
        raise ValueError("table shape %r does not match a %dx%d grid with 4 actions" % (q.shape, world.W, world.H))
    world.set_q(q_from_reference_layout(q))


class CudarlError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("cudarl error %d: %s" % (code, msg))
        self.code = code


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class VecGridWorld:
    """One shard (one GPU): N environments + one Q-table replica, through the C ABI."""

    def __init__(self, cfg):
        self.lib = load()
        self.cfg = cfg.copy()
        self.cfg.struct_size = C.sizeof(Config)
        self.h = C.c_void_p()
        rc = self.lib.cudarl_create(C.byref(self.cfg), C.byref(self.h))
        if rc != 0:
            raise CudarlError(rc, self.lib.cudarl_last_global_error().decode())
        self.N, self.W, self.H = int(cfg.num_envs), int(cfg.width), int(cfg.height)

    def _ck(self, rc):
        if rc != 0:
            raise CudarlError(rc, self.lib.cudarl_last_error(self.h).decode())

    def close(self):
        if self.h:
            self.lib.cudarl_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset_all(self):
        self._ck(self.lib.cudarl_reset_all(self.h))

    def step_actions(self, actions):
        a = np.ascontiguousarray(actions, dtype=np.int32)
        r = np.empty(self.N, np.float32)
        d = np.empty(self.N, np.uint8)
        self._ck(self.lib.cudarl_step_actions(self.h, _ptr(a), _ptr(r), _ptr(d)))
        return r, d

    def train_steps(self, n):
        self._ck(self.lib.cudarl_train_steps(self.h, n))

    def train_steps_eps(self, eps):
        e = np.ascontiguousarray(eps, dtype=np.float32)
        self._ck(self.lib.cudarl_train_steps_eps(self.h, len(e), _ptr(e)))

    def synchronize(self):
        self._ck(self.lib.cudarl_synchronize(self.h))

    def set_trace(self, on=True):
        self._ck(self.lib.cudarl_set_trace(self.h, 1 if on else 0))

    def get_trace(self):
        a, r, d = np.empty(self.N, np.int32), np.empty(self.N, np.float32), np.empty(self.N, np.uint8)
        self._ck(self.lib.cudarl_get_trace(self.h, _ptr(a), _ptr(r), _ptr(d)))
        return a, r, d

    def eval_rollout(self, max_steps):
        s = EvalStats()
        self._ck(self.lib.cudarl_eval_rollout(self.h, max_steps, C.byref(s)))
        return s

    def update_batch(self, sx, sy, a, r, nx, ny, dn):
        arrs = [np.ascontiguousarray(v, dtype=t) for v, t in
                ((sx, np.int32), (sy, np.int32), (a, np.int32), (r, np.float32), (nx, np.int32), (ny, np.int32), (dn, np.uint8))]
        self._ck(self.lib.cudarl_update_batch(self.h, len(arrs[0]), *[_ptr(v) for v in arrs]))

    def get_state(self):
        x, y, t = (np.empty(self.N, np.int32) for _ in range(3))
        self._ck(self.lib.cudarl_get_state(self.h, _ptr(x), _ptr(y), _ptr(t)))
        return x, y, t

    def set_state(self, x=None, y=None, t=None):
        x, y, t = (None if v is None else np.ascontiguousarray(v, dtype=np.int32) for v in (x, y, t))
        self._ck(self.lib.cudarl_set_state(self.h, _ptr(x), _ptr(y), _ptr(t)))

    def get_reward_done(self):
        r, d = np.empty(self.N, np.float32), np.empty(self.N, np.uint8)
        self._ck(self.lib.cudarl_get_reward_done(self.h, _ptr(r), _ptr(d)))
        return r, d

    def get_q(self):
        q = np.empty(self.W * self.H * 4, np.float32)
        self._ck(self.lib.cudarl_get_q(self.h, _ptr(q)))
        return q

    def set_q(self, q):
        q = np.ascontiguousarray(q, dtype=np.float32).ravel()
        assert q.size == self.W * self.H * 4
        self._ck(self.lib.cudarl_set_q(self.h, _ptr(q)))

    def get_cells(self):
        c = np.empty(self.W * self.H, np.uint8)
        self._ck(self.lib.cudarl_get_cells(self.h, _ptr(c)))
        return c

    def add_obstacle(self, x, y):
        self._ck(self.lib.cudarl_add_obstacle(self.h, x, y))

    def set_goal(self, x, y):
        self._ck(self.lib.cudarl_set_goal(self.h, x, y))

    def add_trap(self, x, y, penalty=-0.5):
        self._ck(self.lib.cudarl_add_trap(self.h, x, y, penalty))

    def get_traps(self):
        n = C.c_int32()
        self._ck(self.lib.cudarl_get_traps(self.h, 0, None, None, C.byref(n)))
        cells, pen = np.empty(n.value, np.int32), np.empty(n.value, np.float32)
        self._ck(self.lib.cudarl_get_traps(self.h, n.value, _ptr(cells), _ptr(pen), C.byref(n)))
        return cells, pen

    def get_stats(self):
        s = Stats()
        self._ck(self.lib.cudarl_get_stats(self.h, C.byref(s)))
        return s

    def comm_init(self, id_bytes, rank, nranks):
        buf = C.create_string_buffer(bytes(id_bytes), COMM_ID_BYTES)
        self._ck(self.lib.cudarl_comm_init(self.h, buf, rank, nranks))

    def average_replicas(self):
        self._ck(self.lib.cudarl_average_replicas(self.h))

    def comm_peer_memory(self):
        return bool(self.lib.cudarl_comm_peer_memory(self.h))

    def timer_start(self):
        self._ck(self.lib.cudarl_timer_start(self.h))

    def timer_stop_ms(self):
        ms = C.c_float()
        self._ck(self.lib.cudarl_timer_stop_ms(self.h, C.byref(ms)))
        return ms.value

    def kernel_timing(self, on):
        self._ck(self.lib.cudarl_kernel_timing(self.h, 1 if on else 0))

    def kernel_time_ms(self):
        a, n = C.c_float(), C.c_int64()
        self._ck(self.lib.cudarl_kernel_time_ms(self.h, C.byref(a), C.byref(n)))
        return a.value, n.value

    def debug_set_copy_wait_polls(self, polls):
        self._ck(self.lib.cudarl_debug_set_copy_wait_polls(self.h, polls))


def comm_unique_id():
    buf = C.create_string_buffer(COMM_ID_BYTES)
    rc = load().cudarl_comm_unique_id(buf)
    if rc != 0:
        raise CudarlError(rc, load().cudarl_last_global_error().decode())
    return buf.raw
