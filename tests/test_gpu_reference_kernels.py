"""GPU cross-check against the reference's OWN CUDA kernels (compiled unmodified into oracle/_ref/libref.so
by cudarl-arena_b200/build.py where the reference checkout exists; the .so travels with the tree).
Pins the parts no reference test covers: the obstacle-aware step kernel and both TD-update kernels."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libref.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libref.so not built (needs the reference checkout at build time)")
    L = C.CDLL(REF)
    L.ref_walk.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 5
    L.ref_update.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 7 + [C.c_float, C.c_float]
    return L


def p(a):
    return a.ctypes.data_as(C.c_void_p)


def ref_walk(L, which, w, h, grid, x0, y0, actions):
    n = len(actions)
    xs, ys = np.zeros(n, np.int32), np.zeros(n, np.int32)
    r, d = np.zeros(n, np.float32), np.zeros(n, np.uint8)
    a = np.ascontiguousarray(actions, np.int32)
    g = np.ascontiguousarray(grid, np.float32)
    assert L.ref_walk(which, w, h, p(g), x0, y0, n, p(a), p(xs), p(ys), p(r), p(d)) == 0
    return xs, ys, r, d


def test_step_environment_kernel_of_the_reference(pkg, ref):
    """src/environment.cu:17-48 launched as the reference does (<<<1,1>>> per step) vs step_actions."""
    rng = np.random.RandomState(3)
    for w, h in [(10, 10), (5, 5), (3, 7), (1, 4)]:
        e = pkg.VecGridWorld(pkg.make_config(w, h, 1))
        actions = rng.randint(-1, 6, 150)
        grid = np.zeros(w * h, np.float32); grid[w - 1] = 1.0
        xs, ys, r, d = ref_walk(ref, 0, w, h, grid, w // 2, h // 2, actions)
        for i, a in enumerate(actions):
            rr, dd = e.step_actions([a])
            x, y, _ = e.get_state()
            assert (x[0], y[0], rr[0], dd[0]) == (xs[i], ys[i], r[i], d[i]), (w, h, i)


def test_obstacle_aware_step_kernel_of_the_reference(pkg, ref):
    """src/kernels.cu:13-66 (obstacles block, goal cell ends the episode) vs step_actions on a seeded grid.
    Compared until the first goal hit: after that the two reference kernels themselves disagree
    (one tests the agent's cell, the other the target cell)."""
    rng = np.random.RandomState(4)
    checked = 0
    for trial in range(12):
        w, h = int(rng.randint(4, 14)), int(rng.randint(4, 14))
        cfg = pkg.make_config(w, h, 1, seed=1000 + trial, obstacle_kind=pkg.OBST_BERNOULLI, obstacle_p=0.25,
                              goal_mode=pkg.GOAL_SEEDED, num_goals=2, start_mode=pkg.START_RANDOM)
        e = pkg.VecGridWorld(cfg)
        cells = e.get_cells()
        grid = np.where(cells == 2, 1.0, np.where(cells == 1, -1.0, 0.0)).astype(np.float32)
        x, y, _ = e.get_state()
        actions = rng.randint(0, 4, 200)
        xs, ys, r, d = ref_walk(ref, 1, w, h, grid, int(x[0]), int(y[0]), actions)
        for i, a in enumerate(actions):
            rr, dd = e.step_actions([a])
            xx, yy, _ = e.get_state()
            assert (xx[0], yy[0], rr[0], dd[0]) == (xs[i], ys[i], r[i], d[i]), (trial, i)
            checked += 1
            if d[i]:
                break
    assert checked > 300


def test_trap_rule_of_the_reference_kernel(pkg, ref):
    """src/kernels.cu:61-63: a grid value in (-1, 0) blocks like an obstacle and is charged as the reward.  Traps set with
    cudarl_add_trap (the device trap table) against the reference's own step_environment_kernel on the float grid that
    carries the same penalties; a value of -1 or below is a plain obstacle there and here."""
    rng = np.random.RandomState(6)
    checked = charged = 0
    for trial in range(10):
        w, h = int(rng.randint(5, 12)), int(rng.randint(5, 12))
        cfg = pkg.make_config(w, h, 1, seed=2000 + trial, obstacle_kind=pkg.OBST_BERNOULLI, obstacle_p=0.1,
                              goal_mode=pkg.GOAL_SEEDED, num_goals=1, start_mode=pkg.START_RANDOM)
        e = pkg.VecGridWorld(cfg)
        x, y, _ = e.get_state()
        cells = e.get_cells()
        grid = np.where(cells == 2, 1.0, np.where(cells == 1, -1.0, 0.0)).astype(np.float32)
        free = [k for k in rng.permutation(w * h) if cells[k] == 0 and k != int(y[0]) * w + int(x[0])]
        for j, k in enumerate(free[: max(3, len(free) // 4)]):
            pen = np.float32(-rng.uniform(0.02, 0.98)) if j % 4 else np.float32(-1.5)
            e.add_trap(int(k % w), int(k // w), float(pen))
            grid[k] = pen
        actions = rng.randint(0, 4, 250)
        xs, ys, r, d = ref_walk(ref, 1, w, h, grid, int(x[0]), int(y[0]), actions)
        for i, a in enumerate(actions):
            rr, dd = e.step_actions([a])
            xx, yy, _ = e.get_state()
            assert (xx[0], yy[0], rr[0], dd[0]) == (xs[i], ys[i], r[i], d[i]), (trial, i)
            checked += 1
            charged += int(r[i] != np.float32(-0.01) and r[i] != 1.0)
            if d[i]:
                break
    assert checked > 300 and charged > 20


def race_free_batch(rng, w, h, n):
    """Unique (state, action) keys and no next-state that is also written: the reference kernels have no
    collision handling (plain read-modify-write, src/kernels.cu:99-114), so only such batches are defined."""
    cells = rng.permutation(w * h)
    half = len(cells) // 2
    src, dst = cells[:half], cells[half:]
    s = rng.choice(src, size=n, replace=False)
    s2 = rng.choice(dst, size=n)
    return dict(sx=(s % w).astype(np.int32), sy=(s // w).astype(np.int32), a=rng.randint(0, 4, n).astype(np.int32),
                r=rng.choice([-0.01, 1.0, -0.5], n).astype(np.float32), nx=(s2 % w).astype(np.int32), ny=(s2 // w).astype(np.int32),
                dn=(rng.rand(n) < 0.2).astype(np.uint8))


@pytest.mark.parametrize("which,clamp", [(0, 1), (1, 0)])
def test_td_update_kernels_of_the_reference(pkg, ref, which, clamp):
    """which=0: update_q_values_kernel (src/kernels.cu:68-116, max clamped at 0) vs legacy_clamp=1;
    which=1: cudarl::updateQValuesKernel (src/gpu/kernels.cu:7-54, true max) vs the default.  Bit-exact."""
    rng = np.random.RandomState(10 + which)
    w, h = 40, 30
    for lr, gamma, n in [(0.1, 0.99, 500), (0.5, 0.9, 64), (0.05, 0.995, 599)]:
        q0 = rng.uniform(-1, 1, w * h * 4).astype(np.float32)
        b = race_free_batch(rng, w, h, n)
        e = pkg.VecGridWorld(pkg.make_config(w, h, 1, lr=lr, gamma=gamma, legacy_clamp=clamp))
        e.set_q(q0)
        e.update_batch(**b)
        q = q0.copy()
        assert ref.ref_update(which, p(q), w, h, n, p(b["sx"]), p(b["sy"]), p(b["a"]), p(b["r"]), p(b["nx"]), p(b["ny"]), p(b["dn"]),
                              C.c_float(lr), C.c_float(gamma)) == 0
        assert not np.array_equal(q, q0)
        assert np.array_equal(e.get_q(), q), (which, lr)
