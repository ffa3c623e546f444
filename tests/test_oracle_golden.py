"""CPU tests: pin the oracle (oracle/oracle.cpp) against
  * the published Random123 known-answer vectors for Philox4x32-10,
  * the known-answer cases of the reference's tests/test_environment.cpp,
  * fixtures produced by the reference's own Python CPU code (tests/golden/make_golden.py).
"""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def ref_env(pkg, orc, w=10, h=10, n=1):
    """The reference's default world: no obstacles, goal (W-1,0), start centre (src/environment.cu:9-10,43)."""
    return orc.Oracle(pkg.make_config(w, h, n))


def test_philox_known_answers(orc):
    # Random123 kat_vectors, philox4x32 with 10 rounds
    kat = [([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
           ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
           ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
            [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1])]
    for ctr, key, want in kat:
        assert list(orc.philox(ctr, key)) == want


class TestReferenceCatch2Cases:
    """tests/test_environment.cpp of the reference, case by case."""

    def test_initialisation(self, pkg, orc):          # :6-27
        e = ref_env(pkg, orc)
        x, y, t = e.get_state()
        assert (e.W, e.H) == (10, 10) and (x[0], y[0]) == (5, 5)
        s = e.get_stats()
        assert s.steps == 0

    def test_reset(self, pkg, orc):                   # :29-50
        e = ref_env(pkg, orc)
        e.step_actions([1]); e.step_actions([1])
        e.reset_all()
        x, y, t = e.get_state()
        assert (x[0], y[0], t[0]) == (5, 5, 0)

    @pytest.mark.parametrize("action,pos", [(1, (6, 5)), (2, (5, 6)), (3, (4, 5)), (0, (5, 4))])
    def test_unit_moves(self, pkg, orc, action, pos):  # :52-78
        e = ref_env(pkg, orc)
        r, d = e.step_actions([action])
        x, y, _ = e.get_state()
        assert (x[0], y[0]) == pos and r[0] == np.float32(-0.01) and d[0] == 0   # reward :92-97

    def test_boundary(self, pkg, orc):                # :80-90
        e = ref_env(pkg, orc, 3, 3)
        e.step_actions([1]); assert e.get_state()[0][0] == 2
        e.step_actions([1]); assert e.get_state()[0][0] == 2

    def test_goal(self, pkg, orc):                    # :100-120
        e = ref_env(pkg, orc, 5, 5)
        e.reset_all()
        for a in (1, 1, 0, 0):
            r, d = e.step_actions([a])
        assert d[0] == 1 and r[0] == np.float32(1.0)

    def test_grid(self, pkg, orc):                    # :122-140
        e = ref_env(pkg, orc, 5, 5)
        cells = e.get_cells()
        assert cells.size == 25 and cells[0 * 5 + 4] == 2          # goal value 1.0 at (4,0)


def test_env_walks_match_reference_python(pkg, orc):
    """MockEnvironment of the reference's src/gui.py:84-137 on seeded random walks (incl. invalid actions)."""
    g = np.load(os.path.join(GOLD, "reference_env.npz"))
    k = 0
    while "env%d_wh" % k in g:
        w, h = g["env%d_wh" % k]
        e = ref_env(pkg, orc, int(w), int(h))
        x, y, _ = e.get_state()
        assert (x[0], y[0]) == tuple(g["env%d_start" % k])
        sticky = 0
        for i, a in enumerate(g["env%d_actions" % k]):
            r, d = e.step_actions([int(a)])
            x, y, _ = e.get_state()
            assert (x[0], y[0]) == (g["env%d_x" % k][i], g["env%d_y" % k][i]), (k, i)
            assert r[0] == np.float32(g["env%d_reward" % k][i])
            sticky |= int(g["env%d_done" % k][i])
            assert d[0] == sticky                 # CUDA reference: done is sticky (src/environment.cu:45)
        k += 1
    assert k == 6


def to_native(q_xya):
    """(W,H,A) indexed [x,y,a] (src/train.py:63) -> (y*W+x)*A+a (src/kernels.cu:96)."""
    return np.ascontiguousarray(np.transpose(q_xya, (1, 0, 2))).reshape(-1)


def test_td_update_matches_reference_python(pkg, orc):
    """QTableAgent.update (src/train.py:110-148, float64) vs the oracle's fp32 update; tolerance 1e-5 relative."""
    g = np.load(os.path.join(GOLD, "reference_td.npz"))
    for k in range(3):
        w, h = (int(v) for v in g["td%d_dims" % k])
        lr, gamma = g["td%d_hyper" % k]
        e = orc.Oracle(pkg.make_config(w, h, 1, lr=float(lr), gamma=float(gamma)))
        e.set_q(to_native(g["td%d_q0" % k]).astype(np.float32))
        n = len(g["td%d_a" % k])
        for i in range(n):
            sl = slice(i, i + 1)
            rc = e.update_batch(g["td%d_sx" % k][sl], g["td%d_sy" % k][sl], g["td%d_a" % k][sl], g["td%d_r" % k][sl],
                                g["td%d_nx" % k][sl], g["td%d_ny" % k][sl], g["td%d_done" % k][sl])
            assert rc == 0
        want = to_native(g["td%d_q1" % k])
        np.testing.assert_allclose(e.get_q(), want, rtol=1e-5, atol=2e-6)


def test_greedy_tie_break_matches_reference_python(pkg, orc):
    """np.argmax first-max rule (src/train.py:108) through a train step with epsilon 0."""
    g = np.load(os.path.join(GOLD, "reference_greedy.npz"))
    q, want = g["greedy_q"], g["greedy_action"]
    w, h = q.shape[0], q.shape[1]
    e = orc.Oracle(pkg.make_config(w, h, w * h, eps_kind=pkg.EPS_FIXED, eps0=0.0))
    e.set_q(to_native(q).astype(np.float32))
    xs, ys = np.meshgrid(np.arange(w), np.arange(h), indexing="ij")
    e.set_state(xs.ravel(), ys.ravel(), np.zeros(w * h))
    e.train_steps(1)
    a, _, _ = e.get_trace()
    assert np.array_equal(a.reshape(w, h), want)


def test_epsilon_decay_matches_reference_python(pkg, orc):
    """eps *= 0.995 after every update in float64 (src/train.py:141)."""
    g = np.load(os.path.join(GOLD, "reference_td.npz"))
    eps_after = g["td0_eps"]
    e = orc.Oracle(pkg.make_config(10, 10, 1))          # defaults: eps 1.0, decay 0.995 per step
    for k in range(50):
        e.train_steps(1)
        used = e.get_stats().epsilon
        want = 1.0 if k == 0 else eps_after[k - 1]
        assert used == np.float32(want)
    assert abs(eps_after[499] - 0.995 ** 500) < 1e-12    # 0.082: the value logged in the reference's training.log


def test_collision_fold_order(pkg, orc):
    """Same (state, action) several times in one batch: the reference update applied in index order."""
    e = orc.Oracle(pkg.make_config(4, 4, 1, lr=0.5, gamma=0.9))
    q0 = np.linspace(-1, 1, 64).astype(np.float32)
    e.set_q(q0)
    sx, sy, a = [1, 1, 1, 2], [2, 2, 2, 0], [3, 3, 3, 1]
    r = np.array([1.0, -0.01, 0.25, -0.01], np.float32)
    nx, ny, dn = [0, 3, 1, 2], [0, 3, 2, 1], [0, 1, 0, 0]
    assert e.update_batch(sx, sy, a, r, nx, ny, dn) == 0
    q = q0.copy().reshape(16, 4)
    f32 = np.float32

    def fma(x, y, z):
        return f32(np.float64(x) * np.float64(y) + np.float64(z))   # exact product of two fp32 fits fp64; one rounding
    targets = []
    for i in range(4):
        m = f32(0) if dn[i] else q0.reshape(16, 4)[ny[i] * 4 + nx[i]].max()
        targets.append(fma(f32(0.9), m, r[i]))            # targets come from the table before the batch
    for i in range(4):                                     # applied one after the other: each sees the previous result
        s = sy[i] * 4 + sx[i]
        q[s, a[i]] = fma(f32(0.5), f32(targets[i] - q[s, a[i]]), q[s, a[i]])
    assert np.array_equal(e.get_q(), q.reshape(-1))


def test_grid_generators(pkg, orc):
    c = pkg.preset("C2")
    e = orc.Oracle(c)
    cells = e.get_cells()
    assert (cells == 2).sum() == 1
    frac = (cells == 1).mean()
    assert 0.12 < frac < 0.18
    x, y, t = e.get_state()
    assert np.all(cells[y * 64 + x] == 0) and np.all(t == 0)
    c4 = pkg.preset("C4", num_envs=16)
    c4.width = c4.height = 128
    e4 = orc.Oracle(c4)
    cells = e4.get_cells().reshape(128, 128)
    assert abs((cells == 1).mean() - 0.25) < 0.01
    c1 = pkg.preset("C1")
    e1 = orc.Oracle(c1)
    cells = e1.get_cells().reshape(10, 10)
    assert cells[9, 9] == 2 and cells[0, 0] == 0
    assert tuple(v[0] for v in e1.get_state()) == (0, 0, 0)


def test_auto_reset_and_timeout(pkg, orc):
    c = pkg.make_config(6, 6, 64, start_mode=pkg.START_RANDOM, max_steps=5, eps_kind=pkg.EPS_FIXED, eps0=1.0,
                        obstacle_kind=pkg.OBST_BERNOULLI, obstacle_p=0.2)
    e = orc.Oracle(c)
    for k in range(1, 12):
        e.train_steps(1)
        _, _, t = e.get_state()
        assert t.max() < 5
    s = e.get_stats()
    assert s.episodes == s.goals + s.timeouts and s.timeouts > 0
    assert s.env_steps == 11 * 64


def test_replica_average(pkg, orc):
    cfgs = [pkg.make_config(5, 5, 8, env_offset=8 * r, start_mode=pkg.START_RANDOM, eps_kind=pkg.EPS_FIXED, eps0=0.5) for r in range(4)]
    os_ = [orc.Oracle(c) for c in cfgs]
    for o in os_:
        o.train_steps(7)
    qs = [o.get_q() for o in os_]
    assert not np.array_equal(qs[0], qs[1])
    orc.average_replicas(os_)
    want = (((qs[0] + qs[1]) + qs[2]) + qs[3]) * np.float32(0.25)
    for o in os_:
        assert np.array_equal(o.get_q(), want)


def test_multithreaded_oracle_is_identical(pkg, orc):
    c = pkg.preset("C2", num_envs=8192)
    a, b = orc.Oracle(c), orc.Oracle(c, threads=4)
    a.train_steps(20); b.train_steps(20)
    assert np.array_equal(a.get_q(), b.get_q())
    assert all(np.array_equal(u, v) for u, v in zip(a.get_state(), b.get_state()))
