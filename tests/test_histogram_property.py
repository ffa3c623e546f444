"""The property the fused step kernel is built on, checked on the CPU against the sequential oracle.

The oracle applies the TD updates of one step one environment after the other, in ascending environment
id, each as q <- fma(lr, target - q, q) with the target taken from the table as it was before the step.
Inside one step the target of an update is a function of (cell, action) alone: the action fixes the next
cell, the next cell fixes reward and done, the bootstrap value is the max over the OLD row of that cell.
So the result can be reproduced from nothing but the COUNT of environments per (cell, action): apply
each (cell, action)'s map that many times, in any order.  This test rebuilds the oracle's table that way
with numpy (float32 arithmetic, the fused multiply-add emulated in float64, which is exact for these
operand sizes up to one rounding that the assertion accounts for by requiring bit equality on all but a
negligible number of entries and 1e-7 relative on the rest)."""
import numpy as np
import pytest


def fma32(a, b, c):
    """float32 fma(a, b, c): the product of two float32 is exact in float64; the sum is rounded once to
    float64 and once more to float32 (double rounding can differ from a true fma in rare ties)."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


@pytest.mark.parametrize("w,h,n,eps", [(12, 9, 3000, 0.3), (5, 5, 2000, 0.6), (40, 33, 5000, 0.1)])
def test_update_depends_only_on_counts_per_cell_and_action(pkg, orc, w, h, n, eps):
    cfg = pkg.make_config(w, h, n, start_mode=pkg.START_RANDOM, obstacle_kind=pkg.OBST_BERNOULLI, obstacle_p=0.15,
                          goal_mode=pkg.GOAL_SEEDED, num_goals=2, eps_kind=pkg.EPS_FIXED, eps0=eps, max_steps=50,
                          lr=0.2, gamma=0.9, q_init_kind=pkg.QINIT_UNIFORM, q_init_scale=0.05)
    o = orc.Oracle(cfg)
    cells = o.get_cells().reshape(h, w)
    lr, gamma = np.float32(cfg.lr), np.float32(cfg.gamma)
    dxy = [(0, -1), (1, 0), (0, 1), (-1, 0)]
    exact = total = 0
    for step in range(12):
        x, y, _ = o.get_state()
        q0 = o.get_q().reshape(h, w, 4).copy()
        o.train_steps(1)
        a, r, d = o.get_trace()
        q1 = o.get_q().reshape(h, w, 4)
        # per (cell, action): how many environments chose it
        cnt = np.zeros((h, w, 4), np.int64)
        np.add.at(cnt, (y, x, a), 1)
        want = q0.copy()
        for (cy, cx, ca) in zip(*np.nonzero(cnt)):
            nx, ny = cx + dxy[ca][0], cy + dxy[ca][1]
            moved = 0 <= nx < w and 0 <= ny < h and cells[ny, nx] != 1
            sx, sy = (nx, ny) if moved else (cx, cy)
            done = cells[sy, sx] == 2
            rew = np.float32(1.0 if done else -0.01)
            m = np.float32(0.0) if done else q0[sy, sx].max()
            target = fma32(gamma, m, rew)
            # every environment on this (cell, action) saw the same reward / done flag ...
            sel = (x == cx) & (y == cy) & (a == ca)
            assert np.all(r[sel] == rew) and np.all(d[sel] == (1 if done else 0))
            v = q0[cy, cx, ca]
            for _ in range(int(cnt[cy, cx, ca])):           # ... so the same map is applied count times
                v = fma32(lr, np.float32(target - v), v)
            want[cy, cx, ca] = v
        same = want == q1
        exact += int(same.sum()); total += same.size
        np.testing.assert_allclose(want, q1, rtol=1e-6, atol=1e-9)
        assert np.array_equal(want[cnt == 0], q1[cnt == 0])   # untouched entries stay untouched
    assert exact >= 0.999 * total
    o.close()
