"""GPU parity tests: every call goes through the C ABI of libcudarl.so and is compared with the CPU
oracle on the same seeded inputs.  Integer/byte results (positions, step counters, actions, done flags,
cell classes) and fp32 rewards must be identical; the fp32 Q-table is required to be bit-identical as
well (the stated tolerance is 1e-5 relative, but a 1-ulp difference would eventually flip an argmax)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def pair(pkg, orc, cfg, threads=1):
    return pkg.VecGridWorld(cfg), orc.Oracle(cfg, threads=threads)


def assert_same(gpu, cpu, what=""):
    for name, a, b in zip("xyt", gpu.get_state(), cpu.get_state()):
        assert np.array_equal(a, b), "%s: state %s differs in %d envs" % (what, name, int((a != b).sum()))
    qa, qb = gpu.get_q(), cpu.get_q()
    if not np.array_equal(qa, qb):
        bad = np.flatnonzero(qa != qb)
        raise AssertionError("%s: Q differs in %d entries, first %d: %r vs %r" % (what, bad.size, bad[0], qa[bad[0]], qb[bad[0]]))


def lockstep(gpu, cpu, steps, check_every=1, what=""):
    gpu.set_trace(True)
    for k in range(steps):
        gpu.train_steps(1)
        cpu.train_steps(1)
        ta, tb = gpu.get_trace(), cpu.get_trace()
        for name, a, b in zip(("action", "reward", "done"), ta, tb):
            assert np.array_equal(a, b), "%s step %d: %s differs" % (what, k, name)
        if (k + 1) % check_every == 0 or k == steps - 1:
            assert_same(gpu, cpu, "%s step %d" % (what, k))
    sa, sb = gpu.get_stats(), cpu.get_stats()
    assert sa.device_error == 0
    for f in ("steps", "env_steps", "episodes", "goals", "timeouts", "conflicts"):
        assert getattr(sa, f) == getattr(sb, f), f
    assert sa.epsilon == sb.epsilon and sa.reward_sum == sb.reward_sum
    return sa


# ---- the reference's own known answers, through the CUDA path ---------------------------------------

def ref_world(pkg, w=10, h=10):
    return pkg.VecGridWorld(pkg.make_config(w, h, 1))


def test_reference_catch2_cases(pkg):
    """tests/test_environment.cpp of the reference (:6-140)."""
    e = ref_world(pkg)
    x, y, t = e.get_state()
    assert (x[0], y[0], t[0]) == (5, 5, 0)
    r, d = e.get_reward_done()
    assert r[0] == 0.0 and d[0] == 0
    e.step_actions([1]); e.step_actions([1]); e.reset_all()
    x, y, t = e.get_state()
    r, d = e.get_reward_done()
    assert (x[0], y[0]) == (5, 5) and r[0] == 0.0 and d[0] == 0
    for action, pos in [(1, (6, 5)), (2, (5, 6)), (3, (4, 5)), (0, (5, 4))]:
        e.reset_all()
        r, d = e.step_actions([action])
        x, y, _ = e.get_state()
        assert (x[0], y[0]) == pos and r[0] == np.float32(-0.01) and d[0] == 0
    s = ref_world(pkg, 3, 3)
    s.step_actions([1]); assert s.get_state()[0][0] == 2
    s.step_actions([1]); assert s.get_state()[0][0] == 2
    g = ref_world(pkg, 5, 5)
    for a in (1, 1, 0, 0):
        r, d = g.step_actions([a])
    assert d[0] == 1 and r[0] == np.float32(1.0)
    cells = g.get_cells()
    assert cells.size == 25 and cells[4] == 2


def test_env_walks_match_reference_python(pkg):
    g = np.load(os.path.join(GOLD, "reference_env.npz"))
    for k in range(6):
        w, h = (int(v) for v in g["env%d_wh" % k])
        e = ref_world(pkg, w, h)
        sticky = 0
        for i, a in enumerate(g["env%d_actions" % k]):
            r, d = e.step_actions([int(a)])
            x, y, _ = e.get_state()
            assert (x[0], y[0]) == (g["env%d_x" % k][i], g["env%d_y" % k][i])
            assert r[0] == np.float32(g["env%d_reward" % k][i])
            sticky |= int(g["env%d_done" % k][i])
            assert d[0] == sticky


def to_native(q_xya):
    return np.ascontiguousarray(np.transpose(q_xya, (1, 0, 2))).reshape(-1)


def test_td_update_matches_reference_python(pkg):
    """QTableAgent.update of the reference (float64) vs update_batch, 1e-5 relative."""
    g = np.load(os.path.join(GOLD, "reference_td.npz"))
    for k in range(3):
        w, h = (int(v) for v in g["td%d_dims" % k])
        lr, gamma = g["td%d_hyper" % k]
        e = pkg.VecGridWorld(pkg.make_config(w, h, 1, lr=float(lr), gamma=float(gamma)))
        e.set_q(to_native(g["td%d_q0" % k]).astype(np.float32))
        for i in range(len(g["td%d_a" % k])):
            sl = slice(i, i + 1)
            e.update_batch(g["td%d_sx" % k][sl], g["td%d_sy" % k][sl], g["td%d_a" % k][sl], g["td%d_r" % k][sl],
                           g["td%d_nx" % k][sl], g["td%d_ny" % k][sl], g["td%d_done" % k][sl])
        np.testing.assert_allclose(e.get_q(), to_native(g["td%d_q1" % k]), rtol=1e-5, atol=2e-6)


def test_greedy_tie_break_matches_reference_python(pkg):
    g = np.load(os.path.join(GOLD, "reference_greedy.npz"))
    q, want = g["greedy_q"], g["greedy_action"]
    w, h = q.shape[0], q.shape[1]
    e = pkg.VecGridWorld(pkg.make_config(w, h, w * h, eps_kind=pkg.EPS_FIXED, eps0=0.0))
    e.set_q(to_native(q).astype(np.float32))
    xs, ys = np.meshgrid(np.arange(w), np.arange(h), indexing="ij")
    e.set_state(xs.ravel(), ys.ravel(), np.zeros(w * h))
    e.set_trace(True)
    e.train_steps(1)
    a, _, _ = e.get_trace()
    assert np.array_equal(a.reshape(w, h), want)


# ---- grid / start generators ------------------------------------------------------------------------

@pytest.mark.parametrize("name,kw", [("C1", {}), ("C2", {}), ("C3", {}), ("C4", {"num_envs": 4096}), ("C5", {"num_envs": 4096})])
def test_grid_and_starts_match_oracle(pkg, orc, name, kw):
    cfg = pkg.preset(name, **kw)
    if name in ("C4", "C5"):
        cfg.width = cfg.height = 512
    gpu, cpu = pair(pkg, orc, cfg)
    assert np.array_equal(gpu.get_cells(), cpu.get_cells())
    for a, b in zip(gpu.get_state(), cpu.get_state()):
        assert np.array_equal(a, b)
    assert np.array_equal(gpu.get_q(), cpu.get_q())


# ---- the fused step, in lockstep --------------------------------------------------------------------

def test_lockstep_c1(pkg, orc):
    gpu, cpu = pair(pkg, orc, pkg.preset("C1"))
    s = lockstep(gpu, cpu, 1500, check_every=50, what="C1")
    assert s.episodes > 0


@pytest.mark.parametrize("edge", [0, 8, 16])
def test_lockstep_c2(pkg, orc, edge):
    cfg = pkg.preset("C2")
    cfg.tile_edge = edge                  # 0 = chosen from the population density; the results never depend on it
    gpu, cpu = pair(pkg, orc, cfg)
    s = lockstep(gpu, cpu, 300, check_every=10, what="C2 edge %d" % edge)
    assert s.conflicts > 0


@pytest.mark.parametrize("edge", [8, 16])
def test_lockstep_sparse_population_both_tile_edges(pkg, orc, edge):
    """The benchmark's density (one environment per four cells, 30 % obstacles, several goals) on a grid whose sides are
    not multiples of the tile edge: partial tiles at the right and bottom rims, most tiles on the register-held fast path."""
    cfg = pkg.preset("C5", num_envs=9000)
    cfg.width, cfg.height, cfg.num_goals, cfg.max_steps, cfg.tile_edge = 203, 181, 6, 50, edge
    gpu, cpu = pair(pkg, orc, cfg)
    lockstep(gpu, cpu, 160, check_every=8, what="sparse edge %d" % edge)


def test_lockstep_c3_uniform_q_linear_eps(pkg, orc):
    cfg = pkg.preset("C3")
    cfg.eps_steps = 200           # reach the floor inside the test
    gpu, cpu = pair(pkg, orc, cfg, threads=4)
    lockstep(gpu, cpu, 260, check_every=20, what="C3")


def test_lockstep_dense_collisions(pkg, orc):
    """Tiny grids packed with environments: hundreds to thousands of updates of one (cell, action) per step."""
    for w, h, n, steps in [(3, 3, 512, 40), (5, 5, 4096, 25), (2, 2, 6000, 12), (2, 1, 300, 5)]:
        cfg = pkg.make_config(w, h, n, start_mode=pkg.START_RANDOM, eps_kind=pkg.EPS_FIXED, eps0=0.3, max_steps=7, lr=0.25)
        gpu, cpu = pair(pkg, orc, cfg)
        s = lockstep(gpu, cpu, steps, what="dense %dx%d" % (w, h))
        assert s.long_chains > 0 or n < 512          # cells with more than 24 occupants are counted


def test_lockstep_one_tile_beyond_16_bit_counts(pkg, orc):
    """More environments in one tile than the 16-bit per-action counters of the step kernel hold: the tile counts
    in 32-bit counters in global memory instead."""
    cfg = pkg.make_config(3, 2, 70000, start_mode=pkg.START_RANDOM, eps_kind=pkg.EPS_FIXED, eps0=0.3, max_steps=5, lr=0.2)
    gpu, cpu = pair(pkg, orc, cfg, threads=4)
    lockstep(gpu, cpu, 8, what="70000 on 3x2")


def test_lockstep_with_traps(pkg, orc):
    """Traps (src/kernels.cu:61-63 of the reference): obstacles that charge their penalty.  The fused step must use the
    penalty as the reward of the blocked (state, action) in its TD target, the trace must show it, and caller-driven
    steps must return it."""
    cfg = pkg.make_config(20, 14, 2500, start_mode=pkg.START_RANDOM, goal_mode=pkg.GOAL_SEEDED, num_goals=2, obstacle_kind=pkg.OBST_BERNOULLI,
                          obstacle_p=0.1, eps_kind=pkg.EPS_FIXED, eps0=0.5, max_steps=30, lr=0.2)
    gpu, cpu = pair(pkg, orc, cfg)
    rng = np.random.RandomState(11)
    cells = gpu.get_cells()
    placed = 0
    for k in rng.permutation(20 * 14):
        if cells[k] == 0 and placed < 25:
            pen = float(np.float32(-rng.uniform(0.05, 0.95))) if placed % 5 else -2.0      # every fifth: outside (-1, 0) = a plain obstacle
            gpu.add_trap(int(k % 20), int(k // 20), pen); cpu.add_trap(int(k % 20), int(k // 20), pen)
            placed += 1
    assert np.array_equal(gpu.get_cells(), cpu.get_cells())
    tc, tp = gpu.get_traps()
    assert len(tc) == 20 and np.all(np.diff(tc) > 0) and np.all((tp < 0) & (tp > -1))
    gpu.reset_all(); cpu.reset_all()
    lockstep(gpu, cpu, 60, check_every=5, what="traps")
    gpu.set_trace(True); gpu.train_steps(1); cpu.train_steps(1)
    assert np.array_equal(gpu.get_trace()[1], cpu.get_trace()[1])
    assert (gpu.get_trace()[1] != np.float32(-0.01)).sum() > (gpu.get_trace()[1] == 1.0).sum()    # some penalties were charged
    for _ in range(10):
        a = rng.randint(0, 4, 2500)
        (r1, d1), (r2, d2) = gpu.step_actions(a), cpu.step_actions(a)
        assert np.array_equal(r1, r2) and np.array_equal(d1, d2)
    # a goal or a plain obstacle put on a trap cell removes the trap
    gpu.add_obstacle(int(tc[0] % 20), int(tc[0] // 20)); cpu.add_obstacle(int(tc[0] % 20), int(tc[0] // 20))
    assert len(gpu.get_traps()[0]) == 19
    gpu.train_steps(20); cpu.train_steps(20)
    assert_same(gpu, cpu, "after removing a trap")


def test_copy_wait_that_runs_out_is_reported_not_hung(pkg):
    """The step kernel bounds every wait for a tile copy.  With the bound set to a single look at the barrier the wait runs out
    before the copy can have landed: the warp records the failure, lets its copies land and leaves; the next call that waits
    for the device returns CUDARL_ERR_DEVICE + CUDARL_DEVERR_COPY_TIMEOUT instead of handing out a half-updated table."""
    cfg = pkg.preset("C3", num_envs=20000)
    g = pkg.VecGridWorld(cfg)
    g.train_steps(3); g.synchronize()
    assert g.get_stats().device_error == 0
    g.debug_set_copy_wait_polls(1)
    g.train_steps(1)
    with pytest.raises(pkg.CudarlError) as ei:
        g.synchronize()
    assert ei.value.code == 3000 + 32
    g.debug_set_copy_wait_polls(0)
    with pytest.raises(pkg.CudarlError):
        g.get_q()                                            # the flag is sticky: this context's results are not to be trusted
    g.close()
    h = pkg.VecGridWorld(cfg)                                # the device itself is fine
    h.train_steps(5); h.synchronize()
    assert h.get_stats().device_error == 0


def test_lockstep_legacy_clamp_and_walls(pkg, orc):
    cfg = pkg.preset("C4", num_envs=20000)
    cfg.width = cfg.height = 96
    cfg.legacy_clamp = 1
    gpu, cpu = pair(pkg, orc, cfg)
    lockstep(gpu, cpu, 120, check_every=10, what="walls")


def test_many_steps_per_call_and_schedules(pkg, orc):
    for kind, kw in [(pkg.EPS_MULT_PER_STEP, {}), (pkg.EPS_MULT_PER_EPISODE, {"max_steps": 6}), (pkg.EPS_LINEAR, {"eps_end": 0.1, "eps_steps": 90})]:
        cfg = pkg.make_config(24, 17, 3000, start_mode=pkg.START_RANDOM, obstacle_kind=pkg.OBST_BERNOULLI, obstacle_p=0.2,
                              goal_mode=pkg.GOAL_SEEDED, num_goals=5, eps_kind=kind, eps0=1.0, eps_decay=0.97, **kw)
        gpu, cpu = pair(pkg, orc, cfg)
        for n in (1, 7, 64, 33):
            gpu.train_steps(n); cpu.train_steps(n)
            assert gpu.get_stats().epsilon == cpu.get_stats().epsilon
            assert_same(gpu, cpu, "kind %d after +%d" % (kind, n))


def test_caller_epsilon_array(pkg, orc):
    cfg = pkg.preset("C2", num_envs=1000)
    gpu, cpu = pair(pkg, orc, cfg)
    eps = np.linspace(1.0, 0.0, 40).astype(np.float32)
    gpu.train_steps_eps(eps); cpu.train_steps_eps(eps)
    assert_same(gpu, cpu, "eps array")


def test_state_roundtrip_and_external_steps_then_training(pkg, orc):
    """Caller-driven steps and set_state happen in environment order; training must re-bucket the records."""
    cfg = pkg.preset("C2", num_envs=2048)
    gpu, cpu = pair(pkg, orc, cfg)
    rng = np.random.RandomState(5)
    gpu.train_steps(5); cpu.train_steps(5)
    for _ in range(6):
        a = rng.randint(-1, 6, size=2048)
        ra, da = gpu.step_actions(a)
        rb, db = cpu.step_actions(a)
        assert np.array_equal(ra, rb) and np.array_equal(da, db)
    gpu.train_steps(9); cpu.train_steps(9)
    assert_same(gpu, cpu, "after external steps")
    x, y, t = cpu.get_state()
    perm = rng.permutation(2048)
    gpu.set_state(x[perm], y[perm], t[perm]); cpu.set_state(x[perm], y[perm], t[perm])
    gpu.reset_all(); cpu.reset_all()
    gpu.train_steps(9); cpu.train_steps(9)
    assert_same(gpu, cpu, "after set_state + reset")
    with pytest.raises(pkg.CudarlError):
        gpu.set_state(np.full(2048, 64), y, t)


def test_update_batch_with_duplicates(pkg, orc):
    rng = np.random.RandomState(11)
    cfg = pkg.make_config(9, 7, 1, lr=0.3, gamma=0.95)
    gpu, cpu = pair(pkg, orc, cfg)
    q0 = rng.uniform(-1, 1, 9 * 7 * 4).astype(np.float32)
    gpu.set_q(q0); cpu.set_q(q0)
    for n in (1, 5, 300, 5000, 40000, 40000, 40000):   # far beyond the reference's 1024 cap (src/q_learning.cu:10)
        b = dict(sx=rng.randint(0, 9, n), sy=rng.randint(0, 7, n), a=rng.randint(0, 4, n),
                 r=rng.choice([-0.01, 1.0, 0.5], n).astype(np.float32), nx=rng.randint(0, 9, n), ny=rng.randint(0, 7, n),
                 dn=(rng.rand(n) < 0.2).astype(np.uint8))
        gpu.update_batch(**b)
        assert cpu.update_batch(**b) == 0
        assert np.array_equal(gpu.get_q(), cpu.get_q()), n
    with pytest.raises(pkg.CudarlError):        # "Invalid state or action" (src/q_learning.cu:212-214)
        gpu.update_batch([9], [0], [0], [0.0], [0], [0], [0])
    assert gpu.get_stats().device_error == 0
    # two cells, thousands of transitions each, call after call: the global-scratch sort path every time
    tiny_g, tiny_c = pair(pkg, orc, pkg.make_config(2, 1, 1, lr=0.3, gamma=0.95))
    for _ in range(4):
        n = 4000
        b = dict(sx=rng.randint(0, 2, n), sy=np.zeros(n, np.int32), a=rng.randint(0, 4, n), r=rng.choice([-0.01, 1.0], n).astype(np.float32),
                 nx=rng.randint(0, 2, n), ny=np.zeros(n, np.int32), dn=(rng.rand(n) < 0.2).astype(np.uint8))
        tiny_g.update_batch(**b)
        assert tiny_c.update_batch(**b) == 0
        assert np.array_equal(tiny_g.get_q(), tiny_c.get_q())
    assert tiny_g.get_stats().device_error == 0


def test_eval_rollout(pkg, orc):
    cfg = pkg.preset("C2")
    gpu, cpu = pair(pkg, orc, cfg)
    gpu.train_steps(400); cpu.train_steps(400)
    for cap in (1, 50, 400):
        a, b = gpu.eval_rollout(cap), cpu.eval_rollout(cap)
        assert (a.envs, a.reached, a.total_steps, a.reward_sum) == (b.envs, b.reached, b.total_steps, b.reward_sum)
    gpu.train_steps(3); cpu.train_steps(3)       # training state untouched by the rollouts
    assert_same(gpu, cpu, "after eval")


def test_obstacle_and_goal_edits(pkg, orc):
    cfg = pkg.make_config(8, 8, 64, start_mode=pkg.START_RANDOM, eps_kind=pkg.EPS_FIXED, eps0=0.5)
    gpu, cpu = pair(pkg, orc, cfg)
    for o in ((3, 3), (4, 3), (0, 7)):
        gpu.add_obstacle(*o); cpu.add_obstacle(*o)
    gpu.set_goal(6, 6); cpu.set_goal(6, 6)
    assert np.array_equal(gpu.get_cells(), cpu.get_cells())
    gpu.reset_all(); cpu.reset_all()
    gpu.train_steps(30); cpu.train_steps(30)
    assert_same(gpu, cpu, "edited grid")


def test_determinism_run_twice(pkg):
    cfg = pkg.preset("C3")
    qs = []
    for _ in range(2):
        e = pkg.VecGridWorld(cfg)
        e.train_steps(100)
        qs.append((e.get_q(), e.get_state()))
        e.close()
    assert np.array_equal(qs[0][0], qs[1][0])
    assert all(np.array_equal(a, b) for a, b in zip(qs[0][1], qs[1][1]))


def test_full_size_c5_lockstep_and_properties(pkg, orc):
    """The benchmark workload at full size: 4096x4096 cells, 4,194,304 environments.  Steps against the (multi-threaded)
    oracle that cross a re-sizing of the record regions, with one tile crowded beyond the 16-bit counters and a stream of
    arrivals into one tile that overflows its arrival buffer into the spill list; then invariants that do not need the oracle."""
    cfg = pkg.preset("C5")
    cfg.rebucket_every = 2
    gpu, cpu = pair(pkg, orc, cfg, threads=os.cpu_count() or 8)
    cpu.count_conflicts(False)
    cells = gpu.get_cells().reshape(4096, 4096)
    assert np.array_equal(cells.ravel(), cpu.get_cells())
    x, y, t = gpu.get_state()
    # 70,000 environments on one free cell inside a tile (32-bit counters), 3,000 on a free cell in the top row of another tile
    # whose upper neighbour is free too: with an all-zero table the greedy action is "up", so they all arrive in the tile above
    # in one step -- far more than the 32 arrival slots.
    ys, xs = np.nonzero(cells[1030:1036, 2048:2064] == 0)      # rows 6..11 of the tile: four steps in any direction stay inside it
    x[:70000], y[:70000] = 2048 + xs[0], 1030 + ys[0]
    cand = [(cx, cy) for cy in range(2064, 2400, 16) for cx in range(512, 528) if cells[cy, cx] == 0 and cells[cy - 1, cx] == 0]
    x[70000:73000], y[70000:73000] = cand[0]
    gpu.set_state(x, y, t); cpu.set_state(x, y, t)
    for k in range(4):
        gpu.train_steps(1); cpu.train_steps(1)
    assert_same(gpu, cpu, "C5 full size")
    cpu.close()
    gpu.train_steps(60)
    x, y, t = gpu.get_state()
    cells = gpu.get_cells()
    occ = cells[y.astype(np.int64) * 4096 + x]
    assert np.all(occ == 0)                                  # nobody stands on an obstacle or a goal
    assert t.max() < 16384 and t.min() >= 0
    s = gpu.get_stats()
    assert s.device_error == 0 and s.steps == 64 and s.env_steps == 64 * (1 << 22)
    assert s.episodes == s.goals + s.timeouts
    q = gpu.get_q()
    assert np.isfinite(q).all() and q.max() <= 1.0 and q.min() >= -1.0


def test_region_resizing_never_changes_results(pkg, orc):
    """The per-tile record regions are re-sized from the populations every few steps; any period (and none) must
    give the same bits, and the state must come back in environment order."""
    base = pkg.preset("C3", num_envs=20000)
    base.width = base.height = 96
    ref = orc.Oracle(base, threads=4)
    ref.train_steps(70)
    want_state, want_q = ref.get_state(), ref.get_q()
    for period in (1, 3, 8, 50, -1):
        cfg = base.copy()
        cfg.rebucket_every = period
        g = pkg.VecGridWorld(cfg)
        for n in (1, 9, 60):
            g.train_steps(n)
        for a, b in zip(g.get_state(), want_state):
            assert np.array_equal(a, b), "period %d" % period
        assert np.array_equal(g.get_q(), want_q), "period %d" % period
        assert g.get_stats().device_error == 0
        g.close()


def test_synchronised_step_cap_mass_restart(pkg, orc):
    """Environments that started together and never reach a goal hit the step cap in the same step: nearly all of them draw a
    fresh start cell at once, far more arrivals per tile than an arrival buffer holds, so the spill list carries most of the
    population.  With the re-bucketing that the library schedules right after such a step, and without any re-bucketing
    (every tile then filters the whole spill list), the results are the oracle's."""
    base = pkg.preset("C5", num_envs=60000)
    base.width, base.height, base.num_goals, base.max_steps = 500, 490, 2, 20
    ref = orc.Oracle(base, threads=min(8, os.cpu_count() or 1))
    ref.train_steps(45)
    want_state, want_q, ws = ref.get_state(), ref.get_q(), ref.get_stats()
    assert ws.timeouts > 2 * 50000                      # two mass restarts happened
    for period in (0, -1):
        cfg = base.copy()
        cfg.rebucket_every = period
        g = pkg.VecGridWorld(cfg)
        for n in (19, 1, 1, 24):
            g.train_steps(n)
        for a, b in zip(g.get_state(), want_state):
            assert np.array_equal(a, b), "period %d" % period
        assert np.array_equal(g.get_q(), want_q), "period %d" % period
        gs = g.get_stats()
        assert gs.device_error == 0 and (gs.timeouts, gs.goals) == (ws.timeouts, ws.goals)
        g.close()


def test_step_cap_beyond_the_record_format_is_refused(pkg):
    """A tile record keeps 24 bits of an episode's step count: a larger cap is refused at creation, the largest one is accepted."""
    cfg = pkg.make_config(8, 8, 16, start_mode=pkg.START_RANDOM, eps_kind=pkg.EPS_FIXED, eps0=0.5, max_steps=0xFFFFFF)
    with pytest.raises(pkg.CudarlError):
        pkg.VecGridWorld(cfg)
    cfg.max_steps = 0xFFFFFE
    g = pkg.VecGridWorld(cfg)
    g.train_steps(3)
    assert g.get_stats().device_error == 0
    x, y, t = g.get_state()
    with pytest.raises(pkg.CudarlError):                # a step count the records cannot hold
        g.set_state(x, y, np.full_like(t, 0xFFFFFF))
    g.set_state(x, y, np.full_like(t, 0xFFFFFD))        # one step short of the cap: every environment times out in the next step
    g.train_steps(1)
    assert g.get_stats().timeouts >= 16 - g.get_stats().goals and g.get_stats().device_error == 0
    assert int(g.get_state()[2].max()) <= 1
    g.close()


def test_odd_sizes_and_tiny_populations(pkg, orc):
    for w, h, n in [(1, 7, 5), (7, 1, 33), (13, 11, 1), (31, 3, 257), (5, 5, 0)]:
        cfg = pkg.make_config(w, h, n, start_mode=pkg.START_RANDOM, goal_mode=pkg.GOAL_SEEDED, num_goals=1,
                              obstacle_kind=pkg.OBST_BERNOULLI, obstacle_p=0.1, eps_kind=pkg.EPS_FIXED, eps0=0.4, max_steps=9)
        gpu, cpu = pair(pkg, orc, cfg)
        gpu.train_steps(25); cpu.train_steps(25)
        assert_same(gpu, cpu, "%dx%d n=%d" % (w, h, n))
        a, b = gpu.eval_rollout(20), cpu.eval_rollout(20)
        assert (a.reached, a.total_steps) == (b.reached, b.total_steps)


def test_c2_long_run(pkg, orc):
    """C2 for 10^5 batched steps (4.1e8 environment-steps) in one go: still bit-identical, counters included."""
    cfg = pkg.preset("C2")
    gpu, cpu = pair(pkg, orc, cfg, threads=min(8, os.cpu_count() or 1))
    cpu.count_conflicts(False)
    for _ in range(4):
        gpu.train_steps(25000); cpu.train_steps(25000)
    assert_same(gpu, cpu, "C2 after 1e5 steps")
    sa, sb = gpu.get_stats(), cpu.get_stats()
    assert (sa.steps, sa.episodes, sa.goals, sa.timeouts) == (sb.steps, sb.episodes, sb.goals, sb.timeouts)
    assert sa.device_error == 0 and sa.goals > 100000
    q = gpu.get_q()
    assert np.isfinite(q).all() and q.max() <= 1.0 + 1e-6 and q.min() >= -1.0 - 1e-6     # bounded however crowded a cell gets
    a, b = gpu.eval_rollout(1024), cpu.eval_rollout(1024)
    assert (a.reached, a.total_steps) == (b.reached, b.total_steps) and a.reached > 3000     # it has learnt the way
