"""GPU tests of the reference-facing surfaces: the `cudarl_core` pybind11 module (class Environment with the
ten methods of the reference's src/python_bindings.cpp:8-26, plus aliases) and CudaQLearning."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def pkg():
    from conftest import load_package
    return load_package()


@pytest.fixture(scope="module")
def core():
    sys.path.insert(0, os.path.join(ROOT, "cudarl-arena_b200"))
    import cudarl_core
    return cudarl_core


def test_module_surface(core):
    assert core.__version__ == "0.1.0"
    env = core.Environment(5, 5)
    for name in ("reset", "step", "get_observation", "get_width", "get_height", "get_agent_position",
                 "add_obstacle", "set_goal", "add_trap"):
        assert hasattr(env, name)
    assert (env.get_width(), env.get_height()) == (5, 5)
    assert core.Environment().get_width() == 10 and core.Environment(width=7, height=3).get_height() == 3


def test_environment_like_the_reference_tests(core):
    """tests/test_environment.cpp and tests/test_environment.py of the reference, through Python."""
    env = core.Environment(5, 5)
    obs = env.reset()
    assert isinstance(obs, list) and len(obs) == 25 and obs[4] == 1.0           # goal cell value (:132-133)
    assert env.get_agent_position() == (2, 2)
    obs, reward, done, info = env.step(1)
    assert isinstance(reward, float) and isinstance(done, bool) and isinstance(info, str)
    assert reward < 0 and not done and info == "agent_pos: (3,2)"
    assert abs(reward + 0.01) < 1e-7
    for a in (1, 0, np.int64(0)):                 # src/train.py passes numpy integers from np.argmax
        obs, reward, done, info = env.step(a)
    assert done and reward == 1.0 and env.get_agent_position() == (4, 0)
    assert env.is_done() and env.get_reward() == 1.0 and (env.get_agent_x(), env.get_agent_y()) == (4, 0)
    env.reset()
    assert env.get_agent_position() == (2, 2) and not env.is_done()
    assert (env.width, env.height, env.env_id) == (5, 5, 0)
    assert core.Environment(4, 4, 7).env_id == 7                # third argument of the reference's second binding


def test_packaged_wrapper_duck_type(core):
    """python/cudarl/environment.py:62-89 of the reference drives its backend through reset / step / get_reward / is_done /
    get_agent_x / get_agent_y / get_grid_data; the cases of its tests/test_environment.py:35-66 restated on that duck type."""
    b = core.Environment(width=5, height=5)
    b.reset()
    grid = np.array(b.get_grid_data()).reshape(5, 5)
    assert grid.shape == (5, 5) and grid[0, 4] == 1.0
    b.step(1)
    obs, reward, done, info = np.array(b.get_grid_data()).reshape(5, 5), b.get_reward(), b.is_done(), {"agent_x": b.get_agent_x(), "agent_y": b.get_agent_y()}
    assert isinstance(reward, float) and isinstance(done, bool) and reward < 0 and not done and info == {"agent_x": 3, "agent_y": 2}


def test_cpp_consumer_program():
    """A C++ program written against the reference's header names (environment.h, environment_bridge.h, q_learning.cuh,
    core/environment.h) and linked with libcudarl.so: every case of the reference's tests/test_environment.cpp, the flow
    of src/main.cu, move semantics, getCellValue, the bridge with grid edits."""
    import subprocess
    exe = os.path.join(ROOT, "tests", "cpp", "facade_consumer")
    assert os.path.exists(exe), "tests/cpp/facade_consumer is not built (python cudarl-arena_b200/build.py)"
    r = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0 and " 0 failed" in r.stdout, r.stdout


def test_reference_demo_program_unmodified():
    """The reference's own src/main.cu, compiled without any change against the compatibility headers where its
    checkout was present at build time (the binary travels with the tree)."""
    import subprocess
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_main_demo")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/ref_main_demo not built (needs the reference checkout at build time)")
    r = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0, r.stdout
    assert "Step 0: Agent at (5,5)" in r.stdout and "Performing batch update of Q-values on GPU" in r.stdout and "Demo complete" in r.stdout


def test_obstacle_goal_trap_edits(core):
    env = core.Environment(5, 5)
    env.reset()
    env.add_obstacle(3, 2)
    _, r, d, _ = env.step(1)
    assert env.get_agent_position() == (2, 2) and abs(r + 0.01) < 1e-7           # blocked (src/kernels.cu:39-44)
    env.add_trap(2, 1, -0.5)
    _, r, d, _ = env.step(0)
    assert env.get_agent_position() == (2, 2) and r == -0.5                      # trap penalty (src/kernels.cu:61-63)
    env.set_goal(2, 3)
    obs, r, d, _ = env.step(2)
    assert d and r == 1.0 and obs[3 * 5 + 2] == 1.0 and obs[4] == 0.0 and obs[2 * 5 + 3] == -1.0 and obs[1 * 5 + 2] == -0.5


def test_cuda_q_learning(core):
    q = core.CudaQLearning(6, 4, 4, 0.5, 0.9)
    assert len(q.get_q_table()) == 96 and max(q.get_q_table()) == 0.0
    q.update_batch([(1, 1), (1, 1), (2, 3)], [2, 2, 0], [1.0, 1.0, -0.01], [(1, 2), (1, 2), (2, 2)], [True, True, False])
    f = np.float32
    v1 = f(0.5) * f(1.0)                                                         # 0 + 0.5 * (1 - 0)
    v2 = f(np.float64(f(0.5)) * np.float64(f(1.0) - v1) + np.float64(v1))       # the second update sees the first: 0.75
    assert q.get_q_value(1, 1, 2) == float(v2) and q.get_best_action(1, 1) == 2
    assert q.get_best_action(0, 0) == 0                                          # ties -> lowest index (src/q_learning.cu:196-206)
    with pytest.raises(RuntimeError, match="Inconsistent batch sizes"):
        q.update_batch([(0, 0)], [0, 1], [0.0], [(0, 0)], [False])
    with pytest.raises(RuntimeError, match="Invalid state or action"):
        q.get_q_value(6, 0, 0)
    with pytest.raises(RuntimeError, match="Invalid state"):
        q.get_best_action(0, 4)
    with pytest.raises(RuntimeError, match="Invalid Q-table size"):
        q.set_q_table([0.0] * 5)
    with pytest.raises(RuntimeError, match="Invalid state or action"):
        q.update_batch([(9, 9)], [0], [0.0], [(0, 0)], [False])
    big = 5000                                                                   # beyond the reference's 1024 cap
    q.update_batch([(i % 6, i % 4) for i in range(big)], [i % 4 for i in range(big)], [0.1] * big,
                   [(0, 0)] * big, [False] * big)
    t = q.get_q_table()
    q.set_q_table(t)
    assert q.get_q_table() == t


def test_vec_environment(core):
    v = core.VecEnvironment(width=32, height=32, num_envs=2048, obstacle_kind=1, obstacle_p=0.2, goal_mode=2, num_goals=3,
                            start_mode=2, max_steps=200, eps_kind=0, eps0=0.2)
    v.train_steps(300)
    s = v.stats()
    assert s["steps"] == 300 and s["env_steps"] == 300 * 2048 and s["goals"] > 0
    assert v.q_table().shape == (32, 32, 4) and v.cells().shape == (32, 32)
    r = v.eval_rollout(100)
    assert r["envs"] == 2048 and 0 <= r["reached"] <= 2048
    rew, done = v.step(np.zeros(2048, np.int32))
    assert rew.shape == (2048,) and done.dtype == np.uint8


def test_npy_checkpoint_interop_on_a_trained_world(pkg, tmp_path):
    """QTableAgent.save / load of the reference (src/train.py:150-168) use np.save of a float64 (W, H, A) array indexed [x, y, a].
    A table trained on the GPU goes out in that layout and comes back bit-identical; a file written the reference's way loads."""
    cfg = pkg.preset("C2")
    w = pkg.VecGridWorld(cfg)
    w.train_steps(400)
    q = w.get_q()
    path = str(tmp_path / "qtable_agent.npy")
    pkg.save_q_npy(path, w)
    on_disk = np.load(path)
    assert on_disk.shape == (64, 64, 4) and on_disk.dtype == np.float64
    x, y, a = 17, 42, 3
    assert on_disk[x, y, a] == np.float64(q[(y * 64 + x) * 4 + a])
    w2 = pkg.VecGridWorld(cfg)
    pkg.load_q_npy(path, w2)
    assert np.array_equal(w2.get_q(), q)
    ref_style = np.zeros((64, 64, 4))                       # as QTableAgent.__init__ makes it (src/train.py:63)
    ref_style[5, 9, 2] = 0.625
    np.save(path, ref_style)
    pkg.load_q_npy(path, w2)
    assert w2.get_q()[(9 * 64 + 5) * 4 + 2] == np.float32(0.625) and np.count_nonzero(w2.get_q()) == 1
    with pytest.raises(ValueError):
        np.save(path, np.zeros((3, 3, 4))); pkg.load_q_npy(path, w2)


def test_trainer_shaped_loop_over_the_batched_api(core):
    """Trainer.train of the reference's package (python/cudarl/trainer.py:39-121): per episode reset, step until done or
    max_steps, collect episode reward / length, evaluate every so often -- over VecEnvironment, where one call steps every
    environment and the episode bookkeeping happens on the device."""
    v = core.VecEnvironment(width=48, height=48, num_envs=4096, obstacle_kind=1, obstacle_p=0.15, goal_mode=2, num_goals=2,
                            start_mode=2, max_steps=300, eps_kind=3, eps0=1.0, eps_end=0.05, eps_steps=1500)
    history = {"episodes": [], "mean_length": [], "success_rate": []}
    prev = v.stats()
    for chunk in range(10):                                   # 10 "epochs" of 200 batched steps
        v.train_steps(200)
        s = v.stats()
        ep, st = s["episodes"] - prev["episodes"], s["env_steps"] - prev["env_steps"]
        history["episodes"].append(ep)
        history["mean_length"].append(st / max(ep, 1))
        ev = v.eval_rollout(300)                               # evaluate(): greedy, training state untouched
        history["success_rate"].append(ev["reached"] / ev["envs"])
        prev = s
    assert v.stats()["device_error"] == 0
    assert history["mean_length"][-1] < history["mean_length"][0]          # episodes get shorter
    assert history["success_rate"][-1] > history["success_rate"][0] and history["success_rate"][-1] > 0.5


def test_reference_training_script_shape(core):
    """The loop of the reference's src/train.py:191-222 with its QTableAgent arithmetic restated inline:
    Environment(w,h) positional, reset(), get_agent_position() as NumPy index, step(np.int64), 4-tuple."""
    rng = np.random.RandomState(0)
    env = core.Environment(6, 6)
    q = np.zeros((6, 6, 4))
    eps, lengths = 1.0, []
    for episode in range(60):
        obs = env.reset()
        pos = env.get_agent_position()
        for step in range(200):
            a = rng.randint(0, 4) if rng.rand() < eps else np.argmax(q[pos[0], pos[1]])
            nobs, r, done, info = env.step(a)
            npos = env.get_agent_position()
            nq = 0 if done else np.max(q[npos[0], npos[1]])
            q[pos[0], pos[1], a] += 0.1 * (r + 0.99 * nq - q[pos[0], pos[1], a])
            eps *= 0.995
            pos = npos
            if done:
                break
        lengths.append(step + 1)
    assert np.mean(lengths[-10:]) < np.mean(lengths[:10])       # it learns the way to (5,0)
