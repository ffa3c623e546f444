"""The reference's own drivers -- run_training.py and src/train.py, unmodified -- on this repository's drop-in files.

Two legs.  Without a GPU the native module cannot construct an environment, so the CPU leg puts a stand-in module
`cudarl_core` with the native module's surface (built on the CPU oracle) behind the shim: it proves that the shipped
`python/cudarl/mock_env.py` is what run_training.py picks up and that the scripts accept the surface.  The GPU leg runs
the same scripts on the native module where a reference checkout is present beside it, and in any case drives the native
class through the shim with the call sequence of src/train.py:191-222."""
import os
import sys

import numpy as np
import pytest

import ref_drivers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
needs_ref = pytest.mark.skipif(ref_drivers.reference_root() is None,
                               reason="no checkout of the reference project here (set CUDARL_REFERENCE); its scripts are never copied")

FAKE_CORE = '''
"""Stand-in for the native cudarl_core module on a machine without a GPU: same class, same methods, CPU oracle inside."""
import sys
sys.path.insert(0, %r)
import oracle_lib
from conftest import load_package
pkg = load_package()
__version__ = "0.1.0"
class Environment:
    def __init__(self, width=10, height=10, env_id=0):
        self._o = oracle_lib.Oracle(pkg.make_config(width, height, 1))
        self._w, self._h, self._r, self._d = width, height, 0.0, False
    def _obs(self):
        return [1.0 if c == 2 else (-1.0 if c == 1 else 0.0) for c in self._o.get_cells()]
    def reset(self):
        self._o.reset_all(); self._r, self._d = 0.0, False
        return self._obs()
    def step(self, action):
        r, d = self._o.step_actions([int(action)])
        self._r, self._d = float(r[0]), bool(d[0]) or self._d
        x, y = self.get_agent_position()
        return self._obs(), self._r, self._d, "agent_pos: (%%d,%%d)" %% (x, y)
    def get_agent_position(self):
        x, y, _ = self._o.get_state()
        return (int(x[0]), int(y[0]))
    def get_observation(self): return self._obs()
    def get_width(self): return self._w
    def get_height(self): return self._h
'''


def _check_training_run(rc, out, tmp, episodes):
    assert rc == 0, out[-3000:]
    assert "Training completed" in out and "Done!" in out, out[-3000:]
    assert "Mock environment" not in out                       # the reference's print-only stand-in was NOT what ran
    lengths = ref_drivers.average_lengths(out)
    assert len(lengths) >= 10 and lengths[-1] < lengths[0], lengths     # it learns the way to the goal corner
    q = np.load(os.path.join(tmp, "overlay", "results", "qtable_agent.npy"))
    assert q.shape == (6, 6, 4) and q.dtype == np.float64 and np.abs(q).max() > 0      # QTableAgent.save, src/train.py:150-158


@needs_ref
def test_reference_drivers_pick_up_the_shim_cpu(tmp_path):
    backend = tmp_path / "fake_backend"
    backend.mkdir()
    (backend / "cudarl_core.py").write_text(FAKE_CORE % os.path.join(ROOT, "tests"))
    ov, env = ref_drivers.make_overlay(str(tmp_path), str(backend))
    args = ["--width", "6", "--height", "6", "--episodes", "120", "--max-steps", "100", "--eval-episodes", "2", "--save-agent"]
    rc, out = ref_drivers.run(["run_training.py"] + args, ov, env)
    _check_training_run(rc, out, str(tmp_path), 120)
    rc, out = ref_drivers.run([os.path.join("src", "train.py")] + args, ov, env)           # src/train.py imports cudarl_core by itself
    _check_training_run(rc, out, str(tmp_path), 120)


@pytest.mark.gpu
@needs_ref
def test_reference_drivers_on_the_native_module(tmp_path):
    ov, env = ref_drivers.make_overlay(str(tmp_path), os.path.join(ROOT, "cudarl-arena_b200"))
    args = ["--width", "6", "--height", "6", "--episodes", "120", "--max-steps", "100", "--eval-episodes", "2", "--save-agent"]
    rc, out = ref_drivers.run(["run_training.py"] + args, ov, env)
    _check_training_run(rc, out, str(tmp_path), 120)
    rc, out = ref_drivers.run([os.path.join("src", "train.py")] + args, ov, env)
    _check_training_run(rc, out, str(tmp_path), 120)


@pytest.mark.gpu
def test_shim_is_the_native_environment():
    """What run_training.py:13-14 does with the shim, then the loop of src/train.py:191-222 on it."""
    sys.path.insert(0, ROOT)
    sys.modules.pop("cudarl_core", None)
    import python.cudarl.mock_env as mock_env
    sys.modules["cudarl_core"] = mock_env
    import cudarl_core
    env = cudarl_core.Environment(6, 6)
    assert type(env).__module__ == "cudarl_core" and type(env).__name__ == "Environment"
    rng = np.random.RandomState(0)
    q = np.zeros((6, 6, 4))
    eps, lengths = 1.0, []
    for episode in range(60):
        obs = env.reset()
        pos = env.get_agent_position()
        for step in range(200):
            a = rng.randint(0, 4) if rng.rand() < eps else np.argmax(q[pos[0], pos[1]])
            nobs, r, done, info = env.step(a)
            npos = env.get_agent_position()
            q[pos[0], pos[1], a] += 0.1 * (r + 0.99 * (0 if done else np.max(q[npos[0], npos[1]])) - q[pos[0], pos[1], a])
            eps *= 0.995
            pos = npos
            if done:
                break
        lengths.append(step + 1)
    assert len(obs) == 36 and np.mean(lengths[-10:]) < np.mean(lengths[:10])
    del sys.modules["cudarl_core"]
