#!/usr/bin/env python3
"""Generate tests/golden/*.npz from the reference's OWN Python CPU code.

Run where a checkout of the reference project exists (CUDARL_REFERENCE=<path> selects it):

    python tests/golden/make_golden.py

It imports, unmodified, `MockEnvironment` from the reference's src/gui.py (its CPU restatement of
the CUDA step/reset kernels) and `QTableAgent` from src/train.py (the TD update, epsilon-greedy and
epsilon decay that actually train in the reference), drives them with seeded inputs and stores
inputs and outputs.  matplotlib is not installed here and both files import it at top level, so an
empty stand-in module is put in sys.modules first; src/train.py also insists on importing
`cudarl_core`, for which a dummy module is registered.  Nothing of the reference is copied: only
the numbers its code produces are saved.
"""
import os
import sys
import tempfile
import types

import numpy as np

REF = os.environ.get("CUDARL_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference")
OUT = os.path.dirname(os.path.abspath(__file__))


def _stub(name):
    m = types.ModuleType(name)
    m.__path__ = []
    sys.modules[name] = m
    return m


def import_reference():
    for n in ("matplotlib", "matplotlib.pyplot", "matplotlib.animation", "matplotlib.gridspec", "matplotlib.widgets"):
        _stub(n)
    sys.modules["matplotlib.animation"].FuncAnimation = object
    sys.modules["matplotlib.widgets"].Button = object
    sys.modules["matplotlib.widgets"].Slider = object
    sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
    _stub("cudarl_core").Environment = None   # src/train.py exits at import without the module; never called here
    sys.path.insert(0, REF)
    cwd = os.getcwd()
    os.chdir(tempfile.mkdtemp())  # src/train.py opens ./training.log when imported
    try:
        import src.gui as gui
        import src.train as train
    finally:
        os.chdir(cwd)
    return gui, train


def env_vectors(gui):
    """Random action walks through MockEnvironment (src/gui.py:84-137)."""
    rng = np.random.RandomState(1234)
    out = {}
    for k, (w, h, steps) in enumerate([(10, 10, 400), (5, 5, 200), (3, 3, 100), (7, 4, 300), (1, 1, 10), (2, 9, 120)]):
        env = gui.MockEnvironment(w, h)
        env.reset()
        start = env.get_agent_position()
        actions = rng.randint(-1, 6, size=steps).astype(np.int32)   # includes invalid actions -1, 4, 5
        xs, ys, rs, ds = [], [], [], []
        for a in actions:
            _, r, d, _ = env.step(int(a))
            x, y = env.get_agent_position()
            xs.append(x); ys.append(y); rs.append(r); ds.append(d)
        out["env%d_wh" % k] = np.array([w, h], np.int32)
        out["env%d_start" % k] = np.array(start, np.int32)
        out["env%d_actions" % k] = actions
        out["env%d_x" % k] = np.array(xs, np.int32)
        out["env%d_y" % k] = np.array(ys, np.int32)
        out["env%d_reward" % k] = np.array(rs, np.float64)
        out["env%d_done" % k] = np.array(ds, np.uint8)
    return out


def td_vectors(train):
    """Sequential QTableAgent.update calls (src/train.py:110-148) on random transitions."""
    rng = np.random.RandomState(4321)
    out = {}
    for k, (w, h, n, lr, gamma) in enumerate([(6, 5, 600, 0.1, 0.99), (10, 10, 1500, 0.05, 0.995), (3, 3, 300, 0.5, 0.9)]):
        ag = train.QTableAgent(w, h, 4, learning_rate=lr, discount_factor=gamma, exploration_rate=1.0, exploration_decay=0.995)
        ag.q_table = rng.uniform(-0.5, 1.0, size=(w, h, 4))
        q0 = ag.q_table.copy()
        sx, sy = rng.randint(0, w, n), rng.randint(0, h, n)
        nx, ny = rng.randint(0, w, n), rng.randint(0, h, n)
        a = rng.randint(0, 4, n)
        r = np.where(rng.rand(n) < 0.1, 1.0, -0.01)
        dn = (rng.rand(n) < 0.15)
        eps, tdq, tdt = [], [], []
        for i in range(n):
            m = ag.update(None, int(a[i]), float(r[i]), None, bool(dn[i]), (int(sx[i]), int(sy[i])), (int(nx[i]), int(ny[i])))
            eps.append(m["exploration_rate"]); tdq.append(m["q_value"]); tdt.append(m["target"])
        out["td%d_dims" % k] = np.array([w, h], np.int32)
        out["td%d_hyper" % k] = np.array([lr, gamma], np.float64)
        out["td%d_q0" % k] = q0                       # (W,H,A) float64, indexed [x,y,a]
        out["td%d_q1" % k] = ag.q_table.copy()
        for nm, v in (("sx", sx), ("sy", sy), ("nx", nx), ("ny", ny), ("a", a)):
            out["td%d_%s" % (k, nm)] = v.astype(np.int32)
        out["td%d_r" % k] = r.astype(np.float64)
        out["td%d_done" % k] = dn.astype(np.uint8)
        out["td%d_eps" % k] = np.array(eps, np.float64)      # epsilon after each update (src/train.py:141)
        out["td%d_qvalue" % k] = np.array(tdq, np.float64)
        out["td%d_target" % k] = np.array(tdt, np.float64)
    return out


def greedy_vectors(train):
    """select_action(training=False) = np.argmax over the row (src/train.py:108), with ties."""
    rng = np.random.RandomState(99)
    w, h = 8, 6
    ag = train.QTableAgent(w, h, 4)
    q = rng.randint(-2, 3, size=(w, h, 4)).astype(np.float64) * 0.25     # many exact ties
    ag.q_table = q
    acts = np.zeros((w, h), np.int32)
    for x in range(w):
        for y in range(h):
            acts[x, y] = ag.select_action(None, (x, y), training=False)
    return {"greedy_q": q, "greedy_action": acts}


def main():
    gui, train = import_reference()
    np.savez_compressed(os.path.join(OUT, "reference_env.npz"), **env_vectors(gui))
    np.savez_compressed(os.path.join(OUT, "reference_td.npz"), **td_vectors(train))
    np.savez_compressed(os.path.join(OUT, "reference_greedy.npz"), **greedy_vectors(train))
    print("wrote", [f for f in os.listdir(OUT) if f.endswith(".npz")])


if __name__ == "__main__":
    main()
