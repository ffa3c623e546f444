"""Helpers to run the reference's own driver scripts, unmodified, against this repository's drop-in files.

The reference checkout (CUDARL_REFERENCE, default: a checkout beside this repository's parent named `reference`) is
only read: an overlay directory is built out of symbolic links to its `run_training.py` and `src/`, plus THIS
repository's `python/cudarl/` (the shim that run_training.py installs as `cudarl_core`).  matplotlib is not installed
in the test image and `src/train.py` imports it at top level, so a stand-in package is put on PYTHONPATH.
"""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_root():
    cand = os.environ.get("CUDARL_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    return cand if os.path.isfile(os.path.join(cand, "run_training.py")) and os.path.isfile(os.path.join(cand, "src", "train.py")) else None


def make_overlay(tmp, backend_dir):
    """tmp/: run_training.py and src -> the reference's; python/cudarl -> this repository's shim; stubs/ for matplotlib.
    Returns (overlay directory, environment for the subprocess)."""
    ref = reference_root()
    ov = os.path.join(tmp, "overlay")
    os.makedirs(os.path.join(ov, "python"))
    os.symlink(os.path.join(ref, "run_training.py"), os.path.join(ov, "run_training.py"))
    os.symlink(os.path.join(ref, "src"), os.path.join(ov, "src"))
    os.symlink(os.path.join(ROOT, "python", "cudarl"), os.path.join(ov, "python", "cudarl"))
    stubs = os.path.join(tmp, "stubs", "matplotlib")
    os.makedirs(stubs)
    open(os.path.join(stubs, "__init__.py"), "w").write("")
    open(os.path.join(stubs, "pyplot.py"), "w").write(
        "def __getattr__(name):\n    raise RuntimeError('matplotlib stand-in: plotting is not available in this test')\n")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([os.path.dirname(stubs), backend_dir] + ([env["PYTHONPATH"]] if env.get("PYTHONPATH") else []))
    env["CUDARL_B200_DIR"] = backend_dir
    return ov, env


def run(cmd, cwd, env, timeout=600):
    r = subprocess.run([sys.executable] + cmd, cwd=cwd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout)
    return r.returncode, r.stdout


def average_lengths(log):
    """The 'Avg Length' column of the progress lines of src/train.py:240-250."""
    out = []
    for line in log.splitlines():
        if "Avg Length:" in line:
            out.append(float(line.split("Avg Length:")[1].split("|")[0]))
    return out
