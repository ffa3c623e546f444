"""`python.cudarl.mock_env` backed by the native module.

The reference ships a stand-in of this name whose `Environment` only prints (python/cudarl/mock_env.py:1-16) and
`run_training.py:13-14` installs it as `cudarl_core`.  This file has the same import path and exposes the same class
name with the same constructor (`Environment(width=10, height=10)`) and methods (`reset()`, `step(action)`,
`get_agent_position()`), but the class is the native `cudarl_core.Environment` of libcudarl.so: every step runs on the
GPU.  There is no fallback: if the native module is not built the import fails.

The module is looked up on `sys.path` first (a user who put `cudarl-arena_b200/` on PYTHONPATH), then beside this file
in the layout of this repository (`<root>/python/cudarl/mock_env.py` -> `<root>/cudarl-arena_b200/`), or in the directory
named by the environment variable CUDARL_B200_DIR.
"""
import importlib
import os
import sys


def _native():
    here = os.path.dirname(os.path.abspath(__file__))
    extra = [os.environ.get("CUDARL_B200_DIR"), os.path.join(os.path.dirname(os.path.dirname(here)), "cudarl-arena_b200")]
    mod = sys.modules.get("cudarl_core")
    if mod is not None and hasattr(mod, "Environment") and getattr(mod, "__name__", "") != __name__:
        return mod
    try:
        return importlib.import_module("cudarl_core")
    except ImportError:
        for d in extra:
            if d and os.path.isdir(d) and d not in sys.path:
                sys.path.insert(0, d)
        return importlib.import_module("cudarl_core")


_core = _native()
Environment = _core.Environment
__version__ = getattr(_core, "__version__", "0.1.0")
for _name in ("CudaQLearning", "VecEnvironment"):      # the additions of the native module, for scripts that want them
    if hasattr(_core, _name):
        globals()[_name] = getattr(_core, _name)
