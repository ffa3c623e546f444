"""Drop-in files for a checkout of CudaRL-Arena.

Only `mock_env.py` matters: the reference's `run_training.py:13-14` imports `python.cudarl.mock_env` and installs it
as the module `cudarl_core`.  Copied over the reference's `python/cudarl/mock_env.py`, the file here makes that script
(and `src/train.py`, which it calls) drive the native B200 module instead of the print-only stand-in.  This package
file is deliberately empty: the reference's own `python/cudarl/__init__.py` pulls in its matplotlib trainer, which
`run_training.py` does not need.
"""
