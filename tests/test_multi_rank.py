"""The N>1 path: environment shards with global offsets, one table replica per rank, averaged every K steps.
CPU test with two gloo ranks (runs anywhere); GPU test with one process per GPU over NCCL (needs >= 2 GPUs)."""
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_ranks(n, mode, extra=()):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n),
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(HERE, "multi_rank_worker.py"), "--mode", mode] + list(extra)
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:]
    assert "multi-rank %s ok" % mode in r.stdout, r.stdout[-3000:]


def test_two_cpu_ranks_gloo():
    run_ranks(2, "cpu", ["--steps", "16", "--k", "4", "--envs", "512"])


def gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, timeout=30).stdout
        return sum(1 for l in out.splitlines() if l.startswith("GPU "))
    except Exception:
        return 0


@pytest.mark.gpu
def test_gpu_ranks_nccl():
    n = gpu_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    run_ranks(2, "gpu", ["--steps", "24", "--k", "4", "--envs", "4096"])
    # both forms of the averaging: slices by NCCL send / receive, and read straight out of the peers' IPC-mapped tables
    run_ranks(2, "gpu", ["--steps", "12", "--k", "4", "--envs", "4096", "--avg", "nccl"])
    run_ranks(2, "gpu", ["--steps", "12", "--k", "4", "--envs", "4096", "--avg", "peer"])
    run_ranks(2, "gpu", ["--steps", "12", "--k", "4", "--envs", "8192", "--width", "1001", "--height", "999", "--avg", "nccl"])
    # 999,999 cells: the table does not split into equal slices, the last slice of the averaging runs into the table's padding
    run_ranks(2, "gpu", ["--steps", "12", "--k", "4", "--envs", "8192", "--width", "1001", "--height", "999"])
    if n >= 4:
        run_ranks(4, "gpu", ["--steps", "16", "--k", "4", "--envs", "2048"])
        run_ranks(3, "gpu", ["--steps", "8", "--k", "4", "--envs", "4096", "--width", "1001", "--height", "999"])
