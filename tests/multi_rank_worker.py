"""One rank of the sharded run (launched by the tests with torch.distributed.run, 127.0.0.1).

  --mode cpu : each rank steps its shard with the CPU oracle and the replicas are averaged with a gloo
               all-reduce every K steps -- the host-side sharding logic (global env offsets, averaging cadence,
               id hand-over) without a GPU.
  --mode gpu : each rank owns one GPU, steps its shard with libcudarl.so and averages through NCCL inside
               cudarl_train_steps.
Either way every rank then replays ALL shards with in-process oracles (rank-ordered sum, times 1/R) and
checks that its own shard's state and the averaged table are identical.
"""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from conftest import load_package  # noqa: E402
import oracle_lib  # noqa: E402


SIZE = [0, 0]      # --width / --height: a grid other than the preset's 64x64


def shard_config(pkg, rank, n_local, k):
    cfg = pkg.preset("C2", num_envs=n_local)
    cfg.env_offset = rank * n_local
    cfg.sync_every = k
    if SIZE[0]:
        cfg.width, cfg.height = SIZE
    return cfg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="cpu")
    ap.add_argument("--steps", type=int, default=24)
    ap.add_argument("--k", type=int, default=4)
    ap.add_argument("--envs", type=int, default=1024)
    ap.add_argument("--width", type=int, default=0)
    ap.add_argument("--height", type=int, default=0)
    ap.add_argument("--avg", default="auto", help="gpu mode: 'nccl' forces the send / receive averaging, 'peer' demands the peer-memory one")
    a = ap.parse_args()
    SIZE[:] = [a.width, a.height]
    pkg = load_package()
    dist.init_process_group(backend="gloo")
    rank, world = dist.get_rank(), dist.get_world_size()

    if a.mode == "gpu":
        cfg = shard_config(pkg, rank, a.envs, a.k)
        cfg.device = int(os.environ.get("LOCAL_RANK", rank))
        cfg.avg_over_nccl = 1 if a.avg == "nccl" else 0
        env = pkg.VecGridWorld(cfg)
        ids = [pkg.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        env.comm_init(ids[0], rank, world)
        if a.avg == "nccl":
            assert not env.comm_peer_memory()
        elif a.avg == "peer":
            assert env.comm_peer_memory(), "the peers' tables could not be mapped"
        env.train_steps(a.steps)
        env.synchronize()
        mine_q, mine_state = env.get_q(), env.get_state()
    else:
        ids = [bytes(range(128)) if rank == 0 else None]       # stands in for the communicator id hand-over
        dist.broadcast_object_list(ids, src=0)
        assert ids[0] == bytes(range(128))
        o = oracle_lib.Oracle(shard_config(pkg, rank, a.envs, a.k))
        for s in range(1, a.steps + 1):
            o.train_steps(1)
            if s % a.k == 0:
                q = torch.from_numpy(o.get_q())
                dist.all_reduce(q, op=dist.ReduceOp.SUM)
                o.set_q(q.numpy() * np.float32(1.0 / world))
        mine_q, mine_state = o.get_q(), o.get_state()

    # replay all shards on this rank
    shards = [oracle_lib.Oracle(shard_config(pkg, r, a.envs, a.k)) for r in range(world)]
    for s in range(1, a.steps + 1):
        for sh in shards:
            sh.train_steps(1)
        if s % a.k == 0:
            oracle_lib.average_replicas(shards)
    want_q, want_state = shards[rank].get_q(), shards[rank].get_state()
    for u, v in zip(mine_state, want_state):
        assert np.array_equal(u, v), "rank %d: shard state differs" % rank
    if a.mode == "gpu" or world <= 2:      # the GPU path sums in rank order itself: bit-exact for any world size
        assert np.array_equal(mine_q, want_q), "rank %d: averaged table differs" % rank
    else:   # the gloo all-reduce of the CPU stand-in has no fixed order beyond two ranks
        np.testing.assert_allclose(mine_q, want_q, rtol=1e-5, atol=1e-7)
    dist.barrier()
    if rank == 0:
        print("multi-rank %s ok: world=%d steps=%d k=%d" % (a.mode, world, a.steps, a.k))


if __name__ == "__main__":
    main()
