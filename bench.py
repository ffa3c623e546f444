#!/usr/bin/env python3
"""Benchmark of the fused batched step (grid-world step + epsilon-greedy + TD update + auto-reset).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C5] [--impl ours|reference]

Metric: env-steps/s.  One bench "step" is a window of `window` fused batched steps over all
environments of the shard (window = the configuration's replica-averaging period, 256 for C5), so at
N > 1 every bench step contains exactly one NCCL average of the Q replicas.  Weak scaling: every GPU
holds the configuration's environments (4,194,304 for C5) and its own Q replica.

The line printed by rank 0 carries
  value      whole-job env-steps/s with everything resident in HBM (device events, max over ranks),
  e2e        the same through the host-facing call: every window uploads its epsilon schedule from host
             memory and reads the run statistics back,
  roofline   algorithmic bytes (60 B per env-step) x envs per launch / mean duration of the step kernel
             (k_tile_step; one CUDA event pair around every uninterrupted run of launches), against the
             measured HBM copy bandwidth of MEASURED_PEAKS.json,
  eval       the greedy rollout of all environments that follows training in the workload (k_eval),
  cpu_baseline  the CPU oracle (a C++ port of the same semantics) timed on this box's cores,
  cpu_baseline_reference_python  the reference's own Python loop at its default configuration, where its
             checkout is present,
  multi_gpu_parity / replica_digests_equal  at N > 1: a small sharded run checked bit for bit against the
             rank-ordered oracle replay before timing, and the replicas' tables compared after it.

`--impl reference` times that CPU port with all host threads instead (the reference project itself
only has one-thread-per-environment GPU kernels and a Python loop for this path).
"""
import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.join(ROOT, "cudarl-arena_b200")
ALGO_BYTES_TRAIN = 60      # 12 state in + 12 state out + 16 Q[s] row + 16 Q[s'] row + 4 Q[s,a] write
ALGO_BYTES_EVAL = 40       # greedy rollout step: 24 state + 16 Q[s] row
FALLBACK_HBM_GBS = 6650.0
TRAFFIC_C5 = 455.5e6      # dram__bytes_read.sum + dram__bytes_write.sum of one k_tile_step launch on C5 (one ncu capture of one launch)


def load_pkg():
    name = "cudarl_arena_b200"
    if name not in sys.modules:
        spec = importlib.util.spec_from_file_location(name, os.path.join(PKG_DIR, "__init__.py"),
                                                      submodule_search_locations=[PKG_DIR])
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return sys.modules[name]


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.proc, self.path = device, None, "/tmp/cudarl_clocks_%d.csv" % os.getpid()

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            p = [v.strip() for v in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def dist_setup(n):
    """torch.distributed (gloo) only as plumbing: rendezvous, barrier, max over ranks, id broadcast."""
    if n <= 1 and "RANK" not in os.environ:
        return None, 0, 1
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", str(n)))
    dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    return dist, rank, world


def reduce_max(dist, v):
    if dist is None:
        return v
    import torch
    t = torch.tensor([v], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def barrier(dist):
    if dist is not None:
        dist.barrier()


def cpu_sample(pkg, cfg_name, nsteps, threads, num_envs=None):
    """Time `nsteps` batched steps of the CPU oracle on the full-size workload."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    cfg = pkg.preset(cfg_name, num_envs=num_envs)
    o = oracle_lib.Oracle(cfg, threads=threads)
    o.count_conflicts(False)
    o.train_steps(1)                       # touch memory once, start the worker threads
    t0 = time.perf_counter()
    o.train_steps(nsteps)
    dt = time.perf_counter() - t0
    n = int(cfg.num_envs)
    o.close()
    return n * nsteps / dt, dt


def reference_python_sample(episodes=300, max_steps=500):
    """BASELINE configuration C1 on the reference's OWN CPU path: train() of src/train.py:171-259 driving MockEnvironment of
    src/gui.py:84-137 with QTableAgent, one core (the Python interpreter).  Needs a checkout of the reference beside this
    repository (or CUDARL_REFERENCE); its files are imported where they lie, never copied.  Returns None where it is absent."""
    ref = os.environ.get("CUDARL_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isfile(os.path.join(ref, "src", "train.py")):
        return {"unavailable": "no checkout of the reference project on this machine (its Python files are never copied; "
                               "measured where the checkout exists: 42-49 k env-steps/s on one 2.7 GHz Xeon core)"}
    code = r"""
import sys, os, types, time, tempfile, logging
for n in ("matplotlib", "matplotlib.pyplot", "matplotlib.animation", "matplotlib.gridspec", "matplotlib.widgets"):
    m = types.ModuleType(n); m.__path__ = []; sys.modules[n] = m
sys.modules["matplotlib.animation"].FuncAnimation = object
sys.modules["matplotlib.widgets"].Button = object; sys.modules["matplotlib.widgets"].Slider = object
sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
core = types.ModuleType("cudarl_core"); core.Environment = None; sys.modules["cudarl_core"] = core
sys.path.insert(0, %r); os.chdir(tempfile.mkdtemp())
import src.gui as gui, src.train as train
logging.disable(logging.CRITICAL)
env = gui.MockEnvironment(10, 10)
agent = train.QTableAgent(10, 10)
t0 = time.perf_counter()
m = train.train(env, agent, num_episodes=%d, max_steps=%d)
dt = time.perf_counter() - t0
print("RESULT", sum(m["lengths"]), dt)
""" % (ref, episodes, max_steps)
    try:
        r = subprocess.run([sys.executable, "-c", code], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, timeout=300)
        steps, dt = [l for l in r.stdout.splitlines() if l.startswith("RESULT")][0].split()[1:]
        return {"value": float(steps) / float(dt), "unit": "env-steps/s", "cores": 1, "kind": "reference_python",
                "sample": "C1 (10x10, one environment): %d episodes x <= %d steps = %d steps of the reference's train() + MockEnvironment + QTableAgent, %.1f s"
                          % (episodes, max_steps, int(float(steps)), float(dt))}
    except Exception as e:           # noqa: BLE001
        return {"unavailable": "running the reference's Python path failed: %r" % (e,)}


METRIC = "env-steps/s (step+eps-greedy+TD update)"


def bench_config(name, cfg, window, world):
    return {"workload": workload_name(name, cfg), "window": window,
            "l2": "inputs_exceed_l2" if cfg.width * cfg.height * 16 > 126e6 else "l2_resident",     # the table: 16 B per cell
            "parallelism": "env-sharded x%d, Q replica per GPU, replicas averaged every %d steps" % (world, cfg.sync_every)}


def run_reference(args):
    """The reference arm: the CPU port of the path (persistent worker threads, all host threads) on the same workload;
    rank 0 only.  One bench step times `--cpu-steps-per-sample` of the window's batched steps (a bounded sample)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    pkg = load_pkg()
    threads = os.cpu_count() or 1
    cfg = pkg.preset(args.config, num_envs=args.envs or None)
    window = args.window or (cfg.sync_every if cfg.sync_every > 0 else 256)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    o = oracle_lib.Oracle(cfg, threads=threads)
    o.count_conflicts(False)
    per = args.cpu_steps_per_sample
    for _ in range(args.warmup):
        o.train_steps(per)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        o.train_steps(per)
    dt = time.perf_counter() - t0
    n = int(cfg.num_envs)
    value = n * per * args.steps / dt
    sample = ("each bench step times %d of the %d batched steps of a window of %s (%d environments; at N GPUs the job is N such shards, "
              "which a CPU steps one after the other at this same rate), %d threads" % (per, window, args.config, n, threads))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "env-steps/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.config, cfg, window, max(args.gpus, 1)),
        "cpu_baseline": {"value": value, "unit": "env-steps/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "env-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_name(name, cfg):
    return "%s: %dx%d grid, %d envs/GPU, fused step+eps-greedy+TD update" % (name, cfg.width, cfg.height, cfg.num_envs)


def table_digest(q):
    """Two 64-bit numbers of the table's bits: xor and wrapping sum of its 8-byte words."""
    import numpy as np
    w = np.ascontiguousarray(q).view(np.uint64)
    return int(np.bitwise_xor.reduce(w)), int(np.add.reduce(w, dtype=np.uint64))


def multi_gpu_parity(pkg, dist, rank, world, local):
    """Before anything is timed at N > 1: every rank trains a small shard (C2: 64x64, 4096 environments per rank) for 24 steps
    with the replicas averaged every 4, and replays ALL shards on the CPU oracle with the sum taken in rank order.  State and
    table of the own shard must match bit for bit.  The oracle is the checker here, nothing of it is timed."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    n = 4096
    def shard(r, device):
        c = pkg.preset("C2", num_envs=n, device=device)
        c.env_offset, c.sync_every = r * n, 4
        return c
    env = pkg.VecGridWorld(shard(rank, local))
    ids = [pkg.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    env.comm_init(ids[0], rank, world)
    env.train_steps(24)
    cpus = [oracle_lib.Oracle(shard(r, 0)) for r in range(world)]
    for _ in range(6):
        for o in cpus:
            o.train_steps(4)
        oracle_lib.average_replicas(cpus)
    ok = bool(np.array_equal(env.get_q(), cpus[rank].get_q()) and all(np.array_equal(a, b) for a, b in zip(env.get_state(), cpus[rank].get_state())))
    env.close()
    for o in cpus:
        o.close()
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    return all(flags)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="C5")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--window", type=int, default=0, help="fused steps per bench step (default: averaging period, else 256)")
    ap.add_argument("--envs", type=int, default=0, help="override environments per GPU")
    ap.add_argument("--tile-edge", type=int, default=0, help="tile edge of the step kernel, 8 or 16 (0 = chosen from the density)")
    ap.add_argument("--cpu-steps", type=int, default=24, help="oracle steps timed for cpu_baseline (0 = skip)")
    ap.add_argument("--cpu-steps-per-sample", type=int, default=1)
    ap.add_argument("--eval-steps", type=int, default=1000, help="step cap of the greedy evaluation rollout (0 = skip); 1000 as in src/train.py:282 of the reference")
    ap.add_argument("--profile-steps", type=int, default=0, help="run only this many fused steps and exit (for ncu)")
    ap.add_argument("--profile-eval", type=int, default=0, help="with --profile-steps: then one greedy rollout with this step cap")
    ap.add_argument("--profile-aux", type=int, default=0, help="with --profile-steps: then one caller-driven step of all environments and one update_batch of this many transitions")
    args = ap.parse_args()
    if args.impl == "ours":
        args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)

    import numpy as np
    pkg = load_pkg()
    dist, rank, world = dist_setup(args.gpus)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = pkg.preset(args.config, num_envs=args.envs or None, device=local)
    n_local = int(cfg.num_envs)
    cfg.env_offset = rank * n_local
    cfg.tile_edge = args.tile_edge
    window = args.window or (cfg.sync_every if cfg.sync_every > 0 else 256)

    if args.profile_steps:                      # small fixed run for profilers: no timing, no JSON
        env = pkg.VecGridWorld(cfg)
        env.train_steps(args.profile_steps)
        env.synchronize()
        if args.profile_eval:
            env.eval_rollout(args.profile_eval)
        if args.profile_aux:                    # the caller-driven step and the ordered update_batch, once each at this size
            rng = np.random.RandomState(1)
            env.step_actions(rng.randint(0, 4, n_local).astype(np.int32))
            nb = args.profile_aux
            sx, sy = rng.randint(0, cfg.width, nb).astype(np.int32), rng.randint(0, cfg.height, nb).astype(np.int32)
            env.update_batch(sx, sy, rng.randint(0, 4, nb), np.full(nb, -0.01, np.float32), np.clip(sx + 1, 0, cfg.width - 1), sy, np.zeros(nb, np.uint8))
        print("ran %d fused steps" % args.profile_steps)
        return

    parity = None
    if world > 1:
        parity = multi_gpu_parity(pkg, dist, rank, world, local)
        if not parity:
            raise SystemExit("multi-GPU parity check failed: a rank's shard differs from the rank-ordered oracle replay")
    env = pkg.VecGridWorld(cfg)
    if world > 1:
        ids = [pkg.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        env.comm_init(ids[0], rank, world)

    # ---- device-resident arm -------------------------------------------------------------------
    for _ in range(args.warmup):
        env.train_steps(window)
    env.synchronize(); barrier(dist)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    env.kernel_timing(True)       # one event pair around every uninterrupted run of step-kernel launches of the SAME timed windows
    env.timer_start()
    for _ in range(args.steps):
        env.train_steps(window)
    ms = env.timer_stop_ms()
    env.synchronize(); barrier(dist)
    step_ms, nl = env.kernel_time_ms()
    env.kernel_timing(False)
    clocks = sampler.stop() if rank == 0 else None
    ms = reduce_max(dist, ms)
    total_env_steps = float(n_local) * world * window * args.steps
    value = total_env_steps / (ms * 1e-3)

    # every window ends with an average: all replicas must now hold the same bits
    digests_equal = None
    if world > 1:
        d = [None] * world
        dist.all_gather_object(d, table_digest(env.get_q()))
        digests_equal = all(x == d[0] for x in d)
        if not digests_equal:
            raise SystemExit("replicas differ after an averaging step: %r" % (d,))

    # ---- end-to-end arm: host-facing call, per-window host epsilon array in, statistics out -------
    eps_host = np.full(window, float(cfg.eps0), np.float32)
    for _ in range(2):
        env.train_steps_eps(eps_host); env.get_stats()
    env.synchronize(); barrier(dist)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        env.train_steps_eps(eps_host)
        env.get_stats()                          # synchronising device->host read of the result
    e2e_s = time.perf_counter() - t0
    barrier(dist)
    e2e_s = reduce_max(dist, e2e_s)
    e2e_value = total_env_steps / e2e_s

    # ---- roofline of the dominant kernel, from the event pairs recorded inside the timed windows above --------------------
    peak, peak_kind = hbm_peak()
    step_s = step_ms * 1e-3 / max(nl, 1)
    achieved = ALGO_BYTES_TRAIN * n_local / step_s / 1e9
    stats = env.get_stats()

    # ---- the greedy evaluation rollout of all environments that follows training in the workload ---------------------------
    ev = None
    if args.eval_steps > 0:
        env.eval_rollout(8)                       # warm-up
        env.synchronize(); barrier(dist)
        env.timer_start()
        es = env.eval_rollout(args.eval_steps)
        ev_ms = reduce_max(dist, env.timer_stop_ms())
        tot = [None] * world
        if dist is not None:
            dist.all_gather_object(tot, (int(es.total_steps), int(es.reached)))
        else:
            tot = [(int(es.total_steps), int(es.reached))]
        ev_steps, ev_reached = sum(t[0] for t in tot), sum(t[1] for t in tot)
        ev_rate = ev_steps / (ev_ms * 1e-3)
        ev = {"value": ev_rate, "unit": "env-steps/s", "ms": ev_ms, "step_cap": args.eval_steps, "env_steps": ev_steps,
              "reached_fraction": ev_reached / float(n_local * world),
              "roofline": {"bound": "hbm", "kernel": "k_eval_policy + k_eval", "algorithmic_bytes_per_env_step": ALGO_BYTES_EVAL,
                           "achieved": ALGO_BYTES_EVAL * ev_rate / world / 1e9, "peak": peak, "unit": "GB/s",
                           "frac": ALGO_BYTES_EVAL * ev_rate / world / 1e9 / peak, "peak_kind": peak_kind,
                           "note": "includes the host call and its synchronising read of the result; the rollout folds the table into a "
                                   "one-byte-per-cell policy map once (k_eval_policy) and then reads one byte per environment-step, so "
                                   "against the 40 B per env-step of a rollout that reads Q[s] every step frac can exceed 1"}}

    peer_mem = env.comm_peer_memory() if world > 1 else False
    rebucket = int(cfg.rebucket_every) if int(cfg.rebucket_every) > 0 else 256      # the library's default period
    if rank != 0:
        return
    cpu = None
    if args.cpu_steps > 0:
        threads = os.cpu_count() or 1
        v, dt = cpu_sample(pkg, args.config, args.cpu_steps, threads, num_envs=args.envs or None)
        cpu = {"value": v, "unit": "env-steps/s", "cores": threads, "kind": "port",
               "sample": "%d batched steps of the full %s workload (%d envs) on the CPU oracle, %.1f s" % (args.cpu_steps, args.config, n_local, dt)}
    averaging_kernels = 2 if world > 1 else 0          # per window: the ordered sum of the own slice, the border array rebuilt
    line = {
        "metric": METRIC, "value": value, "unit": "env-steps/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.config, cfg, window, world),
        "e2e": {"value": e2e_value, "unit": "env-steps/s", "h2d_bytes_per_step": int(window * 4), "d2h_bytes_per_step": 128},
        # k_tile_step once per fused step, 5 kernels that re-size the record regions every `rebucket`-th step, the averaging kernels
        "gpu_launches": int(args.steps * (window + (window // rebucket) * 5 + averaging_kernels)),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum of ONE k_tile_step launch on this workload, from an ncu capture
                     # of one launch (not measured by this run)
                     "traffic": TRAFFIC_C5 if (args.config == "C5" and not args.envs) else None,
                     "peak_kind": peak_kind, "kernel": "k_tile_step", "algorithmic_bytes_per_env_step": ALGO_BYTES_TRAIN,
                     "main_kernel_us": step_s * 1e6, "launches_timed": int(nl),
                     "whole_step_frac": ALGO_BYTES_TRAIN * n_local / (ms * 1e-3 / (args.steps * window)) / 1e9 / peak},
        "eval": ev,
        "cpu_baseline": cpu,
        "cpu_baseline_reference_python": reference_python_sample(),
        "averaging": (("peer memory: one kernel per rank reads its slice of every IPC-mapped replica, sums in rank order, stores into every table" if peer_mem else "NCCL send/receive, ordered sum, all-gather") if world > 1 else None),
        "multi_gpu_parity": None if parity is None else "ok",
        "replica_digests_equal": digests_equal,
        "run_stats": {"steps": stats.steps, "goals": stats.goals, "timeouts": stats.timeouts,
                      "conflict_fraction": stats.conflicts / max(stats.env_steps, 1), "chained_fraction": stats.chained / max(stats.env_steps, 1),
                      "long_chains": stats.long_chains},
    }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
