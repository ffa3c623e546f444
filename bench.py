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
             (k_tile_step, CUDA events around every launch), against the measured HBM copy bandwidth of
             MEASURED_PEAKS.json,
  cpu_baseline  the CPU oracle (a C++ port of the same semantics) timed on this box's cores.

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
FALLBACK_HBM_GBS = 6650.0
TRAFFIC_C5 = 655.5e6      # dram__bytes_read.sum + dram__bytes_write.sum of one k_tile_step launch on C5 (profiles/k_tile_step_C5.md)


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
    o.train_steps(1)                       # touch memory once
    t0 = time.perf_counter()
    o.train_steps(nsteps)
    dt = time.perf_counter() - t0
    n = int(cfg.num_envs)
    o.close()
    return n * nsteps / dt, dt


def run_reference(args):
    """The reference arm: the CPU port of the path on all host threads; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    pkg = load_pkg()
    threads = os.cpu_count() or 1
    cfg = pkg.preset(args.config)
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
    sample = "%d batched step(s) of %s (%d envs) per bench step, %d threads" % (per, args.config, n, threads)
    print(json.dumps({
        "impl": "reference", "metric": "env-steps/s (step+eps-greedy+TD update)", "value": value, "unit": "env-steps/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.config, cfg), "window": per},
        "cpu_baseline": {"value": value, "unit": "env-steps/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "env-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_name(name, cfg):
    return "%s: %dx%d grid, %d envs/GPU, fused step+eps-greedy+TD update" % (name, cfg.width, cfg.height, cfg.num_envs)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="C5")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--window", type=int, default=0, help="fused steps per bench step (default: averaging period, else 256)")
    ap.add_argument("--envs", type=int, default=0, help="override environments per GPU")
    ap.add_argument("--cpu-steps", type=int, default=4, help="oracle steps timed for cpu_baseline (0 = skip)")
    ap.add_argument("--cpu-steps-per-sample", type=int, default=1)
    ap.add_argument("--profile-steps", type=int, default=0, help="run only this many fused steps and exit (for ncu)")
    args = ap.parse_args()
    if args.impl == "ours":
        args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)

    pkg = load_pkg()
    dist, rank, world = dist_setup(args.gpus)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = pkg.preset(args.config, num_envs=args.envs or None, device=local)
    n_local = int(cfg.num_envs)
    cfg.env_offset = rank * n_local
    window = args.window or (cfg.sync_every if cfg.sync_every > 0 else 256)
    env = pkg.VecGridWorld(cfg)
    launches_per_step = 1      # k_tile_step (+ 5 kernels that re-size the tile regions every 128th step)

    if args.profile_steps:                      # small fixed run for profilers: no timing, no JSON
        env.train_steps(args.profile_steps)
        env.synchronize()
        print("ran %d fused steps" % args.profile_steps)
        return

    if world > 1:
        ids = [pkg.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        env.comm_init(ids[0], rank, world)
        launches_per_step_window_extra = (cfg.width * cfg.height + (1 << 20) - 1) >> 20     # one averaging kernel per all-gather round of 2^20 cells
    else:
        launches_per_step_window_extra = 0

    # ---- device-resident arm -------------------------------------------------------------------
    for _ in range(args.warmup):
        env.train_steps(window)
    env.synchronize(); barrier(dist)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    env.timer_start()
    for _ in range(args.steps):
        env.train_steps(window)
    ms = env.timer_stop_ms()
    env.synchronize(); barrier(dist)
    clocks = sampler.stop() if rank == 0 else None
    ms = reduce_max(dist, ms)
    total_env_steps = float(n_local) * world * window * args.steps
    value = total_env_steps / (ms * 1e-3)

    # ---- end-to-end arm: host-facing call, per-window host epsilon array in, statistics out -------
    import numpy as np
    eps_host = np.full(window, float(cfg.eps0), np.float32)
    for _ in range(2):
        env.train_steps_eps(eps_host); env.get_stats()
    env.synchronize(); barrier(dist)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        env.train_steps_eps(eps_host)
        st = env.get_stats()                     # synchronising device->host read of the result
    e2e_s = time.perf_counter() - t0
    barrier(dist)
    e2e_s = reduce_max(dist, e2e_s)
    e2e_value = total_env_steps / e2e_s

    # ---- roofline of the dominant kernel: mean main-kernel duration from events around each launch -
    env.kernel_timing(True)
    env.train_steps(min(window, 128))
    main_ms, nl = env.kernel_time_ms(); fix_ms = 0.0
    env.kernel_timing(False)
    peak, peak_kind = hbm_peak()
    main_avg_s = main_ms * 1e-3 / max(nl, 1)
    fix_avg_s = fix_ms * 1e-3 / max(nl, 1)
    achieved = ALGO_BYTES_TRAIN * n_local / main_avg_s / 1e9
    stats = env.get_stats()
    assert stats.device_error == 0, "device error flag set: %d" % stats.device_error

    if rank != 0:
        return
    cpu = None
    if args.cpu_steps > 0:
        threads = os.cpu_count() or 1
        v, dt = cpu_sample(pkg, args.config, args.cpu_steps, threads, num_envs=args.envs or None)
        cpu = {"value": v, "unit": "env-steps/s", "cores": threads, "kind": "port",
               "sample": "%d batched steps of the full %s workload (%d envs) on the CPU oracle, %.1f s" % (args.cpu_steps, args.config, n_local, dt)}
    line = {
        "metric": "env-steps/s (step+eps-greedy+TD update)", "value": value, "unit": "env-steps/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.config, cfg), "window": window, "l2": "inputs_exceed_l2" if cfg.width * cfg.height * 32 > 126e6 else "l2_resident",   # two dense tables of 16 B per cell
                   "parallelism": "env-sharded x%d, Q replica per GPU, NCCL average every %d steps" % (world, cfg.sync_every)},
        "e2e": {"value": e2e_value, "unit": "env-steps/s", "h2d_bytes_per_step": int(window * 4), "d2h_bytes_per_step": 128},
        "gpu_launches": int(args.steps * (window * launches_per_step + (window // 128) * 5 + launches_per_step_window_extra)),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one k_tile_step launch on this workload, from the ncu
                     # capture summarised in profiles/k_tile_step_C5.md (not measured by this run)
                     "traffic": TRAFFIC_C5 if (args.config == "C5" and not args.envs) else None,
                     "peak_kind": peak_kind, "kernel": "k_tile_step", "algorithmic_bytes_per_env_step": ALGO_BYTES_TRAIN,
                     "main_kernel_us": main_avg_s * 1e6, "other_kernels_us": fix_avg_s * 1e6,
                     "whole_step_frac": ALGO_BYTES_TRAIN * n_local / (ms * 1e-3 / (args.steps * window)) / 1e9 / peak},
        "cpu_baseline": cpu,
        "run_stats": {"steps": stats.steps, "goals": stats.goals, "timeouts": stats.timeouts,
                      "conflict_fraction": stats.conflicts / max(stats.env_steps, 1), "chained_fraction": stats.chained / max(stats.env_steps, 1),
                      "long_chains": stats.long_chains},
    }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
