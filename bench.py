#!/usr/bin/env python
"""Benchmark of the batch navigation step + rollout returns.

One bench "step" is one rollout window: T = 32 simulator steps over all N environments of this GPU
(action -> move/turn on the navmesh -> GPS/compass -> A* + funnel geodesic -> reward / done /
info -> on-device episode reset), each step's reward and mask stored into rollout-storage tensors,
followed by one fused GAE + advantage normalisation over the [T+1, N] window.  The metric is
environment steps per second = N * T * windows / time, whole job (all ranks).

Default workload: benchmark config 1 -- one 50x50 m synthetic floor plan with 60 box obstacles
(Recast single-tile build: 446 polygons), 4096 environments per GPU, i.i.d. uniform actions over
{stop, forward, left, right}.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c4]

Keys of the line printed by rank 0 (one JSON object):
  value          device-resident arm: actions already in HBM, results stay in HBM, CUDA-event timed
  e2e            the same metric through the reference-shaped host API: numpy actions in, numpy
                 reward / mask / info / polar out every step (host <-> device traffic inside the
                 timed region).  Measured twice -- one group, and the two groups of a
                 double-buffered generator stepped alternately as the reference's trainer drives
                 it -- and the faster one is reported (e2e.variants holds both)
  roofline       for the kernel with the largest share of step time
  cpu_baseline   the CPU oracle (the reference's compiled PathFinder driven by the simulator
                 restatement, all host cores) on a bounded sample of the same workload
  dense_scene    config 1 read with the polygon count its description quotes (16 407 polygons)
  large_batch    the headline window at 32768 environments per GPU
  c2             benchmark config 2: GAE at T = 32, N = 16384
  shard          benchmark config 3: a fixed global batch (16 scenes, 16384 environments) block-
                 partitioned over the ranks, each rank loading only the scenes of its block
  double_buffered  the headline window with the environments in two groups on two streams
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

T_ROLLOUT = 32
GAMMA, TAU = 0.99, 0.95
# algorithmic bytes (state columns read + written, outputs written) per unit of each launch
BYTES_PER_ENV_STEP = 177          # move + sensor + reward path, per environment step
BYTES_PER_GAE_ELEM = 25.2         # scan 17.2 + normalise 8 per (t, env)
L2_FLUSH_BYTES = 256 << 20
LARGE_BATCH_ENVS = 32768
DENSE_SCENE = "d0"
C2_T, C2_N = 32, 16384
C3_ENVS, C3_SCENES = 16384, [f"m{i:02d}" for i in range(16)]
# dram__bytes_read.sum + dram__bytes_write.sum of one k_step launch, from an ncu capture of this
# script's default workload (one kernel, three launches); other workloads report null
NCU_TRAFFIC_BYTES = {("c1", 4096, "uniform"): 0.95e6}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=["c1", "c4"],
                    help="c1: the headline (config 1); c4: full-box DD-PPO step harness")
    ap.add_argument("--envs", type=int, default=None, help="environments per GPU")
    ap.add_argument("--scene", default="c1")
    ap.add_argument("--mix", default="uniform", choices=["uniform", "policy"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-large-batch", action="store_true")
    ap.add_argument("--no-depth", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the c2 / shard / double-buffered blocks")
    args = ap.parse_args()
    if args.envs is None:
        args.envs = 32768 if args.workload == "c4" else 4096
    return args


def scene_polys(name):
    with open(scene_files(name)[0].replace(".navmesh", ".scene.json")) as fh:
        return int(json.load(fh)["num_polys"])


def workload_string(args):
    """The same words in both arms (the reference arm has no GPU to ask about the scene)."""
    names = args.scene.split(",")
    polys = [scene_polys(nm) for nm in names]
    what = (f"config1: scene {names[0]} ({polys[0]} polys)" if len(names) == 1 else
            f"{len(names)} scenes {args.scene} ({min(polys)}-{max(polys)} polys)")
    return (f"{what}, {args.envs} envs/GPU, one step = T={T_ROLLOUT} sim steps + GAE/normalise, "
            f"{args.mix} actions")


def scene_files(name):
    d = os.path.join(ROOT, "tests", "golden", "scenes")
    return os.path.join(d, f"{name}.navmesh"), os.path.join(d, f"{name}.episodes.npy")


def draw_actions(shape, mix, seed):
    rng = np.random.default_rng(seed)
    if mix == "uniform":
        return rng.integers(0, 4, size=shape, dtype=np.int64)
    u = rng.random(shape)
    a = np.full(shape, 3, np.int64)
    a[u < 0.8025] = 2
    a[u < 0.605] = 1
    a[u < 0.005] = 0
    return a


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a region runs: NVML from a
    thread every few milliseconds (reads only), or nvidia-smi when NVML is not importable."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NVML_REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                    0x4: "sw_power_cap"}

    def __init__(self, gpu):
        self.gpu = gpu
        self.proc = None
        self.thread = None
        self.stop_flag = False
        self.sm, self.mx, self.reasons = [], [], set()

    def _nvml_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.gpu < len(ids) and ids[self.gpu].isdigit():
                return int(ids[self.gpu])
        return self.gpu

    def _poll(self, nv, handle):
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                if reasons_fn is not None:
                    bits = int(reasons_fn(handle))
                    for bit, name in self.NVML_REASONS.items():
                        if bits & bit:
                            self.reasons.add(name)
            except Exception:  # noqa: BLE001 - sampling must never take the bench down
                break
            time.sleep(0.002)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            handle = nv.nvmlDeviceGetHandleByIndex(self._nvml_index())
            self.mx.append(float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM)))
            import threading
            self.thread = threading.Thread(target=self._poll, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            return {"sm_mhz": float(np.median(self.sm)) if self.sm else None,
                    "sm_min_mhz": float(np.min(self.sm)) if self.sm else None,
                    "sm_max_mhz": float(np.max(self.mx)) if self.mx else None,
                    "samples": len(self.sm), "reasons": sorted(self.reasons), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(np.max(mx)) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback 6.65 TB/s (MEASURED_PEAKS.json absent)"


# ------------------------------------------------------------------------------------ CPU arm

def cpu_arm(scene_names, n, mix, seconds=None, windows=None, warmup=0):
    """Times the CPU oracle on rollout windows of the bench workload (T steps over n
    environments + numpy GAE per window): `windows` windows after `warmup` untimed ones, or as
    many as fit into `seconds`.  Returns (env_steps_per_s, details)."""
    from oracle import pyoracle
    if not pyoracle.available():
        raise RuntimeError("oracle libraries missing (oracle/_ref, oracle/_build)")
    scene_list = [(scene_files(nm)[0], np.load(scene_files(nm)[1])) for nm in scene_names]
    cores = len(os.sched_getaffinity(0))
    sim = pyoracle.OracleSim(scene_list, n, seed=1, threads=cores)
    sim.reset()
    T = T_ROLLOUT
    rewards = np.zeros((T + 1, n), np.float32)
    masks = np.ones((T + 1, n), bool)
    values = np.random.default_rng(0).standard_normal((T + 1, n)).astype(np.float32)

    def window(k):
        acts = draw_actions((T, n), mix, 1000 + k)
        ta = time.perf_counter()
        for t in range(T):
            sim.step(acts[t])
            rewards[t] = sim.rewards
            masks[t + 1] = sim.masks != 0
        pyoracle.gae_reference(rewards, values, masks, values[T], GAMMA, TAU, normalize=True)
        return time.perf_counter() - ta

    sim.run(draw_actions((8, n), mix, 99))
    for k in range(warmup):
        window(k)
    busy, k = 0.0, 0
    while True:
        busy += window(warmup + k)
        k += 1
        if (windows is not None and k >= windows) or (windows is None and busy >= seconds):
            break
    sim.close()
    rate = k * T * n / busy
    return rate, {"cores": cores, "windows": k, "seconds": busy,
                  "sample": f"{k} windows of {T} steps x {n} envs on scene "
                            f"{','.join(scene_names)} ({mix} actions) + numpy GAE per window; "
                            "simulator control flow = oracle/oracle_sim.cpp restatement, every "
                            "navmesh query = the reference's compiled PathFinder "
                            "(oracle/_ref/libref_nav.so), one PathFinder replica per thread"}


def cpu_microbench(args, seconds=3.0):
    """One-core rate of the same CPU simulator and microseconds per navmesh query of the
    reference's compiled PathFinder (tryStep, findPath) on the bench scene's episodes."""
    from oracle import pyoracle
    nav, epf = scene_files(args.scene.split(",")[0])
    eps = np.load(epf)
    n = min(args.envs, 1024)
    sim = pyoracle.OracleSim([(nav, eps)], n, seed=1, threads=1)
    sim.reset()
    sim.run(draw_actions((4, n), args.mix, 99))
    steps, busy, k = 0, 0.0, 0
    while busy < seconds:
        acts = draw_actions((16, n), args.mix, 500 + k)
        ta = time.perf_counter()
        sim.run(acts)
        busy += time.perf_counter() - ta
        steps += 16
        k += 1
    sim.close()
    one_core = steps * n / busy
    nq = min(len(eps), 4000)
    start = np.ascontiguousarray(eps[:nq, 0:3], np.float32)   # record = start 3, rotation 4, goal 3
    goal = np.ascontiguousarray(eps[:nq, 7:10], np.float32)
    rn = pyoracle.RefNav(nav)
    s_pos, s_ref = rn.snap(start)
    g_pos, g_ref = rn.snap(goal)
    d = g_pos - s_pos
    d[:, 1] = 0
    d /= np.maximum(np.linalg.norm(d, axis=1, keepdims=True), 1e-6)
    end = (s_pos + 0.25 * d).astype(np.float32)
    rn.try_step(s_pos, s_ref, end)
    t0 = time.perf_counter()
    for _ in range(5):
        rn.try_step(s_pos, s_ref, end)
    us_try = 1e6 * (time.perf_counter() - t0) / (5 * nq)
    rn.geodesic(s_pos, s_ref, g_pos, g_ref)
    t0 = time.perf_counter()
    for _ in range(3):
        rn.geodesic(s_pos, s_ref, g_pos, g_ref)
    us_path = 1e6 * (time.perf_counter() - t0) / (3 * nq)
    rn.close()
    return {"one_core_env_steps_per_s": one_core, "one_core_envs": n,
            "us_per_try_step": us_try, "us_per_find_path_start_to_goal": us_path,
            "queries_timed": nq}


def torch_gae_restatement(rewards, value_preds, masks, returns, next_value, T, gamma, tau):
    """RolloutStorage.compute_returns (bps_nav/common/rollout_storage.py:203-219) restated with the
    same tensor operations: the per-step Python loop whose launch overhead the fused kernel removes."""
    value_preds[T] = next_value
    gae = 0
    for step in reversed(range(T)):
        delta = rewards[step] + gamma * value_preds[step + 1] * masks[step + 1] - value_preds[step]
        gae = delta + gamma * tau * masks[step + 1] * gae
        returns[step] = gae + value_preds[step]
    adv = returns[:T] - value_preds[:T]
    return (adv - adv.mean()) / (adv.std() + 1e-5)


def reference_compute_returns():
    """The reference's own RolloutStorage class (bps_nav/common/rollout_storage.py), loaded by
    file path when the bps-nav tree is on this machine; None otherwise."""
    from oracle import pyoracle
    root = pyoracle.reference_root()
    if not root:
        return None
    import importlib.util
    import types
    common = os.path.join(root, "bps_nav", "common")
    for pkg in ("bps_nav", "bps_nav.common"):
        if pkg not in sys.modules:
            sys.modules[pkg] = types.ModuleType(pkg)
            sys.modules[pkg].__path__ = []
    for mod in ("tree_utils", "rollout_storage"):
        spec = importlib.util.spec_from_file_location(f"bps_nav.common.{mod}",
                                                      os.path.join(common, f"{mod}.py"))
        m = importlib.util.module_from_spec(spec)
        sys.modules[f"bps_nav.common.{mod}"] = m
        spec.loader.exec_module(m)
    return sys.modules["bps_nav.common.rollout_storage"].RolloutStorage


def run_reference(args):
    """The reference arm: the same workload on the host cores.  Under torchrun only rank 0 works
    (the whole job's environments), the other ranks leave at once."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t_start = time.perf_counter()
    if args.workload == "c4":
        print(json.dumps({"impl": "reference", "unavailable":
                          "config 4 needs the reference's renderer (bps3D / Vulkan): unavailable "
                          "on this box"}), flush=True)
        return
    K, W = args.steps, max(args.warmup, 0)
    n_job = args.envs * max(args.gpus, 1)  # the whole job's environments on the host cores
    rate, d = cpu_arm(args.scene.split(","), n_job, args.mix, windows=K, warmup=W)
    ms = 1000.0 * d["seconds"] / max(d["windows"], 1)
    line = {
        "impl": "reference", "metric": "env_steps_per_sec", "value": rate, "unit": "env-steps/s",
        "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_string(args), "envs_per_gpu": args.envs,
                   "rollout_T": T_ROLLOUT},
        "measurement": {"l2": "n/a (CPU)",
                        "timing": "host wall clock around each window, summed"},
        "cpu_baseline": {"value": rate, "unit": "env-steps/s", "cores": d["cores"],
                         "kind": "reference", "sample": d["sample"]},
        "e2e": {"value": rate, "unit": "env-steps/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t_start,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ GPU arm

def run_ours(args):
    import torch
    import torch.distributed as dist

    from bps_nav_b200 import bps_sim, dist_utils, rollout
    from bps_nav_b200.dataset import Scene

    rank, world, local = dist_utils.rank_info()
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def load(nm):
        return Scene(scene_files(nm)[0], np.load(scene_files(nm)[1]), f"{nm}.glb")

    names = args.scene.split(",")
    scenes = [load(nm) for nm in names]
    scene = scenes[0]
    if args.envs % len(scenes):
        raise SystemExit("--envs must be a multiple of the number of scenes")
    N, T, K, W = args.envs, T_ROLLOUT, args.steps, max(args.warmup, 3)
    peak, peak_src = measured_peak()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        return dist_utils.max_over_ranks(x, dev)

    class Storage:
        """Rollout tensors of one group, laid out as the reference's storage lays them out."""

        def __init__(self, n):
            self.n = n
            self.rewards = torch.zeros(T + 1, n, 1, device=dev)
            self.values = torch.randn(T + 1, n, 1, device=dev)
            self.next_value = torch.randn(n, 1, device=dev)
            self.masks = torch.ones(T + 1, n, 1, dtype=torch.bool, device=dev)
            self.returns = torch.zeros(T + 1, n, 1, device=dev)
            self.adv = torch.empty(T, n, 1, device=dev)
            self.rew_rows = [self.rewards[t] for t in range(T)]
            self.mask_rows = [self.masks[t + 1] for t in range(T)]

        def returns_only(self):
            rollout.compute_returns(self.rewards, self.values, self.masks, self.returns,
                                    self.next_value, T, GAMMA, TAU, advantages=self.adv,
                                    normalize=False)

        def returns_and_normalise(self):
            rollout.compute_returns(self.rewards, self.values, self.masks, self.returns,
                                    self.next_value, T, GAMMA, TAU, advantages=self.adv,
                                    normalize=True)

    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)

    def device_windows(scene_set, n, windows, warm, seed0, groups=1, sample_clocks=False,
                       env_scene=None):
        """The device-resident window (T steps with the step's reward / mask landing in the
        rollout rows, then GAE + normalisation) timed with CUDA events per window on the launch
        stream(s), L2 flushed between windows.  With two groups the environments are split
        between them, each group steps on its own stream and the advantages of the two halves
        are normalised together.  Returns (env_steps_per_s of the whole job, ms per window,
        clocks, generator facts)."""
        gen = bps_sim.PointNavRolloutGenerator.from_scenes(
            scene_set, n, gpu_id=local, seed=dist_utils.shard_seed(seed0, rank, n),
            host_mirrors=False, double_buffered=groups == 2, env_scene=env_scene)
        B = n // groups
        store = [Storage(B) for _ in range(groups)]
        streams = [torch.cuda.current_stream()] if groups == 1 else \
            [torch.cuda.Stream() for _ in range(groups)]
        for g in range(groups):
            gen.reset(g)
        acts = torch.from_numpy(draw_actions(((warm + windows) * T, n), args.mix, 7 + rank)).to(dev)
        torch.cuda.synchronize()

        def window(k):
            base = k * T
            if groups == 1:
                st = store[0]
                for t in range(T):
                    gen.step_start(0, acts[base + t], reward_out=st.rew_rows[t],
                                   mask_out=st.mask_rows[t])
                    gen.step_end(0)
                st.returns_and_normalise()
                return
            main = torch.cuda.current_stream()
            for g in range(groups):
                streams[g].wait_stream(main)
            for t in range(T):
                for g in range(groups):
                    with torch.cuda.stream(streams[g]):
                        gen.step_start(g, acts[base + t, g * B:(g + 1) * B],
                                       reward_out=store[g].rew_rows[t],
                                       mask_out=store[g].mask_rows[t])
                        gen.step_end(g)
            for g in range(groups):
                with torch.cuda.stream(streams[g]):
                    store[g].returns_only()
                main.wait_stream(streams[g])
            rollout.normalize_advantages([st.adv for st in store])  # torch.cat(advantages, 1)

        for k in range(warm):
            window(k)
        barrier()
        sampler = ClockSampler(local) if sample_clocks and rank == 0 else None
        if sampler:
            sampler.start()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(windows)]
        t0 = time.perf_counter()
        for k in range(windows):
            flush.fill_(k & 0xFF)  # evict L2 between timed windows (untimed)
            ev[k][0].record()
            window(warm + k)
            ev[k][1].record()
        barrier()
        wall = time.perf_counter() - t0
        clocks = sampler.stop() if sampler else None
        ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in ev))
        facts = {"wall_s": wall, "mean_return": float(store[0].returns[:T].mean().item()),
                 "gen": gen, "store": store, "acts": acts}
        return world * n * T * windows / (ms / 1000.0), ms / windows, clocks, facts

    def kernel_pass(gen, acts, n, windows):
        """CUDA events around every launch of the step (programmatic dependent launch is off
        while they are recorded, so the launches do not overlap): ms per launch of each kernel
        and episode ends per step."""
        gen.profile(0, True)
        m_view = gen.tensor(0, "mask")
        nres = 0.0
        for k in range(windows):
            for t in range(T):
                gen.step_start(0, acts[k * T + t])
                gen.step_end(0)
                nres += float((m_view == 0).sum().item())
        kms, ksteps = gen.profile_read(0)
        gen.profile(0, False)
        return {k: v / max(ksteps, 1) for k, v in kms.items()}, nres / max(ksteps, 1)

    def gae_ms(st, reps=20):
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.returns_and_normalise()
        g0.record()
        for _ in range(reps):
            st.returns_and_normalise()
        g1.record()
        torch.cuda.synchronize()
        return g0.elapsed_time(g1) / reps

    def step_roofline(kms, ms_window, ms_gae, n, scene_key):
        """Roofline object of the step kernel.  Its duration is taken from the timed windows:
        with programmatic dependent launch on, the step kernel is resident from the moment the
        kernel before it starts (it stages its scene, then waits) until the step is complete, so
        one launch lasts (window - GAE) / T.  Units: when the step is one launch (no k_pre) the
        kernel does the whole step of every environment, 177 B each; when k_pre does the
        query-free part, the environments listed for the step kernel (those that moved: a
        quarter of them under uniform actions)."""
        one_launch = kms.get("k_pre", 0.0) == 0.0
        q_step = n * (1.0 if one_launch else 0.25 if args.mix == "uniform" else 0.60)
        ms_launch = (ms_window - ms_gae) / T
        achieved = q_step * BYTES_PER_ENV_STEP / (ms_launch * 1e-3) / 1e9
        share = kms["k_step"] / max(sum(kms.values()), 1e-9)
        return {"bound": "hbm", "kernel": "k_step", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES.get(scene_key), "peak_source": peak_src,
                "ms_per_launch": ms_launch, "units_per_launch": q_step,
                "units": "env-steps (whole step in one launch)" if one_launch
                         else "environments listed for the step kernel",
                "bytes_per_unit": BYTES_PER_ENV_STEP,
                "share_of_step_launches_unoverlapped": share,
                "note": "A* is latency/divergence-bound: its algorithmic HBM bytes are tiny by "
                        "design (tables and scratch stay on chip or in L2); ms_per_launch = "
                        "(timed window - GAE) / T, the step kernel's residency with dependent "
                        "launch on; kernels{} has each launch timed alone"}

    # ---------------- headline: device-resident arm
    value, ms_window, clocks, facts = device_windows(scenes, N, K, W, 1000, sample_clocks=True)
    gen, acts, st0 = facts["gen"], facts["acts"], facts["store"][0]
    info = gen.scene_info(0)
    kms, resets_per_step = kernel_pass(gen, acts, N, min(K, 5))
    ms_gae = gae_ms(st0)
    roofline = step_roofline(kms, ms_window, ms_gae, N, (args.scene, N, args.mix))
    step_ms = sum(kms.values())
    kernels = {k: {"ms_per_launch": v, "share": v / step_ms} for k, v in kms.items()}
    kernels["gae(scan+normalise)"] = {
        "ms_per_launch": ms_gae, "achieved_gbs": T * N * BYTES_PER_GAE_ELEM / (ms_gae * 1e-3) / 1e9}
    whole_step = {"achieved": N * BYTES_PER_ENV_STEP / ((ms_window - ms_gae) / T * 1e-3) / 1e9,
                  "unit": "GB/s"}
    whole_step["frac"] = whole_step["achieved"] / peak
    gen.close()
    mean_return, wall = facts["mean_return"], facts["wall_s"]
    del facts

    # ---------------- the same window at the largest per-GPU batch the benchmark
    # configurations name (32768 environments): the throughput once every warp has several
    # queries to work through
    big = None
    if not args.no_large_batch and N < LARGE_BATCH_ENVS:
        v, _, _, f = device_windows(scenes, LARGE_BATCH_ENVS, 3, 1, 2000)
        f["gen"].close()
        big = {"envs_per_gpu": LARGE_BATCH_ENVS, "windows": 3, "value": v, "unit": "env-steps/s",
               "note": "informational; not the headline workload"}

    # ---------------- config 1 read with the polygon count its description quotes: scene d0
    # (150 x 150 m, 2500 boxes, 16407 polygons; the tables do not fit shared memory, so every
    # search runs against global memory), with its own roofline and its own CPU figure
    dense = None
    if not args.no_large_batch and args.scene == "c1" and os.path.exists(scene_files(DENSE_SCENE)[0]):
        dscene = [load(DENSE_SCENE)]
        dv, dms, _, f = device_windows(dscene, N, 3, 1, 3000)
        dkms, _ = kernel_pass(f["gen"], f["acts"], N, 2)
        dgae = gae_ms(f["store"][0])
        droof = step_roofline(dkms, dms, dgae, N, (DENSE_SCENE, N, args.mix))
        f["gen"].close()
        dbig, _, _, f2 = device_windows(dscene, LARGE_BATCH_ENVS, 3, 1, 3001)
        f2["gen"].close()
        dense = {"scene": DENSE_SCENE, "polys": scene_polys(DENSE_SCENE), "windows": 3,
                 "unit": "env-steps/s", "value": dv, "envs_per_gpu": N, "ms_per_step": dms,
                 "value_large_batch": dbig, "roofline": droof,
                 "kernels": {k: {"ms_per_launch": x} for k, x in dkms.items()},
                 "note": "the '~20k polygons' reading of config 1: same device-resident window "
                         "as the headline on a dense scene (searched in global memory)"}
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            try:
                r, d = cpu_arm([DENSE_SCENE], N, args.mix, seconds=min(args.cpu_seconds, 4.0))
                dense["cpu_baseline"] = {"value": r, "unit": "env-steps/s", "cores": d["cores"],
                                         "kind": "reference", "sample": d["sample"]}
                dense["vs_cpu"] = dv / r
            except Exception as e:  # noqa: BLE001 - a reported figure, not a dependency
                dense["cpu_baseline"] = {"value": None, "sample": f"unavailable: {e}"}

    # ---------------- the environments in the two groups of a double-buffered generator
    # (simulator/simulator.cpp:1377-1399), each group on its own stream and half of the SMs
    dbuf = None
    if not args.no_extras and N % 2 == 0:
        v2, ms2, _, f = device_windows(scenes, N, min(K, 10), 2, 1000, groups=2)
        f["gen"].close()
        dbuf = {"groups": 2, "envs_per_group": N // 2, "value": v2, "unit": "env-steps/s",
                "ms_per_step": ms2,
                "note": "same workload and metric as `value`, environments split over two "
                        "groups whose steps overlap on the GPU; advantages of the two halves "
                        "normalised together"}

    # ---------------- benchmark config 2: GAE at T = 32, N = 16384
    c2 = None
    if not args.no_extras and rank == 0:
        st = Storage(C2_N)
        st.masks.copy_(torch.rand(C2_T + 1, C2_N, 1, device=dev) >= 0.002)
        st.rewards.normal_()
        ms = gae_ms(st, reps=50)
        gbs = C2_T * C2_N * BYTES_PER_GAE_ELEM / (ms * 1e-3) / 1e9
        c2 = {"T": C2_T, "N": C2_N, "fused_ms": ms, "achieved_gbs": gbs, "frac_of_hbm": gbs / peak,
              "algorithmic_bytes": C2_T * C2_N * BYTES_PER_GAE_ELEM,
              "note": "two launches (reverse scan, normalise); launch-latency-bound at this size"}
        # the same kernels where the arrays are large enough for bandwidth to count
        big_n = 16 * C2_N
        stb = Storage(big_n)
        stb.masks.copy_(torch.rand(C2_T + 1, big_n, 1, device=dev) >= 0.002)
        stb.rewards.normal_()
        msb = gae_ms(stb, reps=20)
        gbsb = C2_T * big_n * BYTES_PER_GAE_ELEM / (msb * 1e-3) / 1e9
        c2["at_16x_N"] = {"N": big_n, "fused_ms": msb, "achieved_gbs": gbsb,
                          "frac_of_hbm": gbsb / peak}
        del stb
        if world == 1:
            c2.update(gae_reference_times(st, torch))

    # ---------------- benchmark config 3: a fixed global batch block-partitioned over the ranks
    shard = None
    if not args.no_extras and all(os.path.exists(scene_files(nm)[0]) for nm in C3_SCENES) and \
            C3_ENVS % world == 0:
        first, count, scene_ids, env_scene = dist_utils.shard_plan(C3_ENVS, len(C3_SCENES), rank,
                                                                   world)
        sub = [load(C3_SCENES[i]) for i in scene_ids]
        gen3 = bps_sim.PointNavRolloutGenerator.from_scenes(
            sub, count, gpu_id=local, seed=dist_utils.shard_seed(4000, rank, count),
            host_mirrors=False, env_scene=env_scene)
        st = Storage(count)
        gen3.reset(0)
        a3 = torch.from_numpy(draw_actions((4 * T, count), args.mix, 31 + rank)).to(dev)

        def window3(k):
            for t in range(T):
                gen3.step_start(0, a3[k * T + t], reward_out=st.rew_rows[t],
                                mask_out=st.mask_rows[t])
                gen3.step_end(0)
            st.returns_and_normalise()

        window3(0)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(3):
            window3(1 + k)
        e1.record()
        barrier()
        ms3 = max_over_ranks(e0.elapsed_time(e1))
        gen3.close()
        shard = {"global_envs": C3_ENVS, "scenes": len(C3_SCENES), "envs_per_rank": count,
                 "scenes_per_rank": len(scene_ids), "windows": 3, "scaling": "strong",
                 "value": C3_ENVS * T * 3 / (ms3 / 1000.0), "unit": "env-steps/s",
                 "note": "config 3: rank r owns environments [r N/G, (r+1) N/G) of the global "
                         "batch and loads only the scenes that block touches "
                         "(dist_utils.shard_plan); no collective on the data path"}

    # ---------------- depth sensor (optional observation path; informational)
    depth_info = None
    if not args.no_depth and scene.floor is not None:
        RW, RH = 64, 64
        gend = bps_sim.PointNavRolloutGenerator.from_scenes(
            scenes, N, gpu_id=local, seed=dist_utils.shard_seed(3000, rank, N),
            host_mirrors=False, depth=True, render_resolution=(RW, RH))
        gend.reset(0)
        for t in range(8):
            gend.step(0, acts[t])
        torch.cuda.synchronize()
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 20
        d0.record()
        for _ in range(reps):
            gend.render(0)
        d1.record()
        torch.cuda.synchronize()
        d_ms = max_over_ranks(d0.elapsed_time(d1)) / reps
        nbox = int(np.mean([len(sc.boxes) for sc in scenes]))
        depth_info = {"resolution": [RW, RH], "boxes": nbox, "ms_per_render": d_ms,
                      "rays_per_s": world * N * RW * RH / (d_ms * 1e-3),
                      "image_write_gbs": N * RW * RH * 4 / (d_ms * 1e-3) / 1e9,
                      "note": "k_depth: analytic ray / box sensor, fp32-pipe-bound; not part of "
                              "the headline metric (the benchmark configuration disables rendering)"}
        gend.close()

    # ---------------- end-to-end through the reference-shaped host API: numpy actions in (H2D),
    # numpy reward / mask / info / polar out (D2H) every step; the rollout rows are filled on
    # the device by the same launch; one device -> host read of the window's result
    e2e = None
    if not args.no_e2e:
        hacts = draw_actions(((W + K) * T, N), args.mix, 7 + rank)

        def e2e_run(groups):
            gen2 = bps_sim.PointNavRolloutGenerator.from_scenes(
                scenes, N, gpu_id=local, seed=dist_utils.shard_seed(1000, rank, N),
                host_mirrors=True, double_buffered=groups == 2)
            B = N // groups
            store = [Storage(B) for _ in range(groups)]
            views = [(gen2.get_rewards(g), gen2.get_masks(g), gen2.get_infos(g), gen2.get_polars(g))
                     for g in range(groups)]
            for g in range(groups):
                gen2.reset(g)
            sink = [0.0]

            def read(g):
                r, m, i, p = views[g]
                sink[0] += (float(p[0, 0]) + float(i["distanceToGoal"][0]) + float(r[0]) +
                            float(m[0]))

            def window(k):
                base = k * T
                if groups == 1:
                    st = store[0]
                    for t in range(T):
                        gen2.step_start(0, hacts[base + t], reward_out=st.rew_rows[t],
                                        mask_out=st.mask_rows[t])
                        gen2.step_end(0)
                        read(0)
                    st.returns_and_normalise()
                    return float(st.adv.mean().item())
                # the trainer's alternation (bps_nav/rl/ppo/ppo_trainer.py:245-275): while one
                # group's step runs on the GPU the host collects the other group's results and
                # starts its next step
                for g in range(groups):
                    gen2.step_start(g, hacts[base, g * B:(g + 1) * B],
                                    reward_out=store[g].rew_rows[0], mask_out=store[g].mask_rows[0])
                for t in range(1, T + 1):
                    for g in range(groups):
                        gen2.step_end(g)
                        read(g)
                        if t < T:
                            gen2.step_start(g, hacts[base + t, g * B:(g + 1) * B],
                                            reward_out=store[g].rew_rows[t],
                                            mask_out=store[g].mask_rows[t])
                for st in store:
                    st.returns_only()
                rollout.normalize_advantages([st.adv for st in store])
                return float(store[0].adv.mean().item())

            for k in range(W):
                window(k)
            barrier()
            t0 = time.perf_counter()
            for k in range(K):
                window(W + k)
            barrier()
            secs = max_over_ranks(time.perf_counter() - t0)
            gen2.close()
            return {"value": world * N * T * K / secs, "ms_per_step": 1000 * secs / K}

        variants = {"one_group": e2e_run(1)}
        if N % 2 == 0:
            variants["double_buffered"] = e2e_run(2)
        best = max(variants, key=lambda k: variants[k]["value"])
        h2d = T * N                               # actions cross the bus as one byte each
        d2h = T * (N * 4 + N + N * 12 + N * 8) + 4  # reward, mask, info, polar (+ window result)
        e2e = {"value": variants[best]["value"], "unit": "env-steps/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": variants[best]["ms_per_step"], "variant": best,
               "variants": variants,
               "how": "host wall clock, barrier + synchronize on both sides, max over ranks; "
                      "variant = how the host API was driven (one group, or the two groups of a "
                      "double-buffered generator alternately, the reference trainer's way)"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            rate, d = cpu_arm(names, N, args.mix, seconds=args.cpu_seconds)
            cpu = {"value": rate, "unit": "env-steps/s", "cores": d["cores"], "kind": "reference",
                   "sample": d["sample"], "seconds": d["seconds"]}
            cpu.update(cpu_microbench(args))
        except Exception as e:  # the baseline is a reported figure, not a dependency
            cpu = {"value": None, "unit": "env-steps/s", "cores": 0, "kind": "reference",
                   "sample": f"unavailable: {e}"}

    if rank == 0:
        # small batches of fixed scenes run the whole step as one launch (no k_pre)
        launches_per_step = 2 if kms.get("k_pre", 0.0) > 0.0 else 1
        line = {
            "metric": "env_steps_per_sec", "value": value, "unit": "env-steps/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms_window, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_string(args), "envs_per_gpu": N, "rollout_T": T},
            "measurement": {"l2": f"flushed between timed windows ({L2_FLUSH_BYTES >> 20} MiB write)",
                            "timing": "CUDA events per window on the launch stream, summed, max "
                                      "over ranks",
                            "polys": info["num_polys"], "islands": info["num_islands"]},
            "clocks": clocks, "e2e": e2e, "roofline": roofline, "roofline_whole_step": whole_step,
            "kernels": kernels, "cpu_baseline": cpu, "dense_scene": dense, "large_batch": big,
            "double_buffered": dbuf, "c2": c2, "shard": shard, "depth_sensor": depth_info,
            "gpu_launches": K * (T * launches_per_step + 2), "resets_per_step": resets_per_step,
            "mean_return": mean_return, "wall_s_device_arm": wall,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def gae_reference_times(st, torch):
    """Config 2 beside the reference: RolloutStorage.compute_returns + the get_advantages
    formula on CUDA tensors (what the reference's trainer runs) and on CPU tensors -- the
    reference's own class when the bps-nav tree is on this machine, otherwise the restatement of
    its loop (labelled).  Median wall time per call including launches and a synchronize."""
    T, N = C2_T, C2_N

    def med(fn, reps, sync):
        ts = []
        for _ in range(reps):
            if sync:
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            fn()
            if sync:
                torch.cuda.synchronize()
            ts.append(time.perf_counter() - t0)
        return 1000.0 * float(np.median(ts))

    RS = None
    try:
        RS = reference_compute_returns()
    except Exception:  # noqa: BLE001 - fall back to the restatement
        RS = None
    out = {}
    for where in ("cuda", "cpu"):
        r, v, m = st.rewards.to(where), st.values.to(where), st.masks.to(where)
        nv = st.next_value.to(where)
        if RS is not None:
            class _Space:
                spaces = {}
            rs = RS(T, N, _Space(), None, 8, 1)
            rs.to(where)
            sb = rs.storage_buffers
            sb["rewards"].copy_(r)
            sb["value_preds"].copy_(v)
            sb["masks"].copy_(m)
            rs.step = T

            def fn():
                rs.compute_returns(nv, True, GAMMA, TAU)
                a = sb["returns"][:-1] - sb["value_preds"][:-1]
                return (a - a.mean()) / (a.std() + 1e-5)
        else:
            ret = torch.zeros_like(r)

            def fn():
                return torch_gae_restatement(r, v, m, ret, nv, T, GAMMA, TAU)
        out[f"reference_loop_{where}_ms"] = med(fn, 20 if where == "cuda" else 5, where == "cuda")
    out["reference_loop_is"] = ("the reference's RolloutStorage.compute_returns (loaded by path)"
                                if RS is not None else
                                "restatement of its per-step tensor-op loop (bps-nav tree absent)")
    return out


def run_c4(args):
    """Benchmark config 4, a load generator around the simulator path: per GPU 32768
    environments over 64 scene slots, double-buffered; every step = simulator step + 64 x 64
    depth render + policy inference on the observations; after T = 32 steps GAE and one PPO
    epoch (clipped surrogate, value and entropy terms, two minibatches of environments, BPTT
    through the LSTM) with the gradients all-reduced over NCCL by DistributedDataParallel.
    The policy is a plain-torch stand-in of the architecture the configuration names -- a
    ResNet-18 at half width (32 base planes, GroupNorm) on the depth image, the GPS/compass and
    previous-action embeddings, a 2-layer LSTM of 512 units, actor and critic heads -- with
    random weights, run in fp16 autocast.  It is not an optimisation target: the figures of
    interest are the simulator path's rate and its share of the step time
    (bps_nav/rl/ppo/ppo_trainer.py:200-284 keeps the same split)."""
    import torch
    import torch.distributed as dist
    import torch.nn as nn
    import torch.nn.functional as F

    from bps_nav_b200 import bps_pytorch, bps_sim, dist_utils, rollout
    from bps_nav_b200.dataset import Scene

    rank, world, local = dist_utils.rank_info()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    N, T, K, W = args.envs, T_ROLLOUT, max(1, min(args.steps, 3)), 1
    SLOTS, RES, MB = 64, (64, 64), 8
    names = [C3_SCENES[i % len(C3_SCENES)] for i in range(SLOTS)]
    scenes = [Scene(scene_files(nm)[0], np.load(scene_files(nm)[1]), f"{nm}_{i}.glb")
              for i, nm in enumerate(names)]
    gen = bps_sim.PointNavRolloutGenerator.from_scenes(
        scenes, N, gpu_id=local, seed=dist_utils.shard_seed(5000, rank, N), host_mirrors=False,
        depth=True, render_resolution=RES, double_buffered=True)
    B = N // 2

    def block(cin, cout, stride):
        return nn.ModuleDict({
            "c1": nn.Conv2d(cin, cout, 3, stride, 1, bias=False), "n1": nn.GroupNorm(16, cout),
            "c2": nn.Conv2d(cout, cout, 3, 1, 1, bias=False), "n2": nn.GroupNorm(16, cout),
            "sc": nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), nn.GroupNorm(16, cout))
            if stride != 1 or cin != cout else nn.Identity()})

    class Policy(nn.Module):
        def __init__(self, base=32, hidden=512):
            super().__init__()
            self.stem = nn.Sequential(nn.Conv2d(1, base, 7, 2, 3, bias=False), nn.GroupNorm(16, base),
                                      nn.ReLU(True), nn.MaxPool2d(3, 2, 1))
            cfg = [(base, base, 1), (base, base, 1), (base, 2 * base, 2), (2 * base, 2 * base, 1),
                   (2 * base, 4 * base, 2), (4 * base, 4 * base, 1), (4 * base, 8 * base, 2),
                   (8 * base, 8 * base, 1)]
            self.blocks = nn.ModuleList([block(*c) for c in cfg])
            self.compress = nn.Sequential(nn.Conv2d(8 * base, 64, 3, 1, 1, bias=False),
                                          nn.GroupNorm(1, 64), nn.ReLU(True))
            self.fc = nn.Sequential(nn.Flatten(), nn.Linear(64 * 2 * 2, hidden), nn.ReLU(True))
            self.goal = nn.Linear(3, 32)
            self.prev_action = nn.Embedding(5, 32)
            self.rnn = nn.LSTM(hidden + 64, hidden, num_layers=2)
            self.actor = nn.Linear(hidden, 4)
            self.critic = nn.Linear(hidden, 1)

        def encode(self, depth, polar, prev_a):
            x = self.stem(depth)
            for b in self.blocks:
                y = F.relu(b["n1"](b["c1"](x)))
                y = b["n2"](b["c2"](y))
                x = F.relu(y + b["sc"](x))
            x = self.fc(self.compress(x))
            g = torch.stack([polar[:, 0], torch.cos(-polar[:, 1]), torch.sin(-polar[:, 1])], -1)
            return torch.cat([x, self.goal(g.to(x.dtype)), self.prev_action(prev_a)], -1)

        def forward(self, depth, polar, prev_a, hc, masks, steps=1):
            """depth [steps * n, 1, H, W] ...; hc = (h, c) each [2, n, hidden]; masks [steps * n]
            (0 where an episode began: the state is reset there)."""
            f = self.encode(depth, polar, prev_a).view(steps, -1, 512 + 64)
            m = masks.view(steps, 1, -1, 1).to(f.dtype)
            outs = []
            h, c = hc
            for t in range(steps):
                o, (h, c) = self.rnn(f[t:t + 1], (h * m[t], c * m[t]))
                outs.append(o)
            o = torch.cat(outs, 0).view(-1, 512)
            return self.actor(o), self.critic(o), (h, c)

    torch.manual_seed(1 + rank)
    policy = Policy().to(dev)
    ddp = nn.parallel.DistributedDataParallel(policy, device_ids=[local]) if world > 1 else policy
    opt = torch.optim.Adam(policy.parameters(), lr=5e-4, eps=1e-5)

    class Buf:
        def __init__(self):
            self.depth = torch.zeros(T + 1, B, 1, RES[1], RES[0], dtype=torch.float16, device=dev)
            self.polar = torch.zeros(T + 1, B, 2, device=dev)
            self.prev_a = torch.zeros(T + 1, B, dtype=torch.long, device=dev)
            self.actions = torch.zeros(T, B, dtype=torch.long, device=dev)
            self.logp = torch.zeros(T, B, device=dev)
            self.rewards = torch.zeros(T + 1, B, 1, device=dev)
            self.values = torch.zeros(T + 1, B, 1, device=dev)
            self.masks = torch.ones(T + 1, B, 1, dtype=torch.bool, device=dev)
            self.returns = torch.zeros(T + 1, B, 1, device=dev)
            self.adv = torch.zeros(T, B, 1, device=dev)
            self.h0 = torch.zeros(2, B, 512, device=dev, dtype=torch.float16)
            self.c0 = torch.zeros(2, B, 512, device=dev, dtype=torch.float16)
            self.hc = (self.h0.clone(), self.c0.clone())

    bufs = [Buf(), Buf()]
    depth_view = [bps_pytorch.make_depth_tensor(gen.depth(g), local, B, RES) for g in range(2)]
    polar_view = [gen.tensor(g, "polar") for g in range(2)]
    for g in range(2):
        gen.reset(g)
        gen.render(g)
        bufs[g].depth[0, :, 0] = depth_view[g].clamp(max=10.0) / 10.0
        bufs[g].polar[0] = polar_view[g]
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    rollout_clocks = []

    def rollout_and_learn(timed):
        t_sim = t_pol = 0.0
        marks = []
        for g in range(2):
            b = bufs[g]
            b.h0.copy_(b.hc[0])
            b.c0.copy_(b.hc[1])
        # the SM clock while the rollout (policy inference + simulator + depth) runs: the
        # simulator's steps are latency-bound and follow it
        sampler = ClockSampler(local) if timed and rank == 0 else None
        if sampler:
            torch.cuda.synchronize()
            sampler.start()
        for t in range(T):
            for g in range(2):
                b = bufs[g]
                e0, e1, e2, e3 = ev(), ev(), ev(), ev()
                e0.record()
                with torch.no_grad(), torch.autocast("cuda", dtype=torch.float16):
                    logits, value, b.hc = policy(b.depth[t], b.polar[t], b.prev_a[t], b.hc,
                                                 b.masks[t, :, 0])
                    dist_ = torch.distributions.Categorical(logits=logits.float())
                    a = dist_.sample()
                    b.actions[t] = a
                    b.logp[t] = dist_.log_prob(a)
                    b.values[t] = value.float()
                e1.record()
                gen.step_start(g, a, reward_out=b.rewards[t], mask_out=b.masks[t + 1],
                               polar_out=b.polar[t + 1])
                gen.step_end(g)
                e2.record()
                gen.render(g)
                e3.record()
                b.depth[t + 1, :, 0] = depth_view[g].clamp(max=10.0) / 10.0
                b.prev_a[t + 1] = (a + 1) * b.masks[t + 1, :, 0]
                marks.append((e0, e1, e2, e3))
        if sampler:
            torch.cuda.synchronize()
            rollout_clocks.append(sampler.stop())
        l0, lg, l1, l2 = ev(), ev(), ev(), ev()
        l0.record()
        nvs = []
        for g in range(2):
            b = bufs[g]
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.float16):
                _, nv, _ = policy(b.depth[T], b.polar[T], b.prev_a[T], b.hc, b.masks[T, :, 0])
            nvs.append(nv.float())
        lg.record()
        for g in range(2):
            b = bufs[g]
            rollout.compute_returns(b.rewards, b.values, b.masks, b.returns, nvs[g], T, GAMMA,
                                    TAU, advantages=b.adv, normalize=False)
        rollout.normalize_advantages([bufs[0].adv, bufs[1].adv])
        l1.record()
        per = B // (MB // 2)
        for g in range(2):
            b = bufs[g]
            for s in range(0, B, per):
                sl = slice(s, s + per)
                with torch.autocast("cuda", dtype=torch.float16):
                    logits, value, _ = ddp(
                        b.depth[:T, sl].reshape(-1, 1, RES[1], RES[0]), b.polar[:T, sl].reshape(-1, 2),
                        b.prev_a[:T, sl].reshape(-1), (b.h0[:, sl], b.c0[:, sl]),
                        b.masks[:T, sl, 0].reshape(-1), steps=T)
                d = torch.distributions.Categorical(logits=logits.float())
                ratio = torch.exp(d.log_prob(b.actions[:, sl].reshape(-1)) - b.logp[:, sl].reshape(-1))
                adv = b.adv[:, sl, 0].reshape(-1)
                act_loss = -torch.min(ratio * adv, ratio.clamp(0.8, 1.2) * adv).mean()
                v_loss = 0.5 * (b.returns[:T, sl, 0].reshape(-1) - value.float().view(-1)).pow(2).mean()
                loss = act_loss + 0.5 * v_loss - 0.01 * d.entropy().mean()
                opt.zero_grad(set_to_none=True)
                loss.backward()   # DDP all-reduces the gradients over NCCL here
                nn.utils.clip_grad_norm_(policy.parameters(), 0.25)
                opt.step()
        l2.record()
        for g in range(2):
            b = bufs[g]
            b.depth[0].copy_(b.depth[T])
            b.polar[0].copy_(b.polar[T])
            b.prev_a[0].copy_(b.prev_a[T])
            b.masks[0].copy_(b.masks[T])
        torch.cuda.synchronize()
        if timed:
            t_render = 0.0
            for e0, e1, e2, e3 in marks:
                t_pol += e0.elapsed_time(e1)
                t_sim += e1.elapsed_time(e2)
                t_render += e2.elapsed_time(e3)
            t_pol += l0.elapsed_time(lg)  # the value of the last observation
            return t_sim, t_pol, lg.elapsed_time(l1), l1.elapsed_time(l2), t_render
        return None

    for _ in range(W):
        rollout_and_learn(False)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    tot = np.zeros(5)
    w0 = time.perf_counter()
    for _ in range(K):
        tot += np.array(rollout_and_learn(True))
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - w0
    sim_ms, pol_ms, gae_ms_, learn_ms, render_ms = [dist_utils.max_over_ranks(x, dev) / K
                                                   for x in tot]
    wall = dist_utils.max_over_ranks(wall, dev) / K
    gen.close()
    if rank == 0:
        sim_path_ms = sim_ms + gae_ms_
        step_ms = sim_ms + render_ms + pol_ms + gae_ms_ + learn_ms
        line = {
            "metric": "env_steps_per_sec", "workload": "c4",
            "value": world * N * T / (sim_path_ms / 1000.0), "unit": "env-steps/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"config4: {N} envs/GPU over {SLOTS} scene slots (two groups), "
                                   f"T={T} sim steps + 64x64 depth + GAE feeding a random-init "
                                   "ResNet-18-half + 2-layer LSTM-512 policy, one PPO epoch of "
                                   f"{MB} minibatches, DDP gradient all-reduce over NCCL",
                       "envs_per_gpu": N, "rollout_T": T},
            "sim_path": {"ms_per_window": sim_path_ms, "share_of_step_time": sim_path_ms / step_ms,
                         "steps_ms": sim_ms, "gae_ms": gae_ms_,
                         "what": "the simulator steps of both groups over T steps (navmesh move, "
                                 "geodesic, sensor, reward / done / reset; CUDA events around "
                                 "them) + GAE and advantage normalisation"},
            "clocks_during_rollout": rollout_clocks[-1] if rollout_clocks else None,
            "depth_render_ms": render_ms, "depth_render_share": render_ms / step_ms,
            "policy_inference_ms": pol_ms, "learner_ms": learn_ms,
            "whole_window_env_steps_per_s": world * N * T / wall,
            "wall_ms_per_window": 1000 * wall,
            "note": "value = the simulator path's own rate (environment steps of the window / "
                    "time spent in the simulator steps + GAE); the depth sensor, the policy and "
                    "the learner are reported beside it and are load, not optimisation targets",
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "c4":
        run_c4(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
