"""Generates every fixture under tests/golden/ (run from the repository root, on a machine that
has the bps-nav tree; BPS_NAV_REFERENCE names its root):

    export BPS_NAV_REFERENCE=/path/to/bps-nav
    make -C oracle ref sim && python tests/golden/make_fixtures.py

What it writes
  scenes/<name>.navmesh         synthetic floor plans built by oracle/_ref/gen_scene (the
                                reference's own Recast + dtCreateNavMeshData, unmodified)
  scenes/<name>.scene.json      the generator's manifest (obstacle boxes, Recast parameters, counts)
  scenes/<name>.episodes.npy    float32 [n, 10] episodes: start xyz, start rotation xyzw, goal xyz;
                                start/goal = area-weighted random navigable points
                                (dtNavMeshQuery::findRandomPoint), kept iff the reference geodesic
                                start -> goal is finite and within [1, 30] m
  queries_<name>.npz            inputs and reference outputs of snapPoint / tryStep / findPath
  c0_traj.npz                   64 envs x 500 steps of the oracle simulator on scene c0 with the
                                "uniform" action stream: per-step reward / mask / info / polar and
                                state snapshots
  c0_policy_traj.npz            the same with the "policy" action mix (long episodes)
  gae_ref.npz                   inputs and outputs of the reference's own Python
                                RolloutStorage.compute_returns (loaded from the reference tree by
                                file path) and of the get_advantages formula
  gae_c2_16384.npz              the same at benchmark config 2's full size (T = 32, N = 16384):
                                the inputs come from a seeded numpy generator that the tests
                                re-run (gae_c2_inputs below), the file holds the reference's
                                outputs for every 16th environment, CRC-32 of the full returns /
                                advantages arrays and their sums

Scene list: c0 = benchmark config 0 (20x20 m, 12 boxes, seed 1000); c1 = config 1 (50x50 m, 60
boxes, seed 1001); d0 = a dense plan with the polygon count that config 1's description quotes
(150x150 m, 2500 boxes, seed 1002: 16407 polygons); m00..m15 = config 3's mixed batch (sides U(10,80) m, 5..150 boxes, interior
walls with door gaps; seeds 2000+i).
"""
import importlib.util
import os
import subprocess
import sys
import types
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import pyoracle  # noqa: E402

GOLD = os.path.join(ROOT, "tests", "golden")
SCENES = os.path.join(GOLD, "scenes")


def scene_specs():
    specs = [("c0", dict(size=20, boxes=12, walls=0, seed=1000), 256),
             ("c1", dict(size=50, boxes=60, walls=0, seed=1001), 4096),
             ("d0", dict(size=150, boxes=2500, walls=0, seed=1002), 4096)]
    rng = np.random.default_rng(20240)
    for i in range(16):
        sx = float(np.round(rng.uniform(10, 80), 1))
        sz = float(np.round(rng.uniform(10, 80), 1))
        area = sx * sz
        boxes = int(np.clip(rng.integers(5, 151) * area / 3200.0, 5, 150))
        walls = int(np.clip(round((sx + sz) / 12.0), 1, 12))
        specs.append((f"m{i:02d}", dict(size=sx, size_z=sz, boxes=boxes, walls=walls,
                                        seed=2000 + i), 1024))
    return specs


def build_scene(name, spec):
    out = os.path.join(SCENES, name)
    cmd = [pyoracle.GEN_SCENE, "--size", str(spec["size"]), "--boxes", str(spec["boxes"]),
           "--walls", str(spec["walls"]), "--seed", str(spec["seed"]), "--out", out]
    if "size_z" in spec:
        cmd += ["--size-z", str(spec["size_z"])]
    res = subprocess.run(cmd, check=True, capture_output=True, text=True)
    print("  ", res.stdout.strip())
    return out + ".navmesh"


def make_episodes(nav, n, seed):
    pool, _ = nav.random_points(8 * n + 2048, seed)
    rng = np.random.default_rng(seed)
    eps = np.zeros((0, 10), np.float32)
    tries = 0
    while len(eps) < n and tries < 40:
        tries += 1
        i = rng.integers(0, len(pool), 4 * n)
        j = rng.integers(0, len(pool), 4 * n)
        s, sr = nav.snap(pool[i])
        g, gr = nav.snap(pool[j])
        d = nav.geodesic(s, sr, g, gr)
        ok = np.isfinite(d) & (d >= 1.0) & (d <= 30.0)
        yaw = rng.uniform(0, 2 * np.pi, ok.sum()).astype(np.float32)
        rot = np.stack([np.zeros_like(yaw), np.sin(yaw / 2), np.zeros_like(yaw), np.cos(yaw / 2)], 1)
        batch = np.concatenate([pool[i][ok], rot.astype(np.float32), pool[j][ok]], 1)
        eps = np.concatenate([eps, batch.astype(np.float32)], 0)
    if len(eps) < n:
        raise RuntimeError("could not sample enough episodes")
    return np.ascontiguousarray(eps[:n])


def make_queries(nav, name, n, seed):
    rng = np.random.default_rng(seed)
    pts, _ = nav.random_points(n, seed + 1)
    q = pts + rng.normal(0, 0.7, pts.shape).astype(np.float32) * np.array([1, 0.5, 1], np.float32)
    q[::17] += 30.0  # far outside: snap fails (NaN, ref 0)
    q[5] = [np.nan, 0, 0]
    q[6] = [np.inf, 0, 0]
    snap_xyz, snap_ref = nav.snap(q)
    ok = ~np.isnan(snap_xyz[:, 0])
    s, sr = snap_xyz[ok], snap_ref[ok]
    m = len(s)
    ang = rng.uniform(0, 2 * np.pi, m).astype(np.float32)
    step = np.where(np.arange(m) % 5 == 0, 2.5, 0.25).astype(np.float32)
    e = s + np.stack([np.cos(ang) * step, np.zeros(m, np.float32), np.sin(ang) * step], 1)
    e = e.astype(np.float32)
    ts_xyz, ts_ref = nav.try_step(s, sr, e)
    b = rng.permutation(m)
    b[::11] = np.arange(m)[::11]  # identical endpoints -> 0 via the isApprox early-out
    ga, gar, gb, gbr = ts_xyz, ts_ref, ts_xyz[b], ts_ref[b]
    # a few queries with an unsnapped (ref 0 / NaN) endpoint
    gb = gb.copy()
    gbr = gbr.copy()
    gb[3] = np.nan
    gbr[3] = 0
    dist = nav.geodesic(ga, gar, gb, gbr)
    np.savez_compressed(os.path.join(GOLD, f"queries_{name}.npz"), snap_in=q, snap_xyz=snap_xyz,
                        snap_ref=snap_ref.astype(np.uint32), step_start=s,
                        step_start_ref=sr.astype(np.uint32), step_end=e, step_xyz=ts_xyz,
                        step_ref=ts_ref.astype(np.uint32), geo_a=ga, geo_a_ref=gar.astype(np.uint32),
                        geo_b=gb, geo_b_ref=gbr.astype(np.uint32), geo_dist=dist)
    print(f"   queries_{name}: snap {len(q)} (fail {int((~ok).sum())}), step {m}, geodesic inf "
          f"{int(np.isinf(dist).sum())}")


def make_traj(navmesh, episodes, fname, num_envs, steps, seed, act_seed, mix):
    sim = pyoracle.OracleSim([(navmesh, episodes)], num_envs, seed)
    actions = pyoracle.philox_actions(steps, num_envs, act_seed, mix)
    sim.reset()
    snaps = {}
    st = sim.state()
    snaps[0] = st
    polar0 = sim.polars.copy()
    R = np.zeros((steps, num_envs), np.float32)
    M = np.zeros((steps, num_envs), np.uint8)
    I = np.zeros((steps, num_envs, 3), np.float32)
    P = np.zeros((steps, num_envs, 2), np.float32)
    keep = sorted(set([1, 2, 5, 10, 50, 100, 250, steps]))
    for t in range(steps):
        sim.step(actions[t])
        R[t], M[t], I[t], P[t] = sim.rewards, sim.masks, sim.infos, sim.polars
        if (t + 1) in keep:
            snaps[t + 1] = sim.state()
    out = dict(actions=actions.astype(np.int8), reward=R, mask=M, info=I, polar=P, polar0=polar0,
               seed=np.uint64(seed), act_seed=np.uint64(act_seed),
               snap_steps=np.array(sorted(snaps), np.int32))
    for k in sorted(snaps):
        for name, v in snaps[k].items():
            out[f"s{k}_{name}"] = v
    np.savez_compressed(os.path.join(GOLD, fname), **out)
    c = sim.counters()
    print(f"   {fname}: {steps} steps x {num_envs} envs; oracle calls {c}; resets/step "
          f"{(1 - M.mean()):.3f}; non-finite rewards {int((~np.isfinite(R)).sum())}")


def make_gae(reference_root):
    """Runs the reference's own rollout_storage.py (loaded by path; `import bps_nav` needs gym)."""
    import torch
    common = os.path.join(reference_root, "bps_nav", "common")
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
    RS = sys.modules["bps_nav.common.rollout_storage"].RolloutStorage

    class _Space:
        spaces = {}

    out = {}
    for tag, (T, N, pdone) in {"small": (16, 256, 0.05), "c2": (32, 2048, 0.002)}.items():
        torch.manual_seed(0 if tag == "c2" else 1)
        rs = RS(T, N, _Space(), None, 8, 1)
        sb = rs.storage_buffers
        sb["rewards"].copy_(torch.randn(T + 1, N, 1))
        sb["value_preds"].copy_(torch.randn(T + 1, N, 1))
        sb["masks"].copy_(torch.rand(T + 1, N, 1) >= pdone)
        next_value = torch.randn(N, 1)
        rs.step = T
        out[f"{tag}_rewards"] = sb["rewards"].numpy().copy()
        out[f"{tag}_values"] = sb["value_preds"].numpy().copy()
        out[f"{tag}_masks"] = sb["masks"].numpy().copy()
        out[f"{tag}_next_value"] = next_value.numpy().copy()
        rs.compute_returns(next_value, True, 0.99, 0.95)
        out[f"{tag}_returns"] = sb["returns"].numpy().copy()
        adv = sb["returns"][:-1] - sb["value_preds"][:-1]  # ppo.py:193-195
        out[f"{tag}_adv"] = adv.numpy().copy()
        out[f"{tag}_adv_norm"] = ((adv - adv.mean()) / (adv.std() + 1e-5)).numpy().copy()
    np.savez_compressed(os.path.join(GOLD, "gae_ref.npz"), **out)
    print("   gae_ref.npz written from the reference's RolloutStorage.compute_returns")

    # benchmark config 2 at its full size
    T, N = 32, 16384
    r, v, m, nv = gae_c2_inputs(T, N)
    rs = RS(T, N, _Space(), None, 8, 1)
    sb = rs.storage_buffers
    sb["rewards"].copy_(torch.from_numpy(r)[..., None])
    sb["value_preds"].copy_(torch.from_numpy(v)[..., None])
    sb["masks"].copy_(torch.from_numpy(m)[..., None])
    rs.step = T
    rs.compute_returns(torch.from_numpy(nv)[:, None], True, 0.99, 0.95)
    ret = sb["returns"][:T, :, 0]
    adv = ret - sb["value_preds"][:T, :, 0]                     # ppo.py:193-195
    advn = (adv - adv.mean()) / (adv.std() + 1e-5)               # ppo.py:201
    # per range of 4096 environments (the reference's minibatches are sets of environments,
    # rollout_storage.py:228-238); the same formula on each range
    advr = torch.cat([(adv[:, s:s + 4096] - adv[:, s:s + 4096].mean()) /
                      (adv[:, s:s + 4096].std() + 1e-5) for s in range(0, N, 4096)], 1)
    cols = np.arange(0, N, 16)
    np.savez_compressed(
        os.path.join(GOLD, "gae_c2_16384.npz"), cols=cols.astype(np.int32),
        returns_cols=ret.numpy()[:, cols].copy(), adv_cols=adv.numpy()[:, cols].copy(),
        adv_norm_cols=advn.numpy()[:, cols].copy(), adv_range_norm_cols=advr.numpy()[:, cols].copy(),
        returns_crc=np.uint32(zlib.crc32(np.ascontiguousarray(ret.numpy()).tobytes())),
        adv_crc=np.uint32(zlib.crc32(np.ascontiguousarray(adv.numpy()).tobytes())),
        returns_sum=np.float64(ret.double().sum().item()),
        adv_mean=np.float64(adv.double().mean().item()),
        adv_std=np.float64(adv.double().std().item()),
        adv_mean_f32=np.float32(adv.mean().item()), adv_std_f32=np.float32(adv.std().item()))
    print("   gae_c2_16384.npz written (T = 32, N = 16384)")


def gae_c2_inputs(T=32, N=16384, seed=20250):
    """Benchmark config 2's inputs: rewards, values ~ N(0, 1) float32 [T+1, N], masks = not
    Bernoulli(0.002) bool [T+1, N], next_value float32 [N], from numpy's PCG64 (the same arrays on
    every machine)."""
    rng = np.random.default_rng(seed)
    r = rng.standard_normal((T + 1, N), dtype=np.float32)
    v = rng.standard_normal((T + 1, N), dtype=np.float32)
    m = rng.random((T + 1, N)) >= 0.002
    nv = rng.standard_normal(N, dtype=np.float32)
    return r, v, m, nv


def main():
    if not pyoracle.available():
        raise SystemExit("build the oracle first: make -C oracle ref sim")
    os.makedirs(SCENES, exist_ok=True)
    only = set(sys.argv[1:])
    for name, spec, neps in scene_specs():
        if only and name not in only and "scenes" not in only:
            continue
        print(name, spec)
        path = build_scene(name, spec)
        nav = pyoracle.RefNav(path)
        eps = make_episodes(nav, neps, spec["seed"])
        np.save(os.path.join(SCENES, f"{name}.episodes.npy"), eps)
        if name in ("c0", "c1", "m03"):
            make_queries(nav, name, 3000, spec["seed"] + 7)
        nav.close()
    if not only or "traj" in only:
        c0 = os.path.join(SCENES, "c0.navmesh")
        eps = np.load(os.path.join(SCENES, "c0.episodes.npy"))
        make_traj(c0, eps, "c0_traj.npz", 64, 500, seed=12345, act_seed=777, mix="uniform")
        make_traj(c0, eps, "c0_policy_traj.npz", 64, 500, seed=12345, act_seed=778, mix="policy")
    if not only or "gae" in only:
        ref = pyoracle.reference_root()
        if ref:
            make_gae(ref)
        else:
            print("   GAE fixtures skipped: set BPS_NAV_REFERENCE to the root of the bps-nav tree")


if __name__ == "__main__":
    main()
