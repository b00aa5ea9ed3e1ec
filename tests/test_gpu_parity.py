"""GPU parity tests: CUDA path (through the C ABI) against golden vectors recorded from the
oracle (the reference's compiled PathFinder + the simulator restatement) and, when the oracle
libraries are present on the box, against the oracle run live on larger cases.

Tolerances (from the task statement): integer outputs (mask, success, polygon refs, step and
episode counters) bit-exact; poses within 1e-5 m; geodesic distance and reward within 1e-4
relative; GAE returns within 1e-5 relative.  Polar (GPS/compass) is a sensor output computed with
atan2f, whose device and host implementations differ by ulps: 1e-5 absolute on rho, 1e-5 rad on phi.
"""
import os

import numpy as np
import pytest

from conftest import GOLD, load_scene

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _gen(scenes, n, **kw):
    from bps_nav_b200 import bps_sim
    return bps_sim.PointNavRolloutGenerator.from_scenes(scenes, n, **kw)


def _close(a, b, rel, abs_=0.0):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    same = (a == b) | (np.isnan(a) & np.isnan(b))
    with np.errstate(invalid="ignore"):
        near = np.abs(a - b) <= abs_ + rel * np.abs(b)
    return same | near


@pytest.mark.parametrize("name", ["c0", "c1", "m03"])
def test_queries_match_golden(name):
    q = np.load(os.path.join(GOLD, f"queries_{name}.npz"))
    gen = _gen([load_scene(name)], 64)
    dev = "cuda:0"
    xyz, ref = gen.query_snap(0, torch.from_numpy(q["snap_in"]).to(dev))
    assert np.array_equal(ref.cpu().numpy().view(np.uint32), q["snap_ref"])
    assert _close(xyz.cpu().numpy(), q["snap_xyz"], 0, 1e-5).all()
    xyz, ref = gen.query_try_step(0, torch.from_numpy(q["step_start"]).to(dev),
                                  torch.from_numpy(q["step_start_ref"].view(np.int32)).to(dev),
                                  torch.from_numpy(q["step_end"]).to(dev))
    assert np.array_equal(ref.cpu().numpy().view(np.uint32), q["step_ref"])
    assert _close(xyz.cpu().numpy(), q["step_xyz"], 0, 1e-5).all()
    d, st = gen.query_geodesic(0, torch.from_numpy(q["geo_a"]).to(dev),
                               torch.from_numpy(q["geo_a_ref"].view(np.int32)).to(dev),
                               torch.from_numpy(q["geo_b"]).to(dev),
                               torch.from_numpy(q["geo_b_ref"].view(np.int32)).to(dev))
    d = d.cpu().numpy()
    assert np.array_equal(np.isinf(d), np.isinf(q["geo_dist"]))
    assert _close(d, q["geo_dist"], 1e-4).all()
    # the arithmetic is ordered like the reference's: expect bit-exact, report if not
    exact = (d == q["geo_dist"]).mean()
    assert exact > 0.999, f"only {exact:.4f} of geodesic distances are bit-exact"
    gen.close()


@pytest.mark.parametrize("fname,host_actions", [("c0_traj.npz", True), ("c0_policy_traj.npz", False),
                                                ("c0_traj.npz", "pinned")])
def test_trajectory_matches_golden(fname, host_actions):
    # actions as numpy rows (validated and staged by the call), as rows of a CUDA tensor, or as
    # rows of a tensor in page-locked host memory that the kernels read in place
    g = np.load(os.path.join(GOLD, fname))
    actions = g["actions"].astype(np.int64)
    steps, n = actions.shape
    gen = _gen([load_scene("c0")], n, seed=int(g["seed"]))
    gen.reset(0)
    assert _close(gen.get_polars(0), g["polar0"], 0, 1e-5).all()
    snaps = set(int(s) for s in g["snap_steps"])

    def check_state(k):
        torch.cuda.synchronize()
        for name, key in [("nav_poly", "nav_poly"), ("goal_poly", "goal_poly"), ("step", "step"),
                          ("episode", "episode"), ("reset_count", "reset_count")]:
            got = gen.tensor(0, name).cpu().numpy().view(np.uint32)
            assert np.array_equal(got, g[f"s{k}_{key}"]), f"step {k}: {name}"
        for name, key in [("position", "position"), ("rotation", "rotation"), ("goal", "goal"),
                          ("nav_position", "nav_position")]:
            got = gen.tensor(0, name).cpu().numpy().T
            assert _close(got, g[f"s{k}_{key}"], 0, 1e-5).all(), f"step {k}: {name}"
        for name, key in [("prev_dist", "prev_dist"), ("cum_travel", "cum_travel"),
                          ("init_dist", "init_dist")]:
            got = gen.tensor(0, name).cpu().numpy()
            assert _close(got, g[f"s{k}_{key}"], 1e-4, 1e-6).all(), f"step {k}: {name}"

    check_state(0)
    dact = torch.from_numpy(actions).cuda()
    pact = torch.from_numpy(actions).pin_memory()
    for t in range(steps):
        if host_actions == "pinned":
            gen.step(0, pact[t])
        elif host_actions:
            gen.step(0, actions[t])
        else:
            gen.step(0, dact[t])
        assert np.array_equal(gen.get_masks(0), g["mask"][t]), f"mask, step {t}"
        info = gen.get_infos(0)
        assert np.array_equal(info["success"], g["info"][t, :, 0]), f"success, step {t}"
        assert _close(info["spl"], g["info"][t, :, 1], 1e-4, 1e-6).all(), f"spl, step {t}"
        assert _close(info["distanceToGoal"], g["info"][t, :, 2], 1e-4, 1e-6).all(), f"dist, step {t}"
        assert _close(gen.get_rewards(0), g["reward"][t], 1e-4, 1e-5).all(), f"reward, step {t}"
        assert _close(gen.get_polars(0), g["polar"][t], 0, 1e-5).all(), f"polar, step {t}"
        if (t + 1) in snaps:
            check_state(t + 1)
    assert int(gen.tensor(0, "status").cpu().numpy().view(np.uint32).max() & 0xA0) == 0
    # running episode statistics kept on the device == PPOTrainer._update_stats
    # (bps_nav/rl/ppo/ppo_trainer.py:286-319) replayed in float32 on the golden outputs
    cur = np.zeros(n, np.float32)
    acc = np.zeros((5, n), np.float32)
    for t in range(steps):
        cur = cur + g["reward"][t]
        done = g["mask"][t] == 0
        acc[0] += np.where(done, cur, np.float32(0))
        acc[1] += done.astype(np.float32)
        for k in range(3):
            acc[2 + k] += np.where(done, g["info"][t, :, k], np.float32(0))
        cur = np.where(done, np.float32(0), cur)
    got = gen.tensor(0, "episode_stats").cpu().numpy()
    assert np.array_equal(got[1], acc[1]) and np.array_equal(got[2], acc[2])
    assert _close(got, acc, 1e-4, 1e-5).all()
    assert _close(gen.tensor(0, "episode_reward").cpu().numpy(), cur, 1e-4, 1e-5).all()
    gen.close()


@pytest.mark.parametrize("tag", ["small", "c2"])
def test_gae_matches_reference_python(tag):
    from bps_nav_b200 import rollout
    g = np.load(os.path.join(GOLD, "gae_ref.npz"))
    rewards = torch.from_numpy(g[f"{tag}_rewards"]).cuda()
    values = torch.from_numpy(g[f"{tag}_values"]).cuda()
    masks = torch.from_numpy(g[f"{tag}_masks"]).cuda()
    nv = torch.from_numpy(g[f"{tag}_next_value"]).cuda()
    T = rewards.shape[0] - 1
    returns = torch.zeros_like(rewards)
    adv = torch.empty(T, rewards.shape[1], 1, device="cuda")
    rollout.compute_returns(rewards, values, masks, returns, nv, T, 0.99, 0.95, advantages=adv,
                            normalize=False)
    torch.cuda.synchronize()
    ref = g[f"{tag}_returns"]
    got = returns.cpu().numpy()
    assert _close(got[:T], ref[:T], 1e-5, 1e-6).all()
    assert (got[:T] == ref[:T]).mean() > 0.999  # same op order: expect bit-exact
    assert np.array_equal(values[T].cpu().numpy(), g[f"{tag}_next_value"])
    assert _close(adv.cpu().numpy(), g[f"{tag}_adv"], 1e-5, 1e-6).all()
    rollout.compute_returns(rewards, values, masks, returns, nv, T, 0.99, 0.95, advantages=adv,
                            normalize=True)
    torch.cuda.synchronize()
    assert _close(adv.cpu().numpy(), g[f"{tag}_adv_norm"], 1e-5, 2e-6).all()


def _c2():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_fixtures",
                                                  os.path.join(GOLD, "make_fixtures.py"))
    mf = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mf)
    r, v, m, nv = mf.gae_c2_inputs()
    return r, v, m, nv, np.load(os.path.join(GOLD, "gae_c2_16384.npz"))


def _c2_device(r, v, m, nv):
    rewards = torch.from_numpy(r)[..., None].cuda()
    values = torch.from_numpy(v)[..., None].cuda()
    masks = torch.from_numpy(m)[..., None].cuda()
    next_value = torch.from_numpy(nv)[:, None].cuda()
    return rewards, values, masks, next_value


def test_gae_config2_full_size_matches_reference_python():
    """Benchmark config 2 (T = 32, N = 16384): every element against the oracle restatement
    (itself pinned to the reference's output bit for bit, CRC-32 over the whole arrays), the
    reference's own values on every 16th environment, and the CRC of the whole returns array."""
    import zlib
    from bps_nav_b200 import rollout
    from oracle import pyoracle
    r, v, m, nv, g = _c2()
    T, N = 32, 16384
    rewards, values, masks, next_value = _c2_device(r, v, m, nv)
    returns = torch.zeros_like(rewards)
    adv = torch.empty(T, N, 1, device="cuda")
    rollout.compute_returns(rewards, values, masks, returns, next_value, T, 0.99, 0.95,
                            advantages=adv, normalize=False)
    torch.cuda.synchronize()
    ref_ret, ref_adv, _ = pyoracle.gae_reference(r, v, m, nv, 0.99, 0.95)
    got = returns[:T, :, 0].cpu().numpy()
    assert _close(got, ref_ret[:T], 1e-5, 1e-6).all()
    assert zlib.crc32(np.ascontiguousarray(got).tobytes()) == int(g["returns_crc"])  # bit-exact
    cols = g["cols"]
    assert np.array_equal(got[:, cols], g["returns_cols"])
    got_adv = adv[..., 0].cpu().numpy()
    assert _close(got_adv, ref_adv, 1e-5, 1e-6).all()
    assert zlib.crc32(np.ascontiguousarray(got_adv).tobytes()) == int(g["adv_crc"])
    rollout.compute_returns(rewards, values, masks, returns, next_value, T, 0.99, 0.95,
                            advantages=adv, normalize=True)
    torch.cuda.synchronize()
    _, ref_advn, _ = pyoracle.gae_reference(r, v, m, nv, 0.99, 0.95, normalize=True)
    got_advn = adv[..., 0].cpu().numpy()
    assert _close(got_advn, ref_advn, 1e-5, 2e-6).all()
    assert _close(got_advn[:, cols], g["adv_norm_cols"], 1e-5, 2e-6).all()


def test_advantage_normalisation_over_ranges_and_buffers():
    """bpsn_adv_normalize against the torch formula of PPO.get_advantages
    (bps_nav/rl/ppo/ppo.py:190-201): (a) per range of 4096 environments -- also against the
    values the fixture script computed beside the reference's own returns --, (b) the two halves
    of a double-buffered rollout normalised together, as torch.cat(advantages, 1) is, (c) ragged
    ranges that do not cover the batch."""
    from bps_nav_b200 import rollout
    from oracle import pyoracle
    r, v, m, nv, g = _c2()
    T, N = 32, 16384
    _, ref_adv, _ = pyoracle.gae_reference(r, v, m, nv, 0.99, 0.95)
    base = torch.from_numpy(ref_adv)  # float32 [T, N], CPU

    def torch_norm(a):
        return (a - a.mean()) / (a.std() + 1e-5)

    # (a)
    adv = base.clone()[..., None].cuda()
    ranges = [(s, s + 4096) for s in range(0, N, 4096)]
    rollout.normalize_advantages(adv, ranges=ranges)
    want = torch.cat([torch_norm(base[:, s:e]) for s, e in ranges], 1).numpy()
    got = adv[..., 0].cpu().numpy()
    assert _close(got, want, 1e-5, 2e-6).all()
    assert _close(got[:, g["cols"]], g["adv_range_norm_cols"], 1e-5, 2e-6).all()
    # (b)
    a0 = base[:, :N // 2].contiguous().cuda()
    a1 = base[:, N // 2:].contiguous().cuda()
    rollout.normalize_advantages([a0, a1])
    want = torch_norm(base).numpy()
    assert _close(a0.cpu().numpy(), want[:, :N // 2], 1e-5, 2e-6).all()
    assert _close(a1.cpu().numpy(), want[:, N // 2:], 1e-5, 2e-6).all()
    assert _close(a0.cpu().numpy()[:, g["cols"][g["cols"] < N // 2]],
                  g["adv_norm_cols"][:, g["cols"] < N // 2], 1e-5, 2e-6).all()
    # (c) ragged ranges; columns outside every range stay as they were
    adv = base.clone().cuda()
    ragged = [(0, 1), (5, 1000), (1000, 1003), (9000, 16384)]
    rollout.normalize_advantages(adv, ranges=ragged)
    got = adv.cpu().numpy()
    want = base.clone()
    for s, e in ragged:
        if e - s > 1:
            want[:, s:e] = torch_norm(base[:, s:e])
    for s, e in ragged:
        if e - s > 1:
            assert _close(got[:, s:e], want[:, s:e].numpy(), 1e-5, 2e-6).all(), (s, e)
    assert np.array_equal(got[:, 1:5], base[:, 1:5].numpy())
    assert np.array_equal(got[:, 1003:9000], base[:, 1003:9000].numpy())
    # argument checking: overlapping ranges, empty range, CPU tensor
    with pytest.raises(RuntimeError, match="overlap"):
        rollout.normalize_advantages(adv, ranges=[(0, 10), (5, 20)])
    with pytest.raises(RuntimeError, match="start < end"):
        rollout.normalize_advantages(adv, ranges=[(7, 7)])
    with pytest.raises(RuntimeError, match="CUDA"):
        rollout.normalize_advantages(base.clone())


def test_ema_mean_baseline_matches_ddppo_formula():
    """bpsn_adv_mean + bpsn_adv_ema_shift against the recurrences of
    DecentralizedDistributedMixin._get_advantages_distributed (bps_nav/rl/ddppo/algo/ddppo.py:
    46-64) evaluated with torch on the CPU over three successive updates, single worker and
    with a stand-in for the all-reduce over two workers."""
    from bps_nav_b200 import rollout
    rng = np.random.default_rng(5)
    T, N = 32, 2048
    updates = [torch.from_numpy((rng.standard_normal((T, N)) * (k + 1) + 0.3 * k).astype(np.float32))
               for k in range(3)]
    for workers in (1, 2):
        ema = rollout.EmaMeanBaseline("cuda", beta=0.8)
        biased = torch.tensor(0.0)
        unbias = torch.tensor(0.0)
        for a in updates:
            other = torch.tensor(0.25)  # the second worker's mean

            def all_reduce(mean_dev):
                mean_dev.add_(other.item()).div_(2)

            halves = [a[:, :N // 2].contiguous().cuda(), a[:, N // 2:].contiguous().cuda()]
            ema(halves, all_reduce=all_reduce if workers == 2 else None)
            mean = a.mean()
            if workers == 2:
                mean = (mean + other) / 2
            biased = biased * 0.8 + (1 - 0.8) * mean
            unbias = unbias * 0.8 + (1 - 0.8)
            want = (a - biased / unbias).numpy()
            got = np.concatenate([h.cpu().numpy() for h in halves], 1)
            assert _close(got, want, 1e-5, 2e-6).all()
        st = ema.state.cpu().numpy()
        assert abs(st[0] - float(biased)) < 1e-6 and abs(st[1] - float(unbias)) < 1e-6


def test_exact_sqrt_is_ieee_for_every_float():
    """The hand-written square root of the navmesh queries returns sqrtf's bits for every
    fp32 operand (all 2^32 bit patterns: zero, denormals, normals, inf, NaN, negatives)."""
    import ctypes as C
    from bps_nav_b200 import _lib as L
    lib = L.load()
    bad = C.c_uint64(1)
    L.check(lib.bpsn_selftest_sqrt(0, 0x00000000, 0xFFFFFFFF, C.byref(bad)))
    assert bad.value == 0
