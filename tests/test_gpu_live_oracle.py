"""GPU parity against the oracle run live on the same box (the reference's compiled PathFinder
under the simulator restatement).  Skipped when oracle/_ref is not present.

Same tolerances as test_gpu_parity.py: integer outputs bit-exact, poses 1e-5 m, geodesic / reward
1e-4 relative, polar 1e-5.
"""
import numpy as np
import pytest

from conftest import load_scene, scene_path

from oracle import pyoracle

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not pyoracle.available(), reason="oracle libraries not built")]

torch = pytest.importorskip("torch")


def _close(a, b, rel, abs_=0.0):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    same = (a == b) | (np.isnan(a) & np.isnan(b))
    with np.errstate(invalid="ignore"):
        near = np.abs(a - b) <= abs_ + rel * np.abs(b)
    return same | near


def _compare_run(scene_names, n, steps, seed, mix, threads=8, check_state_every=16,
                 search_count=None, want_status=0, num_active=None, visited=None,
                 force_batched=None, actions=None, exact_done=None, **gen_kw):
    """Steps the CUDA generator and the CPU oracle side by side and compares every output of
    every step.  ``num_active``: fewer scenes in use than the list has, the others rotate in;
    ``visited`` (a set) then collects the scenes the environments were seen in."""
    from bps_nav_b200 import bps_sim
    scenes = [load_scene(s) for s in scene_names]
    gen = bps_sim.PointNavRolloutGenerator.from_scenes(scenes, n, seed=seed,
                                                       num_active_scenes=num_active, **gen_kw)
    if search_count is not None:
        for g in range(gen.num_groups):
            gen.debug_set_search_count(g, search_count)
    if force_batched is not None:
        for g in range(gen.num_groups):
            gen.debug_force_batched(g, force_batched)
    osim = pyoracle.OracleSim([(scene_path(s), sc.episodes) for s, sc in zip(scene_names, scenes)],
                              n, seed, threads=threads,
                              active_scenes=gen._active_scenes if num_active else None,
                              num_groups=gen.num_groups,
                              swap_interval=gen_kw.get("swap_interval", 0))
    groups = gen.num_groups
    B = gen.envs_per_group
    for g in range(groups):
        gen.reset(g)
    osim.reset()
    pol = np.concatenate([gen.get_polars(g) for g in range(groups)])
    assert _close(pol, osim.polars, 0, 1e-5).all()
    if actions is None:
        actions = pyoracle.philox_actions(steps, n, seed + 99, mix)
    ties = 0
    for t in range(steps):
        for g in range(groups):
            gen.step(g, actions[t, g * B:(g + 1) * B])
        assert osim.step(actions[t]) == 0
        mask = np.concatenate([gen.get_masks(g) for g in range(groups)])
        info = np.concatenate([gen.get_infos(g) for g in range(groups)])
        rew = np.concatenate([gen.get_rewards(g) for g in range(groups)])
        pol = np.concatenate([gen.get_polars(g) for g in range(groups)])
        assert np.array_equal(mask, osim.masks), f"mask, step {t}"
        assert np.array_equal(info["success"], osim.infos[:, 0]), f"success, step {t}"
        assert _close(info["spl"], osim.infos[:, 1], 1e-4, 1e-6).all(), f"spl, step {t}"
        assert _close(info["distanceToGoal"], osim.infos[:, 2], 1e-4, 1e-6).all(), f"dist, step {t}"
        if exact_done is not None:  # [episode ends, of which the distance matches bit for bit]
            ended = mask == 0
            exact_done[0] += int(ended.sum())
            exact_done[1] += int((info["distanceToGoal"][ended].view(np.uint32) ==
                                  osim.infos[ended, 2].astype(np.float32).view(np.uint32)).sum())
        assert _close(rew, osim.rewards, 1e-4, 1e-5).all(), f"reward, step {t}"
        assert _close(pol, osim.polars, 0, 1e-5).all(), f"polar, step {t}"
        if (t + 1) % check_state_every == 0 or t + 1 == steps:
            torch.cuda.synchronize()
            st = osim.state()
            for name in ("nav_poly", "goal_poly", "step", "episode", "reset_count"):
                got = np.concatenate([gen.tensor(g, name).cpu().numpy().view(np.uint32)
                                      for g in range(groups)])
                assert np.array_equal(got, st[name]), f"{name}, step {t}"
            for name in ("position", "rotation", "nav_position"):
                got = np.concatenate([gen.tensor(g, name).cpu().numpy().T for g in range(groups)])
                assert _close(got, st[name], 0, 1e-5).all(), f"{name}, step {t}"
            if num_active:
                want_scene, want_swaps = osim.scenes()
                got_scene = np.concatenate([gen.tensor(g, "scene").cpu().numpy()
                                            for g in range(groups)])
                assert np.array_equal(got_scene, want_scene), f"scene of the envs, step {t}"
                rate, in_use, per_scene = gen.swap_stats
                assert abs(rate - 100.0 * want_swaps / ((t + 1) * n)) < 1e-9
                per_group = [len(set(want_scene[g * B:(g + 1) * B])) for g in range(groups)]
                assert in_use == sum(per_group)
                assert abs(per_scene - sum(B / k for k in per_group)) < 1e-3
                if visited is not None:
                    visited.update(int(x) for x in want_scene)
    status = np.concatenate([gen.tensor(g, "status").cpu().numpy().view(np.uint32)
                             for g in range(groups)])
    ties = int(((status >> 8) & 1).sum())
    assert int(np.bitwise_or.reduce(status) & 0xA0) == 0  # no iteration cap, no bad action
    assert int(np.bitwise_or.reduce(status)) & want_status == want_status
    assert all(gen.device_errors(g) == 0 for g in range(groups))
    gen.close()
    osim.close()
    return ties


def test_single_scene_large_batch_uniform_actions():
    # benchmark config 1 shape; 4096 envs also exercise the exact-heap fallback on open-list ties
    _compare_run(["c1"], 4096, 96, seed=321, mix="uniform")


def test_single_scene_policy_like_actions_long_episodes():
    _compare_run(["c1"], 1024, 600, seed=17, mix="policy", check_state_every=100)


def test_mixed_scene_batch():
    # benchmark config 3 shape, scaled: 16 scenes, envs split scene-major
    names = [f"m{i:02d}" for i in range(16)]
    _compare_run(names, 2048, 64, seed=5, mix="uniform")
    _compare_run(names, 512, 300, seed=6, mix="policy", check_state_every=100)


def test_generic_kernel_matches_oracle():
    _compare_run(["c1"], 512, 64, seed=11, mix="uniform", generic_kernel=True)
    _compare_run(["m01", "m04"], 256, 128, seed=12, mix="policy", generic_kernel=True)


def test_exact_heap_search_matches_oracle():
    # every A* search through the shared-memory binary heap (normally only after a tie)
    assert _compare_run(["c1"], 2048, 64, seed=23, mix="uniform", exact_heap=True) > 0
    _compare_run(["m03", "m07"], 512, 128, seed=24, mix="policy", exact_heap=True)


def test_scenes_in_shared_and_in_global_memory_in_one_step():
    # with the shared-memory budget cut to 96 KB the larger scenes (m04: 1304 polygons, m07, m01)
    # do not fit and are worked on in global memory (slabs of three different sizes side by
    # side), the small ones in shared memory, in the same group and launch
    _compare_run(["m04", "m13", "m07", "m15", "m01", "c0"], 1536, 64, seed=41, mix="uniform",
                 small_smem=True)


def test_everything_in_global_memory():
    # the global-only instance of the step kernel (two CTAs per SM) on scenes that would fit
    # shared memory
    _compare_run(["c1"], 2048, 48, seed=31, mix="uniform", global_memory=True)
    _compare_run(["m03", "m10", "c0", "m12"], 1024, 96, seed=32, mix="policy", global_memory=True,
                 check_state_every=32)


def test_open_list_ties_resolved_in_place():
    # long episodes on a grid-aligned scene produce a tie for the minimum every other step at
    # this batch; most are two-way ties whose order cannot matter and are expanded in place
    # (status bit 10), the rest are redone on the slab heap (bit 8): results as the oracle's
    _compare_run(["c1"], 4096, 160, seed=91, mix="policy", threads=16, check_state_every=40,
                 want_status=(1 << 10))
    _compare_run(["d0"], 2048, 60, seed=92, mix="policy", threads=16, check_state_every=20,
                 want_status=(1 << 10) | (1 << 8))


def test_sixty_four_scene_slots():
    # the widest configuration the benchmark names: 64 scene slots in one group (the 16 mixed
    # floor plans, each loaded four times), first with every scene in shared memory, then at a
    # batch that is large enough for the planner to move the group to global memory
    names = [f"m{i:02d}" for i in range(16)] * 4
    _compare_run(names, 4096, 24, seed=64, mix="uniform", threads=16, check_state_every=8)
    _compare_run(names, 16384, 12, seed=65, mix="uniform", threads=16, check_state_every=6)


def test_dense_scene_16k_polygons():
    # 16407 polygons: the tables (and 394 KB of nodes per warp) stay in global memory; paths
    # of up to 30 m cross a few hundred polygons
    _compare_run(["d0"], 1024, 48, seed=77, mix="uniform", threads=16)
    _compare_run(["d0"], 256, 32, seed=78, mix="uniform", threads=16, generic_kernel=True)
    _compare_run(["d0", "c0"], 512, 200, seed=79, mix="policy", threads=16, check_state_every=50)


def test_global_memory_search_numbering_wraps():
    # Node arrays in global memory are not wiped between searches: a node is "visited" when it
    # carries the number of the running search.  Start every array's numbering just below the
    # 15-bit limit, so that each wraps (and is wiped once) within a few steps; the arrays hold
    # the marks of earlier searches at that point.
    _compare_run(["c1"], 2048, 24, seed=33, mix="uniform", global_memory=True)  # fresh numbering
    _compare_run(["c1"], 4096, 96, seed=34, mix="uniform", global_memory=True, search_count=32760)
    _compare_run(["m04", "m13", "m07", "c0"], 2048, 96, seed=35, mix="uniform", small_smem=True,
                 search_count=32764)


def test_mixed_scene_batch_large_enough_for_the_throughput_plan():
    # benchmark config 3 at a batch where the planner moves every scene with room for fewer
    # than 8 slabs (m01, m04, m06, m07) to global memory
    names = [f"m{i:02d}" for i in range(16)]
    _compare_run(names, 12288, 24, seed=9, mix="uniform", check_state_every=8)


def test_benchmark_config1_at_full_length():
    # config 1 as the benchmark states it: scene c1, 4096 environments, 1000 steps, uniform
    # actions, every step of every environment compared; then the policy-like mix (long episodes)
    _compare_run(["c1"], 4096, 1000, seed=101, mix="uniform", threads=16, check_state_every=100)
    _compare_run(["c1"], 4096, 500, seed=102, mix="policy", threads=16, check_state_every=100)


def test_benchmark_config3_at_full_length():
    # config 3: 16 mixed floor plans, 16384 environments, 2000 steps
    names = [f"m{i:02d}" for i in range(16)]
    _compare_run(names, 16384, 2000, seed=103, mix="uniform", threads=16, check_state_every=250)


def test_dense_scene_at_benchmark_batch():
    # the 16 407-polygon plan at the headline batch size
    _compare_run(["d0"], 4096, 150, seed=104, mix="uniform", threads=16, check_state_every=50)
    _compare_run(["d0"], 4096, 100, seed=105, mix="policy", threads=16, check_state_every=50)


def test_scenes_rotate_through_the_whole_dataset():
    """32 scenes, 8 in use at a time: every slot of 64 environments moves on to a waiting scene
    whenever all of its environments have arrived, each environment following at the end of
    its episode (simulator/simulator.cpp:1063-1154, 1284-1308, 1636-1640).  Every step is
    compared with the oracle, the environments' scenes too, and every scene must get its turn."""
    names = [f"m{i:02d}" for i in range(16)] * 2
    seen = set()
    _compare_run(names, 512, 400, seed=71, mix="uniform", threads=16, check_state_every=8,
                 num_active=8, visited=seen)
    assert seen == set(range(32)), sorted(set(range(32)) - seen)


def test_scenes_rotate_with_two_groups_and_mixed_memory():
    # two groups, each rotating through its own share of the waiting scenes; a 96 KB
    # shared-memory budget puts the larger scenes in global memory, so slots change between
    # shared and global memory as they move from scene to scene
    names = ["c0", "m04", "m13", "c1", "m15", "m07", "m02", "m10", "m01", "m14"]
    seen = set()
    _compare_run(names, 256, 300, seed=72, mix="uniform", threads=16, check_state_every=10,
                 num_active=4, visited=seen, double_buffered=True, small_smem=True)
    assert len(seen) == len(names)
    # long episodes: slots stay between two scenes for many steps
    _compare_run(names, 128, 400, seed=73, mix="policy", threads=16, check_state_every=20,
                 num_active=2, global_memory=True)


def test_scenes_rotate_at_a_set_pace():
    # swap_interval: a group starts at most one move every so many of its steps (the pace of
    # the reference's single background loader) instead of one per slot as soon as the slot is
    # whole; one and two groups, compared with the oracle step by step, scenes and swap
    # statistics included
    names = [f"m{i:02d}" for i in range(12)]
    _compare_run(names, 512, 300, seed=74, mix="uniform", threads=16, check_state_every=10,
                 num_active=4, swap_interval=16)
    _compare_run(names, 512, 300, seed=75, mix="uniform", threads=16, check_state_every=10,
                 num_active=4, swap_interval=5, double_buffered=True)
    from bps_nav_b200 import bps_sim
    scenes = [load_scene(s) for s in names]
    rates = []
    for interval in (0, 16):
        gen = bps_sim.PointNavRolloutGenerator.from_scenes(scenes, 512, seed=74, num_active_scenes=4,
                                                           swap_interval=interval)
        gen.reset(0)
        acts = pyoracle.philox_actions(200, 512, 173, "uniform")
        for t in range(200):
            gen.step(0, acts[t])
        rates.append(gen.swap_stats[0])
        gen.close()
    assert rates[1] < rates[0] and rates[1] <= 100.0 * (200 // 16 + 1) / (200 * 512) + 1e-9


def test_large_batch_finishes_thirty_two_entries_at_a_time():
    # batches that give every warp several entries per step: the warp searches 32 entries,
    # then every lane pulls the string through one corridor and finishes one environment --
    # in shared memory (c1), in global memory (the 16 mixed scenes, d0), and with Flee's rule
    # that only moves need a query
    # (the form is chosen step by step from the number of entries the step before listed;
    # forced here, then left to the choice: the policy-like mix lists enough entries at this
    # size for the choice to switch forms after the first step)
    _compare_run(["c1"], 32768, 24, seed=121, mix="uniform", threads=16, check_state_every=12,
                 force_batched=1)
    _compare_run(["c1"], 20480, 40, seed=122, mix="policy", threads=16, check_state_every=20)
    names = [f"m{i:02d}" for i in range(16)]
    _compare_run(names, 65536, 16, seed=123, mix="uniform", threads=16, check_state_every=8,
                 force_batched=1)


def test_episodes_that_end_without_a_move():
    # An episode that ends on a stop (or on the step limit during a turn) reports the distance
    # goal -> agent from where the agent stands: the last move's search, or, before the first
    # move, the episode table's goal -> start distance -- no search at that step.  Patterns
    # that end episodes at once, after turns only, right after a move and after a move and
    # turns, in shared memory (one launch and two), in global memory and with rotating scenes.
    pattern = np.array([0, 2, 0, 1, 0, 1, 3, 0, 1, 1, 2, 2, 0, 3, 3, 0, 1, 2, 1, 0], np.int64)
    steps = 60
    for names, n, kw in ((["c1"], 2048, {}), (["c1"], 2048, {"two_launches": True}),
                         (["m03", "m11"], 1024, {"global_memory": True}),
                         (["m00", "m03", "m07", "m12"], 1024, {"num_active": 2})):
        t = np.arange(steps)[:, None]
        e = np.arange(n)[None, :]
        actions = pattern[(t + 7 * e) % len(pattern)]
        counts = [0, 0]
        _compare_run(names, n, steps, seed=131, mix="uniform", actions=actions,
                     check_state_every=20, exact_done=counts, **kw)
        assert counts[0] > n * steps // 8
        assert counts[1] >= 0.999 * counts[0], counts


def test_two_launch_step_on_small_batches():
    # small batches of fixed scenes run a step as one launch; the two-launch form (k_pre, then
    # the step kernel on work lists in global memory) must give the same results on them
    _compare_run(["c1"], 4096, 64, seed=111, mix="uniform", threads=16, two_launches=True)
    _compare_run(["c0", "m13", "m15"], 96, 64, seed=112, mix="policy", two_launches=True)


def test_odd_batch_sizes():
    # partial warps in k_pre's warp-aggregated list appends, fewer environments than warps
    for n, seed in ((1, 50), (7, 51), (33, 52), (100, 53)):
        _compare_run(["c0"], n, 40, seed=seed, mix="uniform")
    _compare_run(["m13", "m15", "c0"], 99, 40, seed=54, mix="policy")


def test_double_buffered_groups():
    _compare_run(["c0", "m15", "m13", "m14"], 256, 64, seed=3, mix="uniform", double_buffered=True)


@pytest.mark.parametrize("task,cls_name", [("flee", "FleeRolloutGenerator"),
                                           ("exploration", "ExplorationRolloutGenerator")])
@pytest.mark.parametrize("generic", [False, True])
def test_other_tasks_match_oracle(task, cls_name, generic):
    """Flee and Exploration generators (simulator/simulator.cpp:830-999) on two scenes."""
    from bps_nav_b200 import bps_sim
    names = ["c1", "m10"]
    n, steps, seed = 512, 200, 31
    scenes = [load_scene(s) for s in names]
    gen = getattr(bps_sim, cls_name).from_scenes(scenes, n, seed=seed, generic_kernel=generic)
    osim = pyoracle.OracleSim([(scene_path(s), sc.episodes) for s, sc in zip(names, scenes)], n,
                              seed, threads=8, task=task)
    gen.reset(0)
    osim.reset()
    actions = pyoracle.philox_actions(steps, n, seed + 1, "policy")
    actions[::7] = pyoracle.philox_actions(steps, n, seed + 2, "uniform")[::7]  # some resets
    field = "distanceFromStart" if task == "flee" else "numVisited"
    for t in range(steps):
        gen.step(0, actions[t])
        osim.step(actions[t])
        assert np.array_equal(gen.get_masks(0), osim.masks), f"mask, step {t}"
        info = gen.get_infos(0)
        assert info.dtype.names == (field,)
        if task == "exploration":
            assert np.array_equal(info[field], osim.infos[:, 0]), f"info, step {t}"
            assert np.array_equal(gen.get_rewards(0), osim.rewards), f"reward, step {t}"
        else:
            assert _close(info[field], osim.infos[:, 0], 1e-4, 1e-6).all(), f"info, step {t}"
            assert _close(gen.get_rewards(0), osim.rewards, 1e-4, 1e-5).all(), f"reward, step {t}"
        assert _close(gen.get_polars(0), osim.polars, 0, 1e-5).all(), f"polar, step {t}"
    torch.cuda.synchronize()
    st = osim.state()
    for name in ("nav_poly", "step", "episode", "reset_count"):
        assert np.array_equal(gen.tensor(0, name).cpu().numpy().view(np.uint32), st[name]), name
    assert gen.device_errors(0) == 0
    gen.close()
    osim.close()


def test_step_protocol_errors():
    from bps_nav_b200 import bps_sim
    gen = bps_sim.PointNavRolloutGenerator.from_scenes([load_scene("c0")], 32, seed=1)
    gen.reset(0)
    acts = np.zeros(32, np.int64)
    with pytest.raises(RuntimeError, match="Simulation already done"):
        gen.step_end(0)
    gen.step_start(0, acts)
    with pytest.raises(RuntimeError, match="Not done with previous simulation"):
        gen.step_start(0, acts)
    gen.step_end(0)
    bad = acts.copy()
    bad[5] = 9
    with pytest.raises(RuntimeError, match="Unknown action: 9"):
        gen.step_start(0, bad)
    # a rejected call steps nothing and leaves the generator usable
    before = gen.tensor(0, "step").clone()
    gen.step(0, np.full(32, 2, np.int64))
    assert torch.equal(gen.tensor(0, "step"), before + 1)
    # device-side actions out of range: flagged, pose untouched, no fault
    dact = torch.full((32,), 2, dtype=torch.int64, device="cuda")
    dact[7] = 77
    rot = gen.tensor(0, "rotation").clone()
    gen.step(0, dact)
    torch.cuda.synchronize()
    st = gen.tensor(0, "status").cpu().numpy().view(np.uint32)
    assert st[7] & 0x80 and not (np.delete(st, 7) & 0x80).any()
    assert torch.equal(gen.tensor(0, "rotation")[:, 7], rot[:, 7])
    with pytest.raises(RuntimeError):
        gen.step_start(3, acts)
    gen.close()


def test_rollout_rows_written_by_the_step():
    from bps_nav_b200 import bps_sim
    gen = bps_sim.PointNavRolloutGenerator.from_scenes([load_scene("c0")], 64, seed=2)
    gen.reset(0)
    T = 8
    rewards = torch.zeros(T + 1, 64, 1, device="cuda")
    masks = torch.ones(T + 1, 64, 1, dtype=torch.bool, device="cuda")
    obs = torch.zeros(T + 1, 64, 2, device="cuda")
    acts = pyoracle.philox_actions(T, 64, 4, "uniform")
    for t in range(T):
        gen.step_start(0, acts[t], reward_out=rewards[t], mask_out=masks[t + 1],
                       polar_out=obs[t + 1])
        gen.step_end(0)
        assert np.array_equal(rewards[t, :, 0].cpu().numpy(), gen.get_rewards(0))
        assert np.array_equal(masks[t + 1, :, 0].cpu().numpy(), gen.get_masks(0) != 0)
        assert np.array_equal(obs[t + 1].cpu().numpy(), gen.get_polars(0))
    gen.close()


def test_depth_sensor_matches_cpu_restatement():
    """Depth images of the box-world sensor against the fp32 numpy restatement, after the
    agents have moved and turned for a while (two scenes, wide and square images)."""
    from bps_nav_b200 import bps_sim, bps_pytorch
    for names, n, res in ((["c0"], 32, (64, 64)), (["m03", "m07"], 16, (96, 48))):
        scenes = [load_scene(s) for s in names]
        gen = bps_sim.PointNavRolloutGenerator.from_scenes(scenes, n, seed=77, depth=True,
                                                           render_resolution=res)
        gen.reset(0)
        actions = pyoracle.philox_actions(40, n, 5, "policy")
        for t in range(40):
            gen.step(0, actions[t])  # step() renders, like the reference's
        gen.wait_for_frame(0)
        t = bps_pytorch.make_depth_tensor(gen.depth(0), 0, n, res)
        # the reference's order of dimensions (simulator/pytorch.cpp:36): [B, res[0], res[1]]
        # with res = [width, height]; the memory is `height` rows of `width` pixels
        assert tuple(t.shape) == (n, res[0], res[1])
        img = t.reshape(n, res[1], res[0]).cpu().numpy()
        pos = gen.tensor(0, "position").cpu().numpy().T
        rot = gen.tensor(0, "rotation").cpu().numpy().T
        scn = gen.tensor(0, "scene").cpu().numpy().view(np.uint32)
        assert (img < 1000.0).mean() > 0.3  # the images are not empty
        for e in range(n):
            sc = scenes[int(scn[e])]
            want = pyoracle.depth_reference(pos[e], rot[e], sc.floor, sc.boxes, res[0], res[1])
            assert np.array_equal(img[e], want), f"env {e}: {np.abs(img[e] - want).max()}"
        gen.close()
    # without a render size the entry point refuses and depth() stays a zero-filled stub
    gen = bps_sim.PointNavRolloutGenerator.from_scenes([load_scene("c0")], 8, seed=1)
    gen.reset(0)
    gen.render(0)
    assert float(bps_pytorch.make_depth_tensor(gen.depth(0), 0, 8, (64, 64)).abs().sum()) == 0.0
    gen.close()
