"""The reference-shaped way in: a dataset directory on disk, the constructor with the
reference's positional arguments (simulator/simulator.cpp:1785-1809) and the call sequence of
``construct_envs`` (bps_nav/common/env_utils.py:32-118), which wraps the generator's buffers in
torch tensors once and then only calls ``step_start`` / ``step_end`` / ``render`` /
``wait_for_frame``.  When the bps-nav tree is on the machine (BPS_NAV_REFERENCE, or a directory
named ``reference`` beside the repository) its own ``env_utils.py`` is loaded by path and run
unmodified against this package; otherwise the same sequence is walked by the restatement
below.  Results are compared with the CPU oracle driven with the same scenes, active-scene
selection and actions.
"""
import importlib.util
import os
import sys
import types
from collections import OrderedDict

import numpy as np
import pytest

from conftest import load_scene, scene_path

from oracle import pyoracle

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not pyoracle.available(), reason="oracle libraries not built")]

torch = pytest.importorskip("torch")

NAMES = ["c0", "m13", "m14", "m15", "m02", "m10"]


class _Sync:
    def __init__(self, envs, idx):
        self._envs, self._idx = envs, idx

    def wait(self):
        self._envs.wait_for_frame(self._idx)


def _construct_envs_restated(config, num_worker_groups=4, double_buffered=True):
    """The statements of construct_envs (env_utils.py:32-118), in its order."""
    import bps_sim
    import bps_pytorch
    batch_size = config.SIM_BATCH_SIZE
    episodes_folder = os.path.join(os.path.dirname(
        config.TASK_CONFIG.DATASET.DATA_PATH.format(split=config.TASK_CONFIG.DATASET.SPLIT)),
        "content")
    envs = bps_sim.PointNavRolloutGenerator(
        episodes_folder, "data/scene_datasets", batch_size, num_worker_groups, -1,
        config.SIMULATOR_GPU_ID, config.RESOLUTION, config.COLOR, config.DEPTH, double_buffered,
        config.TASK_CONFIG.SEED, True)
    observations, rewards, masks, infos, syncs = [], [], [], [], []
    for i in range(2 if double_buffered else 1):
        observation = OrderedDict()
        per_group = batch_size // (2 if double_buffered else 1)
        if config.COLOR:
            observation["rgb"] = bps_pytorch.make_color_tensor(
                envs.rgba(i), config.SIMULATOR_GPU_ID, per_group,
                config.RESOLUTION)[..., 0:3].permute(0, 3, 1, 2)
        if config.DEPTH:
            observation["depth"] = bps_pytorch.make_depth_tensor(
                envs.depth(i), config.SIMULATOR_GPU_ID, per_group, config.RESOLUTION).unsqueeze(1)
        observation["pointgoal_with_gps_compass"] = torch.from_numpy(envs.get_polars(i))
        packed_info = envs.get_infos(i)
        info = {k: torch.from_numpy(packed_info[k]).view(-1, 1) for k in packed_info.dtype.names}
        observations.append(observation)
        rewards.append(torch.from_numpy(envs.get_rewards(i)).view(-1, 1))
        masks.append(torch.from_numpy(envs.get_masks(i)).view(-1, 1))
        infos.append(info)
        syncs.append(_Sync(envs, i))
    return envs, observations, rewards, masks, infos, syncs


def _config(root, n, res, depth):
    ns = types.SimpleNamespace
    return ns(SIM_BATCH_SIZE=n, TASK="PointNav", SIMULATOR_GPU_ID=0, RESOLUTION=list(res),
              COLOR=False, DEPTH=depth,
              TASK_CONFIG=ns(SEED=17, DATASET=ns(
                  SPLIT="train",
                  DATA_PATH=os.path.join(root, "data/datasets/pointnav/synth/{split}/{split}.json.gz"))))


@pytest.fixture
def dataset_on_disk(tmp_path, monkeypatch):
    """Six scenes written in the layout the reference reads; cwd is the directory that holds
    ``data/`` (construct_envs names the asset folder relative to it)."""
    from bps_nav_b200 import bps_pytorch, bps_sim, dataset
    scenes = [load_scene(s) for s in NAMES]
    root = str(tmp_path)
    dataset.write_dataset(scenes, os.path.join(root, "data/datasets/pointnav/synth/train/content"),
                          os.path.join(root, "data/scene_datasets"))
    monkeypatch.chdir(root)
    # the names the reference imports
    monkeypatch.setitem(sys.modules, "bps_sim", bps_sim)
    monkeypatch.setitem(sys.modules, "bps_pytorch", bps_pytorch)
    return root, scenes


def _reference_construct_envs():
    root = pyoracle.reference_root()
    if not root:
        return None
    path = os.path.join(root, "bps_nav", "common", "env_utils.py")
    spec = importlib.util.spec_from_file_location("_ref_env_utils", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.construct_envs


def _oracle_for(envs, n):
    # file-name order of the dataset = the order the generator holds its scenes in
    order = sorted(range(len(NAMES)), key=lambda i: f"{NAMES[i]}.json.gz")
    names = [NAMES[i] for i in order]
    return pyoracle.OracleSim([(scene_path(s), load_scene(s).episodes) for s in names], n, 17,
                              threads=8, active_scenes=envs._active_scenes,
                              num_groups=envs.num_groups), names


@pytest.mark.parametrize("which", ["restated", "reference file"])
def test_construct_envs_sequence(dataset_on_disk, which):
    root, _ = dataset_on_disk
    construct = _construct_envs_restated if which == "restated" else _reference_construct_envs()
    if construct is None:
        pytest.skip("bps-nav tree not on this machine")
    n, res = 256, (64, 64)
    envs, observations, rewards, masks, infos, syncs = construct(_config(root, n, res, True))
    assert envs.num_groups == 2 and envs.num_active_scenes == 4 and len(envs._scenes) == 6
    B = n // 2
    for i in range(2):
        assert observations[i]["depth"].shape == (B, 1, 64, 64) and observations[i]["depth"].is_cuda
        assert observations[i]["pointgoal_with_gps_compass"].shape == (B, 2)
        assert rewards[i].shape == (B, 1) and masks[i].dtype == torch.uint8
        assert set(infos[i]) == {"success", "spl", "distanceToGoal"}
    osim, _ = _oracle_for(envs, n)
    # the trainer's loop (bps_nav/rl/ddppo/algo/ddppo_trainer.py:546-558, ppo_trainer.py:245-275)
    for i in range(2):
        envs.reset(i)
        syncs[i].wait()
    osim.reset()
    pol = torch.cat([o["pointgoal_with_gps_compass"] for o in observations]).numpy()
    assert np.allclose(pol, osim.polars, atol=1e-5)
    actions = pyoracle.philox_actions(120, n, 5, "uniform")
    for t in range(120):
        for i in range(2):
            envs.step_start(i, actions[t, i * B:(i + 1) * B])
        for i in range(2):
            envs.step_end(i)
            envs.render(i)
            syncs[i].wait()
        assert osim.step(actions[t]) == 0
        # the tensors made once at construction alias the generator's buffers
        assert np.array_equal(torch.cat(masks).numpy()[:, 0], osim.masks), t
        assert np.allclose(torch.cat(rewards).numpy()[:, 0], osim.rewards, rtol=1e-4, atol=1e-5,
                           equal_nan=True), t
        got = torch.cat([inf["distanceToGoal"] for inf in infos]).numpy()[:, 0]
        assert np.allclose(got, osim.infos[:, 2], rtol=1e-4, atol=1e-6, equal_nan=True), t
        pol = torch.cat([o["pointgoal_with_gps_compass"] for o in observations]).numpy()
        assert np.allclose(pol, osim.polars, atol=1e-5), t
    d = observations[0]["depth"]
    assert torch.isfinite(d).all() and float(d.min()) > 0.0 and float(d.max()) <= 1000.0
    stats = envs.swap_stats
    assert len(stats) == 3 and stats[1] >= 4
    del envs


def test_constructor_argument_forms(dataset_on_disk):
    from bps_nav_b200 import bps_sim
    root, _ = dataset_on_disk
    folder = os.path.join(root, "data/datasets/pointnav/synth/train/content")
    assets = os.path.join(root, "data/scene_datasets")
    # 11 positional arguments (should_set_affinity defaults to true), then all 12
    a = bps_sim.PointNavRolloutGenerator(folder, assets, 64, 2, 4, 0, [64, 64], False, False,
                                         False, 3)
    b = bps_sim.PointNavRolloutGenerator(folder, assets, 64, 2, 4, 0, [64, 64], False, False,
                                         False, 3, False)
    for g in (a, b):
        g.reset(0)
        g.step(0, np.ones(64, np.int64))
    assert np.array_equal(a.get_rewards(0), b.get_rewards(0))
    assert a.get_infos(0).dtype.names == ("success", "spl", "distanceToGoal")
    # the reference aborts on these (simulator.cpp:1503-1508, 1536-1538)
    with pytest.raises(RuntimeError):
        bps_sim.PointNavRolloutGenerator(folder, assets, 64, 3, 4, 0, [64, 64], False, False,
                                         False, 3)      # 64 % 3
    with pytest.raises(RuntimeError):
        bps_sim.PointNavRolloutGenerator(folder, assets, 64, 1, 4, 0, [64, 64], False, False,
                                         True, 3)       # one active scene, two groups
    with pytest.raises(RuntimeError):
        bps_sim.PointNavRolloutGenerator(folder, assets, 64, 8, 4, 0, [64, 64], False, False,
                                         False, 3)      # more active scenes than the dataset has
    a.close()
    b.close()
