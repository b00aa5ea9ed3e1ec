"""Multi-GPU plumbing for the environment shards: one process per GPU, no data-path collective.

Environments never interact (reference: ``simulator/simulator.cpp:1626-1644`` touches one env per
work item; DD-PPO runs one generator per rank with a rank-offset seed,
``bps_nav/rl/ddppo/algo/ddppo_trainer.py:354-359``), so ranks only meet for a start barrier and to
agree on the slowest rank's time.
"""
import os


def rank_info():
    """(rank, world_size, local_rank) from the torchrun environment (defaults: single process)."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def shard_seed(base_seed, rank, envs_per_rank):
    """Seed of a rank's generator: ``base + rank * envs_per_rank`` as the reference offsets it."""
    return int(base_seed) + int(rank) * int(envs_per_rank)


def max_over_ranks(value, device=None):
    """Maximum of a python float over all ranks (identity when not distributed)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value, device=None):
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def shard_plan(num_envs, num_scenes, rank, world):
    """Block partition of a fixed global batch over ``world`` ranks.

    The global batch has ``num_envs`` environments in scene-major order, ``num_envs /
    num_scenes`` consecutive environments per scene (the reference's layout,
    ``simulator/simulator.cpp:1205-1221``).  Rank ``r`` owns environments
    ``[r * num_envs / world, (r + 1) * num_envs / world)`` and needs only the scenes that block
    touches.  Returns ``(first_env, count, scene_ids, env_scene)``: the block, the global indices
    of the scenes to load on this rank (ascending) and, for every environment of the block, the
    position of its scene in ``scene_ids``."""
    num_envs, num_scenes, rank, world = int(num_envs), int(num_scenes), int(rank), int(world)
    if num_envs % world or num_envs % num_scenes:
        raise ValueError("num_envs must be a multiple of the number of ranks and of scenes")
    per_scene = num_envs // num_scenes
    count = num_envs // world
    first = rank * count
    scene_of = [(first + i) // per_scene for i in range(count)]
    scene_ids = sorted(set(scene_of))
    local = {s: k for k, s in enumerate(scene_ids)}
    return first, count, scene_ids, [local[s] for s in scene_of]
