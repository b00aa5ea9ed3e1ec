"""Rollout returns and advantages on the GPU, as calls into the C ABI.

* ``compute_returns`` -- ``RolloutStorage.compute_returns``
  (``bps_nav/common/rollout_storage.py:203-219``): GAE reverse scan, fused with the advantage
  ``returns[:T] - value_preds[:T]`` and, optionally, its normalisation over the one buffer given
  (``bpsn_gae``).
* ``normalize_advantages`` -- ``PPO.get_advantages`` (``bps_nav/rl/ppo/ppo.py:190-201``) on one or
  several advantage tensors at once (the reference concatenates the two halves of a
  double-buffered rollout before it takes mean and std), or per range of environments
  (``bpsn_adv_normalize``).
* ``EmaMeanBaseline`` -- what DD-PPO installs instead
  (``DecentralizedDistributedMixin._get_advantages_distributed``,
  ``bps_nav/rl/ddppo/algo/ddppo.py:46-64``): advantages minus the bias-corrected running mean of
  their mean (``bpsn_adv_mean`` / ``bpsn_adv_ema_shift``).

Tensors are laid out as the reference's rollout storage lays them out: ``rewards / value_preds /
returns`` float32 ``[T+1, N, 1]``, ``masks`` bool ``[T+1, N, 1]`` (``rollout_storage.py:83-101``).
There is no CPU implementation: CPU tensors are rejected.
"""
import ctypes as C

import torch

from . import _lib as L

EPS_PPO = 1e-5  # bps_nav/rl/ppo/ppo.py:34

_workspaces = {}


def _device_index(device):
    return device.index if device.index is not None else torch.cuda.current_device()


def _workspace(device, nbytes, kind):
    key = (_device_index(device), kind, nbytes)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _stream(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _check(t, name, dtype):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU implementation)")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _rows_by_envs(t, name, rows):
    """Number of environments of a ``[rows(+), N]`` or ``[rows(+), N, 1]`` tensor."""
    if t.dim() == 3 and t.shape[2] != 1:
        raise RuntimeError(f"{name}: trailing dimension must be 1, got {tuple(t.shape)}")
    if t.dim() not in (2, 3):
        raise RuntimeError(f"{name} must be [rows, N] or [rows, N, 1], got {tuple(t.shape)}")
    if t.shape[0] < rows:
        raise RuntimeError(f"{name} needs at least {rows} rows, got {t.shape[0]}")
    return int(t.shape[1])


def compute_returns(rewards, value_preds, masks, returns, next_value, num_steps, gamma, tau,
                    advantages=None, normalize=False, eps=EPS_PPO):
    """Fills ``returns[:num_steps]`` (and ``value_preds[num_steps] = next_value``) in place.

    If ``advantages`` (float32 ``[num_steps, N, 1]``) is given it receives
    ``returns[:T] - value_preds[:T]``, normalised as ``(a - mean) / (std + eps)`` over all of its
    elements when ``normalize`` is true.  That covers one storage buffer; a double-buffered rollout,
    whose two halves the reference normalises together, calls this once per buffer with
    ``normalize=False`` and then ``normalize_advantages([adv0, adv1])``.
    """
    lib = L.load()
    T = int(num_steps)
    _check(rewards, "rewards", torch.float32)
    _check(value_preds, "value_preds", torch.float32)
    _check(returns, "returns", torch.float32)
    if masks.dtype not in (torch.bool, torch.uint8):
        raise RuntimeError("masks must be bool or uint8")
    if not masks.is_cuda or not masks.is_contiguous():
        raise RuntimeError("masks must be a contiguous CUDA tensor")
    N = _rows_by_envs(rewards, "rewards", T + 1)
    for t, name in ((value_preds, "value_preds"), (masks, "masks"), (returns, "returns")):
        if _rows_by_envs(t, name, T + 1) != N:
            raise RuntimeError(f"{name} has {t.shape[1]} environments, rewards has {N}")
    nv = None
    if next_value is not None:
        nv = next_value.contiguous().float()
        if nv.numel() != N:
            raise RuntimeError("next_value must hold one value per environment")
    adv_ptr = None
    if advantages is not None:
        _check(advantages, "advantages", torch.float32)
        if advantages.numel() != T * N:
            raise RuntimeError("advantages must have num_steps * N elements")
        adv_ptr = advantages.data_ptr()
    elif normalize:
        raise RuntimeError("normalize=True needs the advantages tensor")
    ws = _workspace(rewards.device, lib.bpsn_gae_workspace_bytes(N), "gae")
    L.check(lib.bpsn_gae(rewards.data_ptr(), value_preds.data_ptr(), masks.data_ptr(),
                         nv.data_ptr() if nv is not None else None, returns.data_ptr(), adv_ptr, T,
                         N, float(gamma), float(tau), 1 if normalize else 0, float(eps),
                         ws.data_ptr(), _stream(rewards.device)))
    return returns


def _segments(advantages, ranges, per_range_groups):
    """ctypes segment array for ``advantages`` (one tensor or a list of tensors, each
    ``[T, N]`` / ``[T, N, 1]``) and optional ``ranges`` of environments."""
    tensors = list(advantages) if isinstance(advantages, (list, tuple)) else [advantages]
    if not tensors:
        raise RuntimeError("no advantage tensor given")
    T = int(tensors[0].shape[0])
    segs = []
    for i, a in enumerate(tensors):
        _check(a, f"advantages[{i}]", torch.float32)
        if a.device != tensors[0].device:
            raise RuntimeError("all advantage tensors must be on one device")
        if int(a.shape[0]) != T:
            raise RuntimeError("all advantage tensors must have the same number of steps")
        n = _rows_by_envs(a, f"advantages[{i}]", T)
        if ranges is None:
            segs.append((a.data_ptr(), n, 0, n, 0))
        else:
            if len(tensors) != 1:
                raise RuntimeError("ranges apply to a single advantage tensor")
            for k, (s, e) in enumerate(ranges):
                segs.append((a.data_ptr(), n, int(s), int(e), k if per_range_groups else 0))
    if len(segs) > L.MAX_ADV_SEGMENTS:
        raise RuntimeError(f"at most {L.MAX_ADV_SEGMENTS} segments per call")
    arr = (L.AdvSegment * len(segs))(*[L.AdvSegment(*s) for s in segs])
    return arr, len(segs), T, tensors[0].device


def normalize_advantages(advantages, ranges=None, eps=EPS_PPO):
    """``(a - mean) / (std + eps)`` in place, ``std`` unbiased (``PPO.get_advantages``).

    ``advantages``: one float32 CUDA tensor ``[T, N]`` / ``[T, N, 1]``, or a list of them
    (normalised together, like the reference's ``torch.cat(advantages, 1)`` over the buffers of a
    double-buffered rollout).  ``ranges``: optional list of ``(start, end)`` environment ranges
    of a single tensor; each range is then normalised on its own statistics (per-minibatch
    normalisation over contiguous blocks of environments)."""
    lib = L.load()
    arr, n, T, device = _segments(advantages, ranges, per_range_groups=True)
    ws = _workspace(device, lib.bpsn_adv_workspace_bytes(), "adv")
    L.check(lib.bpsn_adv_normalize(arr, n, T, float(eps), ws.data_ptr(), _stream(device)))
    return advantages


class EmaMeanBaseline:
    """``advantages - EMA(mean(advantages))`` with the bias correction of
    ``bps_nav/rl/ddppo/algo/ddppo.py:46-64`` (``beta = 0.8`` there); the state -- the two
    scalars ``adv_mean_biased`` / ``adv_mean_unbias`` -- lives in a 3-float device tensor.

    ``all_reduce``: optional callable applied to the 1-element device tensor holding this
    worker's mean; it must leave the mean over all workers in it (e.g.
    ``lambda m: (dist.all_reduce(m), m.div_(world_size))``), which is where
    ``distributed_mean_and_var`` (``ddppo.py:18-42``) puts its collective."""

    def __init__(self, device, beta=0.8):
        self.beta = float(beta)
        self.state = torch.zeros(3, dtype=torch.float32, device=device)
        self.mean = torch.zeros(1, dtype=torch.float32, device=device)

    def __call__(self, advantages, all_reduce=None):
        lib = L.load()
        arr, n, T, device = _segments(advantages, None, per_range_groups=False)
        ws = _workspace(device, lib.bpsn_adv_workspace_bytes(), "adv")
        L.check(lib.bpsn_adv_mean(arr, n, T, self.mean.data_ptr(), ws.data_ptr(), _stream(device)))
        if all_reduce is not None:
            all_reduce(self.mean)
        L.check(lib.bpsn_adv_ema_shift(arr, n, T, self.state.data_ptr(), self.mean.data_ptr(),
                                       self.beta, _stream(device)))
        return advantages
