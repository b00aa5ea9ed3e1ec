"""Rollout returns on the GPU: GAE reverse scan fused with advantage computation and
whole-batch normalisation, as one call into the C ABI (``bpsn_gae``).

Mirrors ``RolloutStorage.compute_returns`` (``bps_nav/common/rollout_storage.py:203-219``) and
``PPO.get_advantages`` (``bps_nav/rl/ppo/ppo.py:190-201``) on tensors laid out as the reference's
rollout storage lays them out: ``rewards / value_preds / returns`` float32 ``[T+1, N, 1]``,
``masks`` bool ``[T+1, N, 1]`` (``rollout_storage.py:83-101``).
"""
import ctypes as C

import torch

from . import _lib as L

EPS_PPO = 1e-5  # bps_nav/rl/ppo/ppo.py:34

_workspaces = {}


def _workspace(device, n):
    lib = L.load()
    need = lib.bpsn_gae_workspace_bytes(n)
    key = (device.index, need)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _check(t, name, dtype):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU implementation)")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def compute_returns(rewards, value_preds, masks, returns, next_value, num_steps, gamma, tau,
                    advantages=None, normalize=False, eps=EPS_PPO):
    """Fills ``returns[:num_steps]`` (and ``value_preds[num_steps] = next_value``) in place.

    If ``advantages`` (float32 ``[num_steps, N, 1]``) is given it receives
    ``returns[:T] - value_preds[:T]``, normalised as ``(a - mean) / (std + eps)`` over all
    elements when ``normalize`` is true.
    """
    lib = L.load()
    T = int(num_steps)
    N = rewards.shape[1]
    _check(rewards, "rewards", torch.float32)
    _check(value_preds, "value_preds", torch.float32)
    _check(returns, "returns", torch.float32)
    if masks.dtype not in (torch.bool, torch.uint8):
        raise RuntimeError("masks must be bool or uint8")
    if not masks.is_cuda or not masks.is_contiguous():
        raise RuntimeError("masks must be a contiguous CUDA tensor")
    if rewards.shape[0] < T + 1 or value_preds.shape[0] < T + 1 or masks.shape[0] < T + 1:
        raise RuntimeError("rollout tensors need at least num_steps + 1 rows")
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
    ws = _workspace(rewards.device, N)
    stream = C.c_void_p(torch.cuda.current_stream(rewards.device).cuda_stream)
    L.check(lib.bpsn_gae(rewards.data_ptr(), value_preds.data_ptr(), masks.data_ptr(),
                         nv.data_ptr() if nv is not None else None, returns.data_ptr(), adv_ptr, T,
                         N, float(gamma), float(tau), 1 if normalize else 0, float(eps),
                         ws.data_ptr(), stream))
    return returns
