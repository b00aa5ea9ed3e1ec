"""B200-native batch PointGoal-navigation step and rollout returns.

Modules mirror the reference's Python-visible surface for this path:

* ``bps_sim``      -- ``PointNavRolloutGenerator`` (reference: pybind11 module ``bps_sim``,
  ``simulator/simulator.cpp:1785-1823``)
* ``bps_pytorch``  -- capsule <-> CUDA tensor helpers (reference: ``simulator/pytorch.cpp:69-75``)
* ``rollout``      -- ``compute_returns`` / ``get_advantages`` on rollout-storage tensors
  (reference: ``bps_nav/common/rollout_storage.py:203-219``, ``bps_nav/rl/ppo/ppo.py:190-201``)

Everything computes in hand-written CUDA kernels behind the C ABI of ``include/bpsn.h``;
PyTorch is used for tensor hand-off only.
"""
from . import _lib  # noqa: F401

__all__ = ["bps_sim", "bps_pytorch", "rollout", "dataset"]
