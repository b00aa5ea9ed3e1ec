"""Drop-in for the reference's ``bps_sim`` extension module (PointNav, Flee and Exploration
generators).

Class and method names, argument order and meaning follow the pybind11 bindings at
``simulator/simulator.cpp:1785-1823`` (``RolloutGenerator`` at ``:1332-1460``).  The work that the
reference fans out over CPU threads (``:1619-1653``) is done by CUDA kernels behind the C ABI of
``include/bpsn.h``.

Kept from the reference:

* constructor signature, and ``step / step_start / step_end / render / reset / rgba / depth /
  get_rewards / get_masks / get_infos / get_polars / wait_for_frame / swap_stats``;
* ``get_*`` return numpy arrays that alias fixed host buffers for the life of the generator
  (``makeFlatNumpyArray``, ``:1001-1009``) and are up to date when ``step_end`` returns;
* environment order: group-major, then ``num_environments / num_active_scenes`` consecutive
  environments per scene (``:1205-1221, 1581-1592``);
* after a finished episode the environment is reset inside the same step: reward / mask / info
  describe the terminal transition, polar the first state of the new episode (``:1636-1642``).

Added (not in the reference): device-resident views of every result and state array
(``tensor(group, name)``), and ``step_start`` accepting a CUDA int64 tensor of actions, so a
trainer can keep the whole rollout on the GPU.

Not reproduced: the colour renderer (``rgba`` exposes a zero-filled device buffer; ``depth`` is
the analytic sensor of box-world scenes).  Scenes rotate through the active slots as in the
reference, with one deterministic rule in place of its background loader's timing (see
``include/bpsn.h``, ``num_active_scenes``).
"""
import ctypes as C

import numpy as np

from . import _lib as L
from . import dataset as _dataset

try:  # compiled binding of the per-step calls (csrc/pyext.c); ctypes does the same, slower
    from . import _bpsn_fast as _fast
except ImportError:
    _fast = None

INFO_DTYPE = np.dtype([("success", "<f4"), ("spl", "<f4"), ("distanceToGoal", "<f4")])
# StepInfo records of the three tasks (simulator/simulator.cpp:738-742, 834-836, 893-895, 1814-1821)
_TASKS = {
    "pointnav": (L.TASK_POINTNAV, INFO_DTYPE),
    "flee": (L.TASK_FLEE, np.dtype([("distanceFromStart", "<f4")])),
    "exploration": (L.TASK_EXPLORATION, np.dtype([("numVisited", "<f4")])),
}

_FIELDS = {
    # name: (field id, numpy dtype, shape as function of B)
    "reward": (L.FIELD_REWARD, np.float32, lambda B: (B,)),
    "mask": (L.FIELD_MASK, np.uint8, lambda B: (B,)),
    "info": (L.FIELD_INFO, np.float32, lambda B: (B, 3)),
    "polar": (L.FIELD_POLAR, np.float32, lambda B: (B, 2)),
    "position": (L.FIELD_POSITION, np.float32, lambda B: (3, B)),
    "rotation": (L.FIELD_ROTATION, np.float32, lambda B: (4, B)),
    "goal": (L.FIELD_GOAL, np.float32, lambda B: (3, B)),
    "nav_position": (L.FIELD_NAV_POSITION, np.float32, lambda B: (3, B)),
    "nav_poly": (L.FIELD_NAV_POLY, np.uint32, lambda B: (B,)),
    "goal_poly": (L.FIELD_GOAL_POLY, np.uint32, lambda B: (B,)),
    "step": (L.FIELD_STEP, np.uint32, lambda B: (B,)),
    "episode": (L.FIELD_EPISODE, np.uint32, lambda B: (B,)),
    "reset_count": (L.FIELD_RESET_COUNT, np.uint32, lambda B: (B,)),
    "status": (L.FIELD_STATUS, np.uint32, lambda B: (B,)),
    "prev_dist": (L.FIELD_PREV_DIST, np.float32, lambda B: (B,)),
    "cum_travel": (L.FIELD_CUM_TRAVEL, np.float32, lambda B: (B,)),
    "init_dist": (L.FIELD_INIT_DIST, np.float32, lambda B: (B,)),
    "scene": (L.FIELD_SCENE, np.uint32, lambda B: (B,)),
    "episode_reward": (L.FIELD_EPISODE_REWARD, np.float32, lambda B: (B,)),
    "episode_stats": (L.FIELD_EPISODE_STATS, np.float32, lambda B: (5, B)),
}


class _DeviceArray:
    """Minimal ``__cuda_array_interface__`` carrier for a raw device pointer (non-owning)."""

    def __init__(self, ptr, shape, dtype):
        self.__cuda_array_interface__ = {
            "shape": tuple(shape), "typestr": np.dtype(dtype).str, "data": (int(ptr), False),
            "version": 3, "strides": None,
        }


def _new_capsule(ptr):
    f = C.pythonapi.PyCapsule_New
    f.restype = C.py_object
    f.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p]
    return f(ptr, None, None)


class _RolloutGenerator:
    _task = None

    def __init__(self, dataset_path, asset_path, num_environments, num_active_scenes, num_workers,
                 gpu_id, render_resolution, color, depth, double_buffered, seed,
                 should_set_affinity=True, *, swap_interval=0):
        # num_workers / should_set_affinity configure the reference's CPU worker pool; a kernel
        # launch replaces that pool, so they are accepted and ignored.  swap_interval (added,
        # keyword only): see from_scenes.
        del num_workers, should_set_affinity
        scenes = _dataset.load_dataset(dataset_path, asset_path)
        self._setup(scenes, num_environments, num_active_scenes, gpu_id, render_resolution, color,
                    depth, double_buffered, seed, host_mirrors=True, swap_interval=swap_interval)

    @classmethod
    def from_scenes(cls, scenes, num_environments, num_active_scenes=None, gpu_id=0,
                    render_resolution=(64, 64), color=False, depth=False, double_buffered=False,
                    seed=0, host_mirrors=True, generic_kernel=False, exact_heap=False,
                    small_smem=False, global_memory=False, env_scene=None, two_launches=False,
                    swap_interval=0):
        """Builds a generator from in-memory ``dataset.Scene`` objects (no JSON involved).
        ``env_scene``: optional explicit scene (index into ``scenes``) of every environment, for
        layouts other than equal consecutive blocks; only with every scene active.
        ``swap_interval``: with fewer active scenes than scenes, steps of a group between two
        scene changes at least (0: a slot changes scene as soon as it is whole again)."""
        self = cls.__new__(cls)
        if num_active_scenes is None:
            num_active_scenes = len(scenes)
        self._setup(list(scenes), num_environments, num_active_scenes, gpu_id, render_resolution,
                    color, depth, double_buffered, seed, host_mirrors, generic_kernel, exact_heap,
                    small_smem, global_memory, env_scene, two_launches, swap_interval)
        return self

    def _setup(self, scenes, num_environments, num_active_scenes, gpu_id, render_resolution, color,
               depth, double_buffered, seed, host_mirrors, generic_kernel=False, exact_heap=False,
               small_smem=False, global_memory=False, env_scene=None, two_launches=False,
               swap_interval=0):
        if self._task not in _TASKS:
            raise NotImplementedError(f"{type(self).__name__}: unknown task")
        self._task_id, self._info_dtype = _TASKS[self._task]
        self._info_width = len(self._info_dtype.names)
        self._lib = L.load()
        self._h = C.c_void_p()
        num_groups = 2 if double_buffered else 1
        if num_active_scenes > len(scenes):
            raise RuntimeError("num_active_scenes exceeds the number of scenes in the dataset")
        # Every scene of the dataset is uploaded (navigation meshes are small); the ones drawn
        # here are in use first and the others rotate in as episodes end (SceneSwapper,
        # simulator/simulator.cpp:1063-1154).  (The reference's assert that the dataset has more
        # scenes than are active, :1516, is compiled out of its RelWithDebInfo build; with equal
        # counts nothing ever rotates, there as here.)
        active, inactive = _dataset.select_active_scenes(len(scenes), num_active_scenes, seed)
        self._active_scenes = active
        self._inactive_scenes = inactive
        self._scenes = list(scenes)
        self.num_active_scenes = int(num_active_scenes)
        self.num_environments = int(num_environments)
        self.num_groups = num_groups
        self.gpu_id = int(gpu_id)
        self._color = bool(color)
        self._depth = bool(depth)
        self._res = (int(render_resolution[0]), int(render_resolution[1]))
        self._host_mirrors = bool(host_mirrors)
        cfg = L.Config(gpu_id=self.gpu_id, num_envs=self.num_environments, num_groups=num_groups,
                       num_scenes=len(self._scenes), seed=int(seed) & (2**64 - 1),
                       flags=(L.FLAG_HOST_MIRRORS if host_mirrors else 0) |
                       (L.FLAG_GENERIC_KERNEL if generic_kernel else 0) |
                       (L.FLAG_EXACT_HEAP if exact_heap else 0) |
                       (L.FLAG_SMEM_96K if small_smem else 0) |
                       (L.FLAG_GLOBAL_MEMORY if global_memory else 0) |
                       (L.FLAG_TWO_LAUNCHES if two_launches else 0),
                       task=self._task_id,
                       render_width=self._res[0] if self._depth else 0,
                       render_height=self._res[1] if self._depth else 0,
                       num_active_scenes=self.num_active_scenes,
                       swap_interval=int(swap_interval))
        L.check(self._lib.bpsn_create(C.byref(cfg), C.byref(self._h)))
        try:
            act = np.ascontiguousarray(active, np.uint32)
            L.check(self._lib.bpsn_set_active_scenes(self._h, act.ctypes.data, len(act)), self._h)
            if env_scene is not None:
                es = np.ascontiguousarray(env_scene, np.uint32)
                L.check(self._lib.bpsn_set_env_scenes(self._h, es.ctypes.data, len(es)), self._h)
            for i, sc in enumerate(self._scenes):
                L.check(self._lib.bpsn_set_navmesh_file(self._h, i, sc.navmesh_path.encode()),
                        self._h)
                eps = np.ascontiguousarray(sc.episodes)
                L.check(self._lib.bpsn_set_episodes(self._h, i, eps.ctypes.data, len(eps)),
                        self._h)
                if self._depth and getattr(sc, "floor", None) is not None:
                    floor = np.asarray(sc.floor, np.float32)
                    boxes = np.ascontiguousarray(sc.boxes, np.float32)
                    L.check(self._lib.bpsn_set_scene_geometry(
                        self._h, i, floor.ctypes.data, boxes.ctypes.data if len(boxes) else None,
                        len(boxes)), self._h)
            L.check(self._lib.bpsn_finalize(self._h), self._h)
        except Exception:
            self._lib.bpsn_destroy(self._h)
            self._h = C.c_void_p()
            raise
        import torch
        self._hv = self._h.value
        self._out_cache = {}
        self._raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or (
            lambda dev: torch.cuda.current_stream(dev).cuda_stream)
        self._group_streams = None
        if num_groups == 2 and host_mirrors:
            with torch.cuda.device(self.gpu_id):
                self._group_streams = [torch.cuda.Stream() for _ in range(num_groups)]
            self._group_stream_ptrs = [st.cuda_stream for st in self._group_streams]
        self.envs_per_group = self.num_environments // num_groups
        self.envs_per_scene = self.num_environments // self.num_active_scenes
        self._num_steps_taken = 0
        self._host_views = {}
        self._dev_tensors = {}
        self._render_bufs = {}
        self._keepalive = []

    # ------------------------------------------------------------------ lifecycle
    def close(self):
        h = getattr(self, "_h", None)
        if h is not None and h.value:
            self._lib.bpsn_destroy(h)
            self._h = C.c_void_p()
            self._hv = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ stepping
    def _stream(self, group_idx=0):
        """The CUDA stream a group's work is enqueued on.  A double-buffered generator with
        host result arrays (the reference's way of use: ``step_end`` returns when the numpy
        arrays are complete) gives each group a stream of its own, so that the two groups'
        steps overlap on the GPU as the reference's two groups overlap on its worker threads
        (simulator/simulator.cpp:1377-1399).  Otherwise work goes to torch's current stream and
        is ordered with the caller's tensor operations."""
        if self._group_streams is not None:
            return C.c_void_p(self._group_streams[group_idx].cuda_stream)
        return self._current_stream()

    def _current_stream(self):
        import torch
        raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)  # same value, less overhead
        if raw is not None:
            return C.c_void_p(raw(self.gpu_id))
        return C.c_void_p(torch.cuda.current_stream(self.gpu_id).cuda_stream)

    def reset(self, group_idx):
        L.check(self._lib.bpsn_reset(self._h, group_idx, self._stream(group_idx)), self._h)

    def step_start(self, group_idx, actions, reward_out=None, mask_out=None, polar_out=None):
        """``actions``: C-contiguous int64 numpy array of length ``envs_per_group`` (reference
        signature: validated and staged by the call), or an int64 tensor of the same length
        that the device can read where it lies -- a CUDA tensor, or a CPU tensor in page-locked
        memory (``pin_memory()``), which the kernels then read over the bus.  A tensor is not
        validated (an out-of-range value marks the environment, which does not move) and must
        stay unchanged until the step has run.

        ``reward_out`` / ``mask_out`` (added): contiguous CUDA tensors of ``envs_per_group``
        float32 / 1-byte elements that also receive this step's reward and mask, e.g.
        ``rollouts.rewards[t]`` and ``rollouts.masks[t + 1]``; ``polar_out``: CUDA float32
        ``[B, 2]`` that also receives the GPS/compass observation (``observations[t + 1]``)."""
        ro = mo = po = None
        if reward_out is not None or mask_out is not None or polar_out is not None:
            # validated once per set of tensor objects (a trainer passes the same row views
            # window after window); the entry keeps them alive, so the ids stay theirs
            key = (id(reward_out), id(mask_out), id(polar_out))
            hit = self._out_cache.get(key)
            if hit is None:
                if len(self._out_cache) > 4096:
                    self._out_cache.clear()
                hit = self._out_ptrs(reward_out, mask_out, polar_out) + (
                    (reward_out, mask_out, polar_out),)
                self._out_cache[key] = hit
            ro, mo, po = hit[0], hit[1], hit[2]
        streams = self._group_streams
        if streams is not None:
            stream = self._group_stream_ptrs[group_idx]
        else:
            stream = self._raw_stream(self.gpu_id)
        if type(actions) is np.ndarray:
            self._keepalive = actions
            if _fast is not None:
                rc = _fast.step_start(self._hv, group_idx, actions, self.envs_per_group, stream,
                                      ro, mo, po)
            else:
                if actions.dtype != np.int64 or not actions.flags.c_contiguous:
                    actions = np.ascontiguousarray(actions, dtype=np.int64)
                if actions.shape[0] != self.envs_per_group:
                    raise RuntimeError("actions length must equal the number of envs in the group")
                self._keepalive = actions
                rc = self._lib.bpsn_step_start_ex(self._h, group_idx,
                                                  actions.__array_interface__["data"][0],
                                                  L.MEM_HOST, stream, ro, mo, po)
        else:
            import torch
            if not (isinstance(actions, torch.Tensor) and actions.dtype == torch.int64 and
                    actions.is_contiguous() and (actions.is_cuda or actions.is_pinned())):
                raise RuntimeError("actions must be an int64 numpy array, a contiguous CUDA "
                                   "int64 tensor or a contiguous int64 tensor in pinned memory")
            if actions.numel() != self.envs_per_group:
                raise RuntimeError("actions length must equal the number of envs in the group")
            self._keepalive = actions
            if _fast is not None:
                rc = _fast.step_start_device(self._hv, group_idx, actions.data_ptr(), stream,
                                             ro, mo, po)
            else:
                rc = self._lib.bpsn_step_start_ex(self._h, group_idx, actions.data_ptr(),
                                                  L.MEM_DEVICE, stream, ro, mo, po)
        if rc:
            L.check(rc, self._h)
        self._num_steps_taken += self.envs_per_group

    def _out_ptrs(self, reward_out, mask_out, polar_out):
        B = self.envs_per_group
        po = polar_out.data_ptr() if polar_out is not None else None
        if polar_out is not None and (polar_out.numel() != 2 * B or polar_out.element_size() != 4 or
                                      not polar_out.is_contiguous() or not polar_out.is_cuda):
            raise RuntimeError("polar_out must be a contiguous CUDA float32 tensor of B x 2")
        ro = reward_out.data_ptr() if reward_out is not None else None
        mo = mask_out.data_ptr() if mask_out is not None else None
        if reward_out is not None and (reward_out.numel() != B or reward_out.element_size() != 4 or
                                       not reward_out.is_contiguous() or not reward_out.is_cuda):
            raise RuntimeError("reward_out must be a contiguous CUDA float32 tensor of B elements")
        if mask_out is not None and (mask_out.numel() != B or mask_out.element_size() != 1 or
                                     not mask_out.is_contiguous() or not mask_out.is_cuda):
            raise RuntimeError("mask_out must be a contiguous CUDA 1-byte tensor of B elements")
        return ro, mo, po

    def step_end(self, group_idx):
        if _fast is not None:
            rc = _fast.step_end(self._hv, group_idx)
        else:
            rc = self._lib.bpsn_step_end(self._h, group_idx)
        if rc:
            L.check(rc, self._h)

    def render(self, group_idx):
        """Renders the depth sensor of the group (when the generator was built with
        ``depth=True``) from the current poses, asynchronously on the current stream;
        otherwise a no-op kept so that call sites need no change.  There is no colour
        renderer: ``rgba`` stays zero-filled."""
        if self._depth:
            L.check(self._lib.bpsn_render(self._h, group_idx, self._stream(group_idx)), self._h)

    def step(self, group_idx, actions):
        self.step_start(group_idx, actions)
        self.step_end(group_idx)
        self.render(group_idx)

    def wait_for_frame(self, group_idx):
        import torch
        if self._group_streams is not None:
            self._group_streams[group_idx].synchronize()
        else:
            torch.cuda.current_stream(self.gpu_id).synchronize()

    # ------------------------------------------------------------------ result views (host)
    def _host_array(self, group_idx, name):
        key = (group_idx, name)
        if key not in self._host_views:
            fid, dt, shape = _FIELDS[name]
            p, n = C.c_void_p(), C.c_size_t()
            L.check(self._lib.bpsn_get_ptr(self._h, group_idx, fid, L.MEM_HOST, C.byref(p),
                                           C.byref(n)), self._h)
            buf = (C.c_uint8 * n.value).from_address(p.value)
            arr = np.frombuffer(buf, dtype=dt).reshape(self._shape(name, shape))
            self._host_views[key] = arr
        return self._host_views[key]

    def _shape(self, name, shape):
        if name == "info":  # [B, 3] for PointNav, [B, 1] for Flee / Exploration
            return (self.envs_per_group, self._info_width)
        return shape(self.envs_per_group)

    def get_rewards(self, group_idx):
        return self._host_array(group_idx, "reward")

    def get_masks(self, group_idx):
        return self._host_array(group_idx, "mask")

    def get_infos(self, group_idx):
        return self._host_array(group_idx, "info").view(self._info_dtype).reshape(-1)

    def get_polars(self, group_idx):
        return self._host_array(group_idx, "polar")

    # ------------------------------------------------------------------ device views (added)
    def tensor(self, group_idx, name):
        """Zero-copy CUDA tensor over a per-group array; names are the keys of ``_FIELDS``
        (``reward mask info polar position rotation goal nav_position nav_poly goal_poly step
        episode reset_count status prev_dist cum_travel init_dist scene episode_reward
        episode_stats``).  uint32 arrays are
        exposed as int32 tensors (same bits)."""
        import torch
        key = (group_idx, name)
        if key not in self._dev_tensors:
            fid, dt, shape = _FIELDS[name]
            p, n = C.c_void_p(), C.c_size_t()
            L.check(self._lib.bpsn_get_ptr(self._h, group_idx, fid, L.MEM_DEVICE, C.byref(p),
                                           C.byref(n)), self._h)
            if dt == np.uint32:
                dt = np.int32
            carrier = _DeviceArray(p.value, self._shape(name, shape), dt)
            self._dev_tensors[key] = torch.as_tensor(carrier, device=f"cuda:{self.gpu_id}")
        return self._dev_tensors[key]

    # ------------------------------------------------------------------ image buffers (stubs)
    def _render_buffer(self, group_idx, kind):
        import torch
        key = (group_idx, kind)
        if key not in self._render_bufs:
            B = self.envs_per_group
            H, W = self._res[1], self._res[0]
            if kind == "rgba":
                t = torch.zeros(B, H, W, 4, dtype=torch.uint8, device=f"cuda:{self.gpu_id}")
            else:
                t = torch.zeros(B, H, W, dtype=torch.float32, device=f"cuda:{self.gpu_id}")
            self._render_bufs[key] = t
        return self._render_bufs[key]

    def rgba(self, group_idx):
        return _new_capsule(self._render_buffer(group_idx, "rgba").data_ptr())

    def depth(self, group_idx):
        if self._depth:  # the library's own float32 [B, H, W] image
            p, n = C.c_void_p(), C.c_size_t()
            L.check(self._lib.bpsn_get_ptr(self._h, group_idx, L.FIELD_DEPTH, L.MEM_DEVICE,
                                           C.byref(p), C.byref(n)), self._h)
            return _new_capsule(p.value)
        return _new_capsule(self._render_buffer(group_idx, "depth").data_ptr())

    # ------------------------------------------------------------------ misc
    @property
    def swap_stats(self):
        # (scene swaps per 100 environment steps, scenes in use, mean envs per scene), the last
        # two summed over the groups, as RolloutGenerator::swapStats (simulator.cpp:1412-1424)
        n, scenes, per = C.c_uint64(), C.c_float(), C.c_float()
        L.check(self._lib.bpsn_swap_stats(self._h, C.byref(n), C.byref(scenes), C.byref(per)),
                self._h)
        steps = max(self._num_steps_taken, 1)
        return (100.0 * n.value / steps, float(scenes.value), float(per.value))

    def device_errors(self, group_idx):
        """Sticky device-side error flags of a group (0 in normal operation); synchronises."""
        v = C.c_uint32()
        L.check(self._lib.bpsn_device_error_flags(self._h, group_idx, C.byref(v)), self._h)
        return int(v.value)

    def debug_set_search_count(self, group_idx, count):
        """Diagnostic: presets the search numbering of the group's global-memory node arrays
        (bpsn_debug_set_search_count), e.g. to just below the point where it wraps."""
        L.check(self._lib.bpsn_debug_set_search_count(self._h, group_idx, int(count)), self._h)

    def debug_force_batched(self, group_idx, mode):
        """Diagnostic: form of the step kernel on large batches (bpsn_debug_force_batched):
        1 always 32 entries at a time where the group has that form, 2 never, 0 chosen step
        by step."""
        L.check(self._lib.bpsn_debug_force_batched(self._h, group_idx, int(mode)), self._h)

    KERNEL_NAMES = ("k_pre", "k_step")

    def profile(self, group_idx, enable=True):
        """Turns per-kernel CUDA-event timing of the step on or off (totals are cleared)."""
        L.check(self._lib.bpsn_profile_enable(self._h, group_idx, 1 if enable else 0), self._h)

    def profile_read(self, group_idx):
        """Returns ({kernel name: total ms}, steps) accumulated since ``profile(.., True)``."""
        ms = (C.c_double * 2)()
        n = C.c_uint64()
        L.check(self._lib.bpsn_profile_read(self._h, group_idx, ms, C.byref(n)), self._h)
        return dict(zip(self.KERNEL_NAMES, list(ms))), int(n.value)

    def scene_info(self, scene_idx):
        a, b, c = C.c_int32(), C.c_int32(), C.c_int32()
        L.check(self._lib.bpsn_scene_info(self._h, scene_idx, C.byref(a), C.byref(b), C.byref(c)),
                self._h)
        return {"num_polys": a.value, "num_disabled": b.value, "num_islands": c.value}

    # batched navmesh queries on device tensors (PathFinder API in batch form)
    def query_snap(self, scene_idx, points):
        import torch
        pts = points.contiguous().float()
        n = pts.shape[0]
        out = torch.empty_like(pts)
        refs = torch.empty(n, dtype=torch.int32, device=pts.device)
        L.check(self._lib.bpsn_query_snap(self._h, scene_idx, n, pts.data_ptr(), out.data_ptr(),
                                          refs.data_ptr(), self._current_stream()), self._h)
        return out, refs

    def query_try_step(self, scene_idx, start, start_refs, end):
        import torch
        s, e = start.contiguous().float(), end.contiguous().float()
        r = start_refs.contiguous().to(torch.int32)
        n = s.shape[0]
        out = torch.empty_like(s)
        refs = torch.empty(n, dtype=torch.int32, device=s.device)
        L.check(self._lib.bpsn_query_try_step(self._h, scene_idx, n, s.data_ptr(), r.data_ptr(),
                                              e.data_ptr(), out.data_ptr(), refs.data_ptr(),
                                              self._current_stream()), self._h)
        return out, refs

    def query_geodesic(self, scene_idx, start, start_refs, end, end_refs):
        import torch
        s, e = start.contiguous().float(), end.contiguous().float()
        sr = start_refs.contiguous().to(torch.int32)
        er = end_refs.contiguous().to(torch.int32)
        n = s.shape[0]
        out = torch.empty(n, dtype=torch.float32, device=s.device)
        status = torch.empty(n, dtype=torch.int32, device=s.device)
        L.check(self._lib.bpsn_query_geodesic(self._h, scene_idx, n, s.data_ptr(), sr.data_ptr(),
                                              e.data_ptr(), er.data_ptr(), out.data_ptr(),
                                              status.data_ptr(), self._current_stream()), self._h)
        return out, status


class PointNavRolloutGenerator(_RolloutGenerator):
    _task = "pointnav"


class FleeRolloutGenerator(_RolloutGenerator):
    """Flee task (``simulator/simulator.cpp:830-887, 1818-1819``): info = geodesic distance from
    the episode start, reward = its increase."""
    _task = "flee"


class ExplorationRolloutGenerator(_RolloutGenerator):
    """Exploration task (``simulator/simulator.cpp:889-999, 1821-1822``): info = visited 1 m cells
    minus one, reward = 0.25 per new cell."""
    _task = "exploration"
