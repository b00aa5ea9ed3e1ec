"""TEST INFRASTRUCTURE ONLY: Python access to the parity oracle.

* ``RefNav``    -- the reference's compiled ``esp::nav::PathFinder`` (oracle/_ref/libref_nav.so,
  built by ``oracle/Makefile`` from the reference's own Detour + PathFinder sources).
* ``OracleSim`` -- the CPU restatement of the per-environment PointNav simulator
  (``oracle/oracle_sim.cpp``) running on top of ``RefNav``.  Doubles as the timed CPU baseline.
* ``philox_actions`` -- the synthetic action streams shared by oracle and CUDA runs.
* ``gae_reference`` -- numpy restatement of ``RolloutStorage.compute_returns`` +
  ``PPO.get_advantages`` (bps_nav/common/rollout_storage.py:203-219, bps_nav/rl/ppo/ppo.py:190-201).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` import this module; the shipped package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_LIB = os.path.join(HERE, "_ref", "libref_nav.so")
GEN_SCENE = os.path.join(HERE, "_ref", "gen_scene")
SIM_LIB = os.path.join(HERE, "_build", "liboracle_sim.so")

_fp = C.POINTER(C.c_float)
_u64p = C.POINTER(C.c_uint64)
_u32p = C.POINTER(C.c_uint32)


def available():
    return os.path.exists(REF_LIB) and os.path.exists(SIM_LIB)


def reference_root():
    """Root of the bps-nav tree on this machine: $BPS_NAV_REFERENCE, else a directory named
    ``reference`` beside the repository; None when neither exists."""
    cand = os.environ.get("BPS_NAV_REFERENCE")
    if not cand:
        cand = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "simulator")) else None


def build(root=None):
    """Builds oracle/_ref (needs the reference sources) and oracle/_build.  Returns True when both
    libraries exist afterwards."""
    root = root or reference_root()
    if root:
        subprocess.run(["make", "-C", HERE, "ref", f"REF={root}"], check=True,
                       capture_output=True)
    if os.path.exists(REF_LIB):
        subprocess.run(["make", "-C", HERE, "sim"], check=True, capture_output=True)
    return available()


_ref = None
_sim = None


def ref_lib():
    global _ref
    if _ref is None:
        if not os.path.exists(REF_LIB):
            raise RuntimeError(f"{REF_LIB} missing: run `make -C oracle ref` where the reference "
                               "sources are present")
        lib = C.CDLL(REF_LIB)
        lib.refnav_create.restype = C.c_void_p
        lib.refnav_create.argtypes = [C.c_char_p]
        lib.refnav_destroy.argtypes = [C.c_void_p]
        lib.refnav_snap_batch.argtypes = [C.c_void_p, C.c_int, _fp, _fp, _u64p]
        lib.refnav_try_step_batch.argtypes = [C.c_void_p, C.c_int, _fp, _u64p, _fp, _fp, _u64p]
        lib.refnav_find_path_batch.argtypes = [C.c_void_p, C.c_int, _fp, _u64p, _fp, _u64p, _fp]
        lib.refnav_bounds.argtypes = [C.c_void_p, _fp, _fp]
        lib.refdt_create.restype = C.c_void_p
        lib.refdt_create.argtypes = [C.c_char_p]
        lib.refdt_destroy.argtypes = [C.c_void_p]
        lib.refdt_seed.argtypes = [C.c_uint64]
        lib.refdt_random_point.argtypes = [C.c_void_p, _u32p, _fp]
        lib.refdt_poly_count.argtypes = [C.c_void_p]
        _ref = lib
    return _ref


def _p(a, t):
    return a.ctypes.data_as(t)


class RefNav:
    """Batch wrappers over the reference PathFinder for one navmesh file."""

    def __init__(self, navmesh_path):
        lib = ref_lib()
        self._lib = lib
        self.path = navmesh_path
        self._h = C.c_void_p(lib.refnav_create(navmesh_path.encode()))
        if not self._h.value:
            raise RuntimeError(f"reference PathFinder failed to load {navmesh_path}")
        self._dt = C.c_void_p(lib.refdt_create(navmesh_path.encode()))

    def close(self):
        if self._h.value:
            self._lib.refnav_destroy(self._h)
            self._h = C.c_void_p()
        if self._dt.value:
            self._lib.refdt_destroy(self._dt)
            self._dt = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def poly_count(self):
        return self._lib.refdt_poly_count(self._dt)

    def snap(self, pts):
        pts = np.ascontiguousarray(pts, np.float32).reshape(-1, 3)
        n = len(pts)
        out = np.zeros((n, 3), np.float32)
        ref = np.zeros(n, np.uint64)
        self._lib.refnav_snap_batch(self._h, n, _p(pts, _fp), _p(out, _fp), _p(ref, _u64p))
        return out, ref

    def try_step(self, start, start_ref, end):
        start = np.ascontiguousarray(start, np.float32).reshape(-1, 3)
        end = np.ascontiguousarray(end, np.float32).reshape(-1, 3)
        sref = np.ascontiguousarray(start_ref, np.uint64)
        n = len(start)
        out = np.zeros((n, 3), np.float32)
        ref = np.zeros(n, np.uint64)
        self._lib.refnav_try_step_batch(self._h, n, _p(start, _fp), _p(sref, _u64p), _p(end, _fp),
                                        _p(out, _fp), _p(ref, _u64p))
        return out, ref

    def geodesic(self, start, start_ref, end, end_ref):
        start = np.ascontiguousarray(start, np.float32).reshape(-1, 3)
        end = np.ascontiguousarray(end, np.float32).reshape(-1, 3)
        sref = np.ascontiguousarray(start_ref, np.uint64)
        eref = np.ascontiguousarray(end_ref, np.uint64)
        n = len(start)
        out = np.zeros(n, np.float32)
        self._lib.refnav_find_path_batch(self._h, n, _p(start, _fp), _p(sref, _u64p),
                                         _p(end, _fp), _p(eref, _u64p), _p(out, _fp))
        return out

    def random_points(self, n, seed):
        """Area-weighted random navigable points (dtNavMeshQuery::findRandomPoint)."""
        self._lib.refdt_seed(C.c_uint64(seed))
        pts = np.zeros((n, 3), np.float32)
        refs = np.zeros(n, np.uint32)
        r = C.c_uint32()
        p = (C.c_float * 3)()
        for i in range(n):
            self._lib.refdt_random_point(self._dt, C.byref(r), p)
            pts[i] = p[:]
            refs[i] = r.value
        return pts, refs


def sim_lib():
    global _sim
    if _sim is None:
        if not os.path.exists(SIM_LIB):
            raise RuntimeError(f"{SIM_LIB} missing: run `make -C oracle sim`")
        ref_lib()
        lib = C.CDLL(SIM_LIB)
        lib.osim_create.restype = C.c_void_p
        lib.osim_create.argtypes = [C.c_int, C.POINTER(C.c_char_p), _fp, C.POINTER(C.c_int),
                                    C.c_int, C.POINTER(C.c_int), C.c_uint64, C.c_int, C.c_int]
        lib.osim_destroy.argtypes = [C.c_void_p]
        lib.osim_reset.argtypes = [C.c_void_p, C.c_int, C.c_int]
        lib.osim_step.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int64)]
        lib.osim_run.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int64)]
        for name in ("osim_rewards", "osim_infos", "osim_polars"):
            getattr(lib, name).restype = _fp
            getattr(lib, name).argtypes = [C.c_void_p]
        lib.osim_masks.restype = C.POINTER(C.c_uint8)
        lib.osim_masks.argtypes = [C.c_void_p]
        lib.osim_enable_rotation.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int)]
        lib.osim_set_swap_interval.argtypes = [C.c_void_p, C.c_uint32]
        lib.osim_scenes.restype = C.c_uint64
        lib.osim_scenes.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
        lib.osim_get_state.argtypes = [C.c_void_p, _fp, _u32p]
        lib.osim_counters.argtypes = [C.c_void_p, _u64p]
        lib.osim_philox.argtypes = [C.c_uint32] * 6 + [_u32p]
        _sim = lib
    return _sim


STATE_F = ["position", "rotation", "goal", "nav_position", "nav_goal", "prev_dist", "cum_travel",
           "init_dist", "prev_pos"]
_STATE_F_SLICES = {"position": (0, 3), "rotation": (3, 7), "goal": (7, 10),
                   "nav_position": (10, 13), "nav_goal": (13, 16), "prev_dist": (16, 17),
                   "cum_travel": (17, 18), "init_dist": (18, 19), "prev_pos": (19, 22)}
_STATE_U = {"nav_poly": 0, "goal_poly": 1, "step": 2, "episode": 3, "reset_count": 4}


class OracleSim:
    """CPU oracle over a list of (navmesh_path, episodes[n,10]) scenes."""

    TASKS = {"pointnav": 0, "flee": 1, "exploration": 2}

    def __init__(self, scenes, num_envs, seed, env_scene=None, threads=1, task="pointnav",
                 active_scenes=None, num_groups=1, swap_interval=0):
        """``active_scenes``: turns scene rotation on -- the scenes in use first, one per slot of
        ``num_envs / len(active_scenes)`` consecutive environments; the others rotate in,
        at most one per group every ``swap_interval`` steps (0: as soon as a slot is whole)."""
        lib = sim_lib()
        self._lib = lib
        self.num_envs = num_envs
        ns = len(scenes)
        paths = (C.c_char_p * ns)(*[s[0].encode() for s in scenes])
        eps = [np.ascontiguousarray(s[1]).view(np.float32).reshape(-1, 10) for s in scenes]
        offs = np.zeros(ns + 1, np.int32)
        offs[1:] = np.cumsum([len(e) for e in eps])
        allep = np.ascontiguousarray(np.concatenate(eps, 0), np.float32)
        if env_scene is None:
            per = num_envs // ns
            env_scene = np.arange(num_envs, dtype=np.int32) // per
        env_scene = np.ascontiguousarray(env_scene, np.int32)
        self._h = C.c_void_p(lib.osim_create(ns, paths, _p(allep, _fp),
                                             offs.ctypes.data_as(C.POINTER(C.c_int)), num_envs,
                                             env_scene.ctypes.data_as(C.POINTER(C.c_int)),
                                             C.c_uint64(seed), threads, self.TASKS[task]))
        if not self._h.value:
            raise RuntimeError("oracle simulator creation failed")
        if active_scenes is not None:
            act = np.ascontiguousarray(active_scenes, np.int32)
            if lib.osim_enable_rotation(self._h, len(act), num_groups,
                                        act.ctypes.data_as(C.POINTER(C.c_int))) != 0:
                raise RuntimeError("oracle: bad scene rotation parameters")
            lib.osim_set_swap_interval(self._h, int(swap_interval))
        n = num_envs
        self.rewards = np.ctypeslib.as_array(lib.osim_rewards(self._h), (n,))
        self.masks = np.ctypeslib.as_array(lib.osim_masks(self._h), (n,))
        self.infos = np.ctypeslib.as_array(lib.osim_infos(self._h),
                                           (n, 3 if task == "pointnav" else 1))
        self.polars = np.ctypeslib.as_array(lib.osim_polars(self._h), (n, 2))

    def close(self):
        if self._h.value:
            self._lib.osim_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset(self, first=0, count=None):
        self._lib.osim_reset(self._h, first, self.num_envs if count is None else count)

    def step(self, actions, first=0):
        a = np.ascontiguousarray(actions, np.int64)
        return self._lib.osim_step(self._h, first, len(a), a.ctypes.data_as(C.POINTER(C.c_int64)))

    def run(self, actions):
        """actions[steps, num_envs]; runs without returning to Python between steps."""
        a = np.ascontiguousarray(actions, np.int64)
        return self._lib.osim_run(self._h, a.shape[0], a.ctypes.data_as(C.POINTER(C.c_int64)))

    def state(self):
        f = np.zeros((self.num_envs, 22), np.float32)
        u = np.zeros((self.num_envs, 5), np.uint32)
        self._lib.osim_get_state(self._h, _p(f, _fp), _p(u, _u32p))
        out = {k: f[:, a:b].copy() if b - a > 1 else f[:, a].copy()
               for k, (a, b) in _STATE_F_SLICES.items()}
        out.update({k: u[:, i].copy() for k, i in _STATE_U.items()})
        return out

    def scenes(self):
        """(scene of every environment, scene moves started since set-up)."""
        out = np.zeros(self.num_envs, np.int32)
        n = self._lib.osim_scenes(self._h, out.ctypes.data_as(C.POINTER(C.c_int)))
        return out, int(n)

    def counters(self):
        c = np.zeros(3, np.uint64)
        self._lib.osim_counters(self._h, _p(c, _u64p))
        return {"try_step": int(c[0]), "find_path": int(c[1]), "snap": int(c[2])}


# --------------------------------------------------------------------------- action streams

def _philox4x32(c0, c1, c2, c3, k0, k1):
    """Vectorised Philox-4x32-10; all inputs uint32 arrays (broadcastable) or ints."""
    c0, c1, c2, c3 = [np.asarray(c, np.uint64) & 0xFFFFFFFF for c in np.broadcast_arrays(c0, c1, c2, c3)]
    k0 = np.uint64(k0)
    k1 = np.uint64(k1)
    M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = M0 * c0
        p1 = M1 * c2
        n0 = ((p1 >> np.uint64(32)) ^ c1 ^ k0) & mask
        n1 = p1 & mask
        n2 = ((p0 >> np.uint64(32)) ^ c3 ^ k1) & mask
        n3 = p0 & mask
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return c0.astype(np.uint32), c1.astype(np.uint32), c2.astype(np.uint32), c3.astype(np.uint32)


def philox_actions(steps, num_envs, seed, mix="uniform", env_base=0):
    """int64 actions[steps, num_envs] keyed by (seed, env, t).

    mix = "uniform": i.i.d. uniform over {0 stop, 1 forward, 2 left, 3 right};
    mix = "policy" : stop 0.5 %, forward 60 %, left / right 19.75 % each (closer to a trained
    policy's action statistics: long episodes, few resets).
    """
    env = (np.arange(num_envs, dtype=np.uint64) + np.uint64(env_base))[None, :]
    t = np.arange(steps, dtype=np.uint64)[:, None]
    r0, _, _, _ = _philox4x32(env, t, 0, 0, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    if mix == "uniform":
        return (r0 & 3).astype(np.int64)
    if mix == "policy":
        u = r0.astype(np.float64) / 4294967296.0
        a = np.full(u.shape, 3, np.int64)
        a[u < 0.8025] = 2
        a[u < 0.605] = 1
        a[u < 0.005] = 0
        return a
    raise ValueError(mix)


# --------------------------------------------------------------------------- GAE

def gae_reference(rewards, values, masks, next_value, gamma, tau, normalize=False, eps=1e-5):
    """numpy fp32 restatement of compute_returns + get_advantages.

    rewards / values: float32 [T+1, N]; masks: bool [T+1, N]; next_value: float32 [N].
    Returns (returns[T+1, N] with row T untouched (zero), advantages[T, N]).  Each arithmetic op
    is rounded to float32 separately, in the reference's evaluation order; gamma * tau is folded in
    double first, as Python does before the scalar meets the tensor.
    """
    rewards = np.asarray(rewards, np.float32)
    values = np.array(values, np.float32, copy=True)
    m = np.asarray(masks).astype(np.float32)
    T = rewards.shape[0] - 1
    values[T] = next_value
    returns = np.zeros_like(values)
    g = np.float32(gamma)
    gt = np.float32(gamma * tau)
    gae = np.zeros(rewards.shape[1], np.float32)
    for t in reversed(range(T)):
        delta = (rewards[t] + (g * values[t + 1]) * m[t + 1]) - values[t]
        gae = delta + (gt * gae) * m[t + 1]
        returns[t] = gae + values[t]
    adv = returns[:T] - values[:T]
    if normalize:
        a64 = adv.astype(np.float64)
        mean = a64.mean()
        std = a64.std(ddof=1)
        adv = ((adv - np.float32(mean)) / (np.float32(std) + np.float32(eps))).astype(np.float32)
    return returns, adv, values


# ----------------------------------------------------------------------------- depth sensor
def depth_reference(position, rotation, floor, boxes, width, height):
    """Depth image [H, W] float32 of one environment: CPU restatement, in fp32 numpy with the
    same operation order, of the analytic box-world sensor (camera of simulator/simulator.cpp:
    651-663 and :1216: eye = position + 1.25 up, looking down -Z of the agent frame, 90 degree
    vertical field of view, near 0.1, far 1000; value = view-space depth, far where nothing is
    hit).  Parity unpinned: the reference renders with bps3D, which is not in its tree, so there
    is no reference image to pin this against; it checks the CUDA kernel against an independent
    evaluation of the same geometry."""
    f = np.float32
    qx, qy, qz, qw = (f(x) for x in rotation)
    ox, oy, oz = f(position[0]), f(position[1]) + f(1.25), f(position[2])
    qxx, qyy, qzz = qx * qx, qy * qy, qz * qz
    qxz, qxy, qyz = qx * qz, qx * qy, qy * qz
    qwx, qwy, qwz = qw * qx, qw * qy, qw * qz
    one, two = f(1), f(2)
    m00, m01, m02 = one - two * (qyy + qzz), two * (qxy + qwz), two * (qxz - qwy)
    m10, m11, m12 = two * (qxy - qwz), one - two * (qxx + qzz), two * (qyz + qwx)
    m20, m21, m22 = two * (qxz + qwy), two * (qyz - qwx), one - two * (qxx + qyy)
    aspect = f(width) / f(height)
    px = np.arange(width, dtype=np.float32)
    py = np.arange(height, dtype=np.float32)
    u = ((px + f(0.5)) / f(width) * two - one) * aspect
    v = one - (py + f(0.5)) / f(height) * two
    U, V = np.meshgrid(u, v)  # [H, W]
    dx = (m00 * U + m10 * V) - m20
    dy = (m01 * U + m11 * V) - m21
    dz = (m02 * U + m12 * V) - m22
    near, far = f(0.1), f(1000.0)
    t = np.full((height, width), far, np.float32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        tf = (f(0) - oy) / dy
        hx, hz = ox + tf * dx, oz + tf * dz
        fl = [f(x) for x in floor]
        hit = ((dy < 0) & (tf >= near) & (tf < t) & (hx >= fl[0]) & (hx <= fl[2]) &
               (hz >= fl[1]) & (hz <= fl[3]))
        t = np.where(hit, tf, t).astype(np.float32)
        ix, iy, iz = one / dx, one / dy, one / dz
        for b in np.asarray(boxes, np.float32).reshape(-1, 6):
            tx0, tx1 = (b[0] - ox) * ix, (b[3] - ox) * ix
            ty0, ty1 = (b[1] - oy) * iy, (b[4] - oy) * iy
            tz0, tz1 = (b[2] - oz) * iz, (b[5] - oz) * iz
            tenter = np.fmax(np.fmax(np.fmin(tx0, tx1), np.fmin(ty0, ty1)), np.fmin(tz0, tz1))
            texit = np.fmin(np.fmin(np.fmax(tx0, tx1), np.fmax(ty0, ty1)), np.fmax(tz0, tz1))
            hit = (tenter <= texit) & (tenter >= near) & (tenter < t)
            t = np.where(hit, tenter, t).astype(np.float32)
    return t
