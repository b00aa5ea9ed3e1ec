"""ctypes binding of the C ABI declared in ``include/bpsn.h``.

Loading fails loudly when ``libbpsn.so`` is missing: there is no Python or CPU
implementation to fall back to.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libbpsn.so")

# every symbol include/bpsn.h declares
SYMBOLS = [
    "bpsn_create", "bpsn_destroy", "bpsn_set_navmesh_file", "bpsn_set_navmesh_blob",
    "bpsn_set_episodes", "bpsn_set_active_scenes", "bpsn_swap_stats", "bpsn_set_env_scenes", "bpsn_set_scene_geometry", "bpsn_finalize", "bpsn_reset", "bpsn_step_start", "bpsn_step_start_ex",
    "bpsn_step_end", "bpsn_render", "bpsn_get_ptr", "bpsn_device_error_flags", "bpsn_profile_enable", "bpsn_profile_read", "bpsn_scene_info", "bpsn_query_snap", "bpsn_query_try_step",
    "bpsn_query_geodesic", "bpsn_gae_workspace_bytes", "bpsn_gae", "bpsn_gae_static", "bpsn_adv_workspace_bytes",
    "bpsn_adv_normalize", "bpsn_adv_mean", "bpsn_adv_ema_shift", "bpsn_selftest_sqrt", "bpsn_dataset_open", "bpsn_dataset_num_scenes", "bpsn_dataset_scene",
    "bpsn_dataset_close", "bpsn_last_error",
    "bpsn_version",
]

# exports for the tests only (bps_nav_b200/csrc/bpsn_test_hooks.h)
TEST_HOOKS = ["bpsn_debug_set_search_count", "bpsn_debug_force_batched"]

OK = 0
ERR_INVALID_ARG, ERR_BAD_NAVMESH, ERR_CUDA, ERR_STATE, ERR_BAD_ACTION, ERR_IO, ERR_NO_DEVICE = range(1, 8)
ERR_NAMES = {
    1: "BPSN_ERR_INVALID_ARG", 2: "BPSN_ERR_BAD_NAVMESH", 3: "BPSN_ERR_CUDA", 4: "BPSN_ERR_STATE",
    5: "BPSN_ERR_BAD_ACTION", 6: "BPSN_ERR_IO", 7: "BPSN_ERR_NO_DEVICE",
}
FLAG_HOST_MIRRORS = 1
FLAG_GENERIC_KERNEL = 2
FLAG_EXACT_HEAP = 4
FLAG_SMEM_96K = 8
FLAG_GLOBAL_MEMORY = 16
FLAG_TWO_LAUNCHES = 32
TASK_POINTNAV, TASK_FLEE, TASK_EXPLORATION = 0, 1, 2
MEM_DEVICE, MEM_HOST = 0, 1
(FIELD_REWARD, FIELD_MASK, FIELD_INFO, FIELD_POLAR, FIELD_POSITION, FIELD_ROTATION, FIELD_GOAL,
 FIELD_NAV_POSITION, FIELD_NAV_POLY, FIELD_GOAL_POLY, FIELD_STEP, FIELD_EPISODE, FIELD_RESET_COUNT,
 FIELD_STATUS, FIELD_PREV_DIST, FIELD_CUM_TRAVEL, FIELD_INIT_DIST, FIELD_SCENE,
 FIELD_EPISODE_REWARD, FIELD_EPISODE_STATS, FIELD_DEPTH) = range(21)


class Config(C.Structure):
    _fields_ = [("gpu_id", C.c_int32), ("num_envs", C.c_uint32), ("num_groups", C.c_uint32),
                ("num_scenes", C.c_uint32), ("seed", C.c_uint64), ("flags", C.c_uint32),
                ("task", C.c_uint32), ("render_width", C.c_uint32), ("render_height", C.c_uint32),
                ("num_active_scenes", C.c_uint32),
                ("swap_interval", C.c_uint32)]


class AdvSegment(C.Structure):
    _fields_ = [("advantages", C.c_void_p), ("N", C.c_uint32), ("start", C.c_uint32),
                ("end", C.c_uint32), ("group", C.c_uint32)]


MAX_ADV_SEGMENTS = 64


class Episode(C.Structure):
    _fields_ = [("start_position", C.c_float * 3), ("start_rotation", C.c_float * 4),
                ("goal", C.c_float * 3)]


_lib = None


def load():
    """Returns the loaded library, raising if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m bps_nav_b200.build` "
            "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    vp, u32, i32, sz = C.c_void_p, C.c_uint32, C.c_int32, C.c_size_t
    lib.bpsn_create.argtypes = [C.POINTER(Config), C.POINTER(vp)]
    lib.bpsn_destroy.argtypes = [vp]
    lib.bpsn_set_navmesh_file.argtypes = [vp, u32, C.c_char_p]
    lib.bpsn_set_navmesh_blob.argtypes = [vp, u32, vp, sz]
    lib.bpsn_set_episodes.argtypes = [vp, u32, vp, u32]
    lib.bpsn_set_env_scenes.argtypes = [vp, vp, u32]
    lib.bpsn_set_active_scenes.argtypes = [vp, vp, u32]
    lib.bpsn_swap_stats.argtypes = [vp, C.POINTER(C.c_uint64), C.POINTER(C.c_float),
                                    C.POINTER(C.c_float)]
    lib.bpsn_set_scene_geometry.argtypes = [vp, u32, vp, vp, u32]
    lib.bpsn_render.argtypes = [vp, u32, vp]
    lib.bpsn_finalize.argtypes = [vp]
    lib.bpsn_reset.argtypes = [vp, u32, vp]
    lib.bpsn_step_start.argtypes = [vp, u32, vp, i32, vp]
    lib.bpsn_step_start_ex.argtypes = [vp, u32, vp, i32, vp, vp, vp, vp]
    lib.bpsn_step_end.argtypes = [vp, u32]
    lib.bpsn_get_ptr.argtypes = [vp, u32, i32, i32, C.POINTER(vp), C.POINTER(sz)]
    lib.bpsn_device_error_flags.argtypes = [vp, u32, C.POINTER(C.c_uint32)]
    lib.bpsn_profile_enable.argtypes = [vp, u32, i32]
    lib.bpsn_profile_read.argtypes = [vp, u32, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]
    lib.bpsn_scene_info.argtypes = [vp, u32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)]
    lib.bpsn_query_snap.argtypes = [vp, u32, u32, vp, vp, vp, vp]
    lib.bpsn_query_try_step.argtypes = [vp, u32, u32, vp, vp, vp, vp, vp, vp]
    lib.bpsn_query_geodesic.argtypes = [vp, u32, u32, vp, vp, vp, vp, vp, vp, vp]
    lib.bpsn_gae_workspace_bytes.argtypes = [u32]
    lib.bpsn_gae_workspace_bytes.restype = sz
    lib.bpsn_gae.argtypes = [vp, vp, vp, vp, vp, vp, u32, u32, C.c_double, C.c_double, i32,
                             C.c_float, vp, vp]
    lib.bpsn_gae_static.argtypes = [vp, vp, vp, vp, vp, vp, u32, u32, C.c_double, C.c_double, i32,
                                    C.c_float, vp]
    lib.bpsn_adv_workspace_bytes.argtypes = []
    lib.bpsn_adv_workspace_bytes.restype = sz
    lib.bpsn_adv_normalize.argtypes = [C.POINTER(AdvSegment), u32, u32, C.c_float, vp, vp]
    lib.bpsn_adv_mean.argtypes = [C.POINTER(AdvSegment), u32, u32, vp, vp, vp]
    lib.bpsn_adv_ema_shift.argtypes = [C.POINTER(AdvSegment), u32, u32, vp, vp, C.c_float, vp]
    lib.bpsn_selftest_sqrt.argtypes = [i32, u32, u32, C.POINTER(C.c_uint64)]
    lib.bpsn_debug_set_search_count.argtypes = [C.c_void_p, u32, u32]
    lib.bpsn_debug_force_batched.argtypes = [C.c_void_p, u32, C.c_int32]
    lib.bpsn_dataset_open.argtypes = [C.c_char_p, C.c_char_p, u32, C.POINTER(vp)]
    lib.bpsn_dataset_num_scenes.argtypes = [vp]
    lib.bpsn_dataset_num_scenes.restype = u32
    lib.bpsn_dataset_scene.argtypes = [vp, u32, C.POINTER(C.c_char_p), C.POINTER(C.c_char_p),
                                       C.POINTER(vp), C.POINTER(u32)]
    lib.bpsn_dataset_close.argtypes = [vp]
    lib.bpsn_dataset_close.restype = None
    lib.bpsn_last_error.argtypes = [vp]
    lib.bpsn_last_error.restype = C.c_char_p
    lib.bpsn_version.restype = C.c_char_p
    for name in SYMBOLS + TEST_HOOKS:
        fn = getattr(lib, name)
        if name not in ("bpsn_gae_workspace_bytes", "bpsn_adv_workspace_bytes", "bpsn_last_error", "bpsn_version",
                        "bpsn_dataset_num_scenes", "bpsn_dataset_close"):
            fn.restype = i32
    _lib = lib
    return lib


def check(rc, handle=None):
    """Raises RuntimeError with the library's message for a non-zero status."""
    if rc == OK:
        return
    lib = load()
    msg = lib.bpsn_last_error(handle)
    msg = msg.decode() if msg else ""
    raise RuntimeError(f"{ERR_NAMES.get(rc, rc)}: {msg}")
