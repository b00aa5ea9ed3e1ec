"""Episode datasets and scene lists (host side).

Reads the on-disk layout the reference's ``Dataset`` class reads
(``simulator/simulator.cpp:190-359``): every ``*.json.gz`` under ``dataset_path`` holds the
episodes of one scene, ``{"episodes": [{"start_position": [x,y,z], "start_rotation": [x,y,z,w],
"goals": [{"position": [x,y,z]}], "scene_id": "dir/name.glb"}, ...]}``; the scene's navigation
mesh is ``asset_path/<scene_id without extension>.navmesh`` (``:292-311``).  Files are visited
in sorted order (the reference's order depends on directory iteration and thread timing).
"""
import glob
import gzip
import json
import os

import numpy as np

EPISODE_DTYPE = np.dtype([("start_position", "<f4", 3), ("start_rotation", "<f4", 4),
                          ("goal", "<f4", 3)])


class Scene:
    """One scene: navmesh file, episode records and, optionally, the render geometry of the depth
    sensor (``floor`` = (xmin, zmin, xmax, zmax) at y = 0, ``boxes`` = float32 [K, 6] min/max
    corners).  When not given, geometry is read from ``<navmesh stem>.scene.json`` if that file
    exists (keys ``size_x``, ``size_z``, ``boxes``), the sidecar the synthetic scene generator
    writes; scenes without geometry render as empty space."""

    def __init__(self, navmesh_path, episodes, scene_id="", floor=None, boxes=None):
        self.navmesh_path = navmesh_path
        self.scene_id = scene_id
        if floor is None and boxes is None:
            side = os.path.splitext(navmesh_path)[0] + ".scene.json"
            if os.path.exists(side):
                with open(side) as f:
                    doc = json.load(f)
                if "size_x" in doc and "size_z" in doc:
                    floor = (0.0, 0.0, float(doc["size_x"]), float(doc["size_z"]))
                    boxes = doc.get("boxes", [])
        self.floor = None if floor is None else tuple(float(x) for x in floor)
        self.boxes = (np.zeros((0, 6), np.float32) if boxes is None else
                      np.ascontiguousarray(np.asarray(boxes, np.float32).reshape(-1, 6)))
        episodes = np.ascontiguousarray(episodes)
        if episodes.dtype != EPISODE_DTYPE:
            flat = np.asarray(episodes, dtype=np.float32).reshape(-1, 10)
            episodes = np.ascontiguousarray(flat).view(EPISODE_DTYPE).reshape(-1)
        self.episodes = episodes


def load_dataset(dataset_path, asset_path, num_threads=None):
    """Reads a directory of ``*.json.gz`` episode files with the library's native reader
    (``bpsn_dataset_open``: zlib + its own JSON parser, one thread per file up to
    ``num_threads``) and returns ``Scene`` objects in file-name order."""
    import ctypes as C
    from . import _lib as L
    lib = L.load()
    if num_threads is None:
        num_threads = max(1, len(os.sched_getaffinity(0)))
    h = C.c_void_p()
    L.check(lib.bpsn_dataset_open(os.fsencode(dataset_path), os.fsencode(asset_path),
                                  int(num_threads), C.byref(h)))
    try:
        scenes = []
        for i in range(lib.bpsn_dataset_num_scenes(h)):
            sid, nav, eps, n = C.c_char_p(), C.c_char_p(), C.c_void_p(), C.c_uint32()
            L.check(lib.bpsn_dataset_scene(h, i, C.byref(sid), C.byref(nav), C.byref(eps),
                                           C.byref(n)))
            buf = (C.c_char * (n.value * EPISODE_DTYPE.itemsize)).from_address(eps.value)
            arr = np.frombuffer(buf, dtype=EPISODE_DTYPE).copy()
            scenes.append(Scene(nav.value.decode(), arr, sid.value.decode()))
        return scenes
    finally:
        lib.bpsn_dataset_close(h)


def load_dataset_py(dataset_path, asset_path):
    """The same reader in plain Python (gzip + json modules); kept as the cross-check of the
    native one."""
    files = sorted(glob.glob(os.path.join(dataset_path, "*.json.gz")))
    if not files:
        raise RuntimeError(f"no *.json.gz episode files under {dataset_path}")
    scenes = []
    for fn in files:
        with gzip.open(fn, "rt") as f:
            doc = json.load(f)
        eps = doc["episodes"]
        if not eps:
            continue
        scene_id = eps[0]["scene_id"]
        arr = np.zeros(len(eps), dtype=EPISODE_DTYPE)
        for i, ep in enumerate(eps):
            if ep["scene_id"] != scene_id:
                raise RuntimeError("Loading code assumes json file contains data for one scene")
            arr["start_position"][i] = ep["start_position"]
            arr["start_rotation"][i] = ep["start_rotation"]
            arr["goal"][i] = ep["goals"][0]["position"]
        dot = scene_id.rfind(".")
        if dot < 0:
            raise RuntimeError(f"Invalid scene id: {scene_id}")
        nav = os.path.join(asset_path, scene_id[:dot] + ".navmesh")
        scenes.append(Scene(nav, arr, scene_id))
    return scenes


def write_dataset(scenes, dataset_path, asset_path):
    """Writes scenes in the layout ``load_dataset`` reads (navmesh files are copied)."""
    import shutil
    os.makedirs(dataset_path, exist_ok=True)
    os.makedirs(asset_path, exist_ok=True)
    for i, sc in enumerate(scenes):
        name = sc.scene_id or f"scene_{i:03d}.glb"
        stem = name[:name.rfind(".")]
        dst = os.path.join(asset_path, stem + ".navmesh")
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        if os.path.abspath(dst) != os.path.abspath(sc.navmesh_path):
            shutil.copyfile(sc.navmesh_path, dst)
        eps = [{"episode_id": str(j), "scene_id": name,
                "start_position": [float(x) for x in e["start_position"]],
                "start_rotation": [float(x) for x in e["start_rotation"]],
                "goals": [{"position": [float(x) for x in e["goal"]], "radius": None}]}
               for j, e in enumerate(sc.episodes)]
        with gzip.open(os.path.join(dataset_path, os.path.basename(stem) + ".json.gz"), "wt") as f:
            json.dump({"episodes": eps}, f)


class _MT19937:
    """std::mt19937 (32-bit Mersenne twister), enough of it for the active-scene draw."""

    def __init__(self, seed):
        self.mt = [0] * 624
        self.mt[0] = seed & 0xFFFFFFFF
        for i in range(1, 624):
            self.mt[i] = (1812433253 * (self.mt[i - 1] ^ (self.mt[i - 1] >> 30)) + i) & 0xFFFFFFFF
        self.idx = 624

    def next_u32(self):
        if self.idx >= 624:
            mt = self.mt
            for k in range(624):
                y = (mt[k] & 0x80000000) | (mt[(k + 1) % 624] & 0x7FFFFFFF)
                mt[k] = mt[(k + 397) % 624] ^ (y >> 1) ^ (0x9908B0DF if y & 1 else 0)
            self.idx = 0
        y = self.mt[self.idx]
        self.idx += 1
        y ^= y >> 11
        y ^= (y << 7) & 0x9D2C5680
        y ^= (y << 15) & 0xEFC60000
        y ^= y >> 18
        return y & 0xFFFFFFFF

    def canonical_double(self):
        # std::generate_canonical<double, 53>: two 32-bit draws, low word first
        lo = self.next_u32()
        hi = self.next_u32()
        r = (lo + hi * 4294967296.0) / 18446744073709551616.0
        return r if r < 1.0 else float(np.nextafter(1.0, 0.0))


def select_active_scenes(num_scenes, num_active, seed):
    """Selection sampling of the initially active scenes, as ``simulator/simulator.cpp:1518-1534``
    does with ``std::mt19937(seed)`` and ``uniform_real_distribution<>(0, 1)``."""
    rng = _MT19937(seed)
    active, inactive = [], []
    idx = 0
    while idx < num_scenes and len(active) < num_active:
        weight = float(np.float32(rng.canonical_double()))
        if np.float32(weight) * np.float32(num_scenes - idx) < np.float32(num_active - len(active)):
            active.append(idx)
        else:
            inactive.append(idx)
        idx += 1
    inactive.extend(range(idx, num_scenes))
    return active, inactive
