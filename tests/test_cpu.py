"""CPU-only tests (no GPU): the oracle against the golden vectors, host-side logic, and that the
C-ABI library loads and exports every declared symbol."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from conftest import GOLD, ROOT, SCENES, scene_path

from oracle import pyoracle

needs_oracle = pytest.mark.skipif(not pyoracle.available(),
                                  reason="oracle/_ref not built (needs the reference sources)")

HARNESS_DIR = os.path.join(ROOT, "tests", "host_harness")
HARNESS_LIB = os.path.join(HARNESS_DIR, "_build", "libnav_host_check.so")


@pytest.fixture(scope="session")
def harness():
    """nav_query.cuh compiled for the host (test harness only)."""
    src = [os.path.join(HARNESS_DIR, "nav_host_check.cpp"),
           os.path.join(ROOT, "bps_nav_b200", "csrc", "navmesh_host.cpp")]
    deps = src + [os.path.join(ROOT, "bps_nav_b200", "csrc", f)
                  for f in ("nav_query.cuh", "nav_types.h", "navmesh_host.h")]
    if (not os.path.exists(HARNESS_LIB) or
            any(os.path.getmtime(d) > os.path.getmtime(HARNESS_LIB) for d in deps)):
        os.makedirs(os.path.dirname(HARNESS_LIB), exist_ok=True)
        subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-shared"] + src +
                       ["-o", HARNESS_LIB], check=True)
    lib = C.CDLL(HARNESS_LIB)
    lib.hchk_load.restype = C.c_void_p
    lib.hchk_load.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
    lib.hchk_free.argtypes = [C.c_void_p]
    lib.hchk_info.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
    return lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def _same(a, b):
    return ((a == b) | (np.isnan(a) & np.isnan(b))).all()


# ------------------------------------------------------------------ oracle vs golden vectors

@needs_oracle
@pytest.mark.parametrize("name", ["c0", "c1", "m03"])
def test_reference_pathfinder_reproduces_golden_queries(name):
    q = np.load(os.path.join(GOLD, f"queries_{name}.npz"))
    nav = pyoracle.RefNav(scene_path(name))
    xyz, ref = nav.snap(q["snap_in"])
    assert np.array_equal(ref.astype(np.uint32), q["snap_ref"]) and _same(xyz, q["snap_xyz"])
    xyz, ref = nav.try_step(q["step_start"], q["step_start_ref"].astype(np.uint64), q["step_end"])
    assert np.array_equal(ref.astype(np.uint32), q["step_ref"]) and _same(xyz, q["step_xyz"])
    d = nav.geodesic(q["geo_a"], q["geo_a_ref"].astype(np.uint64), q["geo_b"],
                     q["geo_b_ref"].astype(np.uint64))
    assert _same(d, q["geo_dist"])
    nav.close()


@needs_oracle
@pytest.mark.parametrize("fname,mix", [("c0_traj.npz", "uniform"), ("c0_policy_traj.npz", "policy")])
def test_oracle_simulator_reproduces_golden_trajectory(fname, mix):
    g = np.load(os.path.join(GOLD, fname))
    eps = np.load(os.path.join(SCENES, "c0.episodes.npy"))
    steps, n = g["actions"].shape
    # the action stream is a pure function of (seed, env, t)
    acts = pyoracle.philox_actions(steps, n, int(g["act_seed"]), mix)
    assert np.array_equal(acts, g["actions"].astype(np.int64))
    sim = pyoracle.OracleSim([(scene_path("c0"), eps)], n, int(g["seed"]), threads=2)
    sim.reset()
    assert _same(sim.polars, g["polar0"])
    for t in range(steps):
        assert sim.step(acts[t]) == 0
        assert np.array_equal(sim.masks, g["mask"][t])
        assert _same(sim.rewards, g["reward"][t]) and _same(sim.infos, g["info"][t])
        assert _same(sim.polars, g["polar"][t])
    st = sim.state()
    for k in ("nav_poly", "goal_poly", "step", "episode", "reset_count"):
        assert np.array_equal(st[k], g[f"s{steps}_{k}"])
    sim.close()


@needs_oracle
def test_oracle_rejects_unknown_action():
    eps = np.load(os.path.join(SCENES, "c0.episodes.npy"))
    sim = pyoracle.OracleSim([(scene_path("c0"), eps)], 4, 1)
    sim.reset()
    assert sim.step(np.array([0, 1, 7, 2], np.int64)) == -1
    sim.close()


def test_gae_restatement_matches_reference_python_fixture():
    g = np.load(os.path.join(GOLD, "gae_ref.npz"))
    for tag in ("small", "c2"):
        r, v, m = g[f"{tag}_rewards"][..., 0], g[f"{tag}_values"][..., 0], g[f"{tag}_masks"][..., 0]
        T = r.shape[0] - 1
        ret, adv, _ = pyoracle.gae_reference(r, v, m, g[f"{tag}_next_value"][:, 0], 0.99, 0.95)
        assert np.array_equal(ret[:T], g[f"{tag}_returns"][:T, :, 0])  # bit-exact
        assert np.array_equal(adv, g[f"{tag}_adv"][..., 0])
        _, advn, _ = pyoracle.gae_reference(r, v, m, g[f"{tag}_next_value"][:, 0], 0.99, 0.95,
                                            normalize=True)
        assert np.allclose(advn, g[f"{tag}_adv_norm"][..., 0], rtol=1e-5, atol=2e-6)


def _c2_inputs():
    """The C2 inputs of tests/golden/make_fixtures.py::gae_c2_inputs (seeded numpy PCG64)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_fixtures",
                                                  os.path.join(GOLD, "make_fixtures.py"))
    mf = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mf)
    return mf.gae_c2_inputs()


def test_gae_restatement_at_config2_size_matches_reference_python():
    # T = 32, N = 16384: the reference's RolloutStorage.compute_returns wrote the fixture; the
    # numpy restatement must reproduce the whole arrays bit for bit (CRC-32 of the bytes)
    import zlib
    g = np.load(os.path.join(GOLD, "gae_c2_16384.npz"))
    r, v, m, nv = _c2_inputs()
    T = 32
    ret, adv, _ = pyoracle.gae_reference(r, v, m, nv, 0.99, 0.95)
    assert zlib.crc32(np.ascontiguousarray(ret[:T]).tobytes()) == int(g["returns_crc"])
    assert zlib.crc32(np.ascontiguousarray(adv).tobytes()) == int(g["adv_crc"])
    cols = g["cols"]
    assert np.array_equal(ret[:T][:, cols], g["returns_cols"])
    assert np.array_equal(adv[:, cols], g["adv_cols"])
    _, advn, _ = pyoracle.gae_reference(r, v, m, nv, 0.99, 0.95, normalize=True)
    assert np.allclose(advn[:, cols], g["adv_norm_cols"], rtol=1e-5, atol=2e-6)
    assert abs(float(adv.astype(np.float64).mean()) - float(g["adv_mean"])) < 1e-9
    assert abs(float(adv.astype(np.float64).std(ddof=1)) - float(g["adv_std"])) < 1e-9


def test_philox_known_answers():
    # Random123 known-answer vectors for philox4x32-10
    out = pyoracle._philox4x32(0, 0, 0, 0, 0, 0)
    assert [int(x) for x in out] == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    out = pyoracle._philox4x32(0xffffffff, 0xffffffff, 0xffffffff, 0xffffffff, 0xffffffff, 0xffffffff)
    assert [int(x) for x in out] == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    if pyoracle.available():
        lib = pyoracle.sim_lib()
        o = (C.c_uint32 * 4)()
        lib.osim_philox(0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344, 0xa4093822, 0x299f31d0, o)
        assert list(o) == [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


# ------------------------------------------------------------------ host-compiled device functions

@needs_oracle
@pytest.mark.parametrize("name", ["c0", "c1", "m03"])
def test_query_functions_bit_exact_on_host(harness, name):
    q = np.load(os.path.join(GOLD, f"queries_{name}.npz"))
    err = C.create_string_buffer(256)
    h = C.c_void_p(harness.hchk_load(scene_path(name).encode(), err, 256))
    assert h.value, err.value
    n = len(q["snap_in"])
    xyz = np.zeros((n, 3), np.float32)
    ref = np.zeros(n, np.uint32)
    harness.hchk_snap_batch(h, n, _p(np.ascontiguousarray(q["snap_in"]), C.c_float),
                            _p(xyz, C.c_float), _p(ref, C.c_uint32))
    assert np.array_equal(ref, q["snap_ref"]) and _same(xyz, q["snap_xyz"])
    m = len(q["step_start"])
    xyz = np.zeros((m, 3), np.float32)
    ref = np.zeros(m, np.uint32)
    harness.hchk_try_step_batch(h, m, _p(np.ascontiguousarray(q["step_start"]), C.c_float),
                                _p(np.ascontiguousarray(q["step_start_ref"]), C.c_uint32),
                                _p(np.ascontiguousarray(q["step_end"]), C.c_float),
                                _p(xyz, C.c_float), _p(ref, C.c_uint32))
    assert np.array_equal(ref, q["step_ref"]) and _same(xyz, q["step_xyz"])
    d = np.zeros(m, np.float32)
    st = np.zeros(m, np.uint32)
    harness.hchk_geodesic_batch(h, m, _p(np.ascontiguousarray(q["geo_a"]), C.c_float),
                                _p(np.ascontiguousarray(q["geo_a_ref"]), C.c_uint32),
                                _p(np.ascontiguousarray(q["geo_b"]), C.c_float),
                                _p(np.ascontiguousarray(q["geo_b_ref"]), C.c_uint32),
                                _p(d, C.c_float), _p(st, C.c_uint32))
    assert _same(d, q["geo_dist"])
    harness.hchk_free(h)


def test_navmesh_parser_rejects_bad_input(harness, tmp_path):
    good = open(scene_path("c0"), "rb").read()
    cases = {
        "short": good[:20],
        "magic": b"XXXX" + good[4:],
        "version": good[:4] + (2).to_bytes(4, "little") + good[8:],
        "truncated_tile": good[:len(good) // 2],
        "tile_magic": good[:48] + b"\0\0\0\0" + good[52:],
        "two_tiles": good[:8] + (2).to_bytes(4, "little") + good[12:] + good[40:],
    }
    for name, blob in cases.items():
        p = tmp_path / f"{name}.navmesh"
        p.write_bytes(blob)
        err = C.create_string_buffer(256)
        h = harness.hchk_load(str(p).encode(), err, 256)
        assert not h, name
        assert err.value.startswith(b"navmesh:"), (name, err.value)
    err = C.create_string_buffer(256)
    h = C.c_void_p(harness.hchk_load(scene_path("c0").encode(), err, 256))
    info = (C.c_int * 6)()
    harness.hchk_info(h, info)
    assert info[0] == 87 and info[3] == 0 and info[4] == 23  # polys, disabled, islands
    harness.hchk_free(h)


# ------------------------------------------------------------------ C ABI

def test_library_exports_every_declared_symbol():
    from bps_nav_b200 import _lib
    hdr = open(os.path.join(ROOT, "include", "bpsn.h")).read()
    declared = set(re.findall(r"\b(bpsn_[a-z_0-9]+)\s*\(", hdr))
    declared -= {"bpsn_sim"}
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    lib = _lib.load()
    for name in declared:
        assert getattr(lib, name) is not None
    assert b"sm_100a" in lib.bpsn_version()


def test_create_validates_arguments_and_needs_a_gpu():
    import torch
    from bps_nav_b200 import _lib as L
    lib = L.load()
    h = C.c_void_p()
    bad = L.Config(gpu_id=0, num_envs=10, num_groups=1, num_scenes=3, seed=0, flags=0, task=0)
    assert lib.bpsn_create(C.byref(bad), C.byref(h)) == L.ERR_INVALID_ARG
    assert b"multiple" in lib.bpsn_last_error(None)
    assert lib.bpsn_create(None, C.byref(h)) == L.ERR_INVALID_ARG
    if not torch.cuda.is_available():
        ok = L.Config(gpu_id=0, num_envs=8, num_groups=1, num_scenes=1, seed=0, flags=0, task=0)
        assert lib.bpsn_create(C.byref(ok), C.byref(h)) == L.ERR_NO_DEVICE
        # the Python mirror surfaces it as an exception: no silent CPU fallback
        from bps_nav_b200 import bps_sim
        from conftest import load_scene
        with pytest.raises(RuntimeError, match="BPSN_ERR_NO_DEVICE"):
            bps_sim.PointNavRolloutGenerator.from_scenes([load_scene("c0")], 8)
        from bps_nav_b200 import rollout
        t = torch.zeros(3, 4, 1)
        with pytest.raises(RuntimeError, match="CUDA"):
            rollout.compute_returns(t, t, t.bool(), t, None, 2, 0.99, 0.95)
    assert lib.bpsn_gae(None, None, None, None, None, None, 1, 1, 0.99, 0.95, 0, 1e-5, None,
                        None) == L.ERR_INVALID_ARG


@needs_oracle
def test_oracle_flee_and_exploration_invariants():
    """Flee: info = geodesic distance from the start, reward = its change; Exploration: info =
    visited cells - 1 (non-decreasing within an episode), reward = 0.25 per new cell."""
    eps = np.load(os.path.join(SCENES, "c0.episodes.npy"))
    acts = pyoracle.philox_actions(120, 32, 5, "policy")
    for task in ("flee", "exploration"):
        sim = pyoracle.OracleSim([(scene_path("c0"), eps)], 32, 9, task=task)
        sim.reset()
        prev = np.zeros(32, np.float32)
        for t in range(120):
            sim.step(acts[t])
            info = sim.infos[:, 0].copy()
            scale = np.float32(0.25) if task == "exploration" else np.float32(1)
            assert np.array_equal(sim.rewards, scale * (info - prev))
            if task == "exploration":
                assert (info >= prev).all() and (info == np.round(info)).all()
            done = sim.masks == 0
            assert np.array_equal(done, (acts[t] == 0) | (sim.state()["step"] == 1))
            prev = np.where(done, np.float32(0), info)
        sim.close()


# ------------------------------------------------------------------ dataset / host logic

def test_dataset_round_trip(tmp_path):
    from bps_nav_b200 import dataset
    from conftest import load_scene
    scenes = [load_scene("c0"), load_scene("m15")]
    scenes[0].episodes = scenes[0].episodes[:17]
    scenes[1].episodes = scenes[1].episodes[:5]
    dataset.write_dataset(scenes, str(tmp_path / "eps"), str(tmp_path / "assets"))
    back = dataset.load_dataset(str(tmp_path / "eps"), str(tmp_path / "assets"))
    assert [len(s.episodes) for s in back] == [17, 5]
    for a, b in zip(scenes, back):
        assert os.path.exists(b.navmesh_path)
        for f in ("start_position", "start_rotation", "goal"):
            assert np.array_equal(a.episodes[f], b.episodes[f])
    with pytest.raises(RuntimeError):
        dataset.load_dataset(str(tmp_path / "assets"), str(tmp_path / "assets"))
    # the native reader and the plain-Python one agree record for record
    py = dataset.load_dataset_py(str(tmp_path / "eps"), str(tmp_path / "assets"))
    assert [s.scene_id for s in py] == [s.scene_id for s in back]
    assert [s.navmesh_path for s in py] == [s.navmesh_path for s in back]
    for a, b in zip(py, back):
        assert a.episodes.tobytes() == b.episodes.tobytes()


def test_native_dataset_reader_edge_cases(tmp_path):
    """JSON the writer above never produces: escapes, exponents, nested extras, whitespace,
    an empty file (skipped), two scenes in one file (rejected), malformed input (rejected)."""
    import gzip
    import json
    from bps_nav_b200 import dataset
    d = tmp_path / "eps"
    d.mkdir()
    doc = r'''{ "config" : {"a": [1, 2, {"b": null}], "s": "q\\\"\u00e9\n"},
 "episodes":[
 {"episode_id":"0","scene_id":"dir\/A.glb","start_position":[1e0,-2.5E-1,3],
  "start_rotation":[0,0.70710678,0,0.70710678],"goals":[{"position":[4,5.25,6],"radius":null}],
  "info":{"geodesic_distance":7.5},"shortest_paths":null},
 {"scene_id":"dir/A.glb","goals":[{"radius":0.2,"position":[0.1,0.2,0.3]}],
  "start_rotation":[0,0,0,1],"start_position":[7,8,9],"extra":[true,false]}
]}'''
    with gzip.open(d / "a.json.gz", "wt") as f:
        f.write(doc)
    with gzip.open(d / "b.json.gz", "wt") as f:
        json.dump({"episodes": []}, f)
    got = dataset.load_dataset(str(d), "/assets", num_threads=3)
    assert len(got) == 1 and got[0].scene_id == "dir/A.glb"
    assert got[0].navmesh_path == "/assets/dir/A.navmesh"
    e = got[0].episodes
    assert e["start_position"].tolist() == [[1.0, -0.25, 3.0], [7.0, 8.0, 9.0]]
    assert np.array_equal(e["start_rotation"][0],
                          np.array([0, 0.70710678, 0, 0.70710678], np.float32))
    assert np.array_equal(e["goal"], np.array([[4, 5.25, 6], [0.1, 0.2, 0.3]], np.float32))
    ref = dataset.load_dataset_py(str(d), "/assets")
    assert ref[0].episodes.tobytes() == e.tobytes()
    with gzip.open(d / "c.json.gz", "wt") as f:
        json.dump({"episodes": [
            {"scene_id": "X.glb", "start_position": [0, 0, 0], "start_rotation": [0, 0, 0, 1],
             "goals": [{"position": [1, 1, 1]}]},
            {"scene_id": "Y.glb", "start_position": [0, 0, 0], "start_rotation": [0, 0, 0, 1],
             "goals": [{"position": [1, 1, 1]}]}]}, f)
    with pytest.raises(RuntimeError, match="one scene"):
        dataset.load_dataset(str(d), "/assets")
    os.remove(d / "c.json.gz")
    with gzip.open(d / "c.json.gz", "wt") as f:
        f.write('{"episodes": [ {"scene_id": "X.glb", ')
    with pytest.raises(RuntimeError):
        dataset.load_dataset(str(d), "/assets")
    os.remove(d / "c.json.gz")
    (d / "c.json.gz").write_bytes(b"this is not gzip")  # zlib reads it as plain text: bad JSON
    with pytest.raises(RuntimeError):
        dataset.load_dataset(str(d), "/assets")


def test_active_scene_selection_matches_std_mt19937(tmp_path):
    """Selection sampling of simulator.cpp:1518-1534 against the C++ standard library itself."""
    from bps_nav_b200 import dataset
    src = tmp_path / "sel.cpp"
    src.write_text(r'''
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>
int main(int argc, char** argv) {
  unsigned long long seed = strtoull(argv[1], 0, 10); unsigned n = atoi(argv[2]), k = atoi(argv[3]);
  std::mt19937 rgen(seed); std::uniform_real_distribution<> d(0.f, 1.f); std::vector<unsigned> act;
  for (unsigned i = 0; i < n && act.size() < k; i++) {
    float w = d(rgen);
    if (w * float(n - i) < float(k - act.size())) act.push_back(i);
  }
  for (unsigned a : act) printf("%u ", a);
  return 0;
}''')
    exe = tmp_path / "sel"
    subprocess.run(["g++", "-O1", "-o", str(exe), str(src)], check=True)
    for seed, n, k in [(0, 10, 3), (5, 72, 16), (12345, 64, 64), (7, 100, 1)]:
        out = subprocess.run([str(exe), str(seed), str(n), str(k)], capture_output=True, text=True,
                             check=True).stdout.split()
        active, inactive = dataset.select_active_scenes(n, k, seed)
        assert active == [int(x) for x in out]
        assert sorted(active + inactive) == list(range(n))


def test_bench_reference_arm_prints_contract_line():
    if not pyoracle.available():
        pytest.skip("oracle not built")
    import json
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                          "--steps", "1", "--warmup", "0", "--envs", "256", "--cpu-seconds", "0.2"],
                         capture_output=True, text=True, check=True).stdout.strip().splitlines()[-1]
    line = json.loads(out)
    assert line["impl"] == "reference" and line["value"] > 0
    assert line["cpu_baseline"]["cores"] >= 1 and line["e2e"]["h2d_bytes_per_step"] == 0


# ------------------------------------------------------------------ N > 1 plumbing (gloo, CPU)

def _dist_worker(rank, world, port, q):
    import torch.distributed as dist
    from bps_nav_b200 import dist_utils
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    assert dist_utils.rank_info() == (rank, world, rank)
    dist.barrier()
    mx = dist_utils.max_over_ranks(10.0 + rank)
    sm = dist_utils.sum_over_ranks(4096)
    seed = dist_utils.shard_seed(1000, rank, 4096)
    # each rank's episode stream is its own: same env index, different key
    r = pyoracle._philox4x32(np.arange(8), 0, 0, 0, seed & 0xffffffff, seed >> 32)[0]
    q.put((rank, mx, sm, seed, r.tolist()))
    dist.destroy_process_group()


def test_two_rank_sharding_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_dist_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert [r[1] for r in res] == [11.0, 11.0]          # max over ranks, same on every rank
    assert [r[2] for r in res] == [8192.0, 8192.0]      # whole-job env count
    assert res[0][3] == 1000 and res[1][3] == 1000 + 4096
    assert res[0][4] != res[1][4]


def test_shard_plan_partitions_a_fixed_global_batch():
    from bps_nav_b200 import dist_utils
    # benchmark config 3: 16384 environments over 16 scenes, on 1 / 2 / 4 / 8 ranks
    for world in (1, 2, 4, 8):
        seen_envs, seen_scenes = [], set()
        for rank in range(world):
            first, count, scene_ids, env_scene = dist_utils.shard_plan(16384, 16, rank, world)
            assert count == 16384 // world and first == rank * count
            assert len(scene_ids) == 16 // world and len(env_scene) == count
            # every environment keeps the scene it has in the global batch
            assert all(scene_ids[env_scene[i]] == (first + i) // 1024 for i in range(0, count, 97))
            seen_envs.extend(range(first, first + count))
            seen_scenes.update(scene_ids)
        assert seen_envs == list(range(16384)) and seen_scenes == set(range(16))
    # more ranks than scenes: ranks share a scene, each with its part of the environments
    first, count, scene_ids, env_scene = dist_utils.shard_plan(4096, 2, 3, 8)
    assert (first, count, scene_ids) == (1536, 512, [0]) and set(env_scene) == {0}
    # a block that straddles two scenes
    first, count, scene_ids, env_scene = dist_utils.shard_plan(600, 3, 1, 2)
    assert scene_ids == [1, 2] and env_scene.count(0) == 100 and env_scene.count(1) == 200
    with pytest.raises(ValueError):
        dist_utils.shard_plan(1000, 16, 0, 3)


def test_depth_oracle_known_answers():
    """The CPU restatement of the depth sensor on a scene whose image is known in closed form."""
    from oracle import pyoracle
    # agent at (5, 0, 5), identity rotation = looking down -Z; a 2 m high box face at z = 3
    d = pyoracle.depth_reference([5, 0, 5], [0, 0, 0, 1], (0, 0, 10, 10), [[4, 0, 2, 6, 2, 3]],
                                 64, 64)
    assert d.shape == (64, 64) and d.dtype == np.float32
    assert d[32, 32] == np.float32(2.0)              # optical axis hits the face 2 m ahead
    assert d[0, 32] == np.float32(1000.0)            # 45 degrees up: over the box, nothing there
    v = 1.0 - (63 + 0.5) / 64 * 2.0                  # bottom row: the floor, depth = 1.25 / |v|
    assert abs(d[63, 32] - 1.25 / abs(v)) < 1e-5
    # turned by 180 degrees about +Y the agent looks at the floor's far edge and then the void
    d2 = pyoracle.depth_reference([5, 0, 5], [0, 1, 0, 0], (0, 0, 10, 10), [[4, 0, 2, 6, 2, 3]],
                                  64, 64)
    assert d2[32, 32] == np.float32(1000.0) and d2[63, 32] == d[63, 32]
