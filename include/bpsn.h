/*
 * bpsn -- batch PointGoal-navigation environment step and rollout returns on
 * one NVIDIA B200 (sm_100a).  Plain C ABI: opaque handle, pointers and sizes
 * only.  Every entry point returns 0 on success or a BPSN_ERR_* code; none of
 * them aborts the process or throws.  bpsn_last_error() gives a message for
 * the most recent failure on a handle (or for handle-less calls, a
 * thread-local message when called with NULL).
 *
 * What each group of entry points replaces in the reference (paths relative
 * to the bps-nav tree):
 *
 *   bpsn_create / bpsn_destroy / bpsn_set_navmesh* / bpsn_set_episodes /
 *   bpsn_finalize
 *       RolloutGenerator construction: dataset + navmesh loading, environment
 *       groups, per-thread PathFinder replicas.
 *       simulator/simulator.cpp:1463-1617, 1712-1730; PathFinder::loadNavMesh,
 *       simulator/external/habitat-sim-geodesic/habitat_sim_geodesic/csrc/PathFinder.cpp:330-408
 *   bpsn_reset
 *       RolloutGenerator::reset(group)          simulator/simulator.cpp:1377-1380, 601-618
 *   bpsn_step_start / bpsn_step_end
 *       RolloutGenerator::stepStart / stepEnd   simulator/simulator.cpp:1382-1399,
 *       the work loop :1619-1653 and BaseSimulator::step :620-641
 *   bpsn_get_ptr
 *       getRewards / getMasks / getInfos / getPolars (zero-copy result views)
 *                                               simulator/simulator.cpp:1242-1262, 1426-1445
 *   bpsn_query_snap / bpsn_query_try_step / bpsn_query_geodesic
 *       PathFinder::snapPoint / tryStep / findPath in batch form
 *                                               .../csrc/PathFinder.h:99-227
 *   bpsn_gae
 *       RolloutStorage.compute_returns          bps_nav/common/rollout_storage.py:203-219
 *       PPO.get_advantages                      bps_nav/rl/ppo/ppo.py:190-201
 *   bpsn_adv_normalize
 *       PPO.get_advantages over concatenated buffers or per range of environments
 *   bpsn_adv_mean / bpsn_adv_ema_shift
 *       DecentralizedDistributedMixin._get_advantages_distributed
 *                                               bps_nav/rl/ddppo/algo/ddppo.py:18-64
 */
#ifndef BPSN_H
#define BPSN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct bpsn_sim bpsn_sim;

enum {
  BPSN_OK = 0,
  BPSN_ERR_INVALID_ARG = 1,   /* null pointer, index out of range, bad size */
  BPSN_ERR_BAD_NAVMESH = 2,   /* navmesh file/blob rejected; see bpsn_last_error */
  BPSN_ERR_CUDA = 3,          /* a CUDA runtime call failed */
  BPSN_ERR_STATE = 4,         /* call order violated (e.g. step_start twice) */
  BPSN_ERR_BAD_ACTION = 5,    /* an action outside {0,1,2,3} */
  BPSN_ERR_IO = 6,            /* file could not be read */
  BPSN_ERR_NO_DEVICE = 7      /* no usable CUDA device */
};

/* Episode record: simulator/simulator.cpp:83-87 (rotation stored x, y, z, w). */
typedef struct {
  float start_position[3];
  float start_rotation[4];
  float goal[3];
} bpsn_episode;

typedef struct {
  int32_t gpu_id;            /* CUDA device ordinal */
  uint32_t num_envs;         /* environments over all groups */
  uint32_t num_groups;       /* 1, or 2 for double buffering */
  uint32_t num_scenes;       /* scenes resident on the device */
  uint64_t seed;             /* seeds the episode-selection stream */
  uint32_t flags;            /* BPSN_FLAG_* */
  uint32_t task;             /* BPSN_TASK_* */
  uint32_t render_width;     /* depth sensor image width  (0 with render_height 0: no sensor) */
  uint32_t render_height;    /* depth sensor image height                                    */
  uint32_t num_active_scenes; /* scenes in use at a time; 0 = all of them.  With fewer than
                                 num_scenes the others wait in a pool and the environments move
                                 through the whole dataset, num_envs / num_active_scenes
                                 consecutive environments (a "slot") at a time: when all
                                 environments of a slot have reached its scene the slot draws
                                 another one from the pool, and each environment follows at the
                                 end of its running episode (SceneSwapper / EnvironmentGroup::
                                 swapScene, simulator/simulator.cpp:1063-1154, 1284-1308,
                                 1636-1640).  Every scene's navigation mesh stays resident. */
  uint32_t swap_interval;    /* 0: a slot draws its next scene as soon as all of its
                                 environments have arrived.  k > 0: a group starts at most one
                                 such move every k of its steps -- the pace of the reference's
                                 single background loader, which hands over one scene at a time
                                 (BackgroundSceneLoader, simulator/simulator.cpp:462-550). */
} bpsn_config;

/* Tasks of the reference's three generators (simulator/simulator.cpp:734-999,
 * 1812-1822).  They share motion, sensor, done rule and reset; they differ in
 * the info record and the reward:
 *   POINTNAV     info {success, spl, distanceToGoal}; reward -dGeodesic + 2.5*spl - 0.01
 *   FLEE         info {distanceFromStart} (geodesic, refreshed on moves); reward = its increase
 *   EXPLORATION  info {numVisited} 1 m cells visited - 1;               reward 0.25 per new cell */
enum { BPSN_TASK_POINTNAV = 0, BPSN_TASK_FLEE = 1, BPSN_TASK_EXPLORATION = 2 };

enum {
  /* keep pinned host copies of reward/mask/info/polar, refreshed by every
     step/reset and complete when bpsn_step_end returns (reference behaviour:
     the result arrays are host memory) */
  BPSN_FLAG_HOST_MIRRORS = 1u << 0,
  /* always use the generic one-thread-per-environment step kernel (tables and
     A* scratch in global memory) instead of the shared-memory warp kernel;
     it is otherwise chosen only for scenes too large for shared memory */
  BPSN_FLAG_GENERIC_KERNEL = 1u << 1,
  /* warp kernel only: run every A* search with the reference's binary heap kept
     in shared memory, the path otherwise taken only when the register open list
     cannot decide the pop order (a tie for the minimum) -- for testing that path */
  BPSN_FLAG_EXACT_HEAP = 1u << 2,
  /* plan the step kernels as if a CTA had 96 KB of shared memory instead of 227 KB:
     medium-sized scenes then go to the generic kernel while small ones stay on the
     warp kernel -- for testing groups that need both kernels in one step */
  BPSN_FLAG_SMEM_96K = 1u << 3,
  /* work on every scene in global memory (tables and A* slabs L2 / L1 resident, two CTAs
     per SM) whatever its size; the planner otherwise does this only for large batches
     that contain a scene too big to share an SM's shared memory with 8 slabs */
  BPSN_FLAG_GLOBAL_MEMORY = 1u << 4,
  /* always run a step as two launches (k_pre, then the step kernel on work lists in global
     memory); small batches of fixed scenes otherwise use one launch that does both -- for
     testing the two-launch form on batches of any size */
  BPSN_FLAG_TWO_LAUNCHES = 1u << 5
};

/* Fields addressable through bpsn_get_ptr.  All arrays are indexed by the
 * environment's position inside its group. */
enum {
  BPSN_FIELD_REWARD = 0,     /* float32 [B]                               */
  BPSN_FIELD_MASK = 1,       /* uint8   [B]   1 = episode continues       */
  BPSN_FIELD_INFO = 2,       /* float32 [B,3] success, spl, distanceToGoal (PointNav);
                                float32 [B] distanceFromStart (Flee) / numVisited (Exploration) */
  BPSN_FIELD_POLAR = 3,      /* float32 [B,2] rho, -phi                   */
  BPSN_FIELD_POSITION = 4,   /* float32 [3,B] x | y | z                   */
  BPSN_FIELD_ROTATION = 5,   /* float32 [4,B] x | y | z | w               */
  BPSN_FIELD_GOAL = 6,       /* float32 [3,B]                             */
  BPSN_FIELD_NAV_POSITION = 7, /* float32 [3,B] position on the navmesh   */
  BPSN_FIELD_NAV_POLY = 8,   /* uint32  [B]   Detour polygon ref          */
  BPSN_FIELD_GOAL_POLY = 9,  /* uint32  [B]                               */
  BPSN_FIELD_STEP = 10,      /* uint32  [B]   step counter (starts at 1)  */
  BPSN_FIELD_EPISODE = 11,   /* uint32  [B]   index of the current episode*/
  BPSN_FIELD_RESET_COUNT = 12, /* uint32 [B]  episodes started so far     */
  BPSN_FIELD_STATUS = 13,    /* uint32  [B]   sticky diagnostic bits      */
  BPSN_FIELD_PREV_DIST = 14, /* float32 [B]                               */
  BPSN_FIELD_CUM_TRAVEL = 15,/* float32 [B]                               */
  BPSN_FIELD_INIT_DIST = 16, /* float32 [B]                               */
  BPSN_FIELD_SCENE = 17,     /* uint32  [B]   scene index of the env      */
  BPSN_FIELD_EPISODE_REWARD = 18, /* float32 [B] reward accumulated in the running episode */
  BPSN_FIELD_EPISODE_STATS = 19,  /* float32 [5,B] sums over finished episodes: reward | count |
                                     success | spl | distanceToGoal (what PPOTrainer._update_stats
                                     keeps, bps_nav/rl/ppo/ppo_trainer.py:286-319); zero them to
                                     restart a window */
  BPSN_FIELD_DEPTH = 20,     /* float32 [B,H,W] depth sensor image of the last bpsn_render
                                (only when the handle was created with a render size)    */
  BPSN_FIELD_COUNT = 21
};

enum { BPSN_MEM_DEVICE = 0, BPSN_MEM_HOST = 1 };

int32_t bpsn_create(const bpsn_config* cfg, bpsn_sim** out);
int32_t bpsn_destroy(bpsn_sim* sim);

/* Scene `scene` <- a `.navmesh` file (MSET container, one Detour tile). */
int32_t bpsn_set_navmesh_file(bpsn_sim* sim, uint32_t scene, const char* path);
int32_t bpsn_set_navmesh_blob(bpsn_sim* sim, uint32_t scene, const void* data, size_t size);
/* Episode list of a scene (copied). */
int32_t bpsn_set_episodes(bpsn_sim* sim, uint32_t scene, const bpsn_episode* episodes,
                          uint32_t count);
/* Optional: the scenes that are in use first, one per slot (count = num_active_scenes;
 * default 0 .. num_active_scenes - 1).  The reference draws them with std::mt19937(seed)
 * (simulator/simulator.cpp:1518-1534). */
int32_t bpsn_set_active_scenes(bpsn_sim* sim, const uint32_t* scenes, uint32_t count);
/* Scene rotation so far (RolloutGenerator::swapStats, simulator/simulator.cpp:1412-1424):
 * moves of a slot to another scene started since creation, the number of different scenes
 * the environments are in right now and the mean number of environments per such scene, both
 * summed over the groups as the reference does.  Waits for the steps in flight. */
int32_t bpsn_swap_stats(bpsn_sim* sim, uint64_t* num_swaps, float* scenes_in_use,
                        float* envs_per_scene);
/* Optional: explicit scene per environment (default: num_envs / num_scenes
 * consecutive environments per scene, group-major then scene-major, as in
 * simulator/simulator.cpp:1205-1221, 1581-1592).  Only with every scene active. */
int32_t bpsn_set_env_scenes(bpsn_sim* sim, const uint32_t* env_scene, uint32_t count);
/* Uploads scenes and episodes, allocates state, outputs and query scratch. */
/* Render geometry of a scene for the depth sensor: the floor rectangle at y = 0
 * (floor4 = xmin, zmin, xmax, zmax) and `num_boxes` axis-aligned boxes of 6 floats
 * each (min xyz, max xyz).  Stands in for the render asset the reference loads per
 * scene (Dataset::getScenePath + AssetLoader::loadScene, simulator/simulator.cpp:
 * 330-342, 1209-1210).  Optional; before bpsn_finalize.  Scenes without geometry
 * render as empty space (every pixel at the far plane). */
int32_t bpsn_set_scene_geometry(bpsn_sim* sim, uint32_t scene, const float* floor4,
                                const float* boxes, uint32_t num_boxes);

int32_t bpsn_finalize(bpsn_sim* sim);

/* Starts a fresh episode in every environment of the group.  Asynchronous on
 * `stream` (a cudaStream_t, NULL = default stream). */
int32_t bpsn_reset(bpsn_sim* sim, uint32_t group, void* stream);

/* actions: int64 [B], one of {0 stop, 1 forward, 2 left, 3 right}.
 * actions_mem = BPSN_MEM_HOST: validated, staged and copied by the call;
 * BPSN_MEM_DEVICE: read by the kernels as is (an out-of-range value sets the
 * environment's BAD_ACTION status bit and that environment does not move); any
 * address the device can read will do, page-locked host memory included (the
 * kernels then read the actions over the bus; they must stay unchanged until
 * the step has run).
 * The step is enqueued on `stream`; bpsn_step_end waits for it when host
 * mirrors are enabled and otherwise only closes the start/end pairing. */
int32_t bpsn_step_start(bpsn_sim* sim, uint32_t group, const int64_t* actions,
                        int32_t actions_mem, void* stream);
/* As bpsn_step_start, and the step's reward (float32 [B]), mask (uint8 [B])
 * and GPS/compass observation (float32 [B,2]) are also written to the given
 * DEVICE arrays when non-NULL -- e.g. rows rewards[t], masks[t+1] and
 * observations[t+1] of rollout storage, which the reference fills with separate
 * copies (RolloutStorage.insert, bps_nav/common/rollout_storage.py:130-183). */
int32_t bpsn_step_start_ex(bpsn_sim* sim, uint32_t group, const int64_t* actions,
                           int32_t actions_mem, void* stream, float* reward_out,
                           uint8_t* mask_out, float* polar_out);
int32_t bpsn_step_end(bpsn_sim* sim, uint32_t group);

/* RolloutGenerator::render (simulator/simulator.cpp:1400-1410): renders the depth
 * image of every environment of the group from its current pose into
 * BPSN_FIELD_DEPTH, asynchronously on `stream`.  Camera as the reference sets it
 * up: eye = position + 1.25 * up, looking down -Z of the agent frame, 90 degree
 * vertical field of view, near 0.1, far 1000 (simulator.cpp:651-663, 1216); pixel
 * value = view-space depth in metres, 1000 where nothing is hit.  The geometry is
 * what bpsn_set_scene_geometry gave (the reference rasterises a mesh with bps3D,
 * which is not part of its tree).  BPSN_ERR_STATE without a render size. */
int32_t bpsn_render(bpsn_sim* sim, uint32_t group, void* stream);

/* Pointer to a per-group array; mem selects device memory or (for the four
 * result fields, when BPSN_FLAG_HOST_MIRRORS is set) the pinned host copy.
 * Addresses are stable for the life of the handle. */
int32_t bpsn_get_ptr(bpsn_sim* sim, uint32_t group, int32_t field, int32_t mem, void** ptr,
                     size_t* bytes);

/* Sticky device-side error word of a group (synchronous read; no counterpart
 * in the reference, which aborts on inconsistencies).  Bit 0: a step kernel gave
 * up waiting for its scene tables to arrive in shared memory and skipped its
 * work.  Zero in normal operation.  With host mirrors bpsn_step_end also checks the word
 * and returns BPSN_ERR_CUDA once it is set. */
int32_t bpsn_device_error_flags(bpsn_sim* sim, uint32_t group, uint32_t* flags);

/* Per-kernel device timing of the step (no counterpart in the reference; its
 * Python side times phases with wall clocks, bps_nav/common/utils.py:387-436).
 * While enabled, bpsn_step_end waits for the step and adds the CUDA-event
 * duration of each of its two launches, in order: pre (action decode, turns,
 * sensor, envs that need no navmesh query) and step (forward move, geodesic,
 * reward, reset), to running totals in milliseconds. */
int32_t bpsn_profile_enable(bpsn_sim* sim, uint32_t group, int32_t enable);
int32_t bpsn_profile_read(bpsn_sim* sim, uint32_t group, double* ms2, uint64_t* steps);

/* Number of polygons / disabled polygons / islands of a loaded scene. */
int32_t bpsn_scene_info(bpsn_sim* sim, uint32_t scene, int32_t* num_polys, int32_t* num_disabled,
                        int32_t* num_islands);

/* Batched navigation queries on one scene.  All pointers are DEVICE pointers;
 * positions are float32 [n,3], polygon refs uint32 [n]. */
int32_t bpsn_query_snap(bpsn_sim* sim, uint32_t scene, uint32_t n, const float* points,
                        float* out_points, uint32_t* out_refs, void* stream);
int32_t bpsn_query_try_step(bpsn_sim* sim, uint32_t scene, uint32_t n, const float* start,
                            const uint32_t* start_refs, const float* end, float* out_points,
                            uint32_t* out_refs, void* stream);
int32_t bpsn_query_geodesic(bpsn_sim* sim, uint32_t scene, uint32_t n, const float* start,
                            const uint32_t* start_refs, const float* end,
                            const uint32_t* end_refs, float* out_dist, uint32_t* out_status,
                            void* stream);

/* Generalised advantage estimation over a rollout of T steps and N
 * environments; every pointer is a DEVICE pointer.
 *   rewards, values, returns : float32 [T+1, N]   (row-major; trailing 1 dims ok)
 *   masks                    : uint8/bool [T+1, N], masks[t+1] = not done after step t
 *   next_value               : float32 [N] or NULL; when given it is stored to
 *                              values[T] first (compute_returns does the same)
 *   advantages               : float32 [T, N] or NULL; = returns[:T] - values[:T],
 *                              then, if normalize != 0, (a - mean) / (std + eps)
 *                              with the unbiased std over all T*N elements
 *   gamma, tau               : doubles, because the reference folds gamma*tau in
 *                              double before rounding to float32
 *   workspace                : device scratch of at least bpsn_gae_workspace_bytes(N)
 */
size_t bpsn_gae_workspace_bytes(uint32_t N);
int32_t bpsn_gae(const float* rewards, float* values, const uint8_t* masks,
                 const float* next_value, float* returns, float* advantages, uint32_t T,
                 uint32_t N, double gamma, double tau, int32_t normalize, float eps,
                 void* workspace, void* stream);

/* Advantage normalisation over segments of environments; every tensor pointer is a DEVICE
 * pointer, the segment list itself is HOST memory (read during the call).
 *
 * A segment is a range of environment columns [start, end) of one float32 [T, N] advantage
 * tensor (row-major; rows of N).  Segments with the same `group` number are normalised
 * together, over all T * (end - start) elements of all of them:
 *   - one segment {adv, N, 0, N, 0}: the whole batch, PPO.get_advantages
 *     (bps_nav/rl/ppo/ppo.py:190-201): (a - mean) / (std + eps), unbiased std;
 *   - the two halves of a double-buffered rollout as two segments of one group: what the
 *     reference computes on torch.cat(advantages, 1) (ppo.py:191-198);
 *   - k ranges of environments with k different group numbers: each range on its own
 *     statistics (per-minibatch normalisation; the reference's minibatches are sets of
 *     environments, bps_nav/common/rollout_storage.py:228-238).
 * Segments must not overlap.  At most BPSN_MAX_ADV_SEGMENTS per call.  `workspace`: device
 * scratch of at least bpsn_adv_workspace_bytes() bytes. */
#define BPSN_MAX_ADV_SEGMENTS 64
typedef struct {
  float* advantages; /* device, [T, N] */
  uint32_t N;        /* row length of that tensor */
  uint32_t start;    /* first environment column of the segment */
  uint32_t end;      /* one past the last */
  uint32_t group;    /* segments with equal group numbers share mean and std */
} bpsn_adv_segment;
size_t bpsn_adv_workspace_bytes(void);
int32_t bpsn_adv_normalize(const bpsn_adv_segment* segments, uint32_t num_segments, uint32_t T,
                           float eps, void* workspace, void* stream);

/* The advantage baseline DD-PPO installs instead (DecentralizedDistributedMixin.
 * _get_advantages_distributed, bps_nav/rl/ddppo/algo/ddppo.py:46-64): advantages minus the
 * bias-corrected exponential moving average of their mean; no division by the std.
 *   bpsn_adv_mean       *mean_out (device float) <- mean over every element of every segment.
 *                       With several workers the caller all-reduces it and divides by the
 *                       world size, as distributed_mean_and_var does (ddppo.py:18-42).
 *   bpsn_adv_ema_shift  ema_state (device float[3]: biased, unbias, last shift; start at 0):
 *                       biased = beta * biased + (1 - beta) * mean; unbias = beta * unbias +
 *                       (1 - beta); every element of every segment -= biased / unbias.
 *                       The reference uses beta = 0.8. */
int32_t bpsn_adv_mean(const bpsn_adv_segment* segments, uint32_t num_segments, uint32_t T,
                      float* mean_out, void* workspace, void* stream);
int32_t bpsn_adv_ema_shift(const bpsn_adv_segment* segments, uint32_t num_segments, uint32_t T,
                           float* ema_state, const float* mean, float beta, void* stream);

/* bpsn_gae without any allocation.  No counterpart in the reference.
 *
 * Some hosts of this library may not allocate GPU memory at the moment they
 * need returns computed: a trainer that sized its memory pool up front and
 * treats any later cudaMalloc as a bug, an embedding process whose allocator
 * is owned by another runtime, or code running between two phases that must
 * not disturb the allocator's state.  bpsn_gae asks such a caller for a device
 * workspace; this variant does not.  Its per-block scratch is a fixed 48 KB
 * array inside the library image (every GPU that loads the library carries it
 * until the process exits), and the call itself performs no cudaMalloc /
 * cudaFree / host allocation.  Inputs and outputs are still the caller's.
 *
 *   - Limit: N <= 262144 environments per call; larger N is rejected with
 *     BPSN_ERR_INVALID_ARG (use bpsn_gae with your own workspace).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current).  Make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one array.  Two calls whose kernels can
 *     overlap on the GPU (different streams, no ordering between them) race on
 *     it; serialise them.  Nothing in the array needs clearing between calls.
 * Arguments and results are those of bpsn_gae, minus `workspace`. */
int32_t bpsn_gae_static(const float* rewards, float* values, const uint8_t* masks,
                        const float* next_value, float* returns, float* advantages, uint32_t T,
                        uint32_t N, double gamma, double tau, int32_t normalize, float eps,
                        void* stream);

/* Self-test of the library's arithmetic contract.  Navigation-mesh queries take
 * square roots with a hand-written estimate-and-correct sequence that must
 * return exactly what IEEE sqrtf returns (results feed discrete decisions:
 * A* pop order, funnel side tests).  This compares the two on the GPU for every
 * fp32 bit pattern in [first_bits, last_bits] and returns the number of
 * operands on which they differ (expected: 0 for any range, including zero,
 * denormals, negatives, inf and NaN patterns).  The whole positive range
 * 0x00000000..0x7f800000 takes about a second.  Allocates 8 bytes of device
 * memory for the duration of the call. */
int32_t bpsn_selftest_sqrt(int32_t gpu_id, uint32_t first_bits, uint32_t last_bits,
                           uint64_t* mismatches);

/* Episode datasets on disk (Dataset, simulator/simulator.cpp:190-359): a directory of
 * `*.json.gz` Habitat PointNav episode files, one scene per file.  bpsn_dataset_open
 * reads them all on up to `num_threads` host threads; scenes come back in file-name
 * order.  bpsn_dataset_scene returns pointers into the dataset object (valid until
 * bpsn_dataset_close): the scene id as written in the file, the navmesh path derived
 * from it (asset_path / scene id with its extension replaced by ".navmesh") and the
 * episode records, ready for bpsn_set_navmesh_file / bpsn_set_episodes.  On failure
 * the message is available from bpsn_last_error(NULL).  No GPU is involved. */
typedef struct bpsn_dataset bpsn_dataset;
int32_t bpsn_dataset_open(const char* dataset_path, const char* asset_path, uint32_t num_threads,
                          bpsn_dataset** out);
uint32_t bpsn_dataset_num_scenes(const bpsn_dataset* ds);
int32_t bpsn_dataset_scene(const bpsn_dataset* ds, uint32_t index, const char** scene_id,
                           const char** navmesh_path, const bpsn_episode** episodes,
                           uint32_t* num_episodes);
void bpsn_dataset_close(bpsn_dataset* ds);

const char* bpsn_last_error(const bpsn_sim* sim);
/* Library build identification, e.g. "bpsn sm_100a". */
const char* bpsn_version(void);

#ifdef __cplusplus
}
#endif

#endif /* BPSN_H */
