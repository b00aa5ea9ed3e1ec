// Per-environment PointNav state machine as CUDA kernels.
//
// One environment step of the reference (BaseSimulator::step followed by the
// in-loop auto-reset, simulator/simulator.cpp:620-641, 1626-1644) is two
// launches:
//
//   k_pre   one thread per env: decode the action, advance the step counter,
//           apply a turn (handleMovement :696-703) and refresh the GPS/compass
//           (updateObservationState :651-677).  An env that did not move needs
//           no navmesh query: on a turn it reports the distance of the step
//           before (InfoFunctor::step :784-786); when its episode ends it
//           reports the distance kept for that (GroupDev::doneDist) and is
//           reset by table lookup.  Its info / reward / mask are written here.
//           Envs that moved forward are appended to their slot's work list.
//   k_step_warp / k_step_thread
//           one warp (scene tables in shared memory, geo_warp.cuh) or one
//           thread (tables in global memory) per listed env: forward move
//           (PathFinder::tryStep, handleMovement :684-695), GPS/compass,
//           geodesic goal -> agent (InfoFunctor::step :758-790), success / SPL /
//           reward / mask (RewardFunctor::step :808-822) and, when the episode
//           finished, the reset (BaseSimulator::reset :601-618,
//           InfoFunctor::reset :744-756, RewardFunctor::reset :801-806).
// (Small batches of fixed scenes run both parts in one launch, geo_warp.cuh.)
//
// Tasks.  PointNav is described above.  Flee (simulator.cpp:830-887): the info is the
// geodesic distance from the episode's snapped start to the agent, refreshed only when
// the agent moved, reward = its increase; the start point is kept in the navGoal /
// goalRef columns so the same query code serves both tasks.  Exploration
// (simulator.cpp:889-999): the info is the number of 1 m grid cells (in the frame of
// the initial pose) visited so far minus one, reward = 0.25 per new cell; no
// geodesic query at all.
//
// Everything reset() derives from the chosen episode alone -- the snapped
// start point, the snapped goal and the initial geodesic distance agent ->
// goal (:611-612, :747-752) -- is a pure function of the episode record, so it
// is evaluated once per episode when the scenes are uploaded (k_episode_table,
// same device functions) and a reset becomes a table lookup.  The values are
// bit-identical to evaluating them at every reset as the reference does.
//
// State is structure-of-arrays per group so that each phase reads and writes
// coalesced 4-byte columns.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "nav_query.cuh"

namespace bpsn {

enum Task : uint32_t { kTaskPointNav = 0, kTaskFlee = 1, kTaskExploration = 2 };

// work-list entries: environment index in the low 30 bits, the action's outcome above
constexpr uint32_t kListEnvMask = 0x3fffffffu;
constexpr uint32_t kListDone = 1u << 30;   // the episode ends with this step
constexpr uint32_t kListMoved = 1u << 31;  // MoveForward

constexpr uint32_t kVisitedSlots = 1024;  // per-env open-addressing table of visited grid cells

struct GroupDev {
  uint32_t B;          // environments in this group
  uint32_t envBase;    // global index of the group's first environment
  uint32_t task;       // Task
  uint32_t infoWidth;  // floats per env in `info`: 3 (PointNav) or 1 (Flee, Exploration)
  uint32_t exactHeap;  // test switch: every warp search uses the slab heap (geo_warp.cuh)
  uint32_t numScenes;  // scenes of the simulator (length of the per-scene tables)
  uint32_t numLists;   // work lists of the group: two per slot (see `slot` below)
  uint32_t rotation;   // scenes rotate through the slots (more scenes than slots)
  uint32_t slabPerEnv;  // global-memory slabs are indexed by environment, not by warp (geo_warp.cuh)
  uint32_t globalPcap;  // node capacity every global-memory slab is laid out for
  // pose / task state, each [B] (vectors are component-major: x[B] y[B] z[B])
  float* pos;      // [3][B]  position_
  float* rot;      // [4][B]  rotation_ (x y z w)
  float* goal;     // [3][B]  goal_
  float* navPos;   // [3][B]  navmeshPosition_.xyz
  float* navGoal;  // [3][B]  navmeshGoal_.xyz
  float* prevPos;  // [3][B]  prev_position_
  float* prevDist;
  float* cumTravel;
  float* initDist;
  // What InfoFunctor::step would find if the episode ended now without a move (it searches
  // goal -> agent on every `done`, simulator.cpp:763-767): the distance of the last move's
  // search -- the agent has not left that spot -- or, before the first move, the episode
  // table's goal -> start distance.  An episode that ends on a stop or a turn needs no search.
  float* doneDist;
  uint32_t* navRef;
  uint32_t* goalRef;
  uint32_t* step;
  uint32_t* episode;
  uint32_t* resetCount;
  uint32_t* status;
  uint32_t* scene;
  // outputs
  float* reward;  // [B]
  uint8_t* mask;  // [B]
  float* info;    // [B][infoWidth]
  float* polar;   // [B][2]
  // optional second destination of this step's reward / mask / polar (e.g. rows
  // of rollout storage); null when unused
  float* rewardOut;
  uint8_t* maskOut;
  float* polarOut;  // [B][2]
  // host mirrors of reward / mask / info / polar in mapped pinned memory (null when the
  // handle keeps none): the kernels store every result a second time there, which puts
  // the transfer inside the step instead of a copy after it
  float* hReward;
  uint8_t* hMask;
  float* hInfo;
  float* hPolar;
  uint32_t* hErr;  // host-visible copy of errFlags[0] (same mapped block), null without mirrors
  // Publishing the results to the host in one piece: when pubDst is set the step kernels leave
  // the four mirrors above alone (they are null in the copy of this struct those kernels get);
  // the CTA of the step kernel that finishes last copies the device block [reward | mask |
  // info | polar] to its pinned twin with 16-byte stores and then raises *hStepFlag to stepId.
  // (Thousands of 4-byte stores from single lanes cross the bus as one packet each and cost
  // the step ~10 us; the same bytes in 128-byte packets take ~2 us.)
  const uint4* pubSrc;
  uint4* pubDst;
  uint32_t pubVec;       // 16-byte pieces to copy
  uint32_t* doneCount;   // [1] CTAs of the running step kernel that are through (device)
  uint32_t* hStepFlag;   // mapped host word: number of the last step whose results are out
  uint32_t stepId;
  // running episode statistics, the device-side form of PPOTrainer._update_stats
  // (bps_nav/rl/ppo/ppo_trainer.py:286-319)
  float* episodeReward;  // [B]     reward accumulated in the current episode
  // Exploration task only (simulator/simulator.cpp:889-999)
  float* explInit;       // [7][B]  initial position xyz, inverse initial rotation xyzw
  uint32_t* visited;     // [B][kVisitedSlots] visited cells (0 = empty slot)
  uint32_t* numCells;    // [B]     cells in the set
  float* stats;          // [5][B]  sums over finished episodes: reward, count, success,
                         //         spl, distanceToGoal
  // Slots.  A slot is a fixed set of environments that share a scene: one per scene of the
  // group when the scenes are fixed; `environments / active scenes` consecutive environments
  // when the dataset has more scenes than are active at a time
  // (simulator/simulator.cpp:1205-1221).  Then a slot moves on to another scene whenever all
  // of its environments have reached the current one: every environment follows at the end of
  // its running episode (EnvironmentGroup::swapReady / swapScene, :1284-1308, called from the
  // work loop :1636-1640), so a slot's environments are in at most two scenes at a time, the
  // one it is moving to (`slotScene`) and the one before (`slotPrev`).
  uint32_t* slot;           // [B] slot of each environment (fixed)
  uint32_t* envEpoch;       // [B] number of the slot's move this environment has caught up with
  uint32_t* slotScene;      // [slots] scene the slot's environments are in, or moving to
  uint32_t* slotPrev;       // [slots] scene of those that have not moved yet
  uint32_t* slotEpoch;      // [slots] moves started so far
  uint32_t* slotRemaining;  // [slots] environments that still have to follow the current move
  uint32_t* slotSize;       // [slots] environments of the slot
  uint32_t* slotEnvs;       // [B] the environments ordered by slot (fixed)
  uint32_t* slotEnvBase;    // [slots] where each slot's environments start in slotEnvs
  uint32_t* ovList;         // one-launch step: per CTA, the list entries beyond one per warp
  uint32_t* ovMeta;         // ... and per CTA {count, cursor, step number, -} (geo_warp.cuh)
  uint16_t* batchStage;     // batched step: per warp 32 corridors of up to 256 polygons
  uint32_t* hListed;        // mapped host word: list entries of the last step (the host picks
                            // the next step's form by it)
  uint32_t* pool;           // [poolSize] scenes waiting for a slot
  uint32_t* swapCount;      // [2] moves started (RolloutGenerator::swapStats, :1412-1424); the
                            // step at which the group started its last one
  uint32_t swapInterval;    // steps of the group between two moves at least (0: no limit)
  uint32_t numSlots;
  uint32_t poolSize;
  uint32_t slotBase;        // number of the group's first slot among all slots
  // geodesic work lists, two per slot: list 2 * s holds the slot's listed environments that are
  // in slotScene[s], list 2 * s + 1 those still in slotPrev[s]; list l owns
  // geoList[listBase[l] ...], counts[l] entries are valid this step
  uint32_t* geoList;         // [2 * B]
  uint32_t* counts;          // [2 * numLists]: list lengths, then work-queue cursors
  uint32_t* countsNext;      // the next step's `counts`: the step kernel zeroes it, so that no
                             // separate clearing pass sits between two steps
  uint32_t* errFlags;        // [1] sticky device-side error bits (never cleared by kernels)
  const uint32_t* listBase;  // [numLists]
};

// Per-episode results of reset()'s navmesh queries.
struct alignas(16) EpisodeNav {
  float navStart[3];
  uint32_t startRef;
  float navGoal[3];
  uint32_t goalRef;
  float initDist;      // start -> goal (InfoFunctor::reset)
  uint32_t status;
  float initDistRev;   // goal -> start: what a `done` before the first move reports
  uint32_t statusRev;
};
static_assert(sizeof(EpisodeNav) == 48, "EpisodeNav is 48 bytes");

struct SceneTable {
  const NavScene* scenes;
  const float* episodes;      // 10 floats per record, all scenes concatenated
  const EpisodeNav* epNav;    // one per episode record
  const uint32_t* epOffset;   // [numScenes]
  const uint32_t* epCount;    // [numScenes]
};

// Programmatic dependent launch: a kernel lets the next one in the stream start
// its prologue early (launchDependents) and the next one waits for the whole of
// its predecessor, memory included, before it touches anything the predecessor
// writes (waitForPredecessor).  Both are no-ops for an ordinary launch.
__device__ __forceinline__ void launchDependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void waitForPredecessor() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// How the step kernels divide a group's scenes between them.  A scene whose staged
// image leaves room for at least one warp slab in a CTA's shared memory is handled by
// the warp kernel with `warps` active warps per CTA on `ctas` CTAs; warps == 0 sends the
// scene's environments to the one-thread-per-environment kernel.
struct WarpPlan {
  uint32_t pcap;        // polygon capacity of a slab of this scene (multiple of 16)
  uint32_t slabOffset;  // bytes from the start of dynamic shared memory to the first slab, or
                        // kSlabInGlobal: tables and slabs of this scene stay in global memory
  uint32_t warps;
  uint32_t ctas;
};
constexpr uint32_t kSlabInGlobal = 0xffffffffu;

struct TurnConsts {  // +/-10 degrees about +Y, evaluated once on the host
  float lx, ly, lz, lw;
  float rx, ry, rz, rw;
};

constexpr float kSuccessReward = 2.5f;    // simulator/simulator.cpp:47
constexpr float kSlackReward = 1e-2f;     // :48
constexpr float kSuccessDistance = 0.2f;  // :49
constexpr float kMaxSteps = 500.f;        // :50
constexpr float kForwardStep = 0.25f;     // :51

// Philox-4x32-10 (Salmon et al., SC'11): the episode-selection stream.
__host__ __device__ __forceinline__ uint32_t mulHi32(uint32_t a, uint32_t b) {
  return static_cast<uint32_t>((static_cast<uint64_t>(a) * b) >> 32);
}
__host__ __device__ __forceinline__ uint32_t philoxFirst(uint32_t c0, uint32_t c1, uint32_t c2,
                                                         uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = mulHi32(0xD2511F53u, c0);
    const uint32_t lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = mulHi32(0xCD9E8D57u, c2);
    const uint32_t lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0;
    const uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0;
    c1 = lo1;
    c2 = n2;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

// GPS/compass: polar coordinates of the goal in the agent frame.
__device__ __forceinline__ void writePolar(const GroupDev& g, uint32_t e, float px, float py,
                                           float pz, float qx, float qy, float qz, float qw,
                                           float gx, float gy, float gz) {
  const float qxx = qx * qx, qyy = qy * qy, qzz = qz * qz;
  const float qxz = qx * qz, qxy = qx * qy, qyz = qy * qz;
  const float qwx = qw * qx, qwy = qw * qy, qwz = qw * qz;
  const float m00 = 1.f - 2.f * (qyy + qzz), m01 = 2.f * (qxy + qwz), m02 = 2.f * (qxz - qwy);
  const float m20 = 2.f * (qxz + qwy), m21 = 2.f * (qyz - qwx), m22 = 1.f - 2.f * (qxx + qyy);
  const float tx = gx - px, ty = gy - py, tz = gz - pz;
  const float vx = m00 * tx + m01 * ty + m02 * tz;
  const float vz = m20 * tx + m21 * ty + m22 * tz;
  const float ax = -vz, ay = vx;
  const float rho = sqrtExact(ax * ax + ay * ay);
  const float phi = atan2f(ay, ax);
  reinterpret_cast<float2*>(g.polar)[e] = make_float2(rho, -phi);
  if (g.polarOut)
    reinterpret_cast<float2*>(g.polarOut)[e] = make_float2(rho, -phi);
  if (g.hPolar)
    reinterpret_cast<float2*>(g.hPolar)[e] = make_float2(rho, -phi);
}

// Exploration: cell of the current position in the initial pose's frame,
// InfoFunctor::update (simulator.cpp:897-904).  Returns true if the cell is new.
__device__ __forceinline__ bool explVisit(const GroupDev& g, uint32_t e, float px, float py,
                                          float pz) {
  const uint32_t B = g.B;
  const float dx = px - g.explInit[e];
  const float dy = py - g.explInit[B + e];
  const float dz = pz - g.explInit[2 * B + e];
  const float qx = g.explInit[3 * B + e], qy = g.explInit[4 * B + e];
  const float qz = g.explInit[5 * B + e], qw = g.explInit[6 * B + e];
  // q * v = v + 2 * (w * (q x v) + q x (q x v)), then / cell_size (1.0)
  const float uvx = qy * dz - dy * qz;
  const float uvy = qz * dx - dz * qx;
  const float uvz = qx * dy - dx * qy;
  const float uuvx = qy * uvz - uvy * qz;
  const float uuvy = qz * uvx - uvz * qx;
  const float uuvz = qx * uvy - uvx * qy;
  const float gx = (dx + ((uvx * qw) + uuvx) * 2.f) / 1.0f;
  const float gy = (dy + ((uvy * qw) + uuvy) * 2.f) / 1.0f;
  const float gz = (dz + ((uvz * qw) + uuvz) * 2.f) / 1.0f;
  const int ix = static_cast<int>(gx), iy = static_cast<int>(gy), iz = static_cast<int>(gz);
  // an episode has at most 499 moves of 0.25 m: |cell| <= 125 fits 10 bits
  const uint32_t key = 0x80000000u | ((static_cast<uint32_t>(ix) & 0x3ffu) << 20) |
                       ((static_cast<uint32_t>(iy) & 0x3ffu) << 10) |
                       (static_cast<uint32_t>(iz) & 0x3ffu);
  uint32_t* tab = g.visited + static_cast<size_t>(e) * kVisitedSlots;
  uint32_t h = (key * 2654435761u) >> 22;  // 10 bits
  for (uint32_t probe = 0; probe < kVisitedSlots; ++probe) {
    const uint32_t cur = tab[h];
    if (cur == key)
      return false;
    if (cur == 0u) {
      tab[h] = key;
      g.numCells[e] += 1u;
      return true;
    }
    h = (h + 1u) & (kVisitedSlots - 1u);
  }
  return false;  // table full: cannot happen within one episode (<= 500 cells)
}

// BaseSimulator::reset + InfoFunctor::reset + RewardFunctor::reset for one env.
// (`sceneIdx` = g.scene[e] and `rc` = g.resetCount[e], read by the caller together with whatever
// else it needs from the environment's columns, so that all of it is one trip to memory)
__device__ __forceinline__ void resetEnvLoaded(const GroupDev& g, const SceneTable& st, uint32_t e,
                                               uint32_t sceneIdx, uint32_t rc, uint32_t seedLo,
                                               uint32_t seedHi) {
  const uint32_t B = g.B;
  const uint32_t r = philoxFirst(g.envBase + e, rc, 0u, 0u, seedLo, seedHi);
  const uint32_t nEp = st.epCount[sceneIdx];
  const uint32_t idx = __umulhi(r, nEp);
  g.resetCount[e] = rc + 1;
  g.episode[e] = idx;
  g.step[e] = 1;
  const size_t rec = static_cast<size_t>(st.epOffset[sceneIdx]) + idx;
  const float* ep = st.episodes + 10 * rec;
  const float sx = ep[0], sy = ep[1], sz = ep[2];
  const float qx = ep[3], qy = ep[4], qz = ep[5], qw = ep[6];
  const float gx = ep[7], gy = ep[8], gz = ep[9];
  const uint4* nv = reinterpret_cast<const uint4*>(st.epNav + rec);
  const uint4 n0 = __ldg(nv), n1 = __ldg(nv + 1), n2 = __ldg(nv + 2);
  g.pos[e] = sx;
  g.pos[B + e] = sy;
  g.pos[2 * B + e] = sz;
  g.rot[e] = qx;
  g.rot[B + e] = qy;
  g.rot[2 * B + e] = qz;
  g.rot[3 * B + e] = qw;
  g.goal[e] = gx;
  g.goal[B + e] = gy;
  g.goal[2 * B + e] = gz;
  g.navPos[e] = __uint_as_float(n0.x);
  g.navPos[B + e] = __uint_as_float(n0.y);
  g.navPos[2 * B + e] = __uint_as_float(n0.z);
  g.navRef[e] = n0.w;
  g.navGoal[e] = __uint_as_float(n1.x);
  g.navGoal[B + e] = __uint_as_float(n1.y);
  g.navGoal[2 * B + e] = __uint_as_float(n1.z);
  g.goalRef[e] = n1.w;
  const float init = __uint_as_float(n2.x);
  g.initDist[e] = init;
  g.prevDist[e] = init;
  g.doneDist[e] = __uint_as_float(n2.z);
  if (n2.y | n2.w)
    g.status[e] |= n2.y | n2.w;
  g.cumTravel[e] = 0.f;
  g.prevPos[e] = sx;
  g.prevPos[B + e] = sy;
  g.prevPos[2 * B + e] = sz;
  writePolar(g, e, sx, sy, sz, qx, qy, qz, qw, gx, gy, gz);
  if (g.task == kTaskFlee) {
    // Flee::InfoFunctor::reset: the reference point of the distance is the snapped
    // start; distance and the reward's previous distance start at 0
    g.navGoal[e] = __uint_as_float(n0.x);
    g.navGoal[B + e] = __uint_as_float(n0.y);
    g.navGoal[2 * B + e] = __uint_as_float(n0.z);
    g.goalRef[e] = n0.w;
    g.initDist[e] = 0.f;
    g.prevDist[e] = 0.f;
  } else if (g.task == kTaskExploration) {
    // Exploration::InfoFunctor::reset: empty set, remember the initial pose
    // (glm::inverse(q) = conjugate(q) / dot(q, q)), visit the first cell
    uint4* tab = reinterpret_cast<uint4*>(g.visited + static_cast<size_t>(e) * kVisitedSlots);
    for (uint32_t i = 0; i < kVisitedSlots / 4; ++i)
      tab[i] = make_uint4(0u, 0u, 0u, 0u);
    g.numCells[e] = 0u;
    const float nrm = qx * qx + qy * qy + qz * qz + qw * qw;
    g.explInit[e] = sx;
    g.explInit[B + e] = sy;
    g.explInit[2 * B + e] = sz;
    g.explInit[3 * B + e] = -qx / nrm;
    g.explInit[4 * B + e] = -qy / nrm;
    g.explInit[5 * B + e] = -qz / nrm;
    g.explInit[6 * B + e] = qw / nrm;
    explVisit(g, e, sx, sy, sz);
    g.initDist[e] = 0.f;
    g.prevDist[e] = 0.f;  // numVisited = size - 1 = 0
  }
}
__device__ __forceinline__ void resetEnv(const GroupDev& g, const SceneTable& st, uint32_t e,
                                         uint32_t seedLo, uint32_t seedHi) {
  resetEnvLoaded(g, st, e, g.scene[e], g.resetCount[e], seedLo, seedHi);
}

// InfoFunctor::step + RewardFunctor::step, then the in-loop reset when done.
// `d` is the geodesic distance of this step (ignored when the task or the
// action did not ask for one).
// (`prev` = g.prevDist[e] and `epr0` = g.episodeReward[e], read by the caller)
__device__ __forceinline__ void finishEnvLoaded(const GroupDev& g, const SceneTable& st, uint32_t e,
                                                bool done, bool moved, float d, float prev,
                                                float epr0, uint32_t seedLo, uint32_t seedHi) {
  const uint32_t B = g.B;
  // Everything this function reads from the environment's columns is requested here, before
  // the first store: the columns may alias as far as the compiler knows, so a load placed
  // after a store waits for it, and each such wait is a trip to L2.
  const bool pointNav = g.task == kTaskPointNav;
  float init = 0.f, cum = 0.f, px = 0.f, py = 0.f, pz = 0.f, qx = 0.f, qy = 0.f, qz = 0.f;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f, s4 = 0.f;
  uint32_t sceneIdx = 0u, rc = 0u, slotIdx = 0u, myEpoch = 0u, slotEpoch = 0u, slotScene = 0u;
  if (done) {
    s0 = g.stats[e];
    s1 = g.stats[B + e];
    s2 = g.stats[2 * B + e];
    s3 = g.stats[3 * B + e];
    s4 = g.stats[4 * B + e];
    sceneIdx = g.scene[e];
    rc = g.resetCount[e];
    if (pointNav) {
      init = g.initDist[e];
      cum = g.cumTravel[e];
    }
    if (g.rotation) {
      slotIdx = g.slot[e];
      myEpoch = g.envEpoch[e];
      slotEpoch = g.slotEpoch[slotIdx];
      slotScene = g.slotScene[slotIdx];
    }
  } else if (moved && pointNav) {
    cum = g.cumTravel[e];
    px = g.pos[e];
    py = g.pos[B + e];
    pz = g.pos[2 * B + e];
    qx = g.prevPos[e];
    qy = g.prevPos[B + e];
    qz = g.prevPos[2 * B + e];
  }
  float success = 0, spl = 0, reward;
  if (pointNav) {
    if (done) {
      success = d < kSuccessDistance ? 1.f : 0.f;
      const float mx = (init < cum) ? cum : init;  // std::max(init, cum)
      spl = success * init / mx;
    } else if (moved) {
      const float dx = px - qx;
      const float dy = py - qy;
      const float dz = pz - qz;
      g.cumTravel[e] = cum + sqrtExact(dx * dx + dy * dy + dz * dz);
      g.prevDist[e] = d;
      g.doneDist[e] = d;
      g.prevPos[e] = px;
      g.prevPos[B + e] = py;
      g.prevPos[2 * B + e] = pz;
    } else {
      d = prev;
    }
    reward = -kSlackReward;
    if (done)
      reward += kSuccessReward * spl;
    else
      reward += prev - d;
    g.info[3 * e + 0] = success;
    g.info[3 * e + 1] = spl;
    g.info[3 * e + 2] = d;
    if (g.hInfo) {
      g.hInfo[3 * e + 0] = success;
      g.hInfo[3 * e + 1] = spl;
      g.hInfo[3 * e + 2] = d;
    }
  } else if (g.task == kTaskFlee) {
    // Flee::InfoFunctor::step / RewardFunctor::step (simulator.cpp:846-880)
    if (!moved)
      d = prev;
    reward = d - prev;
    g.prevDist[e] = d;
    g.info[e] = d;
    if (g.hInfo)
      g.hInfo[e] = d;
    success = d;  // first info column, for the running statistics below
  } else {
    // Exploration (simulator.cpp:919-993); the set itself was updated by the caller
    d = static_cast<float>(g.numCells[e] - 1u);
    reward = 0.25f * (d - prev);
    g.prevDist[e] = d;
    g.info[e] = d;
    if (g.hInfo)
      g.hInfo[e] = d;
    success = d;
  }
  g.reward[e] = reward;
  g.mask[e] = done ? 0 : 1;
  if (g.rewardOut)
    g.rewardOut[e] = reward;
  if (g.maskOut)
    g.maskOut[e] = done ? 0 : 1;
  if (g.hReward) {
    g.hReward[e] = reward;
    g.hMask[e] = done ? 0 : 1;
  }
  // current_episode_reward += reward; on done the episode's totals go to the
  // running sums and the accumulator restarts (same fp32 operations, in step
  // order, as the trainer's tensor code)
  const float epr = epr0 + reward;
  if (done) {
    g.stats[e] = s0 + epr;
    g.stats[B + e] = s1 + 1.f;
    g.stats[2 * B + e] = s2 + success;
    g.stats[3 * B + e] = s3 + spl;
    g.stats[4 * B + e] = s4 + d;
    g.episodeReward[e] = 0.f;
    if (myEpoch != slotEpoch) {
      // the slot has moved on: this environment follows now, at the end of its episode, and
      // starts its next one in the new scene (swapScene, simulator.cpp:1292-1308)
      sceneIdx = slotScene;
      g.scene[e] = slotScene;
      g.envEpoch[e] = slotEpoch;
      atomicSub(&g.slotRemaining[slotIdx], 1u);
    }
    resetEnvLoaded(g, st, e, sceneIdx, rc, seedLo, seedHi);
  } else {
    g.episodeReward[e] = epr;
  }
}
__device__ __forceinline__ void finishEnv(const GroupDev& g, const SceneTable& st, uint32_t e,
                                          bool done, bool moved, float d, uint32_t seedLo,
                                          uint32_t seedHi) {
  finishEnvLoaded(g, st, e, done, moved, d, g.prevDist[e], g.episodeReward[e], seedLo, seedHi);
}

// MoveForward of handleMovement: target = position + rotation * (0, 0, -0.25),
// PathFinder::tryStep from the navmesh position, then position = result and the
// GPS/compass is refreshed.  `sc` may point at shared-memory tables.
__device__ __forceinline__ void forwardMove(const GroupDev& g, const NavScene& sc, uint32_t e) {
  const uint32_t B = g.B;
  const float px = g.pos[e], py = g.pos[B + e], pz = g.pos[2 * B + e];
  const float qx = g.rot[e], qy = g.rot[B + e], qz = g.rot[2 * B + e], qw = g.rot[3 * B + e];
  // delta = rot * v :  v + 2 * (w * (q x v) + q x (q x v))
  const float vx = 0.f * kForwardStep, vy = 0.f * kForwardStep, vz = -1.f * kForwardStep;
  const float uvx = qy * vz - vy * qz;
  const float uvy = qz * vx - vz * qx;
  const float uvz = qx * vy - vx * qy;
  const float uuvx = qy * uvz - uvy * qz;
  const float uuvy = qz * uvx - uvz * qx;
  const float uuvz = qx * uvy - uvx * qy;
  float endPos[3];
  endPos[0] = px + (vx + ((uvx * qw) + uuvx) * 2.f);
  endPos[1] = py + (vy + ((uvy * qw) + uuvy) * 2.f);
  endPos[2] = pz + (vz + ((uvz * qw) + uuvz) * 2.f);
  float np[3] = {g.navPos[e], g.navPos[B + e], g.navPos[2 * B + e]};
  uint32_t ref = g.navRef[e];
  tryStep(sc, np, &ref, endPos);
  g.navPos[e] = np[0];
  g.navPos[B + e] = np[1];
  g.navPos[2 * B + e] = np[2];
  g.navRef[e] = ref;
  g.pos[e] = np[0];
  g.pos[B + e] = np[1];
  g.pos[2 * B + e] = np[2];
  writePolar(g, e, np[0], np[1], np[2], qx, qy, qz, qw, g.goal[e], g.goal[B + e],
             g.goal[2 * B + e]);
}

// The part of a step that needs no navmesh query, for one environment: decode the action,
// advance the step counter, apply a turn and refresh the GPS/compass.  An environment that did
// not move is complete after this (info / reward / mask written here, the reset included when
// its episode ended); one that moved gets its work-list entry in *entry and its list in
// *listIdx, and true is returned.
__device__ __forceinline__ bool preEnv(const GroupDev& g, const SceneTable& st, uint32_t e,
                                       const int64_t* __restrict__ actions,
                                       const uint8_t* __restrict__ actions8, const TurnConsts& tc,
                                       uint32_t seedLo, uint32_t seedHi, uint32_t* entry,
                                       uint32_t* listIdxOut) {
  const uint32_t B = g.B;
  // host-supplied actions arrive validated and narrowed to one byte each, in pinned
  // host memory that the kernel reads in place (no staging copy in the stream)
  const int64_t action = actions8 ? static_cast<int64_t>(actions8[e]) : actions[e];
  // every column value any branch below needs is requested now, together with the action
  // (which may come over the bus), so that the branches do not add trips to memory
  const uint32_t step = g.step[e] + 1;
  float qx = g.rot[e], qy = g.rot[B + e], qz = g.rot[2 * B + e], qw = g.rot[3 * B + e];
  const float px = g.pos[e], py = g.pos[B + e], pz = g.pos[2 * B + e];
  const float gx = g.goal[e], gy = g.goal[B + e], gz = g.goal[2 * B + e];
  const uint32_t slotIdx = g.slot[e];
  uint32_t listIdx = 2u * slotIdx;
  if (g.rotation)  // still in the scene the slot is leaving?
    listIdx += g.envEpoch[e] != g.slotEpoch[slotIdx] ? 1u : 0u;
  const float prev = g.prevDist[e];
  const float epr0 = g.episodeReward[e];
  g.step[e] = step;
  bool done = static_cast<float>(step) >= kMaxSteps;
  bool moved = false;
  if (action == 0) {
    done = true;
  } else if (action == 1) {
    moved = true;
  } else {
    if (action == 2 || action == 3) {
      const float ox = action == 2 ? tc.lx : tc.rx;
      const float oy = action == 2 ? tc.ly : tc.ry;
      const float oz = action == 2 ? tc.lz : tc.rz;
      const float ow = action == 2 ? tc.lw : tc.rw;
      const float rw = qw * ow - qx * ox - qy * oy - qz * oz;
      const float rx = qw * ox + qx * ow + qy * oz - qz * oy;
      const float ry = qw * oy + qy * ow + qz * ox - qx * oz;
      const float rz = qw * oz + qz * ow + qx * oy - qy * ox;
      qx = rx;
      qy = ry;
      qz = rz;
      qw = rw;
      g.rot[e] = qx;
      g.rot[B + e] = qy;
      g.rot[2 * B + e] = qz;
      g.rot[3 * B + e] = qw;
    } else {
      // The reference aborts the process here; this implementation flags the
      // environment and leaves its pose untouched.
      g.status[e] |= kStatBadAction;
    }
    writePolar(g, e, px, py, pz, qx, qy, qz, qw, gx, gy, gz);
  }
  if (moved) {
    // the list entry carries what the step kernel has to know about the action
    *entry = e | (done ? kListDone : 0u) | kListMoved;
    *listIdxOut = listIdx;
    return true;
  }
  // No move, no navmesh query: a step that goes on reports the distance of the step before
  // (:783-785), one that ends the episode the distance kept for that (GroupDev::doneDist);
  // the in-loop reset is a table lookup.
  const float dEnd = (done && g.task == kTaskPointNav) ? g.doneDist[e] : 0.f;
  finishEnvLoaded(g, st, e, done, false, dEnd, prev, epr0, seedLo, seedHi);
  return false;
}

__global__ void __launch_bounds__(256)
k_pre(GroupDev g, SceneTable st, const int64_t* __restrict__ actions,
      const uint8_t* __restrict__ actions8, TurnConsts tc, uint32_t seedLo, uint32_t seedHi) {
  launchDependents();
  waitForPredecessor();
  const uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= g.B)
    return;
  uint32_t entry = 0u, listIdx = 0u;
  const bool listed = preEnv(g, st, e, actions, actions8, tc, seedLo, seedHi, &entry, &listIdx);
  const unsigned running = __activemask();
  const unsigned listedMask = __ballot_sync(running, listed);
  if (listed) {
    // one atomic per (warp, list) instead of one per environment
    const unsigned grp = __match_any_sync(listedMask, listIdx);
    const int leader = __ffs(grp) - 1;
    const int lane = threadIdx.x & 31;
    uint32_t base = 0;
    if (lane == leader)
      base = atomicAdd(&g.counts[listIdx], static_cast<uint32_t>(__popc(grp)));
    base = __shfl_sync(grp, base, leader);
    const uint32_t at = base + __popc(grp & ((1u << lane) - 1u));
    g.geoList[g.listBase[listIdx] + at] = entry;
  }
}

// Generic path: one thread per listed env, tables and A* scratch in global
// memory (grid.y = scene).  Used when a scene does not fit the shared-memory
// kernel of geo_warp.cuh.
__global__ void __launch_bounds__(128)
k_step_thread(GroupDev g, SceneTable st, const WarpPlan* __restrict__ plan,
              AStarScratch* __restrict__ scratch, uint32_t seedLo, uint32_t seedHi) {
  launchDependents();
  const uint32_t listIdx = blockIdx.y;
  waitForPredecessor();
  const uint32_t sceneIdx =
      (listIdx & 1u) ? g.slotPrev[listIdx >> 1] : g.slotScene[listIdx >> 1];
  if (plan && plan[sceneIdx].warps != 0)
    return;  // the warp kernel has this scene
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t n = g.counts[listIdx];
  if (t == 0) {  // the next step starts from empty lists
    g.countsNext[listIdx] = 0u;
    g.countsNext[g.numLists + listIdx] = 0u;
  }
  if (t >= n)
    return;
  const uint32_t at = g.listBase[listIdx] + t;
  if (at >= 2u * g.B)
    return;
  const uint32_t entry = g.geoList[at];
  const uint32_t e = entry & kListEnvMask;
  const uint32_t B = g.B;
  const NavScene sc = st.scenes[sceneIdx];
  const bool done = entry & kListDone, moved = entry & kListMoved;
  if (moved)
    forwardMove(g, sc, e);
  float d = 0.f;
  if (g.task == kTaskPointNav || (g.task == kTaskFlee && moved)) {
    const float a[3] = {g.navPos[e], g.navPos[B + e], g.navPos[2 * B + e]};
    const float b[3] = {g.navGoal[e], g.navGoal[B + e], g.navGoal[2 * B + e]};
    uint32_t status = 0;
    d = geodesic(sc, scratch + e, b, g.goalRef[e], a, g.navRef[e], &status);
    if (status)
      g.status[e] |= status;
  } else if (g.task == kTaskExploration && moved) {
    explVisit(g, e, g.pos[e], g.pos[B + e], g.pos[2 * B + e]);
  }
  finishEnv(g, st, e, done, moved, d, seedLo, seedHi);
}

// After a step of a group whose scenes rotate: every slot whose environments have all reached
// the slot's scene starts its next move (SceneSwapper::postStep / startSceneSwap,
// simulator/simulator.cpp:1094-1129): a scene is drawn from the pool of waiting scenes and
// trades places with the slot's scene, which can be drawn again at once, also while some
// other slot's environments are still leaving it.  Slots are visited in order by one thread,
// as the reference visits its swappers in order at the end of a step.  The reference draws
// from the generator's std::mt19937, whose state at that point depends on how its worker
// threads were scheduled, and makes the new scene available when a background thread has
// loaded it; here the draw is Philox-4x32-10 keyed by the seed with counter (slot, move
// number, 1, 0), index = mulhi32(r, pool size), and the new scene is available from the
// next step on (every scene's navigation mesh is resident).
__global__ void k_swap(GroupDev g, uint32_t seedLo, uint32_t seedHi) {
  launchDependents();
  waitForPredecessor();
  if (blockIdx.x != 0 || threadIdx.x != 0 || g.poolSize == 0)
    return;
  // (with an interval: one move at a time, and only so many steps after the last one)
  if (g.swapInterval != 0u && g.stepId - g.swapCount[1] < g.swapInterval)
    return;
  uint32_t swaps = 0;
  for (uint32_t s = 0; s < g.numSlots; ++s) {
    if (g.slotRemaining[s] != 0u)
      continue;
    if (g.swapInterval != 0u && swaps != 0u)
      break;
    const uint32_t epoch = g.slotEpoch[s] + 1u;
    const uint32_t r = philoxFirst(g.slotBase + s, epoch, 1u, 0u, seedLo, seedHi);
    const uint32_t at = mulHi32(r, g.poolSize);
    const uint32_t cur = g.slotScene[s];
    g.slotPrev[s] = cur;
    g.slotScene[s] = g.pool[at];
    g.pool[at] = cur;
    g.slotEpoch[s] = epoch;
    g.slotRemaining[s] = g.slotSize[s];
    ++swaps;
  }
  if (swaps) {
    g.swapCount[0] += swaps;
    g.swapCount[1] = g.stepId;
  }
}

__global__ void __launch_bounds__(256)
k_reset_all(GroupDev g, SceneTable st, uint32_t seedLo, uint32_t seedHi) {
  const uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= g.B)
    return;
  resetEnv(g, st, e, seedLo, seedHi);
}

// One thread per episode record of one scene: snapPoint(start), snapPoint(goal)
// and the geodesic distance start -> goal, exactly what reset() asks of the
// navmesh (simulator.cpp:611-612, 747-752).
__global__ void __launch_bounds__(128)
k_episode_table(const NavScene* scene, const float* __restrict__ episodes, uint32_t count,
                AStarScratch* __restrict__ scratch, uint32_t nslots, EpisodeNav* out,
                unsigned long long* searchWork) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nslots)
    return;
  const NavScene sc = *scene;
  // nodes opened by the episodes' searches and how many searches there were: how much work a
  // query on this scene is (the step kernel's CTAs are dealt to the scenes by it)
  unsigned long long nodesSum = 0ull, searches = 0ull;
  for (uint32_t i = t; i < count; i += nslots) {
    const float* ep = episodes + 10 * static_cast<size_t>(i);
    const float start[3] = {ep[0], ep[1], ep[2]};
    const float goal[3] = {ep[7], ep[8], ep[9]};
    EpisodeNav r;
    snapPoint(sc, start, r.navStart, &r.startRef);
    snapPoint(sc, goal, r.navGoal, &r.goalRef);
    uint32_t status = 0;
    if (r.startRef == 0 || r.goalRef == 0)
      status |= kStatSnapFailed;
    uint32_t opened = 0u;
    r.initDist = geodesic(sc, scratch + t, r.navStart, r.startRef, r.navGoal, r.goalRef, &status,
                          &opened);
    if (opened) {
      nodesSum += opened;
      searches++;
    }
    r.status = status;
    uint32_t statusRev = 0;
    r.initDistRev = geodesic(sc, scratch + t, r.navGoal, r.goalRef, r.navStart, r.startRef,
                             &statusRev);
    r.statusRev = statusRev;
    out[i] = r;
  }
  if (searches) {
    atomicAdd(searchWork, nodesSum);
    atomicAdd(searchWork + 1, searches);
  }
}

// ------------------------------------------------------------ query kernels

__global__ void __launch_bounds__(128)
k_query_snap(const NavScene* scene, uint32_t n, const float* __restrict__ pts, float* out,
             uint32_t* outRef) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n)
    return;
  const NavScene sc = *scene;
  const float p[3] = {pts[3 * i], pts[3 * i + 1], pts[3 * i + 2]};
  float o[3];
  uint32_t r;
  snapPoint(sc, p, o, &r);
  out[3 * i] = o[0];
  out[3 * i + 1] = o[1];
  out[3 * i + 2] = o[2];
  outRef[i] = r;
}

__global__ void __launch_bounds__(128)
k_query_try_step(const NavScene* scene, uint32_t n, const float* __restrict__ start,
                 const uint32_t* __restrict__ startRef, const float* __restrict__ end, float* out,
                 uint32_t* outRef) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n)
    return;
  const NavScene sc = *scene;
  float p[3] = {start[3 * i], start[3 * i + 1], start[3 * i + 2]};
  const float q[3] = {end[3 * i], end[3 * i + 1], end[3 * i + 2]};
  uint32_t r = startRef[i];
  tryStep(sc, p, &r, q);
  out[3 * i] = p[0];
  out[3 * i + 1] = p[1];
  out[3 * i + 2] = p[2];
  outRef[i] = r;
}

__global__ void __launch_bounds__(128)
k_query_geodesic(const NavScene* scene, AStarScratch* __restrict__ scratch, uint32_t nslots,
                 uint32_t n, const float* __restrict__ start,
                 const uint32_t* __restrict__ startRef, const float* __restrict__ end,
                 const uint32_t* __restrict__ endRef, float* out, uint32_t* outStatus) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nslots)
    return;
  const NavScene sc = *scene;
  for (uint32_t i = t; i < n; i += nslots) {
    const float a[3] = {start[3 * i], start[3 * i + 1], start[3 * i + 2]};
    const float b[3] = {end[3 * i], end[3 * i + 1], end[3 * i + 2]};
    uint32_t status = 0;
    out[i] = geodesic(sc, scratch + t, a, startRef[i], b, endRef[i], &status);
    if (outStatus)
      outStatus[i] = status;
  }
}

}  // namespace bpsn
