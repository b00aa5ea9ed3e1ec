// TEST INFRASTRUCTURE ONLY -- the parity oracle and the timed CPU baseline.
// Nothing in the shipped library includes, links or calls this file.
//
// Scalar CPU restatement of the reference's per-environment PointNav state
// machine, written from a reading of simulator/simulator.cpp:
//   * BaseSimulator::reset / step / updateObservationState / handleMovement
//       (simulator/simulator.cpp:601-618, 620-641, 651-677, 680-710)
//   * PointNav::InfoFunctor::reset / step        (:744-756, 758-790)
//   * PointNav::RewardFunctor::reset / step      (:801-806, 808-822)
//   * constants                                   (:46-61)
//   * the batch loop with in-loop auto-reset      (:1619-1653)
//   * Flee::InfoFunctor / RewardFunctor           (:830-887)
//   * Exploration::InfoFunctor / RewardFunctor    (:889-999; the visited set is a
//     std::set of integer cells -- only its size is observable, so the
//     reference's hash function plays no role)
// All navigation-mesh arithmetic (snapPoint, tryStep, findPath) is done by
// the reference's own compiled PathFinder through oracle/_ref/libref_nav.so
// (see ref_capi.cpp); this file only restates the control flow around it and
// the glm quaternion/matrix formulas the reference pulls from an un-vendored
// submodule (angleAxis, quat*quat, quat*vec3, mat3_cast, transpose, length).
//
//   * scene rotation: SceneSwapper, EnvironmentGroup::swapReady / swapScene and their
//     call sites (:1063-1154, 1284-1308, 1385, 1397-1398, 1594, 1636-1640)
// One deliberate difference, shared with the CUDA implementation: the
// reference draws the episode index from the *calling worker thread's*
// std::mt19937 (:605-607, :1736), which makes the sequence depend on thread
// scheduling.  Here the index is a pure function of (seed, env id, number of
// resets that env has had): Philox-4x32-10 with key = (seed_lo, seed_hi),
// counter = (env, reset_count, 0, 0); index = mulhi32(out[0], num_episodes).
// The same holds for scene rotation: the reference picks the next scene of a slot with that
// generator too and makes it available when a background thread has loaded it.  Here the
// pick is Philox with counter = (slot, move number, 1, 0), index = mulhi32(out[0], pool
// size); the new scene is available from the next step on; and every group draws from its
// own share of the waiting scenes (dealt in turn, ascending), so that the order in which the
// groups are stepped plays no role.

#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <set>
#include <tuple>
#include <string>
#include <thread>
#include <vector>

extern "C" {
// from ref_capi.cpp (compiled reference PathFinder)
void* refnav_create(const char* navmesh_path);
void refnav_destroy(void* h);
void refnav_snap(void* h, const float* pt, float* out_xyz, uint64_t* out_poly);
void refnav_try_step(void* h, const float* start_xyz, uint64_t start_poly, const float* end_xyz,
                     float* out_xyz, uint64_t* out_poly);
float refnav_find_path(void* h, const float* s_xyz, uint64_t s_poly, const float* e_xyz,
                       uint64_t e_poly, float* out_pts, int max_pts, int* out_npts);
}

namespace {

constexpr float kSuccessReward = 2.5f;
constexpr float kSlackReward = 1e-2f;
constexpr float kSuccessDistance = 0.2f;
constexpr float kMaxSteps = 500.f;
constexpr float kForwardStep = 0.25f;

struct Quat {
  float x, y, z, w;
};
struct Vec3 {
  float x, y, z;
};

inline Quat quatMul(const Quat& p, const Quat& q) {
  Quat r;
  r.w = p.w * q.w - p.x * q.x - p.y * q.y - p.z * q.z;
  r.x = p.w * q.x + p.x * q.w + p.y * q.z - p.z * q.y;
  r.y = p.w * q.y + p.y * q.w + p.z * q.x - p.x * q.z;
  r.z = p.w * q.z + p.z * q.w + p.x * q.y - p.y * q.x;
  return r;
}

inline Vec3 cross(const Vec3& a, const Vec3& b) {
  return Vec3{a.y * b.z - b.y * a.z, a.z * b.x - b.z * a.x, a.x * b.y - b.x * a.y};
}

// v' = v + 2 * (w * (q x v) + q x (q x v))
inline Vec3 quatRotate(const Quat& q, const Vec3& v) {
  Vec3 qv{q.x, q.y, q.z};
  Vec3 uv = cross(qv, v);
  Vec3 uuv = cross(qv, uv);
  return Vec3{v.x + ((uv.x * q.w) + uuv.x) * 2.f, v.y + ((uv.y * q.w) + uuv.y) * 2.f,
              v.z + ((uv.z * q.w) + uuv.z) * 2.f};
}

// Philox-4x32-10 (Salmon et al., SC'11).
inline void philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                       uint32_t out[4]) {
  for (int r = 0; r < 10; ++r) {
    uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
    uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
    uint32_t n1 = static_cast<uint32_t>(p1);
    uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
    uint32_t n3 = static_cast<uint32_t>(p0);
    c0 = n0;
    c1 = n1;
    c2 = n2;
    c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0;
  out[1] = c1;
  out[2] = c2;
  out[3] = c3;
}

struct Episode {  // simulator/simulator.cpp:83-87, rotation stored x,y,z,w
  float start[3];
  float rot[4];
  float goal[3];
};

struct Env {
  int scene = 0;
  int slot = 0;        // scene rotation: the slot this environment belongs to
  uint32_t epoch = 0;  // ... and the number of the slot's move it has caught up with
  uint32_t resetCount = 0;
  uint32_t episodeIdx = 0;
  Vec3 position{};
  Quat rotation{};
  Vec3 goal{};
  float navPos[3] = {0, 0, 0};
  uint64_t navPoly = 0;
  uint32_t step = 0;
  bool positionUpdated = false;
  // InfoFunctor
  float prevDist = 0, cumTravel = 0, initDist = 0;
  Vec3 prevPos{};
  float navGoal[3] = {0, 0, 0};
  uint64_t navGoalPoly = 0;
  // RewardFunctor
  float rewardPrevDist = 0;
  // Exploration
  Vec3 initialPosition{};
  Quat inverseInitialRotation{};
  std::set<std::tuple<int, int, int>> visited;
};

struct Sim {
  int nScenes = 0;
  std::vector<std::string> navPaths;
  std::vector<std::vector<Episode>> episodes;
  int nEnvs = 0;
  int task = 0;  // 0 PointNav, 1 Flee, 2 Exploration
  uint64_t seed = 0;
  std::vector<Env> envs;
  // outputs (simulator/simulator.cpp:1194-1197)
  std::vector<float> rewards;
  std::vector<uint8_t> masks;
  int infoWidth = 3;
  std::vector<float> infos;   // PointNav: 3 per env (success, spl, distanceToGoal); else 1
  std::vector<float> polars;  // 2 per env
  Quat leftRot{}, rightRot{};

  // thread pool; pathfinders[thread][scene]
  int nThreads = 1;
  std::vector<std::vector<void*>> pathfinders;
  std::vector<std::thread> workers;
  std::mutex mu;
  std::condition_variable cvStart, cvDone;
  uint64_t generation = 0;
  int pending = 0;
  bool exiting = false;
  std::atomic<int> nextEnv{0};
  int rangeFirst = 0, rangeCount = 0;
  const int64_t* actions = nullptr;
  bool triggerReset = false;
  // instrumentation
  std::atomic<uint64_t> nTryStep{0}, nFindPath{0}, nSnap{0};
  // scene rotation (off unless osim_enable_rotation was called)
  bool rotation = false;
  int numSlots = 0, numGroups = 1, perSlot = 0;
  std::vector<int> slotScene, slotPrev;
  std::vector<uint32_t> slotEpoch;
  std::vector<std::atomic<int>> slotRemaining;
  std::vector<std::vector<int>> pools;  // per group
  uint32_t swapInterval = 0;            // steps of a group between two of its moves (0: no limit)
  std::vector<uint32_t> groupSteps, groupLastSwap;
  uint64_t numSwaps = 0;
};

// SceneSwapper::postStep + startSceneSwap (simulator.cpp:1094-1129) for the slots that lie
// inside [first, first + count), in slot order: a slot all of whose environments have reached
// its scene draws the next one from its group's pool; the scene it leaves goes into the pool.
void swapPass(Sim& s, int first, int count, bool atSetup = false) {
  const int slotsPerGroup = s.numSlots / s.numGroups;
  // with an interval: every group whose environments were stepped counts a step, and starts
  // at most one move, and only so many of its steps after its last one
  std::vector<char> mayStart(s.numGroups, 1);
  if (!atSetup) {
    const int perGroup = s.nEnvs / s.numGroups;
    for (int g = 0; g < s.numGroups; ++g) {
      if (g * perGroup < first || (g + 1) * perGroup > first + count)
        continue;
      s.groupSteps[g]++;
      if (s.swapInterval != 0u && s.groupSteps[g] - s.groupLastSwap[g] < s.swapInterval)
        mayStart[g] = 0;
    }
  }
  for (int sl = 0; sl < s.numSlots; ++sl) {
    if (sl * s.perSlot < first || (sl + 1) * s.perSlot > first + count)
      continue;
    const int grp = sl / slotsPerGroup;
    std::vector<int>& pool = s.pools[grp];
    if (pool.empty() || s.slotRemaining[sl].load() != 0)
      continue;
    if (!atSetup && !mayStart[grp])
      continue;
    if (!atSetup && s.swapInterval != 0u) {
      mayStart[grp] = 0;  // one move at a time
      s.groupLastSwap[grp] = s.groupSteps[grp];
    }
    const uint32_t epoch = s.slotEpoch[sl] + 1;
    uint32_t r[4];
    philox4x32(static_cast<uint32_t>(sl), epoch, 1u, 0u, static_cast<uint32_t>(s.seed),
               static_cast<uint32_t>(s.seed >> 32), r);
    const uint32_t at =
        static_cast<uint32_t>((static_cast<uint64_t>(r[0]) * pool.size()) >> 32);
    const int cur = s.slotScene[sl];
    s.slotPrev[sl] = cur;
    s.slotScene[sl] = pool[at];
    pool[at] = cur;
    s.slotEpoch[sl] = epoch;
    s.slotRemaining[sl].store(s.perSlot);
    s.numSwaps++;
  }
}

inline float geoDist(Sim& s, void* pf, const float* a, uint64_t ap, const float* b, uint64_t bp) {
  s.nFindPath.fetch_add(1, std::memory_order_relaxed);
  return refnav_find_path(pf, a, ap, b, bp, nullptr, 0, nullptr);
}

void updateObservation(Sim& s, int e) {
  Env& v = s.envs[e];
  const Quat& q = v.rotation;
  // mat3_cast(q), column-major m[col][row]
  float qxx = q.x * q.x, qyy = q.y * q.y, qzz = q.z * q.z;
  float qxz = q.x * q.z, qxy = q.x * q.y, qyz = q.y * q.z;
  float qwx = q.w * q.x, qwy = q.w * q.y, qwz = q.w * q.z;
  float m00 = 1.f - 2.f * (qyy + qzz), m01 = 2.f * (qxy + qwz), m02 = 2.f * (qxz - qwy);
  float m10 = 2.f * (qxy - qwz), m11 = 1.f - 2.f * (qxx + qzz), m12 = 2.f * (qyz + qwx);
  float m20 = 2.f * (qxz + qwy), m21 = 2.f * (qyz - qwx), m22 = 1.f - 2.f * (qxx + qyy);
  (void)m10;
  (void)m11;
  (void)m12;
  float tx = v.goal.x - v.position.x, ty = v.goal.y - v.position.y, tz = v.goal.z - v.position.z;
  // transpose(m) * t : component i = dot(column i of m, t)
  float vx = m00 * tx + m01 * ty + m02 * tz;
  float vz = m20 * tx + m21 * ty + m22 * tz;
  float px = -vz, py = vx;
  float rho = sqrtf(px * px + py * py);
  float phi = atan2f(py, px);
  s.polars[2 * e + 0] = rho;
  s.polars[2 * e + 1] = -phi;
}

// Exploration::InfoFunctor::update (:897-904)
void explorationUpdate(Env& v) {
  Vec3 d{v.position.x - v.initialPosition.x, v.position.y - v.initialPosition.y,
         v.position.z - v.initialPosition.z};
  Vec3 g = quatRotate(v.inverseInitialRotation, d);
  const float cell = 1.0f;
  v.visited.emplace(int(g.x / cell), int(g.y / cell), int(g.z / cell));
}

void resetEnv(Sim& s, int e, std::vector<void*>& pfs) {
  Env& v = s.envs[e];
  void* pf = pfs[v.scene];
  v.step = 1;
  const std::vector<Episode>& eps = s.episodes[v.scene];
  uint32_t r[4];
  philox4x32(static_cast<uint32_t>(e), v.resetCount, 0u, 0u, static_cast<uint32_t>(s.seed),
             static_cast<uint32_t>(s.seed >> 32), r);
  uint32_t n = static_cast<uint32_t>(eps.size());
  v.episodeIdx = static_cast<uint32_t>((static_cast<uint64_t>(r[0]) * n) >> 32);
  v.resetCount++;
  const Episode& ep = eps[v.episodeIdx];
  v.position = Vec3{ep.start[0], ep.start[1], ep.start[2]};
  v.rotation = Quat{ep.rot[0], ep.rot[1], ep.rot[2], ep.rot[3]};
  v.goal = Vec3{ep.goal[0], ep.goal[1], ep.goal[2]};
  s.nSnap.fetch_add(2, std::memory_order_relaxed);
  refnav_snap(pf, ep.start, v.navPos, &v.navPoly);

  updateObservation(s, e);

  if (s.task == 1) {
    // Flee::InfoFunctor::reset / RewardFunctor::reset: reference point = snapped start
    v.navGoal[0] = v.navPos[0];
    v.navGoal[1] = v.navPos[1];
    v.navGoal[2] = v.navPos[2];
    v.navGoalPoly = v.navPoly;
    v.prevDist = 0;
    v.rewardPrevDist = 0;
    return;
  }
  if (s.task == 2) {
    // Exploration::InfoFunctor::reset; glm::inverse(q) = conjugate(q) / dot(q, q)
    v.visited.clear();
    v.initialPosition = v.position;
    const Quat& q = v.rotation;
    const float nrm = q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
    v.inverseInitialRotation = Quat{-q.x / nrm, -q.y / nrm, -q.z / nrm, q.w / nrm};
    explorationUpdate(v);
    v.prevDist = float(v.visited.size() - 1);
    v.rewardPrevDist = v.prevDist;
    return;
  }

  // InfoFunctor::reset
  refnav_snap(pf, ep.goal, v.navGoal, &v.navGoalPoly);
  v.cumTravel = 0;
  v.initDist = geoDist(s, pf, v.navPos, v.navPoly, v.navGoal, v.navGoalPoly);
  v.prevDist = v.initDist;
  v.prevPos = v.position;
  // RewardFunctor::reset
  v.rewardPrevDist = v.prevDist;
}

// returns done; -1 on an action outside {0,1,2,3} (reference aborts there)
int stepEnv(Sim& s, int e, int64_t action, std::vector<void*>& pfs) {
  Env& v = s.envs[e];
  void* pf = pfs[v.scene];
  v.step++;
  bool done = static_cast<float>(v.step) >= kMaxSteps;
  v.positionUpdated = false;
  if (action == 0) {
    done = true;
  } else {
    if (action == 1) {
      Vec3 delta = quatRotate(v.rotation, Vec3{0.f * kForwardStep, 0.f * kForwardStep,
                                               -1.f * kForwardStep});
      float np[3] = {v.position.x + delta.x, v.position.y + delta.y, v.position.z + delta.z};
      float out[3];
      uint64_t op;
      s.nTryStep.fetch_add(1, std::memory_order_relaxed);
      refnav_try_step(pf, v.navPos, v.navPoly, np, out, &op);
      v.navPos[0] = out[0];
      v.navPos[1] = out[1];
      v.navPos[2] = out[2];
      v.navPoly = op;
      v.position = Vec3{out[0], out[1], out[2]};
      v.positionUpdated = true;
    } else if (action == 2) {
      v.rotation = quatMul(v.rotation, s.leftRot);
    } else if (action == 3) {
      v.rotation = quatMul(v.rotation, s.rightRot);
    } else {
      return -1;
    }
    updateObservation(s, e);
  }

  if (s.task != 0) {
    float info;
    float reward;
    if (s.task == 1) {
      // Flee::InfoFunctor::step / RewardFunctor::step
      if (v.positionUpdated)
        v.prevDist = geoDist(s, pf, v.navGoal, v.navGoalPoly, v.navPos, v.navPoly);
      info = v.prevDist;
      reward = info - v.rewardPrevDist;
    } else {
      // Exploration::InfoFunctor::step / RewardFunctor::step
      if (v.positionUpdated)
        explorationUpdate(v);
      info = float(v.visited.size() - 1);
      reward = static_cast<float>(0.25 * (info - v.rewardPrevDist));
    }
    v.rewardPrevDist = info;
    s.rewards[e] = reward;
    s.masks[e] = done ? 0 : 1;
    s.infos[e] = info;
    return done ? 1 : 0;
  }

  // InfoFunctor::step
  float d = 0, success = 0, spl = 0;
  if (done) {
    d = geoDist(s, pf, v.navGoal, v.navGoalPoly, v.navPos, v.navPoly);
    success = static_cast<float>(d < kSuccessDistance);
    spl = success * v.initDist / std::max(v.initDist, v.cumTravel);
  } else if (v.positionUpdated) {
    d = geoDist(s, pf, v.navGoal, v.navGoalPoly, v.navPos, v.navPoly);
    float dx = v.position.x - v.prevPos.x, dy = v.position.y - v.prevPos.y,
          dz = v.position.z - v.prevPos.z;
    v.cumTravel += sqrtf(dx * dx + dy * dy + dz * dz);
    v.prevDist = d;
    v.prevPos = v.position;
  } else {
    d = v.prevDist;
  }

  // RewardFunctor::step
  float reward = -kSlackReward;
  if (done)
    reward += kSuccessReward * spl;
  else
    reward += v.rewardPrevDist - d;
  v.rewardPrevDist = d;

  s.rewards[e] = reward;
  s.masks[e] = done ? 0 : 1;
  s.infos[3 * e + 0] = success;
  s.infos[3 * e + 1] = spl;
  s.infos[3 * e + 2] = d;
  return done ? 1 : 0;
}

std::atomic<int> g_badAction{0};

void simulate(Sim& s, int tid) {
  std::vector<void*>& pfs = s.pathfinders[tid];
  int i;
  while ((i = s.nextEnv.fetch_add(1, std::memory_order_acq_rel)) < s.rangeCount) {
    int e = s.rangeFirst + i;
    if (s.triggerReset) {
      resetEnv(s, e, pfs);
    } else {
      int done = stepEnv(s, e, s.actions[i], pfs);
      if (done < 0)
        g_badAction.store(1);
      else if (done) {
        if (s.rotation) {
          // swapReady / swapScene (simulator.cpp:1284-1308): the slot has moved on and
          // this environment follows now; its next episode is one of the new scene's
          Env& v = s.envs[e];
          if (v.epoch != s.slotEpoch[v.slot]) {
            v.scene = s.slotScene[v.slot];
            v.epoch = s.slotEpoch[v.slot];
            s.slotRemaining[v.slot].fetch_sub(1);
          }
        }
        resetEnv(s, e, pfs);
      }
    }
  }
}

void workerMain(Sim* s, int tid) {
  uint64_t seen = 0;
  while (true) {
    {
      std::unique_lock<std::mutex> lk(s->mu);
      s->cvStart.wait(lk, [&] { return s->exiting || s->generation != seen; });
      if (s->exiting)
        return;
      seen = s->generation;
    }
    simulate(*s, tid);
    {
      std::lock_guard<std::mutex> lk(s->mu);
      if (--s->pending == 0)
        s->cvDone.notify_all();
    }
  }
}

void runRange(Sim& s, int first, int count, const int64_t* actions, bool reset) {
  s.rangeFirst = first;
  s.rangeCount = count;
  s.actions = actions;
  s.triggerReset = reset;
  s.nextEnv.store(0);
  if (s.nThreads > 1) {
    {
      std::lock_guard<std::mutex> lk(s.mu);
      s.pending = s.nThreads - 1;
      s.generation++;
    }
    s.cvStart.notify_all();
  }
  simulate(s, 0);  // the caller participates as worker 0 (simulator.cpp:1691)
  if (s.nThreads > 1) {
    std::unique_lock<std::mutex> lk(s.mu);
    s.cvDone.wait(lk, [&] { return s.pending == 0; });
  }
}

}  // namespace

extern "C" {

// episodes: concatenated records of 10 floats (start xyz, rot xyzw, goal xyz);
// ep_offsets[n_scenes + 1] indexes records per scene; env_scene[n_envs] gives
// each environment's scene.
void* osim_create(int n_scenes, const char** navmesh_paths, const float* episodes,
                  const int* ep_offsets, int n_envs, const int* env_scene, uint64_t seed,
                  int n_threads, int task) {
  Sim* s = new Sim();
  s->task = task;
  s->infoWidth = task == 0 ? 3 : 1;
  s->nScenes = n_scenes;
  s->seed = seed;
  s->nEnvs = n_envs;
  s->episodes.resize(n_scenes);
  for (int i = 0; i < n_scenes; ++i) {
    s->navPaths.push_back(navmesh_paths[i]);
    for (int j = ep_offsets[i]; j < ep_offsets[i + 1]; ++j) {
      Episode ep;
      memcpy(&ep, episodes + 10 * static_cast<size_t>(j), sizeof(Episode));
      s->episodes[i].push_back(ep);
    }
  }
  s->envs.resize(n_envs);
  for (int e = 0; e < n_envs; ++e)
    s->envs[e].scene = env_scene[e];
  s->rewards.assign(n_envs, 0.f);
  s->masks.assign(n_envs, 0);
  s->infos.assign(3 * static_cast<size_t>(n_envs), 0.f);
  s->polars.assign(2 * static_cast<size_t>(n_envs), 0.f);
  // glm::angleAxis(radians(10.f), +Y): (sin(a/2) * axis, cos(a/2))
  const float a = 10.f * 0.01745329251994329576923690768489f;
  const float sn = sinf(a * 0.5f), cs = cosf(a * 0.5f);
  const float na = -a;
  const float sn2 = sinf(na * 0.5f), cs2 = cosf(na * 0.5f);
  s->leftRot = Quat{0.f * sn, 1.f * sn, 0.f * sn, cs};
  s->rightRot = Quat{0.f * sn2, 1.f * sn2, 0.f * sn2, cs2};

  s->nThreads = n_threads < 1 ? 1 : n_threads;
  s->pathfinders.resize(s->nThreads);
  for (int t = 0; t < s->nThreads; ++t) {
    for (int i = 0; i < n_scenes; ++i) {
      void* pf = refnav_create(navmesh_paths[i]);
      if (!pf) {
        fprintf(stderr, "oracle: failed to load navmesh %s\n", navmesh_paths[i]);
        return nullptr;
      }
      s->pathfinders[t].push_back(pf);
    }
  }
  for (int t = 1; t < s->nThreads; ++t)
    s->workers.emplace_back(workerMain, s, t);
  return s;
}

void osim_destroy(void* h) {
  Sim* s = static_cast<Sim*>(h);
  if (!s)
    return;
  {
    std::lock_guard<std::mutex> lk(s->mu);
    s->exiting = true;
  }
  s->cvStart.notify_all();
  for (auto& t : s->workers)
    t.join();
  for (auto& v : s->pathfinders)
    for (void* pf : v)
      refnav_destroy(pf);
  delete s;
}

void osim_reset(void* h, int first, int count) {
  runRange(*static_cast<Sim*>(h), first, count, nullptr, true);
}

// actions[count] for envs [first, first+count); returns 0, or -1 if any
// action was outside {0,1,2,3}.
int osim_step(void* h, int first, int count, const int64_t* actions) {
  g_badAction.store(0);
  Sim& s = *static_cast<Sim*>(h);
  runRange(s, first, count, actions, false);
  if (s.rotation)
    swapPass(s, first, count);
  return g_badAction.load() ? -1 : 0;
}

// Turns scene rotation on: num_active slots of n_envs / num_active consecutive environments,
// slot i starting in scene active_scenes[i]; the other scenes wait in the groups' pools.
// Every slot starts its first move at once (simulator.cpp:1594).  Call before the first reset.
int osim_enable_rotation(void* h, int num_active, int num_groups, const int* active_scenes) {
  Sim& s = *static_cast<Sim*>(h);
  if (num_active <= 0 || num_groups <= 0 || s.nEnvs % num_active || num_active % num_groups)
    return -1;
  s.rotation = true;
  s.numSlots = num_active;
  s.numGroups = num_groups;
  s.perSlot = s.nEnvs / num_active;
  s.slotScene.assign(active_scenes, active_scenes + num_active);
  s.slotPrev = s.slotScene;
  s.slotEpoch.assign(num_active, 0u);
  s.slotRemaining = std::vector<std::atomic<int>>(num_active);
  for (auto& r : s.slotRemaining)
    r.store(0);
  std::vector<char> active(s.nScenes, 0);
  for (int sc : s.slotScene)
    active[sc] = 1;
  s.pools.assign(num_groups, std::vector<int>());
  int k = 0;
  for (int sc = 0; sc < s.nScenes; ++sc)
    if (!active[sc])
      s.pools[k++ % num_groups].push_back(sc);
  for (int e = 0; e < s.nEnvs; ++e) {
    s.envs[e].slot = e / s.perSlot;
    s.envs[e].scene = s.slotScene[s.envs[e].slot];
    s.envs[e].epoch = 0;
  }
  s.groupSteps.assign(num_groups, 0u);
  s.groupLastSwap.assign(num_groups, 0u);
  swapPass(s, 0, s.nEnvs, /*atSetup=*/true);
  s.numSwaps = 0;
  return 0;
}

// Pace of the rotation: steps of a group between two of its moves at least (0: no limit).
void osim_set_swap_interval(void* h, uint32_t interval) {
  static_cast<Sim*>(h)->swapInterval = interval;
}

// scene of every environment right now, and the moves started since set-up
uint64_t osim_scenes(void* h, int* env_scene) {
  Sim& s = *static_cast<Sim*>(h);
  for (int e = 0; e < s.nEnvs; ++e)
    env_scene[e] = s.envs[e].scene;
  return s.numSwaps;
}

float* osim_rewards(void* h) { return static_cast<Sim*>(h)->rewards.data(); }
uint8_t* osim_masks(void* h) { return static_cast<Sim*>(h)->masks.data(); }
float* osim_infos(void* h) { return static_cast<Sim*>(h)->infos.data(); }
float* osim_polars(void* h) { return static_cast<Sim*>(h)->polars.data(); }

// Snapshot of per-env state, one row per env:
//   f[0:3] position, f[3:7] rotation xyzw, f[7:10] goal, f[10:13] navmesh pos,
//   f[13:16] snapped goal, f[16] prev_dist, f[17] cum_travel, f[18] init_dist,
//   f[19:22] prev_pos          (22 floats)
//   u[0] nav poly, u[1] goal poly, u[2] step, u[3] episode index,
//   u[4] reset count            (5 uint32)
void osim_get_state(void* h, float* f, uint32_t* u) {
  Sim* s = static_cast<Sim*>(h);
  for (int e = 0; e < s->nEnvs; ++e) {
    const Env& v = s->envs[e];
    float* o = f + 22 * static_cast<size_t>(e);
    o[0] = v.position.x; o[1] = v.position.y; o[2] = v.position.z;
    o[3] = v.rotation.x; o[4] = v.rotation.y; o[5] = v.rotation.z; o[6] = v.rotation.w;
    o[7] = v.goal.x; o[8] = v.goal.y; o[9] = v.goal.z;
    o[10] = v.navPos[0]; o[11] = v.navPos[1]; o[12] = v.navPos[2];
    o[13] = v.navGoal[0]; o[14] = v.navGoal[1]; o[15] = v.navGoal[2];
    o[16] = v.prevDist; o[17] = v.cumTravel; o[18] = v.initDist;
    o[19] = v.prevPos.x; o[20] = v.prevPos.y; o[21] = v.prevPos.z;
    uint32_t* q = u + 5 * static_cast<size_t>(e);
    q[0] = static_cast<uint32_t>(v.navPoly);
    q[1] = static_cast<uint32_t>(v.navGoalPoly);
    q[2] = v.step;
    q[3] = v.episodeIdx;
    q[4] = v.resetCount;
  }
}

void osim_counters(void* h, uint64_t* out3) {
  Sim* s = static_cast<Sim*>(h);
  out3[0] = s->nTryStep.load();
  out3[1] = s->nFindPath.load();
  out3[2] = s->nSnap.load();
}

// Runs `steps` steps over all envs with actions[steps][n_envs] without
// returning to the caller in between: the timed CPU-baseline loop.
int osim_run(void* h, int steps, const int64_t* actions) {
  Sim* s = static_cast<Sim*>(h);
  int rc = 0;
  for (int t = 0; t < steps; ++t)
    rc |= osim_step(h, 0, s->nEnvs, actions + static_cast<size_t>(t) * s->nEnvs);
  return rc;
}

void osim_philox(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                 uint32_t* out4) {
  philox4x32(c0, c1, c2, c3, k0, k1, out4);
}

}  // extern "C"
