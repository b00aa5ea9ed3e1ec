// C-ABI implementation (see include/bpsn.h).  Host-side bookkeeping only: it
// owns device buffers, uploads flattened navmeshes and episodes, and launches
// the kernels of sim_kernels.cuh / gae_kernels.cuh.  There is no CPU
// execution path: every compute entry point launches CUDA kernels or fails.

#include "../../include/bpsn.h"
#include "bpsn_test_hooks.h"

#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "dataset_host.h"
#include "depth_kernels.cuh"
#include "gae_kernels.cuh"
#include "geo_warp.cuh"
#include "navmesh_host.h"
#include "sim_kernels.cuh"

using namespace bpsn;

namespace {

thread_local std::string g_lastError;

struct DeviceScene {
  HostScene host;
  bool loaded = false;
  void* blob = nullptr;  // one device allocation holding every array
  NavScene dev{};
  std::vector<bpsn_episode> episodes;
  // render geometry (optional): floor rectangle and boxes
  float floor[4] = {0.f, 0.f, 0.f, 0.f};
  std::vector<float> boxes;
};

struct Group {
  GroupDev dev{};
  void* stateBlob = nullptr;
  size_t stateBytes = 0;
  // pinned host mirrors of the four result arrays
  uint8_t* hOut = nullptr;   // one pinned block mirroring [reward | mask | info | polar]
  size_t outBytes = 0;       // bytes from d.reward to the end of d.polar
  float* hReward = nullptr;  // views into hOut
  uint8_t* hMask = nullptr;
  float* hInfo = nullptr;
  float* hPolar = nullptr;
  volatile uint32_t* hErr = nullptr;  // host view of the device error word (with mirrors)
  volatile uint32_t* hStepFlag = nullptr;  // host view of the published-step counter
  bool publish = false;   // the step kernel's last CTA copies the results to the mirrors
  bool fused = false;     // one launch per step: the step kernel does k_pre's part itself
  bool batched = false;   // funnel and finish for 32 entries at a time, one per lane
  uint16_t* dBatchStage = nullptr;
  volatile uint32_t* hListed = nullptr;  // host view of the last step's number of list entries
  uint32_t batchMinListed = 0;           // the batched form pays from this many entries on
  int batchForce = 0;                    // test hook: 1 always batched, 2 never
  uint32_t stepCounter = 0;
  uint32_t* dDoneCount = nullptr;
  uint32_t* dOvList = nullptr;   // one-launch step: per-CTA overflow segments and their headers
  uint32_t* dOvMeta = nullptr;
  uint8_t* hActions = nullptr;  // pinned, device-mapped staging of host-supplied actions
  const uint8_t* dActions8 = nullptr;  // the same buffer as the device addresses it
  AStarScratch* scratch = nullptr;
  // launch plan of the geodesic phase
  uint32_t maxListLen = 0;      // longest work list (environments of the largest slot)
  bool warpGeo = false;         // some scene of the group runs on the shared-memory warp kernel
  bool anyWarpScene = false;
  bool anyThreadScene = false;  // some scene needs the generic kernel
  uint32_t numCtas = 0;         // grid of the warp kernel
  int warpMode = 0;             // which instance of k_step_warp: 0 shared, 1 global, 2 both
  size_t geoSmem = 0;
  WarpPlan* dPlan = nullptr;    // [numScenes]
  uint8_t* globalSlabs = nullptr;  // warp slabs of the scenes that are worked on in global memory
  size_t globalSlabStride = 0;     // bytes between consecutive slabs there (the largest scene's)
  size_t numGlobalSlabs = 0;       // one per warp of the grid, or one per environment
  uint4* dCtaMap = nullptr;     // [numCtas] (slot, number among the slot's CTAs, their count)
  AStarScratch* fallbackScratch = nullptr;
  float* depth = nullptr;  // [B][H][W] when a render size was configured
  cudaEvent_t done = nullptr;
  bool inFlight = false;
  // optional per-kernel timing (bpsn_profile_enable)
  bool profiling = false;
  cudaEvent_t prof[3] = {};
  double profMs[2] = {0, 0};
  uint64_t profSteps = 0;
  // offsets of each field inside stateBlob (for bpsn_get_ptr)
  void* fieldPtr[BPSN_FIELD_COUNT] = {};
  size_t fieldBytes[BPSN_FIELD_COUNT] = {};
};

}  // namespace

struct bpsn_dataset {
  std::vector<DatasetScene> scenes;
};

struct bpsn_sim {
  bpsn_config cfg{};
  std::vector<DeviceScene> scenes;
  std::vector<uint32_t> envScene;
  bool envSceneExplicit = false;
  // scene rotation (num_active_scenes < num_scenes)
  uint32_t numActive = 0;
  bool rotation = false;
  std::vector<uint32_t> activeScenes;       // [numActive] scene of every slot at the start
  std::vector<std::vector<uint32_t>> pools;  // per group: scenes waiting for a slot
  std::vector<Group> groups;
  bool finalized = false;
  std::string lastError;
  // device tables
  NavScene* dScenes = nullptr;
  float* dEpisodes = nullptr;
  EpisodeNav* dEpNav = nullptr;
  uint32_t* dEpOffset = nullptr;
  uint32_t* dEpCount = nullptr;
  SceneTable table{};
  RenderTable render{};
  float* dBoxes = nullptr;
  uint32_t* dBoxOffset = nullptr;
  uint32_t* dBoxCount = nullptr;
  float* dFloor = nullptr;
  TurnConsts turn{};
  // scratch for the bpsn_query_* entry points
  AStarScratch* queryScratch = nullptr;
  uint32_t querySlots = 0;
  std::vector<double> queryCost;  // per scene: work of one query, in opened nodes (bpsn_finalize)
};

namespace {

int32_t fail(bpsn_sim* sim, int32_t code, const std::string& msg) {
  if (sim)
    sim->lastError = msg;
  g_lastError = msg;
  return code;
}

#define BPSN_CUDA(sim, expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess)                                                                \
      return fail(sim, BPSN_ERR_CUDA,                                                     \
                  std::string(#expr) + ": " + cudaGetErrorString(_e));                    \
  } while (0)

inline size_t alignUp(size_t x, size_t a) {
  return (x + a - 1) / a * a;
}

int32_t uploadScene(bpsn_sim* sim, DeviceScene& ds) {
  const HostScene& h = ds.host;
  size_t off = 0;
  auto place = [&](size_t bytes) {
    size_t o = off;
    off = alignUp(off + bytes, 256);
    return o;
  };
  const size_t oVerts = place(h.verts.size() * sizeof(float));
  const size_t oPolys = place(h.polys.size() * sizeof(NavPoly));
  const size_t oDetail = place(h.detail.size() * sizeof(NavDetail));
  const size_t oDverts = place(h.dverts.size() * sizeof(float) + 16);
  const size_t oDtris = place(h.dtris.size());
  const size_t oBv = place(h.bv.size() * sizeof(NavBVNode) + 16);
  const size_t oIsland = place(h.island.size() * sizeof(int32_t));
  // shared-memory image for k_step_warp (layout = stagedLayout())
  const NavScene hv = h.view();
  const StagedLayout lay = stagedLayout(hv.nverts, hv.npolys, hv.ndtris, hv.ndverts);
  std::vector<uint8_t> img(lay.total, 0);
  {
    float* v4 = reinterpret_cast<float*>(img.data() + lay.verts);
    for (int i = 0; i < hv.nverts; ++i) {
      v4[4 * i + 0] = h.verts[3 * i + 0];
      v4[4 * i + 1] = h.verts[3 * i + 1];
      v4[4 * i + 2] = h.verts[3 * i + 2];
      v4[4 * i + 3] = 0.f;
    }
    NavPoly* sp = reinterpret_cast<NavPoly*>(img.data() + lay.polys);
    for (int i = 0; i < hv.npolys; ++i) {
      NavPoly q = h.polys[i];
      // links to neighbours the filter rejects do not exist for the search and are
      // walls for moveAlongSurface either way
      for (int j = 0; j < kVertsPerPoly; ++j) {
        uint16_t v = j < q.vertCount ? q.neis[j] : 0;
        if (v && !(v & kExtLink) && (h.polys[v - 1].flags & kFlagWalk) == 0)
          v = 0;
        q.neis[j] = v;
      }
      bool dup = false;
      for (int j = 1; j < kVertsPerPoly; ++j)
        for (int k = 0; k < j; ++k)
          if (q.neis[j] && !(q.neis[j] & kExtLink) && q.neis[j] == q.neis[k])
            dup = true;
      q.pad = dup ? 1 : 0;
      sp[i] = q;
    }
    memcpy(img.data() + lay.detail, h.detail.data(), h.detail.size() * sizeof(NavDetail));
    memcpy(img.data() + lay.dtris, h.dtris.data(), h.dtris.size());
    if (!h.dverts.empty())
      memcpy(img.data() + lay.dverts, h.dverts.data(), h.dverts.size() * sizeof(float));
    memcpy(img.data() + lay.island, h.island.data(), h.island.size() * sizeof(int32_t));
  }
  const size_t oStaged = place(img.size());
  BPSN_CUDA(sim, cudaMalloc(&ds.blob, off));
  uint8_t* base = static_cast<uint8_t*>(ds.blob);
  auto up = [&](size_t o, const void* src, size_t bytes) -> cudaError_t {
    if (!bytes)
      return cudaSuccess;
    return cudaMemcpy(base + o, src, bytes, cudaMemcpyHostToDevice);
  };
  BPSN_CUDA(sim, up(oVerts, h.verts.data(), h.verts.size() * sizeof(float)));
  BPSN_CUDA(sim, up(oPolys, h.polys.data(), h.polys.size() * sizeof(NavPoly)));
  BPSN_CUDA(sim, up(oDetail, h.detail.data(), h.detail.size() * sizeof(NavDetail)));
  BPSN_CUDA(sim, up(oDverts, h.dverts.data(), h.dverts.size() * sizeof(float)));
  BPSN_CUDA(sim, up(oDtris, h.dtris.data(), h.dtris.size()));
  BPSN_CUDA(sim, up(oBv, h.bv.data(), h.bv.size() * sizeof(NavBVNode)));
  BPSN_CUDA(sim, up(oIsland, h.island.data(), h.island.size() * sizeof(int32_t)));
  BPSN_CUDA(sim, up(oStaged, img.data(), img.size()));
  NavScene s = h.view();
  s.verts = reinterpret_cast<const float*>(base + oVerts);
  s.polys = reinterpret_cast<const NavPoly*>(base + oPolys);
  s.detail = reinterpret_cast<const NavDetail*>(base + oDetail);
  s.dverts = reinterpret_cast<const float*>(base + oDverts);
  s.dtris = reinterpret_cast<const uint8_t*>(base + oDtris);
  s.bv = reinterpret_cast<const NavBVNode*>(base + oBv);
  s.island = reinterpret_cast<const int32_t*>(base + oIsland);
  s.staged = base + oStaged;
  s.stagedBytes = static_cast<uint32_t>(img.size());
  ds.dev = s;
  return BPSN_OK;
}

int32_t allocGroup(bpsn_sim* sim, Group& g, uint32_t B, uint32_t envBase, uint32_t groupIdx) {
  const uint32_t ns = sim->cfg.num_scenes;
  const uint32_t* envScene = sim->envScene.data() + envBase;
  const bool rotation = sim->rotation;
  // ---- slots (see GroupDev::slot): one per scene when the scenes are fixed, else
  // `active scenes / groups` slots of equal size
  const uint32_t numSlots = rotation ? sim->numActive / sim->cfg.num_groups : ns;
  const uint32_t slotBase = groupIdx * numSlots;
  std::vector<uint32_t> envSlot(B), slotSize(numSlots, 0u), slotScene(numSlots, 0u);
  if (rotation) {
    const uint32_t perSlot = B / numSlots;
    for (uint32_t e = 0; e < B; ++e)
      envSlot[e] = e / perSlot;
    for (uint32_t s2 = 0; s2 < numSlots; ++s2)
      slotScene[s2] = sim->activeScenes[slotBase + s2];
  } else {
    for (uint32_t e = 0; e < B; ++e)
      envSlot[e] = envScene[e];
    for (uint32_t s2 = 0; s2 < numSlots; ++s2)
      slotScene[s2] = s2;
  }
  for (uint32_t e = 0; e < B; ++e)
    slotSize[envSlot[e]]++;
  const std::vector<uint32_t>& pool = sim->pools[groupIdx];
  const uint32_t poolSize = static_cast<uint32_t>(pool.size());
  const uint32_t numLists = 2u * numSlots;

  size_t off = 0;
  auto place = [&](size_t bytes) {
    size_t o = off;
    off = alignUp(off + bytes, 256);
    return o;
  };
  const size_t f = sizeof(float), u = sizeof(uint32_t);
  const size_t oPos = place(3 * B * f), oRot = place(4 * B * f), oGoal = place(3 * B * f);
  const size_t oNavPos = place(3 * B * f), oNavGoal = place(3 * B * f),
               oPrevPos = place(3 * B * f);
  const size_t oPrevDist = place(B * f), oCum = place(B * f), oInit = place(B * f),
               oTmp = place(B * f);
  const size_t oNavRef = place(B * u), oGoalRef = place(B * u), oStep = place(B * u),
               oEpisode = place(B * u), oResetCount = place(B * u), oStatus = place(B * u),
               oScene = place(B * u);
  const size_t oReward = place(B * f), oMask = place(B), oInfo = place(3 * B * f),
               oPolar = place(2 * B * f);
  const size_t oEpReward = place(B * f), oStats = place(5 * B * f);
  const bool expl = sim->cfg.task == BPSN_TASK_EXPLORATION;
  const size_t oExplInit = place(expl ? 7 * B * f : 16), oNumCells = place(expl ? B * u : 16),
               oVisited = place(expl ? static_cast<size_t>(B) * kVisitedSlots * u : 16);
  const size_t oGeoList = place(2 * static_cast<size_t>(B) * u),
               oCounts = place((2 * numLists + 4) * u), oCounts2 = place((2 * numLists + 4) * u),
               oErr = place(4 * u), oListBase = place((numLists + 4) * u);
  const size_t oSlot = place(B * u), oEnvEpoch = place(B * u);
  const size_t oSlotScene = place(numSlots * u), oSlotPrev = place(numSlots * u),
               oSlotEpoch = place(numSlots * u), oSlotRemaining = place(numSlots * u),
               oSlotSize = place(numSlots * u), oPool = place((poolSize + 4) * u),
               oSwapCount = place(4 * u), oSlotEnvs = place(B * u),
               oSlotEnvBase = place(numSlots * u);
  g.stateBytes = off;
  BPSN_CUDA(sim, cudaMalloc(&g.stateBlob, off));
  BPSN_CUDA(sim, cudaMemset(g.stateBlob, 0, off));
  uint8_t* b = static_cast<uint8_t*>(g.stateBlob);
  GroupDev& d = g.dev;
  {
    uint32_t* hl = nullptr;
    BPSN_CUDA(sim, cudaHostAlloc(&hl, 64, cudaHostAllocMapped));
    *hl = 0u;
    g.hListed = hl;
    void* dp = nullptr;
    BPSN_CUDA(sim, cudaHostGetDevicePointer(&dp, hl, 0));
    d.hListed = static_cast<uint32_t*>(dp);
  }
  d.B = B;
  d.envBase = envBase;
  d.task = sim->cfg.task;
  d.infoWidth = sim->cfg.task == BPSN_TASK_POINTNAV ? 3u : 1u;
  d.exactHeap = (sim->cfg.flags & BPSN_FLAG_EXACT_HEAP) ? 1u : 0u;
  d.numScenes = ns;
  d.numLists = numLists;
  d.rotation = rotation ? 1u : 0u;
  d.numSlots = numSlots;
  d.poolSize = poolSize;
  d.slotBase = slotBase;
  d.explInit = reinterpret_cast<float*>(b + oExplInit);
  d.numCells = reinterpret_cast<uint32_t*>(b + oNumCells);
  d.visited = reinterpret_cast<uint32_t*>(b + oVisited);
  d.pos = reinterpret_cast<float*>(b + oPos);
  d.rot = reinterpret_cast<float*>(b + oRot);
  d.goal = reinterpret_cast<float*>(b + oGoal);
  d.navPos = reinterpret_cast<float*>(b + oNavPos);
  d.navGoal = reinterpret_cast<float*>(b + oNavGoal);
  d.prevPos = reinterpret_cast<float*>(b + oPrevPos);
  d.prevDist = reinterpret_cast<float*>(b + oPrevDist);
  d.cumTravel = reinterpret_cast<float*>(b + oCum);
  d.initDist = reinterpret_cast<float*>(b + oInit);
  d.doneDist = reinterpret_cast<float*>(b + oTmp);
  d.navRef = reinterpret_cast<uint32_t*>(b + oNavRef);
  d.goalRef = reinterpret_cast<uint32_t*>(b + oGoalRef);
  d.step = reinterpret_cast<uint32_t*>(b + oStep);
  d.episode = reinterpret_cast<uint32_t*>(b + oEpisode);
  d.resetCount = reinterpret_cast<uint32_t*>(b + oResetCount);
  d.status = reinterpret_cast<uint32_t*>(b + oStatus);
  d.scene = reinterpret_cast<uint32_t*>(b + oScene);
  d.reward = reinterpret_cast<float*>(b + oReward);
  d.mask = reinterpret_cast<uint8_t*>(b + oMask);
  d.info = reinterpret_cast<float*>(b + oInfo);
  d.polar = reinterpret_cast<float*>(b + oPolar);
  d.episodeReward = reinterpret_cast<float*>(b + oEpReward);
  d.stats = reinterpret_cast<float*>(b + oStats);
  d.geoList = reinterpret_cast<uint32_t*>(b + oGeoList);
  d.counts = reinterpret_cast<uint32_t*>(b + oCounts);
  d.countsNext = reinterpret_cast<uint32_t*>(b + oCounts2);
  d.errFlags = reinterpret_cast<uint32_t*>(b + oErr);
  d.listBase = reinterpret_cast<const uint32_t*>(b + oListBase);
  d.slot = reinterpret_cast<uint32_t*>(b + oSlot);
  d.envEpoch = reinterpret_cast<uint32_t*>(b + oEnvEpoch);
  d.slotScene = reinterpret_cast<uint32_t*>(b + oSlotScene);
  d.slotPrev = reinterpret_cast<uint32_t*>(b + oSlotPrev);
  d.slotEpoch = reinterpret_cast<uint32_t*>(b + oSlotEpoch);
  d.slotRemaining = reinterpret_cast<uint32_t*>(b + oSlotRemaining);
  d.slotSize = reinterpret_cast<uint32_t*>(b + oSlotSize);
  d.pool = reinterpret_cast<uint32_t*>(b + oPool);
  d.swapCount = reinterpret_cast<uint32_t*>(b + oSwapCount);
  d.swapInterval = rotation ? sim->cfg.swap_interval : 0u;
  d.slotEnvs = reinterpret_cast<uint32_t*>(b + oSlotEnvs);
  d.slotEnvBase = reinterpret_cast<uint32_t*>(b + oSlotEnvBase);
  {
    // two work lists per slot, each as long as the slot has environments
    std::vector<uint32_t> base(numLists + 4, 0u), initScene(B);
    uint32_t acc = 0;
    g.maxListLen = 0;
    for (uint32_t s2 = 0; s2 < numSlots; ++s2) {
      base[2 * s2] = acc;
      base[2 * s2 + 1] = acc + slotSize[s2];
      acc += 2 * slotSize[s2];
      if (slotSize[s2] > g.maxListLen)
        g.maxListLen = slotSize[s2];
    }
    for (uint32_t e = 0; e < B; ++e)
      initScene[e] = slotScene[envSlot[e]];
    auto up = [&](size_t o, const void* src, size_t bytes) {
      return bytes ? cudaMemcpy(b + o, src, bytes, cudaMemcpyHostToDevice) : cudaSuccess;
    };
    BPSN_CUDA(sim, up(oListBase, base.data(), u * (numLists + 4)));
    BPSN_CUDA(sim, up(oScene, initScene.data(), u * B));
    BPSN_CUDA(sim, up(oSlot, envSlot.data(), u * B));
    // every environment is in its slot's scene, no move under way (the first is started by
    // bpsn_finalize); slotRemaining and slotEpoch start at 0 (memset above)
    BPSN_CUDA(sim, up(oSlotScene, slotScene.data(), u * numSlots));
    BPSN_CUDA(sim, up(oSlotPrev, slotScene.data(), u * numSlots));
    BPSN_CUDA(sim, up(oSlotSize, slotSize.data(), u * numSlots));
    BPSN_CUDA(sim, up(oPool, pool.data(), u * poolSize));
    // the environments ordered by slot (for the step kernel that serves a share of a slot)
    std::vector<uint32_t> envBase(numSlots, 0u), fill(numSlots, 0u), bySlot(B);
    for (uint32_t s2 = 1; s2 < numSlots; ++s2)
      envBase[s2] = envBase[s2 - 1] + slotSize[s2 - 1];
    for (uint32_t e = 0; e < B; ++e)
      bySlot[envBase[envSlot[e]] + fill[envSlot[e]]++] = e;
    BPSN_CUDA(sim, up(oSlotEnvs, bySlot.data(), u * B));
    BPSN_CUDA(sim, up(oSlotEnvBase, envBase.data(), u * numSlots));
  }
  {
    // Scenes this group can ever work on: those of its slots and, when scenes rotate, the
    // ones waiting in its pool.
    std::vector<uint8_t> used(ns, 0);
    for (uint32_t s2 = 0; s2 < numSlots; ++s2)
      if (slotSize[s2])
        used[slotScene[s2]] = 1;
    for (uint32_t sc : pool)
      used[sc] = 1;
    // Shared-memory plan, scene by scene: a CTA works on one scene at a time with 227 KB of
    // shared memory = the scene's staged image + as many warp slabs (24 B per polygon +
    // 512 B) as fit, at most 16.  A scene that leaves no room for a slab goes to global memory.
    // CTAs are dealt to the slots in proportion to environments / warps-per-CTA of the slot's
    // first scene, so that every slot's list drains in about the same time.
    const size_t kSlabPerEnvAbove = size_t(512) << 20;  // bytes of per-warp slabs from which on ...
    const size_t kSlabPerEnvBudget = size_t(32) << 30;  // ... and bytes of per-env slabs up to which
    const size_t kSmemMax = ((sim->cfg.flags & BPSN_FLAG_SMEM_96K) ? 96 : 227) * 1024 - 512;  // per CTA, minus the kernel's static shared memory
    const uint32_t kBlockWarps = 16;
    std::vector<WarpPlan> plan(ns, WarpPlan{16u, 0u, 0u, 0u});
    size_t maxGlobalSlab = 0;
    uint32_t maxGlobalPcap = 16;
    const double kGlobalWarpSpeed = 0.6;  // queries per unit time of a warp in global memory
                                          // relative to one in shared memory (measured)
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, sim->cfg.gpu_id);
    const bool throughputBound = B / 2 > 2u * static_cast<uint32_t>(sms) * kBlockWarps;
    const bool forceGeneric = (sim->cfg.flags & BPSN_FLAG_GENERIC_KERNEL) != 0;
    g.anyThreadScene = false;
    g.anyWarpScene = false;
    // Pass 1: how many slabs fit next to each scene's image in shared memory.
    std::vector<uint32_t> smemWarps(ns, 0u);
    std::vector<size_t> slabBytes(ns, 0), sceneBytes(ns, 0);
    bool anyCramped = false;  // some scene has room for fewer than 8 slabs
    for (uint32_t s2 = 0; s2 < ns; ++s2) {
      if (!used[s2])
        continue;
      const HostScene& h = sim->scenes[s2].host;
      const NavScene hv = h.view();
      const size_t sb = stagedLayout(hv.nverts, hv.npolys, hv.ndtris, hv.ndverts).total;
      const uint32_t pcap = (static_cast<uint32_t>(h.polys.size()) + 15u) / 16u * 16u;
      const size_t slab = warpGeoSlabBytes(static_cast<int>(pcap));
      uint32_t w = 0;
      if (sb + slab <= kSmemMax)
        w = static_cast<uint32_t>((kSmemMax - sb) / slab);
      if (w > kBlockWarps)
        w = kBlockWarps;
      smemWarps[s2] = w;
      slabBytes[s2] = slab;
      sceneBytes[s2] = sb;
      plan[s2].pcap = pcap;
      if (w < 8 && h.polys.size() < 65000)
        anyCramped = true;
    }
    // Pass 2: where each scene is worked on.
    //  * A scene that leaves no room for a slab is worked on in global memory (tables and
    //    slabs L2-resident, all 16 warps of the CTA active).
    //  * When the group has more queries per step than two rounds of every warp of the GPU,
    //    throughput counts, and a scene with room for fewer than 8 slabs gets through more
    //    queries with 16 warps at cache latency than with a few warps at shared-memory
    //    latency.  Such a group is then put in global memory as a whole: a kernel that uses no
    //    shared memory leaves the entire unified cache to L1, which is what makes global
    //    memory competitive (16 scenes of 91-1304 polygons, 16384 envs: 105 M env-steps/s all
    //    in global memory, 95 M mixed, 90 M all in shared memory).
    //  * With fewer queries the step lasts as long as its slowest query, which shared
    //    memory shortens: everything that fits stays there.
    const bool allGlobal = (throughputBound && anyCramped) ||
                           (sim->cfg.flags & BPSN_FLAG_GLOBAL_MEMORY) != 0;
    std::vector<double> speedOf(ns, 1.0);
    bool anyShared = false, anyGlobal = false;
    for (uint32_t s2 = 0; s2 < ns; ++s2) {
      if (!used[s2])
        continue;
      const HostScene& h = sim->scenes[s2].host;
      uint32_t w = smemWarps[s2];
      plan[s2].slabOffset = static_cast<uint32_t>(sceneBytes[s2]);
      const bool indexable = h.polys.size() < 65000;  // 16-bit polygon indices in the slabs
      if (forceGeneric || !indexable) {
        w = 0;
      } else if (allGlobal || w == 0) {
        w = kBlockWarps;
        plan[s2].slabOffset = kSlabInGlobal;
        if (slabBytes[s2] > maxGlobalSlab)
          maxGlobalSlab = slabBytes[s2];
        if (plan[s2].pcap > maxGlobalPcap)
          maxGlobalPcap = plan[s2].pcap;
      }
      plan[s2].warps = w;
      if (w) {
        g.anyWarpScene = true;
        if (plan[s2].slabOffset == kSlabInGlobal)
          anyGlobal = true;
        else
          anyShared = true;
        // a warp working in global memory beside shared-memory CTAs (small L1) gets
        // through its queries more slowly
        speedOf[s2] = (plan[s2].slabOffset == kSlabInGlobal && !allGlobal) ? kGlobalWarpSpeed : 1.0;
      } else {
        g.anyThreadScene = true;
      }
    }
    g.warpGeo = g.anyWarpScene;
    d.globalPcap = maxGlobalPcap;
    if (g.anyWarpScene) {
      g.warpMode = anyShared ? (anyGlobal ? 2 : 0) : 1;
      // A group whose scenes are all searched in global memory and whose step lasts as long as
      // its slowest query runs on the instance without the 64-register cap (one CTA per SM: the
      // cap buys a second CTA, which such a step has no use for, and costs each query 10-20 %):
      // 16 407 polygons, 4096 envs: 204 -> 169 us per step.  (Global memory by request keeps
      // the capped instance, so that tests reach it with small batches.)
      if (g.warpMode == 1 && !throughputBound && !(sim->cfg.flags & BPSN_FLAG_GLOBAL_MEMORY))
        g.warpMode = 2;
      // The steps of a double-buffered generator's two groups are in flight together
      // (simulator/simulator.cpp:1377-1399; bps_nav/rl/ddppo/algo/ddppo_trainer.py:205-270).
      // A small batch's step lasts as long as its slowest query whatever the number of CTAs,
      // so each group gets half of the SMs and the two kernels run side by side instead of
      // one waiting for the other's last warp.
      const int groupsSharing = throughputBound ? 1 : static_cast<int>(sim->cfg.num_groups);
      // the global-only instance fits two CTAs on an SM (64 registers, no shared memory)
      const int ctaBudget = sms * (g.warpMode == 1 ? 2 : 1) / groupsSharing;
      double workSum = 0.0;
      std::vector<double> work(numSlots, 0.0);
      for (uint32_t s2 = 0; s2 < numSlots; ++s2) {
        const WarpPlan& pl = plan[slotScene[s2]];
        if (!slotSize[s2] || !pl.warps)
          continue;
        work[s2] = static_cast<double>(slotSize[s2]) / (pl.warps * speedOf[slotScene[s2]]);
        // Fixed scenes differ in work per query (a search on a scene of long corridors opens
        // several times the nodes of one on a small room): CTAs in proportion to work, not to
        // environments (16 scenes of 91-1304 polygons: 16384 envs 114 -> 121 M env-steps/s,
        // 65536 envs 165 -> 195 M).  A rotating slot meets every scene in turn.
        if (!rotation)
          work[s2] *= sim->queryCost[slotScene[s2]];
        workSum += work[s2];
      }
      // Shares of the budget: whole CTAs by largest remainder, so that the grid does not
      // exceed what is resident at once (a CTA that has to wait for another one to finish
      // starts its first queries when the others are nearly through); at least one per slot.
      std::vector<uint32_t> ctas(numSlots, 0u);
      {
        std::vector<std::pair<double, uint32_t>> rest;
        int dealt = 0;
        for (uint32_t s2 = 0; s2 < numSlots; ++s2) {
          if (!slotSize[s2])
            continue;
          const WarpPlan& pl = plan[slotScene[s2]];
          if (pl.warps && workSum > 0.0) {
            const double share = ctaBudget * work[s2] / workSum;
            const uint32_t need = (slotSize[s2] + pl.warps - 1) / pl.warps;
            uint32_t c = static_cast<uint32_t>(share);
            if (c >= need) {
              c = need;  // never more warps than environments
            } else {
              rest.push_back({share - c, s2});
            }
            if (c == 0) {
              c = 1;
              if (!rest.empty() && rest.back().second == s2)
                rest.pop_back();
            }
            ctas[s2] = c;
          } else if (rotation) {
            ctas[s2] = 1;
          }  // else: a fixed scene of the generic kernel, no CTA of this one
          dealt += static_cast<int>(ctas[s2]);
        }
        std::sort(rest.begin(), rest.end(), [](const auto& a, const auto& b2) {
          return a.first > b2.first || (a.first == b2.first && a.second < b2.second);
        });
        for (size_t i = 0; i < rest.size() && dealt < ctaBudget; ++i, ++dealt)
          ctas[rest[i].second]++;
      }
      std::vector<uint4> ctaMap;
      for (uint32_t s2 = 0; s2 < numSlots; ++s2)
        for (uint32_t r = 0; r < ctas[s2]; ++r)
          ctaMap.push_back(make_uint4(s2, r, ctas[s2], 0u));
      if (ctaMap.empty())
        ctaMap.push_back(make_uint4(0u, 0u, 1u, 0u));
      g.numCtas = static_cast<uint32_t>(ctaMap.size());
      // One launch per step (k_step_warp<.., kFused>) when every CTA's share of its slot is
      // small enough for its warps to take about one query each (the environments that
      // moved need one); larger batches drain a slot's list with all of its CTAs.
      {
        uint32_t maxShare = 0;
        for (const uint4& cm : ctaMap) {
          const uint32_t share = (slotSize[cm.x] + cm.z - 1) / cm.z;
          if (share > maxShare)
            maxShare = share;
        }
        g.fused = !rotation && g.warpMode == 0 && !g.anyThreadScene &&
                  maxShare <= kFusedMaxShare && !(sim->cfg.flags & BPSN_FLAG_TWO_LAUNCHES);
        // Steps that give every warp several entries: funnel and finish 32 at a time.  How
        // many entries a step lists depends on the actions (a quarter of the environments
        // under uniform actions, 60 % under a trained policy's), so the form is chosen step by
        // step from the number the step before listed (GroupDev::hListed).  Measured, entries
        // per warp -> batched against entry by entry: shared memory 1.7 -> -16 %, 3.5 -> -1 %,
        // 4.2 -> -1 %, 6.9 -> +13 %, 8.3 -> +14 %; global memory 3.5 -> -11 %, 8.3 -> +5 %.
        const uint32_t kBatchMinPerWarp = g.warpMode == 0 ? 5 : 6;
        g.batched = !rotation && g.warpMode != 2 && !g.anyThreadScene && !g.fused &&
                    B >= kBatchMinPerWarp * g.numCtas * kBlockWarps;
        g.batchMinListed = kBatchMinPerWarp * g.numCtas * kBlockWarps;
        if (g.batched) {
          const size_t bytes = sizeof(uint16_t) * 32 * kMaxPathPolys * g.numCtas * kBlockWarps;
          BPSN_CUDA(sim, cudaMalloc(&g.dBatchStage, bytes));
          d.batchStage = g.dBatchStage;
        }
        if (g.fused) {
          BPSN_CUDA(sim, cudaMalloc(&g.dOvList, sizeof(uint32_t) * kFusedMaxShare * g.numCtas));
          BPSN_CUDA(sim, cudaMalloc(&g.dOvMeta, sizeof(uint32_t) * 4 * g.numCtas));
          BPSN_CUDA(sim, cudaMemset(g.dOvMeta, 0, sizeof(uint32_t) * 4 * g.numCtas));
          d.ovList = g.dOvList;
          d.ovMeta = g.dOvMeta;
        }
      }
      BPSN_CUDA(sim, cudaMalloc(&g.dCtaMap, sizeof(uint4) * ctaMap.size()));
      BPSN_CUDA(sim, cudaMemcpy(g.dCtaMap, ctaMap.data(), sizeof(uint4) * ctaMap.size(),
                                cudaMemcpyHostToDevice));
      // dynamic shared memory of a CTA: what the largest of the group's shared-memory scenes
      // needs, not the whole SM
      g.geoSmem = 0;
      for (uint32_t s2 = 0; s2 < ns; ++s2)
        if (used[s2] && plan[s2].warps && plan[s2].slabOffset != kSlabInGlobal) {
          const size_t need = sceneBytes[s2] + plan[s2].warps * slabBytes[s2];
          if (need > g.geoSmem)
            g.geoSmem = need;
        }
      if (g.geoSmem > kSmemMax)
        return fail(sim, BPSN_ERR_INVALID_ARG, "step plan: shared memory of a CTA exceeds the limit");
      // The function attribute is the hardware limit whatever this handle's plan asks for: it
      // belongs to the function, so every handle of the process shares it.
      const int kSmemAttr = 227 * 1024 - 512;
      if (g.warpMode == 0) {
        BPSN_CUDA(sim, cudaFuncSetAttribute(rotation  ? k_step_warp<0, true>
                                            : g.fused ? k_step_warp<0, false, true>
                                                      : k_step_warp<0, false>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAttr));
        if (g.batched)
          BPSN_CUDA(sim, cudaFuncSetAttribute(k_step_warp<0, false, false, true>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              kSmemAttr));
      }
      else if (g.warpMode == 2)
        BPSN_CUDA(sim, cudaFuncSetAttribute(rotation ? k_step_warp<2, true> : k_step_warp<2, false>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAttr));
      BPSN_CUDA(sim, cudaMalloc(&g.fallbackScratch, sizeof(AStarScratch) *
                                                        static_cast<size_t>(g.numCtas) * kBlockWarps));
      g.globalSlabStride = maxGlobalSlab ? maxGlobalSlab + kGlobalSlabExtra : 0;
      if (maxGlobalSlab) {
        // One slab per warp of the grid; one per environment instead when the warps' slabs
        // together would not stay in L2 anyway and the environments' fit a memory budget.
        const size_t warpSlabs = static_cast<size_t>(g.numCtas) * kBlockWarps;
        const bool perEnv = warpSlabs * g.globalSlabStride > kSlabPerEnvAbove &&
                            static_cast<size_t>(B) * g.globalSlabStride <= kSlabPerEnvBudget;
        g.numGlobalSlabs = perEnv ? static_cast<size_t>(B) : warpSlabs;
        d.slabPerEnv = perEnv ? 1u : 0u;
        // zeroed: search counters at 0, no node carries a visit tag
        const size_t bytes = g.globalSlabStride * g.numGlobalSlabs;
        BPSN_CUDA(sim, cudaMalloc(&g.globalSlabs, bytes));
        BPSN_CUDA(sim, cudaMemset(g.globalSlabs, 0, bytes));
      }
    }
    // Every index the step kernels form from this plan, checked against what was allocated
    // above (a plan that fails here would make a kernel read or write past an allocation;
    // nothing is launched with it):
    //   shared memory  slabOffset + warps * slab  <=  the CTA's dynamic shared memory
    //   global slabs   (CTA * 16 + warp) or env   <   numGlobalSlabs, slab + counter <= stride
    //   fallback       CTA * 16 + warp            <   numCtas * 16 scratch blocks
    //   work lists     two per slot, each as long as the slot: 2 * B entries in all
    for (uint32_t s2 = 0; s2 < ns; ++s2) {
      const WarpPlan& pl = plan[s2];
      if (!used[s2] || !pl.warps)
        continue;
      std::string bad;
      if (pl.warps > kBlockWarps)
        bad = "more query warps than the block has";
      else if (pl.slabOffset == kSlabInGlobal) {
        if (warpGeoSlabBytes(static_cast<int>(maxGlobalPcap)) + kGlobalSlabExtra >
            g.globalSlabStride)
          bad = "global slab larger than the slab stride";
        else if (g.numGlobalSlabs < (d.slabPerEnv ? static_cast<size_t>(B)
                                                  : static_cast<size_t>(g.numCtas) * kBlockWarps))
          bad = "fewer global slabs than warps (or environments)";
      } else if (pl.slabOffset + static_cast<size_t>(pl.warps) * slabBytes[s2] > g.geoSmem) {
        bad = "slabs run past the CTA's shared memory";
      }
      if (!bad.empty())
        return fail(sim, BPSN_ERR_INVALID_ARG,
                    "step plan of scene " + std::to_string(s2) + ": " + bad);
    }
    BPSN_CUDA(sim, cudaMalloc(&g.dPlan, sizeof(WarpPlan) * ns));
    BPSN_CUDA(sim, cudaMemcpy(g.dPlan, plan.data(), sizeof(WarpPlan) * ns, cudaMemcpyHostToDevice));
  }

  auto setField = [&](int id, void* p, size_t bytes) {
    g.fieldPtr[id] = p;
    g.fieldBytes[id] = bytes;
  };
  setField(BPSN_FIELD_REWARD, d.reward, B * f);
  setField(BPSN_FIELD_MASK, d.mask, B);
  setField(BPSN_FIELD_INFO, d.info, d.infoWidth * B * f);
  setField(BPSN_FIELD_POLAR, d.polar, 2 * B * f);
  setField(BPSN_FIELD_POSITION, d.pos, 3 * B * f);
  setField(BPSN_FIELD_ROTATION, d.rot, 4 * B * f);
  setField(BPSN_FIELD_GOAL, d.goal, 3 * B * f);
  setField(BPSN_FIELD_NAV_POSITION, d.navPos, 3 * B * f);
  setField(BPSN_FIELD_NAV_POLY, d.navRef, B * u);
  setField(BPSN_FIELD_GOAL_POLY, d.goalRef, B * u);
  setField(BPSN_FIELD_STEP, d.step, B * u);
  setField(BPSN_FIELD_EPISODE, d.episode, B * u);
  setField(BPSN_FIELD_RESET_COUNT, d.resetCount, B * u);
  setField(BPSN_FIELD_STATUS, d.status, B * u);
  setField(BPSN_FIELD_PREV_DIST, d.prevDist, B * f);
  setField(BPSN_FIELD_CUM_TRAVEL, d.cumTravel, B * f);
  setField(BPSN_FIELD_INIT_DIST, d.initDist, B * f);
  setField(BPSN_FIELD_SCENE, d.scene, B * u);
  setField(BPSN_FIELD_EPISODE_REWARD, d.episodeReward, B * f);
  setField(BPSN_FIELD_EPISODE_STATS, d.stats, 5 * B * f);
  if (sim->cfg.render_width && sim->cfg.render_height) {
    const size_t bytes = static_cast<size_t>(B) * sim->cfg.render_width * sim->cfg.render_height * f;
    BPSN_CUDA(sim, cudaMalloc(&g.depth, bytes));
    BPSN_CUDA(sim, cudaMemset(g.depth, 0, bytes));
    setField(BPSN_FIELD_DEPTH, g.depth, bytes);
  }

  if (g.anyThreadScene)  // per-slot A* scratch is only used by the generic (global-memory) kernel
    BPSN_CUDA(sim, cudaMalloc(&g.scratch, sizeof(AStarScratch) * static_cast<size_t>(B)));
  BPSN_CUDA(sim, cudaHostAlloc(&g.hActions, B, cudaHostAllocMapped));
  {
    void* dp = nullptr;
    BPSN_CUDA(sim, cudaHostGetDevicePointer(&dp, g.hActions, 0));
    g.dActions8 = static_cast<const uint8_t*>(dp);
  }
  if (sim->cfg.flags & BPSN_FLAG_HOST_MIRRORS) {
    // the four result arrays are adjacent in the state block: one pinned
    // block with the same relative layout lets a step publish them in one copy
    g.outBytes = (oPolar + 2 * B * f) - oReward;
    // mapped: the kernels write the mirrors themselves (GroupDev::hReward ...)
    // (+ two words behind the arrays: the host-visible copy of the device error flags and the
    // number of the last step whose results were published)
    const size_t outPadded = alignUp(g.outBytes, 16);
    BPSN_CUDA(sim, cudaHostAlloc(&g.hOut, outPadded + 32, cudaHostAllocMapped));
    memset(g.hOut, 0, outPadded + 32);
    g.hErr = reinterpret_cast<volatile uint32_t*>(g.hOut + outPadded);
    g.hStepFlag = reinterpret_cast<volatile uint32_t*>(g.hOut + outPadded + 16);
    g.hReward = reinterpret_cast<float*>(g.hOut);
    g.hMask = g.hOut + (oMask - oReward);
    g.hInfo = reinterpret_cast<float*>(g.hOut + (oInfo - oReward));
    g.hPolar = reinterpret_cast<float*>(g.hOut + (oPolar - oReward));
    void* dOut = nullptr;
    BPSN_CUDA(sim, cudaHostGetDevicePointer(&dOut, g.hOut, 0));
    uint8_t* db = static_cast<uint8_t*>(dOut);
    d.hReward = reinterpret_cast<float*>(db);
    d.hMask = db + (oMask - oReward);
    d.hInfo = reinterpret_cast<float*>(db + (oInfo - oReward));
    d.hPolar = reinterpret_cast<float*>(db + (oPolar - oReward));
    d.hErr = reinterpret_cast<uint32_t*>(db + outPadded);
    // one-piece publishing needs the warp step kernel to be the last writer of results
    g.publish = g.anyWarpScene && !g.anyThreadScene;
    if (g.publish) {
      BPSN_CUDA(sim, cudaMalloc(&g.dDoneCount, sizeof(uint32_t)));
      BPSN_CUDA(sim, cudaMemset(g.dDoneCount, 0, sizeof(uint32_t)));
      d.pubSrc = reinterpret_cast<const uint4*>(b + oReward);
      d.pubDst = reinterpret_cast<uint4*>(db);
      d.pubVec = static_cast<uint32_t>(outPadded / 16);
      d.doneCount = g.dDoneCount;
      d.hStepFlag = reinterpret_cast<uint32_t*>(db + outPadded + 16);
    }
  }
  BPSN_CUDA(sim, cudaEventCreateWithFlags(&g.done, cudaEventDisableTiming));
  return BPSN_OK;
}

// D2H of the result arrays + completion event
int32_t finishLaunch(bpsn_sim* sim, Group& g, cudaStream_t s, bool polarOnly) {
  // host mirrors need no copy: the kernels have stored into them (mapped pinned memory);
  // they are complete for the host once this event has been waited for
  (void)polarOnly;
  BPSN_CUDA(sim, cudaEventRecord(g.done, s));
  return BPSN_OK;
}

inline uint32_t blocksFor(uint32_t n, uint32_t bs) {
  return (n + bs - 1) / bs;
}

}  // namespace

// sqrtExact(x) == sqrtf(x), bit for bit, for every operand in [lo, hi]?
__global__ void __launch_bounds__(256)
k_selftest_sqrt(uint32_t lo, uint32_t hi, unsigned long long* mismatches) {
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  unsigned long long bad = 0;
  for (uint64_t i = lo + static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i <= hi;
       i += stride) {
    const float x = __uint_as_float(static_cast<uint32_t>(i));
    const uint32_t want = __float_as_uint(sqrtf(x));
    if (__float_as_uint(sqrtExact(x)) != want)
      bad++;
    if (sqrtCoreValid(x) && __float_as_uint(sqrtCore(x)) != want)
      bad++;  // the bare sequence on the range it claims
  }
  if (bad)
    atomicAdd(mismatches, bad);
}

extern "C" {

const char* bpsn_version(void) {
  return "bpsn 0.1 sm_100a";
}

const char* bpsn_last_error(const bpsn_sim* sim) {
  if (sim)
    return sim->lastError.c_str();
  return g_lastError.c_str();
}

int32_t bpsn_create(const bpsn_config* cfg, bpsn_sim** out) {
  if (!cfg || !out)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_create: null argument");
  *out = nullptr;
  if (cfg->task > BPSN_TASK_EXPLORATION)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_create: unknown task");
  if (cfg->num_envs == 0 || cfg->num_scenes == 0 || cfg->num_groups == 0 || cfg->num_groups > 2)
    return fail(nullptr, BPSN_ERR_INVALID_ARG,
                "bpsn_create: num_envs, num_scenes must be > 0 and num_groups 1 or 2");
  // the reference aborts on these (simulator/simulator.cpp:1503-1508, 1536-1538)
  if ((cfg->render_width == 0) != (cfg->render_height == 0) || cfg->render_width > 4096 ||
      cfg->render_height > 4096)
    return fail(nullptr, BPSN_ERR_INVALID_ARG,
                "bpsn_create: render_width and render_height must both be 0 or both in 1..4096");
  if (cfg->num_envs > kListEnvMask)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_create: at most 2^30 - 1 environments");
  const uint32_t numActive = cfg->num_active_scenes ? cfg->num_active_scenes : cfg->num_scenes;
  if (numActive > cfg->num_scenes)
    return fail(nullptr, BPSN_ERR_INVALID_ARG,
                "bpsn_create: more active scenes than scenes");
  if (cfg->num_envs % numActive != 0)
    return fail(nullptr, BPSN_ERR_INVALID_ARG,
                "Num environments is not a multiple of the number of active scenes");
  // (the reference also wants the active scenes to be a multiple of num_groups,
  // simulator.cpp:1536-1538, because each group renders its own scenes; here the groups share
  // the scene tables, so a single fixed scene may serve both groups: the Python constructor
  // keeps the reference's rule)
  const bool rotating = numActive < cfg->num_scenes;
  if (cfg->num_envs % cfg->num_groups != 0 ||
      (numActive % cfg->num_groups != 0 && (rotating || numActive != 1)))
    return fail(nullptr, BPSN_ERR_INVALID_ARG,
                "num_envs and the number of active scenes must be multiples of num_groups");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
    return fail(nullptr, BPSN_ERR_NO_DEVICE, "bpsn_create: no CUDA device available");
  if (cfg->gpu_id < 0 || cfg->gpu_id >= ndev)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_create: gpu_id out of range");
  bpsn_sim* sim = new bpsn_sim();
  sim->cfg = *cfg;
  sim->scenes.resize(cfg->num_scenes);
  sim->envScene.resize(cfg->num_envs);
  sim->numActive = numActive;
  sim->rotation = rotating;
  sim->activeScenes.resize(numActive);
  for (uint32_t i = 0; i < numActive; ++i)
    sim->activeScenes[i] = i;
  // glm::angleAxis(radians(+/-10), +Y) = (sin(a/2) * axis, cos(a/2)), on the
  // host libm as the reference does at static-init time (simulator.cpp:52-60)
  const float a = 10.f * 0.01745329251994329576923690768489f;
  const float sl = sinf(a * 0.5f), cl = cosf(a * 0.5f);
  const float na = -a;
  const float sr = sinf(na * 0.5f), cr = cosf(na * 0.5f);
  sim->turn = TurnConsts{0.f * sl, 1.f * sl, 0.f * sl, cl, 0.f * sr, 1.f * sr, 0.f * sr, cr};
  *out = sim;
  return BPSN_OK;
}

int32_t bpsn_destroy(bpsn_sim* sim) {
  if (!sim)
    return BPSN_OK;
  cudaSetDevice(sim->cfg.gpu_id);
  cudaDeviceSynchronize();
  for (auto& g : sim->groups) {
    cudaFree(g.stateBlob);
    cudaFree(g.scratch);
    cudaFree(g.fallbackScratch);
    cudaFree(g.dPlan);
    cudaFree(g.globalSlabs);
    cudaFree(g.dCtaMap);
    cudaFree(g.dDoneCount);
    cudaFree(g.dBatchStage);
    cudaFreeHost(const_cast<uint32_t*>(g.hListed));
    cudaFree(g.dOvList);
    cudaFree(g.dOvMeta);
    cudaFree(g.depth);
    cudaFreeHost(g.hActions);
    cudaFreeHost(g.hOut);
    if (g.done)
      cudaEventDestroy(g.done);
    for (cudaEvent_t ev : g.prof)
      if (ev)
        cudaEventDestroy(ev);
  }
  for (auto& s : sim->scenes)
    cudaFree(s.blob);
  cudaFree(sim->dScenes);
  cudaFree(sim->dEpisodes);
  cudaFree(sim->dEpNav);
  cudaFree(sim->dEpOffset);
  cudaFree(sim->dEpCount);
  cudaFree(sim->dBoxes);
  cudaFree(sim->dBoxOffset);
  cudaFree(sim->dBoxCount);
  cudaFree(sim->dFloor);
  cudaFree(sim->queryScratch);
  delete sim;
  return BPSN_OK;
}

int32_t bpsn_set_navmesh_blob(bpsn_sim* sim, uint32_t scene, const void* data, size_t size) {
  if (!sim || !data)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_navmesh_blob: null argument");
  if (sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_set_navmesh_blob: already finalized");
  if (scene >= sim->scenes.size())
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_navmesh_blob: scene index out of range");
  HostScene hs;
  std::string err = parseNavmesh(data, size, &hs);
  if (!err.empty())
    return fail(sim, BPSN_ERR_BAD_NAVMESH, err);
  sim->scenes[scene].host = std::move(hs);
  sim->scenes[scene].loaded = true;
  return BPSN_OK;
}

int32_t bpsn_set_navmesh_file(bpsn_sim* sim, uint32_t scene, const char* path) {
  if (!sim || !path)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_navmesh_file: null argument");
  FILE* fp = fopen(path, "rb");
  if (!fp)
    return fail(sim, BPSN_ERR_IO, std::string("Failed to load navmesh: ") + path);
  std::vector<uint8_t> buf;
  fseek(fp, 0, SEEK_END);
  long n = ftell(fp);
  fseek(fp, 0, SEEK_SET);
  if (n < 0) {
    fclose(fp);
    return fail(sim, BPSN_ERR_IO, std::string("Failed to load navmesh: ") + path);
  }
  buf.resize(static_cast<size_t>(n));
  size_t got = n ? fread(buf.data(), 1, buf.size(), fp) : 0;
  fclose(fp);
  if (got != buf.size())
    return fail(sim, BPSN_ERR_IO, std::string("Failed to load navmesh: ") + path);
  return bpsn_set_navmesh_blob(sim, scene, buf.data(), buf.size());
}

int32_t bpsn_set_episodes(bpsn_sim* sim, uint32_t scene, const bpsn_episode* episodes,
                          uint32_t count) {
  if (!sim || !episodes || count == 0)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_episodes: null or empty episode list");
  if (sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_set_episodes: already finalized");
  if (scene >= sim->scenes.size())
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_episodes: scene index out of range");
  sim->scenes[scene].episodes.assign(episodes, episodes + count);
  return BPSN_OK;
}

int32_t bpsn_set_env_scenes(bpsn_sim* sim, const uint32_t* env_scene, uint32_t count) {
  if (!sim || !env_scene)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_env_scenes: null argument");
  if (sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_set_env_scenes: already finalized");
  if (count != sim->cfg.num_envs)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_env_scenes: count != num_envs");
  for (uint32_t e = 0; e < count; ++e)
    if (env_scene[e] >= sim->cfg.num_scenes)
      return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_env_scenes: scene index out of range");
  if (sim->rotation)
    return fail(sim, BPSN_ERR_STATE,
                "bpsn_set_env_scenes: environments follow their slot's scene when scenes rotate");
  sim->envScene.assign(env_scene, env_scene + count);
  sim->envSceneExplicit = true;
  return BPSN_OK;
}

int32_t bpsn_set_active_scenes(bpsn_sim* sim, const uint32_t* scenes, uint32_t count) {
  if (!sim || !scenes)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_active_scenes: null argument");
  if (sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_set_active_scenes: already finalized");
  if (count != sim->numActive)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_active_scenes: count != num_active_scenes");
  for (uint32_t i = 0; i < count; ++i) {
    if (scenes[i] >= sim->cfg.num_scenes)
      return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_active_scenes: scene index out of range");
    for (uint32_t j = 0; j < i; ++j)
      if (scenes[j] == scenes[i])
        return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_active_scenes: a scene is listed twice");
  }
  sim->activeScenes.assign(scenes, scenes + count);
  return BPSN_OK;
}

int32_t bpsn_finalize(bpsn_sim* sim) {
  if (!sim)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_finalize: null handle");
  if (sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_finalize: already finalized");
  for (size_t i = 0; i < sim->scenes.size(); ++i) {
    if (!sim->scenes[i].loaded)
      return fail(sim, BPSN_ERR_STATE, "bpsn_finalize: scene " + std::to_string(i) + " has no navmesh");
    if (sim->scenes[i].episodes.empty())
      return fail(sim, BPSN_ERR_STATE, "bpsn_finalize: scene " + std::to_string(i) + " has no episodes");
  }
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  const uint32_t ns = sim->cfg.num_scenes;
  std::vector<NavScene> table(ns);
  std::vector<uint32_t> epOff(ns), epCnt(ns);
  std::vector<float> eps;
  for (uint32_t i = 0; i < ns; ++i) {
    int32_t rc = uploadScene(sim, sim->scenes[i]);
    if (rc)
      return rc;
    table[i] = sim->scenes[i].dev;
    epOff[i] = static_cast<uint32_t>(eps.size() / 10);
    epCnt[i] = static_cast<uint32_t>(sim->scenes[i].episodes.size());
    for (const bpsn_episode& ep : sim->scenes[i].episodes) {
      eps.insert(eps.end(), ep.start_position, ep.start_position + 3);
      eps.insert(eps.end(), ep.start_rotation, ep.start_rotation + 4);
      eps.insert(eps.end(), ep.goal, ep.goal + 3);
    }
  }
  BPSN_CUDA(sim, cudaMalloc(&sim->dScenes, sizeof(NavScene) * ns));
  BPSN_CUDA(sim, cudaMemcpy(sim->dScenes, table.data(), sizeof(NavScene) * ns,
                            cudaMemcpyHostToDevice));
  BPSN_CUDA(sim, cudaMalloc(&sim->dEpisodes, sizeof(float) * eps.size()));
  BPSN_CUDA(sim, cudaMemcpy(sim->dEpisodes, eps.data(), sizeof(float) * eps.size(),
                            cudaMemcpyHostToDevice));
  BPSN_CUDA(sim, cudaMalloc(&sim->dEpOffset, sizeof(uint32_t) * ns));
  BPSN_CUDA(sim, cudaMemcpy(sim->dEpOffset, epOff.data(), sizeof(uint32_t) * ns,
                            cudaMemcpyHostToDevice));
  BPSN_CUDA(sim, cudaMalloc(&sim->dEpCount, sizeof(uint32_t) * ns));
  BPSN_CUDA(sim, cudaMemcpy(sim->dEpCount, epCnt.data(), sizeof(uint32_t) * ns,
                            cudaMemcpyHostToDevice));
  sim->querySlots = 16384;
  BPSN_CUDA(sim, cudaMalloc(&sim->queryScratch, sizeof(AStarScratch) * sim->querySlots));
  const size_t totalEps = eps.size() / 10;
  BPSN_CUDA(sim, cudaMalloc(&sim->dEpNav, sizeof(EpisodeNav) * totalEps));
  unsigned long long* dSearchWork = nullptr;
  BPSN_CUDA(sim, cudaMalloc(&dSearchWork, sizeof(unsigned long long) * 2 * ns));
  BPSN_CUDA(sim, cudaMemset(dSearchWork, 0, sizeof(unsigned long long) * 2 * ns));
  for (uint32_t i = 0; i < ns; ++i) {
    const uint32_t slots = epCnt[i] < sim->querySlots ? epCnt[i] : sim->querySlots;
    k_episode_table<<<blocksFor(slots, 128), 128>>>(sim->dScenes + i,
                                                    sim->dEpisodes + 10 * static_cast<size_t>(epOff[i]),
                                                    epCnt[i], sim->queryScratch, slots,
                                                    sim->dEpNav + epOff[i], dSearchWork + 2 * i);
  }
  BPSN_CUDA(sim, cudaGetLastError());
  BPSN_CUDA(sim, cudaDeviceSynchronize());
  {
    // Work of one query per scene, in opened nodes: what the episodes' own searches (start ->
    // goal, the same pairs the steps will search between) needed on average, plus the part
    // of a query that does not depend on the search (move, funnel, finish: about six nodes'
    // worth of instructions).
    std::vector<unsigned long long> w(2 * ns);
    BPSN_CUDA(sim, cudaMemcpy(w.data(), dSearchWork, sizeof(unsigned long long) * 2 * ns,
                              cudaMemcpyDeviceToHost));
    BPSN_CUDA(sim, cudaFree(dSearchWork));
    sim->queryCost.assign(ns, 1.0);
    for (uint32_t i = 0; i < ns; ++i)
      sim->queryCost[i] = 6.0 + (w[2 * i + 1] ? static_cast<double>(w[2 * i]) / w[2 * i + 1] : 10.0);
  }
  sim->table.scenes = sim->dScenes;
  sim->table.episodes = sim->dEpisodes;
  sim->table.epNav = sim->dEpNav;
  sim->table.epOffset = sim->dEpOffset;
  sim->table.epCount = sim->dEpCount;

  if (sim->cfg.render_width && sim->cfg.render_height) {
    std::vector<float> boxes, floors(4 * static_cast<size_t>(ns), 0.f);
    std::vector<uint32_t> bOff(ns), bCnt(ns);
    for (uint32_t i = 0; i < ns; ++i) {
      bOff[i] = static_cast<uint32_t>(boxes.size() / 6);
      bCnt[i] = static_cast<uint32_t>(sim->scenes[i].boxes.size() / 6);
      boxes.insert(boxes.end(), sim->scenes[i].boxes.begin(), sim->scenes[i].boxes.end());
      for (int k = 0; k < 4; ++k)
        floors[4 * static_cast<size_t>(i) + k] = sim->scenes[i].floor[k];
    }
    BPSN_CUDA(sim, cudaMalloc(&sim->dBoxes, sizeof(float) * (boxes.size() + 6)));
    if (!boxes.empty())
      BPSN_CUDA(sim, cudaMemcpy(sim->dBoxes, boxes.data(), sizeof(float) * boxes.size(),
                                cudaMemcpyHostToDevice));
    BPSN_CUDA(sim, cudaMalloc(&sim->dBoxOffset, sizeof(uint32_t) * ns));
    BPSN_CUDA(sim, cudaMemcpy(sim->dBoxOffset, bOff.data(), sizeof(uint32_t) * ns,
                              cudaMemcpyHostToDevice));
    BPSN_CUDA(sim, cudaMalloc(&sim->dBoxCount, sizeof(uint32_t) * ns));
    BPSN_CUDA(sim, cudaMemcpy(sim->dBoxCount, bCnt.data(), sizeof(uint32_t) * ns,
                              cudaMemcpyHostToDevice));
    BPSN_CUDA(sim, cudaMalloc(&sim->dFloor, sizeof(float) * 4 * ns));
    BPSN_CUDA(sim, cudaMemcpy(sim->dFloor, floors.data(), sizeof(float) * 4 * ns,
                              cudaMemcpyHostToDevice));
    sim->render.boxes = sim->dBoxes;
    sim->render.boxOffset = sim->dBoxOffset;
    sim->render.boxCount = sim->dBoxCount;
    sim->render.floor = sim->dFloor;
  }

  const uint32_t ng = sim->cfg.num_groups;
  const uint32_t B = sim->cfg.num_envs / ng;
  sim->groups.resize(ng);
  if (!sim->envSceneExplicit) {
    // num_envs / num_active_scenes consecutive environments per slot, group-major then
    // slot-major (simulator/simulator.cpp:1205-1221, 1581-1592)
    const uint32_t perSlot = sim->cfg.num_envs / sim->numActive;
    for (uint32_t e = 0; e < sim->cfg.num_envs; ++e)
      sim->envScene[e] = sim->activeScenes[e / perSlot];
  }
  // The scenes that wait for a slot, in ascending order (the reference's inactive_scenes_,
  // simulator.cpp:1518-1534), dealt to the groups in turn: each group then rotates through
  // its own share, whatever the other group is doing at the time (the groups' steps may
  // overlap on the GPU).  The reference has one list for all groups.
  sim->pools.assign(ng, std::vector<uint32_t>());
  if (sim->rotation) {
    std::vector<uint8_t> active(ns, 0);
    for (uint32_t sc : sim->activeScenes)
      active[sc] = 1;
    uint32_t k = 0;
    for (uint32_t sc = 0; sc < ns; ++sc)
      if (!active[sc])
        sim->pools[k++ % ng].push_back(sc);
  }
  for (uint32_t gi = 0; gi < ng; ++gi) {
    int32_t rc = allocGroup(sim, sim->groups[gi], B, gi * B, gi);
    if (rc)
      return rc;
  }
  if (sim->rotation) {
    // Every slot starts its first move right away (RolloutGenerator's constructor calls
    // startSceneSwap on every swapper, simulator.cpp:1594): the environments begin in the
    // first scenes and follow at the end of their first episodes.
    for (uint32_t gi = 0; gi < ng; ++gi) {
      GroupDev first = sim->groups[gi].dev;
      first.swapInterval = 0u;  // all slots, whatever the pace of the later moves
      first.stepId = 0u;
      k_swap<<<1, 32>>>(first, static_cast<uint32_t>(sim->cfg.seed),
                        static_cast<uint32_t>(sim->cfg.seed >> 32));
    }
    BPSN_CUDA(sim, cudaGetLastError());
    BPSN_CUDA(sim, cudaDeviceSynchronize());
  }
  sim->finalized = true;
  return BPSN_OK;
}

int32_t bpsn_swap_stats(bpsn_sim* sim, uint64_t* num_swaps, float* scenes_in_use,
                        float* envs_per_scene) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_swap_stats: handle not finalized");
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  BPSN_CUDA(sim, cudaDeviceSynchronize());
  uint64_t swaps = 0;
  float scenes = 0.f, perScene = 0.f;
  std::vector<uint32_t> envScene;
  for (Group& g : sim->groups) {
    uint32_t c = 0;
    BPSN_CUDA(sim, cudaMemcpy(&c, g.dev.swapCount, sizeof(c), cudaMemcpyDeviceToHost));
    // (the first move of every slot is started at set-up and not counted, as in the reference)
    const uint32_t atSetup = g.dev.poolSize ? g.dev.numSlots : 0u;
    swaps += c > atSetup ? c - atSetup : 0u;
    envScene.resize(g.dev.B);
    BPSN_CUDA(sim, cudaMemcpy(envScene.data(), g.dev.scene, sizeof(uint32_t) * g.dev.B,
                              cudaMemcpyDeviceToHost));
    // EnvironmentGroup::sceneStats (simulator.cpp:1212-1227)
    std::vector<uint32_t> count(sim->cfg.num_scenes, 0u);
    for (uint32_t sc : envScene)
      count[sc]++;
    uint32_t distinct = 0;
    for (uint32_t c2 : count)
      distinct += c2 ? 1u : 0u;
    scenes += static_cast<float>(distinct);
    perScene += distinct ? static_cast<float>(g.dev.B) / static_cast<float>(distinct) : 0.f;
  }
  if (num_swaps)
    *num_swaps = swaps;
  if (scenes_in_use)
    *scenes_in_use = scenes;
  if (envs_per_scene)
    *envs_per_scene = perScene;
  return BPSN_OK;
}

int32_t bpsn_reset(bpsn_sim* sim, uint32_t group, void* stream) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_reset: handle not finalized");
  if (group >= sim->groups.size())
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_reset: group out of range");
  Group& g = sim->groups[group];
  if (g.inFlight)
    return fail(sim, BPSN_ERR_STATE, "Not done with previous simulation");
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint32_t B = g.dev.B;
  k_reset_all<<<blocksFor(B, 256), 256, 0, s>>>(g.dev, sim->table,
                                                static_cast<uint32_t>(sim->cfg.seed),
                                                static_cast<uint32_t>(sim->cfg.seed >> 32));
  BPSN_CUDA(sim, cudaGetLastError());
  int32_t rc = finishLaunch(sim, g, s, /*polarOnly=*/true);
  if (rc)
    return rc;
  if (sim->cfg.flags & BPSN_FLAG_HOST_MIRRORS)
    BPSN_CUDA(sim, cudaEventSynchronize(g.done));
  return BPSN_OK;
}

int32_t bpsn_step_start(bpsn_sim* sim, uint32_t group, const int64_t* actions,
                        int32_t actions_mem, void* stream) {
  return bpsn_step_start_ex(sim, group, actions, actions_mem, stream, nullptr, nullptr, nullptr);
}

int32_t bpsn_step_start_ex(bpsn_sim* sim, uint32_t group, const int64_t* actions,
                           int32_t actions_mem, void* stream, float* reward_out,
                           uint8_t* mask_out, float* polar_out) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_step_start: handle not finalized");
  if (group >= sim->groups.size())
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_step_start: group out of range");
  if (!actions)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_step_start: null actions");
  Group& g = sim->groups[group];
  if (g.inFlight)
    return fail(sim, BPSN_ERR_STATE, "Not done with previous simulation");
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint32_t B = g.dev.B;
  const int64_t* dAct = actions;
  const uint8_t* dAct8 = nullptr;
  if (actions_mem == BPSN_MEM_HOST) {
    // The staging buffer is read in place by the kernel of this step; without host
    // mirrors step_end does not wait for the device, so make sure the previous step
    // is through with the buffer before overwriting it.
    if (!(sim->cfg.flags & BPSN_FLAG_HOST_MIRRORS))
      BPSN_CUDA(sim, cudaEventSynchronize(g.done));
    // one pass: narrow and validate (a bad action leaves the buffer half written, which
    // is harmless: nothing is launched)
    uint64_t bad = 0;
    for (uint32_t i = 0; i < B; ++i) {
      const uint64_t a = static_cast<uint64_t>(actions[i]);
      bad |= a;
      g.hActions[i] = static_cast<uint8_t>(a);
    }
    if (bad > 3) {
      for (uint32_t i = 0; i < B; ++i)
        if (actions[i] < 0 || actions[i] > 3)
          return fail(sim, BPSN_ERR_BAD_ACTION, "Unknown action: " + std::to_string(actions[i]));
    }
    dAct = nullptr;
    dAct8 = g.dActions8;
  } else if (actions_mem != BPSN_MEM_DEVICE) {
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_step_start: actions_mem must be host or device");
  }
  // The work-list counters alternate between two arrays: this step fills one and
  // zeroes the other for the step after it (both start zeroed).
  std::swap(g.dev.counts, g.dev.countsNext);
  const bool prof = g.profiling;
  GroupDev gd = g.dev;
  gd.stepId = ++g.stepCounter;  // (never 0: the headers of the overflow segments start zeroed)
  if (g.publish) {
    // the step kernels write device memory only; the last CTA publishes (GroupDev::pubDst)
    gd.hReward = nullptr;
    gd.hMask = nullptr;
    gd.hInfo = nullptr;
    gd.hPolar = nullptr;
  }
  gd.rewardOut = reward_out;
  gd.maskOut = mask_out;
  gd.polarOut = polar_out;
  const uint32_t seedLo = static_cast<uint32_t>(sim->cfg.seed);
  const uint32_t seedHi = static_cast<uint32_t>(sim->cfg.seed >> 32);
  // Both kernels are launched with programmatic stream serialization: each may
  // become resident while its predecessor in the stream is still running and
  // does its read-only prologue (the step kernel: the copy of the scene image
  // into shared memory) before it waits for the predecessor to finish.  Not
  // while per-launch times are being recorded.
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t lc = {};
  lc.stream = s;
  lc.attrs = pdl;
  lc.numAttrs = prof ? 0 : 1;
  if (prof) cudaEventRecord(g.prof[0], s);
  lc.gridDim = dim3(blocksFor(B, 256));
  lc.blockDim = dim3(256);
  lc.dynamicSmemBytes = 0;
  if (!g.fused)
    BPSN_CUDA(sim, cudaLaunchKernelEx(&lc, k_pre, gd, sim->table, dAct, dAct8, sim->turn, seedLo,
                                      seedHi));
  if (prof) cudaEventRecord(g.prof[1], s);
  if (g.anyWarpScene) {
    lc.gridDim = dim3(g.numCtas);
    lc.blockDim = dim3(512);
    lc.dynamicSmemBytes = g.geoSmem;
    const bool rot = g.dev.rotation != 0u;
    const bool batchedNow = g.batched && g.batchForce != 2 &&
                            (g.batchForce == 1 || *g.hListed >= g.batchMinListed);
    auto* kernel = g.fused           ? k_step_warp<0, false, true>
                   : batchedNow      ? (g.warpMode == 0 ? k_step_warp<0, false, false, true>
                                                        : k_step_warp<1, false, false, true>)
                   : g.warpMode == 0 ? (rot ? k_step_warp<0, true> : k_step_warp<0, false>)
                   : g.warpMode == 1 ? (rot ? k_step_warp<1, true> : k_step_warp<1, false>)
                                     : (rot ? k_step_warp<2, true> : k_step_warp<2, false>);
    BPSN_CUDA(sim, cudaLaunchKernelEx(&lc, kernel, gd, sim->table,
                                      static_cast<const WarpPlan*>(g.dPlan),
                                      static_cast<const uint4*>(g.dCtaMap), g.fallbackScratch,
                                      g.globalSlabs, g.globalSlabStride, seedLo, seedHi, dAct,
                                      dAct8, sim->turn));
  }
  if (g.anyThreadScene) {  // meshes the warp kernel cannot index (it skips the other scenes)
    if (g.anyWarpScene)
      lc.numAttrs = 0;  // behind the warp kernel: plain stream order, no early start
    lc.gridDim = dim3(blocksFor(g.maxListLen, 128), g.dev.numLists);
    lc.blockDim = dim3(128);
    lc.dynamicSmemBytes = 0;
    BPSN_CUDA(sim, cudaLaunchKernelEx(&lc, k_step_thread, gd, sim->table,
                                      static_cast<const WarpPlan*>(g.dPlan), g.scratch, seedLo,
                                      seedHi));
  }
  if (prof) cudaEventRecord(g.prof[2], s);
  if (g.dev.rotation && g.dev.poolSize) {  // slots that are complete start their next move
    lc.numAttrs = prof ? 0 : 1;
    lc.gridDim = dim3(1);
    lc.blockDim = dim3(32);
    lc.dynamicSmemBytes = 0;
    BPSN_CUDA(sim, cudaLaunchKernelEx(&lc, k_swap, gd, seedLo, seedHi));
  }
  BPSN_CUDA(sim, cudaGetLastError());
  int32_t rc = finishLaunch(sim, g, s, /*polarOnly=*/false);
  if (rc)
    return rc;
  g.inFlight = true;
  return BPSN_OK;
}

int32_t bpsn_set_scene_geometry(bpsn_sim* sim, uint32_t scene, const float* floor4,
                                const float* boxes, uint32_t num_boxes) {
  if (!sim || !floor4 || (num_boxes && !boxes))
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_scene_geometry: null argument");
  if (sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_set_scene_geometry: already finalized");
  if (scene >= sim->scenes.size())
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_set_scene_geometry: scene index out of range");
  DeviceScene& ds = sim->scenes[scene];
  for (int k = 0; k < 4; ++k)
    ds.floor[k] = floor4[k];
  ds.boxes.assign(boxes, boxes + 6 * static_cast<size_t>(num_boxes));
  for (uint32_t b = 0; b < num_boxes; ++b)
    for (int k = 0; k < 3; ++k)
      if (!(ds.boxes[6 * b + k] <= ds.boxes[6 * b + 3 + k]))
        return fail(sim, BPSN_ERR_INVALID_ARG,
                    "bpsn_set_scene_geometry: box " + std::to_string(b) + " has min > max");
  return BPSN_OK;
}

int32_t bpsn_render(bpsn_sim* sim, uint32_t group, void* stream) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_render: handle not finalized");
  if (group >= sim->groups.size())
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_render: group out of range");
  Group& g = sim->groups[group];
  if (!g.depth)
    return fail(sim, BPSN_ERR_STATE, "bpsn_render: the handle was created without a render size");
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  k_depth<<<g.dev.B, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g.dev, sim->render, g.depth, sim->cfg.render_width, sim->cfg.render_height);
  BPSN_CUDA(sim, cudaGetLastError());
  return BPSN_OK;
}

int32_t bpsn_step_end(bpsn_sim* sim, uint32_t group) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_step_end: handle not finalized");
  if (group >= sim->groups.size())
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_step_end: group out of range");
  Group& g = sim->groups[group];
  if (!g.inFlight)
    return fail(sim, BPSN_ERR_STATE, "Simulation already done");
  g.inFlight = false;
  if (sim->cfg.flags & BPSN_FLAG_HOST_MIRRORS) {
    bool out = false;
    if (g.publish) {
      // The results are complete on the host once the flag shows this step's number (written
      // behind them, with a system-wide fence in between): poll it for a while before falling
      // back to the event, which also covers a step that could not publish.
      const uint32_t want = g.stepCounter;
      for (int spin = 0; spin < 200000 && !out; ++spin) {
        out = *g.hStepFlag == want;
        if (!out)
          __builtin_ia32_pause();
      }
    }
    if (!out)
      BPSN_CUDA(sim, cudaEventSynchronize(g.done));
    if (g.hErr && *g.hErr)
      return fail(sim, BPSN_ERR_CUDA,
                  "bpsn_step_end: a step kernel gave up waiting for its scene tables; the "
                  "environments it served keep the outputs of the step before "
                  "(bpsn_device_error_flags)");
  }
  if (g.profiling) {
    BPSN_CUDA(sim, cudaEventSynchronize(g.prof[2]));
    for (int k = 0; k < 2; ++k) {
      float ms = 0.f;
      BPSN_CUDA(sim, cudaEventElapsedTime(&ms, g.prof[k], g.prof[k + 1]));
      if (k == 0 && g.fused) ms = 0.f;  // one launch per step: no k_pre between the two events
      g.profMs[k] += ms;
    }
    g.profSteps++;
  }
  return BPSN_OK;
}

int32_t bpsn_device_error_flags(bpsn_sim* sim, uint32_t group, uint32_t* flags) {
  if (!sim || !sim->finalized || group >= sim->groups.size() || !flags)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_device_error_flags: bad argument");
  Group& g = sim->groups[group];
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  BPSN_CUDA(sim, cudaMemcpy(flags, g.dev.errFlags, sizeof(uint32_t),
                            cudaMemcpyDeviceToHost));
  return BPSN_OK;
}

int32_t bpsn_profile_enable(bpsn_sim* sim, uint32_t group, int32_t enable) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_profile_enable: handle not finalized");
  if (group >= sim->groups.size())
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_profile_enable: group out of range");
  Group& g = sim->groups[group];
  if (g.inFlight)
    return fail(sim, BPSN_ERR_STATE, "bpsn_profile_enable: a step is in flight");
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  if (enable && !g.prof[0])
    for (cudaEvent_t& ev : g.prof)
      BPSN_CUDA(sim, cudaEventCreate(&ev));
  g.profiling = enable != 0;
  for (double& v : g.profMs)
    v = 0;
  g.profSteps = 0;
  return BPSN_OK;
}

int32_t bpsn_profile_read(bpsn_sim* sim, uint32_t group, double* ms2, uint64_t* steps) {
  if (!sim || !sim->finalized || group >= sim->groups.size() || !ms2)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_profile_read: bad argument");
  Group& g = sim->groups[group];
  for (int k = 0; k < 2; ++k)
    ms2[k] = g.profMs[k];
  if (steps)
    *steps = g.profSteps;
  return BPSN_OK;
}

int32_t bpsn_get_ptr(bpsn_sim* sim, uint32_t group, int32_t field, int32_t mem, void** ptr,
                     size_t* bytes) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_get_ptr: handle not finalized");
  if (group >= sim->groups.size() || field < 0 || field >= BPSN_FIELD_COUNT || !ptr)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_get_ptr: bad group, field or null output");
  Group& g = sim->groups[group];
  if (mem == BPSN_MEM_DEVICE) {
    *ptr = g.fieldPtr[field];
  } else if (mem == BPSN_MEM_HOST) {
    if (!(sim->cfg.flags & BPSN_FLAG_HOST_MIRRORS))
      return fail(sim, BPSN_ERR_STATE, "bpsn_get_ptr: host mirrors were not enabled at creation");
    switch (field) {
      case BPSN_FIELD_REWARD: *ptr = g.hReward; break;
      case BPSN_FIELD_MASK: *ptr = g.hMask; break;
      case BPSN_FIELD_INFO: *ptr = g.hInfo; break;
      case BPSN_FIELD_POLAR: *ptr = g.hPolar; break;
      default:
        return fail(sim, BPSN_ERR_INVALID_ARG,
                    "bpsn_get_ptr: only reward, mask, info and polar have host mirrors");
    }
  } else {
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_get_ptr: mem must be host or device");
  }
  if (bytes)
    *bytes = g.fieldBytes[field];
  return BPSN_OK;
}

int32_t bpsn_scene_info(bpsn_sim* sim, uint32_t scene, int32_t* num_polys, int32_t* num_disabled,
                        int32_t* num_islands) {
  if (!sim || scene >= sim->scenes.size() || !sim->scenes[scene].loaded)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_scene_info: scene not loaded");
  const HostScene& h = sim->scenes[scene].host;
  if (num_polys)
    *num_polys = static_cast<int32_t>(h.polys.size());
  if (num_disabled)
    *num_disabled = h.numDisabled;
  if (num_islands)
    *num_islands = h.numIslands;
  return BPSN_OK;
}

int32_t bpsn_query_snap(bpsn_sim* sim, uint32_t scene, uint32_t n, const float* points,
                        float* out_points, uint32_t* out_refs, void* stream) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_query_snap: handle not finalized");
  if (scene >= sim->scenes.size() || !points || !out_points || !out_refs)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_query_snap: bad argument");
  if (n == 0)
    return BPSN_OK;
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  k_query_snap<<<blocksFor(n, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      sim->dScenes + scene, n, points, out_points, out_refs);
  BPSN_CUDA(sim, cudaGetLastError());
  return BPSN_OK;
}

int32_t bpsn_query_try_step(bpsn_sim* sim, uint32_t scene, uint32_t n, const float* start,
                            const uint32_t* start_refs, const float* end, float* out_points,
                            uint32_t* out_refs, void* stream) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_query_try_step: handle not finalized");
  if (scene >= sim->scenes.size() || !start || !start_refs || !end || !out_points || !out_refs)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_query_try_step: bad argument");
  if (n == 0)
    return BPSN_OK;
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  k_query_try_step<<<blocksFor(n, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      sim->dScenes + scene, n, start, start_refs, end, out_points, out_refs);
  BPSN_CUDA(sim, cudaGetLastError());
  return BPSN_OK;
}

int32_t bpsn_query_geodesic(bpsn_sim* sim, uint32_t scene, uint32_t n, const float* start,
                            const uint32_t* start_refs, const float* end,
                            const uint32_t* end_refs, float* out_dist, uint32_t* out_status,
                            void* stream) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_query_geodesic: handle not finalized");
  if (scene >= sim->scenes.size() || !start || !start_refs || !end || !end_refs || !out_dist)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_query_geodesic: bad argument");
  if (n == 0)
    return BPSN_OK;
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  const uint32_t slots = n < sim->querySlots ? n : sim->querySlots;
  k_query_geodesic<<<blocksFor(slots, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      sim->dScenes + scene, sim->queryScratch, slots, n, start, start_refs, end, end_refs,
      out_dist, out_status);
  BPSN_CUDA(sim, cudaGetLastError());
  return BPSN_OK;
}


size_t bpsn_gae_workspace_bytes(uint32_t N) {
  return sizeof(GaeStat) * (static_cast<size_t>(blocksFor(N, kGaeBlock)) + 1);
}

int32_t bpsn_gae(const float* rewards, float* values, const uint8_t* masks,
                 const float* next_value, float* returns, float* advantages, uint32_t T,
                 uint32_t N, double gamma, double tau, int32_t normalize, float eps,
                 void* workspace, void* stream) {
  if (!rewards || !values || !masks || !returns)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_gae: null tensor");
  if (T == 0 || N == 0)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_gae: T and N must be positive");
  if (normalize && (!advantages || !workspace))
    return fail(nullptr, BPSN_ERR_INVALID_ARG,
                "bpsn_gae: normalisation needs the advantages output and a workspace");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint32_t blocks = blocksFor(N, kGaeBlock);
  GaeStat* partials = normalize ? static_cast<GaeStat*>(workspace) : nullptr;
  k_gae_scan<<<blocks, kGaeBlock, 0, s>>>(rewards, values, masks, next_value, returns, advantages,
                                          T, N, static_cast<float>(gamma),
                                          static_cast<float>(gamma * tau), partials);
  if (normalize) {
    const size_t total = static_cast<size_t>(T) * N;
    uint32_t nb = static_cast<uint32_t>((total + 256 * 4 - 1) / (256 * 4));
    if (nb > 148 * 8)
      nb = 148 * 8;
    if (nb == 0)
      nb = 1;
    // resident and waiting when the scan ends (gaeWaitForPredecessor)
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(nb);
    lc.blockDim = dim3(256);
    lc.stream = s;
    lc.attrs = pdl;
    lc.numAttrs = 1;
    const GaeStat* cpartials = partials;
    cudaError_t le = cudaLaunchKernelEx(&lc, k_gae_normalize, advantages, total, cpartials, blocks,
                                        eps);
    if (le != cudaSuccess)
      return fail(nullptr, BPSN_ERR_CUDA, std::string("bpsn_gae launch: ") + cudaGetErrorString(le));
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(nullptr, BPSN_ERR_CUDA, std::string("bpsn_gae launch: ") + cudaGetErrorString(e));
  return BPSN_OK;
}

// ---------------------------------------------------------------------------
// Advantage normalisation over segments (see gae_kernels.cuh)

namespace {
constexpr uint32_t kAdvMaxBlocksPerSeg = 592;  // 4 x 148 SMs when a single segment is given

int32_t buildAdvList(const char* who, const bpsn_adv_segment* segments, uint32_t num_segments,
                     uint32_t T, AdvSegmentList* out) {
  if (!segments || num_segments == 0 || num_segments > BPSN_MAX_ADV_SEGMENTS)
    return fail(nullptr, BPSN_ERR_INVALID_ARG,
                std::string(who) + ": between 1 and " + std::to_string(BPSN_MAX_ADV_SEGMENTS) +
                    " segments");
  if (T == 0)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, std::string(who) + ": T must be positive");
  size_t largest = 0;
  for (uint32_t i = 0; i < num_segments; ++i) {
    const bpsn_adv_segment& sg = segments[i];
    if (!sg.advantages || sg.start >= sg.end || sg.end > sg.N)
      return fail(nullptr, BPSN_ERR_INVALID_ARG,
                  std::string(who) + ": segment " + std::to_string(i) +
                      " needs a tensor and 0 <= start < end <= N");
    for (uint32_t j = 0; j < i; ++j)
      if (segments[j].advantages == sg.advantages && segments[j].start < sg.end &&
          sg.start < segments[j].end)
        return fail(nullptr, BPSN_ERR_INVALID_ARG,
                    std::string(who) + ": segments " + std::to_string(j) + " and " +
                        std::to_string(i) + " overlap");
    out->seg[i] = AdvSegment{sg.advantages, sg.N, sg.start, sg.end, sg.group};
    const size_t elems = static_cast<size_t>(T) * (sg.end - sg.start);
    if (elems > largest)
      largest = elems;
  }
  out->count = num_segments;
  out->T = T;
  uint32_t bps = static_cast<uint32_t>((largest + 2047) / 2048);
  const uint32_t cap = kAdvMaxBlocksPerSeg / num_segments ? kAdvMaxBlocksPerSeg / num_segments : 1u;
  if (bps > cap)
    bps = cap;
  if (bps == 0)
    bps = 1;
  out->blocksPerSeg = bps;
  return BPSN_OK;
}
}  // namespace

size_t bpsn_adv_workspace_bytes(void) {
  return sizeof(GaeStat) * static_cast<size_t>(kAdvMaxBlocksPerSeg + BPSN_MAX_ADV_SEGMENTS);
}

int32_t bpsn_adv_normalize(const bpsn_adv_segment* segments, uint32_t num_segments, uint32_t T,
                           float eps, void* workspace, void* stream) {
  if (!workspace)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_adv_normalize: null workspace");
  AdvSegmentList list{};
  int32_t rc = buildAdvList("bpsn_adv_normalize", segments, num_segments, T, &list);
  if (rc)
    return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  GaeStat* partials = static_cast<GaeStat*>(workspace);
  const dim3 grid(list.blocksPerSeg, list.count);
  k_adv_stats<<<grid, kAdvBlock, 0, s>>>(list, partials);
  k_adv_normalize<<<grid, kAdvBlock, 0, s>>>(list, partials, eps);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(nullptr, BPSN_ERR_CUDA,
                std::string("bpsn_adv_normalize launch: ") + cudaGetErrorString(e));
  return BPSN_OK;
}

int32_t bpsn_adv_mean(const bpsn_adv_segment* segments, uint32_t num_segments, uint32_t T,
                      float* mean_out, void* workspace, void* stream) {
  if (!workspace || !mean_out)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_adv_mean: null workspace or output");
  AdvSegmentList list{};
  int32_t rc = buildAdvList("bpsn_adv_mean", segments, num_segments, T, &list);
  if (rc)
    return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  GaeStat* partials = static_cast<GaeStat*>(workspace);
  k_adv_stats<<<dim3(list.blocksPerSeg, list.count), kAdvBlock, 0, s>>>(list, partials);
  k_adv_mean<<<1, 32, 0, s>>>(list, partials, mean_out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(nullptr, BPSN_ERR_CUDA, std::string("bpsn_adv_mean launch: ") + cudaGetErrorString(e));
  return BPSN_OK;
}

int32_t bpsn_adv_ema_shift(const bpsn_adv_segment* segments, uint32_t num_segments, uint32_t T,
                           float* ema_state, const float* mean, float beta, void* stream) {
  if (!ema_state || !mean)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_adv_ema_shift: null state or mean");
  if (!(beta >= 0.f && beta < 1.f))
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_adv_ema_shift: beta must be in [0, 1)");
  AdvSegmentList list{};
  int32_t rc = buildAdvList("bpsn_adv_ema_shift", segments, num_segments, T, &list);
  if (rc)
    return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  k_adv_ema_update<<<1, 32, 0, s>>>(ema_state, mean, beta);
  k_adv_shift<<<dim3(list.blocksPerSeg, list.count), kAdvBlock, 0, s>>>(list, ema_state);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(nullptr, BPSN_ERR_CUDA,
                std::string("bpsn_adv_ema_shift launch: ") + cudaGetErrorString(e));
  return BPSN_OK;
}

// ---------------------------------------------------------------------------
// bpsn_gae_static: the same two GAE launches as bpsn_gae, for callers that are
// not able to provide a device workspace.  The per-block advantage statistics
// go to a fixed array that is part of the library image, so the call performs
// no device or host allocation of any kind.

constexpr uint32_t kGaeStaticMaxEnvs = 262144;  // environments per call
constexpr uint32_t kGaeStaticMaxBlocks = kGaeStaticMaxEnvs / kGaeBlock;

// 2048 x 24 bytes = 48 KB, resident on every GPU that loads this library.
static __device__ __align__(256) GaeStat g_gaeStaticPartials[kGaeStaticMaxBlocks];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_gaeStaticMutex;
GaeStat* g_gaeStaticPtr[kMaxDevices] = {};
}  // namespace

int32_t bpsn_gae_static(const float* rewards, float* values, const uint8_t* masks,
                        const float* next_value, float* returns, float* advantages, uint32_t T,
                        uint32_t N, double gamma, double tau, int32_t normalize, float eps,
                        void* stream) {
  if (!rewards || !values || !masks || !returns)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_gae_static: null tensor");
  if (T == 0 || N == 0)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_gae_static: T and N must be positive");
  if (N > kGaeStaticMaxEnvs)
    return fail(nullptr, BPSN_ERR_INVALID_ARG,
                "bpsn_gae_static: N = " + std::to_string(N) + " exceeds the built-in scratch (" +
                    std::to_string(kGaeStaticMaxEnvs) +
                    " environments per call); use bpsn_gae with a caller-provided workspace");
  if (normalize && !advantages)
    return fail(nullptr, BPSN_ERR_INVALID_ARG,
                "bpsn_gae_static: normalisation needs the advantages output");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(nullptr, BPSN_ERR_CUDA, "bpsn_gae_static: cannot identify the current device");
  GaeStat* partials = nullptr;
  {
    // Once per device, with that device current: turn the array's host-side
    // symbol into the device address kernels can use.  The symbol itself is
    // not a device pointer and must never be handed to a kernel.
    std::lock_guard<std::mutex> lock(g_gaeStaticMutex);
    if (!g_gaeStaticPtr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_gaeStaticPartials);
      if (e != cudaSuccess || !p)
        return fail(nullptr, BPSN_ERR_CUDA,
                    std::string("bpsn_gae_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
      g_gaeStaticPtr[dev] = static_cast<GaeStat*>(p);
    }
    partials = g_gaeStaticPtr[dev];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint32_t blocks = blocksFor(N, kGaeBlock);
  // Every block overwrites its own slot before the second launch reads slots
  // [0, blocks): nothing in the array has to start at zero.
  k_gae_scan<<<blocks, kGaeBlock, 0, s>>>(rewards, values, masks, next_value, returns, advantages,
                                          T, N, static_cast<float>(gamma),
                                          static_cast<float>(gamma * tau),
                                          normalize ? partials : nullptr);
  if (normalize) {
    const size_t total = static_cast<size_t>(T) * N;
    uint32_t nb = static_cast<uint32_t>((total + 256 * 4 - 1) / (256 * 4));
    if (nb > 148 * 8)
      nb = 148 * 8;
    if (nb == 0)
      nb = 1;
    k_gae_normalize<<<nb, 256, 0, s>>>(advantages, total, partials, blocks, eps);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(nullptr, BPSN_ERR_CUDA,
                std::string("bpsn_gae_static launch: ") + cudaGetErrorString(e));
  return BPSN_OK;
}

// Step form of large batches (diagnostic): 0 chosen step by step, 1 always 32 entries at a
// time where the group allows it, 2 always entry by entry.
int32_t bpsn_debug_force_batched(bpsn_sim* sim, uint32_t group, int32_t mode) {
  if (!sim || !sim->finalized || group >= sim->groups.size() || mode < 0 || mode > 2)
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_debug_force_batched: bad argument");
  sim->groups[group].batchForce = mode;
  return BPSN_OK;
}

// Presets the search counter of every global-memory slab of a group (diagnostic: lets a test
// drive the counters across the point where the 15-bit visit tag wraps and the slabs are wiped).
int32_t bpsn_debug_set_search_count(bpsn_sim* sim, uint32_t group, uint32_t count) {
  if (!sim || !sim->finalized)
    return fail(sim, BPSN_ERR_STATE, "bpsn_debug_set_search_count: handle not finalized");
  if (group >= sim->groups.size())
    return fail(sim, BPSN_ERR_INVALID_ARG, "bpsn_debug_set_search_count: group out of range");
  Group& g = sim->groups[group];
  if (g.inFlight)
    return fail(sim, BPSN_ERR_STATE, "bpsn_debug_set_search_count: a step is in flight");
  if (!g.globalSlabs)
    return BPSN_OK;  // every slab of this group lives in shared memory
  BPSN_CUDA(sim, cudaSetDevice(sim->cfg.gpu_id));
  BPSN_CUDA(sim, cudaDeviceSynchronize());
  const size_t slabs = g.numGlobalSlabs;
  std::vector<uint32_t> h(slabs, count);
  BPSN_CUDA(sim, cudaMemcpy2D(g.globalSlabs + g.globalSlabStride - kGlobalSlabExtra,
                              g.globalSlabStride, h.data(), sizeof(uint32_t), sizeof(uint32_t),
                              slabs, cudaMemcpyHostToDevice));
  return BPSN_OK;
}

// Self-test of sqrtExact() against the compiler's IEEE sqrtf over every fp32
// bit pattern in [first_bits, last_bits]; counts the operands whose results
// differ in any bit.
int32_t bpsn_selftest_sqrt(int32_t gpu_id, uint32_t first_bits, uint32_t last_bits,
                           uint64_t* mismatches) {
  if (!mismatches || first_bits > last_bits)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_selftest_sqrt: bad arguments");
  if (cudaSetDevice(gpu_id) != cudaSuccess)
    return fail(nullptr, BPSN_ERR_NO_DEVICE, "bpsn_selftest_sqrt: no such device");
  unsigned long long* dCount = nullptr;
  cudaError_t e = cudaMalloc(&dCount, sizeof(unsigned long long));
  if (e == cudaSuccess)
    e = cudaMemset(dCount, 0, sizeof(unsigned long long));
  if (e == cudaSuccess) {
    k_selftest_sqrt<<<148 * 8, 256>>>(first_bits, last_bits, dCount);
    e = cudaGetLastError();
  }
  unsigned long long h = 0;
  if (e == cudaSuccess)
    e = cudaMemcpy(&h, dCount, sizeof(h), cudaMemcpyDeviceToHost);
  cudaFree(dCount);
  if (e != cudaSuccess)
    return fail(nullptr, BPSN_ERR_CUDA,
                std::string("bpsn_selftest_sqrt: ") + cudaGetErrorString(e));
  *mismatches = h;
  return BPSN_OK;
}

int32_t bpsn_dataset_open(const char* dataset_path, const char* asset_path, uint32_t num_threads,
                          bpsn_dataset** out) {
  if (!dataset_path || !asset_path || !out)
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_dataset_open: null argument");
  bpsn_dataset* ds = new bpsn_dataset();
  std::string err;
  if (!loadDataset(dataset_path, asset_path, num_threads, &ds->scenes, &err)) {
    delete ds;
    return fail(nullptr, BPSN_ERR_IO, err);
  }
  *out = ds;
  return BPSN_OK;
}

uint32_t bpsn_dataset_num_scenes(const bpsn_dataset* ds) {
  return ds ? static_cast<uint32_t>(ds->scenes.size()) : 0u;
}

int32_t bpsn_dataset_scene(const bpsn_dataset* ds, uint32_t index, const char** scene_id,
                           const char** navmesh_path, const bpsn_episode** episodes,
                           uint32_t* num_episodes) {
  if (!ds || index >= ds->scenes.size())
    return fail(nullptr, BPSN_ERR_INVALID_ARG, "bpsn_dataset_scene: bad dataset or index");
  const DatasetScene& s = ds->scenes[index];
  if (scene_id)
    *scene_id = s.sceneId.c_str();
  if (navmesh_path)
    *navmesh_path = s.navmeshPath.c_str();
  if (episodes)
    *episodes = s.episodes.data();
  if (num_episodes)
    *num_episodes = static_cast<uint32_t>(s.episodes.size());
  return BPSN_OK;
}

void bpsn_dataset_close(bpsn_dataset* ds) {
  delete ds;
}

}  // extern "C"
