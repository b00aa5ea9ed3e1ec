// Warp-cooperative geodesic distance on a scene staged in shared memory.
//
// Same function as geodesic() in nav_query.cuh (PathFinder::Impl::findPathInternal,
// PathFinder.cpp:485-526: island check, dtNavMeshQuery::findPath A*,
// findStraightPath funnel, polyline length) with the work of one query spread
// over the 32 lanes of a warp and every table it touches held on chip:
//
//   * the scene's vertex and polygon tables are copied once per CTA into shared
//     memory (plain 16-byte loads/stores; no multicast);
//   * A* nodes are direct-mapped, one slot per polygon (a single tile has one
//     search node per polygon: dtNavMeshQuery::findPath only creates extra
//     nodes per polygon for tile-border links, DetourNavMeshQuery.cpp:1040-1045),
//     structure-of-arrays in the warp's private shared-memory slab;
//   * the open list is an *unordered* array; "pop" is a warp-parallel arg-min.
//     A binary heap and an arg-min return the same node whenever the minimum
//     `total` is unique.  When two open nodes tie for the minimum the result
//     would depend on the reference heap's internal order
//     (dtNodeQueue, Detour/Source/DetourNode.cpp:172-200), so the warp abandons
//     the fast path and lane 0 reruns the query with the exact sequential
//     emulation (geodesic()) on a global-memory scratch slab.  Ties are rare
//     (totals are sums of square roots of mesh coordinates);
//   * the up-to-six neighbours of the popped polygon are evaluated by six
//     lanes at once (portal midpoint, cost, heuristic, skip test, node update,
//     open-list append).  Two edges leading to the same neighbour produce
//     bit-identical candidates, of which the second can never pass the
//     reference's `total >= node->total` test, so only the lowest edge acts;
//   * `lastBestNode` bookkeeping is dropped: it only matters for partial
//     paths, which PathFinder turns into +inf anyway (PathFinder.cpp:506).
//
// The funnel runs on lane 0 against the shared-memory scene.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "nav_query.cuh"
#include "sim_kernels.cuh"

namespace bpsn {

// Shared-memory bytes for a scene with nverts / npolys (tables only).
__host__ __device__ inline size_t warpGeoSceneBytes(int nverts, int npolys) {
  const size_t v = (static_cast<size_t>(nverts) * 12 + 15) / 16 * 16;
  return v + static_cast<size_t>(npolys) * sizeof(NavPoly);
}
// Per-warp slab for node capacity pcap (multiple of 16).
__host__ __device__ inline size_t warpGeoSlabBytes(int pcap) {
  return static_cast<size_t>(pcap) * 31 + 1024;
}

struct WarpSlab {
  float* px;
  float* py;
  float* pz;
  float* cost;
  float* total;
  float* listTotal;
  uint16_t* listPoly;
  uint16_t* parent;
  uint16_t* listPos;
  uint8_t* flags;
  uint32_t* path;  // [256]
};

__device__ __forceinline__ WarpSlab carveSlab(uint8_t* base, int pcap) {
  WarpSlab s;
  float* f = reinterpret_cast<float*>(base);
  s.px = f;
  s.py = f + pcap;
  s.pz = f + 2 * pcap;
  s.cost = f + 3 * pcap;
  s.total = f + 4 * pcap;
  s.listTotal = f + 5 * pcap;
  uint16_t* h = reinterpret_cast<uint16_t*>(f + 6 * pcap);
  s.listPoly = h;
  s.parent = h + pcap;
  s.listPos = h + 2 * pcap;
  s.flags = reinterpret_cast<uint8_t*>(h + 3 * pcap);
  s.path = reinterpret_cast<uint32_t*>(s.flags + pcap);
  return s;
}

// One query by one warp.  `sc` has verts/polys pointing into shared memory.
// Returns the distance in every lane.  *needFallback is set (uniformly) when
// the open list had a tie for the minimum.
__device__ __forceinline__ float warpGeodesic(const NavScene& sc, const WarpSlab& w, int lane,
                                              const float* startPos, uint32_t startRef,
                                              const float* endPos, uint32_t endRef,
                                              uint32_t* status, bool* needFallback) {
  *needFallback = false;
  // (i) trivial path
  {
    const float dx = startPos[0] - endPos[0];
    const float dy = startPos[1] - endPos[1];
    const float dz = startPos[2] - endPos[2];
    const float d2 = sum3Tree(dx * dx, dy * dy, dz * dz);
    const float n1 = sum3Tree(startPos[0] * startPos[0], startPos[1] * startPos[1],
                              startPos[2] * startPos[2]);
    const float n2 = sum3Tree(endPos[0] * endPos[0], endPos[1] * endPos[1], endPos[2] * endPos[2]);
    const float prec = 1e-5f;
    const float mn = n2 < n1 ? n2 : n1;
    if (d2 <= prec * prec * mn)
      return 0.0f;
  }
  // (ii) island check
  if (!validRef(sc, startRef) || !validRef(sc, endRef)) {
    *status |= kStatNoIsland;
    return BPSN_INF;
  }
  const uint32_t startIdx = startRef & sc.polyMask;
  const uint32_t endIdx = endRef & sc.polyMask;
  if (sc.island[startIdx] != sc.island[endIdx]) {
    *status |= kStatNoIsland;
    return BPSN_INF;
  }
  if (!finite3(startPos) || !finite3(endPos))
    return BPSN_INF;

  int pathSize = 0;
  if (startIdx == endIdx) {
    if (lane == 0)
      w.path[0] = startIdx;
    pathSize = 1;
    __syncwarp();
  } else {
    const int P = sc.npolys;
    // clear node flags
    {
      uint32_t* f32 = reinterpret_cast<uint32_t*>(w.flags);
      const int words = (P + 3) / 4;
      for (int i = lane; i < words; i += 32)
        f32[i] = 0u;
    }
    __syncwarp();
    if (lane == 0) {
      w.px[startIdx] = startPos[0];
      w.py[startIdx] = startPos[1];
      w.pz[startIdx] = startPos[2];
      w.cost[startIdx] = 0.f;
      const float t0 = vdist(startPos, endPos) * 0.999f;
      w.total[startIdx] = t0;
      w.parent[startIdx] = 0xffffu;
      w.flags[startIdx] = 1;
      w.listTotal[0] = t0;
      w.listPoly[0] = static_cast<uint16_t>(startIdx);
      w.listPos[startIdx] = 0;
    }
    __syncwarp();
    int size = 1;
    int nodeCount = 1;
    bool reached = false;
    bool outOfNodes = false;
    int guard = 0;

    while (size > 0) {
      if (++guard > 32 * kMaxAStarNodes) {
        *status |= kStatIterCap;
        return BPSN_INF;
      }
      // ---- pop: warp arg-min over the open list, with tie detection
      float lmin = BPSN_INF;
      int lidx = -1;
      int lcnt = 0;
      for (int i = lane; i < size; i += 32) {
        const float t = w.listTotal[i];
        if (t < lmin) {
          lmin = t;
          lidx = i;
          lcnt = 1;
        } else if (t == lmin) {
          lcnt++;
        }
      }
      float m = lmin;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
        m = fminf(m, __shfl_xor_sync(0xffffffffu, m, off));
      const uint32_t minMask = __ballot_sync(0xffffffffu, lmin == m && lidx >= 0);
      if (minMask == 0u || __popc(minMask) > 1) {
        *needFallback = true;
        return 0.f;
      }
      const int winLane = __ffs(minMask) - 1;
      const int winCnt = __shfl_sync(0xffffffffu, lcnt, winLane);
      if (winCnt > 1) {
        *needFallback = true;
        return 0.f;
      }
      const int slot = __shfl_sync(0xffffffffu, lidx, winLane);
      const uint32_t best = w.listPoly[slot];
      __syncwarp();
      if (lane == 0) {
        const int last = size - 1;
        if (slot != last) {
          const uint16_t lp = w.listPoly[last];
          w.listPoly[slot] = lp;
          w.listTotal[slot] = w.listTotal[last];
          w.listPos[lp] = static_cast<uint16_t>(slot);
        }
        w.flags[best] = 2;  // closed
      }
      size--;
      __syncwarp();

      if (best == endIdx) {
        reached = true;
        break;
      }

      // ---- expand: one lane per edge of the popped polygon
      const NavPoly* bp = &sc.polys[best];
      const int nv = bp->vertCount;
      const float bx = w.px[best], by = w.py[best], bz = w.pz[best];
      const float bcost = w.cost[best];
      const uint32_t parentPoly = w.parent[best] == 0xffffu ? 0xffffffffu : w.parent[best];

      bool act = false;
      uint32_t nei = 0xffff0000u + lane;  // unique dummy for inactive lanes
      if (lane < nv) {
        const uint16_t ne = bp->neis[lane];
        if (ne && !(ne & kExtLink)) {
          const uint32_t idx = static_cast<uint32_t>(ne - 1);
          if (idx != parentPoly && (sc.polys[idx].flags & kFlagWalk) != 0) {
            act = true;
            nei = idx;
          }
        }
      }
      const uint32_t grp = __match_any_sync(0xffffffffu, nei);
      if (act && (__ffs(grp) - 1) != lane)
        act = false;  // same neighbour through a lower edge: that lane acts

      uint8_t nf = 0;
      if (act)
        nf = w.flags[nei];
      const bool isNew = act && nf == 0;
      const uint32_t newMask = __ballot_sync(0xffffffffu, isNew);
      if (nodeCount + __popc(newMask) > kMaxAStarNodes) {
        outOfNodes = true;  // some getNode() would have failed: status gets DT_OUT_OF_NODES
        break;
      }
      nodeCount += __popc(newMask);

      bool upd = false;
      float ntotal = 0.f;
      if (act) {
        float nx, ny, nz;
        if (isNew) {
          const float* l = sc.verts + 3 * static_cast<size_t>(bp->verts[lane]);
          const int e1 = (lane + 1) % nv;
          const float* r = sc.verts + 3 * static_cast<size_t>(bp->verts[e1]);
          nx = (l[0] + r[0]) * 0.5f;
          ny = (l[1] + r[1]) * 0.5f;
          nz = (l[2] + r[2]) * 0.5f;
        } else {
          nx = w.px[nei];
          ny = w.py[nei];
          nz = w.pz[nei];
        }
        const float bpos[3] = {bx, by, bz};
        const float npos[3] = {nx, ny, nz};
        const float curCost = vdist(bpos, npos) * 1.0f;
        float cost, heuristic;
        if (nei == endIdx) {
          const float endCost = vdist(npos, endPos) * 1.0f;
          cost = bcost + curCost + endCost;
          heuristic = 0.f;
        } else {
          cost = bcost + curCost;
          heuristic = vdist(npos, endPos) * 0.999f;
        }
        ntotal = cost + heuristic;
        upd = isNew || !(ntotal >= w.total[nei]);
        if (upd) {
          if (isNew) {
            w.px[nei] = nx;
            w.py[nei] = ny;
            w.pz[nei] = nz;
          }
          w.parent[nei] = static_cast<uint16_t>(best);
          w.cost[nei] = cost;
          w.total[nei] = ntotal;
          w.flags[nei] = 1;  // open (closed bit cleared)
          if (nf & 1)
            w.listTotal[w.listPos[nei]] = ntotal;
        }
      }
      const bool app = upd && !(nf & 1);
      const uint32_t appMask = __ballot_sync(0xffffffffu, app);
      if (app) {
        const int s = size + __popc(appMask & ((1u << lane) - 1u));
        w.listTotal[s] = ntotal;
        w.listPoly[s] = static_cast<uint16_t>(nei);
        w.listPos[nei] = static_cast<uint16_t>(s);
      }
      size += __popc(appMask);
      __syncwarp();
    }

    if (outOfNodes) {
      *status |= kStatOutOfNodes;
      return BPSN_INF;
    }
    if (!reached) {
      *status |= kStatPartial;
      return BPSN_INF;
    }
    // corridor: walk parents from the end polygon, then reverse
    int length = 0;
    if (lane == 0) {
      uint32_t cur = endIdx;
      while (cur != 0xffffu && length <= kMaxAStarNodes) {
        length++;
        cur = w.parent[cur];
      }
      if (length <= kMaxPathPolys) {
        cur = endIdx;
        for (int i = length - 1; i >= 0; --i) {
          w.path[i] = cur;
          cur = w.parent[cur];
        }
      }
    }
    length = __shfl_sync(0xffffffffu, length, 0);
    __syncwarp();
    if (length > kMaxPathPolys) {
      *status |= kStatPathTooLong;
      return BPSN_INF;
    }
    pathSize = length;
  }

  float d = 0.f;
  uint32_t st = 0;
  if (lane == 0)
    d = funnelLength(sc, startPos, endPos, w.path, pathSize, &st);
  d = __shfl_sync(0xffffffffu, d, 0);
  st = __shfl_sync(0xffffffffu, st, 0);
  *status |= st;
  return d;
}

// Step geodesics (goal -> agent) for the environments listed per scene.
//   grid  = (blocksPerScene, numScenes), block = warpsPerBlock * 32 threads
//   smem  = scene tables of blockIdx.y's scene + warpsPerBlock slabs
// listBase[s] is the first slot of scene s in geoList; counts[s] its length.
__global__ void __launch_bounds__(512)
k_geo_warp(GroupDev g, SceneTable st, const uint32_t* __restrict__ listBase, int pcap,
           AStarScratch* __restrict__ fallbackScratch) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int sceneIdx = blockIdx.y;
  const uint32_t n = g.counts[sceneIdx];
  const int warpsPerBlock = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (static_cast<uint32_t>(blockIdx.x) * warpsPerBlock >= n)
    return;

  NavScene sc = st.scenes[sceneIdx];
  const NavScene scGlobal = sc;
  const size_t vbytes = (static_cast<size_t>(sc.nverts) * 12 + 15) / 16 * 16;
  {
    const uint4* src = reinterpret_cast<const uint4*>(scGlobal.verts);
    uint4* dst = reinterpret_cast<uint4*>(smem);
    const int nv4 = static_cast<int>(vbytes / 16);
    for (int i = threadIdx.x; i < nv4; i += blockDim.x)
      dst[i] = src[i];
    const uint4* psrc = reinterpret_cast<const uint4*>(scGlobal.polys);
    uint4* pdst = reinterpret_cast<uint4*>(smem + vbytes);
    const int np4 = sc.npolys * 2;
    for (int i = threadIdx.x; i < np4; i += blockDim.x)
      pdst[i] = psrc[i];
  }
  __syncthreads();
  sc.verts = reinterpret_cast<const float*>(smem);
  sc.polys = reinterpret_cast<const NavPoly*>(smem + vbytes);
  uint8_t* slabBase = smem + vbytes + static_cast<size_t>(sc.npolys) * sizeof(NavPoly) +
                      static_cast<size_t>(warp) * warpGeoSlabBytes(pcap);
  const WarpSlab w = carveSlab(slabBase, pcap);

  const uint32_t B = g.B;
  const uint32_t base = listBase[sceneIdx];
  const uint32_t stride = gridDim.x * warpsPerBlock;
  for (uint32_t q = blockIdx.x * warpsPerBlock + warp; q < n; q += stride) {
    const uint32_t e = g.geoList[base + q];
    const float a[3] = {g.navPos[e], g.navPos[B + e], g.navPos[2 * B + e]};
    const float b[3] = {g.navGoal[e], g.navGoal[B + e], g.navGoal[2 * B + e]};
    const uint32_t aref = g.navRef[e];
    const uint32_t bref = g.goalRef[e];
    uint32_t status = 0;
    bool fallback = false;
    float d = warpGeodesic(sc, w, lane, b, bref, a, aref, &status, &fallback);
    if (fallback) {
      status = 0;
      if (lane == 0) {
        const size_t slot = static_cast<size_t>(blockIdx.y) * gridDim.x * warpsPerBlock +
                            static_cast<size_t>(blockIdx.x) * warpsPerBlock + warp;
        d = geodesic(scGlobal, fallbackScratch + slot, b, bref, a, aref, &status);
        status |= kStatTieFallback;
      }
    }
    if (lane == 0) {
      if (status)
        g.status[e] |= status;
      g.tmpDist[e] = d;
    }
    __syncwarp();
  }
}

}  // namespace bpsn
