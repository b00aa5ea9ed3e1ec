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

// Shared-memory layout of a staged scene: vertices | polygons | detail bases |
// detail triangles | detail vertices, each section padded to 16 bytes.
struct StagedLayout {
  size_t verts, polys, detail, dtris, dverts, total;
};
__host__ __device__ inline size_t pad16(size_t x) {
  return (x + 15) / 16 * 16;
}
__host__ __device__ inline StagedLayout stagedLayout(int nverts, int npolys, int ndtris,
                                                     int ndverts) {
  StagedLayout l;
  l.verts = 0;
  l.polys = pad16(static_cast<size_t>(nverts) * 12);
  l.detail = l.polys + static_cast<size_t>(npolys) * sizeof(NavPoly);
  l.dtris = l.detail + pad16(static_cast<size_t>(npolys) * sizeof(NavDetail));
  l.dverts = l.dtris + pad16(static_cast<size_t>(ndtris + 1) * 4);
  l.total = l.dverts + pad16(static_cast<size_t>(ndverts) * 12);
  return l;
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

// closestPointOnPolyBoundary (DetourNavMeshQuery.cpp:538-586) for the first and
// the last corridor polygon at once: lanes 0-5 take the edges of the first
// polygon, lanes 8-13 those of the last.
__device__ __forceinline__ void warpClosestOnBoundary(const NavScene& sc, int lane,
                                                      uint32_t polyA, const float* posA,
                                                      uint32_t polyB, const float* posB,
                                                      float* outA, float* outB) {
  const int grp = (lane >> 3) & 1;
  const int j = lane & 7;
  const uint32_t ip = grp ? polyB : polyA;
  const float ptx = grp ? posB[0] : posA[0];
  const float pty = grp ? posB[1] : posA[1];
  const float ptz = grp ? posB[2] : posA[2];
  const NavPoly* p = &sc.polys[ip];
  const int nv = p->vertCount;
  const bool act = lane < 16 && j < nv;
  float ed = BPSN_INF, et = 0.f;
  bool cross = false;
  float vj[3] = {0, 0, 0}, vi[3] = {0, 0, 0};
  if (act) {
    const int i = (j + 1 == nv) ? 0 : j + 1;
    const float* a = sc.verts + 3 * static_cast<size_t>(p->verts[j]);
    const float* b = sc.verts + 3 * static_cast<size_t>(p->verts[i]);
    vj[0] = a[0]; vj[1] = a[1]; vj[2] = a[2];
    vi[0] = b[0]; vi[1] = b[1]; vi[2] = b[2];
    const float pt[3] = {ptx, pty, ptz};
    cross = ((vi[2] > ptz) != (vj[2] > ptz)) &&
            (ptx < (vj[0] - vi[0]) * (ptz - vi[2]) / (vj[2] - vi[2]) + vi[0]);
    ed = distPtSegSqr2D(pt, vj, vi, et);
  }
  const uint32_t gmask = 0xffu << (grp * 8);
  const uint32_t crossBits = __ballot_sync(0xffffffffu, cross) & gmask;
  const bool inside = (__popc(crossBits) & 1) != 0;
  // first edge (lowest index) attaining the minimum squared distance
  const uint32_t edBits = __float_as_uint(ed);  // non-negative floats order like uints
  uint32_t mn = edBits;
  mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, 1));
  mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, 2));
  mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, 4));
  const uint32_t winBits = __ballot_sync(0xffffffffu, act && edBits == mn);
  float c[3] = {ptx, pty, ptz};
  if (!inside && act) {
    c[0] = vj[0] + (vi[0] - vj[0]) * et;
    c[1] = vj[1] + (vi[1] - vj[1]) * et;
    c[2] = vj[2] + (vi[2] - vj[2]) * et;
  }
  const uint32_t winA = winBits & 0xffu, winB = (winBits >> 8) & 0xffu;
  const int srcA = winA ? (__ffs(winA) - 1) : 0;
  const int srcB = winB ? (8 + __ffs(winB) - 1) : 8;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    outA[k] = __shfl_sync(0xffffffffu, c[k], srcA);
    outB[k] = __shfl_sync(0xffffffffu, c[k], srcB);
  }
}

// findStraightPath (options = 0) + polyline length over the corridor in
// w.path[0..pathSize), same decisions as funnelLength() in nav_query.cuh.
// Portal end points of every corridor edge are extracted by all lanes first
// (they only depend on the corridor), into the slab's node arrays, which the
// finished search no longer needs; lane 0 then walks the funnel.
__device__ __forceinline__ float warpFunnel(const NavScene& sc, const WarpSlab& w, int lane,
                                            const float* startPos, const float* endPos,
                                            int pathSize, uint32_t* status) {
  float closestStart[3], closestEnd[3];
  warpClosestOnBoundary(sc, lane, w.path[0], startPos, w.path[pathSize - 1], endPos, closestStart,
                        closestEnd);
  float* lx = w.px;
  float* ly = w.py;
  float* lz = w.pz;
  float* rx = w.cost;
  float* ry = w.total;
  float* rz = w.listTotal;
  bool bad = false;
  for (int i = lane; i + 1 < pathSize; i += 32) {
    const NavPoly* from = &sc.polys[w.path[i]];
    const uint32_t to = w.path[i + 1];
    const int nv = from->vertCount;
    int e = -1;
    for (int k = 0; k < nv; ++k) {
      const uint16_t ne = from->neis[k];
      if (ne && !(ne & kExtLink) && static_cast<uint32_t>(ne - 1) == to) {
        e = k;
        break;
      }
    }
    if (e < 0) {
      bad = true;
    } else {
      const float* l = sc.verts + 3 * static_cast<size_t>(from->verts[e]);
      const int e1 = (e + 1 == nv) ? 0 : e + 1;
      const float* r = sc.verts + 3 * static_cast<size_t>(from->verts[e1]);
      lx[i] = l[0];
      ly[i] = l[1];
      lz[i] = l[2];
      rx[i] = r[0];
      ry[i] = r[1];
      rz[i] = r[2];
    }
  }
  if (__any_sync(0xffffffffu, bad)) {
    *status |= kStatPartial;  // corridor polygons not adjacent: reference returns a partial path
    return BPSN_INF;
  }
  __syncwarp();

  float result = 0.f;
  uint32_t st = 0;
  if (lane == 0) {
    PathAcc acc;
    acc.count = 0;
    acc.length = 0.f;
    acc.last[0] = acc.last[1] = acc.last[2] = 0.f;
    int stat = appendVertex(acc, closestStart, false);
    bool finished = false;
    if (pathSize > 1) {
      float apex[3], pl[3], pr[3];
      vcopy(apex, closestStart);
      vcopy(pl, apex);
      vcopy(pr, apex);
      int apexIndex = 0, leftIndex = 0, rightIndex = 0;
      bool leftIsEnd = false, rightIsEnd = false;
      int guard = 0;
      for (int i = 0; i < pathSize; ++i) {
        if (++guard > 64 * kMaxPathPolys) {
          st |= kStatIterCap;
          result = BPSN_INF;
          finished = true;
          break;
        }
        float left[3], right[3];
        const bool isPortal = i + 1 < pathSize;
        if (isPortal) {
          left[0] = lx[i]; left[1] = ly[i]; left[2] = lz[i];
          right[0] = rx[i]; right[1] = ry[i]; right[2] = rz[i];
          if (i == 0) {
            float t;
            if (distPtSegSqr2D(apex, left, right, t) < (0.001f * 0.001f))
              continue;
          }
        } else {
          vcopy(left, closestEnd);
          vcopy(right, closestEnd);
        }
        if (triArea2D(apex, pr, right) <= 0.0f) {
          if (vequal(apex, pr) || triArea2D(apex, pl, right) > 0.0f) {
            vcopy(pr, right);
            rightIsEnd = !isPortal;
            rightIndex = i;
          } else {
            vcopy(apex, pl);
            apexIndex = leftIndex;
            stat = appendVertex(acc, apex, leftIsEnd);
            if (stat == 2) {
              st |= kStatFunnelOverflow;
              result = BPSN_INF;
              finished = true;
              break;
            }
            if (stat == 1) {
              result = acc.length;
              finished = true;
              break;
            }
            vcopy(pl, apex);
            vcopy(pr, apex);
            leftIndex = apexIndex;
            rightIndex = apexIndex;
            i = apexIndex;
            continue;
          }
        }
        if (triArea2D(apex, pl, left) >= 0.0f) {
          if (vequal(apex, pl) || triArea2D(apex, pr, left) < 0.0f) {
            vcopy(pl, left);
            leftIsEnd = !isPortal;
            leftIndex = i;
          } else {
            vcopy(apex, pr);
            apexIndex = rightIndex;
            stat = appendVertex(acc, apex, rightIsEnd);
            if (stat == 2) {
              st |= kStatFunnelOverflow;
              result = BPSN_INF;
              finished = true;
              break;
            }
            if (stat == 1) {
              result = acc.length;
              finished = true;
              break;
            }
            vcopy(pl, apex);
            vcopy(pr, apex);
            leftIndex = apexIndex;
            rightIndex = apexIndex;
            i = apexIndex;
            continue;
          }
        }
      }
    }
    if (!finished) {
      appendVertex(acc, closestEnd, true);
      if (acc.count >= kMaxPathPolys) {
        st |= kStatFunnelOverflow;
        result = BPSN_INF;
      } else {
        result = acc.length;
      }
    }
  }
  result = __shfl_sync(0xffffffffu, result, 0);
  st = __shfl_sync(0xffffffffu, st, 0);
  *status |= st;
  return result;
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
      // totals are non-negative floats, so their bit patterns order like
      // unsigned integers: one hardware warp reduction finds the minimum
      const uint32_t mbits = __reduce_min_sync(0xffffffffu, __float_as_uint(lmin));
      const uint32_t minMask =
          __ballot_sync(0xffffffffu, __float_as_uint(lmin) == mbits && lidx >= 0);
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
        // the staged copy keeps only links to walkable neighbours
        const uint16_t ne = bp->neis[lane];
        if (ne && !(ne & kExtLink)) {
          const uint32_t idx = static_cast<uint32_t>(ne - 1);
          if (idx != parentPoly) {
            act = true;
            nei = idx;
          }
        }
      }
      if (bp->pad & 1) {  // polygon shares more than one edge with some neighbour (rare)
        const uint32_t grp = __match_any_sync(0xffffffffu, nei);
        if (act && (__ffs(grp) - 1) != lane)
          act = false;  // same neighbour through a lower edge: that lane acts
      }

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
          const int e1 = (lane + 1 == nv) ? 0 : lane + 1;
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

  return warpFunnel(sc, w, lane, startPos, endPos, pathSize, status);
}

// One simulator step for the environments listed per scene (see sim_kernels.cuh
// for the phase split): forward move, GPS/compass, geodesic goal -> agent,
// info / reward / mask and the in-loop reset.
//   grid  = (blocksPerScene, numScenes), block = warpsPerBlock * 32 threads
//   smem  = staged tables of blockIdx.y's scene + warpsPerBlock slabs
// Warps pull list slots from a per-scene cursor until the list is drained.
__global__ void __launch_bounds__(512, 1)
k_step_warp(GroupDev g, SceneTable st, int pcap, size_t slabOffset,
            AStarScratch* __restrict__ fallbackScratch, uint32_t seedLo, uint32_t seedHi) {
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
  const StagedLayout lay = stagedLayout(sc.nverts, sc.npolys, sc.ndtris, sc.ndverts);
  {
    auto copy16 = [&](size_t dstOff, const void* srcPtr, size_t bytes) {
      const uint4* src = reinterpret_cast<const uint4*>(srcPtr);
      uint4* dst = reinterpret_cast<uint4*>(smem + dstOff);
      const int n16 = static_cast<int>(pad16(bytes) / 16);
      for (int i = threadIdx.x; i < n16; i += blockDim.x)
        dst[i] = src[i];
    };
    // every source array is followed by at least 16 bytes of padding in the
    // scene's device allocation, so the rounded-up 16-byte reads stay inside it
    copy16(lay.verts, scGlobal.verts, static_cast<size_t>(sc.nverts) * 12);
    copy16(lay.polys, scGlobal.polys, static_cast<size_t>(sc.npolys) * sizeof(NavPoly));
    copy16(lay.detail, scGlobal.detail, static_cast<size_t>(sc.npolys) * sizeof(NavDetail));
    copy16(lay.dtris, scGlobal.dtris, static_cast<size_t>(sc.ndtris + 1) * 4);
    copy16(lay.dverts, scGlobal.dverts, static_cast<size_t>(sc.ndverts) * 12);
  }
  __syncthreads();
  // tables for the forward move: an unmodified copy (wall tests look at links
  // to non-walkable neighbours through the neighbour's flags)
  sc.verts = reinterpret_cast<const float*>(smem + lay.verts);
  sc.polys = reinterpret_cast<const NavPoly*>(smem + lay.polys);
  sc.detail = reinterpret_cast<const NavDetail*>(smem + lay.detail);
  sc.dtris = smem + lay.dtris;
  sc.dverts = reinterpret_cast<const float*>(smem + lay.dverts);
  // a second polygon table for the search: links to neighbours the filter
  // rejects are dropped (the search and the funnel never cross them) and
  // polygons that reach one neighbour through two edges are flagged
  NavPoly* sp = reinterpret_cast<NavPoly*>(smem + lay.total);
  for (int i = threadIdx.x; i < sc.npolys; i += blockDim.x) {
    NavPoly q = sc.polys[i];
    const int nvp = q.vertCount;
    for (int j = 0; j < kVertsPerPoly; ++j) {
      uint16_t v = j < nvp ? q.neis[j] : 0;
      if (v && !(v & kExtLink) && (sc.polys[v - 1].flags & kFlagWalk) == 0)
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
  __syncthreads();
  NavScene scSearch = sc;
  scSearch.polys = sp;

  uint8_t* slabBase = smem + slabOffset + static_cast<size_t>(warp) * warpGeoSlabBytes(pcap);
  const WarpSlab w = carveSlab(slabBase, pcap);

  const uint32_t B = g.B;
  const uint32_t base = g.listBase[sceneIdx];
  uint32_t* cursor = g.counts + gridDim.y + sceneIdx;  // zeroed with the counts every step
  while (true) {
    uint32_t q = 0;
    if (lane == 0)
      q = atomicAdd(cursor, 1u);
    q = __shfl_sync(0xffffffffu, q, 0);
    if (q >= n)
      break;
    const uint32_t e = g.geoList[base + q];
    const uint32_t f = g.flags[e];
    const bool done = f & 1u, moved = f & 2u;
    if (moved) {
      if (lane == 0)
        forwardMove(g, sc, e);
      __syncwarp();
      __threadfence_block();
    }
    const float a[3] = {g.navPos[e], g.navPos[B + e], g.navPos[2 * B + e]};
    const float b[3] = {g.navGoal[e], g.navGoal[B + e], g.navGoal[2 * B + e]};
    const uint32_t aref = g.navRef[e];
    const uint32_t bref = g.goalRef[e];
    uint32_t status = 0;
    bool fallback = false;
    float d = warpGeodesic(scSearch, w, lane, b, bref, a, aref, &status, &fallback);
    if (lane == 0) {
      if (fallback) {
        status = 0;
        const size_t slot = static_cast<size_t>(blockIdx.y) * gridDim.x * warpsPerBlock +
                            static_cast<size_t>(blockIdx.x) * warpsPerBlock + warp;
        d = geodesic(scGlobal, fallbackScratch + slot, b, bref, a, aref, &status);
        status |= kStatTieFallback;
      }
      if (status)
        g.status[e] |= status;
      finishEnv(g, st, e, done, moved, d, seedLo, seedHi);
    }
    __syncwarp();
  }
}

}  // namespace bpsn
