// Warp-cooperative simulator step on a scene staged in shared memory.
//
// One warp takes one listed environment through forward move, geodesic
// distance, reward and reset.  The geodesic is the same function as
// geodesic() in nav_query.cuh (PathFinder::Impl::findPathInternal,
// PathFinder.cpp:485-526: island check, dtNavMeshQuery::findPath A*,
// findStraightPath funnel, polyline length) with the work of one query spread
// over the 32 lanes and every table it touches held on chip:
//
//   * the scene's vertex (padded to 16 bytes each), polygon, detail-mesh and
//     island tables are copied once per CTA into shared memory with one bulk
//     asynchronous copy of an image laid out for it at set-up (this CTA's own
//     shared memory; no multicast).  In the staged polygon table links to
//     neighbours the query filter rejects are cleared: for the search they do
//     not exist and for moveAlongSurface they are walls either way
//     (DetourNavMeshQuery.cpp:2118-2132);
//   * the forward move (moveAlongSurface, getPolyHeight) takes one lane per edge
//     of the polygon at the head of its queue and 32 detail triangles at a time;
//   * A* nodes are direct-mapped, one slot per polygon (a single tile has one
//     search node per polygon: dtNavMeshQuery::findPath only creates extra
//     nodes per polygon for tile-border links, DetourNavMeshQuery.cpp:1040-1045)
//     in the warp's private shared-memory slab;
//   * the open list lives in registers, three (total, polygon) entries per lane;
//     "pop" is three hardware warp reductions (minimum total, how many entries
//     hold it, the holder's polygon).  A binary heap and an arg-min return the
//     same node whenever the minimum `total` is unique.  When two live entries
//     tie for the minimum the result depends on the reference heap's internal
//     order (dtNodeQueue, Detour/Source/DetourNode.cpp:172-200), so the search
//     is redone with that heap itself, kept in the slab (astarExactSlab); only
//     if the heap outgrows the slab does lane 0 rerun the query with the
//     one-thread emulation (geodesic()) on a global-memory scratch slab.
//     An open node that gets a better total (dtNodeQueue::modify) is not
//     updated in place: a second entry is added and the superseded one is
//     discarded when it is popped (its total no longer matches the node's).
//     The exact search is also taken if a lane runs out of entries (128 in all);
//   * the up-to-six neighbours of the popped polygon are evaluated by six
//     lanes at once (portal midpoint, cost, heuristic, skip test, node update).
//     Two edges leading to the same neighbour produce bit-identical
//     candidates, of which the second can never pass the reference's
//     `total >= node->total` test, so only the lowest edge acts;
//   * `lastBestNode` bookkeeping is dropped: it only matters for partial
//     paths, which PathFinder turns into +inf anyway (PathFinder.cpp:506);
//   * the funnel's portal end points are extracted by all lanes, its
//     sequential scan runs on lane 0.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "nav_query.cuh"
#include "sim_kernels.cuh"

namespace bpsn {

constexpr uint32_t kInfBits = 0x7f800000u;
constexpr int kOpenSlots = 4;  // register open-list entries per lane (128 per warp)
// nodeB.y = parent (16 bits) | kNodeOpen | visit tag (15 bits).  A node belongs to the running
// search iff its tag is the search's; anything else (zero, or the tag of an earlier search on
// the same slab) reads as "not visited yet".
constexpr uint32_t kNodeOpen = 0x10000u;  // exact search only: the node is in the heap
constexpr uint32_t kNodeTagMask = 0xfffe0000u;
constexpr uint32_t kNodeTagOne = 0x20000u;
constexpr uint32_t kNodeTagMax = 32767u;

// Shared-memory layout of a staged scene (byte offsets, each 16-byte aligned).
struct StagedLayout {
  size_t verts;   // float4 per vertex
  size_t polys;   // NavPoly per polygon (links filtered)
  size_t detail;  // NavDetail per polygon
  size_t dtris;   // 4 bytes per detail triangle (+1 padding entry)
  size_t dverts;  // 3 floats per extra detail vertex
  size_t island;  // int32 per polygon
  size_t total;
};
__host__ __device__ inline size_t pad16(size_t x) {
  return (x + 15) / 16 * 16;
}
__host__ __device__ inline StagedLayout stagedLayout(int nverts, int npolys, int ndtris,
                                                     int ndverts) {
  StagedLayout l;
  l.verts = 0;
  l.polys = static_cast<size_t>(nverts) * 16;
  l.detail = l.polys + static_cast<size_t>(npolys) * sizeof(NavPoly);
  l.dtris = l.detail + pad16(static_cast<size_t>(npolys) * sizeof(NavDetail));
  l.dverts = l.dtris + pad16(static_cast<size_t>(ndtris + 1) * 4);
  l.island = l.dverts + pad16(static_cast<size_t>(ndverts) * 12);
  l.total = l.island + pad16(static_cast<size_t>(npolys) * 4);
  return l;
}

// Per-warp slab for node capacity pcap (a multiple of 16):
//   nodeA  float4 {x, y, z, cost}                      16 B / polygon
//   nodeB  uint2  {total bits, parent | open | tag}      8 B / polygon
//   path   uint16 corridor, at most 256 polygons       512 B
// After the search the node arrays are reused for the corridor's portals.
// A slab in global memory keeps its contents from one search (and launch) to the next and
// carries, in the last 16 bytes of its stride, the number of searches it has seen: that number
// is the visit tag, so a search does not have to wipe the node array first (on a
// 16 000-polygon mesh wiping costs as much as the search).  Shared-memory slabs start every
// search from a wiped array.
__host__ __device__ inline size_t warpGeoSlabBytes(int pcap) {
  return static_cast<size_t>(pcap) * 24 + 512;
}
constexpr size_t kGlobalSlabExtra = 16;  // the search counter of a global-memory slab

struct WarpSlab {
  float4* nodeA;
  uint2* nodeB;
  uint16_t* path;
  uint32_t* searches;  // global-memory slabs only: the search counter
  int cap;             // node slots of the slab (what carveSlab was given)
};

__device__ __forceinline__ WarpSlab carveSlab(uint8_t* base, int pcap) {
  WarpSlab s;
  s.nodeA = reinterpret_cast<float4*>(base);
  s.nodeB = reinterpret_cast<uint2*>(base + static_cast<size_t>(pcap) * 16);
  s.path = reinterpret_cast<uint16_t*>(base + static_cast<size_t>(pcap) * 24);
  s.searches = nullptr;
  s.cap = pcap;
  return s;
}

// The staged tables as the search sees them.  Passed by value so that the
// pointers live in registers: a NavScene whose address escapes to a called
// function sits in local memory, and every shared-memory store could alias it.
struct StagedView {
  const NavPoly* polys;
  const float4* verts;
  const NavDetail* detail;
  const uint8_t* dtris;
  const float* dverts;
  const int32_t* island;
  int32_t npolys;
  uint32_t polyMask;
  uint32_t refBase;
};

__device__ __forceinline__ float4 ldVert4(const StagedView& sc, uint32_t iv) {
  return sc.verts[iv];
}

__device__ __forceinline__ bool validRef(const StagedView& sc, uint32_t ref) {
  if (!ref)
    return false;
  if ((ref & ~sc.polyMask) != sc.refBase)
    return false;
  return (ref & sc.polyMask) < static_cast<uint32_t>(sc.npolys);
}

// closestPointOnPolyBoundary (DetourNavMeshQuery.cpp:538-586) for the first and
// the last corridor polygon at once: lanes 0-5 take the edges of the first
// polygon, lanes 8-13 those of the last.
__device__ __forceinline__ void warpClosestOnBoundary(const StagedView sc, int lane,
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
    const float4 a = ldVert4(sc, p->verts[j]);
    const float4 b = ldVert4(sc, p->verts[i]);
    vj[0] = a.x; vj[1] = a.y; vj[2] = a.z;
    vi[0] = b.x; vi[1] = b.y; vi[2] = b.z;
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
// (they only depend on the corridor) into the slab's node arrays, which the
// finished search no longer needs; lane 0 then walks the funnel.
__device__ __forceinline__ float warpFunnel(const StagedView sc, const WarpSlab w, int lane,
                                            const float* startPos, const float* endPos,
                                            int pathSize, uint32_t* status) {
  float closestStart[3], closestEnd[3];
  warpClosestOnBoundary(sc, lane, w.path[0], startPos, w.path[pathSize - 1], endPos, closestStart,
                        closestEnd);
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
      const float4 l = ldVert4(sc, from->verts[e]);
      const int e1 = (e + 1 == nv) ? 0 : e + 1;
      const float4 r = ldVert4(sc, from->verts[e1]);
      w.nodeA[i] = make_float4(l.x, l.y, l.z, r.x);
      w.nodeB[i] = make_uint2(__float_as_uint(r.y), __float_as_uint(r.z));
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
      // The scan is a chain of dependent decisions; a branch costs about as much here
      // as a shared-memory load.  Per portal all five signed areas and the two
      // coincidence tests are evaluated up front (they are independent) and the
      // tightening of the funnel is done with selects, which leaves two rarely taken
      // branches (a corner on the left, a corner on the right).  The float operations
      // and comparisons are those of the sequential form in funnelLength().
      int guard = 0;
      const int lastPortal = pathSize - 2;  // portals are 0 .. pathSize - 2
      float4 curA = w.nodeA[0];
      uint2 curB = w.nodeB[0];
      // The first portal is skipped when the start lies on it (DetourNavMeshQuery.cpp:
      // 1858-1863).  The body only ever runs with i == 0 here, at the start: a restart
      // resumes behind its apex.
      int i = 0;
      {
        const float l0[3] = {curA.x, curA.y, curA.z};
        const float r0[3] = {curA.w, __uint_as_float(curB.x), __uint_as_float(curB.y)};
        float t;
        if (distPtSegSqr2D(apex, l0, r0, t) < (0.001f * 0.001f)) {
          i = 1;
          const int ri = (1 <= lastPortal) ? 1 : lastPortal;
          curA = w.nodeA[ri];
          curB = w.nodeB[ri];
        }
      }
      constexpr int kFunnelCap = 64 * kMaxPathPolys;
      for (; i < pathSize && guard < kFunnelCap; ++i) {
        ++guard;
        // portal i is in cur; fetch the next one now, it is needed a whole iteration later
        const int ni = (i + 1 <= lastPortal) ? i + 1 : lastPortal;
        const float4 nxtA = w.nodeA[ni];
        const uint2 nxtB = w.nodeB[ni];
        const bool isPortal = i + 1 < pathSize;
        float left[3], right[3];
        left[0] = isPortal ? curA.x : closestEnd[0];
        left[1] = isPortal ? curA.y : closestEnd[1];
        left[2] = isPortal ? curA.z : closestEnd[2];
        right[0] = isPortal ? curA.w : closestEnd[0];
        right[1] = isPortal ? __uint_as_float(curB.x) : closestEnd[1];
        right[2] = isPortal ? __uint_as_float(curB.y) : closestEnd[2];
        curA = nxtA;
        curB = nxtB;
        const float aR = triArea2D(apex, pr, right);
        const float aRL = triArea2D(apex, pl, right);
        const float aL = triArea2D(apex, pl, left);
        const float aLRold = triArea2D(apex, pr, left);
        const float aLRnew = triArea2D(apex, right, left);
        const bool eqR = vequal(apex, pr);
        const bool eqL = vequal(apex, pl);
        const bool rHit = aR <= 0.0f;
        const bool rTight = rHit && (eqR || aRL > 0.0f);
        const bool cornerLeft = rHit && !rTight;  // the right side crossed over the left
        // the left vertex is looked at only if the right one made no corner; its test uses
        // the right point as just tightened: triArea2D(apex, pr, left) with the new pr
        const float aLR = rTight ? aLRnew : aLRold;
        const bool lHit = aL >= 0.0f;
        const bool lTight = lHit && (eqL || aLR < 0.0f);
        const bool cornerRight = !cornerLeft && lHit && !lTight;
        if (!cornerLeft) {
          pr[0] = rTight ? right[0] : pr[0];
          pr[1] = rTight ? right[1] : pr[1];
          pr[2] = rTight ? right[2] : pr[2];
          rightIsEnd = rTight ? !isPortal : rightIsEnd;
          rightIndex = rTight ? i : rightIndex;
        }
        if (cornerLeft || cornerRight) {
          // a corner: the opposite side's point becomes the apex and the scan resumes there
          if (cornerLeft) {
            vcopy(apex, pl);
            apexIndex = leftIndex;
            stat = appendVertex(acc, apex, leftIsEnd);
          } else {
            vcopy(apex, pr);
            apexIndex = rightIndex;
            stat = appendVertex(acc, apex, rightIsEnd);
          }
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
          const int ri = (i + 1 <= lastPortal) ? i + 1 : lastPortal;
          curA = w.nodeA[ri];
          curB = w.nodeB[ri];
          continue;
        }
        pl[0] = lTight ? left[0] : pl[0];
        pl[1] = lTight ? left[1] : pl[1];
        pl[2] = lTight ? left[2] : pl[2];
        leftIsEnd = lTight ? !isPortal : leftIsEnd;
        leftIndex = lTight ? i : leftIndex;
      }
      if (!finished && guard >= kFunnelCap && i < pathSize) {
        st |= kStatIterCap;
        result = BPSN_INF;
        finished = true;
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

// Vertex k of a detail triangle of polygon `p`: a polygon vertex or an extra detail vertex.
__device__ __forceinline__ void stagedDetailVert(const StagedView& sc, const NavPoly* p, int nv,
                                                 const NavDetail pd, uint32_t k, float* out) {
  if (k < static_cast<uint32_t>(nv)) {
    const float4 v = ldVert4(sc, p->verts[k]);
    out[0] = v.x;
    out[1] = v.y;
    out[2] = v.z;
  } else {
    const float* v = sc.dverts + 3 * static_cast<size_t>(pd.vertBase + (k - nv));
    out[0] = v[0];
    out[1] = v[1];
    out[2] = v[2];
  }
}

// dtNavMesh::getPolyHeight (DetourNavMesh.cpp:677-726) by one warp: the point-in-
// polygon test takes one lane per edge (the parity of crossings does not depend on
// the order), the detail triangles are tested 32 at a time and the first triangle
// (lowest index) that contains the point gives the height, as in the sequential
// loop.  Returns false, *height untouched, when pos is outside the polygon in xz.
// The result is the same in every lane.
__device__ __forceinline__ bool warpPolyHeight(const StagedView sc, const NavScene& scFull,
                                               int lane, uint32_t ip, const float* pos,
                                               float* height) {
  const NavPoly* p = &sc.polys[ip];
  if ((p->areaAndType >> 6) == 1)  // off-mesh connection
    return false;
  const int nv = p->vertCount;
  bool cross = false;
  if (lane < nv) {
    const float4 vi = ldVert4(sc, p->verts[lane]);
    const float4 vj = ldVert4(sc, p->verts[(lane == 0) ? nv - 1 : lane - 1]);
    cross = ((vi.z > pos[2]) != (vj.z > pos[2])) &&
            (pos[0] < (vj.x - vi.x) * (pos[2] - vi.z) / (vj.z - vi.z) + vi.x);
  }
  if ((__popc(__ballot_sync(0xffffffffu, cross)) & 1) == 0)
    return false;
  const NavDetail pd = sc.detail[ip];
  const int ntris = p->detailTriCount;
  for (int base = 0; base < ntris; base += 32) {
    const int t = base + lane;
    bool hit = false;
    float h = 0.f;
    if (t < ntris) {
      const uchar4 tq =
          *reinterpret_cast<const uchar4*>(sc.dtris + 4 * static_cast<size_t>(pd.triBase + t));
      float v[3][3];
      stagedDetailVert(sc, p, nv, pd, tq.x, v[0]);
      stagedDetailVert(sc, p, nv, pd, tq.y, v[1]);
      stagedDetailVert(sc, p, nv, pd, tq.z, v[2]);
      hit = closestHeightPointTriangle(pos, v[0], v[1], v[2], h);
    }
    const uint32_t hits = __ballot_sync(0xffffffffu, hit);
    if (hits) {
      *height = __shfl_sync(0xffffffffu, h, __ffs(hits) - 1);
      return true;
    }
  }
  // inside the polygon but in none of its detail triangles (numerical edge case)
  float closest[3] = {0.f, 0.f, 0.f};
  if (lane == 0) {
    const NavPoly pc = loadPoly(scFull, ip);
    closestOnDetailEdges(scFull, ip, pc, pos, false, closest);
  }
  *height = __shfl_sync(0xffffffffu, closest[1], 0);
  return true;
}

// dtNavMeshQuery::moveAlongSurface as PathFinder::tryStep uses it (see
// moveAlongSurface() in nav_query.cuh for the one-thread form, whose decisions
// this reproduces): breadth-first over the polygons near the step, one lane per
// edge of the polygon at the head of the queue.
//   * end point inside the polygon: crossing parity over the edge lanes;
//   * wall edges: the sequential loop keeps the first edge with the strictly
//     smallest squared distance, i.e. the minimum with the lowest edge index;
//   * neighbour edges: node allocation, the visited bit and the FIFO push depend
//     on the order of the edges, so they are replayed edge by edge (the distance
//     test of each was already evaluated by its lane).
// The tiny node pool (64 ids) and the FIFO live in the warp's corridor array,
// which nothing else uses during the move.  Results are the same in every lane.
__device__ __forceinline__ bool warpMoveAlongSurface(const StagedView sc, const WarpSlab w,
                                                     int lane, const float* navPos,
                                                     uint32_t startRef, const float* endPos,
                                                     float* bestPos, uint32_t* endIdxOut) {
  if (!validRef(sc, startRef) || !finite3(navPos) || !finite3(endPos))
    return false;
  uint16_t* ids = w.path;           // [kMovePool]
  uint16_t* queue = w.path + kMovePool;  // [kMovePool] each node enters once
  int nnodes = 1, qhead = 0, qtail = 1;
  unsigned long long closedBits = 1ull;
  __syncwarp();
  if (lane == 0) {
    ids[0] = static_cast<uint16_t>(startRef & sc.polyMask);
    queue[0] = 0;
  }
  __syncwarp();
  vcopy(bestPos, navPos);
  float bestDist = 3.402823466e+38f;
  int bestNode = -1;
  float searchPos[3];
  vlerp(searchPos, navPos, endPos, 0.5f);
  const float rad = vdist(navPos, endPos) / 2.0f + 0.001f;
  const float searchRadSqr = rad * rad;

  while (qhead < qtail) {
    const int cur = queue[qhead++];
    const uint32_t curIdx = ids[cur];
    const NavPoly* poly = &sc.polys[curIdx];
    const int nv = poly->vertCount;
    // lane i: edge from vertex j = i - 1 (cyclic) to vertex i, neighbour code neis[j]
    const bool act = lane < nv;
    const int i = act ? lane : 0;
    const int j = (i == 0) ? nv - 1 : i - 1;
    const float4 vi4 = ldVert4(sc, poly->verts[i]);
    const float4 vj4 = ldVert4(sc, poly->verts[j]);
    const uint16_t ne = poly->neis[j];
    const float vi[3] = {vi4.x, vi4.y, vi4.z};
    const float vj[3] = {vj4.x, vj4.y, vj4.z};
    const bool cross = act && ((vi[2] > endPos[2]) != (vj[2] > endPos[2])) &&
                       (endPos[0] < (vj[0] - vi[0]) * (endPos[2] - vi[2]) / (vj[2] - vi[2]) + vi[0]);
    if (__popc(__ballot_sync(0xffffffffu, cross)) & 1) {
      bestNode = cur;
      vcopy(bestPos, endPos);
      break;
    }
    // links to polygons the filter rejects were cleared when the scene was staged
    const bool isNei = act && ne != 0 && !(ne & kExtLink);
    const bool isWall = act && !isNei;
    float tseg = 0.f;
    const float dq = distPtSegSqr2D(isWall ? endPos : searchPos, vj, vi, tseg);
    // walls
    const uint32_t key = isWall ? __float_as_uint(dq) : 0xffffffffu;
    const uint32_t kmin = __reduce_min_sync(0xffffffffu, key);
    if (kmin != 0xffffffffu && __uint_as_float(kmin) < bestDist) {
      const int src = __ffs(__ballot_sync(0xffffffffu, key == kmin)) - 1;
      float cand[3];
      vlerp(cand, vj, vi, tseg);
      bestPos[0] = __shfl_sync(0xffffffffu, cand[0], src);
      bestPos[1] = __shfl_sync(0xffffffffu, cand[1], src);
      bestPos[2] = __shfl_sync(0xffffffffu, cand[2], src);
      bestDist = __uint_as_float(kmin);
      bestNode = cur;
    }
    // neighbours, in edge order
    const uint32_t neiMask = __ballot_sync(0xffffffffu, isNei);
    const uint32_t nearMask = __ballot_sync(0xffffffffu, isNei && !(dq > searchRadSqr));
    for (uint32_t m = neiMask; m; m &= m - 1) {
      const int L = __ffs(m) - 1;
      const uint32_t nei = __shfl_sync(0xffffffffu, static_cast<uint32_t>(ne) - 1u, L);
      // getNode: find or allocate
      const uint32_t lo = __ballot_sync(0xffffffffu, lane < nnodes && ids[lane] == nei);
      const uint32_t hi = __ballot_sync(0xffffffffu, lane + 32 < nnodes && ids[lane + 32] == nei);
      int node;
      if (lo) {
        node = __ffs(lo) - 1;
      } else if (hi) {
        node = 32 + __ffs(hi) - 1;
      } else {
        if (nnodes >= kMovePool)
          continue;
        node = nnodes++;
        if (lane == 0)
          ids[node] = static_cast<uint16_t>(nei);
        __syncwarp();
      }
      if ((closedBits >> node) & 1ull)
        continue;
      if (!((nearMask >> L) & 1u))
        continue;
      if ((qtail - qhead) < kMoveStack) {
        closedBits |= 1ull << node;
        if (lane == 0)
          queue[qtail] = static_cast<uint16_t>(node);
        qtail++;
      }
    }
    __syncwarp();
  }
  if (bestNode < 0)
    return false;  // numPolys == 0
  *endIdxOut = ids[bestNode];
  return true;
}

// MoveForward of handleMovement for one environment by one warp (see forwardMove()
// in sim_kernels.cuh for the one-thread form).  The new navmesh position and
// polygon ref are returned in every lane; lane 0 writes pose and GPS/compass back.
__device__ __forceinline__ void warpForwardMove(const GroupDev& g, const StagedView sv,
                                                const NavScene& scFull, const WarpSlab w, int lane,
                                                uint32_t e, float* navOut, uint32_t* refOut) {
  const uint32_t B = g.B;
  // every lane loads the pose (same addresses: one transaction each)
  const float px = g.pos[e], py = g.pos[B + e], pz = g.pos[2 * B + e];
  const float qx = g.rot[e], qy = g.rot[B + e], qz = g.rot[2 * B + e], qw = g.rot[3 * B + e];
  float np[3] = {g.navPos[e], g.navPos[B + e], g.navPos[2 * B + e]};
  uint32_t ref = g.navRef[e];
  const float gx = g.goal[e], gy = g.goal[B + e], gz = g.goal[2 * B + e];
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
  float best[3];
  uint32_t endIdx = 0;
  const bool ok = warpMoveAlongSurface(sv, w, lane, np, ref, endPos, best, &endIdx);
  if (ok) {
    float h = best[1];
    if (finitef(best[0]) && finitef(best[2]))
      warpPolyHeight(sv, scFull, lane, endIdx, best, &h);
    np[0] = best[0];
    np[1] = h;
    np[2] = best[2];
    ref = sv.refBase | endIdx;
  }
  if (lane == 0) {
    g.navPos[e] = np[0];
    g.navPos[B + e] = np[1];
    g.navPos[2 * B + e] = np[2];
    g.navRef[e] = ref;
    g.pos[e] = np[0];
    g.pos[B + e] = np[1];
    g.pos[2 * B + e] = np[2];
    writePolar(g, e, np[0], np[1], np[2], qx, qy, qz, qw, gx, gy, gz);
  }
  navOut[0] = np[0];
  navOut[1] = np[1];
  navOut[2] = np[2];
  *refOut = ref;
}

constexpr int kSlabHeapCap = kMaxPathPolys;  // the corridor array doubles as the heap

// Start of a search on slab `w`: returns the tag that marks this search's nodes.
template <bool kGlobal>
__device__ __forceinline__ uint32_t beginSearch(const WarpSlab w, int P, int lane) {
  uint32_t count = 1u;
  bool wipe = true;
  if (kGlobal) {
    __syncwarp();
    count = *w.searches + 1u;  // same address in every lane
    wipe = count > kNodeTagMax;  // the 15-bit tag wraps: wipe once and start over
    count = wipe ? 1u : count;
    __syncwarp();
    if (lane == 0)
      *w.searches = count;
  }
  if (wipe) {
    // (a global-memory slab serves scenes of different sizes over time and keeps their marks:
    // when its numbering starts over, all of it is wiped, not just this scene's share)
    const int len = kGlobal ? w.cap : P;
    for (int i = lane; i < len; i += 32)
      w.nodeB[i] = make_uint2(0u, 0u);
  }
  __syncwarp();
  return count * kNodeTagOne;
}

// dtNodeQueue on the slab: the heap holds polygon indices (uint16) in w.path and
// compares the nodes' current totals (nodeB.x), exactly like the reference's
// heap of node pointers (Detour/Source/DetourNode.cpp:172-200).  Every lane runs
// the same code on the same addresses and writes the same values, so each lane
// reads back what it wrote itself and no synchronisation is needed in here.
__device__ __forceinline__ float slabTotal(const WarpSlab& w, uint32_t node) {
  return __uint_as_float(w.nodeB[node].x);
}
__device__ __forceinline__ void slabBubbleUp(const WarpSlab& w, int i, uint32_t node) {
  const float tn = slabTotal(w, node);
  int parent = (i - 1) / 2;
  while (i > 0) {
    const uint32_t pn = w.path[parent];
    if (!(slabTotal(w, pn) > tn))
      break;
    w.path[i] = static_cast<uint16_t>(pn);
    i = parent;
    parent = (i - 1) / 2;
  }
  w.path[i] = static_cast<uint16_t>(node);
}
__device__ __forceinline__ void slabTrickleDown(const WarpSlab& w, int size, int i,
                                                uint32_t node) {
  int child = i * 2 + 1;
  while (child < size) {
    if ((child + 1) < size && slabTotal(w, w.path[child]) > slabTotal(w, w.path[child + 1]))
      child++;
    w.path[i] = w.path[child];
    i = child;
    child = i * 2 + 1;
  }
  slabBubbleUp(w, i, node);
}

enum AStarOutcome : int {
  kAStarReached = 0,
  kAStarExhausted = 1,  // open list ran empty before the end polygon was popped
  kAStarIterCap = 2,
  kAStarHeapFull = 3,   // exact slab search only: more than kSlabHeapCap open nodes
};

// dtNavMeshQuery::findPath (DetourNavMeshQuery.cpp:945-1137) with the reference's
// own open list, a binary heap, kept in the slab: taken when the register open
// list cannot decide the pop order (two live entries tie for the minimum) or is
// full.  The neighbours of the popped polygon are still evaluated by one lane
// each; their node updates and heap operations then happen one edge after the
// other in edge order, as in the reference's loop, because a heap operation
// compares against the totals the earlier edges have already written.
__device__ __noinline__ int astarExactSlab(const StagedView sc, const WarpSlab w, int lane,
                                           const float* startPosIn, const float* endPosIn,
                                           uint32_t startIdx, uint32_t endIdx, uint32_t tag,
                                           int* nodesOut) {
  const float startPos[3] = {startPosIn[0], startPosIn[1], startPosIn[2]};
  const float endPos[3] = {endPosIn[0], endPosIn[1], endPosIn[2]};
  if (lane == 0) {
    const float tot = vdist(startPos, endPos) * 0.999f;
    w.nodeA[startIdx] = make_float4(startPos[0], startPos[1], startPos[2], 0.f);
    w.nodeB[startIdx] = make_uint2(__float_as_uint(tot), 0xffffu | tag | kNodeOpen);
  }
  __syncwarp();
  int heapSize = 1;
  slabBubbleUp(w, 0, startIdx);
  int nodes = 1;
  int outcome = kAStarExhausted;
  int guard = 0;
  while (heapSize > 0) {
    if (++guard > 32 * kMaxAStarNodes) {
      outcome = kAStarIterCap;
      break;
    }
    // pop
    const uint32_t best = w.path[0];
    heapSize--;
    slabTrickleDown(w, heapSize, 0, w.path[heapSize]);
    if (best == endIdx) {
      outcome = kAStarReached;
      break;
    }
    const NavPoly* bp = &sc.polys[best];
    const int nv = bp->vertCount;
    const float4 bA = w.nodeA[best];
    const uint2 bB = w.nodeB[best];
    __syncwarp();
    if (lane == 0)
      w.nodeB[best].y = bB.y & ~kNodeOpen;
    const uint32_t bpar = bB.y & 0xffffu;
    // evaluate: lane j takes edge j
    const int li = lane < kVertsPerPoly ? lane : kVertsPerPoly - 1;
    const uint16_t ne = bp->neis[li];
    bool act = lane < nv && ne != 0 && !(ne & kExtLink) && static_cast<uint32_t>(ne - 1) != bpar;
    uint32_t nei = act ? static_cast<uint32_t>(ne - 1) : best;
    {
      // two edges to the same neighbour: the second candidate is bit-identical to the
      // first and fails the reference's `total >= node->total` test; the lowest edge acts
      const uint32_t grp = __match_any_sync(0xffffffffu, act ? nei : 0xffff0000u + lane);
      if (act && (__ffs(grp) - 1) != lane) {
        act = false;
        nei = best;
      }
    }
    const float4 nA = w.nodeA[nei];
    const uint2 nB = w.nodeB[nei];
    const float4 V0 = ldVert4(sc, bp->verts[li]);
    const float4 V1 = ldVert4(sc, bp->verts[(li + 1 == nv) ? 0 : li + 1]);
    const bool isNew = act && (nB.y & kNodeTagMask) != tag;
    const float nx = isNew ? (V0.x + V1.x) * 0.5f : nA.x;
    const float ny = isNew ? (V0.y + V1.y) * 0.5f : nA.y;
    const float nz = isNew ? (V0.z + V1.z) * 0.5f : nA.z;
    const float bpos[3] = {bA.x, bA.y, bA.z};
    const float npos[3] = {nx, ny, nz};
    const float curCost = act ? vdist(bpos, npos) * 1.0f : 0.f;
    const float toEnd = act ? vdist(npos, endPos) : 0.f;
    const bool atEnd = nei == endIdx;
    const float base = bA.w + curCost;
    const float cost = atEnd ? base + toEnd * 1.0f : base;
    const float heuristic = atEnd ? 0.f : toEnd * 0.999f;
    const float ntotal = cost + heuristic;
    const bool upd = act && (isNew || !(ntotal >= __uint_as_float(nB.x)));
    const bool wasOpen = !isNew && (nB.y & kNodeOpen) != 0;
    nodes += __popc(__ballot_sync(0xffffffffu, isNew));
    // commit edge by edge
    const uint32_t updMask = __ballot_sync(0xffffffffu, upd);
    const uint32_t openMask = __ballot_sync(0xffffffffu, upd && wasOpen);
    bool full = false;
    for (uint32_t m = updMask; m; m &= m - 1) {
      const int j = __ffs(m) - 1;
      const uint32_t node = __shfl_sync(0xffffffffu, nei, j);
      if (lane == j) {
        w.nodeA[nei] = make_float4(nx, ny, nz, cost);
        w.nodeB[nei] = make_uint2(__float_as_uint(ntotal), best | tag | kNodeOpen);
      }
      __syncwarp();
      if ((openMask >> j) & 1u) {
        // dtNodeQueue::modify: find the node, bubble it up from where it is
        int at = -1;
        for (int k0 = 0; k0 < heapSize && at < 0; k0 += 32) {
          const int k = k0 + lane;
          const uint32_t hit = __ballot_sync(0xffffffffu, k < heapSize && w.path[k] == node);
          if (hit)
            at = k0 + __ffs(hit) - 1;
        }
        if (at >= 0)
          slabBubbleUp(w, at, node);
      } else {
        if (heapSize >= kSlabHeapCap) {
          full = true;
          break;
        }
        heapSize++;
        slabBubbleUp(w, heapSize - 1, node);
      }
    }
    if (full) {
      outcome = kAStarHeapFull;
      break;
    }
    __syncwarp();
  }
  __syncwarp();
  *nodesOut = nodes;
  return outcome;
}

// The search part of one query by one warp: everything of findPathInternal
// (PathFinder.cpp:485-526) up to the corridor.  `sc` points at the staged tables (shared or
// global memory).  Returns the corridor's length, the corridor itself being in w.path[0 ..
// length); or 0 when the distance is already known without a funnel -- *early (0 for coincident
// end points, +inf for every failure) -- or when the query has to be redone by the one-thread
// emulation (*needFallback set, uniformly: the register open list could not decide the pop
// order and the slab heap outgrew its array).  The same in every lane.
template <bool kGlobal>
__device__ __forceinline__ int warpSearch(const StagedView sc, const WarpSlab w, int lane,
                                          const float* startPosIn, uint32_t startRef,
                                          const float* endPosIn, uint32_t endRef,
                                          uint32_t* status, uint32_t* needFallback,
                                          bool forceExact, float* early) {

  // private copies: the caller's arrays are also handed to a non-inlined
  // function and therefore live in local memory
  const float startPos[3] = {startPosIn[0], startPosIn[1], startPosIn[2]};
  const float endPos[3] = {endPosIn[0], endPosIn[1], endPosIn[2]};
  *needFallback = 0u;
  // (i) trivial path: Eigen isApprox with precision 1e-5
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
      { *early = 0.0f; return 0; }
  }
  // (ii) island check
  if (!validRef(sc, startRef) || !validRef(sc, endRef)) {
    *status |= kStatNoIsland;
    { *early = BPSN_INF; return 0; }
  }
  const uint32_t startIdx = startRef & sc.polyMask;
  const uint32_t endIdx = endRef & sc.polyMask;
  if (sc.island[startIdx] != sc.island[endIdx]) {
    *status |= kStatNoIsland;
    { *early = BPSN_INF; return 0; }
  }
  if (!finite3(startPos) || !finite3(endPos))
    { *early = BPSN_INF; return 0; }

  int pathSize = 0;
  if (startIdx == endIdx) {
    if (lane == 0)
      w.path[0] = static_cast<uint16_t>(startIdx);
    pathSize = 1;
    __syncwarp();
  } else {
    const uint32_t tag = beginSearch<kGlobal>(w, sc.npolys, lane);
    // open list: kOpenSlots register entries (total, polygon) per lane, kInfBits = empty.
    // All loops over the slots are unrolled, so the arrays live in registers.
    uint32_t t[kOpenSlots], p[kOpenSlots];
#pragma unroll
    for (int k = 0; k < kOpenSlots; ++k) {
      t[k] = kInfBits;
      p[k] = 0;
    }
    int newNodes = 0;  // nodes this lane created (summed over the warp at the end)
    if (lane == 0) {
      const float tot = vdist(startPos, endPos) * 0.999f;
      w.nodeA[startIdx] = make_float4(startPos[0], startPos[1], startPos[2], 0.f);
      w.nodeB[startIdx] = make_uint2(__float_as_uint(tot), 0xffffu | tag);
      t[0] = __float_as_uint(tot);
      p[0] = startIdx;
      newNodes = 1;
    }
    __syncwarp();
    bool reached = false;
    bool overflow = false;  // this lane had to drop an entry, or met a distance outside the bare
                            // square root's range: the query is redone exactly
    // why the search has to be (re)done with the reference's heap
    uint32_t exactWhy = forceExact ? kStatTieFallback : 0u;
    int guard = 0;
    // Edge j of the popped polygon is evaluated by lane (j + rot) & 31 and rot moves on
    // after every pop, so that over a search every lane gets to evaluate neighbours: a
    // new open entry is kept in the *evaluating* lane's own registers, without any
    // cross-lane traffic, and the entries spread over the warp.
    int rot = 0;
    // a two-way tie that is being expanded in place: expansions still to check, the tied
    // total, the polygon that goes second
    int tiePending = 0;
    uint32_t tieTotal = 0u, tieOther = 0u;

    // The loop body has one conditional branch on its common path besides the two
    // uncommon-case tests after the loads (a branch costs about as much as a
    // shared-memory load here): the iteration cap, the state of the open list, the end
    // test and the request to rebalance all leave through the same test.
    if (!forceExact) while (true) {
      ++guard;
      // ---- pop: totals are non-negative floats, so their bit patterns order
      // like unsigned integers and one warp reduction finds the minimum.  A lane
      // that overflowed reports 0 so that the search stops at once.
      uint32_t lm = t[0];
#pragma unroll
      for (int k = 1; k < kOpenSlots; ++k)
        lm = min(lm, t[k]);
      const uint32_t gm = __reduce_min_sync(0xffffffffu, overflow ? 0u : lm);
      bool m[kOpenSlots];
      uint32_t mc = 0, cand = 0xffffffffu;
      bool laneFull = true;
#pragma unroll
      for (int k = kOpenSlots - 1; k >= 0; --k) {
        m[k] = t[k] == gm;
        mc += m[k] ? 1u : 0u;
        cand = m[k] ? p[k] : cand;
        laneFull = laneFull && t[k] != kInfBits;
      }
      // Two more reductions, side by side, instead of vote + find-first-set + shuffle
      // (each of which costs about as much as a reduction): how many entries hold the
      // minimum, and the polygon of the one that does when it is alone.
      // (a lane whose entries are all taken adds 65536: it asks for a rebalance)
      const uint32_t hsum = __reduce_add_sync(0xffffffffu, mc | (laneFull ? 0x10000u : 0u));
      uint32_t best = __reduce_min_sync(0xffffffffu, cand);
      // one branch for everything that is not "a unique minimum that is not the end"
      if ((hsum != 1u) | (best == endIdx) | (guard > 64 * kMaxAStarNodes)) {
        if (guard > 64 * kMaxAStarNodes) {
          *status |= kStatIterCap;
          { *early = BPSN_INF; return 0; }
        }
        if (gm == kInfBits)
          break;  // open list empty: the end polygon was not reached
        const uint32_t holders = hsum & 0xffffu;
        if (holders != 1u) {
          if (__any_sync(0xffffffffu, overflow)) {
            exactWhy = kStatOpenOverflow;
            break;
          }
          // Several entries share the minimum.  Superseded entries do not count: only
          // those whose total is still their node's are in the reference's heap.
          int lc = 0;
          uint32_t livePoly = 0;
#pragma unroll
          for (int k = kOpenSlots - 1; k >= 0; --k) {
            const bool live = m[k] && w.nodeB[p[k]].x == gm;
            lc += live ? 1 : 0;
            livePoly = live ? p[k] : livePoly;
          }
          const uint32_t liveHolders = __ballot_sync(0xffffffffu, lc != 0);
          const bool liveMulti = __any_sync(0xffffffffu, lc > 1);
          if (__popc(liveHolders) > 1 || liveMulti) {
            // A real tie: the heap's order decides which is popped first.  When exactly two
            // polygons tie, neither is the end polygon, they are not adjacent and share no
            // neighbour, and (checked below, after each of the two expansions) neither
            // expansion writes a total at or below the tied one, then both are popped before
            // anything else in either order and the two orders leave the same nodes and the
            // same open set behind: they are expanded one after the other here.  Anything
            // else goes to the exact redo.
            bool resolved = false;
            if (__popc(liveHolders) == 2 && !liveMulti && tiePending == 0) {
              const uint32_t p0 = __shfl_sync(0xffffffffu, livePoly, __ffs(liveHolders) - 1);
              const uint32_t p1 = __shfl_sync(0xffffffffu, livePoly, 31 - __clz(liveHolders));
              const uint32_t first = min(p0, p1), second = max(p0, p1);
              if (first != endIdx && second != endIdx) {
                // lanes 0..5: the neighbours of the first, lanes 6..11: of the second
                uint32_t key = 0xffffffffu;
                const bool sideB = lane >= kVertsPerPoly;
                if (lane < 2 * kVertsPerPoly) {
                  const NavPoly* q = &sc.polys[sideB ? second : first];
                  const int jj = sideB ? lane - kVertsPerPoly : lane;
                  const uint16_t qn = q->neis[jj];
                  if (jj < q->vertCount && qn != 0 && !(qn & kExtLink))
                    key = static_cast<uint32_t>(qn - 1);
                }
                bool touch = false;
#pragma unroll
                for (int jj = 0; jj < kVertsPerPoly; ++jj) {
                  const uint32_t other = __shfl_sync(0xffffffffu, key, jj);
                  touch = touch || (sideB && key == other);
                }
                touch = key != 0xffffffffu && (touch || key == (sideB ? first : second));
                if (!__any_sync(0xffffffffu, touch)) {
                  resolved = true;
                  *status |= kStatTieInPlace;
                  best = first;
                  tieOther = second;
                  tieTotal = gm;
                  tiePending = 2;
                  // the second polygon keeps its entry: it is the minimum of the next pop
#pragma unroll
                  for (int k = 0; k < kOpenSlots; ++k)
                    m[k] = m[k] && p[k] != second;
                }
              }
            }
            if (!resolved) {
              exactWhy = kStatTieFallback;
              break;
            }
          } else {
            if (liveHolders == 0u) {  // only superseded entries surfaced: drop them
#pragma unroll
              for (int k = 0; k < kOpenSlots; ++k)
                t[k] = m[k] ? kInfBits : t[k];
              continue;
            }
            best = __shfl_sync(0xffffffffu, livePoly, __ffs(liveHolders) - 1);
          }
        }
        if (best == endIdx) {
          reached = true;
          break;
        }
        if (hsum >> 16) {
          // A lane whose entries are all taken hands its last one to a lane with room
          // (preferably one with two free pairs), so that it can accept a neighbour below.
          bool f[kOpenSlots];
          int freeCnt = 0;
#pragma unroll
          for (int k = 0; k < kOpenSlots; ++k) {
            t[k] = m[k] ? kInfBits : t[k];  // (the popped entry first)
            m[k] = false;                   // done: the pairs may be refilled just below
            // superseded entries (their total is no longer their node's) only take up room
            const bool stale = t[k] != kInfBits && w.nodeB[p[k]].x != t[k];
            t[k] = stale ? kInfBits : t[k];
            f[k] = t[k] == kInfBits;
            freeCnt += f[k] ? 1 : 0;
          }
          uint32_t fb = __ballot_sync(0xffffffffu, freeCnt == 0);
          uint32_t rb = __ballot_sync(0xffffffffu, freeCnt >= 2);
          const uint32_t rb1 = __ballot_sync(0xffffffffu, freeCnt >= 1);
          if (!rb)
            rb = rb1;
          while (fb && rb) {
            const int src = __ffs(fb) - 1, dst = __ffs(rb) - 1;
            fb &= fb - 1;
            rb &= rb - 1;
            const uint32_t mt = __shfl_sync(0xffffffffu, t[kOpenSlots - 1], src);
            const uint32_t mp = __shfl_sync(0xffffffffu, p[kOpenSlots - 1], src);
            bool placed = lane != dst;  // into the receiver's first free pair
#pragma unroll
            for (int k = 0; k < kOpenSlots; ++k) {
              const bool here = !placed && f[k];
              t[k] = here ? mt : t[k];
              p[k] = here ? mp : p[k];
              placed = placed || here;
            }
            if (lane == src)
              t[kOpenSlots - 1] = kInfBits;
          }
        }
      }
      // the popped entry and, after a resolved tie, the superseded ones beside it
#pragma unroll
      for (int k = 0; k < kOpenSlots; ++k)
        t[k] = m[k] ? kInfBits : t[k];

      // ---- expand: one lane per edge of the popped polygon.  All loads of a
      // round are issued before any of them is used.
      const NavPoly* bp = &sc.polys[best];
      const int ej = (lane - rot) & 31;  // this lane's edge index (>= nv: none)
      const int li = ej < kVertsPerPoly ? ej : kVertsPerPoly - 1;
      const int nv = bp->vertCount;
      const uint32_t dupFlag = bp->pad;
      const uint16_t ne = bp->neis[li];
      const uint16_t va = bp->verts[li];
      // verts[li + 1] stays inside the record (neis follows verts)
      const uint16_t vbNext = (&bp->verts[0])[li + 1];
      const uint16_t vbFirst = bp->verts[0];
      const float4 bA = w.nodeA[best];
      const uint2 bB = w.nodeB[best];

      const uint16_t vb = (li + 1 == nv) ? vbFirst : vbNext;
      const bool hasEdge = ej < nv && ne != 0 && !(ne & kExtLink);
      const uint32_t nei = hasEdge ? static_cast<uint32_t>(ne - 1) : best;
      // The neighbour's node and the edge's end points are requested as soon as the polygon
      // record is there: they do not wait for the popped node's own record (in global
      // memory that is a second trip to L2, now overlapped with this one).
      const float4 nA = w.nodeA[nei];
      const uint2 nB = w.nodeB[nei];
      const float4 V0 = ldVert4(sc, va);
      const float4 V1 = ldVert4(sc, vb);
      const uint32_t bpar = bB.y & 0xffffu;
      bool act = hasEdge && nei != bpar;
      if ((bB.x != gm) | (dupFlag & 1)) {  // one branch for the two uncommon cases
        // Entries are never updated in place: a better total for an open node adds a
        // second entry and the superseded one is dropped here, when it surfaces.  All
        // entries of a node have different totals (each is strictly below the one
        // before), so the live one is the one that matches the node's current total.
        if (bB.x != gm) {
          rot = (rot + 7) & 31;
          continue;
        }
        // the polygon shares more than one edge with some neighbour
        const uint32_t grp = __match_any_sync(0xffffffffu, hasEdge ? nei : 0xffff0000u + lane);
        // bit k of the rotated mask = edge k; the lowest edge of the group acts
        const uint32_t byEdge = __funnelshift_r(grp, grp, rot);
        act = act && (__ffs(byEdge) - 1) == ej;
      }
      const bool isNew = act && (nB.y & kNodeTagMask) != tag;
      newNodes += isNew ? 1 : 0;
      const float nx = isNew ? (V0.x + V1.x) * 0.5f : nA.x;
      const float ny = isNew ? (V0.y + V1.y) * 0.5f : nA.y;
      const float nz = isNew ? (V0.z + V1.z) * 0.5f : nA.z;
      const float bpos[3] = {bA.x, bA.y, bA.z};
      const float npos[3] = {nx, ny, nz};
      // The two distances use the bare square-root sequence (exact for operands from
      // 2^-100 up).  An operand outside that range in a lane that has a neighbour - a zero
      // distance, in practice - marks the search for the exact redo, like a full open list;
      // nothing of this search is kept then.  Lanes without a neighbour compute garbage.
      const float c2 = vdistSqr(bpos, npos);
      const float e2 = vdistSqr(npos, endPos);
      const float curCost = sqrtCore(c2);  // vdist(bpos, npos) * 1.0f
      const float toEnd = sqrtCore(e2);    // vdist(npos, endPos)
      overflow = overflow || (act && !(sqrtCoreValid(c2) & sqrtCoreValid(e2)));
      const bool atEnd = nei == endIdx;
      // end polygon: cost = g + step + distance to the end point, h = 0
      const float base = bA.w + curCost;
      const float cost = atEnd ? base + toEnd * 1.0f : base;
      const float heuristic = atEnd ? 0.f : toEnd * 0.999f;
      const float ntotal = cost + heuristic;
      const uint32_t ntBits = __float_as_uint(ntotal);
      // open or closed alike: skipped unless strictly better (DetourNavMeshQuery.cpp:1075-1080)
      const bool upd = act && (isNew || !(ntotal >= __uint_as_float(nB.x)));
      if (tiePending) {
        // one of the two expansions of a resolved tie (see the pop): it has to be the expected
        // polygon and must not write a total that the other order would have popped first
        if ((tiePending == 1 && best != tieOther) ||
            __any_sync(0xffffffffu, upd && ntBits <= tieTotal)) {
          exactWhy = kStatTieFallback;
          break;
        }
        --tiePending;
      }

      // ---- the new entry goes into this lane's first free register pair
      {
        bool placed = !upd;
#pragma unroll
        for (int k = 0; k < kOpenSlots; ++k) {
          const bool here = !placed && t[k] == kInfBits;
          t[k] = here ? ntBits : t[k];
          p[k] = here ? nei : p[k];
          placed = placed || here;
        }
        overflow = overflow || !placed;
      }
      if (upd) {
        w.nodeA[nei] = make_float4(nx, ny, nz, cost);
        w.nodeB[nei] = make_uint2(ntBits, best | tag);
      }
      rot = (rot + 7) & 31;
      __syncwarp();
    }

    if (!exactWhy && __any_sync(0xffffffffu, overflow))
      exactWhy = kStatOpenOverflow;
    int nodeTotal = __reduce_add_sync(0xffffffffu, newNodes);
    if (exactWhy) {
      const uint32_t exactTag = beginSearch<kGlobal>(w, sc.npolys, lane);
      const int outcome = astarExactSlab(sc, w, lane, startPos, endPos, startIdx, endIdx, exactTag,
                                         &nodeTotal);
      if (outcome == kAStarHeapFull) {
        *needFallback = exactWhy;  // hand the query to the global-memory emulation
        { *early = 0.f; return 0; }
      }
      if (outcome == kAStarIterCap) {
        *status |= kStatIterCap;
        { *early = BPSN_INF; return 0; }
      }
      *status |= exactWhy;
      reached = outcome == kAStarReached;
    }
    // dtNodePool hands out at most kMaxAStarNodes nodes; a search that asks for more
    // ends with DT_OUT_OF_NODES in its status, which PathFinder turns into +inf
    // whatever path was found (PathFinder.cpp:506).
    const bool outOfNodes = nodeTotal > kMaxAStarNodes;
    if (outOfNodes) {
      *status |= kStatOutOfNodes;
      { *early = BPSN_INF; return 0; }
    }
    if (!reached) {
      *status |= kStatPartial;
      { *early = BPSN_INF; return 0; }
    }
    // corridor: walk parents from the end polygon, then reverse
    int length = 0;
    if (lane == 0) {
      uint32_t cur = endIdx;
      while (cur != 0xffffu && length <= kMaxAStarNodes) {
        length++;
        cur = w.nodeB[cur].y & 0xffffu;
      }
      if (length <= kMaxPathPolys) {
        cur = endIdx;
        for (int i = length - 1; i >= 0; --i) {
          w.path[i] = static_cast<uint16_t>(cur);
          cur = w.nodeB[cur].y & 0xffffu;
        }
      }
    }
    length = __shfl_sync(0xffffffffu, length, 0);
    __syncwarp();
    if (length > kMaxPathPolys) {
      *status |= kStatPathTooLong;
      { *early = BPSN_INF; return 0; }
    }
    pathSize = length;
  }

  return pathSize;
}

// One query by one warp: search, then the funnel over the corridor.  Returns the distance in
// every lane; *needFallback as in warpSearch.
template <bool kGlobal>
__device__ __forceinline__ float warpGeodesic(const StagedView sc, const WarpSlab w, int lane,
                                              const float* startPos, uint32_t startRef,
                                              const float* endPos, uint32_t endRef,
                                              uint32_t* status, uint32_t* needFallback,
                                              bool forceExact) {
  float early = 0.f;
  const int pathSize = warpSearch<kGlobal>(sc, w, lane, startPos, startRef, endPos, endRef, status,
                                           needFallback, forceExact, &early);
  if (pathSize == 0)
    return early;
  const float dres = warpFunnel(sc, w, lane, startPos, endPos, pathSize, status);
  if (kGlobal) {
    // the portals sit in the first node slots; what they left in the tag field must not
    // pass for a visit mark of a later search
    __syncwarp();
    for (int i = lane; i + 1 < pathSize; i += 32)
      w.nodeB[i].y = 0u;
  }
  return dres;
}

// Where a warp gets its work-list entries from.  operator() returns false (in every lane)
// when there is nothing left for this warp.
//
// ListSource: a work list in global memory shared by all CTAs of a slot.  Every warp starts on
// the list slot of its own number; the slots beyond the number of warps that share the list
// are handed out through a cursor that starts at zero.
struct ListSource {
  const uint32_t* list;
  uint32_t* cursor;
  uint32_t q;          // first slot of this warp
  uint32_t gridWarps;  // warps that share the list
  uint32_t n;
  bool first;
  __device__ __forceinline__ bool operator()(int lane, uint32_t* entry) {
    if (!first) {
      if (lane == 0)
        q = gridWarps + atomicAdd(cursor, 1u);
      q = __shfl_sync(0xffffffffu, q, 0);
    }
    first = false;
    if (q >= n)
      return false;
    *entry = list[q];
    return true;
  }
};

// FusedSource: the CTA made its own list (see kFused).  Its first entries, one per warp, stay
// in shared memory; the ones beyond sit in the CTA's segment of a global array, with a count,
// a cursor and the number of the step they belong to, and are claimed through the cursor by
// whichever warp has nothing else to do -- one of the CTA's own or one of a CTA that serves the
// same slot (the next few in the slot's ring are looked at).  Nobody waits for anybody: a
// segment that is not marked with this step's number yet is passed over, and its owner's
// warps drain it themselves at the latest.
constexpr uint32_t kFusedMaxShare = 64;  // environments per CTA at most
constexpr uint32_t kStealReach = 8;      // neighbours in the slot's ring a warp looks at
struct FusedSource {
  const uint32_t* local;  // shared memory
  uint32_t nLocal;
  uint32_t* ovList;       // [CTA][kFusedMaxShare]
  uint32_t* ovMeta;       // [CTA][4]: count, cursor, step number, -
  uint32_t ctaBase, rank, slotCtas, stepId;
  int warp;
  uint32_t stage;         // 0: own first entry, 1: own segment, 2...: neighbours
  __device__ __forceinline__ bool operator()(int lane, uint32_t* entry) {
    if (stage == 0) {
      stage = 1;
      if (static_cast<uint32_t>(warp) < nLocal) {
        *entry = local[warp];
        return true;
      }
    }
    // One look at the own segment and the next few of the slot's ring, a lane each (one trip
    // to memory); the first that shows unclaimed entries of this step is tried.  A claim that
    // loses the race for the last entry sends the warp round once more.
    for (int tries = 0; tries < 4; ++tries) {
      const uint32_t k = static_cast<uint32_t>(lane);
      const bool looks = k <= kStealReach && k < slotCtas;
      const uint32_t cta = ctaBase + (rank + (looks ? k : 0u)) % slotCtas;
      uint4 m = make_uint4(0u, 0u, 0u, 0u);
      if (looks)
        m = __ldcg(reinterpret_cast<const uint4*>(ovMeta) + cta);
      const uint32_t has = __ballot_sync(0xffffffffu, looks && m.z == stepId && m.y < m.x);
      if (!has)
        return false;
      const int src = __ffs(has) - 1;
      uint32_t got = 0xffffffffu;
      if (lane == src) {
        volatile uint32_t* meta = ovMeta + 4u * cta;
        __threadfence();  // the step number was seen: the count and the entries are out
        const uint32_t count = meta[0];
        const uint32_t q = atomicAdd(ovMeta + 4u * cta + 1u, 1u);
        if (q < count)
          got = *(volatile uint32_t*)(ovList + static_cast<size_t>(cta) * kFusedMaxShare + q);
      }
      got = __shfl_sync(0xffffffffu, got, src);
      if (got != 0xffffffffu) {
        *entry = got;
        return true;
      }
    }
    return false;
  }
};

// The part of k_step_warp after the scene is in place: the warp's loop over work-list
// entries.  Two instances: tables and slabs in shared memory (the pointers are then known to
// be shared-memory addresses and the accesses compile to shared-memory instructions) or in
// global memory.
// kBatched (batches that give every warp many entries): the funnel and everything after it --
// which are one thread's work -- are not done entry by entry on lane 0 with 31 lanes waiting,
// but for up to 32 entries at a time, one per lane: the warp searches 32 entries one after the
// other, keeping each corridor in a staging row, then every lane pulls the string through its
// own corridor (funnelLength(), the one-thread form) and finishes its own environment.
template <bool kGlobal, bool kBatched, class Source>
__device__ __forceinline__ void stepWarpQueries(const GroupDev& g, const SceneTable& st,
                                                const WarpPlan pl, Source next,
                                                const NavScene& scGlobal,
                                                uint8_t* globalSlabs, size_t globalSlabStride,
                                                AStarScratch* fallbackScratch, uint32_t seedLo,
                                                uint32_t seedHi
) {
  extern __shared__ __align__(16) uint8_t smem[];
  // Slabs in global memory are laid out for the largest scene of the group whatever scene
  // is being worked on: a slab outlives searches, launches and (when scenes rotate) scenes,
  // and its visit marks only mean something if they always sit in the same place.
  const int pcap = static_cast<int>(kGlobal ? g.globalPcap : pl.pcap);
  const int warpsPerBlock = static_cast<int>(pl.warps);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  NavScene sc = scGlobal;
  const StagedLayout lay = stagedLayout(sc.nverts, sc.npolys, sc.ndtris, sc.ndverts);
  const uint8_t* tables = kGlobal ? scGlobal.staged : smem;
  sc.verts = reinterpret_cast<const float*>(tables + lay.verts);
  sc.vstride = 4;
  sc.polys = reinterpret_cast<const NavPoly*>(tables + lay.polys);
  sc.detail = reinterpret_cast<const NavDetail*>(tables + lay.detail);
  sc.dtris = tables + lay.dtris;
  sc.dverts = reinterpret_cast<const float*>(tables + lay.dverts);
  sc.island = reinterpret_cast<const int32_t*>(tables + lay.island);

  StagedView sv;
  sv.polys = sc.polys;
  sv.verts = reinterpret_cast<const float4*>(sc.verts);
  sv.detail = sc.detail;
  sv.dtris = sc.dtris;
  sv.dverts = sc.dverts;
  sv.island = sc.island;
  sv.npolys = sc.npolys;
  sv.polyMask = sc.polyMask;
  sv.refBase = sc.refBase;
  // (global memory: one stride for all scenes, slabs of different sizes must not overlap)
  // (global memory: carved per query below)
  WarpSlab w = carveSlab(
      kGlobal ? globalSlabs : smem + pl.slabOffset + static_cast<size_t>(warp) * warpGeoSlabBytes(pcap),
      pcap);
  // Large slabs (the group's slabs together exceed what L2 holds) belong to environments
  // instead: an environment's searches start from the same goal step after step and touch
  // nearly the same nodes, so its own slab is still warm in L2 from the step before, whereas
  // a warp meets a different environment every step.
  const bool slabPerEnv = kGlobal && g.slabPerEnv != 0u;

  const uint32_t B = g.B;
  (void)warpsPerBlock;
  if constexpr (kBatched) {
    uint16_t* stage = g.batchStage +
                      (static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + warp) * 32u * kMaxPathPolys;
    for (;;) {
      int cnt = 0;
      uint32_t myEntry = 0u, myStatus = 0u;
      int myLen = 0;
      float myD = 0.f, myA[3] = {0.f, 0.f, 0.f}, myB[3] = {0.f, 0.f, 0.f};
      while (cnt < 32) {
        uint32_t entry = 0u;
        if (!next(lane, &entry))
          break;
        const uint32_t e = entry & kListEnvMask;
        if (kGlobal) {
          const size_t slabIdx =
              slabPerEnv ? static_cast<size_t>(e)
                         : static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + static_cast<size_t>(warp);
          uint8_t* slab = globalSlabs + slabIdx * globalSlabStride;
          w = carveSlab(slab, pcap);
          w.searches = reinterpret_cast<uint32_t*>(slab + globalSlabStride - kGlobalSlabExtra);
        }
        const bool moved = entry & kListMoved;
        const float b[3] = {g.navGoal[e], g.navGoal[B + e], g.navGoal[2 * B + e]};
        const uint32_t bref = g.goalRef[e];
        float a[3];
        uint32_t aref;
        if (moved) {
          warpForwardMove(g, sv, sc, w, lane, e, a, &aref);
        } else {
          a[0] = g.navPos[e];
          a[1] = g.navPos[B + e];
          a[2] = g.navPos[2 * B + e];
          aref = g.navRef[e];
        }
        uint32_t status = 0u, fallback = 0u;
        float d = 0.f;
        int len = 0;
        const bool needGeo = g.task == kTaskPointNav || (g.task == kTaskFlee && moved);
        if (needGeo) {
          len = warpSearch<kGlobal>(sv, w, lane, b, bref, a, aref, &status, &fallback,
                                    g.exactHeap != 0, &d);
          if (fallback) {  // (rare) the one-thread emulation, at once
            if (lane == 0) {
              status = 0u;
              const size_t slot = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
              d = geodesic(scGlobal, fallbackScratch + slot, b, bref, a, aref, &status);
              status |= fallback;
            }
            d = __shfl_sync(0xffffffffu, d, 0);
            status = __shfl_sync(0xffffffffu, status, 0);
            len = 0;
          }
          for (int i = lane; i < len; i += 32)
            stage[cnt * kMaxPathPolys + i] = w.path[i];
        }
        if (lane == cnt) {
          myEntry = entry;
          myStatus = status;
          myLen = len;
          myD = d;
          myA[0] = a[0]; myA[1] = a[1]; myA[2] = a[2];
          myB[0] = b[0]; myB[1] = b[1]; myB[2] = b[2];
        }
        ++cnt;
        __syncwarp();
      }
      if (cnt == 0)
        break;
      if (lane < cnt) {
        const uint32_t e = myEntry & kListEnvMask;
        const bool done = myEntry & kListDone, moved = myEntry & kListMoved;
        if (myLen > 0) {
          uint32_t st2 = 0u;
          myD = funnelLength(sc, myB, myA, stage + lane * kMaxPathPolys, myLen, &st2);
          myStatus |= st2;
        }
        if (g.task == kTaskExploration && moved)
          explVisit(g, e, myA[0], myA[1], myA[2]);
        if (myStatus)
          g.status[e] |= myStatus;
        finishEnv(g, st, e, done, moved, myD, seedLo, seedHi);
      }
      __syncwarp();
      if (cnt < 32)
        break;
    }
  } else {
  for (;;) {
    uint32_t entry = 0u;
    if (!next(lane, &entry))
      break;
    const uint32_t e = entry & kListEnvMask;
    if (kGlobal) {
      const size_t slabIdx =
          slabPerEnv ? static_cast<size_t>(e)
                     : static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + static_cast<size_t>(warp);
      uint8_t* slab = globalSlabs + slabIdx * globalSlabStride;
      w = carveSlab(slab, pcap);
      w.searches = reinterpret_cast<uint32_t*>(slab + globalSlabStride - kGlobalSlabExtra);
    }
    const bool done = entry & kListDone, moved = entry & kListMoved;
    const float b[3] = {g.navGoal[e], g.navGoal[B + e], g.navGoal[2 * B + e]};
    const uint32_t bref = g.goalRef[e];
    float a[3];
    uint32_t aref;
    if (moved) {
      warpForwardMove(g, sv, sc, w, lane, e, a, &aref);
    } else {
      a[0] = g.navPos[e];
      a[1] = g.navPos[B + e];
      a[2] = g.navPos[2 * B + e];
      aref = g.navRef[e];
    }
    uint32_t status = 0;
    uint32_t fallback = 0u;
    float d = 0.f;
    // PointNav queries on every listed step, Flee only after a move, Exploration never
    const bool needGeo = g.task == kTaskPointNav || (g.task == kTaskFlee && moved);
    if (needGeo) {
      d = warpGeodesic<kGlobal>(sv, w, lane, b, bref, a, aref, &status, &fallback, g.exactHeap != 0);
    }
    if (lane == 0) {
      if (fallback) {
        status = 0;
        const size_t slot = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
        d = geodesic(scGlobal, fallbackScratch + slot, b, bref, a, aref, &status);
        status |= fallback;
      }
      if (g.task == kTaskExploration && moved)
        explVisit(g, e, a[0], a[1], a[2]);
      if (status)
        g.status[e] |= status;
      finishEnv(g, st, e, done, moved, d, seedLo, seedHi);
    }
    __syncwarp();
  }
  }
}

// One simulator step for the listed environments (see sim_kernels.cuh for the phase split):
// forward move, GPS/compass, geodesic goal -> agent, info / reward / mask and the in-loop
// reset.
//   grid  = CTAs of all slots (ctaMap: slot, number among the slot's CTAs, their count),
//           block = 512 threads
//   smem  = staged tables of the scene being worked on + as many warp slabs as fit
//           (plan[scene].warps)
// A CTA drains the slot's two work lists one after the other: environments in the slot's
// scene, then (only while the slot is moving to another scene) those still in the previous
// one, whose tables are staged in between.  Warps pull list slots from a per-list cursor
// until the list is drained.
// Three instances, chosen by the host from the group's plan, so that a group whose scenes
// all sit in shared memory (the usual case) does not carry the code of the other mode:
//   kMode 0  every scene of the group is staged in shared memory
//   kMode 1  every scene is worked on in global memory (launched without dynamic shared
//            memory, which leaves the whole unified cache to L1)
//   kMode 2  both kinds in one grid
// and each of them for fixed scenes (kRotate false: one list per slot, and which scene the
// slot has is known before the kernel has to wait for its predecessor) and for rotating ones.
// kFused (fixed scenes in shared memory only): the kernel also does the part of the step that
// needs no navmesh query (preEnv, otherwise the kernel k_pre before this one) for a share of
// its slot's environments and works off the list of those it has to query itself, from
// shared memory: one launch per step and no work list in global memory.  For batches in which
// a CTA's share is small enough for its warps to take one query each; with more, the
// lists of all CTAs of a slot are better drained together (k_pre + global lists).
template <int kMode, bool kRotate, bool kFused = false, bool kBatched = false>
__global__ void __launch_bounds__(512, kMode == 1 ? 2 : 1)
k_step_warp(GroupDev g, SceneTable st, const WarpPlan* __restrict__ plan,
            const uint4* __restrict__ ctaMap, AStarScratch* __restrict__ fallbackScratch,
            uint8_t* __restrict__ globalSlabs, size_t globalSlabStride, uint32_t seedLo,
            uint32_t seedHi, const int64_t* __restrict__ actions,
            const uint8_t* __restrict__ actions8, TurnConsts tc) {
  static_assert(!kFused || (kMode == 0 && !kRotate), "fused: fixed scenes in shared memory");
  static_assert(!kBatched || (kMode != 2 && !kRotate && !kFused), "batched: large fixed batches");
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ uint32_t fusedList[kFused ? kFusedMaxShare : 1];
  __shared__ uint32_t fusedCount;
  launchDependents();
  // which slot this CTA serves, its number among that slot's CTAs and how many they are
  // (set-up data)
  const uint4 cm = ctaMap[blockIdx.x];
  const uint32_t slot = cm.x, rank = cm.y, slotCtas = cm.z;
  const int warp = threadIdx.x >> 5;

  // The staged image of a scene was laid out at set-up exactly as stagedLayout() describes
  // (float4 vertices, polygons with filtered links and the duplicate-neighbour flag, detail
  // bases / triangles / vertices, island ids), 16-byte aligned and a multiple of 16 bytes
  // long: one bulk asynchronous copy (TMA, untiled, this CTA's own shared memory, no
  // multicast) brings it in and signals an mbarrier, whose phase alternates from one copy
  // to the next.
  __shared__ __align__(8) unsigned long long stageBar;
  const uint32_t bar = static_cast<uint32_t>(__cvta_generic_to_shared(&stageBar));
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  uint32_t phase = 0u;
  bool inFlight = false, failed = false;
  uint32_t stagedScene = 0xffffffffu;
  auto stage = [&](const NavScene& scn) {
    if (threadIdx.x == 0) {
      const uint32_t bytes = scn.stagedBytes;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                   : "memory");
      asm volatile(
          "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
          ::"r"(dst), "l"(scn.staged), "r"(bytes), "r"(bar)
          : "memory");
    }
    inFlight = true;
  };
  // bounded wait for the copy in flight (a copy of this size lands within microseconds, the
  // bound is ~1 s of polling); false when it did not arrive
  auto landed = [&]() -> bool {
    bool ok = false;
    for (int it = 0; it < (1 << 22) && !ok; ++it) {
      uint32_t r;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(r)
          : "r"(bar), "r"(phase)
          : "memory");
      ok = r != 0;
    }
    const bool all = __syncthreads_and(ok ? 1 : 0) != 0;
    if (all) {
      phase ^= 1u;
      inFlight = false;
    }
    return all;
  };
  if (kMode != 1) {
    if (threadIdx.x == 0) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
  }
  // Fixed scenes: which scene the slot has is set-up data and its image never changes, so
  // all of it is fetched, and the copy started, while the kernel before this one is still at
  // work.
  uint32_t sc0 = 0u;
  WarpPlan pl0{};
  NavScene scn0{};
  if (!kRotate) {
    sc0 = g.slotScene[slot];
    pl0 = plan[sc0];
    scn0 = st.scenes[sc0];
    if (kMode != 1 && pl0.warps != 0 && pl0.slabOffset != kSlabInGlobal) {
      stage(scn0);
      stagedScene = sc0;
    }
  }
  // fused: this CTA's share of the slot's environments (set-up data)
  uint32_t myEnv = 0xffffffffu;
  if (kFused) {
    const uint32_t size = g.slotSize[slot];
    const uint32_t share = (size + slotCtas - 1u) / slotCtas;
    // spread over the warps (lane l of warp w takes the share's environment 16 l + w): the
    // three kinds of step -- a turn, a move, the end of an episode with its reset -- then run
    // side by side in different warps instead of one after the other in one
    const uint32_t mine = (threadIdx.x & 31u) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t at = rank * share + mine;
    if (mine < share && at < size)
      myEnv = g.slotEnvs[g.slotEnvBase[slot] + at];
    if (threadIdx.x == 0)
      fusedCount = 0u;
    __syncthreads();
  }
  // everything below reads what the kernels before this one wrote
  waitForPredecessor();
  if (kFused) {
    if (myEnv != 0xffffffffu) {
      uint32_t entry = 0u, listIdx = 0u;
      if (preEnv(g, st, myEnv, actions, actions8, tc, seedLo, seedHi, &entry, &listIdx))
        fusedList[atomicAdd(&fusedCount, 1u)] = entry;
    }
    __syncthreads();
    // entries beyond one per query warp go to this CTA's segment in global memory, where
    // any warp of the slot's CTAs can claim them (FusedSource)
    const uint32_t nLocal = min(fusedCount, pl0.warps);
    const uint32_t nOver = fusedCount - nLocal;
    if (threadIdx.x < nOver)
      g.ovList[static_cast<size_t>(blockIdx.x) * kFusedMaxShare + threadIdx.x] =
          fusedList[nLocal + threadIdx.x];
    __syncthreads();
    if (threadIdx.x == 0) {
      volatile uint32_t* meta = g.ovMeta + 4u * blockIdx.x;
      meta[0] = nOver;
      meta[1] = 0u;
      __threadfence();
      meta[2] = g.stepId;
    }
    __syncthreads();  // the CTA's own warps see their segment as published
  }

  if (!kFused && blockIdx.x == 0 && warp == 0) {
    // how many entries this step lists, for the host (GroupDev::hListed)
    uint32_t listed = 0u;
    for (uint32_t l = threadIdx.x; l < g.numLists; l += 32u)
      listed += g.counts[l];
    listed = __reduce_add_sync(0xffffffffu, listed);
    if (threadIdx.x == 0)
      *reinterpret_cast<volatile uint32_t*>(g.hListed) = listed;
  }
  constexpr uint32_t kRoles = kRotate ? 2u : 1u;
  // A slot that is between two scenes has entries in both of its lists.  Its CTAs then divide
  // into two parties in proportion to the lists' lengths, one per list, so that the two scenes
  // are worked on side by side and the step lasts as long as the slower of the two, not as
  // their sum (a single CTA, or a slot with one list empty, takes them one after the other).
  uint32_t firstParty = 0u;  // CTAs of the party of list 0; 0: no division
  if (kRotate && slotCtas > 1u) {
    const uint32_t n0 = g.counts[2u * slot], n1 = g.counts[2u * slot + 1u];
    if (n0 != 0u && n1 != 0u) {
      const uint32_t c0 = (slotCtas * n0 + (n0 + n1) / 2u) / (n0 + n1);
      firstParty = min(max(c0, 1u), slotCtas - 1u);
    }
  }
#pragma unroll 1
  for (uint32_t role = 0; role < kRoles; ++role) {
    const uint32_t listIdx = 2u * slot + role;
    // (fused: a CTA without entries of its own may still find some to take over)
    const uint32_t n = kFused ? 1u : g.counts[listIdx];
    if (!kFused && rank == 0 && threadIdx.x == 0) {  // the next step starts from empty lists
      g.countsNext[listIdx] = 0u;
      g.countsNext[g.numLists + listIdx] = 0u;
    }
    if (n == 0)
      continue;
    uint32_t partyRank = rank, partyCtas = slotCtas;
    if (kRotate && firstParty != 0u) {
      if ((role == 0u) != (rank < firstParty))
        continue;  // the other party's list
      partyRank = role == 0u ? rank : rank - firstParty;
      partyCtas = role == 0u ? firstParty : slotCtas - firstParty;
    }
    const uint32_t sceneIdx = !kRotate ? sc0 : (role ? g.slotPrev[slot] : g.slotScene[slot]);
    const WarpPlan pl = !kRotate ? pl0 : plan[sceneIdx];
    if (pl.warps == 0)
      continue;  // a scene of the one-thread-per-environment kernel
    const NavScene scGlobal = !kRotate ? scn0 : st.scenes[sceneIdx];
    // A scene too large to sit in shared memory next to at least one slab is worked on where
    // it lies: the same image, in global memory (L2-resident), and slabs in a global
    // scratch area.  The code is the same either way; only the latency differs.
    const bool inGlobal = kMode == 1 || (kMode == 2 && pl.slabOffset == kSlabInGlobal);
    if (kMode != 1 && !inGlobal) {
      if (stagedScene != sceneIdx) {
        if (inFlight && !landed()) {
          failed = true;
          break;
        }
        __syncthreads();  // every warp is through with the image that is being replaced
        stage(scGlobal);
        stagedScene = sceneIdx;
      }
      if (inFlight && !landed()) {
        failed = true;
        break;
      }
    }
    const int warpsPerBlock = static_cast<int>(pl.warps);  // warps of this CTA that take queries
    if (warp >= warpsPerBlock)
      continue;
#define BPSN_STEP_ARGS scGlobal, globalSlabs, globalSlabStride, fallbackScratch, seedLo, seedHi
    if constexpr (kFused) {
      FusedSource src{fusedList, min(fusedCount, pl.warps), g.ovList, g.ovMeta,
                      blockIdx.x - rank, rank, slotCtas, g.stepId, warp, 0u};
      stepWarpQueries<false, false>(g, st, pl, src, BPSN_STEP_ARGS);
    } else {
      const uint32_t firstQ =
          partyRank * static_cast<uint32_t>(warpsPerBlock) + static_cast<uint32_t>(warp);
      if (firstQ - static_cast<uint32_t>(warp) >= n)
        continue;
      ListSource src{g.geoList + g.listBase[listIdx], g.counts + g.numLists + listIdx, firstQ,
                     partyCtas * static_cast<uint32_t>(warpsPerBlock), n, true};
      if constexpr (kMode == 0) {
        stepWarpQueries<false, kBatched>(g, st, pl, src, BPSN_STEP_ARGS);
      } else if constexpr (kMode == 1) {
        stepWarpQueries<true, kBatched>(g, st, pl, src, BPSN_STEP_ARGS);
      } else {
        if (inGlobal)
          stepWarpQueries<true, false>(g, st, pl, src, BPSN_STEP_ARGS);
        else
          stepWarpQueries<false, false>(g, st, pl, src, BPSN_STEP_ARGS);
      }
    }
#undef BPSN_STEP_ARGS
  }
  if (kMode != 1) {
    // A copy whose list turned out empty, or one that did not arrive in time (never observed):
    // the CTA does not exit under a copy into its own shared memory, it waits once more.  A
    // copy that was late is made visible (bpsn_step_end reports it): the environments this CTA
    // would have served keep the outputs of the step before.
    if (inFlight)
      landed();
    if (failed && threadIdx.x == 0) {
      atomicOr(g.errFlags, 1u);
      if (g.hErr)
        *g.hErr = 1u;
    }
  }
  if (g.pubDst) {
    // The CTA that is through last publishes the step's results (see GroupDev::pubDst).  Every
    // CTA's stores are fenced before it counts itself, the last one fences again before it
    // reads them; the results of the environments that needed no query were written by the
    // kernel before this one.
    __shared__ uint32_t lastCta;
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const uint32_t before = atomicAdd(g.doneCount, 1u);
      lastCta = before == gridDim.x - 1u ? 1u : 0u;
      if (lastCta)
        *g.doneCount = 0u;  // for the next step
    }
    __syncthreads();
    if (lastCta) {
      __threadfence();
      // (four loads in flight per thread before the first store)
      for (uint32_t base = threadIdx.x; base < g.pubVec; base += 4u * blockDim.x) {
        uint4 v[4];
#pragma unroll
        for (uint32_t k = 0; k < 4u; ++k)
          if (base + k * blockDim.x < g.pubVec)
            v[k] = __ldcg(g.pubSrc + base + k * blockDim.x);
#pragma unroll
        for (uint32_t k = 0; k < 4u; ++k)
          if (base + k * blockDim.x < g.pubVec)
            g.pubDst[base + k * blockDim.x] = v[k];
      }
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0)
        *reinterpret_cast<volatile uint32_t*>(g.hStepFlag) = g.stepId;
    }
  }
}

}  // namespace bpsn
