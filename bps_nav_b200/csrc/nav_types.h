// Flattened, read-only navigation-mesh image as the kernels see it, plus the
// per-query scratch layout.  Plain structs shared by the host flattener
// (navmesh_host.cpp) and the device code (nav_query.cuh).
//
// One scene = one Detour tile.  The reference keeps a dtMeshTile with pointer
// fields patched at load time (Detour/Include/DetourNavMesh.h:280-312) and a
// per-polygon linked list of dtLink records; for a single tile every link is
// an internal one and the list order is ascending edge index
// (Detour/Source/DetourNavMesh.cpp:524-559), so the image keeps only the
// neis[] array and recovers neighbour order by scanning edges 0..n-1.
#pragma once

#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define BPSN_HD __host__ __device__ __forceinline__
#define BPSN_HD_NOINLINE __host__ __device__ __noinline__
#else
#define BPSN_HD inline
#define BPSN_HD_NOINLINE
#endif

namespace bpsn {

constexpr int kVertsPerPoly = 6;       // DT_VERTS_PER_POLYGON
constexpr uint16_t kExtLink = 0x8000;  // DT_EXT_LINK
constexpr uint16_t kFlagWalk = 0x01;   // POLYFLAGS_WALK  (PathFinder.cpp:229-234)
constexpr uint16_t kFlagDisabled = 0x04;

constexpr int kMaxAStarNodes = 2048;  // dtNavMeshQuery::init(navMesh, 2048), PathFinder.cpp:247
constexpr int kMaxPathPolys = 256;    // MAX_POLYS, PathFinder.cpp:499
constexpr int kHashBuckets = 512;     // dtNextPow2(maxNodes / 4), DetourNavMeshQuery.cpp:180
constexpr int kMoveStack = 48;        // MAX_STACK, DetourNavMeshQuery.cpp:2040
constexpr int kMovePool = 64;         // tiny node pool, DetourNavMeshQuery.cpp:191

// 32 bytes, two 16-byte loads.  Same information as dtPoly minus firstLink.
struct alignas(16) NavPoly {
  uint16_t verts[kVertsPerPoly];
  uint16_t neis[kVertsPerPoly];
  uint16_t flags;
  uint8_t vertCount;
  uint8_t areaAndType;
  uint8_t detailVertCount;
  uint8_t detailTriCount;
  uint16_t pad;
};
static_assert(sizeof(NavPoly) == 32, "NavPoly must be 32 bytes");

struct alignas(8) NavDetail {  // dtPolyDetail bases
  uint32_t vertBase;
  uint32_t triBase;
};

struct alignas(16) NavBVNode {  // dtBVNode, 16 bytes
  uint16_t bmin[3];
  uint16_t bmax[3];
  int32_t i;
};
static_assert(sizeof(NavBVNode) == 16, "NavBVNode must be 16 bytes");

// Device-resident scene descriptor (pointers are device pointers in the
// shipped library, host pointers in the host-side checks of the flattener).
struct NavScene {
  const float* verts;       // 3 * nverts
  const NavPoly* polys;     // npolys
  const NavDetail* detail;  // npolys
  const float* dverts;      // 3 * ndverts
  const uint8_t* dtris;     // 4 * ndtris
  const NavBVNode* bv;      // nbv (0 => linear scan)
  const int32_t* island;    // npolys, connected-component id per polygon
  const uint8_t* staged;    // ready-to-copy shared-memory image of the tables (may be null)
  uint32_t stagedBytes;
  int32_t npolys;
  int32_t nverts;
  int32_t nbv;
  int32_t ndverts;
  int32_t ndtris;
  int32_t vstride;  // floats between consecutive vertices in `verts` (3, or 4 when staged)
  uint32_t refBase;   // salt/tile bits of every polygon ref of this tile
  uint32_t polyMask;  // (1 << polyBits) - 1
  float bmin[3];
  float bmax[3];
  float bvQuantFactor;
  float walkableClimb;
  // dtNavMeshParams + tile grid location, for queryPolygons' tile lookup
  float orig[3];
  float tileWidth;
  float tileHeight;
  int32_t tileX;
  int32_t tileY;
};

// A* node, 32 bytes: dtNode (Detour/Include/DetourNode.h:36-45) plus the
// hash-chain link and the node's current heap slot (replaces the linear
// search in dtNodeQueue::modify).
struct alignas(16) AStarNode {
  float pos[3];
  float cost;
  float total;
  uint32_t poly;    // polygon index within the tile
  uint16_t parent;  // 1-based node index, 0 = none
  uint16_t next;    // hash chain, 0xffff = end
  uint16_t heapPos;
  uint8_t flags;  // 1 open, 2 closed
  uint8_t pad;
};
static_assert(sizeof(AStarNode) == 32, "AStarNode must be 32 bytes");

struct alignas(8) HeapEntry {
  float total;
  uint32_t node;
};

// Per-query scratch slab (global memory; one per resident query slot).
struct alignas(16) AStarScratch {
  AStarNode nodes[kMaxAStarNodes];
  uint16_t first[kHashBuckets];        // hash heads; cleared with 16-byte stores
  HeapEntry heap[kMaxAStarNodes + 2];  // reused as the corridor after the search
};
static_assert(offsetof(AStarScratch, first) % 16 == 0, "hash heads must be 16-byte aligned");
static_assert(offsetof(AStarScratch, heap) % 16 == 0, "heap must be 16-byte aligned");
static_assert(sizeof(AStarScratch) % 16 == 0, "scratch slabs must tile with 16-byte alignment");

// Per-query status bits (diagnostics only; they never change an output).
enum QueryStatus : uint32_t {
  kStatOutOfNodes = 1u << 0,    // DT_OUT_OF_NODES  -> distance = +inf
  kStatPartial = 1u << 1,       // DT_PARTIAL_RESULT -> +inf
  kStatPathTooLong = 1u << 2,   // corridor > 256 polys -> +inf
  kStatFunnelOverflow = 1u << 3,  // straight path >= 256 points -> +inf
  kStatSnapFailed = 1u << 4,    // findNearestPoly found nothing -> NaN point, ref 0
  kStatIterCap = 1u << 5,       // a defensive loop bound was hit
  kStatNoIsland = 1u << 6,      // start/end on different components -> +inf
  kStatBadAction = 1u << 7,     // action outside {0,1,2,3}
  kStatTieFallback = 1u << 8,   // open-list tie: query rerun with the exact heap emulation
  kStatOpenOverflow = 1u << 9,  // register open list full, or a zero / out-of-range distance in the
                                // fast search: query rerun the same way
  kStatTieInPlace = 1u << 10,   // a two-way open-list tie whose order cannot matter was expanded in place
};

}  // namespace bpsn
