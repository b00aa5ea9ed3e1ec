// TEST INFRASTRUCTURE ONLY -- never linked into or called by the shipped library.
//
// C-ABI shim over the *unmodified* reference navigation library so that the
// oracle simulator (oracle_sim.cpp) and the Python test-suite can call it
// through ctypes.  This translation unit is compiled together with the
// reference's own Detour + PathFinder sources (the same source list that
// simulator/external/CMakeLists.txt:25-44 builds as `habitat_sim_geodesic`)
// into oracle/_ref/libref_nav.so by oracle/Makefile.
//
// Two handle kinds are exposed:
//   * refnav_*  : esp::nav::PathFinder (HSG csrc/PathFinder.h:99-227) --
//                 loadNavMesh / snapPoint / tryStep / findPath, exactly the
//                 calls simulator/simulator.cpp:553-563, 611, 689, 747 make.
//   * refdt_*   : a raw dtNavMesh + dtNavMeshQuery built from the same file
//                 the way PathFinder::Impl::loadNavMesh does
//                 (csrc/PathFinder.cpp:330-408, 245-256), used only to expose
//                 the intermediate results (A* corridor, funnel points,
//                 moveAlongSurface visited list, findNearestPoly) that
//                 PathFinder hides, for unit parity tests of each primitive.

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <string>
#include <vector>

#include "PathFinder.h"

#include "DetourCommon.h"
#include "DetourNavMesh.h"
#include "DetourNavMeshQuery.h"

using esp::vec3f;
using esp::nav::NavMeshPoint;
using esp::nav::PathFinder;
using esp::nav::ShortestPath;

extern "C" {

// ---------------------------------------------------------------- PathFinder

void* refnav_create(const char* navmesh_path) {
  PathFinder* pf = new PathFinder();
  if (!pf->loadNavMesh(std::string(navmesh_path))) {
    delete pf;
    return nullptr;
  }
  return pf;
}

void refnav_destroy(void* h) {
  delete static_cast<PathFinder*>(h);
}

// PathFinder::snapPoint -> xyz (NaN on failure) + polyId.
void refnav_snap(void* h, const float* pt, float* out_xyz, uint64_t* out_poly) {
  PathFinder* pf = static_cast<PathFinder*>(h);
  NavMeshPoint p = pf->snapPoint(vec3f(pt[0], pt[1], pt[2]));
  out_xyz[0] = p.xyz[0];
  out_xyz[1] = p.xyz[1];
  out_xyz[2] = p.xyz[2];
  *out_poly = p.polyId;
}

// PathFinder::tryStep (sliding allowed).
void refnav_try_step(void* h,
                     const float* start_xyz,
                     uint64_t start_poly,
                     const float* end_xyz,
                     float* out_xyz,
                     uint64_t* out_poly) {
  PathFinder* pf = static_cast<PathFinder*>(h);
  NavMeshPoint s{vec3f(start_xyz[0], start_xyz[1], start_xyz[2]), start_poly};
  NavMeshPoint r = pf->tryStep(s, vec3f(end_xyz[0], end_xyz[1], end_xyz[2]));
  out_xyz[0] = r.xyz[0];
  out_xyz[1] = r.xyz[1];
  out_xyz[2] = r.xyz[2];
  *out_poly = r.polyId;
}

// PathFinder::findPath -> geodesic distance (may be +inf); optionally copies
// up to max_pts straight-path points.
float refnav_find_path(void* h,
                       const float* s_xyz,
                       uint64_t s_poly,
                       const float* e_xyz,
                       uint64_t e_poly,
                       float* out_pts,
                       int max_pts,
                       int* out_npts) {
  PathFinder* pf = static_cast<PathFinder*>(h);
  ShortestPath sp;
  sp.requestedStart = NavMeshPoint{vec3f(s_xyz[0], s_xyz[1], s_xyz[2]), s_poly};
  sp.requestedEnd = NavMeshPoint{vec3f(e_xyz[0], e_xyz[1], e_xyz[2]), e_poly};
  pf->findPath(sp);
  if (out_npts)
    *out_npts = static_cast<int>(sp.points.size());
  if (out_pts) {
    int n = static_cast<int>(sp.points.size());
    if (n > max_pts)
      n = max_pts;
    for (int i = 0; i < n; ++i) {
      out_pts[3 * i + 0] = sp.points[i][0];
      out_pts[3 * i + 1] = sp.points[i][1];
      out_pts[3 * i + 2] = sp.points[i][2];
    }
  }
  return sp.geodesicDistance;
}

// Batched versions (one ctypes call for many queries keeps the tests fast).
void refnav_snap_batch(void* h, int n, const float* pts, float* out_xyz, uint64_t* out_poly) {
  for (int i = 0; i < n; ++i)
    refnav_snap(h, pts + 3 * i, out_xyz + 3 * i, out_poly + i);
}

void refnav_try_step_batch(void* h,
                           int n,
                           const float* start_xyz,
                           const uint64_t* start_poly,
                           const float* end_xyz,
                           float* out_xyz,
                           uint64_t* out_poly) {
  for (int i = 0; i < n; ++i)
    refnav_try_step(h, start_xyz + 3 * i, start_poly[i], end_xyz + 3 * i, out_xyz + 3 * i,
                    out_poly + i);
}

void refnav_find_path_batch(void* h,
                            int n,
                            const float* s_xyz,
                            const uint64_t* s_poly,
                            const float* e_xyz,
                            const uint64_t* e_poly,
                            float* out_dist) {
  for (int i = 0; i < n; ++i)
    out_dist[i] = refnav_find_path(h, s_xyz + 3 * i, s_poly[i], e_xyz + 3 * i, e_poly[i], nullptr,
                                   0, nullptr);
}

void refnav_bounds(void* h, float* bmin, float* bmax) {
  PathFinder* pf = static_cast<PathFinder*>(h);
  auto b = pf->bounds();
  for (int i = 0; i < 3; ++i) {
    bmin[i] = b.first[i];
    bmax[i] = b.second[i];
  }
}

// ------------------------------------------------------------- raw Detour

struct RefDt {
  dtNavMesh* mesh = nullptr;
  dtNavMeshQuery* query = nullptr;
  dtQueryFilter filter;
};

namespace {
struct SetHeader {
  int magic;
  int version;
  int numTiles;
  dtNavMeshParams params;
};
struct TileHeader {
  dtTileRef tileRef;
  int dataSize;
};
}  // namespace

void refdt_destroy(void* h) {
  RefDt* r = static_cast<RefDt*>(h);
  if (!r)
    return;
  if (r->query)
    dtFreeNavMeshQuery(r->query);
  if (r->mesh)
    dtFreeNavMesh(r->mesh);
  delete r;
}

// Same steps as PathFinder::Impl::loadNavMesh + removeZeroAreaPolys +
// initNavQuery (minus the island system), on a private dtNavMesh.
void* refdt_create(const char* path) {
  FILE* fp = fopen(path, "rb");
  if (!fp)
    return nullptr;
  SetHeader hdr;
  if (fread(&hdr, sizeof(hdr), 1, fp) != 1) {
    fclose(fp);
    return nullptr;
  }
  RefDt* r = new RefDt();
  r->filter.setIncludeFlags(0x01);
  r->filter.setExcludeFlags(0);
  r->mesh = dtAllocNavMesh();
  if (dtStatusFailed(r->mesh->init(&hdr.params))) {
    fclose(fp);
    refdt_destroy(r);
    return nullptr;
  }
  for (int i = 0; i < hdr.numTiles; ++i) {
    TileHeader th;
    if (fread(&th, sizeof(th), 1, fp) != 1)
      break;
    if (!th.tileRef || !th.dataSize)
      break;
    unsigned char* data = static_cast<unsigned char*>(dtAlloc(th.dataSize, DT_ALLOC_PERM));
    memset(data, 0, th.dataSize);
    if (fread(data, th.dataSize, 1, fp) != 1) {
      dtFree(data);
      break;
    }
    r->mesh->addTile(data, th.dataSize, DT_TILE_FREE_DATA, th.tileRef, 0);
  }
  fclose(fp);

  // Disable polygons whose detail-mesh area is below 1e-5, as
  // PathFinder::Impl::removeZeroAreaPolys does (same arithmetic: Eigen
  // cross/norm in float, accumulated as `area += 0.5 * norm` in double then
  // stored to float).
  const dtNavMesh* cm = r->mesh;
  for (int it = 0; it < r->mesh->getMaxTiles(); ++it) {
    const dtMeshTile* tile = cm->getTile(it);
    if (!tile || !tile->header)
      continue;
    for (int jp = 0; jp < tile->header->polyCount; ++jp) {
      const dtPoly* poly = &tile->polys[jp];
      const dtPolyDetail* pd = &tile->detailMeshes[jp];
      float area = 0;
      for (int j = 0; j < pd->triCount; ++j) {
        const unsigned char* t = &tile->detailTris[(pd->triBase + j) * 4];
        const float* v[3];
        for (int k = 0; k < 3; ++k) {
          if (t[k] < poly->vertCount)
            v[k] = &tile->verts[poly->verts[t[k]] * 3];
          else
            v[k] = &tile->detailVerts[(pd->vertBase + (t[k] - poly->vertCount)) * 3];
        }
        const vec3f w1 = Eigen::Map<const vec3f>(v[1]) - Eigen::Map<const vec3f>(v[0]);
        const vec3f w2 = Eigen::Map<const vec3f>(v[2]) - Eigen::Map<const vec3f>(v[0]);
        area += 0.5 * w1.cross(w2).norm();
      }
      if (area < 1e-5)
        r->mesh->setPolyFlags(cm->encodePolyId(tile->salt, it, jp), 0x04);
    }
  }

  r->query = dtAllocNavMeshQuery();
  if (dtStatusFailed(r->query->init(r->mesh, 2048))) {
    refdt_destroy(r);
    return nullptr;
  }
  return r;
}

// dtNavMeshQuery::findPath -> corridor refs + raw status word.
unsigned int refdt_find_path(void* h,
                             unsigned int start_ref,
                             unsigned int end_ref,
                             const float* start_pos,
                             const float* end_pos,
                             unsigned int* path,
                             int* path_count,
                             int max_path) {
  RefDt* r = static_cast<RefDt*>(h);
  return r->query->findPath(start_ref, end_ref, start_pos, end_pos, &r->filter, path, path_count,
                            max_path);
}

// dtNavMeshQuery::findStraightPath with options = 0.
unsigned int refdt_straight_path(void* h,
                                 const float* start_pos,
                                 const float* end_pos,
                                 const unsigned int* path,
                                 int path_size,
                                 float* out_pts,
                                 int* out_count,
                                 int max_pts) {
  RefDt* r = static_cast<RefDt*>(h);
  return r->query->findStraightPath(start_pos, end_pos, path, path_size, out_pts, 0, 0, out_count,
                                    max_pts, 0);
}

// dtNavMeshQuery::moveAlongSurface (Habitat variant with allowSliding).
unsigned int refdt_move_along_surface(void* h,
                                      unsigned int start_ref,
                                      const float* start_pos,
                                      const float* end_pos,
                                      float* result_pos,
                                      unsigned int* visited,
                                      int* visited_count,
                                      int max_visited,
                                      int allow_sliding) {
  RefDt* r = static_cast<RefDt*>(h);
  return r->query->moveAlongSurface(start_ref, start_pos, end_pos, &r->filter, result_pos, visited,
                                    visited_count, max_visited, allow_sliding != 0);
}

unsigned int refdt_find_nearest_poly(void* h,
                                     const float* center,
                                     const float* half_extents,
                                     unsigned int* nearest_ref,
                                     float* nearest_pt) {
  RefDt* r = static_cast<RefDt*>(h);
  return r->query->findNearestPoly(center, half_extents, &r->filter, nearest_ref, nearest_pt);
}

unsigned int refdt_get_poly_height(void* h, unsigned int ref, const float* pos, float* height) {
  RefDt* r = static_cast<RefDt*>(h);
  return r->query->getPolyHeight(ref, pos, height);
}

// Area-weighted random point (dtNavMeshQuery::findRandomPoint) driven by a
// caller-owned LCG so fixture generation is reproducible and does not touch
// the C library's global rand() state.
static thread_local uint64_t g_lcg = 0x9E3779B97F4A7C15ull;
static float lcg_frand() {
  g_lcg = g_lcg * 6364136223846793005ull + 1442695040888963407ull;
  return static_cast<float>((g_lcg >> 40) & 0xFFFFFF) / static_cast<float>(1 << 24);
}
void refdt_seed(uint64_t s) {
  g_lcg = s * 2862933555777941757ull + 3037000493ull;
}
unsigned int refdt_random_point(void* h, unsigned int* ref, float* pt) {
  RefDt* r = static_cast<RefDt*>(h);
  return r->query->findRandomPoint(&r->filter, lcg_frand, ref, pt);
}

int refdt_poly_count(void* h) {
  RefDt* r = static_cast<RefDt*>(h);
  const dtNavMesh* cm = r->mesh;
  int n = 0;
  for (int it = 0; it < r->mesh->getMaxTiles(); ++it) {
    const dtMeshTile* tile = cm->getTile(it);
    if (tile && tile->header)
      n += tile->header->polyCount;
  }
  return n;
}

}  // extern "C"
