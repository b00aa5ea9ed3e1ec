// TEST / FIXTURE TOOLING ONLY -- never linked into or called by the shipped
// library.
//
// Synthetic floor-plan -> navigation-mesh generator.  It is compiled together
// with the reference's *unmodified* Recast sources and Detour's
// dtCreateNavMeshData (recastnavigation-master/Recast/Source/*.cpp,
// Detour/Source/DetourNavMeshBuilder.cpp) into oracle/_ref/gen_scene by
// oracle/Makefile, and writes a `.navmesh` file in the MSET container that
// esp::nav::PathFinder::loadNavMesh reads (csrc/PathFinder.cpp:258-272,
// 330-408).  The build steps are the standard single-tile Recast sequence
// (Recast/Include/Recast.h:775-1198): rasterise -> filter -> compact ->
// erode -> distance field -> regions -> contours -> poly mesh -> detail mesh.
//
// Scene: a flat SX x SZ metre floor at y = 0 with K axis-aligned box
// obstacles (sides U(0.5, 3) m, height 2 m) and W interior walls (0.2 m
// thick, full span, each with 1-3 door gaps of 1-2 m).  All randomness comes
// from a splitmix64 stream seeded on the command line, so a (size, boxes,
// walls, seed) tuple names one scene for ever.
//
// Recast parameters that the benchmark spec fixes: cs 0.05, agent radius 0.1,
// agent height 1.5, max slope 45 deg.  Parameters it leaves open and this
// tool fixes (also written to the .json manifest): ch 0.2, climb 0.2,
// maxEdgeLen 12 m, maxSimplificationError 1.3, minRegionArea 64 cells,
// mergeRegionArea 400 cells, detailSampleDist 6*cs, detailSampleMaxError 1*ch,
// nvp 6 (overridable).

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "Recast.h"

#include "DetourNavMesh.h"
#include "DetourNavMeshBuilder.h"

namespace {

struct Rng {
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed) {}
  uint64_t next() {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  double uni() { return (next() >> 11) * (1.0 / 9007199254740992.0); }
  double uni(double a, double b) { return a + (b - a) * uni(); }
};

struct Box {
  float mn[3], mx[3];
};

void addQuad(std::vector<float>& v, std::vector<int>& t, const float* a, const float* b,
             const float* c, const float* d) {
  int base = static_cast<int>(v.size() / 3);
  const float* p[4] = {a, b, c, d};
  for (int i = 0; i < 4; ++i)
    for (int k = 0; k < 3; ++k)
      v.push_back(p[i][k]);
  t.push_back(base);
  t.push_back(base + 1);
  t.push_back(base + 2);
  t.push_back(base);
  t.push_back(base + 2);
  t.push_back(base + 3);
}

// Closed box, outward-facing, counter-clockwise triangles (top faces +Y).
void addBox(std::vector<float>& v, std::vector<int>& t, const Box& b) {
  const float x0 = b.mn[0], y0 = b.mn[1], z0 = b.mn[2];
  const float x1 = b.mx[0], y1 = b.mx[1], z1 = b.mx[2];
  float p000[3] = {x0, y0, z0}, p100[3] = {x1, y0, z0}, p010[3] = {x0, y1, z0},
        p110[3] = {x1, y1, z0}, p001[3] = {x0, y0, z1}, p101[3] = {x1, y0, z1},
        p011[3] = {x0, y1, z1}, p111[3] = {x1, y1, z1};
  addQuad(v, t, p010, p011, p111, p110);  // top (+Y)
  addQuad(v, t, p000, p100, p101, p001);  // bottom (-Y)
  addQuad(v, t, p000, p010, p110, p100);  // -Z
  addQuad(v, t, p001, p101, p111, p011);  // +Z
  addQuad(v, t, p000, p001, p011, p010);  // -X
  addQuad(v, t, p100, p110, p111, p101);  // +X
}

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

int main(int argc, char** argv) {
  float sx = 20.f, sz = -1.f;
  int nboxes = 12, nwalls = 0, nvp = 6;
  uint64_t seed = 1000;
  std::string out = "scene";
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto val = [&]() -> const char* { return (i + 1 < argc) ? argv[++i] : ""; };
    if (a == "--size")
      sx = static_cast<float>(atof(val()));
    else if (a == "--size-z")
      sz = static_cast<float>(atof(val()));
    else if (a == "--boxes")
      nboxes = atoi(val());
    else if (a == "--walls")
      nwalls = atoi(val());
    else if (a == "--nvp")
      nvp = atoi(val());
    else if (a == "--seed")
      seed = strtoull(val(), nullptr, 10);
    else if (a == "--out")
      out = val();
    else {
      fprintf(stderr, "unknown argument %s\n", a.c_str());
      return 2;
    }
  }
  if (sz <= 0)
    sz = sx;

  Rng rng(seed);
  std::vector<Box> boxes;
  for (int i = 0; i < nboxes; ++i) {
    float w = static_cast<float>(rng.uni(0.5, 3.0));
    float d = static_cast<float>(rng.uni(0.5, 3.0));
    float cx = static_cast<float>(rng.uni(0.0, sx));
    float cz = static_cast<float>(rng.uni(0.0, sz));
    Box b;
    b.mn[0] = cx - 0.5f * w;
    b.mx[0] = cx + 0.5f * w;
    b.mn[2] = cz - 0.5f * d;
    b.mx[2] = cz + 0.5f * d;
    b.mn[1] = 0.f;
    b.mx[1] = 2.f;
    boxes.push_back(b);
  }
  for (int i = 0; i < nwalls; ++i) {
    bool alongX = (rng.next() & 1) != 0;  // wall runs along x, fixed z
    float span = alongX ? sx : sz;
    float other = alongX ? sz : sx;
    float pos = static_cast<float>(rng.uni(1.5, other - 1.5));
    int ngaps = 1 + static_cast<int>(rng.next() % 3);
    std::vector<std::pair<float, float>> gaps;
    for (int g = 0; g < ngaps; ++g) {
      float gw = static_cast<float>(rng.uni(1.0, 2.0));
      float gc = static_cast<float>(rng.uni(0.5 + 0.5 * gw, span - 0.5 - 0.5 * gw));
      gaps.push_back({gc - 0.5f * gw, gc + 0.5f * gw});
    }
    // sort gaps, emit the solid pieces between them
    for (size_t a = 0; a < gaps.size(); ++a)
      for (size_t b = a + 1; b < gaps.size(); ++b)
        if (gaps[b].first < gaps[a].first)
          std::swap(gaps[a], gaps[b]);
    float cur = 0.f;
    auto emit = [&](float a, float b) {
      if (b - a < 0.05f)
        return;
      Box w;
      w.mn[1] = 0.f;
      w.mx[1] = 2.f;
      if (alongX) {
        w.mn[0] = a;
        w.mx[0] = b;
        w.mn[2] = pos - 0.1f;
        w.mx[2] = pos + 0.1f;
      } else {
        w.mn[2] = a;
        w.mx[2] = b;
        w.mn[0] = pos - 0.1f;
        w.mx[0] = pos + 0.1f;
      }
      boxes.push_back(w);
    };
    for (auto& g : gaps) {
      if (g.first > cur)
        emit(cur, g.first);
      if (g.second > cur)
        cur = g.second;
    }
    emit(cur, span);
  }

  std::vector<float> verts;
  std::vector<int> tris;
  {
    float a[3] = {0, 0, 0}, b[3] = {0, 0, sz}, c[3] = {sx, 0, sz}, d[3] = {sx, 0, 0};
    addQuad(verts, tris, a, b, c, d);  // floor, +Y normal
  }
  for (auto& b : boxes)
    addBox(verts, tris, b);
  const int nverts = static_cast<int>(verts.size() / 3);
  const int ntris = static_cast<int>(tris.size() / 3);

  rcContext ctx(false);
  rcConfig cfg;
  memset(&cfg, 0, sizeof(cfg));
  const float agentHeight = 1.5f, agentRadius = 0.1f, agentClimb = 0.2f;
  cfg.cs = 0.05f;
  cfg.ch = 0.2f;
  cfg.walkableSlopeAngle = 45.f;
  cfg.walkableHeight = static_cast<int>(ceilf(agentHeight / cfg.ch));
  cfg.walkableClimb = static_cast<int>(floorf(agentClimb / cfg.ch));
  cfg.walkableRadius = static_cast<int>(ceilf(agentRadius / cfg.cs));
  cfg.maxEdgeLen = static_cast<int>(12.f / cfg.cs);
  cfg.maxSimplificationError = 1.3f;
  cfg.minRegionArea = 64;
  cfg.mergeRegionArea = 400;
  cfg.maxVertsPerPoly = nvp;
  cfg.detailSampleDist = 6.f * cfg.cs;
  cfg.detailSampleMaxError = 1.f * cfg.ch;
  rcCalcBounds(verts.data(), nverts, cfg.bmin, cfg.bmax);
  rcCalcGridSize(cfg.bmin, cfg.bmax, cfg.cs, &cfg.width, &cfg.height);

  rcHeightfield* solid = rcAllocHeightfield();
  if (!rcCreateHeightfield(&ctx, *solid, cfg.width, cfg.height, cfg.bmin, cfg.bmax, cfg.cs,
                           cfg.ch)) {
    fprintf(stderr, "rcCreateHeightfield failed\n");
    return 1;
  }
  std::vector<unsigned char> triareas(ntris, 0);
  rcMarkWalkableTriangles(&ctx, cfg.walkableSlopeAngle, verts.data(), nverts, tris.data(), ntris,
                          triareas.data());
  if (!rcRasterizeTriangles(&ctx, verts.data(), nverts, tris.data(), triareas.data(), ntris,
                            *solid, cfg.walkableClimb)) {
    fprintf(stderr, "rcRasterizeTriangles failed\n");
    return 1;
  }
  rcFilterLowHangingWalkableObstacles(&ctx, cfg.walkableClimb, *solid);
  rcFilterLedgeSpans(&ctx, cfg.walkableHeight, cfg.walkableClimb, *solid);
  rcFilterWalkableLowHeightSpans(&ctx, cfg.walkableHeight, *solid);

  rcCompactHeightfield* chf = rcAllocCompactHeightfield();
  if (!rcBuildCompactHeightfield(&ctx, cfg.walkableHeight, cfg.walkableClimb, *solid, *chf)) {
    fprintf(stderr, "rcBuildCompactHeightfield failed\n");
    return 1;
  }
  rcFreeHeightField(solid);
  if (!rcErodeWalkableArea(&ctx, cfg.walkableRadius, *chf)) {
    fprintf(stderr, "rcErodeWalkableArea failed\n");
    return 1;
  }
  if (!rcBuildDistanceField(&ctx, *chf) ||
      !rcBuildRegions(&ctx, *chf, 0, cfg.minRegionArea, cfg.mergeRegionArea)) {
    fprintf(stderr, "region build failed\n");
    return 1;
  }
  rcContourSet* cset = rcAllocContourSet();
  if (!rcBuildContours(&ctx, *chf, cfg.maxSimplificationError, cfg.maxEdgeLen, *cset)) {
    fprintf(stderr, "rcBuildContours failed\n");
    return 1;
  }
  rcPolyMesh* pmesh = rcAllocPolyMesh();
  if (!rcBuildPolyMesh(&ctx, *cset, cfg.maxVertsPerPoly, *pmesh)) {
    fprintf(stderr, "rcBuildPolyMesh failed\n");
    return 1;
  }
  rcPolyMeshDetail* dmesh = rcAllocPolyMeshDetail();
  if (!rcBuildPolyMeshDetail(&ctx, *pmesh, *chf, cfg.detailSampleDist, cfg.detailSampleMaxError,
                             *dmesh)) {
    fprintf(stderr, "rcBuildPolyMeshDetail failed\n");
    return 1;
  }
  rcFreeCompactHeightfield(chf);
  rcFreeContourSet(cset);

  // Every walkable polygon: area 0 (ground), flags 0x01 (walk) -- the only
  // flag esp::nav::PathFinder's filter includes (csrc/PathFinder.cpp:229-243).
  for (int i = 0; i < pmesh->npolys; ++i) {
    if (pmesh->areas[i] == RC_WALKABLE_AREA)
      pmesh->areas[i] = 0;
    pmesh->flags[i] = 0x01;
  }

  dtNavMeshCreateParams params;
  memset(&params, 0, sizeof(params));
  params.verts = pmesh->verts;
  params.vertCount = pmesh->nverts;
  params.polys = pmesh->polys;
  params.polyAreas = pmesh->areas;
  params.polyFlags = pmesh->flags;
  params.polyCount = pmesh->npolys;
  params.nvp = pmesh->nvp;
  params.detailMeshes = dmesh->meshes;
  params.detailVerts = dmesh->verts;
  params.detailVertsCount = dmesh->nverts;
  params.detailTris = dmesh->tris;
  params.detailTriCount = dmesh->ntris;
  params.walkableHeight = agentHeight;
  params.walkableRadius = agentRadius;
  params.walkableClimb = agentClimb;
  rcVcopy(params.bmin, pmesh->bmin);
  rcVcopy(params.bmax, pmesh->bmax);
  params.cs = cfg.cs;
  params.ch = cfg.ch;
  params.buildBvTree = true;

  unsigned char* navData = nullptr;
  int navDataSize = 0;
  if (!dtCreateNavMeshData(&params, &navData, &navDataSize)) {
    fprintf(stderr, "dtCreateNavMeshData failed\n");
    return 1;
  }
  const dtMeshHeader* mh = reinterpret_cast<const dtMeshHeader*>(navData);

  // Single-tile MSET container; the dtNavMeshParams are the ones
  // dtNavMesh::init(data, size, flags) derives for a lone tile
  // (Detour/Source/DetourNavMesh.cpp:267-291): orig = tile bmin, tile extent =
  // tile bounds, maxTiles = 1, maxPolys = polyCount.  tileRef = salt 1, tile 0.
  SetHeader sh;
  sh.magic = 'M' << 24 | 'S' << 16 | 'E' << 8 | 'T';
  sh.version = 1;
  sh.numTiles = 1;
  sh.params.orig[0] = mh->bmin[0];
  sh.params.orig[1] = mh->bmin[1];
  sh.params.orig[2] = mh->bmin[2];
  sh.params.tileWidth = mh->bmax[0] - mh->bmin[0];
  sh.params.tileHeight = mh->bmax[2] - mh->bmin[2];
  sh.params.maxTiles = 1;
  sh.params.maxPolys = mh->polyCount;
  unsigned int polyBits = 0;
  {
    unsigned int v = static_cast<unsigned int>(mh->polyCount);
    unsigned int p2 = 1;
    while (p2 < v)
      p2 <<= 1;
    while ((1u << polyBits) < p2)
      ++polyBits;
  }
  TileHeader th;
  th.tileRef = 1u << polyBits;
  th.dataSize = navDataSize;

  std::string navPath = out + ".navmesh";
  FILE* fp = fopen(navPath.c_str(), "wb");
  if (!fp) {
    fprintf(stderr, "cannot write %s\n", navPath.c_str());
    return 1;
  }
  fwrite(&sh, sizeof(sh), 1, fp);
  fwrite(&th, sizeof(th), 1, fp);
  fwrite(navData, navDataSize, 1, fp);
  fclose(fp);

  std::string jsonPath = out + ".scene.json";
  fp = fopen(jsonPath.c_str(), "w");
  if (fp) {
    fprintf(fp,
            "{\"size_x\": %g, \"size_z\": %g, \"seed\": %llu, \"nvp\": %d, \"num_polys\": %d, "
            "\"num_verts\": %d, \"num_detail_verts\": %d, \"num_detail_tris\": %d, "
            "\"num_bv_nodes\": %d,\n \"recast\": {\"cs\": %g, \"ch\": %g, \"slope\": %g, "
            "\"agent_height\": %g, \"agent_radius\": %g, \"agent_climb\": %g, \"max_edge_len\": "
            "%d, \"max_simplification_error\": %g, \"min_region_area\": %d, "
            "\"merge_region_area\": %d, \"detail_sample_dist\": %g, \"detail_sample_max_error\": "
            "%g},\n \"boxes\": [",
            sx, sz, static_cast<unsigned long long>(seed), nvp, mh->polyCount, mh->vertCount,
            mh->detailVertCount, mh->detailTriCount, mh->bvNodeCount, cfg.cs, cfg.ch,
            cfg.walkableSlopeAngle, agentHeight, agentRadius, agentClimb, cfg.maxEdgeLen,
            cfg.maxSimplificationError, cfg.minRegionArea, cfg.mergeRegionArea,
            cfg.detailSampleDist, cfg.detailSampleMaxError);
    for (size_t i = 0; i < boxes.size(); ++i) {
      fprintf(fp, "%s[%.6f, %.6f, %.6f, %.6f, %.6f, %.6f]", i ? ", " : "", boxes[i].mn[0],
              boxes[i].mn[1], boxes[i].mn[2], boxes[i].mx[0], boxes[i].mx[1], boxes[i].mx[2]);
    }
    fprintf(fp, "]}\n");
    fclose(fp);
  }
  printf("%s: %d polys, %d verts, %d bytes\n", navPath.c_str(), mh->polyCount, mh->vertCount,
         navDataSize);
  dtFree(navData);
  rcFreePolyMesh(pmesh);
  rcFreePolyMeshDetail(dmesh);
  return 0;
}
