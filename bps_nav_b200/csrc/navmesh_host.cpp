// `.navmesh` reader and flattener (host).
//
// Input format = what esp::nav::PathFinder::loadNavMesh reads
// (csrc/PathFinder.cpp:258-272, 330-408): a 40-byte NavMeshSetHeader
// {magic 'MSET', version 1, numTiles, dtNavMeshParams}, then per tile an
// 8-byte {tileRef, dataSize} header and a Detour tile blob whose sections are
// laid out as dtNavMesh::addTile expects
// (recastnavigation-master/Detour/Source/DetourNavMesh.cpp:970-989).
//
// After parsing, two load-time passes of the reference are applied so the
// kernels see the same mesh its queries see:
//   * polygons whose detail-mesh area is below 1e-5 get flags = DISABLED
//     (PathFinder::Impl::removeZeroAreaPolys, PathFinder.cpp:307-328, area
//     arithmetic :275-302);
//   * connected components over passable links give an island id per polygon
//     (impl::IslandSystem, PathFinder.cpp:53-170), same visiting order.
//
// Only single-tile meshes are accepted (what Recast's solo build and
// habitat-sim produce); a second non-empty tile is reported as an error.

#include "navmesh_host.h"

#include <math.h>
#include <string.h>

namespace bpsn {

namespace {

struct SetHeader {
  int32_t magic;
  int32_t version;
  int32_t numTiles;
  float orig[3];
  float tileWidth;
  float tileHeight;
  int32_t maxTiles;
  int32_t maxPolys;
};
static_assert(sizeof(SetHeader) == 40, "MSET header is 40 bytes");

struct TileHeader {
  uint32_t tileRef;
  int32_t dataSize;
};

struct MeshHeader {  // dtMeshHeader, 100 bytes
  int32_t magic;
  int32_t version;
  int32_t x, y, layer;
  uint32_t userId;
  int32_t polyCount;
  int32_t vertCount;
  int32_t maxLinkCount;
  int32_t detailMeshCount;
  int32_t detailVertCount;
  int32_t detailTriCount;
  int32_t bvNodeCount;
  int32_t offMeshConCount;
  int32_t offMeshBase;
  float walkableHeight;
  float walkableRadius;
  float walkableClimb;
  float bmin[3];
  float bmax[3];
  float bvQuantFactor;
};
static_assert(sizeof(MeshHeader) == 100, "dtMeshHeader is 100 bytes");

struct RawPoly {  // dtPoly, 32 bytes
  uint32_t firstLink;
  uint16_t verts[6];
  uint16_t neis[6];
  uint16_t flags;
  uint8_t vertCount;
  uint8_t areaAndtype;
};
static_assert(sizeof(RawPoly) == 32, "dtPoly is 32 bytes");

struct RawDetail {  // dtPolyDetail, 12 bytes
  uint32_t vertBase;
  uint32_t triBase;
  uint8_t vertCount;
  uint8_t triCount;
};
static_assert(sizeof(RawDetail) == 12, "dtPolyDetail is 12 bytes");

constexpr int32_t kSetMagic = 'M' << 24 | 'S' << 16 | 'E' << 8 | 'T';
constexpr int32_t kNavMagic = 'D' << 24 | 'N' << 16 | 'A' << 8 | 'V';
constexpr int32_t kNavVersion = 7;

inline size_t align4(size_t x) {
  return (x + 3) & ~static_cast<size_t>(3);
}

inline uint32_t nextPow2(uint32_t v) {
  v--;
  v |= v >> 1;
  v |= v >> 2;
  v |= v >> 4;
  v |= v >> 8;
  v |= v >> 16;
  v++;
  return v;
}

inline uint32_t ilog2(uint32_t v) {
  uint32_t r = 0;
  while (v > 1) {
    v >>= 1;
    ++r;
  }
  return r;
}

}  // namespace

NavScene HostScene::view() const {
  NavScene s;
  s.verts = verts.data();
  s.polys = polys.data();
  s.detail = detail.data();
  s.dverts = dverts.data();
  s.dtris = dtris.data();
  s.bv = bv.data();
  s.island = island.data();
  s.staged = nullptr;
  s.stagedBytes = 0;
  s.npolys = static_cast<int32_t>(polys.size());
  s.nverts = static_cast<int32_t>(verts.size() / 3);
  s.nbv = static_cast<int32_t>(bv.size());
  s.ndverts = static_cast<int32_t>(dverts.size() / 3);
  s.ndtris = static_cast<int32_t>(dtris.size() / 4) - 1;  // the array carries one padding entry
  s.vstride = 3;
  s.refBase = refBase;
  s.polyMask = polyMask;
  for (int k = 0; k < 3; ++k) {
    s.bmin[k] = bmin[k];
    s.bmax[k] = bmax[k];
    s.orig[k] = orig[k];
  }
  s.bvQuantFactor = bvQuantFactor;
  s.walkableClimb = walkableClimb;
  s.tileWidth = tileWidth;
  s.tileHeight = tileHeight;
  s.tileX = tileX;
  s.tileY = tileY;
  return s;
}

std::string parseNavmesh(const void* data, size_t size, HostScene* out) {
  const uint8_t* p = static_cast<const uint8_t*>(data);
  if (!p || size < sizeof(SetHeader))
    return "navmesh: file shorter than the MSET header";
  SetHeader sh;
  memcpy(&sh, p, sizeof(sh));
  if (sh.magic != kSetMagic)
    return "navmesh: bad MSET magic";
  if (sh.version != 1)
    return "navmesh: unsupported MSET version";
  if (sh.maxTiles < 1 || sh.maxPolys < 1)
    return "navmesh: maxTiles/maxPolys must be positive";

  const uint32_t tileBits = ilog2(nextPow2(static_cast<uint32_t>(sh.maxTiles)));
  const uint32_t polyBits = ilog2(nextPow2(static_cast<uint32_t>(sh.maxPolys)));
  if (tileBits + polyBits > 22)
    return "navmesh: fewer than 10 salt bits (dtNavMesh::init would fail)";
  const uint32_t saltBits = (32 - tileBits - polyBits) < 31 ? (32 - tileBits - polyBits) : 31;

  size_t off = sizeof(SetHeader);
  bool haveTile = false;
  for (int t = 0; t < sh.numTiles; ++t) {
    if (off + sizeof(TileHeader) > size)
      return "navmesh: truncated tile header";
    TileHeader th;
    memcpy(&th, p + off, sizeof(th));
    off += sizeof(th);
    if (!th.tileRef || !th.dataSize)
      break;  // loader stops at the first empty tile
    if (th.dataSize < static_cast<int32_t>(sizeof(MeshHeader)) ||
        off + static_cast<size_t>(th.dataSize) > size)
      return "navmesh: truncated tile data";
    if (haveTile)
      return "navmesh: multi-tile meshes are not supported";
    haveTile = true;

    const uint8_t* d = p + off;
    off += static_cast<size_t>(th.dataSize);
    MeshHeader mh;
    memcpy(&mh, d, sizeof(mh));
    if (mh.magic != kNavMagic)
      return "navmesh: bad tile magic";
    if (mh.version != kNavVersion)
      return "navmesh: unsupported tile version";
    if (mh.polyCount < 1 || mh.vertCount < 3 || mh.detailMeshCount != mh.polyCount ||
        mh.maxLinkCount < 0 || mh.detailVertCount < 0 || mh.detailTriCount < 0 ||
        mh.bvNodeCount < 0 || mh.offMeshConCount < 0)
      return "navmesh: inconsistent tile header counts";
    if (mh.offMeshConCount != 0)
      return "navmesh: off-mesh connections are not supported";
    if (static_cast<uint32_t>(mh.polyCount) > (1u << polyBits))
      return "navmesh: polyCount exceeds maxPolys";

    const size_t vertsSize = align4(sizeof(float) * 3 * mh.vertCount);
    const size_t polysSize = align4(sizeof(RawPoly) * mh.polyCount);
    const size_t linksSize = align4(12 * static_cast<size_t>(mh.maxLinkCount));
    const size_t dmeshSize = align4(sizeof(RawDetail) * mh.detailMeshCount);
    const size_t dvertsSize = align4(sizeof(float) * 3 * mh.detailVertCount);
    const size_t dtrisSize = align4(4 * static_cast<size_t>(mh.detailTriCount));
    const size_t bvSize = align4(sizeof(NavBVNode) * mh.bvNodeCount);
    const size_t need = align4(sizeof(MeshHeader)) + vertsSize + polysSize + linksSize +
                        dmeshSize + dvertsSize + dtrisSize + bvSize;
    if (need > static_cast<size_t>(th.dataSize))
      return "navmesh: tile sections exceed tile size";

    const uint8_t* q = d + align4(sizeof(MeshHeader));
    out->verts.resize(3 * static_cast<size_t>(mh.vertCount));
    memcpy(out->verts.data(), q, sizeof(float) * out->verts.size());
    q += vertsSize;
    std::vector<RawPoly> raw(mh.polyCount);
    memcpy(raw.data(), q, sizeof(RawPoly) * raw.size());
    q += polysSize;
    q += linksSize;  // link records are rebuilt at load time by the reference; not needed
    std::vector<RawDetail> rawd(mh.detailMeshCount);
    memcpy(rawd.data(), q, sizeof(RawDetail) * rawd.size());
    q += dmeshSize;
    out->dverts.resize(3 * static_cast<size_t>(mh.detailVertCount));
    if (!out->dverts.empty())
      memcpy(out->dverts.data(), q, sizeof(float) * out->dverts.size());
    q += dvertsSize;
    // +4 bytes of padding so a 4-byte load of the last triangle is in bounds
    out->dtris.assign(4 * static_cast<size_t>(mh.detailTriCount) + 4, 0);
    if (mh.detailTriCount)
      memcpy(out->dtris.data(), q, 4 * static_cast<size_t>(mh.detailTriCount));
    q += dtrisSize;
    out->bv.resize(mh.bvNodeCount);
    if (mh.bvNodeCount)
      memcpy(out->bv.data(), q, sizeof(NavBVNode) * out->bv.size());

    // validate every index the kernels will follow
    out->polys.resize(mh.polyCount);
    out->detail.resize(mh.polyCount);
    for (int i = 0; i < mh.polyCount; ++i) {
      const RawPoly& r = raw[i];
      NavPoly& np = out->polys[i];
      memset(&np, 0, sizeof(np));
      if (r.vertCount < 3 || r.vertCount > kVertsPerPoly)
        return "navmesh: polygon vertex count out of range";
      if ((r.areaAndtype >> 6) != 0)
        return "navmesh: off-mesh polygon types are not supported";
      for (int j = 0; j < r.vertCount; ++j) {
        if (r.verts[j] >= mh.vertCount)
          return "navmesh: polygon vertex index out of range";
        np.verts[j] = r.verts[j];
        const uint16_t ne = r.neis[j];
        if (ne && !(ne & kExtLink) && (ne - 1) >= mh.polyCount)
          return "navmesh: neighbour index out of range";
        np.neis[j] = ne;
      }
      np.flags = r.flags;
      np.vertCount = r.vertCount;
      np.areaAndType = r.areaAndtype;
      const RawDetail& rd = rawd[i];
      if (static_cast<size_t>(rd.triBase) + rd.triCount > static_cast<size_t>(mh.detailTriCount) ||
          static_cast<size_t>(rd.vertBase) + rd.vertCount >
              static_cast<size_t>(mh.detailVertCount))
        return "navmesh: detail mesh range out of bounds";
      np.detailVertCount = rd.vertCount;
      np.detailTriCount = rd.triCount;
      out->detail[i].vertBase = rd.vertBase;
      out->detail[i].triBase = rd.triBase;
      for (int k = 0; k < rd.triCount; ++k) {
        const uint8_t* tri = &out->dtris[4 * (static_cast<size_t>(rd.triBase) + k)];
        for (int c = 0; c < 3; ++c)
          if (tri[c] >= r.vertCount + rd.vertCount)
            return "navmesh: detail triangle vertex out of range";
      }
    }
    for (int i = 0; i < mh.bvNodeCount; ++i) {
      const NavBVNode& n = out->bv[i];
      if (n.i >= mh.polyCount)
        return "navmesh: BV leaf index out of range";
    }

    const uint32_t tileMask = (1u << tileBits) - 1;
    const uint32_t saltMask = saltBits >= 32 ? 0xffffffffu : ((1u << saltBits) - 1);
    const uint32_t tileIdx = (th.tileRef >> polyBits) & tileMask;
    const uint32_t salt = (th.tileRef >> (polyBits + tileBits)) & saltMask;
    if (tileIdx >= static_cast<uint32_t>(sh.maxTiles))
      return "navmesh: tile index out of range";
    out->refBase = (salt << (polyBits + tileBits)) | (tileIdx << polyBits);
    out->polyMask = (1u << polyBits) - 1;
    for (int k = 0; k < 3; ++k) {
      out->bmin[k] = mh.bmin[k];
      out->bmax[k] = mh.bmax[k];
      out->orig[k] = sh.orig[k];
    }
    out->bvQuantFactor = mh.bvQuantFactor;
    out->walkableClimb = mh.walkableClimb;
    out->tileWidth = sh.tileWidth;
    out->tileHeight = sh.tileHeight;
    out->tileX = mh.x;
    out->tileY = mh.y;
  }
  if (!haveTile)
    return "navmesh: no tile data";

  // ---- zero-area polygons -> DISABLED
  const int npolys = static_cast<int>(out->polys.size());
  out->numDisabled = 0;
  for (int i = 0; i < npolys; ++i) {
    NavPoly& poly = out->polys[i];
    const NavDetail& pd = out->detail[i];
    float area = 0;
    for (int j = 0; j < poly.detailTriCount; ++j) {
      const uint8_t* t = &out->dtris[4 * (static_cast<size_t>(pd.triBase) + j)];
      const float* v[3];
      for (int k = 0; k < 3; ++k) {
        if (t[k] < poly.vertCount)
          v[k] = &out->verts[3 * static_cast<size_t>(poly.verts[t[k]])];
        else
          v[k] = &out->dverts[3 * (static_cast<size_t>(pd.vertBase) + (t[k] - poly.vertCount))];
      }
      const float w1[3] = {v[1][0] - v[0][0], v[1][1] - v[0][1], v[1][2] - v[0][2]};
      const float w2[3] = {v[2][0] - v[0][0], v[2][1] - v[0][1], v[2][2] - v[0][2]};
      const float cx = w1[1] * w2[2] - w1[2] * w2[1];
      const float cy = w1[2] * w2[0] - w1[0] * w2[2];
      const float cz = w1[0] * w2[1] - w1[1] * w2[0];
      const float nrm = sqrtf(cx * cx + (cy * cy + cz * cz));
      area = static_cast<float>(static_cast<double>(area) + 0.5 * static_cast<double>(nrm));
    }
    if (static_cast<double>(area) < 1e-5) {
      poly.flags = kFlagDisabled;
      out->numDisabled++;
    }
  }

  // ---- islands
  out->island.assign(npolys, -1);
  int nIslands = 0;
  std::vector<int> stack;
  for (int s = 0; s < npolys; ++s) {
    if (out->island[s] >= 0)
      continue;
    const int id = nIslands++;
    out->island[s] = id;
    stack.clear();
    stack.push_back(s);
    while (!stack.empty()) {
      const int cur = stack.back();
      stack.pop_back();
      const NavPoly& poly = out->polys[cur];
      for (int j = 0; j < poly.vertCount; ++j) {
        const uint16_t ne = poly.neis[j];
        if (!ne || (ne & kExtLink))
          continue;
        const int nb = ne - 1;
        if (out->island[nb] >= 0)
          continue;
        if ((out->polys[nb].flags & kFlagWalk) == 0)
          continue;
        out->island[nb] = id;
        stack.push_back(nb);
      }
    }
  }
  out->numIslands = nIslands;
  return std::string();
}

}  // namespace bpsn
