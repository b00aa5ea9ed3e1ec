// Host-side loader: `.navmesh` (MSET container of Detour tiles) -> flat arrays
// ready to upload as a bpsn::NavScene.
#pragma once

#include <stddef.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "nav_types.h"

namespace bpsn {

struct HostScene {
  std::vector<float> verts;
  std::vector<NavPoly> polys;
  std::vector<NavDetail> detail;
  std::vector<float> dverts;
  std::vector<uint8_t> dtris;
  std::vector<NavBVNode> bv;
  std::vector<int32_t> island;
  uint32_t refBase = 0;
  uint32_t polyMask = 0;
  float bmin[3] = {0, 0, 0};
  float bmax[3] = {0, 0, 0};
  float bvQuantFactor = 0;
  float walkableClimb = 0;
  float orig[3] = {0, 0, 0};
  float tileWidth = 0;
  float tileHeight = 0;
  int32_t tileX = 0;
  int32_t tileY = 0;
  int32_t numDisabled = 0;
  int32_t numIslands = 0;

  // View over the host arrays (for host-side checks of the query code).
  NavScene view() const;
};

// Parses an in-memory `.navmesh` file.  Returns an empty string on success,
// else a description of what is wrong with the input.  Never aborts.
std::string parseNavmesh(const void* data, size_t size, HostScene* out);

}  // namespace bpsn
