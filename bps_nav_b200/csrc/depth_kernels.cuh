// Headless depth sensor for box-world scenes.
//
// The reference renders its observations with bps3D, a Vulkan rasteriser that is
// not part of its source tree; what the tree fixes is the camera: per environment
// view = transpose(mat3(rotation)) about eye = position + 1.25 * up, looking down
// -Z (simulator/simulator.cpp:651-663), vertical field of view 90 degrees, near
// plane 0.1, far plane 1000 (makeEnvironment(scene, I, 90.f, 0.f, 0.1, 1000),
// :1216), image [H, W] float32 per environment (simulator/pytorch.cpp:36-44).
// For scenes that are given as a floor rectangle plus axis-aligned boxes the same
// camera is evaluated here analytically: one ray per pixel centre, ray / plane for
// the floor, slab test for every box that reaches into the view frustum, nearest hit.  The value is the view-space
// depth in metres (distance along the optical axis), `far` where nothing is hit;
// hits in front of the near plane are clipped.
//
// Arithmetic: plain fp32, one rounding per operation (the library is compiled
// without FMA contraction), IEEE division, so a restatement with the same
// operation order in fp32 numpy reproduces the image bit for bit.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "sim_kernels.cuh"

namespace bpsn {

constexpr float kEyeHeight = 1.25f;  // simulator.cpp:659
constexpr float kNearPlane = 0.1f;   // :1216
constexpr float kFarPlane = 1000.f;
constexpr int kDepthBoxChunk = 256;  // boxes staged in shared memory at a time

struct RenderTable {
  const float* boxes;         // 6 floats per box (min xyz, max xyz), all scenes concatenated
  const uint32_t* boxOffset;  // [numScenes]
  const uint32_t* boxCount;   // [numScenes]
  const float* floor;         // [numScenes][4]: xmin, zmin, xmax, zmax of the floor at y = 0
};

// grid = environments of the group, block = 256 threads striding over the pixels
__global__ void __launch_bounds__(256)
k_depth(GroupDev g, RenderTable rt, float* __restrict__ out, uint32_t W, uint32_t H) {
  __shared__ float sBox[kDepthBoxChunk * 6];
  const uint32_t e = blockIdx.x;
  const uint32_t B = g.B;
  const uint32_t sceneIdx = g.scene[e];
  const float qx = g.rot[e], qy = g.rot[B + e], qz = g.rot[2 * B + e], qw = g.rot[3 * B + e];
  const float ox = g.pos[e], oy = g.pos[B + e] + kEyeHeight, oz = g.pos[2 * B + e];
  // mat3_cast(rotation): columns are the camera axes in world space
  const float qxx = qx * qx, qyy = qy * qy, qzz = qz * qz;
  const float qxz = qx * qz, qxy = qx * qy, qyz = qy * qz;
  const float qwx = qw * qx, qwy = qw * qy, qwz = qw * qz;
  const float m00 = 1.f - 2.f * (qyy + qzz), m01 = 2.f * (qxy + qwz), m02 = 2.f * (qxz - qwy);
  const float m10 = 2.f * (qxy - qwz), m11 = 1.f - 2.f * (qxx + qzz), m12 = 2.f * (qyz + qwx);
  const float m20 = 2.f * (qxz + qwy), m21 = 2.f * (qyz - qwx), m22 = 1.f - 2.f * (qxx + qyy);
  const float fxmin = rt.floor[4 * sceneIdx + 0], fzmin = rt.floor[4 * sceneIdx + 1];
  const float fxmax = rt.floor[4 * sceneIdx + 2], fzmax = rt.floor[4 * sceneIdx + 3];
  const uint32_t nb = rt.boxCount[sceneIdx];
  const float* boxes = rt.boxes + 6 * static_cast<size_t>(rt.boxOffset[sceneIdx]);
  const float aspect = static_cast<float>(W) / static_cast<float>(H);
  const uint32_t npix = W * H;
  float* img = out + static_cast<size_t>(e) * npix;

  // Of the scene's first kDepthBoxChunk boxes only those that reach into the view frustum
  // are staged in shared memory (every thread then walks them in the same order: broadcast
  // reads); any boxes beyond that number are read from global memory, unculled.  A box is
  // dropped when all its corners lie outside one of the five planes through the eye that
  // bound the image (behind the near plane, beyond the left / right / top / bottom edge,
  // with a millimetre of slack: pixel centres stay half a pixel inside those edges), so
  // no ray of the image can touch it and the image is the same as without culling.  The
  // order of the survivors does not matter: the nearest hit is a minimum.
  __shared__ uint32_t sCount;
  const uint32_t first = nb < static_cast<uint32_t>(kDepthBoxChunk)
                             ? nb : static_cast<uint32_t>(kDepthBoxChunk);
  if (threadIdx.x == 0)
    sCount = 0u;
  __syncthreads();
  for (uint32_t b = threadIdx.x; b < first; b += blockDim.x) {
    const float* bx = boxes + 6 * static_cast<size_t>(b);
    const float mn[3] = {bx[0], bx[1], bx[2]}, mx[3] = {bx[3], bx[4], bx[5]};
    bool allNear = true, allLeft = true, allRight = true, allUp = true, allDown = true;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float px = ((c & 1) ? mx[0] : mn[0]) - ox;
      const float py = ((c & 2) ? mx[1] : mn[1]) - oy;
      const float pz = ((c & 4) ? mx[2] : mn[2]) - oz;
      // camera space: x right, y up, depth along the optical axis (-z)
      const float cx = m00 * px + m01 * py + m02 * pz;
      const float cy = m10 * px + m11 * py + m12 * pz;
      const float depth = -(m20 * px + m21 * py + m22 * pz);
      const float slack = 1e-3f;
      allNear = allNear && (kNearPlane - depth > slack);
      allRight = allRight && (cx - aspect * depth > slack);
      allLeft = allLeft && (-cx - aspect * depth > slack);
      allUp = allUp && (cy - depth > slack);
      allDown = allDown && (-cy - depth > slack);
    }
    if (!(allNear || allLeft || allRight || allUp || allDown)) {
      const uint32_t slot = atomicAdd(&sCount, 1u);
#pragma unroll
      for (int k = 0; k < 6; ++k)
        sBox[6 * slot + k] = bx[k];
    }
  }
  __syncthreads();
  const uint32_t staged = sCount;
  for (uint32_t pix = threadIdx.x; pix < npix; pix += blockDim.x) {
    const uint32_t px = pix % W, py = pix / W;
    // pixel centre -> camera-space direction with z = -1 (tan(45 deg) = 1)
    const float u = ((static_cast<float>(px) + 0.5f) / static_cast<float>(W) * 2.f - 1.f) * aspect;
    const float v = 1.f - (static_cast<float>(py) + 0.5f) / static_cast<float>(H) * 2.f;
    // world direction = R * (u, v, -1); a ray parameter t is then the view-space depth
    const float dx = (m00 * u + m10 * v) - m20;
    const float dy = (m01 * u + m11 * v) - m21;
    const float dz = (m02 * u + m12 * v) - m22;
    float t = kFarPlane;
    if (dy < 0.f) {  // floor plane y = 0
      const float tf = (0.f - oy) / dy;
      const float hx = ox + tf * dx, hz = oz + tf * dz;
      if (tf >= kNearPlane && tf < t && hx >= fxmin && hx <= fxmax && hz >= fzmin && hz <= fzmax)
        t = tf;
    }
    const float ix = 1.f / dx, iy = 1.f / dy, iz = 1.f / dz;
    const uint32_t total = staged + (nb - first);  // survivors, then the unculled rest
    for (uint32_t b = 0; b < total; ++b) {
      const float* bx = b < staged ? &sBox[6 * b]
                                   : &boxes[6 * static_cast<size_t>(first + (b - staged))];
      const float tx0 = (bx[0] - ox) * ix, tx1 = (bx[3] - ox) * ix;
      const float ty0 = (bx[1] - oy) * iy, ty1 = (bx[4] - oy) * iy;
      const float tz0 = (bx[2] - oz) * iz, tz1 = (bx[5] - oz) * iz;
      // slab test; fminf / fmaxf drop a NaN operand (0 * inf on a face the ray grazes)
      const float tenter = fmaxf(fmaxf(fminf(tx0, tx1), fminf(ty0, ty1)), fminf(tz0, tz1));
      const float texit = fminf(fminf(fmaxf(tx0, tx1), fmaxf(ty0, ty1)), fmaxf(tz0, tz1));
      if (tenter <= texit && tenter >= kNearPlane && tenter < t)
        t = tenter;
    }
    img[pix] = t;
  }
}

}  // namespace bpsn
