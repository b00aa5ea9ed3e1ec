// Rollout returns: generalised advantage estimation as one reverse scan per
// environment column, fused with the advantage (returns - values) and the
// statistics for whole-batch normalisation.
//
// Follows RolloutStorage.compute_returns (bps_nav/common/rollout_storage.py:
// 203-219) and PPO.get_advantages (bps_nav/rl/ppo/ppo.py:190-201).  The float
// expression tree is the one PyTorch evaluates for those lines, each op
// rounded to fp32 on its own (compile without FMA contraction):
//     delta = (r[t] + (gamma * v[t+1]) * m[t+1]) - v[t]
//     gae   = delta + ((gamma*tau) * gae) * m[t+1]      gamma*tau folded in double
//     ret   = gae + v[t]
//     adv   = ret - v[t]
// Normalisation: (adv - mean) / (std + eps), std unbiased over T*N elements;
// per-thread sums and sums of squares are accumulated in double, turned into
// (count, mean, M2) and merged with Chan's pairwise formula, so the statistics
// are at least as accurate as the fp32 reductions of the reference.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace bpsn {

struct GaeStat {  // running (count, mean, M2)
  double n;
  double mean;
  double m2;
};

__device__ __forceinline__ GaeStat gaeMerge(const GaeStat& a, const GaeStat& b) {
  if (b.n == 0.0)
    return a;
  if (a.n == 0.0)
    return b;
  GaeStat r;
  r.n = a.n + b.n;
  const double delta = b.mean - a.mean;
  r.mean = a.mean + delta * (b.n / r.n);
  r.m2 = a.m2 + b.m2 + delta * delta * (a.n * b.n / r.n);
  return r;
}

__device__ __forceinline__ GaeStat gaeWarpReduce(GaeStat s) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    GaeStat o;
    o.n = __shfl_down_sync(0xffffffffu, s.n, off);
    o.mean = __shfl_down_sync(0xffffffffu, s.mean, off);
    o.m2 = __shfl_down_sync(0xffffffffu, s.m2, off);
    s = gaeMerge(s, o);
  }
  return s;
}

constexpr int kGaeBlock = 128;

// Programmatic dependent launch of the normalisation behind the scan: the scan lets its
// dependent become resident at once, the normalisation waits for the whole of the scan (and
// its stores) before it reads anything.  Both instructions are no-ops for an ordinary launch.
__device__ __forceinline__ void gaeLaunchDependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void gaeWaitForPredecessor() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// One thread per environment column.  partials[blockIdx.x] receives the
// block's advantage statistics when `partials` is non-null.
__global__ void __launch_bounds__(kGaeBlock)
k_gae_scan(const float* __restrict__ rewards, float* __restrict__ values,
           const uint8_t* __restrict__ masks, const float* __restrict__ nextValue,
           float* __restrict__ returns, float* __restrict__ adv, uint32_t T, uint32_t N,
           float gamma, float gammaTau, GaeStat* __restrict__ partials) {
  gaeLaunchDependents();
  const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
  GaeStat st;
  st.n = 0.0;
  st.mean = 0.0;
  st.m2 = 0.0;
  if (n < N) {
    float vnext;
    if (nextValue) {
      vnext = nextValue[n];
      values[static_cast<size_t>(T) * N + n] = vnext;
    } else {
      vnext = values[static_cast<size_t>(T) * N + n];
    }
    float gae = 0.f;
    // The recurrence is a 4-flop dependent chain; the cost is load latency.  Rows are
    // fetched kChunk at a time (independent loads, all in flight together) and then
    // scanned from registers (T = 32 takes two rounds of memory latency).  Statistics: plain sums in double (131 072 values of
    // order 1 lose nothing in 53 bits), turned into (n, mean, M2) once per thread.
    constexpr int kChunk = 16;
    double sum = 0.0, sumSq = 0.0;
    int count = 0;
    for (int hi = static_cast<int>(T); hi > 0; hi -= kChunk) {
      float r[kChunk], v[kChunk];
      uint8_t mb[kChunk];
      // Nothing in this loop looks at a loaded value and rows past the start are read
      // from row 0 instead of being skipped, so the 3 * kChunk loads carry no branch and
      // are all in flight before the first one is needed.
#pragma unroll
      for (int k = 0; k < kChunk; ++k) {
        const int t = hi - 1 - k;
        const size_t i = static_cast<size_t>(t > 0 ? t : 0) * N + n;
        r[k] = rewards[i];
        v[k] = values[i];
        mb[k] = masks[i + N];
      }
#pragma unroll
      for (int k = 0; k < kChunk; ++k) {
        const int t = hi - 1 - k;
        if (t >= 0) {
          const size_t i = static_cast<size_t>(t) * N + n;
          const float m = mb[k] ? 1.f : 0.f;
          const float delta = (r[k] + (gamma * vnext) * m) - v[k];
          gae = delta + (gammaTau * gae) * m;
          const float ret = gae + v[k];
          returns[i] = ret;
          if (adv) {
            const float a = ret - v[k];
            adv[i] = a;
            sum += static_cast<double>(a);
            sumSq += static_cast<double>(a) * static_cast<double>(a);
            ++count;
          }
          vnext = v[k];
        }
      }
    }
    if (count > 0) {
      st.n = static_cast<double>(count);
      st.mean = sum / st.n;
      const double m2 = sumSq - sum * st.mean;
      st.m2 = m2 > 0.0 ? m2 : 0.0;
    }
  }
  if (partials) {
    __shared__ GaeStat sh[kGaeBlock / 32];
    st = gaeWarpReduce(st);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0)
      sh[warp] = st;
    __syncthreads();
    if (threadIdx.x == 0) {
      GaeStat acc = sh[0];
      for (int w = 1; w < kGaeBlock / 32; ++w)
        acc = gaeMerge(acc, sh[w]);
      partials[blockIdx.x] = acc;
    }
  }
}

// Every block merges the (few) partials itself, then normalises its slice.
__global__ void __launch_bounds__(256)
k_gae_normalize(float* __restrict__ adv, size_t total, const GaeStat* __restrict__ partials,
                uint32_t numPartials, float eps) {
  __shared__ float sMean, sInv;
  __shared__ GaeStat sWarp[8];
  gaeWaitForPredecessor();
  {
    // every thread merges a share of the block partials, the warps' results are merged by
    // thread 0 (a chain of numPartials / 256 + 5 + 8 merges instead of numPartials / 32 + 5)
    GaeStat st;
    st.n = 0.0;
    st.mean = 0.0;
    st.m2 = 0.0;
    for (uint32_t i = threadIdx.x; i < numPartials; i += blockDim.x)
      st = gaeMerge(st, partials[i]);
    st = gaeWarpReduce(st);
    if ((threadIdx.x & 31u) == 0u)
      sWarp[threadIdx.x >> 5] = st;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (uint32_t w = 1; w < (blockDim.x >> 5); ++w)
        st = gaeMerge(st, sWarp[w]);
      const double var = st.n > 1.0 ? st.m2 / (st.n - 1.0) : __longlong_as_double(0x7ff8000000000000ll);
      const float mean = static_cast<float>(st.mean);
      const float sd = static_cast<float>(sqrt(var));
      sMean = mean;
      sInv = sd + eps;
    }
  }
  __syncthreads();
  const float mean = sMean, denom = sInv;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t first = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if ((reinterpret_cast<uintptr_t>(adv) & 15u) == 0u) {
    // 16 bytes per access and four independent accesses in flight per thread: a plain
    // element-by-element loop waits for each load before it issues the next (the store to the
    // same array in between keeps the compiler from moving loads up)
    float4* a4 = reinterpret_cast<float4*>(adv);
    const size_t nvec = total / 4;
    for (size_t i = first; i < nvec; i += 4 * stride) {
      float4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (i + k * stride < nvec)
          v[k] = a4[i + k * stride];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (i + k * stride < nvec) {
          v[k].x = (v[k].x - mean) / denom;
          v[k].y = (v[k].y - mean) / denom;
          v[k].z = (v[k].z - mean) / denom;
          v[k].w = (v[k].w - mean) / denom;
          a4[i + k * stride] = v[k];
        }
    }
    for (size_t i = nvec * 4 + first; i < total; i += stride)
      adv[i] = (adv[i] - mean) / denom;
  } else {
    for (size_t i = first; i < total; i += stride)
      adv[i] = (adv[i] - mean) / denom;
  }
}

// ---------------------------------------------------------------------------
// Advantage normalisation over segments.  A segment is a range of environment
// columns [start, end) of one [T, N] advantage tensor; segments that carry the
// same group number are normalised together, over all of their elements:
//   * one segment covering the batch      -> PPO.get_advantages (ppo.py:190-201);
//   * the two halves of a double-buffered rollout in one group -> the same call
//     on the concatenation the reference builds with torch.cat(advantages, 1);
//   * one group per range of environments -> per-minibatch statistics.
// Passed to the kernels by value (no device copy of the list).
constexpr int kMaxAdvSegments = 64;
constexpr int kAdvBlock = 256;

struct AdvSegment {
  float* adv;       // [T, N] row-major
  uint32_t N;       // row length of that tensor
  uint32_t start;   // first environment column
  uint32_t end;     // one past the last
  uint32_t group;   // segments with equal numbers share mean and std
};
struct AdvSegmentList {
  AdvSegment seg[kMaxAdvSegments];
  uint32_t count;
  uint32_t blocksPerSeg;
  uint32_t T;
};

// element i of a segment: row i / width, column start + i % width
__device__ __forceinline__ size_t advIndex(const AdvSegment& sg, uint32_t width, size_t i) {
  const size_t row = i / width;
  return row * sg.N + sg.start + (i - row * width);
}

// grid (blocksPerSeg, count): partials[seg * blocksPerSeg + block] <- (n, mean, M2) of the
// block's share of the segment
__global__ void __launch_bounds__(kAdvBlock)
k_adv_stats(const AdvSegmentList L, GaeStat* __restrict__ partials) {
  const AdvSegment sg = L.seg[blockIdx.y];
  const uint32_t width = sg.end - sg.start;
  const size_t total = static_cast<size_t>(L.T) * width;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  double sum = 0.0, sumSq = 0.0;
  unsigned long long count = 0;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const double a = static_cast<double>(sg.adv[advIndex(sg, width, i)]);
    sum += a;
    sumSq += a * a;
    ++count;
  }
  GaeStat st;
  st.n = static_cast<double>(count);
  st.mean = count ? sum / st.n : 0.0;
  const double m2 = count ? sumSq - sum * st.mean : 0.0;
  st.m2 = m2 > 0.0 ? m2 : 0.0;
  __shared__ GaeStat sh[kAdvBlock / 32];
  st = gaeWarpReduce(st);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0)
    sh[warp] = st;
  __syncthreads();
  if (threadIdx.x == 0) {
    GaeStat acc = sh[0];
    for (int w = 1; w < kAdvBlock / 32; ++w)
      acc = gaeMerge(acc, sh[w]);
    partials[blockIdx.y * gridDim.x + blockIdx.x] = acc;
  }
}

// statistics of the group the block's segment belongs to (first warp; result in lane 0)
__device__ __forceinline__ GaeStat advGroupStat(const AdvSegmentList& L, uint32_t group,
                                                const GaeStat* __restrict__ partials) {
  GaeStat st;
  st.n = 0.0;
  st.mean = 0.0;
  st.m2 = 0.0;
  for (uint32_t s = 0; s < L.count; ++s) {
    if (L.seg[s].group != group)
      continue;
    for (uint32_t b = threadIdx.x; b < L.blocksPerSeg; b += 32)
      st = gaeMerge(st, partials[s * L.blocksPerSeg + b]);
  }
  return gaeWarpReduce(st);
}

// mode 0: (a - mean) / (std + eps), unbiased std, per group
__global__ void __launch_bounds__(kAdvBlock)
k_adv_normalize(const AdvSegmentList L, const GaeStat* __restrict__ partials, float eps) {
  const AdvSegment sg = L.seg[blockIdx.y];
  __shared__ float sMean, sDenom;
  if (threadIdx.x < 32) {
    const GaeStat st = advGroupStat(L, sg.group, partials);
    if (threadIdx.x == 0) {
      const double var =
          st.n > 1.0 ? st.m2 / (st.n - 1.0) : __longlong_as_double(0x7ff8000000000000ll);
      sMean = static_cast<float>(st.mean);
      sDenom = static_cast<float>(sqrt(var)) + eps;
    }
  }
  __syncthreads();
  const float mean = sMean, denom = sDenom;
  const uint32_t width = sg.end - sg.start;
  const size_t total = static_cast<size_t>(L.T) * width;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const size_t at = advIndex(sg, width, i);
    sg.adv[at] = (sg.adv[at] - mean) / denom;
  }
}

// mean over every element of every segment -> *meanOut (one block)
__global__ void __launch_bounds__(32)
k_adv_mean(const AdvSegmentList L, const GaeStat* __restrict__ partials, float* meanOut) {
  GaeStat st;
  st.n = 0.0;
  st.mean = 0.0;
  st.m2 = 0.0;
  for (uint32_t i = threadIdx.x; i < L.count * L.blocksPerSeg; i += 32)
    st = gaeMerge(st, partials[i]);
  st = gaeWarpReduce(st);
  if (threadIdx.x == 0)
    *meanOut = static_cast<float>(st.mean);
}

// The running mean DD-PPO subtracts (DecentralizedDistributedMixin._get_advantages_distributed,
// bps_nav/rl/ddppo/algo/ddppo.py:46-64): biased = beta * biased + (1 - beta) * mean,
// unbias = beta * unbias + (1 - beta), shift = biased / unbias.  state = {biased, unbias, shift}.
__global__ void k_adv_ema_update(float* state, const float* mean, float beta) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const float biased = state[0] * beta + (1.f - beta) * *mean;
    const float unbias = state[1] * beta + (1.f - beta);
    state[0] = biased;
    state[1] = unbias;
    state[2] = biased / unbias;
  }
}
__global__ void __launch_bounds__(kAdvBlock)
k_adv_shift(const AdvSegmentList L, const float* __restrict__ state) {
  const AdvSegment sg = L.seg[blockIdx.y];
  const float shift = state[2];
  const uint32_t width = sg.end - sg.start;
  const size_t total = static_cast<size_t>(L.T) * width;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const size_t at = advIndex(sg, width, i);
    sg.adv[at] = sg.adv[at] - shift;
  }
}

}  // namespace bpsn
