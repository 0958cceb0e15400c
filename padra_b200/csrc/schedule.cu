// Prefill scheduling: expert-major pair lists and tile descriptors, built entirely on the device so that the
// whole layer can be recorded in a CUDA graph (no host read of counts, no data-dependent grid).
#include "common.cuh"
#include "kernels.cuh"

namespace padra {
namespace {

constexpr int kMaxPrefillTokens = 2048; // src/runtime/exl3_masked_schedule.h:15-17

// One CTA per expert walks all pairs in order and appends the ones routed to it: lists are stable in pair
// order, which fixes the row order inside every tile.  Semantics: src/cuda/expert_schedule.cuh:11-69.
__global__ void __launch_bounds__(256) GroupKernel(const int *ids, int *groups, int *counts, int tokens, int *bad) {
  if (!ids || !groups || !counts || !bad || tokens < 1 || tokens > kMaxPrefillTokens || blockDim.x != 256 ||
      gridDim.x != kExperts) {
    if (!threadIdx.x && bad)
      Raise(bad);
    return;
  }
  const int expert = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, pairs = tokens * kTopK;
  __shared__ int warp_counts[8], warp_offsets[8], total;
  if (!threadIdx.x)
    total = 0;
  // validation is shared out: this CTA checks the tokens congruent to its expert index
  for (int token = expert + kExperts * (threadIdx.x); token < tokens; token += kExperts * 256) {
    unsigned long long seen = 0;
    for (int s = 0; s < kTopK; ++s) {
      const int e = ids[token * kTopK + s];
      if (e < 0 || e >= kExperts) {
        Raise(bad);
        continue;
      }
      if (seen & (1ull << e))
        Raise(bad); // a token may use an expert once
      seen |= 1ull << e;
    }
  }
  __syncthreads();
  // thread t owns the consecutive pairs [t*per, (t+1)*per): count its matches, scan the counts over the CTA (stable in
  // pair order), then write
  const int per = (pairs + 255) / 256, first = threadIdx.x * per;
  const int last = first + per < pairs ? first + per : pairs;
  const bool wide = per % 4 == 0 && first + per <= pairs && (reinterpret_cast<uintptr_t>(ids) & 15) == 0; // 16-byte groups
  int mine = 0;
  if (wide) {
    for (int pair = first; pair < last; pair += 4) {
      const int4 e = *reinterpret_cast<const int4 *>(ids + pair);
      mine += (e.x == expert) + (e.y == expert) + (e.z == expert) + (e.w == expert);
    }
  } else {
    for (int pair = first; pair < last; ++pair)
      mine += ids[pair] == expert;
  }
  int inclusive = mine;
#pragma unroll
  for (int d = 1; d < 32; d *= 2) {
    const int other = __shfl_up_sync(0xffffffffu, inclusive, d);
    if (lane >= d)
      inclusive += other;
  }
  if (lane == 31)
    warp_counts[warp] = inclusive;
  __syncthreads();
  if (!threadIdx.x) {
    int n = 0;
    for (int w = 0; w < 8; ++w) {
      warp_offsets[w] = n;
      n += warp_counts[w];
    }
    total = n;
  }
  __syncthreads();
  int at = warp_offsets[warp] + inclusive - mine;
  auto append = [&](int id, int pair) {
    if (id == expert) {
      if (at < tokens)
        groups[expert * tokens + at] = pair;
      ++at;
    }
  };
  if (wide) {
    for (int pair = first; pair < last && mine; pair += 4) {
      const int4 e = *reinterpret_cast<const int4 *>(ids + pair);
      append(e.x, pair), append(e.y, pair + 1), append(e.z, pair + 2), append(e.w, pair + 3);
    }
  } else {
    for (int pair = first; pair < last; ++pair)
      append(ids[pair], pair);
  }
  __syncthreads();
  if (!threadIdx.x) {
    if (total > tokens)
      Raise(bad);
    counts[expert] = total < tokens ? total : tokens;
  }
}

// Tiles of at most 32 pairs, experts ascending.  Semantics: src/cuda/expert_exl3_prefill_masked.cuh:12-45.
__global__ void ScheduleKernel(const int *counts, padra_tile *tiles, int *tile_count, int tokens, int *bad) {
  if (!counts || !tiles || !tile_count || !bad || tokens < 1 || tokens > kMaxPrefillTokens || blockDim.x != kExperts ||
      gridDim.x != 1) {
    if (!threadIdx.x && bad)
      Raise(bad);
    if (!threadIdx.x && tile_count)
      *tile_count = 0;
    return;
  }
  __shared__ int offsets[kExperts + 1], ok;
  const int e = threadIdx.x;
  if (!e) {
    ok = *bad == 0;
    int sum = 0, n = 0;
    for (int i = 0; i < kExperts; ++i) {
      const int c = counts[i];
      offsets[i] = n;
      if (c < 0 || c > tokens)
        ok = 0;
      else {
        sum += c;
        n += (c + 31) / 32;
      }
    }
    offsets[kExperts] = n;
    if (sum != tokens * kTopK || n > (tokens * kTopK + 31) / 32 + kExperts)
      ok = 0;
    *tile_count = ok ? n : 0;
    if (!ok)
      Raise(bad);
  }
  __syncthreads();
  if (!ok)
    return;
  const int c = counts[e];
  for (int i = offsets[e]; i < offsets[e + 1]; ++i) {
    const int begin = (i - offsets[e]) * 32;
    tiles[i] = padra_tile{e, begin, c - begin < 32 ? c - begin : 32};
  }
}

} // namespace

int LaunchGroup(const int *ids, int *groups, int *counts, int tokens, int *bad, cudaStream_t stream) {
  if (!ids || !groups || !counts || !bad || tokens < 1 || tokens > kMaxPrefillTokens)
    return PADRA_INVALID_ARGUMENT;
  GroupKernel<<<kExperts, 256, 0, stream>>>(ids, groups, counts, tokens, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchSchedule(const int *counts, padra_tile *tiles, int *tile_count, int tokens, int *bad, cudaStream_t stream) {
  if (!counts || !tiles || !tile_count || !bad || tokens < 1 || tokens > kMaxPrefillTokens)
    return PADRA_INVALID_ARGUMENT;
  ScheduleKernel<<<1, kExperts, 0, stream>>>(counts, tiles, tile_count, tokens, bad);
  return CudaStatus(cudaGetLastError());
}

} // namespace padra
