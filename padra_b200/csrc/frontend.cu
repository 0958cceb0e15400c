// The callers either side of the expert projections: the router's softmax / top-8, the grouping and tile schedule of a
// prefill chunk fused behind it, and the RMS norms that produce the experts' input and consume their output.
//
//   RouteKernel               exact-rank routing, one warp per token.  Semantics: RouteRankExact,
//                             src/cuda/router_rank_exact.cuh:3-81 (softmax with FP64 exp rounded to FP32 and ascending
//                             compensated sums, rank by probability then index, renormalised BF16 weights, ascending ids).
//   RouteGroupScheduleKernel  the same routing, after which the CTA that finishes last builds, for the whole chunk, the
//                             expert-major pair lists (fast_expert::Group, src/cuda/expert_schedule.cuh:11-69) and the
//                             32-pair tile list (exl3_masked::Schedule, src/cuda/expert_exl3_prefill_masked.cuh:12-45):
//                             one launch where the reference has three (src/cuda/inference.cu:3861, :3875, :3890).
//   ResidualNormKernel        x = B(x + residual), normalized = B(B(x * inv) * weight) with the compensated 128-thread
//                             sum of squares.  Semantics: ResidualPostNormWideExact,
//                             src/cuda/residual_norm_wide_exact.cuh:84-131 with Rms128In256Exact, rms_wide_exact.cuh:3-33.
//   CombineNormKernel         the ordered BF16 combine of the eight slots, the residual add and the same norm in one
//                             pass.  Semantics: combine_norm_exact::CombineNorm<false>, src/cuda/combine_norm_exact.cuh:7-68.
// Summation orders are the reference's (thread t owns elements t, t+128, ...; shuffle-down trees), so results are equal
// bit for bit.
#include "common.cuh"
#include "kernels.cuh"

namespace padra {
namespace {

constexpr int kRouteWarps = 32;      // tokens per CTA of the routing kernels
constexpr int kMaxChunkTokens = 2048; // src/runtime/exl3_masked_schedule.h:15-17

// src/cuda/inference.cu:57-59 and :103-109
__device__ __forceinline__ float ExpRN(float x) {
  return __double2float_rn(exp(static_cast<double>(x)));
}
__device__ __forceinline__ void Accumulate(float value, float &sum, float &error) {
  const float next = __fadd_rn(sum, value);
  const float residual = fabsf(sum) >= fabsf(value) ? __fadd_rn(__fsub_rn(sum, next), value) : __fadd_rn(__fsub_rn(value, next), sum);
  error = __fadd_rn(error, residual);
  sum = next;
}

// One warp routes one token.  `slot_*` are eight-entry scratch arrays of the warp in shared memory.
__device__ __forceinline__ void RouteToken(const float *logits, int *ids, float *weights, int *bad, bool abort, float *slot_w,
                                           int *slot_id) {
  const unsigned full = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  const float l0 = logits[lane], l1 = logits[lane + 32];
  abort = abort || !__all_sync(full, isfinite(l0) && isfinite(l1));
  if (abort) { // safe descriptor indices, zero weights, sticky flag: the host rejects the token
    if (lane < kTopK) {
      ids[lane] = 0;
      weights[lane] = 0.f;
    }
    if (!lane)
      Raise(bad);
    return;
  }
  float maximum = fmaxf(l0, l1);
#pragma unroll
  for (int d = 16; d; d /= 2)
    maximum = fmaxf(maximum, __shfl_xor_sync(full, maximum, d));
  const float p0 = ExpRN(__fsub_rn(l0, maximum)), p1 = ExpRN(__fsub_rn(l1, maximum));
  float sum = 0.f, error = 0.f; // every lane forms the same ascending sum
  for (int i = 0; i < 32; ++i)
    Accumulate(__shfl_sync(full, p0, i), sum, error);
  for (int i = 0; i < 32; ++i)
    Accumulate(__shfl_sync(full, p1, i), sum, error);
  const float total = __fadd_rn(sum, error);
  const float q0 = __fdiv_rn(p0, total), q1 = __fdiv_rn(p1, total);
  int rank0 = 0, rank1 = 0; // experts `lane` and `lane + 32`
  for (int i = 0; i < 32; ++i) {
    const float other = __shfl_sync(full, q0, i); // expert i
    rank0 += other > q0 || (other == q0 && i < lane);
    rank1 += other > q1 || other == q1; // i < lane + 32 always
  }
  for (int i = 0; i < 32; ++i) {
    const float other = __shfl_sync(full, q1, i); // expert i + 32
    rank0 += other > q0;                         // i + 32 < lane never
    rank1 += other > q1 || (other == q1 && i < lane);
  }
  if (rank0 < kTopK) {
    slot_id[rank0] = lane;
    slot_w[rank0] = q0;
  }
  if (rank1 < kTopK) {
    slot_id[rank1] = lane + 32;
    slot_w[rank1] = q1;
  }
  __syncwarp();
  sum = 0.f, error = 0.f;
#pragma unroll
  for (int s = 0; s < kTopK; ++s)
    Accumulate(slot_w[s], sum, error);
  const float selected = __fadd_rn(sum, error);
  if (lane < kTopK) {
    const int id = slot_id[lane];
    int place = 0; // ascending expert id
#pragma unroll
    for (int s = 0; s < kTopK; ++s)
      place += slot_id[s] < id;
    ids[place] = id;
    weights[place] = RoundBF16(__fdiv_rn(slot_w[lane], selected));
  }
  if (!lane && !isfinite(selected))
    Raise(bad);
  __syncwarp();
}

__global__ void __launch_bounds__(kRouteWarps * 32) RouteKernel(const float *logits, int *ids, float *weights, int tokens, int *bad) {
  __shared__ float s_w[kRouteWarps][kTopK];
  __shared__ int s_id[kRouteWarps][kTopK];
  const int warp = threadIdx.x >> 5, token = blockIdx.x * kRouteWarps + warp;
  if (token >= tokens)
    return;
  RouteToken(logits + static_cast<size_t>(token) * kExperts, ids + token * kTopK, weights + token * kTopK, bad, *bad != 0, s_w[warp],
             s_id[warp]);
}

// Dynamic shared memory of the scheduling phase: per (expert, thread) the number of the thread's pairs routed to the
// expert, then (in place, widened) the thread's first position inside the expert's list.
struct ScheduleSmem {
  unsigned short position[kExperts][1024];
};

__global__ void __launch_bounds__(1024) RouteGroupScheduleKernel(const float *logits, int *ids, float *weights, int *groups, int *counts,
                                                                 padra_tile *tiles, int *tile_count, int tokens, unsigned *ticket,
                                                                 int *bad) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float s_w[kRouteWarps][kTopK];
  __shared__ int s_id[kRouteWarps][kTopK];
  __shared__ int s_last, s_total[kExperts], s_tile_offset[kExperts + 1], s_ok;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int token = blockIdx.x * kRouteWarps + warp;
  if (token < tokens)
    RouteToken(logits + static_cast<size_t>(token) * kExperts, ids + token * kTopK, weights + token * kTopK, bad, *bad != 0, s_w[warp],
               s_id[warp]);
  // ---- the CTA that finishes last schedules the chunk ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    if (s_last)
      *ticket = 0; // left zero for the next call
  }
  __syncthreads();
  if (!s_last)
    return;
  __threadfence();
  auto &sm = *reinterpret_cast<ScheduleSmem *>(smem);
  const int pairs = tokens * kTopK;
  const int per = (pairs + 1023) / 1024, first = tid * per, last = first + per < pairs ? first + per : pairs; // per <= 16
  if (tid == 0)
    s_ok = __ldcg(bad) == 0;
  for (int e = 0; e < kExperts; ++e)
    sm.position[e][tid] = 0;
  __syncthreads();
  // thread t owns the consecutive pairs [first, last): count per expert (its own column: no races)
  int mine[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int pair = first + i;
    int id = -1;
    if (i < per && pair < last) {
      id = __ldcg(ids + pair);
      if (id < 0 || id >= kExperts) {
        id = -1;
        s_ok = 0;
      } else {
        ++sm.position[id][tid];
      }
    }
    mine[i] = id;
  }
  __syncthreads();
  // exclusive scan of every expert's row over the 1024 threads: warp w scans experts 2w and 2w+1, a lane 32 threads
  for (int e = 2 * warp; e < 2 * warp + 2; ++e) {
    unsigned short *row = sm.position[e];
    int local = 0;
    for (int i = 0; i < 32; ++i)
      local += row[lane * 32 + i];
    int inclusive = local;
#pragma unroll
    for (int d = 1; d < 32; d *= 2) {
      const int other = __shfl_up_sync(0xffffffffu, inclusive, d);
      if (lane >= d)
        inclusive += other;
    }
    int at = inclusive - local;
    for (int i = 0; i < 32; ++i) {
      const int n = row[lane * 32 + i];
      row[lane * 32 + i] = static_cast<unsigned short>(at);
      at += n;
    }
    if (lane == 31)
      s_total[e] = inclusive;
  }
  __syncthreads();
  // lists, stable in pair order (group_stride = tokens, as in the reference)
#pragma unroll
  for (int i = 0; i < 16; ++i)
    if (mine[i] >= 0) {
      const int at = sm.position[mine[i]][tid]++;
      if (at < tokens)
        groups[mine[i] * tokens + at] = first + i;
    }
  // counts and the 32-pair tiles, experts ascending
  if (tid == 0) {
    int sum = 0, n = 0, ok = s_ok;
    for (int e = 0; e < kExperts; ++e) {
      const int c = s_total[e];
      s_tile_offset[e] = n;
      if (c > tokens)
        ok = 0;
      sum += c;
      n += (c + 31) / 32;
    }
    s_tile_offset[kExperts] = n;
    if (sum != pairs || n > (pairs + 31) / 32 + kExperts)
      ok = 0;
    s_ok = ok;
    *tile_count = ok ? n : 0;
    if (!ok)
      Raise(bad);
  }
  __syncthreads();
  if (tid < kExperts)
    counts[tid] = s_total[tid] < tokens ? s_total[tid] : tokens;
  if (!s_ok)
    return;
  for (int i = tid; i < s_tile_offset[kExperts]; i += 1024) {
    int e = 0;
    for (int step = 32; step; step >>= 1)
      if (e + step < kExperts && s_tile_offset[e + step] <= i)
        e += step;
    const int begin = (i - s_tile_offset[e]) * 32, c = s_total[e];
    tiles[i] = padra_tile{e, begin, c - begin < 32 ? c - begin : 32};
  }
}

// Reduction of the 128 per-thread compensated sums: shuffle-down trees inside each of the four warps, then over the
// four warp results (src/cuda/rms_wide_exact.cuh:3-33; src/cuda/inference.cu:110-134 gives the same sum).
// Called by all threads of the CTA; threads >= 128 pass zeros.  Returns the total in thread 0.
__device__ __forceinline__ float ReduceSquares128(float sum, float error, float *scratch) {
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid < 128) {
#pragma unroll
    for (int d = 16; d; d /= 2) {
      const float other = __shfl_down_sync(0xffffffffu, sum, d), low = __shfl_down_sync(0xffffffffu, error, d);
      if (lane + d < 32) {
        Accumulate(other, sum, error);
        Accumulate(low, sum, error);
      }
    }
    if (lane == 0) {
      scratch[tid / 32] = sum;
      scratch[4 + tid / 32] = error;
    }
  }
  __syncthreads();
  sum = tid < 4 ? scratch[tid] : 0.f;
  error = tid < 4 ? scratch[4 + tid] : 0.f;
  if (tid < 4)
#pragma unroll
    for (int d = 2; d; d /= 2) {
      const float other = __shfl_down_sync(0xfu, sum, d, 4), low = __shfl_down_sync(0xfu, error, d, 4);
      if (tid + d < 4) {
        Accumulate(other, sum, error);
        Accumulate(low, sum, error);
      }
    }
  return __fadd_rn(sum, error);
}

__global__ void __launch_bounds__(256) ResidualNormKernel(float *x, const float *residual, float *normalized, const unsigned short *weight,
                                                          int hidden, int *bad, float *statistics) {
  extern __shared__ __align__(16) float row[];
  __shared__ float sums[8], inv;
  const int tid = threadIdx.x;
  x += static_cast<size_t>(blockIdx.x) * hidden;
  normalized += static_cast<size_t>(blockIdx.x) * hidden;
  if (residual)
    residual += static_cast<size_t>(blockIdx.x) * hidden;
  float sum = 0.f, error = 0.f;
  if (tid < 128)
    for (int i = tid; i < hidden; i += 128) {
      const float value = RoundBF16(residual ? __fadd_rn(x[i], residual[i]) : x[i]);
      x[i] = value;
      row[i] = value;
      if (!isfinite(value))
        Raise(bad);
      Accumulate(__fmul_rn(value, value), sum, error);
    }
  sum = ReduceSquares128(sum, error, sums);
  if (tid == 0) {
    if (!isfinite(sum))
      Raise(bad);
    const float variance = __fdiv_rn(sum, static_cast<float>(hidden));
    inv = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(variance, 1e-6f)));
    if (statistics) {
      statistics[blockIdx.x * 2] = variance;
      statistics[blockIdx.x * 2 + 1] = inv;
    }
  }
  __syncthreads();
  for (int i = tid; i < hidden; i += 256) {
    const float value = RoundBF16(__fmul_rn(RoundBF16(__fmul_rn(row[i], inv)), FromBF16Bits(weight[i])));
    normalized[i] = value;
    if (!isfinite(value))
      Raise(bad);
  }
}

__global__ void __launch_bounds__(128) CombineNormKernel(float *x, const float *down, const float *routing, float *normalized,
                                                         const unsigned short *weight, int hidden, int *bad, float *statistics) {
  extern __shared__ __align__(16) float row[];
  __shared__ float sums[8], inv;
  const int tid = threadIdx.x;
  x += static_cast<size_t>(blockIdx.x) * hidden;
  normalized += static_cast<size_t>(blockIdx.x) * hidden;
  down += static_cast<size_t>(blockIdx.x) * kTopK * hidden;
  routing += blockIdx.x * kTopK;
  float w[kTopK];
#pragma unroll
  for (int s = 0; s < kTopK; ++s)
    w[s] = routing[s];
  float sum = 0.f, error = 0.f;
  for (int i = tid; i < hidden; i += 128) {
    float acc = 0.f; // every element sees the slots in order 0..7
#pragma unroll
    for (int s = 0; s < kTopK; ++s)
      acc = RoundBF16(__fadd_rn(acc, RoundBF16(__fmul_rn(down[static_cast<size_t>(s) * hidden + i], w[s]))));
    const float value = RoundBF16(__fadd_rn(x[i], acc));
    x[i] = value;
    row[i] = value;
    if (!isfinite(value))
      Raise(bad);
    Accumulate(__fmul_rn(value, value), sum, error);
  }
  sum = ReduceSquares128(sum, error, sums);
  if (tid == 0) {
    const float variance = __fdiv_rn(sum, static_cast<float>(hidden));
    inv = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(variance, 1e-6f)));
    if (statistics) {
      statistics[blockIdx.x * 2] = variance;
      statistics[blockIdx.x * 2 + 1] = inv;
    }
  }
  __syncthreads();
  for (int i = tid; i < hidden; i += 128) {
    const float value = RoundBF16(__fmul_rn(RoundBF16(__fmul_rn(row[i], inv)), FromBF16Bits(weight[i])));
    normalized[i] = value;
    if (!isfinite(value))
      Raise(bad);
  }
}

} // namespace

int LaunchRoute(const float *logits, int *ids, float *weights, int tokens, int *bad, cudaStream_t stream) {
  if (!logits || !ids || !weights || !bad || tokens < 1)
    return PADRA_INVALID_ARGUMENT;
  RouteKernel<<<(tokens + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, 0, stream>>>(logits, ids, weights, tokens, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchRouteGroupSchedule(const float *logits, int *ids, float *weights, int *groups, int *counts, padra_tile *tiles, int *tile_count,
                             int tokens, unsigned *ticket, int *bad, cudaStream_t stream) {
  if (!logits || !ids || !weights || !groups || !counts || !tiles || !tile_count || !ticket || !bad || tokens < 1 ||
      tokens > kMaxChunkTokens)
    return PADRA_INVALID_ARGUMENT;
  const size_t smem = sizeof(ScheduleSmem);
  if (cudaFuncSetAttribute(RouteGroupScheduleKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return PADRA_RESOURCE_EXHAUSTED;
  RouteGroupScheduleKernel<<<(tokens + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, smem, stream>>>(
      logits, ids, weights, groups, counts, tiles, tile_count, tokens, ticket, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchResidualNorm(float *x, const float *residual, float *normalized, const unsigned short *weight, int rows, int hidden, int *bad,
                       float *statistics, cudaStream_t stream) {
  if (!x || !normalized || x == normalized || !weight || !bad || rows < 1 || hidden < 128 || hidden % 128 || hidden > 12288)
    return PADRA_INVALID_ARGUMENT;
  const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(ResidualNormKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return PADRA_RESOURCE_EXHAUSTED;
  ResidualNormKernel<<<rows, 256, smem, stream>>>(x, residual, normalized, weight, hidden, bad, statistics);
  return CudaStatus(cudaGetLastError());
}

int LaunchCombineNorm(float *x, const float *down, const float *routing, float *normalized, const unsigned short *weight, int rows,
                      int hidden, int *bad, float *statistics, cudaStream_t stream) {
  if (!x || !down || !routing || !normalized || x == normalized || !weight || !bad || rows < 1 || hidden < 128 || hidden % 128 ||
      hidden > 12288)
    return PADRA_INVALID_ARGUMENT;
  const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(CombineNormKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return PADRA_RESOURCE_EXHAUSTED;
  CombineNormKernel<<<rows, 128, smem, stream>>>(x, down, routing, normalized, weight, hidden, bad, statistics);
  return CudaStatus(cudaGetLastError());
}

} // namespace padra
