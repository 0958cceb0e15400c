// Expert-parallel prefill: the device-side pieces around the all-to-all exchange.
//
// With the 64 experts of a layer spread over N GPUs, a rank (1) packs the activation row of every (token, slot) pair
// into BF16 rows ordered by destination rank, (2) exchanges them (NCCL all-to-all, host side), (3) groups the rows
// it received by expert and runs the grouped projections on them (prefill.cu, one input row per pair), (4) sends the
// down rows back, and (5) combines them with the routing weights, reading each pair's row through an index map so
// that no un-permute pass over the rows is needed.  Arithmetic is that of the single-GPU path: rows cross the wire as
// BF16, which is exactly what the projections' inputs and outputs hold.
#include "common.cuh"
#include "kernels.cuh"

namespace padra {
namespace {

constexpr int kMaxRows = 4096 * kTopK; // rows one grouped-projection call takes (received rows may exceed a rank's own)
constexpr int kMaxRanks = 8;

// One CTA per expert walks the rows in order and appends those routed to it (stable, like GroupKernel).  `ids` are
// expert ids 0..63 per row; experts this rank does not own simply get no rows.
__global__ void __launch_bounds__(256) GroupRowsKernel(const int *ids, int *groups, int *counts, int rows, int stride, int *bad) {
  const int expert = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __shared__ int warp_counts[8], warp_offsets[8], total;
  if (!threadIdx.x)
    total = 0;
  __syncthreads();
  for (int base = 0; base < rows; base += 256) {
    const int row = base + threadIdx.x;
    const int id = row < rows ? ids[row] : -1;
    if (row < rows && (id < 0 || id >= kExperts) && expert == 0)
      Raise(bad);
    const bool mine = id == expert;
    const unsigned votes = __ballot_sync(0xffffffffu, mine);
    if (!lane)
      warp_counts[warp] = __popc(votes);
    __syncthreads();
    if (!threadIdx.x) {
      int n = total;
      for (int w = 0; w < 8; ++w) {
        warp_offsets[w] = n;
        n += warp_counts[w];
      }
      total = n;
    }
    __syncthreads();
    if (mine) {
      const int at = warp_offsets[warp] + __popc(votes & ((1u << lane) - 1u));
      if (at < stride)
        groups[static_cast<size_t>(expert) * stride + at] = row;
    }
    __syncthreads();
  }
  if (!threadIdx.x) {
    if (total > stride)
      Raise(bad);
    counts[expert] = total < stride ? total : stride;
  }
}

// The send plan of one rank, one CTA: a stable counting sort of the pairs by destination rank owner[ids[pair]].
//   order[j]      pair that travels as row j          position[pair]  row at which the pair's result comes back
//   send_ids[j]   expert id of row j                  send_counts[r]  rows for rank r (64-bit, as the host API wants)
// Thread t owns the 16 consecutive pairs from 16*t on; a scan over (destination, thread) keeps the order stable.
__global__ void __launch_bounds__(1024) PlanKernel(const int *ids, const int *owner, int *order, int *position, int *send_ids,
                                                   long long *send_counts, int pairs, int world, int *bad) {
  __shared__ int s_owner[kExperts], s_scan[kMaxRanks][1024 + 1], s_base[kMaxRanks + 1];
  const int t = threadIdx.x, per = (pairs + 1023) / 1024, first = t * per;
  if (t < kExperts)
    s_owner[t] = owner[t];
  __syncthreads();
  int mine[kMaxRanks] = {};
  for (int i = 0; i < per; ++i) {
    const int pair = first + i;
    if (pair < pairs) {
      const int e = ids[pair];
      const int r = (e >= 0 && e < kExperts) ? s_owner[e] : -1;
      if (r < 0 || r >= world)
        Raise(bad);
      else
        ++mine[r];
    }
  }
  for (int r = 0; r < world; ++r)
    s_scan[r][t] = mine[r];
  __syncthreads();
  if (t < world) { // one thread per destination: exclusive scan over the 1024 threads' counts
    int sum = 0;
    for (int i = 0; i < 1024; ++i) {
      const int v = s_scan[t][i];
      s_scan[t][i] = sum;
      sum += v;
    }
    s_scan[t][1024] = sum;
  }
  __syncthreads();
  if (t == 0) {
    int sum = 0;
    for (int r = 0; r < world; ++r) {
      s_base[r] = sum;
      sum += s_scan[r][1024];
      send_counts[r] = s_scan[r][1024];
    }
    s_base[world] = sum;
  }
  __syncthreads();
  int cursor[kMaxRanks];
  for (int r = 0; r < world; ++r)
    cursor[r] = s_base[r] + s_scan[r][t];
  for (int i = 0; i < per; ++i) {
    const int pair = first + i;
    if (pair < pairs) {
      const int e = ids[pair];
      const int r = (e >= 0 && e < kExperts) ? s_owner[e] : -1;
      if (r >= 0 && r < world) {
        const int at = cursor[r]++;
        order[at] = pair, send_ids[at] = e, position[pair] = at;
      } else {
        position[pair] = 0;
      }
    }
  }
}

// packed[j] = BF16 bits of activations[order[j] / 8]: order[j] is the (token*8+slot) pair that travels as row j.
__global__ void __launch_bounds__(256) PackRowsKernel(const float *activations, const int *order, unsigned short *packed, int rows,
                                                      int hidden, int *bad) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const int pair = order[row];
    if (pair < 0 || pair >= rows) {
      if (!lane)
        Raise(bad);
      continue;
    }
    const float *from = activations + static_cast<size_t>(pair >> 3) * hidden;
    unsigned short *to = packed + static_cast<size_t>(row) * hidden;
    for (int k = lane * 4; k < hidden; k += 128) {
      const float4 v = *reinterpret_cast<const float4 *>(from + k);
      uint2 bits;
      bits.x = static_cast<unsigned>(BF16Bits(v.x)) | (static_cast<unsigned>(BF16Bits(v.y)) << 16);
      bits.y = static_cast<unsigned>(BF16Bits(v.z)) | (static_cast<unsigned>(BF16Bits(v.w)) << 16);
      *reinterpret_cast<uint2 *>(to + k) = bits;
    }
  }
}

// The combine of src/cuda/expert_exl3_prefill_packed_activations.cuh:86-103 with the down row of pair p found at
// down_rows[position[p]]: x[t] = B(x[t] + sum), sum = B(sum + B(down * w)) over the eight slots in order.
__global__ void __launch_bounds__(128) CombineIndexedKernel(float *x, const unsigned short *down_rows, const int *position,
                                                            const float *weights, int tokens, int hidden, int *bad, bool residual) {
  const int token = blockIdx.y, col = (blockIdx.x * blockDim.x + threadIdx.x) * 4; // four columns per thread
  if (token >= tokens || col >= hidden)
    return;
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < kTopK; ++s) {
    const int at = position[token * kTopK + s];
    if (at < 0 || at >= tokens * kTopK) {
      Raise(bad);
      return;
    }
    const uint2 bits = *reinterpret_cast<const uint2 *>(down_rows + static_cast<size_t>(at) * hidden + col);
    const float w = weights[token * kTopK + s];
    const float d[4] = {FromBF16Bits(bits.x & 0xffffu), FromBF16Bits(bits.x >> 16), FromBF16Bits(bits.y & 0xffffu),
                        FromBF16Bits(bits.y >> 16)};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      sum[j] = RoundBF16(__fadd_rn(sum[j], RoundBF16(__fmul_rn(d[j], w))));
  }
  float4 *target = reinterpret_cast<float4 *>(x + static_cast<size_t>(token) * hidden + col);
  const float4 old = *target;
  float4 v;
  v.x = residual ? RoundBF16(__fadd_rn(old.x, sum[0])) : sum[0];
  v.y = residual ? RoundBF16(__fadd_rn(old.y, sum[1])) : sum[1];
  v.z = residual ? RoundBF16(__fadd_rn(old.z, sum[2])) : sum[2];
  v.w = residual ? RoundBF16(__fadd_rn(old.w, sum[3])) : sum[3];
  if (!isfinite(v.x) || !isfinite(v.y) || !isfinite(v.z) || !isfinite(v.w))
    Raise(bad);
  *target = v;
}

} // namespace

int LaunchGroupRows(const int *ids, int *groups, int *counts, int rows, int group_stride, int *bad, cudaStream_t stream) {
  if (!ids || !groups || !counts || !bad || rows < 1 || rows > kMaxRows || group_stride < 1 || group_stride > rows)
    return PADRA_INVALID_ARGUMENT;
  GroupRowsKernel<<<kExperts, 256, 0, stream>>>(ids, groups, counts, rows, group_stride, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchPlan(const int *ids, const int *owner, int *order, int *position, int *send_ids, long long *send_counts, int pairs,
               int world, int *bad, cudaStream_t stream) {
  if (!ids || !owner || !order || !position || !send_ids || !send_counts || !bad || pairs < 1 || pairs > 2048 * kTopK ||
      world < 1 || world > kMaxRanks)
    return PADRA_INVALID_ARGUMENT;
  PlanKernel<<<1, 1024, 0, stream>>>(ids, owner, order, position, send_ids, send_counts, pairs, world, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchPackRows(const float *activations, const int *order, unsigned short *packed, int rows, int hidden, int *bad,
                   cudaStream_t stream) {
  if (!activations || !order || !packed || !bad || rows < 8 || (rows % kTopK) || hidden < 128 || (hidden % 128) ||
      reinterpret_cast<uintptr_t>(activations) % 16 || reinterpret_cast<uintptr_t>(packed) % 8)
    return PADRA_INVALID_ARGUMENT;
  const int blocks = (rows + 7) / 8;
  PackRowsKernel<<<blocks < 148 * 16 ? blocks : 148 * 16, 256, 0, stream>>>(activations, order, packed, rows, hidden, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchCombineIndexed(float *x, const unsigned short *down_rows, const int *position, const float *weights, int tokens,
                         int *bad, int residual, int hidden, cudaStream_t stream) {
  if (!x || !down_rows || !position || !weights || !bad || tokens < 1 || hidden < 4 || (hidden % 4) ||
      reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(down_rows) % 8)
    return PADRA_INVALID_ARGUMENT;
  CombineIndexedKernel<<<dim3((hidden / 4 + 127) / 128, tokens), 128, 0, stream>>>(x, down_rows, position, weights, tokens, hidden, bad,
                                                                                residual != 0);
  return CudaStatus(cudaGetLastError());
}

} // namespace padra
