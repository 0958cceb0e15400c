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

constexpr int kMaxRows = 2048 * kTopK;

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
__global__ void CombineIndexedKernel(float *x, const unsigned short *down_rows, const int *position, const float *weights, int tokens,
                                     int hidden, int *bad, bool residual) {
  const int token = blockIdx.y, col = blockIdx.x * blockDim.x + threadIdx.x;
  if (token >= tokens || col >= hidden)
    return;
  float sum = 0.f;
#pragma unroll
  for (int s = 0; s < kTopK; ++s) {
    const int at = position[token * kTopK + s];
    if (at < 0 || at >= tokens * kTopK) {
      Raise(bad);
      return;
    }
    const float d = FromBF16Bits(down_rows[static_cast<size_t>(at) * hidden + col]);
    sum = RoundBF16(__fadd_rn(sum, RoundBF16(__fmul_rn(d, weights[token * kTopK + s]))));
  }
  const size_t i = static_cast<size_t>(token) * hidden + col;
  const float v = residual ? RoundBF16(__fadd_rn(x[i], sum)) : sum;
  if (!isfinite(v))
    Raise(bad);
  x[i] = v;
}

} // namespace

int LaunchGroupRows(const int *ids, int *groups, int *counts, int rows, int group_stride, int *bad, cudaStream_t stream) {
  if (!ids || !groups || !counts || !bad || rows < 1 || rows > kMaxRows || group_stride < 1 || group_stride > rows)
    return PADRA_INVALID_ARGUMENT;
  GroupRowsKernel<<<kExperts, 256, 0, stream>>>(ids, groups, counts, rows, group_stride, bad);
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
  if (!x || !down_rows || !position || !weights || !bad || tokens < 1 || hidden < 1)
    return PADRA_INVALID_ARGUMENT;
  CombineIndexedKernel<<<dim3((hidden + 127) / 128, tokens), 128, 0, stream>>>(x, down_rows, position, weights, tokens, hidden, bad,
                                                                                residual != 0);
  return CudaStatus(cudaGetLastError());
}

} // namespace padra
