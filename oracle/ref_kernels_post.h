#include "cuda/router_rank_exact.cuh"
#include "cuda/expert_exl3.cuh"
#include "cuda/expert_exl3_prefill_fp16.cuh"
#include "cuda/expert_exl3_prefill_masked.cuh"
#include "cuda/expert_exl3_prefill_warp.cuh"
#include "cuda/expert_exl3_prefill_packed_activations.cuh"
#include "cuda/expert_exl3_prefill_transport_async64.cuh"
#include "cuda/expert_exl3_decode_dual.cuh"
#include "cuda/mtp_experts.cuh"
#include "cuda/expert_schedule.cuh"
#include "cuda/residual_norm_wide_exact.cuh"
} // namespace
} // namespace mellum16

using namespace mellum16;
#define REF_API extern "C" __attribute__((visibility("default")))
namespace {
int Done() {
  return static_cast<int>(cudaGetLastError());
}
int FormatRate(int rate) {
  return rate == 3 || rate == 4 || rate == 6;
}
} // namespace

// M = 1 decode projection, src/cuda/expert_exl3_decode_dual.cuh:30-131.  The kernel is launched directly
// so that any rows (multiple of 128) and cols (multiple of 128, <= 2304) can be used; its launcher
// (:132-146) hard-codes the Mellum dimensions.
REF_API int ref_decode_dual(const DeviceMatrix *matrices, int layer, int part, const int *ids, const float *input,
                            float *output, float *other, int pairs, int *bad, cudaStream_t stream, int rate,
                            int rows) {
  if (!FormatRate(rate))
    return -1;
  const dim3 grid(rows / 128, pairs, part == 0 ? 2 : 1);
  if (rate == 3)
    exl3_mma_dual::Projection<3><<<grid, 256, 0, stream>>>(matrices, layer, part, ids, input, output, other, pairs, bad);
  else if (rate == 6)
    exl3_mma_dual::Projection<6><<<grid, 256, 0, stream>>>(matrices, layer, part, ids, input, output, other, pairs, bad);
  else
    exl3_mma_dual::Projection<4><<<grid, 256, 0, stream>>>(matrices, layer, part, ids, input, output, other, pairs, bad);
  return Done();
}
// The reference launcher itself (Mellum dimensions only).
REF_API int ref_decode_dual_launch(const DeviceMatrix *matrices, int layer, int part, const int *ids,
                                   const float *input, float *output, float *other, int pairs, int *bad,
                                   cudaStream_t stream, int rate) {
  exl3_mma_dual::Launch(matrices, layer, part, ids, input, output, nullptr, pairs, bad, stream, nullptr, other, rate);
  return Done();
}
// Scalar "represented math" path, src/cuda/expert_exl3.cuh:32-113, any dimensions.
REF_API int ref_simt_linear(const DeviceMatrix *matrices, int layer, int part, const int *ids, const float *input,
                            float *output, float *in_scratch, float *out_scratch, int pairs, int *bad,
                            cudaStream_t stream, int rows, int cols) {
  exl3_expert::InputHad<<<dim3(cols / 128, pairs), 128, 0, stream>>>(matrices, layer, part, ids, input, in_scratch,
                                                                      pairs, bad, false);
  exl3_expert::Dot<<<dim3(rows / 4, pairs), 128, 0, stream>>>(matrices, layer, part, ids, in_scratch, out_scratch,
                                                               pairs, bad);
  exl3_expert::OutputHad<<<dim3(rows / 128, pairs), 128, 0, stream>>>(matrices, layer, part, ids, out_scratch, output,
                                                                       pairs, bad);
  return Done();
}
REF_API int ref_mtp_build_union(const int *ids, unsigned *masks, int *slots, int rows, int *bad, int *active,
                                int *active_count, cudaStream_t stream) {
  mtp_experts::BuildUnion<true><<<1, 64, 0, stream>>>(ids, masks, slots, rows, bad, active, active_count);
  return Done();
}
// M = 2..5 verifier projection, src/cuda/mtp_experts.cuh:42-167, launched directly for any rows/cols.
template <int Rate>
static void MtpRate(const DeviceMatrix *matrices, int layer, int part, const unsigned *masks, const int *slots,
                    int rows, const float *input, float *output, float *up, int *bad, cudaStream_t stream,
                    const int *active, const int *count, int out_rows) {
  const dim3 grid(out_rows / 128, std::min(64, 8 * rows), part == 0 ? 2 : 1);
  switch (rows) {
  case 2:
    mtp_experts::Projection<2, true, Rate><<<grid, 256, 0, stream>>>(matrices, layer, part, masks, slots, rows, input,
                                                                     output, up, bad, active, count);
    break;
  case 3:
    mtp_experts::Projection<3, true, Rate><<<grid, 256, 0, stream>>>(matrices, layer, part, masks, slots, rows, input,
                                                                     output, up, bad, active, count);
    break;
  case 4:
    mtp_experts::Projection<4, true, Rate><<<grid, 256, 0, stream>>>(matrices, layer, part, masks, slots, rows, input,
                                                                     output, up, bad, active, count);
    break;
  default:
    mtp_experts::Projection<5, true, Rate><<<grid, 256, 0, stream>>>(matrices, layer, part, masks, slots, rows, input,
                                                                     output, up, bad, active, count);
    break;
  }
}
REF_API int ref_mtp_projection(const DeviceMatrix *matrices, int layer, int part, const unsigned *masks,
                               const int *slots, int rows, const float *input, float *output, float *up, int *bad,
                               cudaStream_t stream, const int *active, const int *count, int rate, int out_rows) {
  if (!FormatRate(rate) || rows < 2 || rows > 5)
    return -1;
  if (rate == 3)
    MtpRate<3>(matrices, layer, part, masks, slots, rows, input, output, up, bad, stream, active, count, out_rows);
  else if (rate == 6)
    MtpRate<6>(matrices, layer, part, masks, slots, rows, input, output, up, bad, stream, active, count, out_rows);
  else
    MtpRate<4>(matrices, layer, part, masks, slots, rows, input, output, up, bad, stream, active, count, out_rows);
  return Done();
}
REF_API int ref_group(const int *ids, int *groups, int *counts, int tokens, int *bad, cudaStream_t stream) {
  fast_expert::Group<<<64, 128, 0, stream>>>(ids, groups, counts, tokens, bad);
  return Done();
}
REF_API int ref_schedule(const int *counts, void *tiles, int *tile_count, int tokens, int *bad, cudaStream_t stream) {
  exl3_masked::Schedule<<<1, 1, 0, stream>>>(counts, static_cast<exl3_masked::Tile *>(tiles), tile_count, tokens, bad);
  return Done();
}
// Prefill, the reference launchers (Mellum dimensions only): src/cuda/expert_exl3_prefill_transport_async64.cuh:136-157
// for K4 and src/cuda/expert_exl3_prefill_packed_activations.cuh:250-277 for K3/K6.
REF_API int ref_prefill_launch(const DeviceMatrix *matrices, int layer, int part, const int *ids, const int *groups,
                               const int *counts, const void *tiles, const int *tile_count, const float *input,
                               unsigned short *output, const unsigned short *gate, const unsigned short *up,
                               const unsigned short *table, __half *transformed, int tokens, int *bad,
                               cudaStream_t stream, int rate) {
  const auto *t = static_cast<const exl3_masked::Tile *>(tiles);
  try {
    if (rate == 4)
      exl3_transport_async64::Launch(matrices, layer, part, ids, groups, counts, t, tile_count, input, output, gate, up,
                                     table, transformed, tokens, bad, stream, nullptr, true);
    else
      exl3_packed_activations::Launch(matrices, layer, part, ids, groups, counts, t, tile_count, input, output, gate,
                                      up, table, transformed, tokens, bad, stream, nullptr, true, rate);
  } catch (const std::exception &) {
    return -2;
  }
  return Done();
}
// Prefill at any dimensions: the dimension-generic kernels of the same family launched directly.
// Input transform: exl3_masked::Input (src/cuda/expert_exl3_prefill_masked.cuh:46-82); for the down
// projection the activation is first widened with the reference's ActivateToFloat adapter
// (expert_exl3_prefill_packed_activations.cuh:75-80) into `float_scratch` ([pairs][cols] floats).
REF_API int ref_prefill_generic(const DeviceMatrix *matrices, int layer, int part, const int *ids, const int *groups,
                                const void *tiles, const int *tile_count, const float *input, unsigned short *output,
                                const unsigned short *gate, const unsigned short *up, const unsigned short *table,
                                __half *transformed, float *float_scratch, int tokens, int *bad, cudaStream_t stream,
                                int rate, int rows, int cols) {
  if (!FormatRate(rate))
    return -1;
  const int pairs = tokens * 8;
  const auto *t = static_cast<const exl3_masked::Tile *>(tiles);
  if (part == 2) {
    exl3_packed_activations::ActivateToFloat<<<(pairs * cols + 255) / 256, 256, 0, stream>>>(gate, up, table,
                                                                                            float_scratch, pairs * cols, bad);
    exl3_masked::Input<<<dim3(cols / 128, pairs), 128, 0, stream>>>(matrices, layer, part, ids, float_scratch,
                                                                    transformed, pairs, bad);
  } else {
    exl3_masked::Input<<<dim3(cols / 128, pairs), 128, 0, stream>>>(matrices, layer, part, ids, input, transformed,
                                                                    pairs, bad);
  }
  const dim3 grid(rows / 128, exl3_packed_activations::Capacity(tokens));
  if (rate == 4)
    exl3_transport_async64::Projection<<<grid, 256, 0, stream>>>(matrices, layer, part, groups, t, tile_count,
                                                                  transformed, output, tokens, bad);
  else if (rate == 3)
    exl3_packed_activations::Projection<3><<<grid, 256, 0, stream>>>(matrices, layer, part, groups, t, tile_count,
                                                                     transformed, output, tokens, bad);
  else
    exl3_packed_activations::Projection<6><<<grid, 256, 0, stream>>>(matrices, layer, part, groups, t, tile_count,
                                                                     transformed, output, tokens, bad);
  return Done();
}
REF_API int ref_silu_build(unsigned short *table, cudaStream_t stream) {
  exl3_silu_lut::Build<<<256, 256, 0, stream>>>(table);
  return Done();
}
REF_API int ref_silu_activate(float *gate, const float *up, const unsigned short *table, int count, int *bad,
                              cudaStream_t stream) {
  exl3_silu_lut::Activate<<<(count + 127) / 128, 128, 0, stream>>>(gate, up, table, count, bad);
  return Done();
}
// Hidden size 2304 only (hard-coded in the kernels): src/cuda/inference.cu:580-594 and
// src/cuda/expert_exl3_prefill_packed_activations.cuh:86-103.
REF_API int ref_combine(float *x, const float *down, const float *weights, int rows, int *bad, cudaStream_t stream) {
  Combine<<<dim3(18, rows), 128, 0, stream>>>(x, down, weights, bad);
  return Done();
}
REF_API int ref_combine_packed(float *x, const unsigned short *down, const float *weights, int tokens, int *bad,
                               int residual, cudaStream_t stream) {
  exl3_packed_activations::Combine<<<dim3(18, tokens), 128, 0, stream>>>(x, down, weights, tokens, bad, residual != 0);
  return Done();
}
REF_API int ref_route(const float *logits, int *ids, float *weights, int tokens, int *bad, cudaStream_t stream) {
  Route<<<tokens, 1, 0, stream>>>(logits, ids, weights, bad);
  return Done();
}
REF_API int ref_route_rank_exact(const float *logits, int *ids, float *weights, int tokens, int *bad,
                                 cudaStream_t stream) {
  RouteRankExact<<<tokens, 64, 0, stream>>>(logits, ids, weights, bad);
  return Done();
}

// Residual add + post-attention RMS norm, src/cuda/residual_norm_wide_exact.cuh (the default profile's form), launched
// as at src/cuda/inference.cu:2913 and :3358: rows 1..5 of 2304 elements, weight = 2304 BF16 values.
REF_API int ref_residual_post_norm(float *x, const float *residual, float *normalized, const unsigned char *weight, int *bad,
                                   float *statistics, int rows, cudaStream_t stream) {
  DeviceMatrix w{};
  w.data = weight, w.rows = 2304, w.cols = 1, w.format = 0;
  ResidualPostNormWideExact<<<rows, 256, 0, stream>>>(x, residual, normalized, w, bad, statistics, rows);
  return Done();
}

// SwiGLU without the table, src/cuda/inference.cu:575-579, as the MTP draft layer launches it (src/cuda/mtp.cuh:383).
REF_API int ref_activate(float *gate, const float *up, int tokens, cudaStream_t stream) {
  Activate<<<tokens * 56, 128, 0, stream>>>(gate, up, tokens);
  return Done();
}
