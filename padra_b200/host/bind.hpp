// C++ forwarders that bind the C ABI of libpadra_b200.so into the reference's launcher call sites.
//
// The reference (Danmoreng/padra) has no plugin layer for its expert path: each launcher is an inline host function in
// a header of the one translation unit src/cuda/inference.cu.  Every function below keeps the argument list of the
// launcher it replaces (cited beside it), passes the Mellum dimensions the reference hard-codes (hidden 2304,
// intermediate 896) explicitly, and turns a non-zero status into the std::runtime_error the reference's launchers throw
// (RunCudaInferenceCore maps it to Status(kInternal), src/cuda/inference.cu:4324-4328).
//
// Include it after the reference's own declarations of mellum16::DeviceMatrix (src/cuda/device_matrix.cuh:6-13) and
// mellum16::exl3_masked_schedule::Tile (src/runtime/exl3_masked_schedule.h:6-8); a translation unit that has neither
// defines PADRA_B200_BIND_STANDALONE first and gets layout-identical stand-ins.
#pragma once
#include <cstdint>
#include <stdexcept>

#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include "../../include/padra_b200.h"

#ifdef PADRA_B200_BIND_STANDALONE
namespace mellum16 {
struct DeviceMatrix {
  const unsigned char *data = nullptr;
  const unsigned char *scales = nullptr;
  const float *divisor = nullptr;
  int rows = 0, cols = 0, format = 0;
  const std::uint16_t *suh = nullptr;
  const std::uint16_t *svh = nullptr;
};
namespace exl3_masked_schedule {
struct Tile {
  int expert, begin, valid_rows;
};
} // namespace exl3_masked_schedule
} // namespace mellum16
#endif

namespace padra_b200_bind {

constexpr int kHidden = 2304, kInter = 896; // src/cuda/expert_exl3_decode_dual.cuh:136

static_assert(sizeof(mellum16::DeviceMatrix) == sizeof(padra_matrix), "descriptor layouts must agree");
static_assert(sizeof(mellum16::exl3_masked_schedule::Tile) == sizeof(padra_tile), "tile layouts must agree");

inline const padra_matrix *M(const mellum16::DeviceMatrix *m) {
  return reinterpret_cast<const padra_matrix *>(m);
}
inline void Check(int status) {
  if (status != PADRA_OK)
    throw std::runtime_error(padra_status_string(status));
}

// exl3_mma_dual::Launch, src/cuda/expert_exl3_decode_dual.cuh:132-146 (call site inference.cu:2963-2975 via expert())
inline void DecodeLaunch(const mellum16::DeviceMatrix *m, int layer, int part, const int *ids, const float *in, float *out,
                         float *scratch, int pairs, int *bad, cudaStream_t s, unsigned *ranges = nullptr,
                         float *other = nullptr, int rate = 4) {
  Check(padra_exl3_decode_launch(M(m), layer, part, ids, in, out, scratch, pairs, bad, s, ranges, other, rate, kHidden, kInter));
}
// mtp_experts::BuildUnion<true> + mtp_experts::Launch, src/cuda/mtp_experts.cuh:7-40, 225-245 (inference.cu:3375-3392)
inline void MtpUnion(const int *ids, unsigned *masks, int *slots, int rows, int *bad, int *active, int *count, cudaStream_t s) {
  Check(padra_mtp_build_union(ids, masks, slots, rows, bad, active, count, s, /*slot_stride=*/5));
}
inline void MtpLaunch(const mellum16::DeviceMatrix *m, int layer, int part, const unsigned *masks, const int *slots, int rows,
                      const float *in, float *out, float *up, int *bad, cudaStream_t s, const int *active, const int *count,
                      int rate = 4) {
  Check(padra_mtp_experts_launch(M(m), layer, part, masks, slots, rows, in, out, up, bad, s, active, count, rate, kHidden, kInter, 5));
}
// exl3_silu_lut::Build / Activate, src/cuda/exl3_silu_lut.cuh:9-31
inline void SiluBuild(unsigned short *table, cudaStream_t s) {
  Check(padra_exl3_silu_build(table, s));
}
inline void SiluActivate(float *gate, const float *up, const unsigned short *table, int count, int *bad, cudaStream_t s) {
  Check(padra_exl3_silu_activate(gate, up, table, count, bad, s));
}
// Combine<<<dim3(18, rows), 128>>>, src/cuda/inference.cu:580-594
inline void Combine(float *x, const float *down, const float *w, int *bad, int rows, cudaStream_t s) {
  Check(padra_combine(x, down, w, bad, rows, kHidden, s));
}
// fast_expert::Group (src/cuda/expert_schedule.cuh:11-69), exl3_masked::Schedule (expert_exl3_prefill_masked.cuh:12-45)
inline void Group(const int *ids, int *groups, int *counts, int tokens, int *bad, cudaStream_t s) {
  Check(padra_expert_group(ids, groups, counts, tokens, bad, s));
}
inline void Schedule(const int *counts, mellum16::exl3_masked_schedule::Tile *tiles, int *n, int tokens, int *bad, cudaStream_t s) {
  Check(padra_exl3_schedule(counts, reinterpret_cast<padra_tile *>(tiles), n, tokens, bad, s));
}
// exl3_transport_async64::Launch (K4, src/cuda/expert_exl3_prefill_transport_async64.cuh:136-157) and
// exl3_packed_activations::Launch (K3/K6, src/cuda/expert_exl3_prefill_packed_activations.cuh:250-277): inference.cu:3896-3921
inline void PrefillLaunch(const mellum16::DeviceMatrix *m, int layer, int part, const int *ids, const int *groups,
                          const int *counts, const mellum16::exl3_masked_schedule::Tile *tiles, const int *tile_count,
                          const float *in, unsigned short *out, const unsigned short *gate, const unsigned short *up,
                          const unsigned short *table, __half *workspace, int tokens, int *bad, cudaStream_t s,
                          unsigned *stats = nullptr, bool wide = false, int rate = 4) {
  Check(padra_exl3_prefill_launch(M(m), layer, part, ids, groups, counts, reinterpret_cast<const padra_tile *>(tiles), tile_count, in,
                                  out, gate, up, table, workspace, tokens, bad, s, stats, wide ? 1 : 0, rate, kHidden, kInter));
}
// The gate and up launches of a prefill chunk (parts 0 and 1 of the call above, src/cuda/inference.cu:3896-3907) as one:
// both parts' work items form one list.  `workspace` holds 2 * tokens * 8 * 2304 halves.
inline void PrefillGateUpLaunch(const mellum16::DeviceMatrix *m, int layer, const int *groups, const int *counts, const float *in,
                                unsigned short *gate_out, unsigned short *up_out, __half *workspace, int tokens, int *bad,
                                cudaStream_t s, int rate) {
  Check(padra_exl3_prefill_gate_up_launch(M(m), layer, groups, counts, in, gate_out, up_out, workspace, tokens, bad, s, rate, kHidden,
                                          kInter));
}
// exl3_packed_activations::Combine, src/cuda/expert_exl3_prefill_packed_activations.cuh:86-103
inline void CombinePacked(float *x, const unsigned short *down, const float *w, int tokens, int *bad, bool residual, cudaStream_t s) {
  Check(padra_combine_packed(x, down, w, tokens, bad, residual ? 1 : 0, kHidden, s));
}
// exl3_expert::Launch, src/cuda/expert_exl3.cuh:137-151 (T < 4).  The reference's trailing `bool fp32` keeps the
// transformed input unrounded (a diagnostic form, :34,55) and `unsigned *ranges` collects value statistics (:114-136,
// :144-146); this library computes the production form only and keeps no statistics, so both are accepted and dropped.
inline void ExpertLaunch(const mellum16::DeviceMatrix *m, int layer, int part, const int *ids, const float *in, float *out,
                         float *in_scratch, float *out_scratch, int tokens, int *bad, cudaStream_t s, bool fp32 = false,
                         unsigned *ranges = nullptr, int rate = 4) {
  (void)fp32;
  (void)ranges;
  Check(padra_exl3_expert_launch(M(m), layer, part, ids, in, out, in_scratch, out_scratch, tokens, bad, s, rate, kHidden, kInter));
}
// The whole decode layer in one call: replaces expert(l,0) ... Combine of inference.cu:2963-2975 (one token) and
// :3375-3392 (verifier rows).  `workspace` holds padra_exl3_moe_decode_workspace_bytes(rows, ...) bytes and was passed
// to padra_exl3_moe_decode_workspace_init once after allocation.
inline void DecodeLayer(const mellum16::DeviceMatrix *m, int layer, const int *ids, const float *routing, const float *normalized,
                        float *x, int rows, int rate, const unsigned short *table, void *workspace, std::size_t workspace_bytes,
                        int *bad, cudaStream_t s) {
  Check(padra_exl3_moe_decode_layer(M(m), layer, ids, routing, normalized, x, rows, rate, kHidden, kInter, table, workspace,
                                    workspace_bytes, bad, s));
}

// The expert layer of the MTP draft model (src/cuda/mtp.cuh:370-387): one K4 layer with a descriptor table of its own
// (layer 0), one token.  Replaces Projection<4><<<dim3(7, 8, 2)>>> (gate+up), Activate<<<56, 128>>>,
// Projection<4><<<dim3(18, 8)>>> (down) and Combine<<<18, 128>>> with one call; ids and routing weights come from the
// draft's own Route kernel as before.
inline void DraftExpertLayer(const mellum16::DeviceMatrix *draft_descriptors, const int *ids, const float *routing_weights,
                             const float *normalized, float *x, const unsigned short *table, void *workspace,
                             std::size_t workspace_bytes, int *bad, cudaStream_t s) {
  DecodeLayer(draft_descriptors, 0, ids, routing_weights, normalized, x, 1, 4, table, workspace, workspace_bytes, bad, s);
}

// RouteRankExact<<<rows, 64>>> (src/cuda/router_rank_exact.cuh:3-81; inference.cu:2950, :3366).
inline void RouteRankExact(const float *logits, int *ids, float *weights, int rows, int *bad, cudaStream_t s) {
  Check(padra_route(logits, ids, weights, rows, bad, s));
}
// Route + fast_expert::Group + exl3_masked::Schedule of one prefill chunk (inference.cu:3861, :3875, :3890) as one
// launch.  `ticket` is one zeroed word of device memory that every call leaves zero.
inline void RouteGroupSchedule(const float *logits, int *ids, float *weights, int *groups, int *counts,
                               mellum16::exl3_masked_schedule::Tile *tiles, int *tile_count, int tokens, unsigned *ticket,
                               int *bad, cudaStream_t s) {
  Check(padra_route_group_schedule(logits, ids, weights, groups, counts, reinterpret_cast<padra_tile *>(tiles), tile_count,
                                   tokens, ticket, bad, s));
}
// ResidualPostNormWideExact<<<rows, 256>>> (src/cuda/residual_norm_wide_exact.cuh:82-131; inference.cu:2913, :3358).
// The norm weight is a BF16 vector descriptor: its data pointer is passed on.
inline void ResidualPostNorm(float *x, const float *residual, float *normalized, const mellum16::DeviceMatrix &weight, int *bad,
                             float *statistics, int rows, cudaStream_t s) {
  Check(padra_residual_norm(x, residual, normalized, reinterpret_cast<const unsigned short *>(weight.data), rows, kHidden, bad,
                            statistics, s));
}
// combine_norm_exact::CombineNorm<false><<<1, 128>>> (src/cuda/combine_norm_exact.cuh:7-68), extended to `rows` rows.
inline void CombineNorm(float *x, const float *down, const float *routing, float *normalized, const mellum16::DeviceMatrix &weight,
                        int *bad, float *statistics, int rows, cudaStream_t s) {
  Check(padra_combine_norm(x, down, routing, normalized, reinterpret_cast<const unsigned short *>(weight.data), rows, kHidden, bad,
                           statistics, s));
}

} // namespace padra_b200_bind
