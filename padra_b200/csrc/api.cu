// The C ABI of the library: argument checks, then the launchers.  No allocation, no synchronisation.
#include "kernels.cuh"

using namespace padra;

namespace {
cudaStream_t S(padra_stream s) {
  return static_cast<cudaStream_t>(s);
}
bool RateOk(int rate) {
  return rate == 3 || rate == 4 || rate == 6;
}
} // namespace

extern "C" {

int padra_version(void) {
  return 100; // 0.1.0
}

const char *padra_status_string(int status) {
  switch (status) {
  case PADRA_OK:
    return "ok";
  case PADRA_INVALID_ARGUMENT:
    return "invalid argument";
  case PADRA_UNSUPPORTED:
    return "unsupported";
  case PADRA_RESOURCE_EXHAUSTED:
    return "resource exhausted";
  case PADRA_INTERNAL:
    return "internal (CUDA error)";
  default:
    return "unknown status";
  }
}

int padra_device_supported(void) {
  int device = 0, major = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess)
    return PADRA_INTERNAL;
  return major == 10 ? PADRA_OK : PADRA_UNSUPPORTED;
}

int padra_exl3_decode_launch(const padra_matrix *matrices, int layer, int part, const int *ids, const float *input,
                             float *output, float *scratch, int pairs, int *bad, padra_stream stream, unsigned *ranges,
                             float *other_output, int rate, int hidden, int inter) {
  (void)scratch;
  (void)ranges;
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  return LaunchPairProjection(matrices, layer, part, ids, input, output, other_output, pairs, bad, S(stream), rate,
                              hidden, inter);
}

int padra_mtp_build_union(const int *ids, unsigned *masks, int *slots, int rows, int *bad, int *active_experts,
                          int *active_count, padra_stream stream, int slot_stride) {
  return LaunchBuildUnion(ids, masks, slots, rows, slot_stride, bad, active_experts, active_count, S(stream));
}

int padra_mtp_experts_launch(const padra_matrix *matrices, int layer, int part, const unsigned *masks, const int *slots,
                             int rows, const float *input, float *output, float *up, int *bad, padra_stream stream,
                             const int *active_experts, const int *active_count, int rate, int hidden, int inter,
                             int slot_stride) {
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  return LaunchUnionProjection(matrices, layer, part, masks, slots, slot_stride, rows, input, output, up, bad, S(stream),
                               active_experts, active_count, rate, hidden, inter);
}

int padra_exl3_silu_build(unsigned short *table, padra_stream stream) {
  return LaunchSiluBuild(table, S(stream));
}

int padra_exl3_silu_activate(float *gate, const float *up, const unsigned short *table, int count, int *bad,
                             padra_stream stream) {
  return LaunchSiluActivate(gate, up, table, count, bad, S(stream));
}

int padra_combine(float *x, const float *down, const float *weights, int *bad, int rows, int hidden,
                  padra_stream stream) {
  return LaunchCombine(x, down, weights, bad, rows, hidden, S(stream));
}

int padra_combine_packed(float *x, const unsigned short *down, const float *weights, int tokens, int *bad, int residual,
                         int hidden, padra_stream stream) {
  return LaunchCombinePacked(x, down, weights, tokens, bad, residual, hidden, S(stream));
}

int padra_expert_group(const int *ids, int *groups, int *counts, int tokens, int *bad, padra_stream stream) {
  return LaunchGroup(ids, groups, counts, tokens, bad, S(stream));
}

int padra_exl3_schedule(const int *counts, padra_tile *tiles, int *tile_count, int tokens, int *bad,
                        padra_stream stream) {
  return LaunchSchedule(counts, tiles, tile_count, tokens, bad, S(stream));
}

int padra_exl3_prefill_launch(const padra_matrix *matrices, int layer, int part, const int *ids, const int *groups,
                              const int *counts, const padra_tile *tiles, const int *tile_count, const float *input,
                              unsigned short *output, const unsigned short *gate, const unsigned short *up,
                              const unsigned short *table, void *transformed, int tokens, int *bad, padra_stream stream,
                              unsigned *stats, int wide_input, int rate, int hidden, int inter) {
  (void)stats;
  (void)ids;
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  if (tokens < 4 || tokens > 2048 || part < 0 || part > 2) // the reference throws below four tokens
    return PADRA_INVALID_ARGUMENT;
  if (!matrices || !groups || !tiles || !tile_count || !output || !bad || hidden < 128 || inter < 128 ||
      (hidden % 128) || (inter % 128) || (part == 2 ? (!gate || !up || !table) : !input))
    return PADRA_INVALID_ARGUMENT;
  // wide_input: 0 = the 32-pair tile kernel on the tensor-core fragments path, 1 = the tensor-memory grouped GEMM
  // (needs `transformed` and `counts`), which is what a caller with the reference's selected options passes
  // (src/runtime/model_runtime.cpp:22-34 sets exl3_wide_input).
  if (wide_input && transformed && counts)
    return LaunchPrefillTensorMemory(matrices, layer, part, groups, counts, input, output, gate, up, table, transformed, tokens, bad,
                                     S(stream), rate, hidden, inter);
  return LaunchTileProjection(matrices, layer, part, groups, tiles, tile_count, input, output, gate, up, table, tokens,
                              bad, S(stream), rate, hidden, inter);
}

int padra_exl3_prefill_gate_up_launch(const padra_matrix *matrices, int layer, const int *groups, const int *counts,
                                      const float *input, unsigned short *gate_output, unsigned short *up_output, void *transformed,
                                      int tokens, int *bad, padra_stream stream, int rate, int hidden, int inter) {
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  if (tokens < 4 || tokens > 2048)
    return PADRA_INVALID_ARGUMENT;
  if (!matrices || !groups || !counts || !input || !gate_output || !up_output || !transformed || !bad || layer < 0 || hidden < 128 ||
      inter < 128 || (hidden % 128) || (inter % 128))
    return PADRA_INVALID_ARGUMENT;
  return LaunchPrefillGateUp(matrices, layer, groups, counts, input, gate_output, up_output, transformed, tokens, bad, S(stream), rate,
                             hidden, inter);
}

int padra_exl3_prefill_rows_gate_up_launch(const padra_matrix *matrices, int layer, const int *groups, const int *counts,
                                           int group_stride, int rows, const unsigned short *input_rows, unsigned short *gate_output,
                                           unsigned short *up_output, void *transformed, int *bad, padra_stream stream, int rate,
                                           int hidden, int inter) {
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  if (!matrices || !groups || !counts || !input_rows || !gate_output || !up_output || !transformed || !bad || layer < 0 || hidden < 128 ||
      inter < 128 || (hidden % 128) || (inter % 128))
    return PADRA_INVALID_ARGUMENT;
  return LaunchPrefillRowsGateUp(matrices, layer, groups, counts, group_stride, rows, input_rows, gate_output, up_output, transformed, bad,
                                 S(stream), rate, hidden, inter);
}

size_t padra_ep_exchange_bytes(int world, int cap, int hidden, size_t *offsets) {
  return ExchangeBytes(world, cap, hidden, offsets);
}

int padra_ep_dispatch(const float *activations, const int *order, const int *send_ids, const long long *send_counts,
                      const unsigned long long *peer_blocks, int rank, int world, int cap, int pairs, int hidden, unsigned epoch,
                      int *bad, padra_stream stream) {
  return LaunchDispatch(activations, order, send_ids, send_counts, peer_blocks, rank, world, cap, pairs, hidden, epoch, bad, S(stream));
}

int padra_ep_wait(const void *block, int which, int world, int cap, int hidden, unsigned epoch, int *bad, padra_stream stream) {
  return LaunchWaitFlags(block, which, world, cap, hidden, epoch, bad, S(stream));
}

int padra_ep_set_wait_limit_ms(int milliseconds) {
  return SetExchangeWaitLimit(milliseconds);
}

int padra_prefill_set_reserved_sms(int sms) {
  return SetPrefillReservedSms(sms);
}

int padra_ep_group_received(const void *block, int world, int cap, int hidden, int *groups, int *counts, int group_stride, int *bad,
                            padra_stream stream) {
  return LaunchGroupRegions(block, world, cap, hidden, groups, counts, group_stride, bad, S(stream));
}

int padra_ep_return(const unsigned short *down_rows, const unsigned long long *peer_blocks, int rank, int world, int cap, int hidden,
                    unsigned epoch, int *bad, padra_stream stream, int column_begin, int column_count, int announce) {
  return LaunchReturn(down_rows, peer_blocks, rank, world, cap, hidden, epoch, bad, S(stream), column_begin, column_count, announce);
}

int padra_ep_down_return(const padra_matrix *matrices, int layer, const int *groups, const int *counts, int group_stride,
                         const unsigned short *gate, const unsigned short *up, const unsigned short *table, void *transformed,
                         const unsigned long long *peer_blocks, int rank, int world, int cap, unsigned epoch, int *bad,
                         padra_stream stream, int rate, int hidden, int inter) {
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  if (!matrices || !groups || !counts || !gate || !up || !table || !transformed || !peer_blocks || !bad || layer < 0 || hidden < 128 ||
      inter < 128 || (hidden % 128) || (inter % 128))
    return PADRA_INVALID_ARGUMENT;
  return LaunchPrefillDownReturn(matrices, layer, groups, counts, group_stride, gate, up, table, transformed, peer_blocks, rank, world,
                                 cap, epoch, bad, S(stream), rate, hidden, inter);
}

int padra_ep_plan(const int *ids, const int *owner, int *order, int *position, int *send_ids, long long *send_counts, int pairs,
                  int world, int *bad, padra_stream stream) {
  return LaunchPlan(ids, owner, order, position, send_ids, send_counts, pairs, world, bad, S(stream));
}

int padra_ep_pack_rows(const float *activations, const int *order, unsigned short *packed, int rows, int hidden, int *bad,
                       padra_stream stream) {
  return LaunchPackRows(activations, order, packed, rows, hidden, bad, S(stream));
}

int padra_ep_group_rows(const int *ids, int *groups, int *counts, int rows, int group_stride, int *bad, padra_stream stream) {
  return LaunchGroupRows(ids, groups, counts, rows, group_stride, bad, S(stream));
}

int padra_exl3_prefill_rows_launch(const padra_matrix *matrices, int layer, int part, const int *groups, const int *counts,
                                   int group_stride, int rows, const unsigned short *input_rows, unsigned short *output,
                                   const unsigned short *gate, const unsigned short *up, const unsigned short *table,
                                   void *transformed, int *bad, padra_stream stream, int rate, int hidden, int inter,
                                   int block_begin, int block_count) {
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  if (!matrices || !groups || !counts || !output || !transformed || !bad || part < 0 || part > 2 || layer < 0 || hidden < 128 ||
      inter < 128 || (hidden % 128) || (inter % 128) || (part == 2 ? (!gate || !up || !table) : !input_rows))
    return PADRA_INVALID_ARGUMENT;
  return LaunchPrefillRows(matrices, layer, part, groups, counts, group_stride, rows, input_rows, output, gate, up, table,
                           transformed, bad, S(stream), rate, hidden, inter, block_begin, block_count);
}

int padra_ep_combine(float *x, const unsigned short *down_rows, const int *position, const float *weights, int tokens, int *bad,
                     int residual, int hidden, padra_stream stream) {
  return LaunchCombineIndexed(x, down_rows, position, weights, tokens, bad, residual, hidden, S(stream));
}

int padra_exl3_expert_launch(const padra_matrix *matrices, int layer, int part, const int *ids, const float *input,
                             float *output, float *in_scratch, float *out_scratch, int tokens, int *bad,
                             padra_stream stream, int rate, int hidden, int inter) {
  (void)in_scratch;
  (void)out_scratch;
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  if (tokens < 1 || part < 0 || part > 2)
    return PADRA_INVALID_ARGUMENT;
  // one part per call, FP32-held BF16 out, exactly like the reference's small-batch launcher
  return LaunchPairProjection(matrices, layer, part, ids, input, output, nullptr, tokens * kTopK, bad, S(stream), rate,
                              hidden, inter, /*gate_and_up=*/false);
}

size_t padra_exl3_moe_decode_workspace_bytes(int tokens, int hidden, int inter) {
  if (tokens < 1 || tokens > kMaxDecodeRows || hidden < 128 || inter < 128 || (hidden % 128) || (inter % 128))
    return 0;
  return DecodeLayerWorkspaceBytes(tokens, hidden, inter);
}

int padra_exl3_moe_decode_workspace_init(void *workspace, size_t workspace_bytes, padra_stream stream) {
  return InitDecodeLayerWorkspace(workspace, workspace_bytes, S(stream));
}

int padra_exl3_moe_decode_layer(const padra_matrix *matrices, int layer, const int *ids, const float *routing,
                                const float *normalized, float *x, int tokens, int rate, int hidden, int inter,
                                const unsigned short *table, void *workspace, size_t workspace_bytes, int *bad,
                                padra_stream stream) {
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  if (!matrices || !ids || !routing || !normalized || !x || !table || !workspace || !bad || tokens < 1 ||
      tokens > kMaxDecodeRows || hidden < 128 || inter < 128 || (hidden % 128) || (inter % 128) || layer < 0)
    return PADRA_INVALID_ARGUMENT;
  return LaunchDecodeLayer(matrices, layer, ids, routing, normalized, x, tokens, rate, hidden, inter, table, workspace,
                           workspace_bytes, bad, S(stream));
}

int padra_exl3_moe_decode_layer_launches(const padra_matrix *matrices, int layer, const int *ids, const float *routing,
                                         const float *normalized, float *x, int tokens, int rate, int hidden, int inter,
                                         const unsigned short *table, void *workspace, size_t workspace_bytes, int *bad,
                                         padra_stream stream, unsigned launches) {
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  if (!matrices || !ids || !routing || !normalized || !x || !table || !workspace || !bad || tokens < 1 ||
      tokens > kMaxDecodeRows || hidden < 128 || inter < 128 || (hidden % 128) || (inter % 128) || layer < 0 || launches > 3u)
    return PADRA_INVALID_ARGUMENT;
  return LaunchDecodeLayer(matrices, layer, ids, routing, normalized, x, tokens, rate, hidden, inter, table, workspace,
                           workspace_bytes, bad, S(stream), launches);
}

int padra_route(const float *logits, int *ids, float *weights, int tokens, int *bad, padra_stream stream) {
  return LaunchRoute(logits, ids, weights, tokens, bad, S(stream));
}

int padra_route_group_schedule(const float *logits, int *ids, float *weights, int *groups, int *counts, padra_tile *tiles,
                               int *tile_count, int tokens, unsigned *ticket, int *bad, padra_stream stream) {
  return LaunchRouteGroupSchedule(logits, ids, weights, groups, counts, tiles, tile_count, tokens, ticket, bad, S(stream));
}

int padra_residual_norm(float *x, const float *residual, float *normalized, const unsigned short *weight, int rows, int hidden,
                        int *bad, float *statistics, padra_stream stream) {
  return LaunchResidualNorm(x, residual, normalized, weight, rows, hidden, bad, statistics, S(stream));
}

int padra_combine_norm(float *x, const float *down, const float *routing, float *normalized, const unsigned short *weight, int rows,
                       int hidden, int *bad, float *statistics, padra_stream stream) {
  return LaunchCombineNorm(x, down, routing, normalized, weight, rows, hidden, bad, statistics, S(stream));
}

int padra_codec_ceiling_launch(int rate, int form, int iterations, int blocks, unsigned *sink, padra_stream stream) {
  return LaunchCodecCeiling(rate, form, iterations, blocks, sink, S(stream));
}

int padra_exl3_decode_weights_tensor(const padra_matrix *matrix, unsigned short *out, int rows, int cols, int rate, int *bad,
                                     padra_stream stream) {
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  return LaunchDecodeWeightsTensor(matrix, out, rows, cols, rate, bad, S(stream));
}

int padra_exl3_decode_weights(const padra_matrix *matrix, unsigned short *out, int rows, int cols, int rate, int *bad,
                              padra_stream stream) {
  if (!RateOk(rate))
    return PADRA_UNSUPPORTED;
  return LaunchDecodeWeights(matrix, out, rows, cols, rate, bad, S(stream));
}

} // extern "C"
