// Host-side launchers shared between translation units; the C ABI (api.cu) is a thin layer over these.
#pragma once
#include "common.cuh"

namespace padra {

int LaunchPairProjection(const Matrix *matrices, int layer, int part, const int *ids, const float *input, float *output,
                         float *other, int pairs, int *bad, cudaStream_t stream, int rate, int hidden, int inter,
                         bool gate_and_up = true);
int LaunchUnionProjection(const Matrix *matrices, int layer, int part, const unsigned *masks, const int *slots,
                          int slot_stride, int rows, const float *input, float *output, float *up, int *bad,
                          cudaStream_t stream, const int *active, const int *active_count, int rate, int hidden,
                          int inter);
int LaunchBuildUnion(const int *ids, unsigned *masks, int *slots, int rows, int slot_stride, int *bad, int *active,
                     int *active_count, cudaStream_t stream);
int LaunchSiluBuild(unsigned short *table, cudaStream_t stream);
int LaunchSiluActivate(float *gate, const float *up, const unsigned short *table, int count, int *bad,
                       cudaStream_t stream);
int LaunchCombine(float *x, const float *down, const float *weights, int *bad, int rows, int hidden,
                  cudaStream_t stream);
int LaunchCombinePacked(float *x, const unsigned short *down, const float *weights, int tokens, int *bad, int residual,
                        int hidden, cudaStream_t stream);
int LaunchDecodeWeights(const Matrix *matrix, unsigned short *out, int rows, int cols, int rate, int *bad,
                        cudaStream_t stream);

size_t DecodeLayerWorkspaceBytes(int tokens, int hidden, int inter);
int InitDecodeLayerWorkspace(void *workspace, size_t bytes, cudaStream_t stream);
// launches: bit 0 the gate+up kernel, bit 1 the down kernel (both: the whole layer)
int LaunchDecodeLayer(const Matrix *matrices, int layer, const int *ids, const float *routing, const float *normalized, float *x,
                      int tokens, int rate, int hidden, int inter, const unsigned short *table, void *workspace,
                      size_t workspace_bytes, int *bad, cudaStream_t stream, unsigned launches = 3u);
int LaunchRoute(const float *logits, int *ids, float *weights, int tokens, int *bad, cudaStream_t stream);
int LaunchRouteGroupSchedule(const float *logits, int *ids, float *weights, int *groups, int *counts, padra_tile *tiles, int *tile_count,
                             int tokens, unsigned *ticket, int *bad, cudaStream_t stream);
int LaunchResidualNorm(float *x, const float *residual, float *normalized, const unsigned short *weight, int rows, int hidden, int *bad,
                       float *statistics, cudaStream_t stream);
int LaunchCombineNorm(float *x, const float *down, const float *routing, float *normalized, const unsigned short *weight, int rows,
                      int hidden, int *bad, float *statistics, cudaStream_t stream);
int LaunchCodecCeiling(int rate, int form, int iterations, int blocks, unsigned *sink, cudaStream_t stream);
int LaunchDecodeWeightsTensor(const Matrix *matrix, unsigned short *out, int rows, int cols, int rate, int *bad, cudaStream_t stream);
int LaunchTileProjection(const Matrix *matrices, int layer, int part, const int *groups, const padra_tile *tiles,
                         const int *tile_count, const float *input, unsigned short *output,
                         const unsigned short *gate, const unsigned short *up, const unsigned short *table, int tokens,
                         int *bad, cudaStream_t stream, int rate, int hidden, int inter);
int LaunchPrefillRows(const Matrix *matrices, int layer, int part, const int *groups, const int *counts, int group_stride, int rows,
                      const unsigned short *input_rows, unsigned short *output, const unsigned short *gate,
                      const unsigned short *up, const unsigned short *table, void *transformed, int *bad, cudaStream_t stream,
                      int rate, int hidden, int inter, int block_begin = 0, int block_count = 0);
size_t ExchangeBytes(int world, int cap, int hidden, size_t *offsets);
int LaunchDispatch(const float *activations, const int *order, const int *send_ids, const long long *send_counts,
                   const unsigned long long *bases, int rank, int world, int cap, int pairs, int hidden, unsigned epoch, int *bad,
                   cudaStream_t stream);
int SetExchangeWaitLimit(int milliseconds);
int SetPrefillReservedSms(int sms);
int LaunchWaitFlags(const void *block, int which, int world, int cap, int hidden, unsigned epoch, int *bad, cudaStream_t stream);
int LaunchGroupRegions(const void *block, int world, int cap, int hidden, int *groups, int *counts, int group_stride, int *bad,
                       cudaStream_t stream);
int LaunchReturn(const unsigned short *down, const unsigned long long *bases, int rank, int world, int cap, int hidden, unsigned epoch,
                 int *bad, cudaStream_t stream, int column_begin = 0, int column_count = 0, int announce = 1);
int LaunchPlan(const int *ids, const int *owner, int *order, int *position, int *send_ids, long long *send_counts, int pairs,
               int world, int *bad, cudaStream_t stream);
int LaunchPrefillDownReturn(const Matrix *matrices, int layer, const int *groups, const int *counts, int group_stride,
                            const unsigned short *gate, const unsigned short *up, const unsigned short *table, void *transformed,
                            const unsigned long long *bases, int rank, int world, int cap, unsigned epoch, int *bad, cudaStream_t stream,
                            int rate, int hidden, int inter);
int LaunchGroupRows(const int *ids, int *groups, int *counts, int rows, int group_stride, int *bad, cudaStream_t stream);
int LaunchPackRows(const float *activations, const int *order, unsigned short *packed, int rows, int hidden, int *bad,
                   cudaStream_t stream);
int LaunchCombineIndexed(float *x, const unsigned short *down_rows, const int *position, const float *weights, int tokens,
                         int *bad, int residual, int hidden, cudaStream_t stream);
int LaunchPrefillTensorMemory(const Matrix *matrices, int layer, int part, const int *groups, const int *counts, const float *input,
                              unsigned short *output, const unsigned short *gate, const unsigned short *up,
                              const unsigned short *table, void *transformed, int tokens, int *bad, cudaStream_t stream, int rate,
                              int hidden, int inter);
int LaunchPrefillGateUp(const Matrix *matrices, int layer, const int *groups, const int *counts, const float *input,
                        unsigned short *gate_output, unsigned short *up_output, void *transformed, int tokens, int *bad, cudaStream_t stream,
                        int rate, int hidden, int inter);
int LaunchPrefillRowsGateUp(const Matrix *matrices, int layer, const int *groups, const int *counts, int group_stride, int rows,
                            const unsigned short *input_rows, unsigned short *gate_output, unsigned short *up_output, void *transformed,
                            int *bad, cudaStream_t stream, int rate, int hidden, int inter);
int LaunchGroup(const int *ids, int *groups, int *counts, int tokens, int *bad, cudaStream_t stream);
int LaunchSchedule(const int *counts, padra_tile *tiles, int *tile_count, int tokens, int *bad, cudaStream_t stream);
int LaunchPrefill(const Matrix *matrices, int layer, int part, const int *ids, const int *groups, const int *counts,
                  const float *input, unsigned short *output, const unsigned short *gate, const unsigned short *up,
                  const unsigned short *table, void *transformed, int tokens, int *bad, cudaStream_t stream, int rate,
                  int hidden, int inter);

} // namespace padra
