/*
 * padra_b200 -- C ABI of the B200 (sm_100a) EXL3 mixture-of-experts expert kernels.
 *
 * Every entry point takes plain device pointers and sizes, enqueues work on the given CUDA stream and
 * returns at once; none of them allocates, frees, synchronises or reads device memory on the host, so the
 * entry points that stand in for a reference launcher may be recorded into CUDA graphs.  Activations follow the reference's conventions: decode-side
 * buffers are `float` arrays holding BF16-representable values, prefill-side buffers are BF16 bit patterns
 * in `unsigned short`.  Errors discovered on the device (a descriptor that does not fit the call, an expert
 * id outside 0..63, a non-finite or FP16-overflowing value) set the caller's sticky `*bad` flag with an
 * atomic exchange and skip the affected work; nothing traps.  Host-side argument errors are returned as a
 * status code whose values equal mellum16::StatusCode (include/mellum16/status.h:11-21).
 *
 * The reference has no FFI for this path: its launchers are inline host functions in headers of one
 * translation unit.  Each function below names the reference launcher (file:line) whose argument list it
 * keeps; the trailing `hidden` / `inter` arguments replace the Mellum dimensions (2304 / 896) the reference
 * hard-codes, and `stream` is a cudaStream_t.
 */
#ifndef PADRA_B200_H
#define PADRA_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define PADRA_API
#else
#define PADRA_API __attribute__((visibility("default")))
#endif

/* Status codes: numerically mellum16::StatusCode (include/mellum16/status.h:11-21). */
enum {
  PADRA_OK = 0,
  PADRA_INVALID_ARGUMENT = 1,
  PADRA_UNSUPPORTED = 5,
  PADRA_RESOURCE_EXHAUSTED = 6,
  PADRA_INTERNAL = 8
};

/* Weight descriptor: field for field the reference's DeviceMatrix (src/cuda/device_matrix.cuh:6-13),
 * 56 bytes.  rows = outputs, cols = inputs; format 3 = K4, 5 = K6, 6 = K3 (:30-44).  data holds
 * (cols/16)*(rows/16) tiles of 32*rate bytes, input-block-major; suh/svh are FP16 bit patterns. */
typedef struct padra_matrix {
  const unsigned char *data;
  const unsigned char *scales;
  const float *divisor;
  int rows, cols, format;
  const uint16_t *suh;
  const uint16_t *svh;
} padra_matrix;

/* Prefill tile descriptor: src/runtime/exl3_masked_schedule.h:6-8. */
typedef struct padra_tile {
  int expert, begin, valid_rows;
} padra_tile;

typedef void *padra_stream; /* cudaStream_t */

PADRA_API int padra_version(void);
PADRA_API const char *padra_status_string(int status);
/* Returns PADRA_OK when the current device is an sm_100 part this library's kernels were built for. */
PADRA_API int padra_device_supported(void);

/* ---- decode, M = 1 --------------------------------------------------------------------------------
 * exl3_mma_dual::Launch (src/cuda/expert_exl3_decode_dual.cuh:132-146).  matrices is the table indexed
 * (layer*64+expert)*3+part, part 0 = gate, 1 = up, 2 = down.  ids[pairs] are expert ids.  part == 0 computes
 * gate into output and up into other_output in one launch.  Input row is pair/8 for gate/up and pair for
 * down; output row is pair.  scratch and ranges are accepted for signature compatibility and unused. */
PADRA_API int padra_exl3_decode_launch(const padra_matrix *matrices, int layer, int part, const int *ids,
                                       const float *input, float *output, float *scratch, int pairs, int *bad,
                                       padra_stream stream, unsigned *ranges, float *other_output, int rate,
                                       int hidden, int inter);

/* ---- decode, M = 2..16 rows sharing decoded tiles ---------------------------------------------------
 * mtp_experts::BuildUnion<true> (src/cuda/mtp_experts.cuh:7-40): per expert a row mask, the slot each row
 * used, and the ascending list of active experts.  slots is [64][slot_stride]; the reference fixes the
 * stride at 5 (its kRows) and rows at 2..5, this library accepts rows 1..16 with slot_stride >= rows. */
PADRA_API int padra_mtp_build_union(const int *ids, unsigned *masks, int *slots, int rows, int *bad,
                                    int *active_experts, int *active_count, padra_stream stream, int slot_stride);
/* mtp_experts::Launch (src/cuda/mtp_experts.cuh:225-245).  Gate/up read input row r, down reads row
 * r*8+slot; every part writes output row r*8+slot.  part == 0 writes gate to output and up to `up`. */
PADRA_API int padra_mtp_experts_launch(const padra_matrix *matrices, int layer, int part, const unsigned *masks,
                                       const int *slots, int rows, const float *input, float *output, float *up,
                                       int *bad, padra_stream stream, const int *active_experts,
                                       const int *active_count, int rate, int hidden, int inter, int slot_stride);

/* ---- SwiGLU -------------------------------------------------------------------------------------------
 * exl3_silu_lut::Build / Activate (src/cuda/exl3_silu_lut.cuh:9-31): table[65536] maps the BF16 bits of g
 * to the BF16 bits of silu(g); gate[i] = B(table[gate[i]] * up[i]). */
PADRA_API int padra_exl3_silu_build(unsigned short *table, padra_stream stream);
PADRA_API int padra_exl3_silu_activate(float *gate, const float *up, const unsigned short *table, int count,
                                       int *bad, padra_stream stream);

/* ---- combine ------------------------------------------------------------------------------------------
 * Combine (src/cuda/inference.cu:580-594): x[r] = B(x[r] + sum), sum = B(sum + B(down[r][s] * weights[r][s]))
 * over the eight slots in order.  rows tokens, x [rows][hidden], down [rows][8][hidden]. */
PADRA_API int padra_combine(float *x, const float *down, const float *weights, int *bad, int rows, int hidden,
                            padra_stream stream);
/* exl3_packed_activations::Combine (src/cuda/expert_exl3_prefill_packed_activations.cuh:86-103): the same
 * with BF16-bit down rows; residual == 0 stores the sum alone. */
PADRA_API int padra_combine_packed(float *x, const unsigned short *down, const float *weights, int tokens,
                                   int *bad, int residual, int hidden, padra_stream stream);

/* ---- prefill scheduling -------------------------------------------------------------------------------
 * fast_expert::Group (src/cuda/expert_schedule.cuh:11-69): groups[e*tokens + n] = n-th pair (token*8+slot)
 * routed to expert e in ascending pair order, counts[e] their number; validates ids and per-token uniqueness.
 * exl3_masked::Schedule (src/cuda/expert_exl3_prefill_masked.cuh:12-45): tiles of at most 32 pairs,
 * experts ascending; capacity (tokens*8+31)/32+64 (src/runtime/exl3_masked_schedule.h:15-17). */
PADRA_API int padra_expert_group(const int *ids, int *groups, int *counts, int tokens, int *bad,
                                 padra_stream stream);
PADRA_API int padra_exl3_schedule(const int *counts, padra_tile *tiles, int *tile_count, int tokens, int *bad,
                                  padra_stream stream);

/* ---- prefill projection, T >= 4 -----------------------------------------------------------------------
 * exl3_transport_async64::Launch (src/cuda/expert_exl3_prefill_transport_async64.cuh:136-157) for K4 and
 * exl3_packed_activations::Launch (src/cuda/expert_exl3_prefill_packed_activations.cuh:250-277) for K3/K6:
 * one argument list for all three rates.  input is FP32-held BF16 [tokens][hidden] (parts 0, 1); gate/up are
 * BF16-bit [pairs][inter] (part 2, SwiGLU applied while building the down input); output is BF16-bit
 * [pairs][rows]; transformed is workspace of pairs*cols halves.  tiles/tile_count/counts/ids are read only
 * through `groups` and `counts` here; stats is accepted and unused.  wide_input (set by the reference's
 * selected server options) selects the tensor-memory grouped GEMM (tcgen05, 128 outputs x up to 256 tokens per
 * CTA); 0 selects the small-tile kernel (32 pairs per CTA).
 * Returns PADRA_INVALID_ARGUMENT for tokens < 4, where the reference throws. */
PADRA_API int padra_exl3_prefill_launch(const padra_matrix *matrices, int layer, int part, const int *ids,
                                        const int *groups, const int *counts, const padra_tile *tiles,
                                        const int *tile_count, const float *input, unsigned short *output,
                                        const unsigned short *gate, const unsigned short *up,
                                        const unsigned short *table, void *transformed, int tokens, int *bad,
                                        padra_stream stream, unsigned *stats, int wide_input, int rate,
                                        int hidden, int inter);

/* Gate and up of a chunk in ONE launch of the tensor-memory grouped GEMM (the reference launches the two parts one
 * after the other, src/cuda/inference.cu:3896-3907): the work items of both parts form one list, so the persistent CTAs
 * are loaded evenly (1248 equal items on 148 SMs instead of two times 624).  Arguments as padra_exl3_prefill_launch
 * with wide_input = 1; gate_output / up_output are the two parts' [pairs][inter] BF16-bit outputs; transformed is
 * workspace of 2*pairs*hidden halves (both parts' transformed rows).  Results equal those of the two separate calls. */
PADRA_API int padra_exl3_prefill_gate_up_launch(const padra_matrix *matrices, int layer, const int *groups,
                                                const int *counts, const float *input, unsigned short *gate_output,
                                                unsigned short *up_output, void *transformed, int tokens, int *bad,
                                                padra_stream stream, int rate, int hidden, int inter);

/* ---- expert-parallel prefill -----------------------------------------------------------------------------
 * The reference runs on one GPU; these four entry points are what a host needs around an all-to-all exchange when the
 * 64 experts of a layer are spread over several GPUs (the exchange itself is the host's: NCCL).  Arithmetic is that
 * of the single-GPU prefill path; rows travel as BF16, which is what the projections read and write anyway.
 *   padra_ep_plan: the send plan of a rank, a stable sort of its pairs by destination owner[ids[pair]] (owner[64] on
 *     the device, ranks 0..world-1, world <= 8): order[j] = pair sent as row j, position[pair] = row at which the pair's
 *     result returns, send_ids[j] = expert id of row j, send_counts[r] = rows for rank r.
 *   padra_ep_pack_rows: packed[j] = BF16 bits of activations[order[j]/8], j < rows = tokens*8; order lists the
 *     (token*8+slot) pairs in the order in which they are sent (sorted by destination rank).
 *   padra_ep_group_rows: fast_expert::Group for received rows: ids[rows] are expert ids 0..63 (any number of rows
 *     per expert, up to group_stride), groups[e*group_stride + n] = n-th row of expert e in ascending row order.
 *   padra_exl3_prefill_rows_launch: padra_exl3_prefill_launch's tensor-memory GEMM with one BF16 input row per pair
 *     (parts 0, 1: input_rows [rows][hidden]; part 2: gate/up [rows][inter]); output [rows][out] BF16 bits in row
 *     order (row indices may be sparse, up to 2^20; at most 32768 rows may be grouped); transformed is workspace of
 *     32768*max(hidden, inter) halves at most.
 *   padra_exl3_prefill_rows_gate_up_launch: parts 0 and 1 of the same in one launch (see
 *     padra_exl3_prefill_gate_up_launch); transformed holds 2*min(rows, 32768)*hidden halves.
 *   padra_ep_combine: padra_combine_packed with the down row of pair p at down_rows[position[p]]. */
/* The exchange done by the GPUs themselves over NVLink peer memory (no host in the loop, no NCCL on the data path).
 * Every rank owns one exchange block of padra_ep_exchange_bytes(world, cap, hidden, offsets) bytes, zero-filled once,
 * that every rank has mapped (peer_blocks[r] = address of rank r's block in THIS process, 256-byte aligned); cap is the
 * most pairs a rank sends per call.  offsets[0..5] = byte offsets of: received rows [world][cap][hidden] BF16, their
 * expert ids [world][cap], meta, returned rows [cap][hidden] BF16, and the two flag arrays.
 *   padra_ep_dispatch: padra_ep_pack_rows fused with the transfer: row j of the send order is stored into its owner's
 *     block, region `rank`; when all rows are out, the row counts and a flag carrying `epoch` follow.
 *   padra_ep_wait: which = 0 waits until every rank's rows for this call have arrived in `block` (this rank's own),
 *     which = 1 until every rank has returned this rank's rows; bounded (two seconds), then *bad is set.
 *   padra_ep_group_received: padra_ep_group_rows over the regions of `block`; row index = source*cap + k.  Pass that
 *     index space to padra_exl3_prefill_rows_launch: rows = world*cap, input_rows = block + offsets[0].
 *   padra_ep_return: down rows (same index space) go back into their source's block at the send rows they came
 *     from, then a flag with `epoch`; after padra_ep_wait(which = 1), padra_ep_combine reads block + offsets[3].
 *   Splitting a projection: block_begin / block_count of padra_exl3_prefill_rows_launch select the 128-output blocks a
 *     launch computes (0, 0 = all); only the launch with block_begin == 0 runs the input transform, later launches of
 *     the same call reuse `transformed`.  column_begin / column_count of padra_ep_return select the columns that are
 *     sent (0, 0 = all) and announce says whether this launch raises the flags (the last one of a call must).  With
 *     the two, the first half of the down rows can travel while the second half is still being computed.
 *   padra_ep_down_return: the down projection (part 2 of padra_exl3_prefill_rows_launch on the received index space)
 *     fused with padra_ep_return: the epilogue of the grouped GEMM stores every finished row straight into its source's
 *     block, so the transfer overlaps the remaining tiles, and the CTA that finishes last raises the flags.
 * epoch must differ from call to call (count up from 1).  A rank may start call n+1 only after its own combine of call
 * n has been enqueued on the same stream: that order is what makes reuse of the blocks safe. */
PADRA_API size_t padra_ep_exchange_bytes(int world, int cap, int hidden, size_t *offsets);
PADRA_API int padra_ep_dispatch(const float *activations, const int *order, const int *send_ids,
                                const long long *send_counts, const unsigned long long *peer_blocks, int rank, int world,
                                int cap, int pairs, int hidden, unsigned epoch, int *bad, padra_stream stream);
PADRA_API int padra_ep_wait(const void *block, int which, int world, int cap, int hidden, unsigned epoch, int *bad,
                            padra_stream stream);
/* How long padra_ep_wait's kernel polls before it gives up, raises *bad and returns (1..60000 ms, default 2000; a
 * process-wide host setting read at launch).  A wait that expires leaves the stream and the context usable. */
PADRA_API int padra_ep_set_wait_limit_ms(int milliseconds);
/* SMs the tensor-memory grouped GEMM leaves free (0..64, default 0; a process-wide host setting read at launch).  The GEMM
 * is persistent, one CTA per SM; with every SM taken, the kernels of another stream (the exchange of the next chunk:
 * plan, dispatch, return, input transforms) cannot start until its CTAs retire.  A host that overlaps chunks leaves a few
 * SMs to them. */
PADRA_API int padra_prefill_set_reserved_sms(int sms);
PADRA_API int padra_ep_group_received(const void *block, int world, int cap, int hidden, int *groups, int *counts,
                                      int group_stride, int *bad, padra_stream stream);
PADRA_API int padra_ep_return(const unsigned short *down_rows, const unsigned long long *peer_blocks, int rank, int world,
                              int cap, int hidden, unsigned epoch, int *bad, padra_stream stream, int column_begin,
                              int column_count, int announce);
PADRA_API int padra_ep_down_return(const padra_matrix *matrices, int layer, const int *groups, const int *counts,
                                   int group_stride, const unsigned short *gate, const unsigned short *up,
                                   const unsigned short *table, void *transformed, const unsigned long long *peer_blocks,
                                   int rank, int world, int cap, unsigned epoch, int *bad, padra_stream stream, int rate,
                                   int hidden, int inter);
PADRA_API int padra_ep_plan(const int *ids, const int *owner, int *order, int *position, int *send_ids,
                            long long *send_counts, int pairs, int world, int *bad, padra_stream stream);
PADRA_API int padra_ep_pack_rows(const float *activations, const int *order, unsigned short *packed, int rows, int hidden,
                                 int *bad, padra_stream stream);
PADRA_API int padra_ep_group_rows(const int *ids, int *groups, int *counts, int rows, int group_stride, int *bad,
                                  padra_stream stream);
PADRA_API int padra_exl3_prefill_rows_launch(const padra_matrix *matrices, int layer, int part, const int *groups,
                                             const int *counts, int group_stride, int rows,
                                             const unsigned short *input_rows, unsigned short *output,
                                             const unsigned short *gate, const unsigned short *up,
                                             const unsigned short *table, void *transformed, int *bad,
                                             padra_stream stream, int rate, int hidden, int inter, int block_begin,
                                             int block_count);
PADRA_API int padra_exl3_prefill_rows_gate_up_launch(const padra_matrix *matrices, int layer, const int *groups,
                                                     const int *counts, int group_stride, int rows,
                                                     const unsigned short *input_rows, unsigned short *gate_output,
                                                     unsigned short *up_output, void *transformed, int *bad,
                                                     padra_stream stream, int rate, int hidden, int inter);
PADRA_API int padra_ep_combine(float *x, const unsigned short *down_rows, const int *position, const float *weights,
                               int tokens, int *bad, int residual, int hidden, padra_stream stream);

/* ---- the callers either side of the experts: routing and norms -----------------------------------------------
 * padra_route: RouteRankExact (src/cuda/router_rank_exact.cuh:3-81; launched <<<rows, 64>>> at src/cuda/inference.cu:2950
 * and :3366): logits [tokens][64] FP32 -> ids [tokens][8] ascending, weights [tokens][8] BF16-valued.  Softmax with FP64
 * exp rounded to FP32 and ascending compensated sums, rank by probability then index, renormalised over the selection.
 * A raised *bad or a non-finite logit gives ids 0 and weights 0 for the token and raises *bad.
 * padra_route_group_schedule: the same routing and, in the same launch, the chunk's expert-major pair lists and 32-pair
 * tile list (what padra_expert_group and padra_exl3_schedule produce): one launch for the reference's three
 * (src/cuda/inference.cu:3861, :3875, :3890).  tokens <= 2048.  ticket: one word of device memory, zero before the first
 * call and left zero by every call (the CTA that finishes routing last does the scheduling). */
PADRA_API int padra_route(const float *logits, int *ids, float *weights, int tokens, int *bad, padra_stream stream);
PADRA_API int padra_route_group_schedule(const float *logits, int *ids, float *weights, int *groups, int *counts,
                                         padra_tile *tiles, int *tile_count, int tokens, unsigned *ticket, int *bad,
                                         padra_stream stream);
/* padra_residual_norm: ResidualPostNormWideExact (src/cuda/residual_norm_wide_exact.cuh:84-131; call sites
 * src/cuda/inference.cu:2913, :3358): per row x = B(x + residual), normalized = B(B(x * inv) * weight) with
 * inv = 1 / sqrt(mean(x^2) + 1e-6) from the reference's compensated 128-thread sum.  weight: BF16 bits [hidden].
 * residual may be NULL (x is normalised as it is).  statistics (may be NULL) receives [rows][2] = variance, inv.
 * padra_combine_norm: combine_norm_exact::CombineNorm<false> (src/cuda/combine_norm_exact.cuh:7-68): the ordered BF16
 * combine of the eight slots (down [rows][8][hidden], routing [rows][8]), the residual add into x and the same norm. */
PADRA_API int padra_residual_norm(float *x, const float *residual, float *normalized, const unsigned short *weight,
                                  int rows, int hidden, int *bad, float *statistics, padra_stream stream);
PADRA_API int padra_combine_norm(float *x, const float *down, const float *routing, float *normalized,
                                 const unsigned short *weight, int rows, int hidden, int *bad, float *statistics,
                                 padra_stream stream);

/* ---- small-batch projection (T < 4) -------------------------------------------------------------------
 * exl3_expert::Launch (src/cuda/expert_exl3.cuh:137-151): pairs = tokens*8, input row pair/8 (gate/up) or
 * pair (down), FP32-held BF16 in and out.  in_scratch / out_scratch are accepted and unused.  The reference's two
 * trailing parameters are not part of this signature: `bool fp32` (keep the transformed input unrounded, a diagnostic
 * form) and `unsigned *ranges` (value statistics); the serving path passes neither (both default to off). */
PADRA_API int padra_exl3_expert_launch(const padra_matrix *matrices, int layer, int part, const int *ids,
                                       const float *input, float *output, float *in_scratch, float *out_scratch,
                                       int tokens, int *bad, padra_stream stream, int rate, int hidden, int inter);

/* ---- whole expert layer at decode (M = 1..16), one call ------------------------------------------------
 * The call order of the reference's decode layer (src/cuda/inference.cu:2963-2975: gate/up projection,
 * SwiGLU, down projection, combine with residual) behind one entry point.  ids/routing are [tokens][8] (eight
 * distinct experts per token, BF16-valued weights), normalized [tokens][hidden] is the post-norm input,
 * x [tokens][hidden] the residual stream updated in place.  workspace must hold
 * padra_exl3_moe_decode_workspace_bytes() bytes; one workspace serves one stream at a time.
 *
 * padra_exl3_moe_decode_layer enqueues two launches that overlap on the GPU: the split-K projection of gate+up, and the
 * split-K projection of down, whose CTAs wait (bounded) for the gate/up blocks they need, apply SwiGLU and the down input
 * transform to them, and whose last-arriving CTA per 128-output block combines.  (Several tokens: the gate/up CTA that
 * delivers a block's last K-slice runs that epilogue instead.)  The counters at the start of the workspace must be zero
 * before the first call on it: call padra_exl3_moe_decode_workspace_init once after allocating it (it zero-fills the
 * workspace; stream-ordered, not graph-captured work of every step).  Every call leaves the counters zero again, also
 * when it raised *bad.
 * Stream order: ids, routing, normalized, x and *bad are read and written in stream order like any kernel's arguments.
 * `matrices` (the descriptor table) and the packed weights and sidecars it points to are model state: the launches
 * are programmatic dependents of what precedes them on the stream and read that state BEFORE the preceding work has
 * finished, so it must not be written by work that is still in flight on the stream when the call is made. */
PADRA_API size_t padra_exl3_moe_decode_workspace_bytes(int tokens, int hidden, int inter);
PADRA_API int padra_exl3_moe_decode_workspace_init(void *workspace, size_t workspace_bytes, padra_stream stream);
PADRA_API int padra_exl3_moe_decode_layer(const padra_matrix *matrices, int layer, const int *ids,
                                          const float *routing, const float *normalized, float *x, int tokens,
                                          int rate, int hidden, int inter, const unsigned short *table,
                                          void *workspace, size_t workspace_bytes, int *bad, padra_stream stream);
/* Diagnostic: the same pipeline with only the selected launches enqueued (bit 0 the gate+up kernel, bit 1 the down
 * kernel), so that one kernel can be timed or profiled alone on buffers a complete call has filled before. */
PADRA_API int padra_exl3_moe_decode_layer_launches(const padra_matrix *matrices, int layer, const int *ids,
                                                   const float *routing, const float *normalized, float *x,
                                                   int tokens, int rate, int hidden, int inter,
                                                   const unsigned short *table, void *workspace,
                                                   size_t workspace_bytes, int *bad, padra_stream stream,
                                                   unsigned launches);

/* ---- decode layer without any device allocation ------------------------------------------------------------
 * This entry point has no counterpart in the reference.  It is padra_exl3_moe_decode_layer for callers that cannot
 * allocate device memory: a server that gave every free byte of the device to its own arena at start-up, a plugin
 * that is not allowed to touch the allocator, or a latency-critical path that must avoid the device-wide
 * synchronisation of cudaMalloc/cudaFree.  Instead of a caller workspace it uses an array of
 * PADRA_STATIC_SCRATCH_BYTES that is built into the library's device code, and it calls no cudaMalloc, cudaFree or
 * other allocating routine.
 *   - Shapes whose workspace (padra_exl3_moe_decode_workspace_bytes) exceeds the array are refused with
 *     PADRA_RESOURCE_EXHAUSTED and nothing is enqueued.  Hidden 2048 / intermediate 1024 and 2304 / 896 fit at every
 *     batch (1..16 tokens); hidden 4096 / intermediate 2048 fits up to 9 tokens.
 *   - There is one array per device (256-byte aligned) and every call shares it: calls that may overlap on the GPU
 *     race on it and then give wrong results without any error, so the caller orders them (one stream, or events).
 *     The array keeps the last call's contents.  Only the ticket counters at its start have to be zero; the module
 *     loader zero-fills the array and every call leaves them zero, so there is nothing to clear between calls.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current); make that first call outside any stream capture.  That look-up may also be the moment the CUDA runtime
 *     loads this library's device code and backs the array with device memory (lazy module loading): a host that hands
 *     all free device memory to its own arena must make this first call (or any other call into this library that
 *     launches a kernel) BEFORE its arena claims the rest, or the call fails with PADRA_INTERNAL. */
#define PADRA_STATIC_SCRATCH_BYTES (4u << 20)
PADRA_API int padra_exl3_moe_decode_layer_static(const padra_matrix *matrices, int layer, const int *ids,
                                                 const float *routing, const float *normalized, float *x, int tokens,
                                                 int rate, int hidden, int inter, const unsigned short *table, int *bad,
                                                 padra_stream stream);


/* ---- utilities ------------------------------------------------------------------------------------------
 * Full FP16 decode of one matrix through the same codec the kernels use: out[input*rows + output].
 * `matrix` is a device pointer to one descriptor.  For verification; not on the timed path.
 * padra_exl3_decode_weights uses the form with byte sums on the integer pipe (prefill and per-part decode kernels),
 * padra_exl3_decode_weights_tensor the form with byte sums on the tensor cores (the whole-layer decode kernels). */
PADRA_API int padra_exl3_decode_weights(const padra_matrix *matrix, unsigned short *out, int rows, int cols,
                                        int rate, int *bad, padra_stream stream);
PADRA_API int padra_exl3_decode_weights_tensor(const padra_matrix *matrix, unsigned short *out, int rows, int cols,
                                               int rate, int *bad, padra_stream stream);
/* The codec's inner loop on registers alone, for measuring the rate at which the GPU can decode weights at all (the
 * instruction-issue ceiling beside the HBM roofline).  form bit 0: byte sums on the tensor cores instead of dp4a;
 * bit 1: with the FP16 mma that consumes the decoded fragments.  `blocks` CTAs of 256 threads each decode
 * 32 * iterations weights per thread; sink receives blocks * 256 words.  No counterpart in the reference. */
PADRA_API int padra_codec_ceiling_launch(int rate, int form, int iterations, int blocks, unsigned *sink,
                                         padra_stream stream);

#ifdef __cplusplus
}
#endif
#endif
