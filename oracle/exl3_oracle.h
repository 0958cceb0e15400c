/*
 * CPU oracle for the EXL3 MoE expert path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic the reference (Danmoreng/padra) performs on the GPU for
 * its trellis-coded expert layer.  It exists so that the CUDA library can be checked against an
 * independent scalar implementation and so that a host-core baseline can be timed next to the GPU
 * numbers.  Only the tests, the smoke check and the benchmark's CPU-baseline leg may load it; the
 * product library never links or calls it.
 *
 * Parity pin: the trellis decoder (exl3_index / exl3_weight_bits) is checked bit-for-bit against the
 * reference's own Index/Weight source text compiled for the host (oracle/_ref/libref_weight.so, built
 * by oracle/Makefile) and against the committed golden vectors in tests/golden/.  The layer arithmetic
 * is checked on the GPU box against the reference's own kernels compiled for sm_100a
 * (oracle/_ref/libref_kernels.so).
 *
 * Every function names the reference file:line it follows (paths relative to the reference root).
 */
#ifndef EXL3_ORACLE_H
#define EXL3_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* Same seven fields, order and size (56 bytes) as the reference descriptor,
 * src/cuda/device_matrix.cuh:6-13.  Pointers are host pointers here. */
typedef struct exl3_matrix {
  const unsigned char *data;   /* packed trellis tiles */
  const unsigned char *scales; /* unused for EXL3 */
  const float *divisor;        /* unused for EXL3 */
  int rows, cols, format;      /* rows = outputs, cols = inputs; format 3=K4, 5=K6, 6=K3 */
  const uint16_t *suh;         /* FP16 bits, one per input */
  const uint16_t *svh;         /* FP16 bits, one per output */
} exl3_matrix;

/* scalar helpers */
float exl3_bf16_round(float x);              /* B(), src/cuda/inference.cu:52-54 */
uint16_t exl3_f32_to_f16_bits(float x);      /* __float2half_rn */
float exl3_f16_bits_to_f32(uint16_t h);      /* __half2float */
int exl3_rate_of_format(int format);         /* src/cuda/expert_exl3.cuh:9 */
int exl3_format_of_rate(int rate);

/* trellis decoder */
unsigned exl3_index(unsigned input_in_tile, unsigned output_in_tile); /* expert_exl3.cuh:4-7 */
uint16_t exl3_mul1_bits(unsigned state);                               /* expert_exl3.cuh:19-21 */
unsigned exl3_state(const exl3_matrix *m, int input, int output);      /* expert_exl3.cuh:8-18 */
uint16_t exl3_weight_bits(const exl3_matrix *m, int input, int output);/* expert_exl3.cuh:8-22 */
/* out[input * rows + output] = FP16 bits of every weight */
void exl3_decode_matrix(const exl3_matrix *m, uint16_t *out);

/* one EXL3 linear, reference SIMT ("represented math") form */
void exl3_hadamard128(float *x);                                          /* expert_exl3.cuh:48-55 */
int exl3_input_had(const exl3_matrix *m, const float *x, float *xt);      /* expert_exl3.cuh:32-59 */
int exl3_dot(const exl3_matrix *m, const float *xt, float *raw);          /* expert_exl3.cuh:60-87 */
int exl3_output_had(const exl3_matrix *m, const float *raw, float *y);    /* expert_exl3.cuh:88-113 */
int exl3_linear(const exl3_matrix *m, const float *x, float *y);          /* expert_exl3.cuh:137-151 */
/* production (tensor-core) form: FP16 inputs, FP16 x FP16 products, FP32 sequential accumulation,
 * src/cuda/expert_exl3_decode_dual.cuh:65-130 */
int exl3_linear_f16(const exl3_matrix *m, const float *x, float *y);

/* SwiGLU, routing, combine */
float exl3_silu_rounded(float g);                                  /* exl3_silu_lut.cuh:5-8 */
void exl3_silu_table(uint16_t *table65536);                        /* exl3_silu_lut.cuh:9-14 */
int exl3_activate(float *gate, const float *up, int count);        /* inference.cu:575-579 */
int exl3_route(const float *logits64, int *ids8, float *weights8); /* inference.cu:482-536 */
int exl3_combine(float *x, const float *down, const float *weights, int hidden); /* inference.cu:580-594 */

/* the norms either side of the experts: one row of `hidden` elements, weight = BF16 bits, stats (may be NULL) receives
 * the variance and its inverse root */
int exl3_residual_norm(float *x, const float *residual, float *normalized, const uint16_t *weight, int hidden,
                       float *stats); /* residual_norm_wide_exact.cuh:84-131 */
int exl3_combine_norm(float *x, const float *down, const float *routing, float *normalized, const uint16_t *weight,
                      int hidden, float *stats); /* combine_norm_exact.cuh:7-68 */

/* scheduling */
int exl3_group(const int *ids, int *groups, int *counts, int tokens);          /* expert_schedule.cuh:11-69 */
int exl3_schedule(const int *counts, int *tiles3, int *tile_count, int tokens);/* expert_exl3_prefill_masked.cuh:12-45 */

/* Whole MoE layer for `tokens` rows: x[tokens][hidden] (FP32 holding BF16 values) is updated in place
 * with the residual, exactly like the decode call order of inference.cu:2963-2975.
 * matrices = table indexed (layer*64+e)*3+part.  f16_form selects exl3_linear_f16.
 * Optional captures (may be NULL): gate/up/act [tokens*8][inter], down [tokens*8][hidden].
 * Returns nonzero if the sticky `bad` condition would have been raised. */
int exl3_moe_layer(const exl3_matrix *matrices, int layer, const int *ids, const float *weights,
                   float *x, int tokens, int hidden, int inter, int f16_form,
                   float *cap_gate, float *cap_up, float *cap_act, float *cap_down);

void exl3_set_threads(int n); /* OpenMP threads used by the loops over outputs/pairs (0 = default) */
int exl3_get_threads(void);

#ifdef __cplusplus
}
#endif
#endif
