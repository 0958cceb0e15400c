/*
 * CPU oracle for the EXL3 MoE expert path.  TEST INFRASTRUCTURE ONLY -- see exl3_oracle.h.
 *
 * Build with -ffp-contract=off: the reference spells every FP32 operation as an explicit
 * round-to-nearest intrinsic (__fmul_rn, __fadd_rn, __fsub_rn), so no multiply-add may be fused here.
 */
#include "exl3_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 0;
void exl3_set_threads(int n) { g_threads = n; }
int exl3_get_threads(void) {
#ifdef _OPENMP
  return g_threads > 0 ? g_threads : omp_get_max_threads();
#else
  return 1;
#endif
}

static inline uint32_t f32_bits(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  return u;
}
static inline float bits_f32(uint32_t u) {
  float x;
  memcpy(&x, &u, 4);
  return x;
}

/* B(): round FP32 to BF16 (nearest even) and widen back.  src/cuda/inference.cu:52-54 */
float exl3_bf16_round(float x) {
  uint32_t u = f32_bits(x);
  if ((u & 0x7fffffffu) > 0x7f800000u) /* every NaN becomes the canonical BF16 NaN 0x7fff, as __float2bfloat16_rn does */
    return bits_f32(0x7fff0000u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return bits_f32(u & 0xffff0000u);
}

/* __float2half_rn: FP32 -> FP16 bits, nearest even, with subnormals, overflow to infinity. */
uint16_t exl3_f32_to_f16_bits(float x) {
  const uint32_t u = f32_bits(x);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u)
    return (uint16_t)(sign | 0x7fffu);
  if (a >= 0x477ff000u) /* >= 65520 rounds to infinity */
    return (uint16_t)(sign | 0x7c00u);
  if (a < 0x33000001u) /* <= 2^-25 rounds to zero */
    return (uint16_t)sign;
  int exp = (int)(a >> 23) - 127;
  uint32_t man = (a & 0x7fffffu) | 0x800000u;
  int shift;
  uint32_t base;
  if (exp >= -14) {
    shift = 13;
    base = (uint32_t)(exp + 15) << 10;
    man &= 0x7fffffu;
  } else {
    shift = 13 + (-14 - exp);
    base = 0;
  }
  uint32_t q = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u)))
    q += 1;
  return (uint16_t)(sign | (base + q));
}

float exl3_f16_bits_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 31u, man = h & 1023u;
  if (exp == 31)
    return bits_f32(sign | 0x7f800000u | (man << 13));
  if (exp == 0) {
    const float v = (float)man * (1.0f / 16777216.0f); /* man * 2^-24, exact */
    return sign ? -v : v;
  }
  return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

int exl3_rate_of_format(int format) { /* src/cuda/expert_exl3.cuh:9 */
  return format == 6 ? 3 : format == 4 ? 8 : format == 5 ? 6 : 4;
}
int exl3_format_of_rate(int rate) { /* src/cuda/device_matrix.cuh:30-44 */
  return rate == 3 ? 6 : rate == 6 ? 5 : rate == 8 ? 4 : 3;
}

/* Position of weight (input, output) inside a 16x16 tile.  src/cuda/expert_exl3.cuh:4-7 */
unsigned exl3_index(unsigned i, unsigned o) {
  return ((o & 7u) * 4u + ((i & 7u) >> 1)) * 8u + (o >= 8u ? 4u : 0u) + (i >= 8u ? 2u : 0u) + (i & 1u);
}

/* The 16-bit trellis state of one weight: a cyclic MSB-first window over the tile's bit stream.
 * src/cuda/expert_exl3.cuh:8-18 */
unsigned exl3_state(const exl3_matrix *m, int input, int output) {
  const int rate = exl3_rate_of_format(m->format);
  const unsigned char *tile =
      m->data + ((size_t)(input / 16) * (size_t)(m->rows / 16) + (size_t)(output / 16)) * (size_t)(32 * rate);
  const int words = 8 * rate;
  const unsigned p = exl3_index((unsigned)input & 15u, (unsigned)output & 15u);
  const int end = (int)p * rate + rate + 256 * rate; /* one stream length ahead: no negative indices */
  const int begin = end - 16, first = begin / 32, last = (end - 1) / 32, shift = (last + 1) * 32 - end;
  uint32_t lo, hi;
  memcpy(&lo, tile + 4 * (last % words), 4);  /* little-endian u32 words */
  memcpy(&hi, tile + 4 * (first % words), 4);
  const uint64_t both = ((uint64_t)hi << 32) | lo; /* __funnelshift_r(lo, hi, shift) */
  return (unsigned)((both >> shift) & 0xffffu);
}

/* "mul1" codebook: hash the state, sum the four bytes, one fused FP16 multiply-add.
 * (1024+s) * 0x1eee + 0xc931 = ((1024+s)*1774 - 2721792) * 2^-18 exactly; the integer has < 21 bits,
 * so it is exact in FP32 and the FP32 -> FP16 conversion is the single rounding of __hfma.
 * src/cuda/expert_exl3.cuh:19-21 */
uint16_t exl3_mul1_bits(unsigned state) {
  const uint32_t h = (uint32_t)state * 0x83DCD12Du;
  const int s = (int)((h & 255u) + ((h >> 8) & 255u) + ((h >> 16) & 255u) + (h >> 24));
  const int n = (1024 + s) * 1774 - 2721792;
  return exl3_f32_to_f16_bits((float)n * (1.0f / 262144.0f));
}

uint16_t exl3_weight_bits(const exl3_matrix *m, int input, int output) {
  return exl3_mul1_bits(exl3_state(m, input, output));
}

void exl3_decode_matrix(const exl3_matrix *m, uint16_t *out) {
#pragma omp parallel for num_threads(exl3_get_threads()) schedule(static)
  for (int i = 0; i < m->cols; ++i)
    for (int o = 0; o < m->rows; ++o)
      out[(size_t)i * m->rows + o] = exl3_weight_bits(m, i, o);
}

/* 128-point Walsh-Hadamard, stages d = 1,2,...,64, then one scaling by 1/sqrt(128).
 * src/cuda/expert_exl3.cuh:48-55 (same order as the warp form, expert_exl3_codec.cuh:24-43) */
void exl3_hadamard128(float *x) {
  float y[128];
  for (int d = 1; d < 128; d *= 2) {
    for (int t = 0; t < 128; ++t) {
      const float a = x[t], b = x[t ^ d];
      y[t] = (t & d) ? (b - a) : (a + b);
    }
    memcpy(x, y, sizeof y);
  }
  for (int t = 0; t < 128; ++t)
    x[t] = x[t] * 0.08838834764831845f;
}

static int valid_format(const exl3_matrix *m) {
  return m->format == 3 || m->format == 4 || m->format == 5 || m->format == 6;
}

/* xt = B(H128(x * suh)).  src/cuda/expert_exl3.cuh:32-59 */
int exl3_input_had(const exl3_matrix *m, const float *x, float *xt) {
  int bad = !valid_format(m) || (m->cols % 128) != 0;
  for (int b = 0; b + 128 <= m->cols; b += 128) {
    float v[128];
    for (int t = 0; t < 128; ++t)
      v[t] = x[b + t] * exl3_f16_bits_to_f32(m->suh[b + t]);
    exl3_hadamard128(v);
    for (int t = 0; t < 128; ++t) {
      const float r = exl3_bf16_round(v[t]);
      if (!isfinite(r))
        bad = 1;
      xt[b + t] = r;
    }
  }
  return bad;
}

/* Neumaier step.  src/cuda/inference.cu:103-109 */
static inline void accumulate(float value, float *sum, float *error) {
  const float next = *sum + value;
  const float residual = fabsf(*sum) >= fabsf(value) ? ((*sum - next) + value) : ((value - next) + *sum);
  *error = *error + residual;
  *sum = next;
}

/* Compensated per-output dot product, 32 lanes striding the inputs, shuffle-down merge.
 * src/cuda/expert_exl3.cuh:60-87 */
int exl3_dot(const exl3_matrix *m, const float *xt, float *raw) {
  int bad = !valid_format(m);
#pragma omp parallel for num_threads(exl3_get_threads()) schedule(static) reduction(| : bad)
  for (int row = 0; row < m->rows; ++row) {
    float sum[32], err[32];
    for (int lane = 0; lane < 32; ++lane) {
      float s = 0.f, e = 0.f;
      for (int k = lane; k < m->cols; k += 32)
        accumulate(xt[k] * exl3_f16_bits_to_f32(exl3_weight_bits(m, k, row)), &s, &e);
      sum[lane] = s;
      err[lane] = e;
    }
    for (int d = 16; d; d /= 2) {
      for (int lane = 0; lane + d < 32; ++lane) { /* lanes read values the higher lanes held before this step */
        const float other = sum[lane + d], low = err[lane + d];
        accumulate(other, &sum[lane], &err[lane]);
        accumulate(low, &sum[lane], &err[lane]);
      }
    }
    const float v = sum[0] + err[0];
    if (!isfinite(v))
      bad |= 1;
    raw[row] = v;
  }
  return bad;
}

/* y = B((H128(raw)) * svh).  src/cuda/expert_exl3.cuh:88-113 */
int exl3_output_had(const exl3_matrix *m, const float *raw, float *y) {
  int bad = !valid_format(m) || (m->rows % 128) != 0;
  for (int b = 0; b + 128 <= m->rows; b += 128) {
    float v[128];
    memcpy(v, raw + b, sizeof v);
    exl3_hadamard128(v);
    for (int t = 0; t < 128; ++t) {
      const float r = exl3_bf16_round(v[t] * exl3_f16_bits_to_f32(m->svh[b + t]));
      if (!isfinite(r))
        bad = 1;
      y[b + t] = r;
    }
  }
  return bad;
}

int exl3_linear(const exl3_matrix *m, const float *x, float *y) {
  float *xt = (float *)malloc(sizeof(float) * (size_t)m->cols);
  float *raw = (float *)malloc(sizeof(float) * (size_t)m->rows);
  int bad = exl3_input_had(m, x, xt);
  bad |= exl3_dot(m, xt, raw);
  bad |= exl3_output_had(m, raw, y);
  free(xt);
  free(raw);
  return bad;
}

/* Production form: the transformed input is narrowed to FP16 (overflow raises `bad`), each FP16 x FP16
 * product is exact in FP32, and the products are added in FP32 in ascending input order.
 * src/cuda/expert_exl3_decode_dual.cuh:65-130 */
int exl3_linear_f16(const exl3_matrix *m, const float *x, float *y) {
  float *xt = (float *)malloc(sizeof(float) * (size_t)m->cols);
  float *raw = (float *)malloc(sizeof(float) * (size_t)m->rows);
  int bad = exl3_input_had(m, x, xt);
  for (int k = 0; k < m->cols; ++k) {
    const uint16_t h = exl3_f32_to_f16_bits(xt[k]);
    if ((h & 0x7c00u) == 0x7c00u)
      bad = 1;
    xt[k] = exl3_f16_bits_to_f32(h);
  }
#pragma omp parallel for num_threads(exl3_get_threads()) schedule(static)
  for (int row = 0; row < m->rows; ++row) {
    float acc = 0.f;
    for (int k = 0; k < m->cols; ++k)
      acc = acc + xt[k] * exl3_f16_bits_to_f32(exl3_weight_bits(m, k, row));
    raw[row] = acc;
  }
  bad |= exl3_output_had(m, raw, y);
  free(xt);
  free(raw);
  return bad;
}

/* SiLU with the exponential evaluated in FP64 and rounded once to FP32, result rounded to BF16.
 * src/cuda/exl3_silu_lut.cuh:5-8, src/cuda/inference.cu:57-59 */
float exl3_silu_rounded(float g) {
  const float e = (float)exp((double)(-g));
  const float denominator = 1.f + e;
  return exl3_bf16_round(g / denominator);
}

void exl3_silu_table(uint16_t *table) { /* src/cuda/exl3_silu_lut.cuh:9-14 */
  for (uint32_t i = 0; i < 65536u; ++i)
    table[i] = (uint16_t)(f32_bits(exl3_silu_rounded(bits_f32(i << 16))) >> 16);
}

/* gate = B(silu(gate) * up).  src/cuda/inference.cu:575-579; table form exl3_silu_lut.cuh:15-31 */
int exl3_activate(float *gate, const float *up, int count) {
  int bad = 0;
  for (int i = 0; i < count; ++i) {
    const float g = gate[i], u = up[i];
    if (!isfinite(g) || !isfinite(u) || (f32_bits(g) & 65535u)) {
      bad = 1; /* the table form refuses values that are not BF16-representable */
      continue;
    }
    const float v = exl3_bf16_round(exl3_silu_rounded(g) * u);
    if (!isfinite(v))
      bad = 1;
    gate[i] = v;
  }
  return bad;
}

/* Softmax in FP32 with compensated sums, top eight, renormalise, BF16 weights, ascending expert id.
 * src/cuda/inference.cu:482-536 */
int exl3_route(const float *logits, int *ids, float *weights) {
  float p[64], mx = -INFINITY, total = 0.f, total_error = 0.f;
  for (int i = 0; i < 64; ++i)
    mx = fmaxf(mx, logits[i]);
  for (int i = 0; i < 64; ++i) {
    p[i] = (float)exp((double)(logits[i] - mx));
    accumulate(p[i], &total, &total_error);
  }
  total = total + total_error;
  for (int i = 0; i < 64; ++i)
    p[i] = p[i] / total;
  float selected = 0.f, selected_error = 0.f;
  for (int s = 0; s < 8; ++s) {
    int best = -1;
    float q = -1.f;
    for (int i = 0; i < 64; ++i)
      if (p[i] > q) {
        q = p[i];
        best = i;
      }
    ids[s] = best;
    weights[s] = q;
    accumulate(q, &selected, &selected_error);
    p[best] = -1.f;
  }
  selected = selected + selected_error;
  for (int s = 0; s < 8; ++s)
    weights[s] = exl3_bf16_round(weights[s] / selected);
  for (int a = 0; a < 8; ++a)
    for (int b = a + 1; b < 8; ++b)
      if (ids[b] < ids[a]) {
        const int id = ids[a];
        ids[a] = ids[b];
        ids[b] = id;
        const float w = weights[a];
        weights[a] = weights[b];
        weights[b] = w;
      }
  return !isfinite(selected);
}

/* x = B(x + sum_s), sum = B(sum + B(down_s * w_s)) over the eight slots in order.
 * src/cuda/inference.cu:580-594 */
int exl3_combine(float *x, const float *down, const float *weights, int hidden) {
  int bad = 0;
  for (int i = 0; i < hidden; ++i) {
    float sum = 0.f;
    for (int s = 0; s < 8; ++s)
      sum = exl3_bf16_round(sum + exl3_bf16_round(down[(size_t)s * hidden + i] * weights[s]));
    x[i] = exl3_bf16_round(x[i] + sum);
    if (!isfinite(x[i]))
      bad = 1;
  }
  return bad;
}

/* Merge of the 128 per-thread compensated sums: shuffle-down trees inside each of the four warps (every lane reads its
 * partner's values from before the step), then over the four warp results.
 * src/cuda/rms_wide_exact.cuh:3-33 (and AccurateReduce, src/cuda/inference.cu:110-134, which gives the same sum). */
static float reduce_squares128(float *sum, float *err) {
  float wsum[4], werr[4];
  for (int w = 0; w < 4; ++w) {
    float *s = sum + 32 * w, *e = err + 32 * w;
    for (int d = 16; d; d /= 2) {
      float os[32], oe[32];
      for (int l = 0; l < 32; ++l) {
        os[l] = l + d < 32 ? s[l + d] : s[l];
        oe[l] = l + d < 32 ? e[l + d] : e[l];
      }
      for (int l = 0; l + d < 32; ++l) {
        accumulate(os[l], &s[l], &e[l]);
        accumulate(oe[l], &s[l], &e[l]);
      }
    }
    wsum[w] = s[0];
    werr[w] = e[0];
  }
  for (int d = 2; d; d /= 2) {
    float os[4], oe[4];
    for (int l = 0; l < 4; ++l) {
      os[l] = l + d < 4 ? wsum[l + d] : wsum[l];
      oe[l] = l + d < 4 ? werr[l + d] : werr[l];
    }
    for (int l = 0; l + d < 4; ++l) {
      accumulate(os[l], &wsum[l], &werr[l]);
      accumulate(oe[l], &wsum[l], &werr[l]);
    }
  }
  return wsum[0] + werr[0];
}

static float bf16_bits_f32(uint16_t b) {
  return bits_f32((uint32_t)b << 16);
}

/* x = B(x + residual) (residual may be NULL), normalized = B(B(x * inv) * weight), inv = 1 / sqrt(mean(x^2) + 1e-6) with
 * thread t of 128 summing the squares of elements t, t+128, ... compensated.  One row of `hidden` elements.
 * src/cuda/residual_norm_wide_exact.cuh:84-131.  stats (may be NULL) receives variance and inv. */
int exl3_residual_norm(float *x, const float *residual, float *normalized, const uint16_t *weight, int hidden, float *stats) {
  float sum[128], err[128];
  int bad = 0;
  for (int t = 0; t < 128; ++t) {
    sum[t] = 0.f, err[t] = 0.f;
    for (int i = t; i < hidden; i += 128) {
      const float value = exl3_bf16_round(residual ? x[i] + residual[i] : x[i]);
      x[i] = value;
      if (!isfinite(value))
        bad = 1;
      accumulate(value * value, &sum[t], &err[t]);
    }
  }
  const float total = reduce_squares128(sum, err);
  if (!isfinite(total))
    bad = 1;
  const float variance = total / (float)hidden;
  const float inv = 1.f / sqrtf(variance + 1e-6f);
  if (stats)
    stats[0] = variance, stats[1] = inv;
  for (int i = 0; i < hidden; ++i) {
    normalized[i] = exl3_bf16_round(exl3_bf16_round(x[i] * inv) * bf16_bits_f32(weight[i]));
    if (!isfinite(normalized[i]))
      bad = 1;
  }
  return bad;
}

/* The ordered BF16 combine of the eight slots, the residual add and the same norm in one pass, one row.
 * down [8][hidden], routing [8].  src/cuda/combine_norm_exact.cuh:7-68 (EncodeFP8 = false). */
int exl3_combine_norm(float *x, const float *down, const float *routing, float *normalized, const uint16_t *weight, int hidden,
                      float *stats) {
  float sum[128], err[128];
  int bad = 0;
  for (int t = 0; t < 128; ++t) {
    sum[t] = 0.f, err[t] = 0.f;
    for (int i = t; i < hidden; i += 128) {
      float acc = 0.f;
      for (int s = 0; s < 8; ++s)
        acc = exl3_bf16_round(acc + exl3_bf16_round(down[(size_t)s * hidden + i] * routing[s]));
      const float value = exl3_bf16_round(x[i] + acc);
      x[i] = value;
      if (!isfinite(value))
        bad = 1;
      accumulate(value * value, &sum[t], &err[t]);
    }
  }
  const float total = reduce_squares128(sum, err);
  const float variance = total / (float)hidden;
  const float inv = 1.f / sqrtf(variance + 1e-6f);
  if (stats)
    stats[0] = variance, stats[1] = inv;
  for (int i = 0; i < hidden; ++i) {
    normalized[i] = exl3_bf16_round(exl3_bf16_round(x[i] * inv) * bf16_bits_f32(weight[i]));
    if (!isfinite(normalized[i]))
      bad = 1;
  }
  return bad;
}

/* Stable expert-major slot lists.  groups[e*tokens + n] = n-th (token*8+slot) that chose expert e.
 * src/cuda/expert_schedule.cuh:11-69 */
int exl3_group(const int *ids, int *groups, int *counts, int tokens) {
  int bad = 0;
  for (int e = 0; e < 64; ++e)
    counts[e] = 0;
  for (int t = 0; t < tokens; ++t) {
    uint64_t seen = 0;
    for (int s = 0; s < 8; ++s) {
      const int e = ids[t * 8 + s];
      if (e < 0 || e >= 64) {
        bad = 1;
        continue;
      }
      if (seen & (1ull << e))
        bad = 1;
      seen |= 1ull << e;
      if (counts[e] < tokens)
        groups[(size_t)e * tokens + counts[e]] = t * 8 + s;
      counts[e]++;
    }
  }
  for (int e = 0; e < 64; ++e)
    if (counts[e] > tokens) {
      bad = 1;
      counts[e] = tokens;
    }
  return bad;
}

/* Tiles of at most 32 rows per expert, experts ascending.  tiles3 = {expert, begin, valid_rows}.
 * src/cuda/expert_exl3_prefill_masked.cuh:12-45, src/runtime/exl3_masked_schedule.h:6-21 */
int exl3_schedule(const int *counts, int *tiles3, int *tile_count, int tokens) {
  *tile_count = 0;
  if (tokens < 1 || tokens > 2048)
    return 1;
  const int capacity = (tokens * 8 + 31) / 32 + 64;
  int total = 0, sum = 0;
  for (int e = 0; e < 64; ++e) {
    if (counts[e] < 0 || counts[e] > tokens)
      return 1;
    sum += counts[e];
    total += (counts[e] + 31) / 32;
  }
  if (sum != tokens * 8 || total > capacity)
    return 1;
  int at = 0;
  for (int e = 0; e < 64; ++e)
    for (int begin = 0; begin < counts[e]; begin += 32) {
      tiles3[at * 3 + 0] = e;
      tiles3[at * 3 + 1] = begin;
      tiles3[at * 3 + 2] = counts[e] - begin < 32 ? counts[e] - begin : 32;
      ++at;
    }
  *tile_count = at;
  return 0;
}

/* gate/up -> SwiGLU -> down -> combine, per token, in the reference's decode call order
 * (src/cuda/inference.cu:2963-2975). */
int exl3_moe_layer(const exl3_matrix *matrices, int layer, const int *ids, const float *weights,
                   float *x, int tokens, int hidden, int inter, int f16_form,
                   float *cap_gate, float *cap_up, float *cap_act, float *cap_down) {
  int bad = 0;
  const int pairs = tokens * 8;
  float *gate = (float *)malloc(sizeof(float) * (size_t)pairs * inter);
  float *up = (float *)malloc(sizeof(float) * (size_t)pairs * inter);
  float *down = (float *)malloc(sizeof(float) * (size_t)pairs * hidden);
  int (*linear)(const exl3_matrix *, const float *, float *) = f16_form ? exl3_linear_f16 : exl3_linear;
  for (int pair = 0; pair < pairs; ++pair) {
    const int e = ids[pair];
    if (e < 0 || e >= 64) {
      bad = 1;
      continue;
    }
    const exl3_matrix *m = matrices + ((size_t)layer * 64 + e) * 3;
    if (m[0].rows != inter || m[0].cols != hidden || m[1].rows != inter || m[1].cols != hidden ||
        m[2].rows != hidden || m[2].cols != inter) {
      bad = 1;
      continue;
    }
    bad |= linear(m + 0, x + (size_t)(pair / 8) * hidden, gate + (size_t)pair * inter);
    bad |= linear(m + 1, x + (size_t)(pair / 8) * hidden, up + (size_t)pair * inter);
  }
  if (cap_gate)
    memcpy(cap_gate, gate, sizeof(float) * (size_t)pairs * inter);
  if (cap_up)
    memcpy(cap_up, up, sizeof(float) * (size_t)pairs * inter);
  bad |= exl3_activate(gate, up, pairs * inter);
  if (cap_act)
    memcpy(cap_act, gate, sizeof(float) * (size_t)pairs * inter);
  for (int pair = 0; pair < pairs; ++pair) {
    const int e = ids[pair];
    if (e < 0 || e >= 64)
      continue;
    const exl3_matrix *m = matrices + ((size_t)layer * 64 + e) * 3 + 2;
    bad |= linear(m, gate + (size_t)pair * inter, down + (size_t)pair * hidden);
  }
  if (cap_down)
    memcpy(cap_down, down, sizeof(float) * (size_t)pairs * hidden);
  for (int t = 0; t < tokens; ++t)
    bad |= exl3_combine(x + (size_t)t * hidden, down + (size_t)t * 8 * hidden, weights + t * 8, hidden);
  free(gate);
  free(up);
  free(down);
  return bad;
}
