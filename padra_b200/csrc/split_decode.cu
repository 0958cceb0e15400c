// Whole EXL3 expert layer at decode (M = 1..16 rows) as a pipeline of four plain launches:
//
//   1. SplitProjectionKernel, gate+up : every (expert, 128-output block, matrix, K-slice) is one CTA that streams its
//      slice of packed words, decodes in registers and multiplies with mma.m16n8k16 (same lane ownership as
//      decode.cu); the FP32 sums of the slice go to the workspace.
//   2. GateUpEpilogueKernel : per (row, 128-output block) sums the K-slices in ascending order, applies the output
//      Hadamard and svh, SwiGLU, and the down projection's input transform; writes FP16 in the permuted K16 order.
//   3. SplitProjectionKernel, down   : as 1, reading the transformed rows.
//   4. DownEpilogueKernel : per (token, 128-output block) sums the slices of each of the eight slots, output
//      Hadamard, svh, BF16, then the reference's combine with routing weights and residual.
//
// Splitting K over CTAs is what fills the machine at M = 1: 8 experts x 8 blocks x 2 matrices are only 128 work
// items, with four K-slices each they are 512 CTAs of 8 warps, four resident per SM.  Kernel boundaries carry the
// dependencies, so no kernel waits on another CTA.  All summation orders are fixed (ascending slice, ascending slot):
// results are bit-identical run to run.
#include "codec.cuh"
#include "common.cuh"
#include "kernels.cuh"

namespace padra {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxSlices = 4;

__device__ __forceinline__ void MmaF16(const uint32_t (&a)[4], uint32_t b0, uint32_t b1, float (&d)[4]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void Unpack4(uint2 bits, float (&f)[4]) {
  f[0] = HalfBitsToFloat(bits.x & 0xffffu);
  f[1] = HalfBitsToFloat(bits.x >> 16);
  f[2] = HalfBitsToFloat(bits.y & 0xffffu);
  f[3] = HalfBitsToFloat(bits.y >> 16);
}

// Programmatic dependent launch: each kernel of the pipeline is launched with programmatic stream serialization,
// lets its successor start launching at once and itself waits for its predecessor right before the first access
// to data the predecessor produces.  What comes before the wait (unit lookup, descriptor checks, the first packed
// words in flight) overlaps the predecessor's tail.  Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void LetSuccessorLaunch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void WaitForPredecessor() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

struct SplitArgs {
  const Matrix *matrices;
  int layer, phase; // phase 0: gate and up from `normalized`; phase 1: down from `xdown`
  const int *ids;
  int tokens, hidden, inter, slices;
  const float *normalized; // [tokens][hidden]
  const __half *xdown;     // [pairs][inter], permuted K16 order
  float *partials;         // phase 0: [pair][2][slices][inter]; phase 1: [pair][slices][hidden]
  int *bad;
};

// Unit `unit` of the launch: for one token the unit is the slot; for several tokens it is the unit-th active expert
// in ascending id, with the rows (token*8+slot) routed to it.  Every CTA derives this from `ids` alone.
template <int NG>
__device__ __forceinline__ bool ResolveUnit(const int *ids, int tokens, int unit, int &expert, int &count, int (&rows)[8 * NG],
                                            int *bad) {
  __shared__ unsigned s_votes[2];
  __shared__ int s_expert, s_count, s_invalid, s_rows[8 * NG];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    s_expert = -1;
    s_count = 0;
    s_invalid = 0;
  }
  __syncthreads();
  if (tokens == 1) {
    if (tid == 0) {
      const int e = unit < kTopK ? ids[unit] : -1;
      if (unit < kTopK && (e < 0 || e >= kExperts))
        s_invalid = 1;
      s_expert = e;
      s_count = unit < kTopK ? 1 : 0;
      s_rows[0] = unit;
    }
  } else if (tid < kExperts) {
    int n = 0, mine[8 * NG], invalid = 0;
    for (int r = 0; r < tokens; ++r)
      for (int s = 0; s < kTopK; ++s) {
        const int id = ids[r * kTopK + s];
        invalid |= (id < 0 || id >= kExperts);
        if (id == tid) {
          if (n < 8 * NG)
            mine[n] = r * kTopK + s;
          ++n;
        }
      }
    if (invalid || n > 8 * NG)
      atomicOr(&s_invalid, 1);
    const unsigned votes = __ballot_sync(0xffffffffu, n > 0);
    if (!lane)
      s_votes[warp] = votes;
    __syncwarp();
    // both warps of the first 64 threads must see both ballots
    asm volatile("bar.sync 1, 64;" ::: "memory");
    const unsigned own = s_votes[warp];
    const int rank = __popc(own & ((1u << lane) - 1u)) + (warp ? __popc(s_votes[0]) : 0);
    if (n > 0 && rank == unit) {
      s_expert = tid;
      s_count = n < 8 * NG ? n : 8 * NG;
      for (int i = 0; i < s_count; ++i)
        s_rows[i] = mine[i];
    }
  }
  __syncthreads();
  if (s_invalid) {
    if (tid == 0)
      Raise(bad);
    return false;
  }
  expert = s_expert;
  count = s_count;
#pragma unroll
  for (int i = 0; i < 8 * NG; ++i)
    rows[i] = i < count ? s_rows[i] : 0;
  return expert >= 0 && count > 0;
}

template <int Rate, int NG>
__global__ void __launch_bounds__(kThreads) SplitProjectionKernel(SplitArgs a) {
  using L = codec::Lane<Rate>;
  extern __shared__ __align__(16) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  LetSuccessorLaunch();
  int expert, count, rows[8 * NG];
  if (!ResolveUnit<NG>(a.ids, a.tokens, blockIdx.y, expert, count, rows, a.bad)) {
    WaitForPredecessor();
    return;
  }
  const int part = a.phase ? 2 : static_cast<int>(blockIdx.z) / a.slices;
  const int slice = static_cast<int>(blockIdx.z) % a.slices;
  const Matrix m = a.matrices[(static_cast<size_t>(a.layer) * kExperts + expert) * 3 + part];
  const int want_rows = part == 2 ? a.hidden : a.inter, want_cols = part == 2 ? a.inter : a.hidden;
  const int base = blockIdx.x * 128;
  if (m.format != FormatOfRate(Rate) || m.rows != want_rows || m.cols != want_cols || base + 128 > m.rows || !m.data ||
      !m.suh || !m.svh) {
    WaitForPredecessor();
    if (!threadIdx.x)
      Raise(a.bad);
    return;
  }
  const int span = m.cols / a.slices, k_begin = slice * span; // inputs of this slice, a multiple of 128
  const int stride = span + 8;
  __half *xs = reinterpret_cast<__half *>(smem);

  // ---- the first packed words go in flight before anything else is touched ----
  const int g = lane >> 2, t = lane & 3;
  const int tiles_per_kstep = m.rows / 16, column = blockIdx.x * 8 + warp;
  const unsigned char *lane_base =
      m.data + (static_cast<size_t>(k_begin / 16 + t) * tiles_per_kstep + column) * L::kTileBytes + g * L::kBytes;
  const size_t round_bytes = static_cast<size_t>(4) * tiles_per_kstep * L::kTileBytes;
  const int rounds = span / 64; // even: a slice is a whole number of 128-input blocks
  uint32_t fetched[4][Rate];   // four rounds in flight; short slices re-read their last pair instead of branching
#pragma unroll
  for (int d = 0; d < 4; ++d)
    codec::LoadWords<Rate>(lane_base + static_cast<size_t>(d < rounds ? d : rounds - 2 + (d & 1)) * round_bytes, fetched[d]);

  WaitForPredecessor(); // from here on: the activations the predecessor wrote, and this kernel's own stores
  if (*a.bad)
    return;

  // ---- activation rows of the slice, permuted K16 order ----
  if (a.phase == 0) {
    for (int n = 0; n < count; ++n) {
      const float *x = a.normalized + static_cast<size_t>(rows[n] >> 3) * m.cols + k_begin;
      for (int h = warp; h < span / 128; h += 8) {
        const int k = h * 128 + lane * 4;
        const float4 src = __ldg(reinterpret_cast<const float4 *>(x + k));
        float sg[4];
        Unpack4(__ldg(reinterpret_cast<const uint2 *>(m.suh + k_begin + k)), sg);
        float v[4] = {__fmul_rn(src.x, sg[0]), __fmul_rn(src.y, sg[1]), __fmul_rn(src.z, sg[2]), __fmul_rn(src.w, sg[3])};
        WarpHadamard128(v);
        __half hv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float r = RoundBF16(v[j]);
          hv[j] = __float2half_rn(r);
          if (!isfinite(r) || (__half_as_ushort(hv[j]) & 0x7c00) == 0x7c00)
            Raise(a.bad);
        }
        __half *dst = xs + n * stride + (k >> 4) * 16 + 8 * (lane & 1) + 2 * ((lane >> 1) & 1);
        *reinterpret_cast<__half2 *>(dst) = __halves2half2(hv[0], hv[1]);
        *reinterpret_cast<__half2 *>(dst + 4) = __halves2half2(hv[2], hv[3]);
      }
    }
  } else {
    for (int n = 0; n < count; ++n) {
      const __half *x = a.xdown + static_cast<size_t>(rows[n]) * m.cols + k_begin;
      for (int i = threadIdx.x; i < span / 8; i += kThreads)
        *reinterpret_cast<uint4 *>(xs + n * stride + i * 8) = __ldcg(reinterpret_cast<const uint4 *>(x + i * 8));
    }
  }
  __syncthreads();

  // ---- stream, decode, multiply (lane ownership as in decode.cu) ----
  float acc[NG][4];
  const __half *xrow[NG];
#pragma unroll
  for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      acc[ng][j] = 0.f;
    const int n = g + 8 * ng;
    xrow[ng] = xs + (n < count ? n : count - 1) * stride + t * 16;
  }
  auto multiply = [&](const uint32_t (&words)[Rate], int round) {
    const uint32_t previous = __shfl_sync(0xffffffffu, words[Rate - 1], (lane + 28) & 31);
    uint32_t frag[4][4];
    codec::Decode32<Rate>(words, previous, frag);
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
      const uint4 lo = *reinterpret_cast<const uint4 *>(xrow[ng] + round * 64);
      const uint4 hi = *reinterpret_cast<const uint4 *>(xrow[ng] + round * 64 + 8);
      MmaF16(frag[0], lo.x, lo.y, acc[ng]);
      MmaF16(frag[1], lo.z, lo.w, acc[ng]);
      MmaF16(frag[2], hi.x, hi.y, acc[ng]);
      MmaF16(frag[3], hi.z, hi.w, acc[ng]);
    }
  };
  // Two rounds per half-iteration; while one pair is multiplied the pair four rounds ahead is requested.  The
  // prefetch index is clamped to the slice's last pair, so the tail re-reads words instead of branching.
  for (int round = 0; round < rounds; round += 4) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = round + 2 * half;
      if (r < rounds) { // warp-uniform
        uint32_t now_even[Rate], now_odd[Rate];
#pragma unroll
        for (int i = 0; i < Rate; ++i) {
          now_even[i] = fetched[2 * half][i];
          now_odd[i] = fetched[2 * half + 1][i];
        }
        const int ahead = r + 4 < rounds ? r + 4 : rounds - 2;
        codec::LoadWords<Rate>(lane_base + static_cast<size_t>(ahead) * round_bytes, fetched[2 * half]);
        codec::LoadWords<Rate>(lane_base + static_cast<size_t>(ahead + 1) * round_bytes, fetched[2 * half + 1]);
        multiply(now_even, r);
        multiply(now_odd, r + 1);
      }
    }
  }
  // accumulator (row g | g+8, column 2t | 2t+1) -> this slice's sums of the warp's 16 outputs
#pragma unroll
  for (int ng = 0; ng < NG; ++ng)
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int n = 8 * ng + 2 * t + c;
      if (n < count) {
        const size_t pair = rows[n];
        float *p = a.phase ? a.partials + (pair * a.slices + slice) * a.hidden
                           : a.partials + ((pair * 2 + part) * a.slices + slice) * a.inter;
        p[base + warp * 16 + g] = acc[ng][c];
        p[base + warp * 16 + g + 8] = acc[ng][2 + c];
      }
    }
}

// One warp per (pair, 128-output block): reference arithmetic expert_exl3_decode_dual.cuh:116-130 (output side of
// gate and up), exl3_silu_lut.cuh:15-31 (SwiGLU), expert_exl3_decode_dual.cuh:65-85 (input side of down).
__global__ void __launch_bounds__(128) GateUpEpilogueKernel(const Matrix *matrices, int layer, const int *ids, int pairs, int hidden,
                                                            int inter, int slices, const float *partials,
                                                            const unsigned short *table, __half *xdown, int *bad) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pair = blockIdx.y, nb = blockIdx.x * 4 + warp;
  LetSuccessorLaunch();
  // what does not depend on the projection kernel (ids, descriptors, sidecars: the caller's inputs, complete before
  // the pipeline's first kernel started) is fetched before waiting for it: three dependent round trips to L2 less
  const bool in_range = pair < pairs && nb < inter / 128;
  const int expert = in_range ? ids[pair] : -1;
  const bool valid = expert >= 0 && expert < kExperts;
  const Matrix *m = matrices + (static_cast<size_t>(layer) * kExperts + (valid ? expert : 0)) * 3;
  const int out = nb * 128 + lane * 4;
  float svg[4], svu[4], shd[4];
  // a descriptor that does not fit the call was rejected by the projection kernel (sticky flag, checked below); do not
  // read through it here
  if (valid && m[0].svh && m[1].svh && m[2].suh && m[0].rows == inter && m[1].rows == inter && m[2].cols == inter) {
    Unpack4(__ldg(reinterpret_cast<const uint2 *>(m[0].svh + out)), svg);
    Unpack4(__ldg(reinterpret_cast<const uint2 *>(m[1].svh + out)), svu);
    Unpack4(__ldg(reinterpret_cast<const uint2 *>(m[2].suh + out)), shd);
  }
  WaitForPredecessor();
  if (*bad || !in_range)
    return;
  if (!valid) {
    if (!lane)
      Raise(bad);
    return;
  }
  float gsum[4] = {0.f, 0.f, 0.f, 0.f}, usum[4] = {0.f, 0.f, 0.f, 0.f};
  const float *pg = partials + (static_cast<size_t>(pair) * 2 + 0) * slices * inter + out;
  const float *pu = partials + (static_cast<size_t>(pair) * 2 + 1) * slices * inter + out;
  float4 vg[kMaxSlices], vu[kMaxSlices];
#pragma unroll
  for (int s = 0; s < kMaxSlices; ++s)
    if (s < slices) {
      vg[s] = *reinterpret_cast<const float4 *>(pg + static_cast<size_t>(s) * inter);
      vu[s] = *reinterpret_cast<const float4 *>(pu + static_cast<size_t>(s) * inter);
    }
#pragma unroll
  for (int s = 0; s < kMaxSlices; ++s)
    if (s < slices) {
      gsum[0] += vg[s].x, gsum[1] += vg[s].y, gsum[2] += vg[s].z, gsum[3] += vg[s].w;
      usum[0] += vu[s].x, usum[1] += vu[s].y, usum[2] += vu[s].z, usum[3] += vu[s].w;
    }
  WarpHadamard128(gsum);
  WarpHadamard128(usum);
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float gate = RoundBF16(__fmul_rn(gsum[i], svg[i]));
    const float up = RoundBF16(__fmul_rn(usum[i], svu[i]));
    if (!isfinite(gate) || !isfinite(up))
      Raise(bad);
    const float silu = FromBF16Bits(__ldg(table + (__float_as_uint(gate) >> 16)));
    const float act = RoundBF16(__fmul_rn(silu, up));
    if (!isfinite(act))
      Raise(bad);
    v[i] = __fmul_rn(act, shd[i]);
  }
  WarpHadamard128(v);
  __half hv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float r = RoundBF16(v[i]);
    hv[i] = __float2half_rn(r);
    if (!isfinite(r) || (__half_as_ushort(hv[i]) & 0x7c00) == 0x7c00)
      Raise(bad);
  }
  __half *dst = xdown + static_cast<size_t>(pair) * inter + nb * 128 + (lane >> 2) * 16 + 8 * (lane & 1) + 2 * ((lane >> 1) & 1);
  *reinterpret_cast<__half2 *>(dst) = __halves2half2(hv[0], hv[1]);
  *reinterpret_cast<__half2 *>(dst + 4) = __halves2half2(hv[2], hv[3]);
}

// One CTA per (token, 128-output block), one warp per slot; warp 0 then combines the eight slots in order.
// Reference arithmetic: expert_exl3_decode_dual.cuh:116-130 and Combine, src/cuda/inference.cu:580-594.
__global__ void __launch_bounds__(256) DownEpilogueKernel(const Matrix *matrices, int layer, const int *ids, const float *routing,
                                                          int tokens, int hidden, int slices, const float *partials, float *x,
                                                          int *bad) {
  __shared__ float s_down[kTopK][128];
  const int lane = threadIdx.x & 31, slot = threadIdx.x >> 5;
  const int token = blockIdx.y, nb = blockIdx.x;
  LetSuccessorLaunch();
  // ids, descriptors and sidecars do not depend on the projection kernel: fetched before waiting for it
  const int pair = token * kTopK + slot, out = nb * 128 + lane * 4;
  const int expert = token < tokens ? ids[pair] : -1;
  const bool valid = expert >= 0 && expert < kExperts;
  float sc[4] = {0.f, 0.f, 0.f, 0.f};
  if (valid) { // a descriptor that does not fit was rejected by the projection kernel: do not read through it here
    const Matrix &m = matrices[(static_cast<size_t>(layer) * kExperts + expert) * 3 + 2];
    if (m.svh && m.rows == hidden)
      Unpack4(__ldg(reinterpret_cast<const uint2 *>(m.svh + out)), sc);
  }
  WaitForPredecessor();
  if (*bad || token >= tokens)
    return;
  if (!valid && !lane)
    Raise(bad);
  float d[4] = {0.f, 0.f, 0.f, 0.f};
  if (valid) {
    const float *pd = partials + static_cast<size_t>(pair) * slices * hidden + out;
    float4 vd[kMaxSlices];
#pragma unroll
    for (int s = 0; s < kMaxSlices; ++s)
      if (s < slices)
        vd[s] = *reinterpret_cast<const float4 *>(pd + static_cast<size_t>(s) * hidden);
#pragma unroll
    for (int s = 0; s < kMaxSlices; ++s)
      if (s < slices)
        d[0] += vd[s].x, d[1] += vd[s].y, d[2] += vd[s].z, d[3] += vd[s].w;
    WarpHadamard128(d);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      d[i] = RoundBF16(__fmul_rn(d[i], sc[i]));
      if (!isfinite(d[i]))
        Raise(bad);
    }
  }
  *reinterpret_cast<float4 *>(&s_down[slot][lane * 4]) = make_float4(d[0], d[1], d[2], d[3]);
  __syncthreads();
  if (slot == 0) {
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < kTopK; ++s) {
      const float w = routing[token * kTopK + s];
      const float4 dv = *reinterpret_cast<const float4 *>(&s_down[s][lane * 4]);
      sum[0] = RoundBF16(__fadd_rn(sum[0], RoundBF16(__fmul_rn(dv.x, w))));
      sum[1] = RoundBF16(__fadd_rn(sum[1], RoundBF16(__fmul_rn(dv.y, w))));
      sum[2] = RoundBF16(__fadd_rn(sum[2], RoundBF16(__fmul_rn(dv.z, w))));
      sum[3] = RoundBF16(__fadd_rn(sum[3], RoundBF16(__fmul_rn(dv.w, w))));
    }
    float4 xv = *reinterpret_cast<const float4 *>(x + static_cast<size_t>(token) * hidden + out);
    xv.x = RoundBF16(__fadd_rn(xv.x, sum[0]));
    xv.y = RoundBF16(__fadd_rn(xv.y, sum[1]));
    xv.z = RoundBF16(__fadd_rn(xv.z, sum[2]));
    xv.w = RoundBF16(__fadd_rn(xv.w, sum[3]));
    if (!isfinite(xv.x) || !isfinite(xv.y) || !isfinite(xv.z) || !isfinite(xv.w))
      Raise(bad);
    *reinterpret_cast<float4 *>(x + static_cast<size_t>(token) * hidden + out) = xv;
  }
}

struct SplitWorkspace {
  size_t gateup, xdown, down, total;
  SplitWorkspace(int tokens, int hidden, int inter) {
    const size_t pairs = static_cast<size_t>(tokens) * kTopK;
    auto align = [](size_t n) { return (n + 255) & ~static_cast<size_t>(255); };
    size_t at = 0;
    gateup = at, at += align(pairs * 2 * kMaxSlices * inter * sizeof(float));
    xdown = at, at += align(pairs * inter * sizeof(__half));
    down = at, at += align(pairs * kMaxSlices * hidden * sizeof(float));
    total = at;
  }
};

// `programmatic` = the kernel may start before its predecessor in the stream has finished and waits for it itself.
// The first kernel of the pipeline is launched without it: what precedes it is the caller's work (router, norm),
// whose results it reads from its first instruction on.
template <typename... KernelArgs, typename... Args>
int LaunchDependent(bool programmatic, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                    Args... args) {
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = programmatic ? 1 : 0;
  cudaLaunchConfig_t config{};
  config.gridDim = grid, config.blockDim = block, config.dynamicSmemBytes = smem, config.stream = stream;
  config.attrs = &attribute, config.numAttrs = 1;
  return CudaStatus(cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...));
}

// K-slices: enough CTAs to fill the machine about four deep, slices of whole 128-input blocks.
int PickSlices(int cols, int base_ctas) {
  int slices = kMaxSlices;
  while (slices > 1 && ((cols / 128) % slices != 0 || base_ctas * slices > 1024))
    slices /= 2;
  return slices;
}

template <int Rate, int NG> int LaunchSplit(const SplitArgs &a, dim3 grid, size_t smem, cudaStream_t stream) {
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    if (cudaFuncSetAttribute(SplitProjectionKernel<Rate, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
      return PADRA_RESOURCE_EXHAUSTED;
    configured = smem;
  }
  return LaunchDependent(a.phase != 0, SplitProjectionKernel<Rate, NG>, grid, dim3(kThreads), smem, stream, a);
}

int DispatchSplit(const SplitArgs &a, int rate, bool wide, dim3 grid, size_t smem, cudaStream_t stream) {
  switch (rate) {
  case 3:
    return wide ? LaunchSplit<3, 2>(a, grid, smem, stream) : LaunchSplit<3, 1>(a, grid, smem, stream);
  case 4:
    return wide ? LaunchSplit<4, 2>(a, grid, smem, stream) : LaunchSplit<4, 1>(a, grid, smem, stream);
  case 6:
    return wide ? LaunchSplit<6, 2>(a, grid, smem, stream) : LaunchSplit<6, 1>(a, grid, smem, stream);
  default:
    return PADRA_UNSUPPORTED;
  }
}

} // namespace

size_t SplitDecodeWorkspaceBytes(int tokens, int hidden, int inter) {
  return SplitWorkspace(tokens, hidden, inter).total;
}

int LaunchSplitDecodeLayer(const Matrix *matrices, int layer, const int *ids, const float *routing, const float *normalized,
                           float *x, int tokens, int rate, int hidden, int inter, const unsigned short *table, void *workspace,
                           size_t workspace_bytes, int *bad, cudaStream_t stream, unsigned launches) {
  const SplitWorkspace w(tokens, hidden, inter);
  if (workspace_bytes < w.total)
    return PADRA_RESOURCE_EXHAUSTED;
  auto *base = static_cast<unsigned char *>(workspace);
  float *gateup = reinterpret_cast<float *>(base + w.gateup), *down = reinterpret_cast<float *>(base + w.down);
  __half *xdown = reinterpret_cast<__half *>(base + w.xdown);
  const int pairs = tokens * kTopK, units = pairs < kExperts ? pairs : kExperts;
  const bool wide = tokens > 8;
  const int rows = wide ? 16 : 8;

  SplitArgs a{};
  a.matrices = matrices, a.layer = layer, a.ids = ids, a.tokens = tokens, a.hidden = hidden, a.inter = inter;
  a.normalized = normalized, a.xdown = xdown, a.bad = bad;
  // gate + up
  a.phase = 0, a.partials = gateup, a.slices = PickSlices(hidden, (inter / 128) * units * 2);
  size_t smem = static_cast<size_t>(tokens == 1 ? 1 : rows) * (hidden / a.slices + 8) * sizeof(__half);
  int status = PADRA_OK;
  if (launches & 1u)
    status = DispatchSplit(a, rate, wide, dim3(inter / 128, units, 2 * a.slices), smem, stream);
  if (status != PADRA_OK)
    return status;
  if (launches & 2u)
    status = LaunchDependent(true, GateUpEpilogueKernel, dim3((inter / 128 + 3) / 4, pairs), dim3(128), 0, stream, matrices, layer, ids,
                             pairs, hidden, inter, a.slices, static_cast<const float *>(gateup), table, xdown, bad);
  if (status != PADRA_OK)
    return status;
  // down
  a.phase = 1, a.partials = down, a.slices = PickSlices(inter, (hidden / 128) * units);
  smem = static_cast<size_t>(tokens == 1 ? 1 : rows) * (inter / a.slices + 8) * sizeof(__half);
  if ((launches & 4u) && (status = DispatchSplit(a, rate, wide, dim3(hidden / 128, units, a.slices), smem, stream)) != PADRA_OK)
    return status;
  if (launches & 8u)
    status = LaunchDependent(true, DownEpilogueKernel, dim3(hidden / 128, tokens), dim3(256), 0, stream, matrices, layer, ids, routing,
                             tokens, hidden, a.slices, static_cast<const float *>(down), x, bad);
  return status;
}

} // namespace padra
