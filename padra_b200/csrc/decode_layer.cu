// Whole EXL3 expert layer at decode (M = 1..16 rows) as TWO launches:
//
//   1. LayerProjectionKernel<.., 0>, gate+up : every (expert, 128-output block, matrix, K-slice) is one CTA that streams
//      its slice of packed words, decodes in registers (codec.cuh) and multiplies with
//      mma.m16n8k16; the FP32 sums of the slice go to the workspace.  The CTA that delivers the LAST slice of an
//      (expert, block) -- it learns so from a ticket counter -- runs that block's epilogue: slice sums in ascending
//      order, output Hadamard and svh for gate and up, SwiGLU, the down projection's input transform; it writes the
//      block's 128 FP16 inputs of the down projection.
//   2. LayerProjectionKernel<.., 1>, down : the same streaming over the down matrices; the CTA that delivers the last
//      slice of a (token, block) sums the slices of each of the token's eight slots, applies output Hadamard, svh and
//      BF16 rounding, and then the reference's combine with routing weights and residual.
//
// Splitting K over CTAs is what fills the machine at M = 1 (8 experts x 8 blocks x 2 matrices are only 128 work items).
// Reference arithmetic: src/cuda/expert_exl3_decode_dual.cuh:65-130 (input transform, dot, output transform),
// src/cuda/exl3_silu_lut.cuh:15-31 (SwiGLU), src/cuda/inference.cu:580-594 (combine).  All summation orders are fixed
// (ascending slice, ascending slot) whichever CTA happens to run an epilogue: results are bit-identical run to run.
//
// Launch overlap: both kernels are launched with programmatic stream serialization.  The down kernel's CTAs become
// resident while the gate+up kernel drains, look up their unit, check descriptors and put their first packed words in
// flight, and only then wait for the gate+up kernel.  The gate+up kernel waits at its top: its expert ids are the
// caller's preceding work.  The gate+up CTAs also ask L2 to fetch the down matrices of their expert, so that the down
// kernel's loads meet them there.
//
// Tickets: one counter per (unit, block) for gate+up and per (token, block) for down, at the start of the workspace.
// They must be zero before the first call on a workspace (padra_exl3_moe_decode_workspace_init); every CTA that takes
// part takes its ticket whether or not it could do its work (error paths included), and the CTA that takes the last one
// clears the counter, so every call leaves them zero.  No CTA ever waits for another one.
#include <cstdlib>

#include "decode_common.cuh"

namespace padra {
#ifdef PADRA_DECODE_TRACE
namespace decode {
unsigned long long *g_trace = nullptr;
int g_trace_launch = 0;
} // namespace decode
#endif
namespace {
using namespace decode;

struct LayerArgs {
  const Matrix *matrices;
  int layer;
  const int *ids;          // [tokens][8]
  const float *routing;    // [tokens][8]
  const float *normalized; // [tokens][hidden]
  float *x;                // [tokens][hidden], residual in/out
  int tokens, hidden, inter, slices;
  const unsigned short *table; // SwiGLU table
  float *partials;             // gate+up: [pair][2][slices][inter]; down: [pair][slices][hidden]
  __half *xdown;               // [pair][inter], in the order the B fragments are read (codec::PermutedInput per K16 step)
  __half *svh_rows;            // [pair][hidden]: the down matrices' svh, copied beside the partial sums
  unsigned *tickets;           // gate+up: [unit][kMaxBlocks]; down: [token][kMaxBlocks]
  int *bad;
  unsigned long long *trace; // scratch builds only
};


// Unit `unit` of the launch.  One token: the unit is the slot, and it takes part (count = 1) even when its id is
// invalid, because the token's combine counts on eight arrivals.  Several tokens: the unit-th active expert in ascending
// id with the rows (token*8+slot) routed to it; any invalid id refuses the whole step, the same way in every CTA.
// expert < 0: nothing to compute.  count == 0: nothing to do at all.
template <int NG>
__device__ __forceinline__ void ResolveUnit(const int *ids, int tokens, int unit, int &expert, int &count, int (&rows)[8 * NG],
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
    if (tid == 0 && unit < kTopK) {
      const int e = ids[unit];
      if (e < 0 || e >= kExperts)
        Raise(bad);
      else
        s_expert = e;
      s_count = 1;
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
    asm volatile("bar.sync 1, 64;" ::: "memory"); // both warps of the first 64 threads see both ballots
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
    expert = -1, count = 0;
    return;
  }
  expert = s_expert;
  count = s_count;
#pragma unroll
  for (int i = 0; i < 8 * NG; ++i)
    rows[i] = i < count ? s_rows[i] : 0;
}

// Epilogue of one (pair, 128-output block) of gate+up, one warp: the block's 128 inputs of the down projection.
__device__ __forceinline__ void GateUpEpilogue(const LayerArgs &a, const Matrix *m, int pair, int nb, int lane) {
  const int out = nb * 128 + lane * 4;
  float gsum[4] = {0.f, 0.f, 0.f, 0.f}, usum[4] = {0.f, 0.f, 0.f, 0.f};
  const float *pg = a.partials + (static_cast<size_t>(pair) * 2 + 0) * a.slices * a.inter + out;
  const float *pu = a.partials + (static_cast<size_t>(pair) * 2 + 1) * a.slices * a.inter + out;
  float svg[4], svu[4], shd[4];
  Unpack4(__ldg(reinterpret_cast<const uint2 *>(m[0].svh + out)), svg);
  Unpack4(__ldg(reinterpret_cast<const uint2 *>(m[1].svh + out)), svu);
  Unpack4(__ldg(reinterpret_cast<const uint2 *>(m[2].suh + out)), shd);
  for (int s0 = 0; s0 < a.slices; s0 += 4) { // four slices of each matrix in flight, summed in ascending order
    float4 vg[4], vu[4];
#pragma unroll
    for (int s = 0; s < 4; ++s)
      if (s0 + s < a.slices) {
        vg[s] = __ldcg(reinterpret_cast<const float4 *>(pg + static_cast<size_t>(s0 + s) * a.inter));
        vu[s] = __ldcg(reinterpret_cast<const float4 *>(pu + static_cast<size_t>(s0 + s) * a.inter));
      }
#pragma unroll
    for (int s = 0; s < 4; ++s)
      if (s0 + s < a.slices) {
        gsum[0] += vg[s].x, gsum[1] += vg[s].y, gsum[2] += vg[s].z, gsum[3] += vg[s].w;
        usum[0] += vu[s].x, usum[1] += vu[s].y, usum[2] += vu[s].z, usum[3] += vu[s].w;
      }
  }
  WarpHadamard128(gsum);
  WarpHadamard128(usum);
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float gate = RoundBF16(__fmul_rn(gsum[i], svg[i]));
    const float up = RoundBF16(__fmul_rn(usum[i], svu[i]));
    if (!isfinite(gate) || !isfinite(up))
      Raise(a.bad);
    const float silu = FromBF16Bits(__ldg(a.table + (__float_as_uint(gate) >> 16)));
    const float act = RoundBF16(__fmul_rn(silu, up));
    if (!isfinite(act))
      Raise(a.bad);
    v[i] = __fmul_rn(act, shd[i]);
  }
  WarpHadamard128(v);
  __half *dst = a.xdown + static_cast<size_t>(pair) * a.inter;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float r = RoundBF16(v[i]);
    const __half h = __float2half_rn(r);
    if (!isfinite(r) || (__half_as_ushort(h) & 0x7c00) == 0x7c00)
      Raise(a.bad);
    dst[PermutedPlace(out + i)] = h;
  }
}

// Epilogue of one (token, 128-output block) of down, all eight warps (warp = slot), then warp 0 combines.
__device__ __forceinline__ void DownEpilogue(const LayerArgs &a, int token, int nb, float (*s_down)[128]) {
  const int lane = threadIdx.x & 31, slot = threadIdx.x >> 5;
  const int pair = token * kTopK + slot, out = nb * 128 + lane * 4;
  const float *pd = a.partials + static_cast<size_t>(pair) * a.slices * a.hidden + out;
  float4 vd[kMaxSlices];
#pragma unroll
  for (int s = 0; s < kMaxSlices; ++s)
    if (s < a.slices)
      vd[s] = __ldcg(reinterpret_cast<const float4 *>(pd + static_cast<size_t>(s) * a.hidden));
  float sc[4];
  Unpack4(__ldcg(reinterpret_cast<const uint2 *>(a.svh_rows + static_cast<size_t>(pair) * a.hidden + out)), sc);
  float w = 0.f;
  float4 xv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (slot == 0) {
    w = lane < kTopK ? a.routing[token * kTopK + lane] : 0.f;
    xv = *reinterpret_cast<const float4 *>(a.x + static_cast<size_t>(token) * a.hidden + out);
  }
  float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < kMaxSlices; ++s)
    if (s < a.slices)
      d[0] += vd[s].x, d[1] += vd[s].y, d[2] += vd[s].z, d[3] += vd[s].w;
  WarpHadamard128(d);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    d[i] = RoundBF16(__fmul_rn(d[i], sc[i]));
    if (!isfinite(d[i]))
      Raise(a.bad);
  }
  *reinterpret_cast<float4 *>(&s_down[slot][lane * 4]) = make_float4(d[0], d[1], d[2], d[3]);
  __syncthreads();
  if (slot == 0) {
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < kTopK; ++s) {
      const float ws = __shfl_sync(0xffffffffu, w, s);
      const float4 dv = *reinterpret_cast<const float4 *>(&s_down[s][lane * 4]);
      sum[0] = RoundBF16(__fadd_rn(sum[0], RoundBF16(__fmul_rn(dv.x, ws))));
      sum[1] = RoundBF16(__fadd_rn(sum[1], RoundBF16(__fmul_rn(dv.y, ws))));
      sum[2] = RoundBF16(__fadd_rn(sum[2], RoundBF16(__fmul_rn(dv.z, ws))));
      sum[3] = RoundBF16(__fadd_rn(sum[3], RoundBF16(__fmul_rn(dv.w, ws))));
    }
    xv.x = RoundBF16(__fadd_rn(xv.x, sum[0]));
    xv.y = RoundBF16(__fadd_rn(xv.y, sum[1]));
    xv.z = RoundBF16(__fadd_rn(xv.z, sum[2]));
    xv.w = RoundBF16(__fadd_rn(xv.w, sum[3]));
    if (!isfinite(xv.x) || !isfinite(xv.y) || !isfinite(xv.z) || !isfinite(xv.w))
      Raise(a.bad);
    *reinterpret_cast<float4 *>(a.x + static_cast<size_t>(token) * a.hidden + out) = xv;
  }
  __syncthreads(); // s_down may be refilled for the next token
}

// Phase 0: gate and up from `normalized`; Phase 1: down from `xdown`.
template <int Rate, int NG, int Phase>
__global__ void __launch_bounds__(kThreads, 4) LayerProjectionKernel(LayerArgs a) {
  using L = codec::Lane<Rate>;
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ __align__(16) float s_down[Phase ? kTopK : 1][128];
  __shared__ unsigned s_done;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  PADRA_TRACE(a.trace, 0);
  // Gate+up: the ids, activations and the error flag are the work of whatever ran before this call, so it waits first,
  // and lets the down kernel start only then: the down kernel reads the ids before its own wait.
  if (Phase == 0)
    WaitForPredecessor();
  LetSuccessorLaunch();
  PADRA_TRACE(a.trace, 1);
  int expert, count, rows[8 * NG];
  ResolveUnit<NG>(a.ids, a.tokens, blockIdx.y, expert, count, rows, a.bad);
  PADRA_TRACE(a.trace, 2);
  if (count == 0)
    return; // the same in every CTA of the unit: nobody takes this unit's tickets
  const int part = Phase ? 2 : static_cast<int>(blockIdx.z) / a.slices;
  const int slice = static_cast<int>(blockIdx.z) % a.slices;
  const int nb = blockIdx.x, base = nb * 128;
  const Matrix *unit_matrices = a.matrices + (static_cast<size_t>(a.layer) * kExperts + (expert < 0 ? 0 : expert)) * 3;
  Matrix m{};
  bool work = expert >= 0;
  if (work) {
    m = unit_matrices[part];
    const int want_rows = Phase ? a.hidden : a.inter, want_cols = Phase ? a.inter : a.hidden;
    if (m.format != FormatOfRate(Rate) || m.rows != want_rows || m.cols != want_cols || base + 128 > m.rows || !m.data || !m.suh ||
        !m.svh) {
      if (!tid)
        Raise(a.bad);
      work = false;
    }
  }
  PADRA_TRACE(a.trace, 3);
  const int cols = Phase ? a.inter : a.hidden;
  const int span = cols / a.slices, k_begin = slice * span; // inputs of this slice, a multiple of 128
  const int stride = span + 8;
  const int rounds = span / 64; // even
  __half *xs = reinterpret_cast<__half *>(smem);
  const int g = lane >> 2, t = lane & 3;

  // ---- the first packed words go in flight before anything else is touched ----
  const unsigned char *lane_base = nullptr;
  size_t round_bytes = 0;
  uint32_t fetched[4][Rate] = {}; // four rounds in flight; short slices re-read their last pair instead of branching
  uint2 svh_bits = make_uint2(0u, 0u);
  if (work) {
    const int tiles_per_kstep = m.rows / 16, column = nb * 8 + warp;
    lane_base = m.data + (static_cast<size_t>(k_begin / 16 + t) * tiles_per_kstep + column) * L::kTileBytes + g * L::kBytes;
    round_bytes = static_cast<size_t>(4) * tiles_per_kstep * L::kTileBytes;
#pragma unroll
    for (int d = 0; d < 4; ++d)
      codec::LoadWords<Rate>(lane_base + static_cast<size_t>(d < rounds ? d : rounds - 2 + (d & 1)) * round_bytes, fetched[d]);
    if (Phase == 0) {
      // hints for what comes later: the sidecars the block's epilogue reads, this CTA's share of the expert's down matrix
      if (slice == 0 && warp == 1 && lane < 2 && (reinterpret_cast<uintptr_t>(m.svh) & 15) == 0)
        PrefetchL2(reinterpret_cast<const unsigned char *>(m.svh + base) + lane * 128, 128);
      if (warp == 2 && lane == 0) {
        const Matrix &down = unit_matrices[2];
        const unsigned ctas = gridDim.x * gridDim.z, index = blockIdx.z * gridDim.x + blockIdx.x;
        const size_t bytes = static_cast<size_t>(a.hidden) * a.inter * Rate / 8;
        if (down.data && down.format == FormatOfRate(Rate) && down.rows == a.hidden && down.cols == a.inter &&
            bytes % (static_cast<size_t>(ctas) * 16) == 0 && (reinterpret_cast<uintptr_t>(down.data) & 15) == 0)
          PrefetchL2(down.data + index * (bytes / ctas), static_cast<unsigned>(bytes / ctas));
        if (index == 0 && down.suh && down.svh && down.cols == a.inter && down.rows == a.hidden) {
          if ((a.inter * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(down.suh) & 15) == 0)
            PrefetchL2(down.suh, static_cast<unsigned>(a.inter * 2));
          if ((a.hidden * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(down.svh) & 15) == 0)
            PrefetchL2(down.svh, static_cast<unsigned>(a.hidden * 2));
        }
      }
    } else if (slice == 0 && warp == 0) {
      svh_bits = __ldg(reinterpret_cast<const uint2 *>(m.svh + base + lane * 4));
    }
  }
  PADRA_TRACE(a.trace, 4);
  if (Phase == 1)
    WaitForPredecessor(); // from here on: what the gate+up kernel wrote, and this kernel's own stores
  if (__syncthreads_or(LoadFlag(a.bad)))
    work = false; // refused or failed earlier: no work, but the tickets are still taken (one verdict for the whole CTA)
  PADRA_TRACE(a.trace, 5);

  if (work) { // uniform over the CTA
    // ---- activation rows of the slice, in the order the B fragments are read ----
    if (Phase == 0) {
      for (int n = 0; n < count; ++n) {
        const float *x = a.normalized + static_cast<size_t>(rows[n] >> 3) * m.cols + k_begin;
        for (int h = warp; h < span / 128; h += 8) {
          const int k = h * 128 + lane * 4;
          const float4 src = __ldg(reinterpret_cast<const float4 *>(x + k));
          float sg[4];
          Unpack4(__ldg(reinterpret_cast<const uint2 *>(m.suh + k_begin + k)), sg);
          float v[4] = {__fmul_rn(src.x, sg[0]), __fmul_rn(src.y, sg[1]), __fmul_rn(src.z, sg[2]), __fmul_rn(src.w, sg[3])};
          WarpHadamard128(v);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float r = RoundBF16(v[j]);
            const __half hv = __float2half_rn(r);
            if (!isfinite(r) || (__half_as_ushort(hv) & 0x7c00) == 0x7c00)
              Raise(a.bad);
            xs[n * stride + PermutedPlace(k + j)] = hv;
          }
        }
      }
    } else {
      for (int n = 0; n < count; ++n) {
        const __half *x = a.xdown + static_cast<size_t>(rows[n]) * m.cols + k_begin;
        for (int i = tid; i < span / 8; i += kThreads)
          *reinterpret_cast<uint4 *>(xs + n * stride + i * 8) = __ldcg(reinterpret_cast<const uint4 *>(x + i * 8));
      }
    }
    __syncthreads();
    PADRA_TRACE(a.trace, 6);
#ifdef PADRA_DECODE_TRACE
    {
      unsigned probe = fetched[0][0] ^ 1u;
      asm volatile("mov.u32 %0, %0;" : "+r"(probe));
      PADRA_TRACE(a.trace, 7);
    }
#endif

    // ---- stream, decode, multiply ----
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
          if (r + 4 < rounds) {
            codec::LoadWords<Rate>(lane_base + static_cast<size_t>(r + 4) * round_bytes, fetched[2 * half]);
            codec::LoadWords<Rate>(lane_base + static_cast<size_t>(r + 5) * round_bytes, fetched[2 * half + 1]);
          }
          multiply(now_even, r);
          multiply(now_odd, r + 1);
        }
      }
    }
    PADRA_TRACE(a.trace, 8);
    // accumulator (row g | g+8, column 2t | 2t+1) -> this slice's sums of the warp's 16 outputs
#pragma unroll
    for (int ng = 0; ng < NG; ++ng)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int n = 8 * ng + 2 * t + c;
        if (n < count) {
          const size_t pair = rows[n];
          float *p = Phase ? a.partials + (pair * a.slices + slice) * a.hidden : a.partials + ((pair * 2 + part) * a.slices + slice) * a.inter;
          p[base + warp * 16 + g] = acc[ng][c];
          p[base + warp * 16 + g + 8] = acc[ng][2 + c];
        }
      }
    if (Phase == 1 && slice == 0 && warp == 0)
      for (int n = 0; n < count; ++n)
        *reinterpret_cast<uint2 *>(a.svh_rows + static_cast<size_t>(rows[n]) * a.hidden + base + lane * 4) = svh_bits;
  }

  // ---- ticket: which CTA delivered the last slice? ----
  // The tickets are drawn behind the CTA's barrier with release and acquire at device scope: the release covers the sums
  // the CTA's threads stored before the barrier, the acquire (where the ticket turns out to be the last) the other CTAs'.
  auto draw = [](unsigned *ticket) {
    unsigned drawn;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(drawn) : "l"(ticket) : "memory");
    return drawn;
  };
  if (tid == 0)
    s_done = 0;
  __syncthreads();
  PADRA_TRACE(a.trace, 9);
  if (Phase == 0) {
    unsigned *ticket = a.tickets + static_cast<size_t>(blockIdx.y) * kMaxBlocks + nb;
    if (tid == 0 && draw(ticket) == 2u * a.slices - 1u) {
      *ticket = 0; // nobody else touches it before the next call
      s_done = 1;
    }
  } else if (tid < count) {
    unsigned *ticket = a.tickets + static_cast<size_t>(rows[tid] >> 3) * kMaxBlocks + nb;
    if (draw(ticket) == static_cast<unsigned>(kTopK) * a.slices - 1u) {
      *ticket = 0;
      atomicOr(&s_done, 1u << tid);
    }
  }
  __syncthreads();
  PADRA_TRACE(a.trace, 10);
  const unsigned done = s_done;
  if (!done)
    return;
  if (__syncthreads_or(LoadFlag(a.bad)))
    return; // some slice was not computed: leave x and the down inputs alone

  if (Phase == 0) {
    const Matrix *mm = unit_matrices;
    const bool fits = mm[0].svh && mm[1].svh && mm[2].suh && mm[0].rows == a.inter && mm[1].rows == a.inter && mm[2].cols == a.inter;
    if (!fits) {
      if (!tid)
        Raise(a.bad);
      return;
    }
    for (int n = warp; n < count; n += 8)
      GateUpEpilogue(a, mm, rows[n], nb, lane);
  } else {
    for (int n = 0; n < count; ++n) // uniform over the CTA
      if (done & (1u << n))
        DownEpilogue(a, rows[n] >> 3, nb, s_down);
  }
  PADRA_TRACE(a.trace, 11);
}

template <int Rate, int NG, int Phase> int LaunchLayerKernel(const LayerArgs &a, dim3 grid, size_t smem, cudaStream_t stream) {
  if (smem > 48 * 1024 && // per device and cheap: no cache that another device or thread could see half-written
      cudaFuncSetAttribute(LayerProjectionKernel<Rate, NG, Phase>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
          cudaSuccess)
    return PADRA_RESOURCE_EXHAUSTED;
  return LaunchProgrammatic(LayerProjectionKernel<Rate, NG, Phase>, grid, dim3(kThreads), smem, stream, a);
}
template <int Phase> int DispatchLayerKernel(const LayerArgs &a, int rate, bool wide, dim3 grid, size_t smem, cudaStream_t stream) {
  switch (rate) {
  case 3:
    return wide ? LaunchLayerKernel<3, 2, Phase>(a, grid, smem, stream) : LaunchLayerKernel<3, 1, Phase>(a, grid, smem, stream);
  case 4:
    return wide ? LaunchLayerKernel<4, 2, Phase>(a, grid, smem, stream) : LaunchLayerKernel<4, 1, Phase>(a, grid, smem, stream);
  case 6:
    return wide ? LaunchLayerKernel<6, 2, Phase>(a, grid, smem, stream) : LaunchLayerKernel<6, 1, Phase>(a, grid, smem, stream);
  default:
    return PADRA_UNSUPPORTED;
  }
}

} // namespace

size_t DecodeLayerWorkspaceBytes(int tokens, int hidden, int inter) {
  return LayerWorkspace(tokens, hidden, inter).total;
}

int InitDecodeLayerWorkspace(void *workspace, size_t bytes, cudaStream_t stream) {
  if (!workspace || bytes == 0)
    return PADRA_INVALID_ARGUMENT;
  return CudaStatus(cudaMemsetAsync(workspace, 0, bytes, stream));
}

int LaunchDecodeLayer(const Matrix *matrices, int layer, const int *ids, const float *routing, const float *normalized, float *x,
                      int tokens, int rate, int hidden, int inter, const unsigned short *table, void *workspace,
                      size_t workspace_bytes, int *bad, cudaStream_t stream, unsigned launches) {
  if (hidden / 128 > kMaxBlocks || inter / 128 > kMaxBlocks)
    return PADRA_UNSUPPORTED;
  const LayerWorkspace w(tokens, hidden, inter);
  if (workspace_bytes < w.total)
    return PADRA_RESOURCE_EXHAUSTED;
  if (tokens == 1)
    return LaunchSingleTokenLayer(matrices, layer, ids, routing, normalized, x, rate, hidden, inter, table, workspace, bad, stream,
                                  launches);
  auto *base = static_cast<unsigned char *>(workspace);
  const int pairs = tokens * kTopK, units = pairs < kExperts ? pairs : kExperts;
  const bool wide = tokens > 8;
  const int rows = tokens == 1 ? 1 : wide ? 16 : 8;

  LayerArgs a{};
  a.matrices = matrices, a.layer = layer, a.ids = ids, a.routing = routing, a.tokens = tokens, a.hidden = hidden, a.inter = inter;
  a.normalized = normalized, a.x = x, a.table = table, a.bad = bad;
#ifdef PADRA_DECODE_TRACE
  a.trace = g_trace ? g_trace + static_cast<size_t>(g_trace_launch++) * 2 * 1024 * 16 : nullptr;
#endif
  a.xdown = reinterpret_cast<__half *>(base + w.xdown), a.svh_rows = reinterpret_cast<__half *>(base + w.svh);
  int status = PADRA_OK;
  if (launches & 1u) { // gate + up
    a.partials = reinterpret_cast<float *>(base + w.gateup), a.slices = w.slices_gateup;
    a.tickets = reinterpret_cast<unsigned *>(base + w.tickets_gateup);
    const size_t smem = static_cast<size_t>(rows) * (hidden / a.slices + 8) * sizeof(__half);
    status = DispatchLayerKernel<0>(a, rate, wide, dim3(inter / 128, units, 2 * a.slices), smem, stream);
  }
  if (status != PADRA_OK)
    return status;
  if (launches & 2u) { // down
    a.partials = reinterpret_cast<float *>(base + w.down), a.slices = w.slices_down;
    a.tickets = reinterpret_cast<unsigned *>(base + w.tickets_down);
    const size_t smem = static_cast<size_t>(rows) * (inter / a.slices + 8) * sizeof(__half);
#ifdef PADRA_DECODE_TRACE
    if (a.trace)
      a.trace += 1024 * 16;
#endif
    status = DispatchLayerKernel<1>(a, rate, wide, dim3(hidden / 128, units, a.slices), smem, stream);
  }
  return status;
}

#ifdef PADRA_DECODE_TRACE
extern "C" __attribute__((visibility("default"))) void padra_debug_set_decode_trace(unsigned long long *buffer) {
  g_trace = buffer, g_trace_launch = 0;
}
#endif

} // namespace padra
