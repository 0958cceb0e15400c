// Decode-side (M = 1..16 rows) EXL3 expert kernels: streaming projection, SwiGLU, combine, row unions.
//
// Projection layout.  One CTA owns 128 consecutive outputs of one (expert, matrix) and all of its inputs;
// each of its 8 warps owns one 16-output tile column.  Per step a warp covers FOUR K16 tiles of that column:
// lane (g = lane/4, t = lane%4) loads the 4*Rate bytes of row-pair g of the tile at K-step 4*round + t
// (one 16-byte load at K4), i.e. 32 weights for outputs g and g+8 and all 16 inputs of that K-step.  The warp
// then issues four mma.m16n8k16: in the c-th, lane (g, t) supplies inputs {2c, 2c+1, 2c+8, 2c+9} of ITS
// K-step as the logical columns {2t, 2t+1, 2t+8, 2t+9}.  The activation rows are stored in shared memory in
// the matching permuted order (codec::PermutedInput) so that a lane's B fragments for all four MMAs are 32
// contiguous bytes.  Tokens that share the expert occupy B columns 0..7 (and a second accumulator set for
// 8..15), so decoded weights are reused across them.  Accumulation is FP32 inside the tensor core.
#include "codec.cuh"
#include "common.cuh"
#include "kernels.cuh"

namespace padra {
namespace {

constexpr int kThreads = 256;
constexpr int kDepth = 4; // packed-word rounds kept in flight per lane

__device__ __forceinline__ void MmaF16(const uint32_t (&a)[4], uint32_t b0, uint32_t b1, float (&d)[4]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct ProjectionArgs {
  const Matrix *matrices;
  int layer, requested_part;
  // pair mode: one row per unit
  const int *ids;
  int pairs;
  // union mode: rows that chose the same expert share a unit
  const unsigned *masks;
  const int *slots;
  int slot_stride;
  const int *active;
  const int *active_count;
  int rows;
  const float *input;
  float *output, *other;
  int *bad;
  int hidden, inter;
  int row_capacity; // shared-memory rows provisioned per CTA (1, 8, 16 or 32)
  // tile mode (prefill): up to 32 pairs of one expert per unit, BF16-bit activations
  const int *groups;
  const padra_tile *tiles;
  const int *tile_count;
  int tokens;
  const unsigned short *gate_bits, *up_bits, *table;
  unsigned short *output_bits;
};

enum RowMode { kPairRows = 0, kUnionRows = 1, kTileRows = 2 };

// xs row stride in halves: +8 halves (16 bytes) puts odd rows on the banks even rows leave free when the
// four K-steps of a quarter-warp are read with 16-byte loads.
__host__ __device__ constexpr int RowStride(int cols) {
  return cols + 8;
}
__host__ __device__ constexpr size_t ProjectionSmem(int cols, int row_capacity) {
  return static_cast<size_t>(row_capacity) * (RowStride(cols) * sizeof(__half) + 128 * sizeof(float));
}

template <int Rate, int NG, int Mode>
__global__ void __launch_bounds__(kThreads) ProjectionKernel(ProjectionArgs a) {
  using L = codec::Lane<Rate>;
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int s_expert, s_count, s_abort;
  __shared__ int s_in[8 * NG], s_out[8 * NG];

  // a decode call for part 0 computes gate and up side by side over grid.z; a prefill call handles one part
  const int part = (Mode != kTileRows && a.requested_part == 0) ? static_cast<int>(blockIdx.z) : a.requested_part;
  float *out = part == 1 ? a.other : a.output;
  if constexpr (Mode == kTileRows)
    out = reinterpret_cast<float *>(a.output_bits); // only tested for presence below
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int want_rows = part == 2 ? a.hidden : a.inter, want_cols = part == 2 ? a.inter : a.hidden;
  const int base = blockIdx.x * 128;

  if (threadIdx.x == 0) {
    int expert = -1, count = 0, abort = 0, raise = 0;
    if (*a.bad) {
      abort = 1; // a failed step is never continued (the host rejects it); keep indices safe and leave
    } else if (!out || blockDim.x != kThreads || part < 0 || part > 2) {
      abort = raise = 1;
    } else if constexpr (Mode == kTileRows) {
      // tiles were laid out on the device (reference: src/cuda/expert_exl3_prefill_transport_async64.cuh:39-66)
      const int unit = blockIdx.y;
      if (unit >= *a.tile_count) {
        abort = 1;
      } else {
        const padra_tile tile = a.tiles[unit];
        if (tile.expert < 0 || tile.expert >= kExperts || tile.valid_rows < 1 || tile.valid_rows > 8 * NG ||
            tile.valid_rows > a.row_capacity || tile.begin < 0 || tile.begin > a.tokens - tile.valid_rows) {
          abort = raise = 1;
        } else {
          expert = tile.expert;
          for (int r = 0; r < tile.valid_rows; ++r) {
            const int pair = a.groups[tile.expert * a.tokens + tile.begin + r];
            if (pair < 0 || pair >= a.tokens * kTopK) {
              abort = raise = 1;
              break;
            }
            s_in[r] = part == 2 ? pair : pair / kTopK;
            s_out[r] = pair;
          }
          count = tile.valid_rows;
        }
      }
    } else if constexpr (Mode == kUnionRows) {
      int unit = blockIdx.y;
      if (a.active) {
        const int n = *a.active_count;
        if (n < 0 || n > kExperts)
          abort = raise = 1;
        else if (unit >= n)
          abort = 1; // uniform early-out past the active list
        else
          expert = a.active[unit];
      } else {
        expert = unit;
      }
      if (!abort) {
        if (expert < 0 || expert >= kExperts) {
          abort = raise = 1;
        } else {
          const unsigned mask = a.masks[expert];
          for (int r = 0; r < a.rows && !abort; ++r) {
            if (!(mask & (1u << r)))
              continue;
            const int slot = a.slots[expert * a.slot_stride + r];
            if (slot < 0 || slot >= kTopK || count >= 8 * NG || count >= a.row_capacity) {
              abort = raise = 1;
              break;
            }
            s_in[count] = part == 2 ? r * kTopK + slot : r;
            s_out[count] = r * kTopK + slot;
            ++count;
          }
          if (!count)
            abort = 1;
        }
      }
    } else {
      const int pair = blockIdx.y;
      if (pair >= a.pairs) {
        abort = 1;
      } else {
        expert = a.ids[pair];
        if (expert < 0 || expert >= kExperts) {
          abort = raise = 1;
        } else {
          s_in[0] = part == 2 ? pair : pair / kTopK;
          s_out[0] = pair;
          count = 1;
        }
      }
    }
    if (!abort) {
      const Matrix &m = a.matrices[(a.layer * kExperts + expert) * 3 + part];
      if (m.format != FormatOfRate(Rate) || m.rows != want_rows || m.cols != want_cols || base + 128 > m.rows ||
          m.cols < 128 || (m.cols % 128) != 0 || (m.rows % 128) != 0 || !m.data || !m.suh || !m.svh)
        abort = raise = 1;
    }
    if (raise)
      Raise(a.bad);
    s_expert = expert;
    s_count = count;
    s_abort = abort;
  }
  __syncthreads();
  if (s_abort)
    return;
  const int count = s_count;
  const Matrix m = a.matrices[(a.layer * kExperts + s_expert) * 3 + part];
  const int cols = m.cols, stride = RowStride(cols);
  __half *xs = reinterpret_cast<__half *>(smem);
  float *raw = reinterpret_cast<float *>(smem + static_cast<size_t>(a.row_capacity) * stride * sizeof(__half));

  // ---- input side: xs[n] = fp16(B(H128(x * suh))) in permuted K16 order (reference arithmetic:
  // src/cuda/expert_exl3_decode_dual.cuh:65-85) ----
  for (int n = 0; n < count; ++n) {
    for (int h = warp; h < cols / 128; h += 8) {
      const int k = h * 128 + lane * 4;
      float4 src;
      if (Mode == kTileRows && part == 2) {
        // SwiGLU applied while building the down-projection input
        // (reference: src/cuda/expert_exl3_prefill_packed_activations.cuh:17-28, :48-56)
        const uint2 gb = *reinterpret_cast<const uint2 *>(a.gate_bits + static_cast<size_t>(s_in[n]) * cols + k);
        const uint2 ub = *reinterpret_cast<const uint2 *>(a.up_bits + static_cast<size_t>(s_in[n]) * cols + k);
        const unsigned short gs[4] = {static_cast<unsigned short>(gb.x & 0xffffu), static_cast<unsigned short>(gb.x >> 16),
                                      static_cast<unsigned short>(gb.y & 0xffffu), static_cast<unsigned short>(gb.y >> 16)};
        const unsigned short us[4] = {static_cast<unsigned short>(ub.x & 0xffffu), static_cast<unsigned short>(ub.x >> 16),
                                      static_cast<unsigned short>(ub.y & 0xffffu), static_cast<unsigned short>(ub.y >> 16)};
        float act[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float gv = FromBF16Bits(gs[j]), uv = FromBF16Bits(us[j]);
          if (!isfinite(gv) || !isfinite(uv)) {
            Raise(a.bad);
            act[j] = 0.f;
          } else {
            act[j] = RoundBF16(__fmul_rn(FromBF16Bits(a.table[gs[j]]), uv));
            if (!isfinite(act[j]))
              Raise(a.bad);
          }
        }
        src = make_float4(act[0], act[1], act[2], act[3]);
      } else {
        src = *reinterpret_cast<const float4 *>(a.input + static_cast<size_t>(s_in[n]) * cols + k);
      }
      const uint2 sign = *reinterpret_cast<const uint2 *>(m.suh + k);
      float v[4] = {__fmul_rn(src.x, HalfBitsToFloat(sign.x & 0xffffu)), __fmul_rn(src.y, HalfBitsToFloat(sign.x >> 16)),
                    __fmul_rn(src.z, HalfBitsToFloat(sign.y & 0xffffu)), __fmul_rn(src.w, HalfBitsToFloat(sign.y >> 16))};
      WarpHadamard128(v);
      __half hv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float r = RoundBF16(v[j]);
        hv[j] = __float2half_rn(r);
        if (!isfinite(r) || (__half_as_ushort(hv[j]) & 0x7c00) == 0x7c00)
          Raise(a.bad);
      }
      // inputs i = 4*(lane&3) + j of K-step (k >> 4); see codec::PermutedInput
      __half *dst = xs + n * stride + (k >> 4) * 16 + 8 * (lane & 1) + 2 * ((lane >> 1) & 1);
      *reinterpret_cast<__half2 *>(dst) = __halves2half2(hv[0], hv[1]);
      *reinterpret_cast<__half2 *>(dst + 4) = __halves2half2(hv[2], hv[3]);
    }
  }
  __syncthreads();

  // ---- stream, decode, multiply ----
  const int g = lane >> 2, t = lane & 3;
  const int tiles_per_kstep = m.rows / 16, column = blockIdx.x * 8 + warp;
  const unsigned char *lane_base =
      m.data + (static_cast<size_t>(t) * tiles_per_kstep + column) * L::kTileBytes + g * L::kBytes;
  const size_t round_bytes = static_cast<size_t>(4) * tiles_per_kstep * L::kTileBytes;
  const int rounds = cols / 64;
  uint32_t fetched[kDepth][Rate];
#pragma unroll
  for (int d = 0; d < kDepth; ++d)
    if (d < rounds)
      codec::LoadWords<Rate>(lane_base + d * round_bytes, fetched[d]);
  float acc[NG][4];
  const __half *xrow[NG];
#pragma unroll
  for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      acc[ng][j] = 0.f;
    const int n = g + 8 * ng;
    xrow[ng] = xs + (n < count ? n : count - 1) * stride + t * 16; // columns past `count` are never read back
  }
  for (int r = 0; r < rounds; r += kDepth) {
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
      const int round = r + d;
      if (round < rounds) { // warp-uniform
        uint32_t words[Rate];
#pragma unroll
        for (int i = 0; i < Rate; ++i)
          words[i] = fetched[d][i];
        if (round + kDepth < rounds)
          codec::LoadWords<Rate>(lane_base + static_cast<size_t>(round + kDepth) * round_bytes, fetched[d]);
        // the word before this lane's words is the last word of row-pair g-1 (cyclic) of the same tile
        const uint32_t previous = __shfl_sync(0xffffffffu, words[Rate - 1], (lane + 28) & 31);
        uint32_t frag[4][4];
        codec::Decode32<Rate>(words, previous, frag);
#pragma unroll
        for (int ng = 0; ng < NG; ++ng) {
          const uint4 b_lo = *reinterpret_cast<const uint4 *>(xrow[ng] + round * 64);
          const uint4 b_hi = *reinterpret_cast<const uint4 *>(xrow[ng] + round * 64 + 8);
          MmaF16(frag[0], b_lo.x, b_lo.y, acc[ng]);
          MmaF16(frag[1], b_lo.z, b_lo.w, acc[ng]);
          MmaF16(frag[2], b_hi.x, b_hi.y, acc[ng]);
          MmaF16(frag[3], b_hi.z, b_hi.w, acc[ng]);
        }
      }
    }
  }
  // accumulator (row g | g+8, column 2t | 2t+1) -> raw[token][output within the 128 block]
#pragma unroll
  for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int n = 8 * ng + 2 * t + c;
      if (n < count) {
        raw[n * 128 + warp * 16 + g] = acc[ng][c];
        raw[n * 128 + warp * 16 + g + 8] = acc[ng][2 + c];
      }
    }
  }
  __syncthreads();

  // ---- output side: y = B(H128(raw) * svh) (src/cuda/expert_exl3_decode_dual.cuh:116-130) ----
  for (int n = warp; n < count; n += 8) {
    float v[4];
    const float4 r4 = *reinterpret_cast<const float4 *>(raw + n * 128 + lane * 4);
    v[0] = r4.x, v[1] = r4.y, v[2] = r4.z, v[3] = r4.w;
    WarpHadamard128(v);
    const uint2 sign = *reinterpret_cast<const uint2 *>(m.svh + base + lane * 4);
    float4 y;
    y.x = RoundBF16(__fmul_rn(v[0], HalfBitsToFloat(sign.x & 0xffffu)));
    y.y = RoundBF16(__fmul_rn(v[1], HalfBitsToFloat(sign.x >> 16)));
    y.z = RoundBF16(__fmul_rn(v[2], HalfBitsToFloat(sign.y & 0xffffu)));
    y.w = RoundBF16(__fmul_rn(v[3], HalfBitsToFloat(sign.y >> 16)));
    if (!isfinite(y.x) || !isfinite(y.y) || !isfinite(y.z) || !isfinite(y.w))
      Raise(a.bad);
    if constexpr (Mode == kTileRows) {
      const uint2 packed = {static_cast<unsigned>(BF16Bits(y.x)) | (static_cast<unsigned>(BF16Bits(y.y)) << 16),
                            static_cast<unsigned>(BF16Bits(y.z)) | (static_cast<unsigned>(BF16Bits(y.w)) << 16)};
      *reinterpret_cast<uint2 *>(a.output_bits + static_cast<size_t>(s_out[n]) * m.rows + base + lane * 4) = packed;
    } else {
      *reinterpret_cast<float4 *>(out + static_cast<size_t>(s_out[n]) * m.rows + base + lane * 4) = y;
    }
  }
}

template <int Rate, int NG, int Mode> int LaunchProjection(const ProjectionArgs &a, dim3 grid, cudaStream_t stream) {
  const int cols = a.hidden > a.inter ? a.hidden : a.inter; // provision for the wider of the two inputs
  const size_t smem = ProjectionSmem(cols, a.row_capacity);
  // set on every launch that needs it: the attribute belongs to the current device, and the call is cheap
  if (smem > 48 * 1024 && cudaFuncSetAttribute(ProjectionKernel<Rate, NG, Mode>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem)) != cudaSuccess)
    return PADRA_RESOURCE_EXHAUSTED;
  ProjectionKernel<Rate, NG, Mode><<<grid, kThreads, smem, stream>>>(a);
  return CudaStatus(cudaGetLastError());
}

template <int Mode, int NG> int DispatchRate(const ProjectionArgs &a, int rate, dim3 grid, cudaStream_t stream) {
  switch (rate) {
  case 3:
    return LaunchProjection<3, NG, Mode>(a, grid, stream);
  case 4:
    return LaunchProjection<4, NG, Mode>(a, grid, stream);
  case 6:
    return LaunchProjection<6, NG, Mode>(a, grid, stream);
  default:
    return PADRA_UNSUPPORTED;
  }
}
template <int Mode> int DispatchProjection(const ProjectionArgs &a, int rate, dim3 grid, cudaStream_t stream) {
  if constexpr (Mode == kTileRows)
    return DispatchRate<Mode, 4>(a, rate, grid, stream);
  else
    return a.row_capacity > 8 ? DispatchRate<Mode, 2>(a, rate, grid, stream) : DispatchRate<Mode, 1>(a, rate, grid, stream);
}

// ---- row unions (reference: src/cuda/mtp_experts.cuh:7-40) ---------------------------------------------
__global__ void BuildUnionKernel(const int *ids, unsigned *masks, int *slots, int rows, int slot_stride, int *bad,
                                 int *active, int *active_count) {
  const int expert = threadIdx.x;
  if (blockDim.x != kExperts || rows < 1 || rows > kMaxDecodeRows || slot_stride < rows) {
    if (!threadIdx.x)
      Raise(bad);
    if (!threadIdx.x && active_count)
      *active_count = 0;
    return;
  }
  unsigned mask = 0;
  for (int r = 0; r < rows; ++r) {
    int found = -1;
    for (int s = 0; s < kTopK; ++s) {
      const int id = ids[r * kTopK + s];
      if (id < 0 || id >= kExperts)
        Raise(bad);
      if (id == expert)
        found = s;
    }
    slots[expert * slot_stride + r] = found;
    if (found >= 0)
      mask |= 1u << r;
  }
  masks[expert] = mask;
  if (active) {
    __shared__ unsigned warp_masks[2];
    const unsigned here = __ballot_sync(0xffffffffu, mask != 0);
    const int lane = expert & 31;
    if (!lane)
      warp_masks[expert >> 5] = here;
    __syncthreads();
    const int rank = __popc(here & ((1u << lane) - 1u)) + (expert >= 32 ? __popc(warp_masks[0]) : 0);
    if (mask)
      active[rank] = expert; // ascending expert order
    if (!expert)
      *active_count = __popc(warp_masks[0]) + __popc(warp_masks[1]);
  }
}

// ---- SwiGLU (reference: src/cuda/exl3_silu_lut.cuh:5-31) -------------------------------------------------
__global__ void SiluBuildKernel(unsigned short *table) {
  const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 65536u)
    return;
  const float g = __uint_as_float(i << 16);
  const float denominator = __fadd_rn(1.f, __double2float_rn(exp(static_cast<double>(-g))));
  table[i] = BF16Bits(__fdiv_rn(g, denominator));
}
__global__ void SiluActivateKernel(float *gate, const float *up, const unsigned short *table, int count, int *bad) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count)
    return;
  const float g = gate[i], u = up[i];
  const unsigned bits = __float_as_uint(g);
  if (!table || !isfinite(g) || !isfinite(u) || (bits & 0xffffu)) {
    Raise(bad);
    return;
  }
  const float v = RoundBF16(__fmul_rn(FromBF16Bits(table[bits >> 16]), u));
  if (!isfinite(v))
    Raise(bad);
  gate[i] = v;
}

// ---- combine (reference: src/cuda/inference.cu:580-594) --------------------------------------------------
template <typename DownT>
__global__ void CombineKernel(float *x, const DownT *down, const float *weights, int rows, int hidden, int *bad,
                              bool residual) {
  const int row = blockIdx.y, col = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows || col >= hidden)
    return;
  float sum = 0.f;
#pragma unroll
  for (int s = 0; s < kTopK; ++s) {
    float d;
    if constexpr (sizeof(DownT) == 2)
      d = FromBF16Bits(down[(static_cast<size_t>(row) * kTopK + s) * hidden + col]);
    else
      d = down[(static_cast<size_t>(row) * kTopK + s) * hidden + col];
    sum = RoundBF16(__fadd_rn(sum, RoundBF16(__fmul_rn(d, weights[row * kTopK + s]))));
  }
  const size_t i = static_cast<size_t>(row) * hidden + col;
  const float v = residual ? RoundBF16(__fadd_rn(x[i], sum)) : sum;
  if (!isfinite(v))
    Raise(bad);
  x[i] = v;
}

// ---- full FP16 decode of one matrix through the kernel codec ------------------------------------------
template <int Rate>
__global__ void DecodeWeightsKernel(const Matrix *matrix, unsigned short *out, int rows, int cols, int *bad) {
  using L = codec::Lane<Rate>;
  const Matrix m = *matrix;
  if (m.format != FormatOfRate(Rate) || m.rows != rows || m.cols != cols || (rows % 16) || (cols % 64)) {
    if (!threadIdx.x && !blockIdx.x)
      Raise(bad);
    return;
  }
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int tiles_per_kstep = rows / 16, rounds = cols / 64;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < rounds * tiles_per_kstep; item += warps) {
    const int round = item / tiles_per_kstep, column = item % tiles_per_kstep;
    const int kstep = round * 4 + t;
    uint32_t words[Rate];
    codec::LoadWords<Rate>(m.data + (static_cast<size_t>(kstep) * tiles_per_kstep + column) * L::kTileBytes + g * L::kBytes,
                           words);
    const uint32_t previous = __shfl_sync(0xffffffffu, words[Rate - 1], (lane + 28) & 31);
    uint32_t frag[4][4];
    codec::Decode32<Rate>(words, previous, frag);
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int o = column * 16 + g + ((f & 1) ? 8 : 0);
        const int i = kstep * 16 + 2 * c + ((f & 2) ? 8 : 0);
        out[static_cast<size_t>(i) * rows + o] = static_cast<unsigned short>(frag[c][f] & 0xffffu);
        out[static_cast<size_t>(i + 1) * rows + o] = static_cast<unsigned short>(frag[c][f] >> 16);
      }
  }
}

} // namespace

// ---- host-side launchers used by the C ABI ----------------------------------------------------------------
int LaunchPairProjection(const Matrix *matrices, int layer, int part, const int *ids, const float *input, float *output,
                         float *other, int pairs, int *bad, cudaStream_t stream, int rate, int hidden, int inter,
                         bool gate_and_up) {
  if (!matrices || !ids || !input || !output || !bad || pairs < 1 || layer < 0 || part < 0 || part > 2 ||
      (part == 0 && gate_and_up && !other) || hidden < 128 || inter < 128 || (hidden % 128) || (inter % 128))
    return PADRA_INVALID_ARGUMENT;
  ProjectionArgs a{};
  a.matrices = matrices, a.layer = layer, a.requested_part = part, a.ids = ids, a.pairs = pairs, a.input = input;
  a.output = part == 1 ? nullptr : output, a.other = part == 1 ? output : other, a.bad = bad;
  a.hidden = hidden, a.inter = inter, a.row_capacity = 1;
  const int rows = part == 2 ? hidden : inter;
  return DispatchProjection<kPairRows>(a, rate, dim3(rows / 128, pairs, part == 0 && gate_and_up ? 2 : 1), stream);
}

int LaunchUnionProjection(const Matrix *matrices, int layer, int part, const unsigned *masks, const int *slots,
                          int slot_stride, int rows, const float *input, float *output, float *up, int *bad,
                          cudaStream_t stream, const int *active, const int *active_count, int rate, int hidden,
                          int inter) {
  if (!matrices || !masks || !slots || !input || !output || !bad || rows < 1 || rows > kMaxDecodeRows || layer < 0 ||
      part < 0 || part > 2 || (part == 0 && !up) || slot_stride < rows || hidden < 128 || inter < 128 ||
      (hidden % 128) || (inter % 128) || (active != nullptr) != (active_count != nullptr))
    return PADRA_INVALID_ARGUMENT;
  ProjectionArgs a{};
  a.matrices = matrices, a.layer = layer, a.requested_part = part, a.masks = masks, a.slots = slots;
  a.slot_stride = slot_stride, a.active = active, a.active_count = active_count, a.rows = rows, a.input = input;
  a.output = part == 1 ? nullptr : output, a.other = part == 1 ? output : up, a.bad = bad;
  a.hidden = hidden, a.inter = inter, a.row_capacity = rows > 8 ? 16 : 8;
  const int out_rows = part == 2 ? hidden : inter;
  const int units = active ? (rows * kTopK < kExperts ? rows * kTopK : kExperts) : kExperts;
  return DispatchProjection<kUnionRows>(a, rate, dim3(out_rows / 128, units, part == 0 ? 2 : 1), stream);
}

// Prefill projection over the reference's 32-pair tiles (small-tile tensor-core path; the tcgen05 grouped
// GEMM in prefill.cu takes over for large token counts).
int LaunchTileProjection(const Matrix *matrices, int layer, int part, const int *groups, const padra_tile *tiles,
                         const int *tile_count, const float *input, unsigned short *output,
                         const unsigned short *gate, const unsigned short *up, const unsigned short *table, int tokens,
                         int *bad, cudaStream_t stream, int rate, int hidden, int inter) {
  ProjectionArgs a{};
  a.matrices = matrices, a.layer = layer, a.requested_part = part, a.input = input, a.bad = bad;
  a.hidden = hidden, a.inter = inter, a.row_capacity = 32, a.groups = groups, a.tiles = tiles, a.tile_count = tile_count;
  a.tokens = tokens, a.gate_bits = gate, a.up_bits = up, a.table = table, a.output_bits = output;
  const int rows = part == 2 ? hidden : inter;
  const int capacity = (tokens * kTopK + 31) / 32 + kExperts; // src/runtime/exl3_masked_schedule.h:15-17
  return DispatchProjection<kTileRows>(a, rate, dim3(rows / 128, capacity, 1), stream);
}

int LaunchBuildUnion(const int *ids, unsigned *masks, int *slots, int rows, int slot_stride, int *bad, int *active,
                     int *active_count, cudaStream_t stream) {
  if (!ids || !masks || !slots || !bad || rows < 1 || rows > kMaxDecodeRows || slot_stride < rows ||
      (active != nullptr) != (active_count != nullptr))
    return PADRA_INVALID_ARGUMENT;
  BuildUnionKernel<<<1, kExperts, 0, stream>>>(ids, masks, slots, rows, slot_stride, bad, active, active_count);
  return CudaStatus(cudaGetLastError());
}

int LaunchSiluBuild(unsigned short *table, cudaStream_t stream) {
  if (!table)
    return PADRA_INVALID_ARGUMENT;
  SiluBuildKernel<<<256, 256, 0, stream>>>(table);
  return CudaStatus(cudaGetLastError());
}

int LaunchSiluActivate(float *gate, const float *up, const unsigned short *table, int count, int *bad,
                       cudaStream_t stream) {
  if (!gate || !up || !table || !bad || count < 1)
    return PADRA_INVALID_ARGUMENT;
  SiluActivateKernel<<<(count + 255) / 256, 256, 0, stream>>>(gate, up, table, count, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchCombine(float *x, const float *down, const float *weights, int *bad, int rows, int hidden,
                  cudaStream_t stream) {
  if (!x || !down || !weights || !bad || rows < 1 || hidden < 1)
    return PADRA_INVALID_ARGUMENT;
  CombineKernel<float><<<dim3((hidden + 127) / 128, rows), 128, 0, stream>>>(x, down, weights, rows, hidden, bad, true);
  return CudaStatus(cudaGetLastError());
}

// The same with four columns per thread (8-byte loads of BF16 rows, 16-byte accesses of x) for aligned buffers.
__global__ void __launch_bounds__(128) CombinePackedWideKernel(float *x, const unsigned short *down, const float *weights, int rows, int hidden,
                                                               int *bad, bool residual) {
  const int row = blockIdx.y, col = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (row >= rows || col >= hidden)
    return;
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < kTopK; ++s) {
    const uint2 bits = *reinterpret_cast<const uint2 *>(down + (static_cast<size_t>(row) * kTopK + s) * hidden + col);
    const float w = weights[row * kTopK + s];
    const float d[4] = {FromBF16Bits(bits.x & 0xffffu), FromBF16Bits(bits.x >> 16), FromBF16Bits(bits.y & 0xffffu),
                        FromBF16Bits(bits.y >> 16)};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      sum[j] = RoundBF16(__fadd_rn(sum[j], RoundBF16(__fmul_rn(d[j], w))));
  }
  float4 *target = reinterpret_cast<float4 *>(x + static_cast<size_t>(row) * hidden + col);
  const float4 old = *target;
  float4 v;
  v.x = residual ? RoundBF16(__fadd_rn(old.x, sum[0])) : sum[0];
  v.y = residual ? RoundBF16(__fadd_rn(old.y, sum[1])) : sum[1];
  v.z = residual ? RoundBF16(__fadd_rn(old.z, sum[2])) : sum[2];
  v.w = residual ? RoundBF16(__fadd_rn(old.w, sum[3])) : sum[3];
  if (!isfinite(v.x) || !isfinite(v.y) || !isfinite(v.z) || !isfinite(v.w))
    Raise(bad);
  *target = v;
}

int LaunchCombinePacked(float *x, const unsigned short *down, const float *weights, int tokens, int *bad, int residual,
                        int hidden, cudaStream_t stream) {
  if (!x || !down || !weights || !bad || tokens < 1 || hidden < 1)
    return PADRA_INVALID_ARGUMENT;
  if (hidden % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(down) % 8 == 0)
    CombinePackedWideKernel<<<dim3((hidden / 4 + 127) / 128, tokens), 128, 0, stream>>>(x, down, weights, tokens, hidden, bad,
                                                                                       residual != 0);
  else
    CombineKernel<unsigned short>
        <<<dim3((hidden + 127) / 128, tokens), 128, 0, stream>>>(x, down, weights, tokens, hidden, bad, residual != 0);
  return CudaStatus(cudaGetLastError());
}

int LaunchDecodeWeights(const Matrix *matrix, unsigned short *out, int rows, int cols, int rate, int *bad,
                        cudaStream_t stream) {
  if (!matrix || !out || !bad || rows < 16 || cols < 64 || (rows % 16) || (cols % 64))
    return PADRA_INVALID_ARGUMENT;
  const int items = (cols / 64) * (rows / 16);
  const int blocks = (items + 7) / 8 < 1184 ? (items + 7) / 8 : 1184;
  switch (rate) {
  case 3:
    DecodeWeightsKernel<3><<<blocks, 256, 0, stream>>>(matrix, out, rows, cols, bad);
    break;
  case 4:
    DecodeWeightsKernel<4><<<blocks, 256, 0, stream>>>(matrix, out, rows, cols, bad);
    break;
  case 6:
    DecodeWeightsKernel<6><<<blocks, 256, 0, stream>>>(matrix, out, rows, cols, bad);
    break;
  default:
    return PADRA_UNSUPPORTED;
  }
  return CudaStatus(cudaGetLastError());
}

} // namespace padra
