// EXL3 trellis codec for a "row-pair" lane ownership.
//
// A 16x16 weight tile is a cyclic MSB-first bit stream of 256*Rate bits held in 8*Rate little-endian u32
// words.  The weight for (input i, output o) sits at stream position
//     p = ((o&7)*4 + ((i&7)>>1))*8 + [o>=8]*4 + [i>=8]*2 + (i&1)
// and its 16-bit state is the window that ends at bit Rate*(p+1) (reference: src/cuda/expert_exl3.cuh:4-22).
// So the 32 positions with (o&7) == g are the contiguous bits [32*Rate*g, 32*Rate*(g+1)): exactly Rate
// words at word offset Rate*g.  A lane that loads those Rate words (16 bytes at K4) owns the two output
// rows g and g+8 for all sixteen inputs of the tile, and needs only the word just before them (the last
// word of row-pair g-1, cyclically) to complete its first windows.
//
// Position inside the lane's 32: q = 8*c + j with c = (i&7)>>1 and j = [o>=8]*4 + [i>=8]*2 + (i&1).
// Decoded values come out as four groups c = 0..3 of four FP16 pairs in mma.m16n8k16 A-fragment order:
//     a[c][0] = (row g  ; inputs 2c, 2c+1)     a[c][1] = (row g+8; inputs 2c, 2c+1)
//     a[c][2] = (row g  ; inputs 2c+8, 2c+9)   a[c][3] = (row g+8; inputs 2c+8, 2c+9)
// with the even input in the low half.  The same a[c][r] viewed per r over c = 0..3 is one full 16-byte row
// of an 8x8 FP16 core matrix, which is what the tensor-memory (tcgen05) path stores.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

#if defined(__CUDACC__)
#define PADRA_HD __host__ __device__ __forceinline__
#else
#define PADRA_HD inline
#endif

namespace padra {
namespace codec {

// Bytes one lane owns per tile (32 positions * Rate bits).
template <int Rate> struct Lane {
  static_assert(Rate == 3 || Rate == 4 || Rate == 6, "EXL3 rates on this path are K3, K4 and K6");
  static constexpr int kWords = Rate;
  static constexpr int kBytes = 4 * Rate;
  static constexpr int kTileBytes = 32 * Rate;
};

PADRA_HD uint32_t FunnelRight(uint32_t lo, uint32_t hi, int shift) {
#if defined(__CUDA_ARCH__)
  return __funnelshift_r(lo, hi, shift);
#else
  return static_cast<uint32_t>(((static_cast<uint64_t>(hi) << 32) | lo) >> (shift & 31));
#endif
}

// 0x6400 + (sum of the four bytes of state*0x83DCD12D): the FP16 bit pattern of 1024 + s.  The byte sum is at
// most 1020, so it never carries into the exponent.
PADRA_HD uint32_t HashedHalfBits(uint32_t state) {
  const uint32_t h = state * 0x83DCD12Du;
#if defined(__CUDA_ARCH__)
  return __dp4a(h, 0x01010101u, 0x6400u);
#else
  return 0x6400u + (h & 255u) + ((h >> 8) & 255u) + ((h >> 16) & 255u) + (h >> 24);
#endif
}

// (x >> 8) & 0xffff in one byte-permute (the second source is zero).
PADRA_HD uint32_t MiddleHalf(uint32_t x) {
#if defined(__CUDA_ARCH__)
  return __byte_perm(x, 0u, 0x4421);
#else
  return (x >> 8) & 0xffffu;
#endif
}

// The eight states of one K4 word, MSB-first: state j ends at bit 4*(j+1) of the 64-bit value previous:word, i.e.
// s_j = ((previous:word) >> (28 - 4j)) & 0xffff.  Three funnel shifts bring every state to bit 0, 8 or 16 of some
// register, where one instruction (mask, byte-permute with zero, or plain shift) isolates it: 11 operations for
// 8 states instead of 15 with a shift and a mask each.
PADRA_HD void StatesK4(uint32_t word, uint32_t previous, uint32_t (&s)[8]) {
  const uint32_t by4 = FunnelRight(word, previous, 4), by16 = FunnelRight(word, previous, 16),
                 by20 = FunnelRight(word, previous, 20);
  s[7] = word & 0xffffu;
  s[5] = MiddleHalf(word);
  s[3] = word >> 16;
  s[1] = MiddleHalf(by16);
  s[6] = by4 & 0xffffu;
  s[4] = MiddleHalf(by4);
  s[2] = by4 >> 16;
  s[0] = MiddleHalf(by20);
}

#if defined(__CUDACC__)
// Two states -> two FP16 weights: one packed fused multiply-add (1024+s)*0x1eee + 0xc931, rounded once.  The two
// 16-bit patterns are packed with a multiply-add (odd*65536 + even) so that the packing runs on the FMA pipe; the
// integer ALU pipe is the scarcer one in these kernels.
__device__ __forceinline__ uint32_t PairToHalf2(uint32_t even_state, uint32_t odd_state) {
  uint32_t packed;
  asm("mad.lo.u32 %0, %1, 65536, %2;" : "=r"(packed) : "r"(HashedHalfBits(odd_state)), "r"(HashedHalfBits(even_state)));
  const __half2 scale = __halves2half2(__ushort_as_half(0x1eee), __ushort_as_half(0x1eee));
  const __half2 shift = __halves2half2(__ushort_as_half(0xc931), __ushort_as_half(0xc931));
  const __half2 w = __hfma2(*reinterpret_cast<const __half2 *>(&packed), scale, shift);
  return *reinterpret_cast<const uint32_t *>(&w);
}
#endif

// The 32-bit window ending at the end bit of local position q (odd q): low 16 bits are the state of q, bits
// [Rate, Rate+16) the state of q-1.  `words` are the lane's own words, `previous` the word before them.
template <int Rate, int Q>
PADRA_HD uint32_t PairWindow(const uint32_t (&words)[Rate], uint32_t previous) {
  constexpr int end = Rate * (Q + 1);
  constexpr int last = (end - 1) / 32;
  constexpr int shift = (last + 1) * 32 - end;
  const uint32_t lo = words[last];
  const uint32_t hi = last > 0 ? words[last > 0 ? last - 1 : 0] : previous;
  return shift == 0 ? lo : FunnelRight(lo, hi, shift);
}

// State (16 bits) of local position q, for host-side checks and the scalar paths.
template <int Rate> PADRA_HD uint32_t StateAt(const uint32_t (&words)[Rate], uint32_t previous, int q) {
  const int end = Rate * (q + 1);
  const int last = (end - 1) / 32;
  const int shift = (last + 1) * 32 - end;
  const uint32_t lo = words[last];
  const uint32_t hi = last > 0 ? words[last - 1] : previous;
  const uint64_t both = (static_cast<uint64_t>(hi) << 32) | lo;
  return static_cast<uint32_t>(both >> shift) & 0xffffu;
}

// Fragment register index for pair m (positions 8c+2m, 8c+2m+1): m bit0 = [i>=8], bit1 = [o>=8].
PADRA_HD constexpr int FragmentOfPair(int m) {
  return (m >> 1) + 2 * (m & 1);
}

#if defined(__CUDACC__)
template <int Rate, int C, int M>
__device__ __forceinline__ uint32_t DecodePair(const uint32_t (&words)[Rate], uint32_t previous) {
  const uint32_t window = PairWindow<Rate, 8 * C + 2 * M + 1>(words, previous);
  return PairToHalf2((window >> Rate) & 0xffffu, window & 0xffffu);
}
// All 32 weights of the lane.
template <int Rate>
__device__ __forceinline__ void Decode32(const uint32_t (&words)[Rate], uint32_t previous, uint32_t (&a)[4][4]) {
  if constexpr (Rate == 4) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t s[8];
      StatesK4(words[c], c ? words[c > 0 ? c - 1 : 0] : previous, s);
#pragma unroll
      for (int m = 0; m < 4; ++m)
        a[c][FragmentOfPair(m)] = PairToHalf2(s[2 * m], s[2 * m + 1]);
    }
    return;
  }
#define PADRA_DECODE_GROUP(C)                                            \
  a[C][FragmentOfPair(0)] = DecodePair<Rate, C, 0>(words, previous);     \
  a[C][FragmentOfPair(1)] = DecodePair<Rate, C, 1>(words, previous);     \
  a[C][FragmentOfPair(2)] = DecodePair<Rate, C, 2>(words, previous);     \
  a[C][FragmentOfPair(3)] = DecodePair<Rate, C, 3>(words, previous);
  PADRA_DECODE_GROUP(0)
  PADRA_DECODE_GROUP(1)
  PADRA_DECODE_GROUP(2)
  PADRA_DECODE_GROUP(3)
#undef PADRA_DECODE_GROUP
}

// ---- byte sums on the tensor cores ----------------------------------------------------------------------------
// The byte sum of a hash is a dot product of its four bytes with ones, and one integer mma.m16n8k32 (u8 x u8 -> s32)
// does 128 of them: its A operand is 16 rows x 8 hashes (a lane supplies four hashes as its four A registers), its B
// operand the constant selector B[k][n] = (k/4 == n), its C operand the constant 0x6400, so D[r][n] = 0x6400 + byte sum
// of hash (r, n): the FP16 bit pattern of 1024 + s.  One tensor instruction replaces four dp4a, and the integer ALU pipe
// (the busiest unit of these kernels) is left with the state extraction alone.
//
// The instruction also moves values between the four lanes of a quad (lanes 4g..4g+3): lane t supplies the hashes of
// grid columns n = t and t + 4 for rows g and g + 8 and receives the sums of columns 2t and 2t + 1 -- adjacent
// columns, which pack into one half2.  Two such instructions give the four A registers of one FP16 mma.m16n8k16 whose
// logical input k (0..15) is the weight of tile k % 4 (the quad's lane k % 4 owns that tile) at input
// TensorInput(c, k / 4).  Activations are stored in the matching order (TensorPermutedInput).
PADRA_HD constexpr int TensorInput(int c, int quarter) {
  return 2 * c + (quarter & 1) + 8 * (quarter >> 1);
}
// Place, inside the 64 halves of one round (four K16 steps, `tile` = step within the round), of input i of that step:
// lane t' of a quad reads 16 consecutive halves, four per mma (group c), {b0.lo, b0.hi, b1.lo, b1.hi}.
PADRA_HD constexpr int TensorPermutedInput(int tile, int i) {
  const int c = (i & 7) >> 1, quarter = 2 * (i >> 3) + (i & 1);
  const int k = 4 * quarter + tile;
  return ((k & 7) >> 1) * 16 + c * 4 + (k >> 3) * 2 + (k & 1);
}

struct ByteSumSelector {
  uint32_t b0, b1;
};
// B fragment of the selector for this lane: rows k = 4t..4t+3 (b0) and 16+4t.. (b1) of column n = g.
__device__ __forceinline__ ByteSumSelector MakeByteSumSelector(int lane) {
  const int g = lane >> 2, t = lane & 3;
  ByteSumSelector s;
  s.b0 = g == t ? 0x01010101u : 0u;
  s.b1 = g == t + 4 ? 0x01010101u : 0u;
  return s;
}
// d[0], d[1] = 0x6400 + byte sums of (row g; columns 2t, 2t+1), d[2], d[3] the same for row g + 8.
__device__ __forceinline__ void ByteSums(uint32_t h_row_lo, uint32_t h_row8_lo, uint32_t h_row_hi, uint32_t h_row8_hi,
                                         const ByteSumSelector &sel, uint32_t (&d)[4]) {
  const uint32_t bias = 0x6400u;
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(h_row_lo), "r"(h_row8_lo), "r"(h_row_hi), "r"(h_row8_hi), "r"(sel.b0), "r"(sel.b1), "r"(bias));
}
// Two FP16 bit patterns 1024 + s (even in the low half) -> two weights.
__device__ __forceinline__ uint32_t BiasedPairToHalf2(uint32_t even_bits, uint32_t odd_bits) {
  uint32_t packed;
  asm("mad.lo.u32 %0, %1, 65536, %2;" : "=r"(packed) : "r"(odd_bits), "r"(even_bits));
  const __half2 scale = __halves2half2(__ushort_as_half(0x1eee), __ushort_as_half(0x1eee));
  const __half2 shift = __halves2half2(__ushort_as_half(0xc931), __ushort_as_half(0xc931));
  const __half2 w = __hfma2(*reinterpret_cast<const __half2 *>(&packed), scale, shift);
  return *reinterpret_cast<const uint32_t *>(&w);
}
// The eight states of group C (positions 8C .. 8C+7 of the lane's 32): s[j], j = [o>=8]*4 + [i>=8]*2 + (i&1).
template <int Rate, int C>
__device__ __forceinline__ void GroupStates(const uint32_t (&words)[Rate], uint32_t previous, uint32_t (&s)[8]) {
  if constexpr (Rate == 4) {
    StatesK4(words[C], C ? words[C > 0 ? C - 1 : 0] : previous, s);
  } else {
    const uint32_t w0 = PairWindow<Rate, 8 * C + 1>(words, previous), w1 = PairWindow<Rate, 8 * C + 3>(words, previous);
    const uint32_t w2 = PairWindow<Rate, 8 * C + 5>(words, previous), w3 = PairWindow<Rate, 8 * C + 7>(words, previous);
    s[0] = (w0 >> Rate) & 0xffffu, s[1] = w0 & 0xffffu;
    s[2] = (w1 >> Rate) & 0xffffu, s[3] = w1 & 0xffffu;
    s[4] = (w2 >> Rate) & 0xffffu, s[5] = w2 & 0xffffu;
    s[6] = (w3 >> Rate) & 0xffffu, s[7] = w3 & 0xffffu;
  }
}
template <int Rate, int C>
__device__ __forceinline__ void DecodeGroupTensor(const uint32_t (&words)[Rate], uint32_t previous, const ByteSumSelector &sel,
                                                  uint32_t (&a)[4]) {
  uint32_t s[8], lo[4], hi[4];
  GroupStates<Rate, C>(words, previous, s);
#pragma unroll
  for (int j = 0; j < 8; ++j)
    s[j] *= 0x83DCD12Du;
  ByteSums(s[0], s[4], s[1], s[5], sel, lo); // inputs 2C and 2C+1 of both rows -> logical k 0..7
  ByteSums(s[2], s[6], s[3], s[7], sel, hi); // inputs 2C+8 and 2C+9            -> logical k 8..15
  a[0] = BiasedPairToHalf2(lo[0], lo[1]);
  a[1] = BiasedPairToHalf2(lo[2], lo[3]);
  a[2] = BiasedPairToHalf2(hi[0], hi[1]);
  a[3] = BiasedPairToHalf2(hi[2], hi[3]);
}
// All 32 weights of the lane, byte sums on the tensor cores.  a[c] are the A registers of mma number c of the round:
// a[c][0] = (row g; logical k 2t, 2t+1), [1] = (row g+8; same k), [2] = (row g; k 2t+8, 2t+9), [3] = (row g+8; ...),
// logical k = weight of tile k % 4 at input TensorInput(c, k / 4).  All 32 lanes must call this together.
template <int Rate>
__device__ __forceinline__ void Decode32Tensor(const uint32_t (&words)[Rate], uint32_t previous, const ByteSumSelector &sel,
                                               uint32_t (&a)[4][4]) {
  DecodeGroupTensor<Rate, 0>(words, previous, sel, a[0]);
  DecodeGroupTensor<Rate, 1>(words, previous, sel, a[1]);
  DecodeGroupTensor<Rate, 2>(words, previous, sel, a[2]);
  DecodeGroupTensor<Rate, 3>(words, previous, sel, a[3]);
}

// The lane's Rate words of one tile.  `lane_bytes` points at tile + g*4*Rate.  Weights are read exactly once
// per pass, so the loads go through the read-only path without claiming L1 lines.
template <int Rate> __device__ __forceinline__ void LoadWords(const unsigned char *lane_bytes, uint32_t (&w)[Rate]) {
  if constexpr (Rate == 4) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(lane_bytes));
    w[0] = v.x;
    w[1] = v.y;
    w[2] = v.z;
    w[3] = v.w;
  } else if constexpr (Rate == 6) {
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      uint2 v;
      asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(lane_bytes + 8 * i));
      w[2 * i] = v.x;
      w[2 * i + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 3; ++i)
      asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(w[i]) : "l"(lane_bytes + 4 * i));
  }
}
#endif

// Place of input i (0..15) of a K16 step inside the permuted activation row the tensor-core B fragments are
// read from: group c = (i&7)>>1 occupies four consecutive halves {2c, 2c+1, 2c+8, 2c+9}.
PADRA_HD constexpr int PermutedInput(int i) {
  return 4 * ((i & 7) >> 1) + 2 * (i >> 3) + (i & 1);
}

} // namespace codec
} // namespace padra
