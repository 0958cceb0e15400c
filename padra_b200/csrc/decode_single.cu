// The expert layer for ONE token (the decode step proper), two launches built around one observation: at this size the
// step is a chain of dependent memory round trips, not a stream.  Eight experts are 25 MB of packed words, a few
// microseconds of decoding spread over 148 SMs; every dependent load on the way (ids -> descriptor -> words -> ...)
// costs most of a microsecond.  So both kernels do whatever does not depend on their predecessor BEFORE they wait for
// it, ask for everything they need at one point in one go, and a CTA of the second kernel starts as soon as the sixteen
// CTAs of the first one that it depends on have delivered, not when the whole first kernel has drained.
//
//   SingleGateUpKernel   grid (2 matrices x K-slices, intermediate/128, 8 slots): the CTAs of one (slot, 128-output
//                        block) are neighbours in launch order, so blocks complete in order.  Before the wait: the
//                        layer's 64 descriptors of its matrix, into shared memory (model state, not the predecessor's
//                        work).  After it: expert id, error flag and the token's activation slice in one round trip,
//                        then the slice's packed words and suh in a second one; input transform, decode, mma, and the
//                        slice's FP32 sums go to the workspace.  Slice 0 also copies its svh block beside them.  Every
//                        CTA then counts itself into the block's `ready` counter (release), whatever happened to it.
//   SingleDownKernel     grid (K-slices, hidden/128, 8 slots).  It does not wait for the first kernel as a whole.  At
//                        once: id, descriptors, ALL of its packed words (a K-slice of the down matrix is four rounds)
//                        and its sidecars.  Then it polls (bounded) the `ready` counters of the 128-input blocks of ITS
//                        slice and fetches their gate/up sums in one round trip; the warp that owns a block sums the
//                        slices in ascending order, applies output Hadamard and svh, SwiGLU, suh and the input Hadamard
//                        -- the gate/up epilogue, recomputed by each of the CTAs that need the block (a few hundred
//                        instructions) instead of waiting for one CTA to publish it.  SwiGLU evaluates the function the
//                        table tabulates (src/cuda/exl3_silu_lut.cuh:5-8) directly: the same bits, one dependent load
//                        less.  Then decode, mma, slice sums to the workspace, and the CTA that delivers the last of
//                        the token's 8 x slices sums of a 128-output block (a ticket) does output Hadamard, svh, BF16
//                        and the reference's combine; the CTA that finishes the last block clears the counters.
//
// Why polling is safe here: the second kernel is launched programmatically, so none of its CTAs exists before every
// CTA of the first kernel is resident and past its own wait; first-kernel CTAs never wait for anything, so they always
// deliver.  Every poll is bounded in time all the same; on expiry the CTA raises the error flag, skips its work and still
// takes its tickets, so the counters come out right.
//
// Arithmetic and summation orders are those of decode_layer.cu (reference: src/cuda/expert_exl3_decode_dual.cuh:65-130,
// src/cuda/exl3_silu_lut.cuh:15-31, src/cuda/inference.cu:580-594); results are bit-identical run to run.
#include "decode_common.cuh"

namespace padra {
namespace {
using namespace decode;

struct SingleArgs {
  const Matrix *matrices;
  int layer;
  const int *ids;          // [8]
  const float *routing;    // [8]
  const float *normalized; // [hidden]
  float *x;                // [hidden], residual in/out
  int hidden, inter, slices_gateup, slices_down;
  const unsigned short *table;
  float *gateup;     // [slot][2][slices_gateup][inter]
  __half *sidecars;  // [slot][2][inter]: svh of gate and up
  float *down;       // [slot][slices_down][hidden]
  __half *svh_rows;  // [slot][hidden]: svh of down
  unsigned *tickets; // [kMaxBlocks] per output block of down, zero between calls
  unsigned *ready;   // [slot][kMaxBlocks] arrivals per (slot, 128-output block) of gate+up, then one word: blocks combined
  int *bad;
  unsigned long long *trace; // scratch builds only
};

// The 64 descriptors of one matrix kind of the layer, into shared memory (56 bytes each, 8-byte pieces).
__device__ __forceinline__ void LoadDescriptors(const Matrix *matrices, int layer, int part, Matrix *s_m) {
  const int tid = threadIdx.x;
  if (tid < kExperts * 7) { // seven 8-byte pieces per descriptor
    const int e = tid / 7, piece = tid % 7;
    const auto *src = reinterpret_cast<const unsigned long long *>(matrices + (static_cast<size_t>(layer) * kExperts + e) * 3 + part);
    reinterpret_cast<unsigned long long *>(s_m + e)[piece] = __ldg(src + piece);
  }
}
static_assert(kExperts * 7 <= 2 * kThreads, "descriptor copy is written for two passes at most");

template <int Rate> struct Stream {
  using L = codec::Lane<Rate>;
  const unsigned char *lane_base;
  size_t round_bytes;
  __device__ __forceinline__ void Set(const Matrix &m, int k_begin, int column, int lane) {
    const int g = lane >> 2, t = lane & 3, tiles_per_kstep = m.rows / 16;
    lane_base = m.data + (static_cast<size_t>(k_begin / 16 + t) * tiles_per_kstep + column) * L::kTileBytes + g * L::kBytes;
    round_bytes = static_cast<size_t>(4) * tiles_per_kstep * L::kTileBytes;
  }
  __device__ __forceinline__ void Load(int round, uint32_t (&w)[Rate]) const {
    codec::LoadWords<Rate>(lane_base + static_cast<size_t>(round) * round_bytes, w);
  }
};

// Decode and multiply `rounds` rounds (even, >= 2) of one warp's tile column against the activation row in shared
// memory; the first four rounds are already in `fetched`.
template <int Rate>
__device__ __forceinline__ void StreamRounds(const Stream<Rate> &stream, uint32_t (&fetched)[4][Rate], int rounds, const __half *xrow,
                                             int lane, float (&acc)[4]) {
  auto multiply = [&](const uint32_t (&words)[Rate], int round) {
    const uint32_t previous = __shfl_sync(0xffffffffu, words[Rate - 1], (lane + 28) & 31);
    uint32_t frag[4][4];
    codec::Decode32<Rate>(words, previous, frag);
    const uint4 lo = *reinterpret_cast<const uint4 *>(xrow + round * 64);
    const uint4 hi = *reinterpret_cast<const uint4 *>(xrow + round * 64 + 8);
    MmaF16(frag[0], lo.x, lo.y, acc);
    MmaF16(frag[1], lo.z, lo.w, acc);
    MmaF16(frag[2], hi.x, hi.y, acc);
    MmaF16(frag[3], hi.z, hi.w, acc);
  };
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
          stream.Load(r + 4, fetched[2 * half]);
          stream.Load(r + 5, fetched[2 * half + 1]);
        }
        multiply(now_even, r);
        multiply(now_odd, r + 1);
      }
    }
  }
}

__device__ __forceinline__ bool DescriptorFits(const Matrix &m, int rate, int rows, int cols) {
  return m.format == FormatOfRate(rate) && m.rows == rows && m.cols == cols && m.data && m.suh && m.svh;
}

template <int Rate> __global__ void __launch_bounds__(kThreads, 4) SingleGateUpKernel(SingleArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ Matrix s_m[kExperts];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nb = blockIdx.y, slot = blockIdx.z, part = static_cast<int>(blockIdx.x) / a.slices_gateup,
            slice = static_cast<int>(blockIdx.x) % a.slices_gateup;
  const int span = a.hidden / a.slices_gateup, k_begin = slice * span, rounds = span / 64, blocks = span / 128;
  PADRA_TRACE(a.trace, 0);
  PADRA_TRACE_SM(a.trace);
  // model state, not the predecessor's work: fetched while the predecessor still runs
  LoadDescriptors(a.matrices, a.layer, part, s_m);
  if (tid + kThreads < kExperts * 7) {
    const int e = (tid + kThreads) / 7, piece = (tid + kThreads) % 7;
    const auto *src = reinterpret_cast<const unsigned long long *>(a.matrices + (static_cast<size_t>(a.layer) * kExperts + e) * 3 + part);
    reinterpret_cast<unsigned long long *>(s_m + e)[piece] = __ldg(src + piece);
  }
  WaitForPredecessor(); // ids, activations and the error flag are the work of whatever ran before this call
  LetSuccessorLaunch(); // only now: the down kernel reads the ids before its own wait
  PADRA_TRACE(a.trace, 1);
  // one round trip: expert id, error flag, and this lane's four activations
  const int id = __ldcg(a.ids + slot);
  int flagged = LoadFlag(a.bad);
  float4 xv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (warp < blocks)
    xv = __ldcg(reinterpret_cast<const float4 *>(a.normalized + k_begin + warp * 128 + lane * 4));
  __syncthreads(); // descriptors are in shared memory
  const bool valid = id >= 0 && id < kExperts;
  const Matrix m = s_m[valid ? id : 0];
  bool work = valid && DescriptorFits(m, Rate, a.inter, a.hidden); // the same verdict in every thread of the CTA
  if (!work && !tid)
    Raise(a.bad);
  PADRA_TRACE(a.trace, 2);
  // second round trip: the slice's first four rounds of packed words, and suh
  Stream<Rate> stream;
  uint32_t fetched[4][Rate] = {};
  uint2 suh_bits = make_uint2(0u, 0u), svh_bits = make_uint2(0u, 0u);
  if (work) {
    stream.Set(m, k_begin, nb * 8 + warp, lane);
#pragma unroll
    for (int d = 0; d < 4; ++d)
      stream.Load(d < rounds ? d : rounds - 2 + (d & 1), fetched[d]);
    if (warp < blocks)
      suh_bits = __ldg(reinterpret_cast<const uint2 *>(m.suh + k_begin + warp * 128 + lane * 4));
    if (slice == 0 && warp == 7)
      svh_bits = __ldg(reinterpret_cast<const uint2 *>(m.svh + nb * 128 + lane * 4));
  }
  PADRA_TRACE(a.trace, 3);
  // input transform of the slice: warp w owns 128-input block w (more blocks than warps: in turns)
  __half *xs = reinterpret_cast<__half *>(smem);
  if (work)
    for (int block = warp; block < blocks; block += 8) {
      if (block >= 8) { // beyond the registers loaded above
        xv = __ldcg(reinterpret_cast<const float4 *>(a.normalized + k_begin + block * 128 + lane * 4));
        suh_bits = __ldg(reinterpret_cast<const uint2 *>(m.suh + k_begin + block * 128 + lane * 4));
      }
      float sg[4];
      Unpack4(suh_bits, sg);
      float v[4] = {__fmul_rn(xv.x, sg[0]), __fmul_rn(xv.y, sg[1]), __fmul_rn(xv.z, sg[2]), __fmul_rn(xv.w, sg[3])};
      WarpHadamard128(v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float r = RoundBF16(v[j]);
        const __half hv = __float2half_rn(r);
        if (!isfinite(r) || (__half_as_ushort(hv) & 0x7c00) == 0x7c00) {
          Raise(a.bad);
          flagged = 1;
        }
        xs[PermutedPlace(block * 128 + lane * 4 + j)] = hv;
      }
    }
  if (__syncthreads_or(flagged))
    work = false; // refused or failed: nothing is stored, the down kernel sees the flag and leaves x alone
  PADRA_TRACE(a.trace, 4);
  if (work) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    StreamRounds<Rate>(stream, fetched, rounds, xs + (lane & 3) * 16, lane, acc);
    PADRA_TRACE(a.trace, 5);
    // every column of the accumulator holds the token's sums: lanes with t == 0 store rows g and g + 8
    const int g = lane >> 2;
    float *p = a.gateup + ((static_cast<size_t>(slot) * 2 + part) * a.slices_gateup + slice) * a.inter + nb * 128 + warp * 16;
    if ((lane & 3) == 0) {
      p[g] = acc[0];
      p[g + 8] = acc[2];
    }
    if (slice == 0 && warp == 7)
      *reinterpret_cast<uint2 *>(a.sidecars + (static_cast<size_t>(slot) * 2 + part) * a.inter + nb * 128 + lane * 4) = svh_bits;
  }
  // delivered (or given up): the down kernel's CTAs that need this block count the arrivals.  Every warp counts itself
  // as soon as its own stores are out (a release at device scope behind the warp's barrier), without waiting for the
  // CTA's other warps.
  __syncwarp();
  if (lane == 0 && a.ready)
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.ready + slot * kMaxBlocks + nb) : "memory");
  PADRA_TRACE(a.trace, 6);
}

// The function the SwiGLU table tabulates, evaluated directly (src/cuda/exl3_silu_lut.cuh:5-8): the same bits.
__device__ __forceinline__ float SiluRounded(float g) {
  const float denominator = __fadd_rn(1.f, __double2float_rn(exp(static_cast<double>(-g))));
  return RoundBF16(__fdiv_rn(g, denominator));
}

constexpr unsigned long long kReadyWaitNs = 200ull * 1000 * 1000; // a producer that has not delivered by then never will

// Waits (bounded) until `target` CTAs have counted themselves into *counter; false on expiry.
__device__ __forceinline__ bool WaitForArrivals(const unsigned *counter, unsigned target) {
  unsigned long long started = 0;
  for (unsigned spins = 0;; ++spins) {
    unsigned seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    if (seen >= target)
      return true;
    if ((spins & 31u) == 31u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (!started)
        started = now;
      else if (now - started > kReadyWaitNs)
        return false;
    }
    __nanosleep(64);
  }
}

template <int Rate> __global__ void __launch_bounds__(kThreads, 4) SingleDownKernel(SingleArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ Matrix s_m[kExperts];
  __shared__ __align__(16) float s_down[kTopK][128];
  __shared__ int s_last, s_final, s_expired;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nb = blockIdx.y, slot = blockIdx.z, slice = blockIdx.x;
  const int span = a.inter / a.slices_down, k_begin = slice * span, rounds = span / 64, blocks = span / 128;
  PADRA_TRACE(a.trace, 0);
  PADRA_TRACE_SM(a.trace);
  LetSuccessorLaunch();
  // ---- everything that does not depend on the gate+up kernel ----
  const int id = __ldg(a.ids + slot); // the caller's input, complete before the gate+up kernel passed its own wait
  LoadDescriptors(a.matrices, a.layer, 2, s_m);
  if (tid + kThreads < kExperts * 7) {
    const int e = (tid + kThreads) / 7, piece = (tid + kThreads) % 7;
    const auto *src = reinterpret_cast<const unsigned long long *>(a.matrices + (static_cast<size_t>(a.layer) * kExperts + e) * 3 + 2);
    reinterpret_cast<unsigned long long *>(s_m + e)[piece] = __ldg(src + piece);
  }
  if (tid == 0)
    s_expired = 0;
  __syncthreads();
  const bool valid = id >= 0 && id < kExperts;
  const Matrix m = s_m[valid ? id : 0];
  bool work = valid && DescriptorFits(m, Rate, a.hidden, a.inter);
  if (!work && !tid)
    Raise(a.bad);
  PADRA_TRACE(a.trace, 1);
  Stream<Rate> stream;
  uint32_t fetched[4][Rate] = {};
  uint2 svh_bits = make_uint2(0u, 0u), suh_bits = make_uint2(0u, 0u);
  // Where a slice has no more elements than the CTA has threads (two blocks at the graded shape) the SwiGLU of the
  // gate/up epilogue is spread over all threads and needs three float rows and the signs in shared memory; longer slices
  // keep everything in the registers of the block's warp and need the transformed row only.  (The dynamic shared memory
  // is kept small on purpose: a down kernel that asks for much more shared memory per SM than the gate+up kernel makes the
  // SM switch its shared-memory configuration between the two, and they then no longer run side by side.)
  const bool spread = span <= kThreads;
  __half *xs = reinterpret_cast<__half *>(smem);
  float *s_gate = reinterpret_cast<float *>(smem + static_cast<size_t>(span) * sizeof(__half)), *s_up = s_gate + span, *s_act = s_up + span;
  unsigned short *s_suh = reinterpret_cast<unsigned short *>(s_act + span);
  if (work) {
    stream.Set(m, k_begin, nb * 8 + warp, lane);
#pragma unroll
    for (int d = 0; d < 4; ++d)
      stream.Load(d < rounds ? d : rounds - 2 + (d & 1), fetched[d]);
    // the down matrix's input signs of the slice, which the SwiGLU below multiplies by: into shared memory where the
    // SwiGLU is spread over the threads, else in the registers of the warp that owns the block
    if (spread) {
      for (int e = tid; e < span; e += kThreads)
        s_suh[e] = __ldg(m.suh + k_begin + e);
    } else if (warp < blocks) {
      suh_bits = __ldg(reinterpret_cast<const uint2 *>(m.suh + k_begin + warp * 128 + lane * 4));
    }
    if (slice == 0 && warp == 7)
      svh_bits = __ldg(reinterpret_cast<const uint2 *>(m.svh + nb * 128 + lane * 4));
  }
  PADRA_TRACE(a.trace, 2);
  // ---- the gate+up sums of this slice's blocks: the warp that sums a block waits for the block's producers (every warp
  // of 2 x slices CTAs counts itself), then reads the error flag, which a producer raises before it counts itself ----
  const unsigned producers = 2u * a.slices_gateup * (kThreads / 32);
  int flagged = 0;
  // ---- the gate/up epilogue of this slice's 128-input blocks ----
  // Sums and Hadamard transforms need a block's 128 values in one warp (one warp per block); the SwiGLU between them
  // is elementwise and its exact exponential is a long dependent chain, so where a slice has no more elements than the CTA
  // has threads (two blocks at the graded shape: six of the eight warps would idle) it is spread over all threads, one
  // element each.  Longer slices keep every warp busy with a block of its own, and there the block's warp does it.
  if (work)
    for (int block = warp; block < blocks; block += 8) {
      int arrived = 1;
      if (lane == 0 && !WaitForArrivals(a.ready + slot * kMaxBlocks + k_begin / 128 + block, producers)) {
        s_expired = 1;
        Raise(a.bad);
        arrived = 0;
      }
      if (!__shfl_sync(0xffffffffu, arrived, 0)) {
        flagged = 1;
        continue;
      }
      if (block == warp)
        PADRA_TRACE(a.trace, 3);
      flagged |= LoadFlag(a.bad);
      const int out = k_begin + block * 128 + lane * 4; // this lane's four intermediate channels
      const float *pg = a.gateup + (static_cast<size_t>(slot) * 2 + 0) * a.slices_gateup * a.inter + out;
      const float *pu = a.gateup + (static_cast<size_t>(slot) * 2 + 1) * a.slices_gateup * a.inter + out;
      float svg[4], svu[4];
      const uint2 sg = __ldcg(reinterpret_cast<const uint2 *>(a.sidecars + (static_cast<size_t>(slot) * 2 + 0) * a.inter + out));
      const uint2 su = __ldcg(reinterpret_cast<const uint2 *>(a.sidecars + (static_cast<size_t>(slot) * 2 + 1) * a.inter + out));
      float gsum[4] = {0.f, 0.f, 0.f, 0.f}, usum[4] = {0.f, 0.f, 0.f, 0.f};
      for (int s0 = 0; s0 < a.slices_gateup; s0 += 4) { // four slices of each matrix in flight, summed in ascending order
        float4 vg[4], vu[4];
#pragma unroll
        for (int s = 0; s < 4; ++s)
          if (s0 + s < a.slices_gateup) {
            vg[s] = __ldcg(reinterpret_cast<const float4 *>(pg + static_cast<size_t>(s0 + s) * a.inter));
            vu[s] = __ldcg(reinterpret_cast<const float4 *>(pu + static_cast<size_t>(s0 + s) * a.inter));
          }
#pragma unroll
        for (int s = 0; s < 4; ++s)
          if (s0 + s < a.slices_gateup) {
            gsum[0] += vg[s].x, gsum[1] += vg[s].y, gsum[2] += vg[s].z, gsum[3] += vg[s].w;
            usum[0] += vu[s].x, usum[1] += vu[s].y, usum[2] += vu[s].z, usum[3] += vu[s].w;
          }
      }
      PADRA_TRACE(a.trace, 9);
      Unpack4(sg, svg);
      Unpack4(su, svu);
      WarpHadamard128(gsum);
      WarpHadamard128(usum);
      float4 gate, up;
      gate.x = RoundBF16(__fmul_rn(gsum[0], svg[0])), gate.y = RoundBF16(__fmul_rn(gsum[1], svg[1]));
      gate.z = RoundBF16(__fmul_rn(gsum[2], svg[2])), gate.w = RoundBF16(__fmul_rn(gsum[3], svg[3]));
      up.x = RoundBF16(__fmul_rn(usum[0], svu[0])), up.y = RoundBF16(__fmul_rn(usum[1], svu[1]));
      up.z = RoundBF16(__fmul_rn(usum[2], svu[2])), up.w = RoundBF16(__fmul_rn(usum[3], svu[3]));
      if (spread) {
        *reinterpret_cast<float4 *>(s_gate + block * 128 + lane * 4) = gate;
        *reinterpret_cast<float4 *>(s_up + block * 128 + lane * 4) = up;
      } else { // long slices: the block's warp applies the SwiGLU and the input transform itself
        if (block >= 8)
          suh_bits = __ldg(reinterpret_cast<const uint2 *>(m.suh + out));
        float shd[4], v[4];
        Unpack4(suh_bits, shd);
        const float gv[4] = {gate.x, gate.y, gate.z, gate.w}, uv[4] = {up.x, up.y, up.z, up.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const bool finite = isfinite(gv[i]) && isfinite(uv[i]);
          const float act = RoundBF16(__fmul_rn(SiluRounded(finite ? gv[i] : 0.f), uv[i]));
          if (!finite || !isfinite(act)) {
            if (!flagged)
              Raise(a.bad);
            flagged = 1;
          }
          v[i] = __fmul_rn(act, shd[i]);
        }
        WarpHadamard128(v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float r = RoundBF16(v[i]);
          const __half h = __float2half_rn(r);
          if (!isfinite(r) || (__half_as_ushort(h) & 0x7c00) == 0x7c00) {
            if (!flagged)
              Raise(a.bad);
            flagged = 1;
          }
          xs[PermutedPlace(block * 128 + lane * 4 + i)] = h;
        }
      }
      PADRA_TRACE(a.trace, 10);
    }
  __syncthreads();
  const bool recompute = work && !s_expired; // uniform over the CTA
  if (recompute && spread)
    for (int e0 = tid; e0 < span; e0 += 4 * kThreads) { // one element per thread at the graded shape
      // up to four elements a thread at a time, so that their exponentials (long dependent chains) overlap
      float gate[4], up[4], act[4];
      bool finite[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = e0 + j * kThreads;
        gate[j] = e < span ? s_gate[e] : 0.f, up[j] = e < span ? s_up[e] : 0.f;
        finite[j] = isfinite(gate[j]) && isfinite(up[j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        act[j] = e0 + j * kThreads < span ? RoundBF16(__fmul_rn(SiluRounded(finite[j] ? gate[j] : 0.f), up[j])) : 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = e0 + j * kThreads;
        if (e < span) {
          if (!finite[j] || !isfinite(act[j])) {
            if (!flagged) // a flag raised earlier explains garbage here; only a fresh failure is reported
              Raise(a.bad);
            flagged = 1;
          }
          s_act[e] = __fmul_rn(act[j], HalfBitsToFloat(s_suh[e]));
        }
      }
    }
  __syncthreads();
  PADRA_TRACE(a.trace, 11);
  if (recompute && spread)
    for (int block = warp; block < blocks; block += 8) {
      const float4 in = *reinterpret_cast<const float4 *>(s_act + block * 128 + lane * 4);
      float v[4] = {in.x, in.y, in.z, in.w};
      WarpHadamard128(v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float r = RoundBF16(v[i]);
        const __half h = __float2half_rn(r);
        if (!isfinite(r) || (__half_as_ushort(h) & 0x7c00) == 0x7c00) {
          if (!flagged)
            Raise(a.bad);
          flagged = 1;
        }
        xs[PermutedPlace(block * 128 + lane * 4 + i)] = h;
      }
    }
  if (__syncthreads_or(flagged))
    work = false; // refused or failed: no sums from this CTA, but its ticket is still taken
  PADRA_TRACE(a.trace, 4);
  if (work) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    StreamRounds<Rate>(stream, fetched, rounds, xs + (lane & 3) * 16, lane, acc);
    PADRA_TRACE(a.trace, 5);
    const int g = lane >> 2;
    float *p = a.down + (static_cast<size_t>(slot) * a.slices_down + slice) * a.hidden + nb * 128 + warp * 16;
    if ((lane & 3) == 0) {
      p[g] = acc[0];
      p[g + 8] = acc[2];
    }
    if (slice == 0 && warp == 7)
      *reinterpret_cast<uint2 *>(a.svh_rows + static_cast<size_t>(slot) * a.hidden + nb * 128 + lane * 4) = svh_bits;
  }
  // ---- ticket: the CTA that delivers the last of the block's 8 x slices sums combines ----
  // One thread draws the ticket behind the CTA's barrier with release and acquire at device scope: the release covers the
  // sums the CTA's threads stored before the barrier, the acquire (in the CTA that turns out to be last) the other CTAs'.
  __syncthreads();
  PADRA_TRACE(a.trace, 6);
  if (tid == 0) {
    unsigned *ticket = a.tickets + nb;
    unsigned drawn;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(drawn) : "l"(ticket) : "memory");
    const bool last = drawn == static_cast<unsigned>(kTopK) * a.slices_down - 1u;
    if (last)
      *ticket = 0; // nobody else touches it before the next call
    s_last = last;
  }
  __syncthreads();
  PADRA_TRACE(a.trace, 7);
  if (!s_last)
    return;
  // one round trip: flag, the eight slots' sums and sidecars, routing weights, the residual row
  const int out = nb * 128 + lane * 4; // warp = slot from here on
  flagged = LoadFlag(a.bad);
  const float *pd = a.down + static_cast<size_t>(warp) * a.slices_down * a.hidden + out;
  float d[4] = {0.f, 0.f, 0.f, 0.f};
  const uint2 sc_bits = __ldcg(reinterpret_cast<const uint2 *>(a.svh_rows + static_cast<size_t>(warp) * a.hidden + out));
  float w = 0.f;
  float4 xv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (warp == 0) {
    w = lane < kTopK ? __ldcg(a.routing + lane) : 0.f;
    xv = __ldcg(reinterpret_cast<const float4 *>(a.x + out));
  }
  for (int s0 = 0; s0 < a.slices_down; s0 += 4) {
    float4 vd[4];
#pragma unroll
    for (int s = 0; s < 4; ++s)
      if (s0 + s < a.slices_down)
        vd[s] = __ldcg(reinterpret_cast<const float4 *>(pd + static_cast<size_t>(s0 + s) * a.hidden));
#pragma unroll
    for (int s = 0; s < 4; ++s)
      if (s0 + s < a.slices_down)
        d[0] += vd[s].x, d[1] += vd[s].y, d[2] += vd[s].z, d[3] += vd[s].w;
  }
  float sc[4];
  Unpack4(sc_bits, sc);
  WarpHadamard128(d);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    d[i] = RoundBF16(__fmul_rn(d[i], sc[i]));
    if (!isfinite(d[i])) {
      if (!flagged) // a fresh failure; with an earlier flag some sums were never written and garbage is expected
        Raise(a.bad);
      flagged = 1;
    }
  }
  *reinterpret_cast<float4 *>(&s_down[warp][lane * 4]) = make_float4(d[0], d[1], d[2], d[3]);
  const bool refused = __syncthreads_or(flagged) != 0; // the barrier also publishes s_down; refused: x is left alone
  if (warp == 0 && !refused) {
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
    *reinterpret_cast<float4 *>(a.x + out) = xv;
  }
  PADRA_TRACE(a.trace, 8);
  // ---- the CTA that combines the last block clears the arrival counters for the next call: every CTA of this kernel
  // has taken its ticket by then, so nobody polls them any more ----
  if (tid == 0) {
    unsigned *combined = a.ready + kTopK * kMaxBlocks;
    const bool final = atomicAdd(combined, 1u) == gridDim.y - 1u;
    if (final)
      *combined = 0;
    s_final = final;
  }
  __syncthreads();
  if (s_final)
    for (int i = tid; i < kTopK * kMaxBlocks; i += kThreads)
      a.ready[i] = 0;
}

template <int Rate> int LaunchSingle(const SingleArgs &a, unsigned launches, cudaStream_t stream) {
  int status = PADRA_OK;

  if (launches & 1u) {
    const size_t smem = static_cast<size_t>(a.hidden / a.slices_gateup) * sizeof(__half);
    if (smem > 40 * 1024 && cudaFuncSetAttribute(SingleGateUpKernel<Rate>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(smem)) != cudaSuccess)
      return PADRA_RESOURCE_EXHAUSTED;
    status = LaunchProgrammatic(SingleGateUpKernel<Rate>, dim3(2 * a.slices_gateup, a.inter / 128, kTopK), dim3(kThreads), smem, stream, a);
  }
  if (status != PADRA_OK)
    return status;
  if (launches & 2u) {
    // the slice's transformed input row; for slices of at most one element per thread also three float rows of the gate/up
    // epilogue (gate, up, activation) and the input signs
    const size_t span = static_cast<size_t>(a.inter / a.slices_down);
    const size_t smem = span * (span <= static_cast<size_t>(kThreads) ? 2 * sizeof(__half) + 3 * sizeof(float) : sizeof(__half));
    if (smem > 36 * 1024 && cudaFuncSetAttribute(SingleDownKernel<Rate>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(smem)) != cudaSuccess)
      return PADRA_RESOURCE_EXHAUSTED;
    status = LaunchProgrammatic(SingleDownKernel<Rate>, dim3(a.slices_down, a.hidden / 128, kTopK), dim3(kThreads), smem, stream, a);
  }
  return status;
}

} // namespace

int LaunchSingleTokenLayer(const Matrix *matrices, int layer, const int *ids, const float *routing, const float *normalized, float *x,
                           int rate, int hidden, int inter, const unsigned short *table, void *workspace, int *bad, cudaStream_t stream,
                           unsigned launches) {
  const LayerWorkspace w(1, hidden, inter);
  auto *base = static_cast<unsigned char *>(workspace);
  SingleArgs a{};
  a.matrices = matrices, a.layer = layer, a.ids = ids, a.routing = routing, a.normalized = normalized, a.x = x;
  a.hidden = hidden, a.inter = inter, a.slices_gateup = w.slices_gateup, a.slices_down = w.slices_down, a.table = table, a.bad = bad;
  a.gateup = reinterpret_cast<float *>(base + w.gateup), a.sidecars = reinterpret_cast<__half *>(base + w.sidecars);
  a.down = reinterpret_cast<float *>(base + w.down), a.svh_rows = reinterpret_cast<__half *>(base + w.svh);
  a.tickets = reinterpret_cast<unsigned *>(base + w.tickets_down);
  a.ready = reinterpret_cast<unsigned *>(base + w.tickets_gateup); // the gate+up ticket area serves as arrival counters here
  // One kernel alone (a diagnostic: timing or profiling it on buffers a complete call has filled): a lone gate+up kernel
  // does not count its arrivals, a lone down kernel finds the counters set to "everything has arrived" (it clears them).
  if (launches == 1u)
    a.ready = nullptr;
  if (launches == 2u && cudaMemsetAsync(a.ready, 1, static_cast<size_t>(kTopK) * kMaxBlocks * sizeof(unsigned), stream) != cudaSuccess)
    return PADRA_INTERNAL;
#ifdef PADRA_DECODE_TRACE
  a.trace = g_trace ? g_trace + static_cast<size_t>(g_trace_launch++) * 2 * 1024 * 16 : nullptr;
  if (a.trace && (launches & 1u)) {
    SingleArgs first = a;
    int status = rate == 3 ? LaunchSingle<3>(first, 1u, stream) : rate == 6 ? LaunchSingle<6>(first, 1u, stream) : LaunchSingle<4>(first, 1u, stream);
    if (status != PADRA_OK)
      return status;
    a.trace += 1024 * 16;
    launches &= ~1u;
  }
#endif
  switch (rate) {
  case 3:
    return LaunchSingle<3>(a, launches, stream);
  case 4:
    return LaunchSingle<4>(a, launches, stream);
  case 6:
    return LaunchSingle<6>(a, launches, stream);
  default:
    return PADRA_UNSUPPORTED;
  }
}

} // namespace padra
