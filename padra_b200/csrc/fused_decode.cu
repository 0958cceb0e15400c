// Whole EXL3 expert layer at decode (M = 1..16 rows) as ONE persistent cooperative kernel.
//
// Why one kernel: a layer step is 25 MB of packed weights (K4, hidden 2048 / intermediate 1024, eight experts),
// a few microseconds of HBM time.  Separate launches for gate/up, SwiGLU, down and combine spend more time
// starting, draining and waiting on each other than streaming.  Here one CTA per SM walks a static, strided
// list of 128-output x 128-input weight chunks that covers the gate/up matrices of every active expert and then
// the down matrices, so all SMs stream from the first to the last byte, and the dependent steps (split-K
// reduction, output Hadamard, SwiGLU, the down projection's input transform, combine) are done by whichever CTA
// delivers the last chunk of a unit, off the streaming warps' critical path.
//
// Roles inside a CTA (19 warps):
//   * two streaming groups of 8 warps.  A group owns every (2*gridDim)-th chunk; warp w of the group owns tile
//     column w of the chunk (16 outputs) and both of its K-rounds.  Packed words are register-prefetched two
//     chunks ahead, decoded in registers (codec.cuh) and multiplied with mma.m16n8k16 against the chunk's
//     activation tile in shared memory; the FP32 partial sums go straight to the workspace.  The group also
//     stages its own activation tiles one chunk ahead, the rows dealt round-robin over its warps: the input
//     Hadamard of x * suh for a gate/up chunk, a copy of the published SwiGLU output for a down chunk.
//   * one counting warp per group.  It learns from a shared-memory counter that the group has stored the partial
//     sums of one or more chunks and counts them against their units in the workspace (one lane per chunk, so
//     the round trips of a batch overlap).  A chunk that completes its unit is queued for the epilogue warp.
//   * one epilogue warp.  It takes completed units from the queue and runs their epilogue, so that counting is
//     never held up behind an epilogue.  Counting and epilogue warps wait on shared memory of their own CTA only.
//
// Determinism: chunk -> CTA assignment and every summation order are fixed by the shapes alone, so results are
// bit-identical run to run and under CUDA-graph replay.
//
// Waiting rules: the only cross-CTA wait is a streaming warp polling the "ready" word of a gate/up unit before
// it copies a down chunk's tile.  It polls ahead of time only for units whose chunks all lie more than two grid
// strides before the end of the gate/up range, and otherwise only after its group has stored every gate/up
// chunk it owns, so a poll never holds back work the polled unit depends on, for any shape.  Every poll is
// bounded: on expiry the warp records an error and proceeds, so the kernel always terminates.  All CTAs must
// be co-resident, hence the cooperative launch with one CTA per SM.
#include "codec.cuh"
#include "common.cuh"
#include "kernels.cuh"

namespace padra {
namespace {

constexpr int kGroups = 2;
constexpr int kGroupWarps = 8;
constexpr int kStreamWarps = kGroups * kGroupWarps;
constexpr int kCountWarps = 1;                                    // per group
constexpr int kFinishWarp = kStreamWarps + kGroups * kCountWarps; // index of the CTA's epilogue warp
constexpr int kWarps = kFinishWarp + 1;                           // 19
constexpr int kFusedThreads = kWarps * 32;                        // 608
constexpr int kQueue = 16;                                        // completed units waiting for their epilogue
constexpr unsigned kEmpty = 0xffffffffu;
constexpr int kTileBuffers = 3;
constexpr int kXsStride = 128 + 8; // halves per staged activation row (+16 B against bank conflicts)
constexpr int kGroupThreads = kGroupWarps * 32;
constexpr int kMaxBlocks = 64; // 128-wide blocks per dimension the control words provide for
constexpr unsigned kPollLimit = 1u << 20;
constexpr int kChunkTable = 64; // chunks per group described up front; later ones are described on the fly

// Control words at the start of the workspace.  All zero between launches: the last CTA to finish clears them.
struct Control {
  unsigned done;
  unsigned error;
  unsigned pad[2];
  unsigned unit_down[kMaxBlocks];              // arrivals per 128-output block of the down projection
  unsigned unit_gateup[kExperts * kMaxBlocks]; // arrivals per (expert, 128-output block) of gate+up
  unsigned ready[kExperts * kMaxBlocks];       // 1 once the block's down-projection input is published
};

struct FusedArgs {
  const Matrix *matrices;
  int layer;
  const int *ids;          // [tokens][8]
  const float *routing;    // [tokens][8]
  const float *normalized; // [tokens][hidden]
  float *x;                // [tokens][hidden], residual in/out
  int tokens, hidden, inter;
  const unsigned short *table;
  Control *control;
  __half *xdown;   // [pairs][inter], permuted K16 order
  float *partials; // gate/up partial sums, then down partial sums
  int *bad;
  unsigned long long *trace; // optional timeline, kTraceSlots words per CTA (nullptr: off)
};

constexpr int kTraceSlots = 64;
__device__ __forceinline__ unsigned long long GlobalTimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Timeline slots per CTA: 0 start, 1 set-up done, 2 group-0 streaming done, 3 group-0 counting done, 4 end,
// 8.. time after the tile barrier of each chunk of group 0 (warp 0), 36.. time of each counting batch of group 0.
__device__ __forceinline__ void Trace(const FusedArgs &a, int slot) {
  if (a.trace && slot < kTraceSlots)
    a.trace[static_cast<size_t>(blockIdx.x) * kTraceSlots + slot] = GlobalTimer();
}

__device__ __forceinline__ void GroupBarrier(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(kGroupThreads) : "memory");
}
__device__ __forceinline__ unsigned LoadAcquire(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void MmaF16(const uint32_t (&a)[4], uint32_t b0, uint32_t b1, float (&d)[4]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// idx / d for idx < 2^22 with a precomputed reciprocal: two fix-ups make the float estimate exact.
struct Divider {
  int d;
  float inv;
  __device__ __forceinline__ void Set(int v) {
    d = v;
    inv = 1.0f / static_cast<float>(v);
  }
  __device__ __forceinline__ int Div(int idx) const {
    int q = static_cast<int>(static_cast<float>(idx) * inv);
    q -= (q * d > idx);
    q += ((q + 1) * d <= idx);
    return q;
  }
};

// Shape-derived chunk bookkeeping, identical in every thread.
struct Geometry {
  int blocks_inter, blocks_hidden; // 128-wide blocks
  int per_expert_gateup, per_expert_down;
  int chunks_gateup, chunks_total, active;
  Divider by_gateup, by_down, by_2kh, by_kh, by_ki;
  size_t down_partials; // float offset of the down partial sums
};

// One chunk: part 0/1/2, expert, 128-output block `nb`, 128-input block `kc`.
struct Chunk {
  int part, expert, nb, kc, count;
  int order; // position of the expert in the ascending list of active experts
};

// A chunk squeezed into one register for the two prefetch slots.
__device__ __forceinline__ unsigned PackChunk(const Chunk &c) {
  return static_cast<unsigned>(c.part) | (static_cast<unsigned>(c.expert) << 2) | (static_cast<unsigned>(c.nb) << 8) |
         (static_cast<unsigned>(c.kc) << 14) | (static_cast<unsigned>(c.count) << 20) | (static_cast<unsigned>(c.order) << 25);
}
__device__ __forceinline__ Chunk UnpackChunk(unsigned w) {
  Chunk c;
  c.part = w & 3u;
  c.expert = (w >> 2) & 63u;
  c.nb = (w >> 8) & 63u;
  c.kc = (w >> 14) & 63u;
  c.count = (w >> 20) & 31u;
  c.order = (w >> 25) & 63u;
  return c;
}

template <int NG> struct Tables {
  const unsigned char *data[kExperts][3]; // packed words of gate, up, down (validated at start)
  const uint16_t *suh[kExperts][3];
  const uint16_t *svh[kExperts][3];
  unsigned char rows[kExperts][8 * NG]; // token*8+slot of the n-th row routed to the expert
  unsigned char count[kExperts];
  unsigned char active[kExperts]; // ascending ids of experts with at least one row
};

template <int NG>
__device__ __forceinline__ Chunk Describe(int idx, const Geometry &geo, const Tables<NG> &tab) {
  Chunk c;
  int a;
  if (idx < geo.chunks_gateup) {
    a = geo.by_gateup.Div(idx);
    const int rem = idx - a * geo.per_expert_gateup;
    c.nb = geo.by_2kh.Div(rem);
    const int rem2 = rem - c.nb * 2 * geo.blocks_hidden;
    c.part = geo.by_kh.Div(rem2);
    c.kc = rem2 - c.part * geo.blocks_hidden;
  } else {
    const int i2 = idx - geo.chunks_gateup;
    a = geo.by_down.Div(i2);
    const int rem = i2 - a * geo.per_expert_down;
    c.nb = geo.by_ki.Div(rem);
    c.kc = rem - c.nb * geo.blocks_inter;
    c.part = 2;
  }
  c.order = a;
  c.expert = tab.active[a];
  c.count = tab.count[c.expert];
  return c;
}

__device__ __forceinline__ size_t PartialOffset(int part, int nb, int kc, int pair, const Geometry &geo) {
  if (part < 2)
    return ((static_cast<size_t>(pair * geo.blocks_inter + nb) * 2 + part) * geo.blocks_hidden + kc) * 128;
  return geo.down_partials + (static_cast<size_t>(pair * geo.blocks_hidden + nb) * geo.blocks_inter + kc) * 128;
}

__device__ __forceinline__ float4 LoadL2(const float *p) {
  return __ldcg(reinterpret_cast<const float4 *>(p));
}
__device__ __forceinline__ void Unpack4(uint2 bits, float (&f)[4]) {
  f[0] = HalfBitsToFloat(bits.x & 0xffffu);
  f[1] = HalfBitsToFloat(bits.x >> 16);
  f[2] = HalfBitsToFloat(bits.y & 0xffffu);
  f[3] = HalfBitsToFloat(bits.y >> 16);
}

// Registers one warp holds for the (at most NG) tile rows it stages: the raw inputs of a gate/up tile (x and
// the shared suh block) or the finished halves of a down tile.
template <int NG> struct TileRegs {
  float4 x[NG]; // gate/up tile: this lane's four inputs per row; down tile: .x/.y carry the four staged halves
  uint2 sign;   // gate/up tile: suh of this lane's four inputs
  int state;    // 0 nothing loaded, 1 gate/up inputs loaded, 2 down halves loaded
};

template <int Rate, int NG>
__global__ void __launch_bounds__(kFusedThreads, 1) FusedDecodeLayerKernel(FusedArgs a) {
  using L = codec::Lane<Rate>;
  constexpr int kRows = 8 * NG;
  __shared__ Tables<NG> tab;
  __shared__ Geometry geo; // read through shared memory to keep it out of the streaming warps' registers
  __shared__ int s_active_count, s_invalid, s_last;
  __shared__ unsigned s_warp_votes[2];
  __shared__ unsigned s_stored[kGroups]; // warp-chunks whose partial sums are stored, per group
  __shared__ unsigned s_chunks[kGroups][kChunkTable]; // this CTA's chunks, described once (PackChunk)
  __shared__ unsigned s_queue[kQueue];                // completed units (PackChunk of the completing chunk) or kEmpty
  __shared__ unsigned s_queue_tail, s_counting_done;
  __shared__ __align__(16) __half s_xs[kGroups][kTileBuffers][kRows * kXsStride];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  Control *ctl = a.control;
  if (tid == 0)
    Trace(a, 0);

  // ---- which rows use which expert (every CTA builds the same tables) -----------------------------------
  if (tid == 0) {
    s_invalid = 0;
    s_stored[0] = s_stored[1] = 0;
    s_queue_tail = s_counting_done = 0;
  }
  if (tid < kQueue)
    s_queue[tid] = kEmpty;
  __syncthreads();
  if (tid < kExperts) {
    const int expert = tid;
    int n = 0, bad_id = 0;
    for (int r = 0; r < a.tokens; ++r)
      for (int s = 0; s < kTopK; ++s) {
        const int id = a.ids[r * kTopK + s];
        bad_id |= (id < 0 || id >= kExperts);
        if (id == expert) {
          if (n < kRows)
            tab.rows[expert][n] = static_cast<unsigned char>(r * kTopK + s);
          ++n;
        }
      }
    if (bad_id || n > kRows)
      atomicOr(&s_invalid, 1);
    tab.count[expert] = static_cast<unsigned char>(n < kRows ? n : kRows);
    const unsigned votes = __ballot_sync(0xffffffffu, n > 0);
    if (!lane)
      s_warp_votes[warp] = votes;
  }
  __syncthreads();
  if (tid < kExperts) {
    const unsigned mine = s_warp_votes[warp];
    if (mine & (1u << lane)) {
      const int rank = __popc(mine & ((1u << lane) - 1u)) + (warp ? __popc(s_warp_votes[0]) : 0);
      tab.active[rank] = static_cast<unsigned char>(tid);
    }
    if (!tid)
      s_active_count = __popc(s_warp_votes[0]) + __popc(s_warp_votes[1]);
  }
  // descriptors of the active experts: checked once, pointers kept in shared memory
  if (tid < kExperts * 3) {
    const int expert = tid / 3, part = tid - expert * 3;
    if (tab.count[expert]) {
      const Matrix m = a.matrices[(static_cast<size_t>(a.layer) * kExperts + expert) * 3 + part];
      const int want_rows = part == 2 ? a.hidden : a.inter, want_cols = part == 2 ? a.inter : a.hidden;
      if (m.format != FormatOfRate(Rate) || m.rows != want_rows || m.cols != want_cols || !m.data || !m.suh || !m.svh)
        atomicOr(&s_invalid, 2);
      tab.data[expert][part] = m.data;
      tab.suh[expert][part] = m.suh;
      tab.svh[expert][part] = m.svh;
    }
  }
  __syncthreads();
  // Every exit below is taken by all CTAs of the grid or by none: ids and descriptors are the same for all,
  // and `*bad` only ever changes at the very end of a launch.
  if (s_invalid) {
    if (!blockIdx.x && !tid)
      Raise(a.bad);
    return;
  }
  if (*a.bad)
    return;

  if (tid == 0) {
    geo.blocks_inter = a.inter / 128;
    geo.blocks_hidden = a.hidden / 128;
    geo.per_expert_gateup = geo.blocks_inter * 2 * geo.blocks_hidden;
    geo.per_expert_down = geo.blocks_hidden * geo.blocks_inter;
    geo.active = s_active_count;
    geo.chunks_gateup = geo.active * geo.per_expert_gateup;
    geo.chunks_total = geo.chunks_gateup + geo.active * geo.per_expert_down;
    geo.by_gateup.Set(geo.per_expert_gateup);
    geo.by_down.Set(geo.per_expert_down);
    geo.by_2kh.Set(2 * geo.blocks_hidden);
    geo.by_kh.Set(geo.blocks_hidden);
    geo.by_ki.Set(geo.blocks_inter);
    geo.down_partials = static_cast<size_t>(a.tokens) * kTopK * geo.blocks_inter * 2 * geo.blocks_hidden * 128;
  }
  __syncthreads();

  const int group = warp < kStreamWarps ? warp / kGroupWarps : (warp < kFinishWarp ? (warp - kStreamWarps) / kCountWarps : 0);
  const int first = blockIdx.x * kGroups + group, stride = gridDim.x * kGroups;
  const int mine = first < geo.chunks_total ? (geo.chunks_total - first + stride - 1) / stride : 0;
  // the chunk list of both groups, described once instead of once per warp and use
  for (int i = tid; i < kGroups * kChunkTable; i += kFusedThreads) {
    const int grp = i / kChunkTable, j = i - grp * kChunkTable;
    const int idx = blockIdx.x * kGroups + grp + j * stride;
    if (idx < geo.chunks_total)
      s_chunks[grp][j] = PackChunk(Describe<NG>(idx, geo, tab));
  }
  __syncthreads();
  if (tid == 0)
    Trace(a, 1);
  auto j_packed = [&](int j) {
    return j < kChunkTable ? s_chunks[group][j] : PackChunk(Describe<NG>(first + j * stride, geo, tab));
  };
  auto chunk_at = [&](int j) {
    return j < kChunkTable ? UnpackChunk(s_chunks[group][j]) : Describe<NG>(first + j * stride, geo, tab);
  };
  const int my_gateup = first < geo.chunks_gateup ? (geo.chunks_gateup - first + stride - 1) / stride : 0;
  // Permuted K16 position of this lane's four consecutive inputs inside a 128-input block.
  const int permuted = (lane >> 2) * 16 + 8 * (lane & 1) + 2 * ((lane >> 1) & 1);

  if (warp < kStreamWarps) {
    // =============================== streaming warps ===============================
    const int col = warp % kGroupWarps, g = lane >> 2, t = lane & 3;

    // Packed words of chunk `c` for this lane: two rounds of four K16 steps.
    auto fetch = [&](const Chunk &c, uint32_t (&w)[2][Rate]) {
      const unsigned char *data = tab.data[c.expert][c.part];
      const size_t tiles_per_kstep = (c.part == 2 ? a.hidden : a.inter) / 16;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const size_t kstep = c.kc * 8 + r * 4 + t;
        codec::LoadWords<Rate>(data + (kstep * tiles_per_kstep + c.nb * 8 + col) * L::kTileBytes + g * L::kBytes, w[r]);
      }
    };

    // ---- activation tiles: row n of tile j is staged by warp (j + n) % 8 of the group ----
    auto poll_ready = [&](const Chunk &c) {
      const unsigned *flag = &ctl->ready[c.expert * kMaxBlocks + c.kc];
      unsigned polls = 0;
      while (LoadAcquire(flag) == 0u) { // all lanes poll the same word; each gets its own acquire
        if (++polls > kPollLimit) {
          atomicOr(&ctl->error, 2u); // gave up: proceed with whatever is there, the step is rejected
          break;
        }
        __nanosleep(64);
      }
    };
    // true when the gate/up unit a down chunk depends on lies wholly more than two strides before the end of
    // the gate/up range (see the waiting rules at the top)
    auto poll_is_safe = [&](const Chunk &c) {
      const int unit_last = c.order * geo.per_expert_gateup + (c.kc + 1) * 2 * geo.blocks_hidden - 1;
      return unit_last < geo.chunks_gateup - 2 * stride;
    };
    auto tile_load = [&](int j, const Chunk &c, TileRegs<NG> &regs, bool synchronous) {
      regs.state = 0;
      const int n0 = (col - j % kGroupWarps + kGroupWarps) % kGroupWarps; // rows n0, n0+8 are this warp's
      if (n0 >= c.count)
        return;
      if (c.part < 2) {
        regs.sign = __ldg(reinterpret_cast<const uint2 *>(tab.suh[c.expert][c.part] + c.kc * 128 + lane * 4));
#pragma unroll
        for (int u = 0; u < NG; ++u)
          if (n0 + 8 * u < c.count) {
            const int token = tab.rows[c.expert][n0 + 8 * u] >> 3;
            regs.x[u] = __ldg(reinterpret_cast<const float4 *>(a.normalized + static_cast<size_t>(token) * a.hidden + c.kc * 128 + lane * 4));
          }
        regs.state = 1;
      } else {
        if (!synchronous && !poll_is_safe(c)) {
          regs.state = 3; // to be fetched later, once this group holds no gate/up work
          return;
        }
        poll_ready(c);
#pragma unroll
        for (int u = 0; u < NG; ++u)
          if (n0 + 8 * u < c.count) {
            const int pair = tab.rows[c.expert][n0 + 8 * u];
            const uint2 staged = __ldcg(reinterpret_cast<const uint2 *>(a.xdown + static_cast<size_t>(pair) * a.inter + c.kc * 128 + lane * 4));
            regs.x[u].x = __uint_as_float(staged.x);
            regs.x[u].y = __uint_as_float(staged.y);
          }
        regs.state = 2;
      }
    };
    auto tile_store = [&](int j, const Chunk &c, const TileRegs<NG> &regs) {
      const int n0 = (col - j % kGroupWarps + kGroupWarps) % kGroupWarps;
      __half *xs = s_xs[group][j % kTileBuffers];
      if (regs.state == 1) {
        // x~ = fp16(B(H128(x * suh))) (reference: expert_exl3_decode_dual.cuh:65-85)
        float sg[4];
        Unpack4(regs.sign, sg);
#pragma unroll
        for (int u = 0; u < NG; ++u)
          if (n0 + 8 * u < c.count) {
            float v[4] = {__fmul_rn(regs.x[u].x, sg[0]), __fmul_rn(regs.x[u].y, sg[1]), __fmul_rn(regs.x[u].z, sg[2]),
                          __fmul_rn(regs.x[u].w, sg[3])};
            WarpHadamard128(v);
            __half hv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float r = RoundBF16(v[i]);
              hv[i] = __float2half_rn(r);
              if (!isfinite(r) || (__half_as_ushort(hv[i]) & 0x7c00) == 0x7c00)
                atomicOr(&ctl->error, 1u);
            }
            __half *dst = xs + (n0 + 8 * u) * kXsStride + permuted;
            *reinterpret_cast<__half2 *>(dst) = __halves2half2(hv[0], hv[1]);
            *reinterpret_cast<__half2 *>(dst + 4) = __halves2half2(hv[2], hv[3]);
          }
      } else if (regs.state == 2) {
#pragma unroll
        for (int u = 0; u < NG; ++u)
          if (n0 + 8 * u < c.count)
            *reinterpret_cast<uint2 *>(xs + (n0 + 8 * u) * kXsStride + lane * 4) =
                make_uint2(__float_as_uint(regs.x[u].x), __float_as_uint(regs.x[u].y));
      }
    };

    // One chunk.  `slot`/`slot_chunk` hold chunk j on entry and chunk j+2 on exit; `other_chunk` is chunk j+1;
    // `next_tile` holds this warp's rows of tile j+1 (loaded one chunk ago), `later_tile` receives tile j+2.
    auto stream = [&](int j, uint32_t (&slot)[2][Rate], unsigned &slot_chunk, unsigned other_chunk, TileRegs<NG> &next_tile,
                      TileRegs<NG> &later_tile) {
      const Chunk c = UnpackChunk(slot_chunk);
      uint32_t words[2][Rate];
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int i = 0; i < Rate; ++i)
          words[r][i] = slot[r][i];
      later_tile.state = 0;
      if (j + 2 < mine) {
        const Chunk ahead = chunk_at(j + 2);
        slot_chunk = PackChunk(ahead);
        fetch(ahead, slot);
        tile_load(j + 2, ahead, later_tile, /*synchronous=*/false);
      }
      // round 0 is decoded before the barrier (it needs no activations), round 1 after its MMAs were issued
      uint32_t frag[4][4];
      {
        const uint32_t previous = __shfl_sync(0xffffffffu, words[0][Rate - 1], (lane + 28) & 31);
        codec::Decode32<Rate>(words[0], previous, frag);
      }
      GroupBarrier(group); // tile j is complete in shared memory
      if (warp == 0 && lane == 0 && j < 12)
        Trace(a, 8 + j);
      const __half *xs = s_xs[group][j % kTileBuffers];
      float acc[NG][4];
      const __half *xrow[NG];
#pragma unroll
      for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          acc[ng][i] = 0.f;
        const int n = g + 8 * ng;
        xrow[ng] = xs + (n < c.count ? n : c.count - 1) * kXsStride + t * 16;
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (r == 1) {
          const uint32_t previous = __shfl_sync(0xffffffffu, words[1][Rate - 1], (lane + 28) & 31);
          codec::Decode32<Rate>(words[1], previous, frag);
        }
#pragma unroll
        for (int ng = 0; ng < NG; ++ng) {
          const uint4 lo = *reinterpret_cast<const uint4 *>(xrow[ng] + r * 64);
          const uint4 hi = *reinterpret_cast<const uint4 *>(xrow[ng] + r * 64 + 8);
          MmaF16(frag[0], lo.x, lo.y, acc[ng]);
          MmaF16(frag[1], lo.z, lo.w, acc[ng]);
          MmaF16(frag[2], hi.x, hi.y, acc[ng]);
          MmaF16(frag[3], hi.z, hi.w, acc[ng]);
        }
      }
#pragma unroll
      for (int ng = 0; ng < NG; ++ng)
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int n = 8 * ng + 2 * t + cc;
          if (n < c.count) {
            float *p = a.partials + PartialOffset(c.part, c.nb, c.kc, tab.rows[c.expert][n], geo) + col * 16 + g;
            p[0] = acc[ng][cc];
            p[8] = acc[ng][2 + cc];
          }
        }
      __threadfence_block();
      __syncwarp();
      if (lane == 0)
        atomicAdd(&s_stored[group], 1u); // this warp's share of chunk j is in the workspace
      // Tile j+1 goes to buffer (j+1)%3, last read by chunk j-2, which every warp of the group has left.  Its
      // inputs were loaded a whole chunk ago -- except for a down tile whose unit was not safe to poll ahead of
      // time: that one is fetched now, when the group has stored every gate/up chunk it owns.
      if (j + 1 < mine) {
        const Chunk next = UnpackChunk(other_chunk);
        if (next_tile.state == 3)
          tile_load(j + 1, next, next_tile, /*synchronous=*/true);
        tile_store(j + 1, next, next_tile);
      }
    };

    uint32_t slot0[2][Rate], slot1[2][Rate];
    unsigned chunk0 = 0, chunk1 = 0;
    TileRegs<NG> tile0, tile1;
    tile0.state = tile1.state = 0;
    if (mine > 0) {
      const Chunk c0 = chunk_at(0);
      chunk0 = PackChunk(c0);
      fetch(c0, slot0);
      tile_load(0, c0, tile0, /*synchronous=*/true); // nothing of this group is pending yet
      tile_store(0, c0, tile0);
    }
    if (mine > 1) {
      const Chunk c1 = chunk_at(1);
      chunk1 = PackChunk(c1);
      fetch(c1, slot1);
      tile_load(1, c1, tile1, /*synchronous=*/my_gateup == 0);
    }
    for (int j = 0; j < mine; j += 2) {
      stream(j, slot0, chunk0, chunk1, tile1, tile0);
      if (j + 1 < mine)
        stream(j + 1, slot1, chunk1, chunk0, tile0, tile1);
    }
    if (warp == 0 && lane == 0)
      Trace(a, 2);
  } else if (warp < kFinishWarp) {
    // =============================== counting warps ===============================
    int counted = 0; // chunks of this group already counted against their units
    while (counted < mine) {
      // wait (within this CTA only) until all eight warps of the group have stored at least one more chunk
      unsigned stored = 0, polls = 0;
      while ((stored = *reinterpret_cast<volatile unsigned *>(&s_stored[group]) / kGroupWarps) <= static_cast<unsigned>(counted)) {
        if (++polls > 16 * kPollLimit) {
          atomicOr(&ctl->error, 4u);
          stored = mine; // count the rest regardless; the step is rejected
          break;
        }
        __nanosleep(40);
      }
      const int batch = min(static_cast<int>(stored) - counted, 32);
      // one lane per chunk of the batch: release the group's stores, count the chunk, queue a completed unit
      if (lane < batch) {
        const unsigned packed = j_packed(counted + lane);
        const Chunk c = UnpackChunk(packed);
        unsigned *counter = c.part < 2 ? &ctl->unit_gateup[c.expert * kMaxBlocks + c.nb] : &ctl->unit_down[c.nb];
        const unsigned needed = c.part < 2 ? 2u * geo.blocks_hidden : static_cast<unsigned>(geo.active) * geo.blocks_inter;
        __threadfence();
        if (atomicAdd(counter, 1u) == needed - 1) {
          __threadfence();
          const unsigned slot = atomicAdd(&s_queue_tail, 1u) % kQueue;
          unsigned waits = 0;
          while (*reinterpret_cast<volatile unsigned *>(&s_queue[slot]) != kEmpty) { // the epilogue warp is behind
            if (++waits > kPollLimit) {
              atomicOr(&ctl->error, 8u);
              break;
            }
            __nanosleep(100);
          }
          *reinterpret_cast<volatile unsigned *>(&s_queue[slot]) = packed;
        }
      }
      __syncwarp();
      counted += batch;
      if (group == 0 && lane == 0)
        Trace(a, 36 + (counted < 28 ? counted : 27));
    }
    __threadfence_block();
    __syncwarp();
    if (lane == 0)
      atomicAdd(&s_counting_done, 1u);
    if (group == 0 && lane == 0)
      Trace(a, 3);
  } else {
    // =============================== epilogue warp ===============================
    auto note_nonfinite = [&](float v) {
      if (!isfinite(v))
        atomicOr(&ctl->error, 1u);
    };
    int trace_unit = 0;

    // gate/up epilogue for (expert, block nb): split-K sums -> output Hadamard, svh -> SwiGLU -> the down
    // projection's input transform (x suh, Hadamard, BF16, FP16), published for the down chunks.
    // Reference arithmetic: expert_exl3_decode_dual.cuh:116-130, exl3_silu_lut.cuh:15-31, :65-85.
    auto finalize_gateup = [&](const Chunk &c) {
      const int out = c.nb * 128 + lane * 4;
      float svg[4], svu[4], shd[4];
      Unpack4(__ldg(reinterpret_cast<const uint2 *>(tab.svh[c.expert][0] + out)), svg);
      Unpack4(__ldg(reinterpret_cast<const uint2 *>(tab.svh[c.expert][1] + out)), svu);
      Unpack4(__ldg(reinterpret_cast<const uint2 *>(tab.suh[c.expert][2] + out)), shd);
      for (int n = 0; n < c.count; ++n) {
        const int pair = tab.rows[c.expert][n];
        float gsum[4] = {0.f, 0.f, 0.f, 0.f}, usum[4] = {0.f, 0.f, 0.f, 0.f};
        const float *pg = a.partials + PartialOffset(0, c.nb, 0, pair, geo) + lane * 4;
        const float *pu = a.partials + PartialOffset(1, c.nb, 0, pair, geo) + lane * 4;
        for (int kc0 = 0; kc0 < geo.blocks_hidden; kc0 += 8) { // ascending K, sixteen loads in flight
          float4 vg[8], vu[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (kc0 + u < geo.blocks_hidden) {
              vg[u] = LoadL2(pg + (kc0 + u) * 128);
              vu[u] = LoadL2(pu + (kc0 + u) * 128);
            }
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (kc0 + u < geo.blocks_hidden) {
              gsum[0] += vg[u].x, gsum[1] += vg[u].y, gsum[2] += vg[u].z, gsum[3] += vg[u].w;
              usum[0] += vu[u].x, usum[1] += vu[u].y, usum[2] += vu[u].z, usum[3] += vu[u].w;
            }
        }
        if (lane == 0 && n == 0)
          Trace(a, 20 + 3 * trace_unit + 1);
        WarpHadamard128(gsum);
        WarpHadamard128(usum);
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float gate = RoundBF16(__fmul_rn(gsum[i], svg[i]));
          const float up = RoundBF16(__fmul_rn(usum[i], svu[i]));
          note_nonfinite(gate);
          note_nonfinite(up);
          const float silu = FromBF16Bits(__ldg(a.table + (__float_as_uint(gate) >> 16)));
          const float act = RoundBF16(__fmul_rn(silu, up));
          note_nonfinite(act);
          v[i] = __fmul_rn(act, shd[i]);
        }
        WarpHadamard128(v);
        __half hv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float r = RoundBF16(v[i]);
          hv[i] = __float2half_rn(r);
          if (!isfinite(r) || (__half_as_ushort(hv[i]) & 0x7c00) == 0x7c00)
            atomicOr(&ctl->error, 1u);
        }
        __half *dst = a.xdown + static_cast<size_t>(pair) * a.inter + c.nb * 128 + permuted;
        *reinterpret_cast<__half2 *>(dst) = __halves2half2(hv[0], hv[1]);
        *reinterpret_cast<__half2 *>(dst + 4) = __halves2half2(hv[2], hv[3]);
      }
      __threadfence();
      __syncwarp();
      if (lane == 0)
        atomicExch(&ctl->ready[c.expert * kMaxBlocks + c.nb], 1u);
    };

    // down epilogue for output block nb: per row, the eight slots in order -- split-K sum, output Hadamard, svh,
    // BF16 -- combined with the routing weights and the residual exactly like the reference's Combine
    // (src/cuda/inference.cu:580-594).
    auto finalize_down = [&](int nb) {
      const int out = nb * 128 + lane * 4;
      for (int r = 0; r < a.tokens; ++r) {
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < kTopK; ++s) {
          const int pair = r * kTopK + s;
          const int expert = a.ids[pair];
          float sc[4];
          Unpack4(__ldg(reinterpret_cast<const uint2 *>(tab.svh[expert][2] + out)), sc);
          const float *pd = a.partials + PartialOffset(2, nb, 0, pair, geo) + lane * 4;
          float d[4] = {0.f, 0.f, 0.f, 0.f};
          for (int kc0 = 0; kc0 < geo.blocks_inter; kc0 += 8) {
            float4 vd[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (kc0 + u < geo.blocks_inter)
                vd[u] = LoadL2(pd + (kc0 + u) * 128);
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (kc0 + u < geo.blocks_inter)
                d[0] += vd[u].x, d[1] += vd[u].y, d[2] += vd[u].z, d[3] += vd[u].w;
          }
          WarpHadamard128(d);
          const float w = a.routing[pair];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float down = RoundBF16(__fmul_rn(d[i], sc[i]));
            note_nonfinite(down);
            sum[i] = RoundBF16(__fadd_rn(sum[i], RoundBF16(__fmul_rn(down, w))));
          }
        }
        float4 xv = *reinterpret_cast<const float4 *>(a.x + static_cast<size_t>(r) * a.hidden + out);
        xv.x = RoundBF16(__fadd_rn(xv.x, sum[0]));
        xv.y = RoundBF16(__fadd_rn(xv.y, sum[1]));
        xv.z = RoundBF16(__fadd_rn(xv.z, sum[2]));
        xv.w = RoundBF16(__fadd_rn(xv.w, sum[3]));
        note_nonfinite(xv.x), note_nonfinite(xv.y), note_nonfinite(xv.z), note_nonfinite(xv.w);
        *reinterpret_cast<float4 *>(a.x + static_cast<size_t>(r) * a.hidden + out) = xv;
      }
    };

    unsigned head = 0, idle = 0;
    for (;;) {
      trace_unit = head < 5 ? head : 4;
      const unsigned done = *reinterpret_cast<volatile unsigned *>(&s_counting_done); // read before the queue slot
      const unsigned entry = *reinterpret_cast<volatile unsigned *>(&s_queue[head % kQueue]);
      if (entry != kEmpty) {
        if (lane == 0)
          Trace(a, 20 + 3 * trace_unit);
        __threadfence(); // the counting lane saw the unit complete; order this warp's loads after that
        const Chunk c = UnpackChunk(entry);
        if (c.part < 2)
          finalize_gateup(c);
        else
          finalize_down(c.nb);
        __syncwarp();
        if (lane == 0)
          Trace(a, 20 + 3 * trace_unit + 2);
        if (lane == 0)
          *reinterpret_cast<volatile unsigned *>(&s_queue[head % kQueue]) = kEmpty;
        __syncwarp();
        ++head;
        idle = 0;
      } else if (done == static_cast<unsigned>(kGroups * kCountWarps)) {
        break; // both counting warps have finished and queued everything they completed
      } else {
        if (++idle > 64 * kPollLimit) {
          atomicOr(&ctl->error, 16u);
          break;
        }
        __nanosleep(100);
      }
    }
  }

  // ---- leave the control words zero for the next launch ---------------------------------------------------
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    s_last = atomicAdd(&ctl->done, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    const unsigned error = LoadAcquire(&ctl->error);
    if (tid == 0 && error != 0u)
      Raise(a.bad);
    __syncthreads();
    unsigned *words = reinterpret_cast<unsigned *>(ctl);
    for (int i = tid; i < static_cast<int>(sizeof(Control) / sizeof(unsigned)); i += kFusedThreads)
      if (i != 3)
        words[i] = 0u;
    if (tid == 0)
      ctl->pad[1] |= error; // sticky record of what went wrong (1 value, 2 ready poll, 4 store poll, 8 queue, 16 epilogue)
  }
  if (tid == 0)
    Trace(a, 4);
}

struct FusedWorkspace {
  size_t control, xdown, partials, total;
  FusedWorkspace(int tokens, int hidden, int inter) {
    const size_t pairs = static_cast<size_t>(tokens) * kTopK;
    auto align = [](size_t n) { return (n + 255) & ~static_cast<size_t>(255); };
    size_t at = 0;
    control = at, at += align(sizeof(Control));
    xdown = at, at += align(pairs * inter * sizeof(__half));
    const size_t gateup = pairs * (inter / 128) * 2 * (hidden / 128) * 128;
    const size_t down = pairs * (hidden / 128) * (inter / 128) * 128;
    partials = at, at += align((gateup + down) * sizeof(float));
    total = at;
  }
};

unsigned long long *g_trace = nullptr; // set by SetFusedDecodeTrace; host-side only

int SmCount() {
  static int cached = 0;
  if (!cached) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
      cached = 0;
  }
  return cached;
}

template <int Rate, int NG> int LaunchFused(FusedArgs &args, cudaStream_t stream) {
  const int sms = SmCount();
  if (sms < 1)
    return PADRA_INTERNAL;
  void *params[] = {&args};
  return CudaStatus(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(FusedDecodeLayerKernel<Rate, NG>), dim3(sms),
                                                dim3(kFusedThreads), params, 0, stream));
}

} // namespace

int SetFusedDecodeTrace(void *buffer, size_t bytes) {
  const int sms = SmCount();
  if (buffer && (sms < 1 || bytes < static_cast<size_t>(sms) * kTraceSlots * sizeof(unsigned long long)))
    return PADRA_INVALID_ARGUMENT;
  g_trace = static_cast<unsigned long long *>(buffer);
  return PADRA_OK;
}

size_t FusedDecodeWorkspaceBytes(int tokens, int hidden, int inter) {
  return FusedWorkspace(tokens, hidden, inter).total;
}

int InitFusedDecodeWorkspace(void *workspace, size_t bytes, cudaStream_t stream) {
  if (!workspace || bytes < sizeof(Control))
    return PADRA_INVALID_ARGUMENT;
  return CudaStatus(cudaMemsetAsync(workspace, 0, sizeof(Control), stream));
}

int LaunchFusedDecodeLayer(const Matrix *matrices, int layer, const int *ids, const float *routing, const float *normalized,
                           float *x, int tokens, int rate, int hidden, int inter, const unsigned short *table,
                           void *workspace, size_t workspace_bytes, int *bad, cudaStream_t stream) {
  if (hidden / 128 > kMaxBlocks || inter / 128 > kMaxBlocks)
    return PADRA_UNSUPPORTED;
  const FusedWorkspace w(tokens, hidden, inter);
  if (workspace_bytes < w.total)
    return PADRA_RESOURCE_EXHAUSTED;
  auto *base = static_cast<unsigned char *>(workspace);
  FusedArgs args{};
  args.matrices = matrices, args.layer = layer, args.ids = ids, args.routing = routing, args.normalized = normalized;
  args.x = x, args.tokens = tokens, args.hidden = hidden, args.inter = inter, args.table = table;
  args.control = reinterpret_cast<Control *>(base + w.control);
  args.xdown = reinterpret_cast<__half *>(base + w.xdown);
  args.partials = reinterpret_cast<float *>(base + w.partials);
  args.bad = bad;
  args.trace = g_trace;
  const bool wide = tokens > 8;
  switch (rate) {
  case 3:
    return wide ? LaunchFused<3, 2>(args, stream) : LaunchFused<3, 1>(args, stream);
  case 4:
    return wide ? LaunchFused<4, 2>(args, stream) : LaunchFused<4, 1>(args, stream);
  case 6:
    return wide ? LaunchFused<6, 2>(args, stream) : LaunchFused<6, 1>(args, stream);
  default:
    return PADRA_UNSUPPORTED;
  }
}

} // namespace padra
