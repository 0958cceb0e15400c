// Prefill: the grouped per-expert projection on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory), with the trellis decode fused into the producer side of the pipeline.
//
// A work item is a tile of up to 128 tokens x 256 outputs (two 128-output blocks) of one expert:
// D[n][o] = sum_k x~[n][k] * W[k][o].  The kernel is persistent: one CTA per SM walks a list of items (token tiles
// sorted by size, dealt out in snake order so that every CTA gets a similar load; the items of one token tile run at the
// same time on neighbouring CTAs and share the tile's activation rows through L2).  The shape is chosen for the two
// things that bound the kernel: an SM pulls 16 KB of activations per 64-input stage for 256 output columns (half the L2
// traffic per MAC of a 256-token x 128-output item), and every producer warp sees all four ring slots.
//   * the weights are the MMA's N side.  Two sets of eight producer warps, one set per output block of the item and one
//     warp per 16-output tile column, read packed words three stages ahead, decode 32 weights per lane in registers
//     (codec.cuh) and store them as 16-byte pieces of 128-byte rows (one row of 64 inputs per output) in the
//     128-byte-swizzled K-major layout: with the lane <-> (row pair, K-step) ownership of the codec the eight lanes of a
//     quarter-warp hit eight different pieces, so neither these stores nor the tensor cores' reads meet bank conflicts.
//   * the tokens are the M side: the expert's transformed activation rows (FP16, written in expert-grouped order by
//     PrefillInputKernel).  One thread of a copy warp fetches a stage's 128 rows x 64 inputs with ONE tensor copy
//     (cp.async.bulk.tensor, 128-byte swizzle, completion counted in bytes on the stage's barrier); the sixteen decoding
//     warps never touch the activations.  (Gathering them with 16-byte cp.async from those warps cost them three times
//     as many cycles per stage as the decode itself.)
//   * a launch may cover two parts (gate and up): their items then form one list and every item picks its part's
//     matrices, tensor map and output.
//   * one elected thread issues tcgen05.mma (M = 128 tokens, N = 256 outputs, K = 16), four per stage, and commits each
//     stage back to the producers; a 4-stage ring of (32 KB weights + 16 KB activations) that runs on across items.
//   * a thread of the four epilogue warps owns one TOKEN row of the accumulator, so the 128-point output Hadamard of
//     each output block runs over the columns it reads from tensor memory: stages d = 1..16 in registers on 32-column
//     pieces (written back in place), stages d = 32, 64 between the four pieces, then svh, BF16 rounding and 16-byte
//     stores to the row of the (token, slot) pair.  No shuffles, no barriers.
//   * the 512 tensor-memory columns hold TWO accumulators of 256 columns: the epilogue drains item i while the
//     producers and the MMA thread already work on item i+1.
// Every wait on an mbarrier is bounded in time: on expiry the CTA raises the sticky error flag, skips the rest of
// its work, frees its tensor memory and leaves.
#include <atomic>
#include <cuda.h>

#include "codec.cuh"
#include "common.cuh"
#include "exchange.cuh"
#include "kernels.cuh"

namespace padra {
namespace {

constexpr int kStages = 4;
constexpr int kStageK = 64;    // inputs per pipeline stage (four K16 steps)
constexpr int kTileM = 128;    // outputs per item (the MMA's N), and token rows per MMA (its M)
constexpr int kMaxTileN = 128; // tokens per item (one MMA token tile)
constexpr int kItemBlocks = 2; // 128-output blocks per item: 256 accumulator columns
constexpr int kStageABytes = kItemBlocks * kTileM * kStageK * 2; // 32 KB of decoded weights
// Activation stage: 128 token rows of 128 bytes (64 inputs), 128-byte swizzle: what one tensor copy delivers and what
// the MMA's operand descriptor (layout SWIZZLE_128B, 1024 bytes per eight-row group) reads.
constexpr int kStageBBytes = kMaxTileN * kStageK * 2; // 16 KB
constexpr int kEpilogueWarps = 4, kProducerSets = 2, kWarpsPerSet = 8; // set b decodes output block b of the item
constexpr int kMmaWarp = kEpilogueWarps;
constexpr int kFirstProducerWarp = kMmaWarp + 1;
constexpr int kCopyWarp = kFirstProducerWarp + kProducerSets * kWarpsPerSet; // one thread of it fetches the activation tiles
constexpr int kPrefillThreads = (kCopyWarp + 1) * 32; // 704
constexpr int kTmemColumns = 512;                   // two accumulators of 256 columns (128 tokens x 256 outputs)
constexpr int kBufferColumns = 256;
constexpr int kMaxPairs = 4096 * kTopK;              // grouped pairs (rows) one call works on
constexpr int kMaxPairIndex = 1 << 20;              // pair indices may be sparse (received rows in per-source regions)
constexpr int kMaxTiles = kExperts + kMaxPairs / kMaxTileN; // sum over experts of ceil(n_e / 256)
constexpr int kAhead = 2;                           // own stages of packed words in flight per producer lane
constexpr unsigned long long kWaitLimitNs = 1000000000ull; // a wait that lasts a second has failed
constexpr int kMaxTokensPrefill = 2048;

#ifdef PADRA_PREFILL_TRACE
__device__ unsigned long long *g_prefill_trace = nullptr; // [stage record][8], CTA 0 only
#define PF_TRACE(record, slot)                                                     \
  do {                                                                             \
    if (g_prefill_trace && blockIdx.x == 0 && (record) < 8192) {                   \
      g_prefill_trace[static_cast<size_t>(record) * 8 + (slot)] = clock64();       \
    }                                                                              \
  } while (0)
#else
#define PF_TRACE(record, slot)
#endif

struct TileInfo {
  int expert, valid, row_base, begin; // begin = index of the tile's first pair inside the expert's group
};

struct PrefillSmem {
  alignas(1024) unsigned char b[kStages][kStageBBytes]; // swizzled tiles want 1024-byte alignment
  alignas(1024) unsigned char a[kStages][kStageABytes];
  alignas(16) float scale[2][kItemBlocks * kTileM]; // svh of the item being drained / the next one
  alignas(8) unsigned long long full[kStages], empty[kStages], accumulator_ready[2], accumulator_free[2];
  TileInfo tile[kMaxTiles], unsorted[kMaxTiles];
  int pairs[2][kMaxTileN]; // (token*8+slot) of the rows of the item being drained / the next one
  int scan[4];
  int from[kMaxRanks]; // return_to_peers: first send row of each source's region
  unsigned tmem_base;
  int abort, tiles, last;
};

struct PrefillArgs {
  const Matrix *matrices;
  int layer, part;
  int parts; // 1, or 2: the launch computes parts `part` and `part + 1` (gate and up) as one list of items
  const int *groups, *counts;
  const __half *transformed; // [pairs][cols] in expert-grouped order
  unsigned short *output;    // [pairs][rows] BF16 bits, pair order
  unsigned short *output_second; // parts == 2: the rows of the second part
  int group_stride; // rows of `groups` per expert = the most pairs one expert can hold
  int pairs_total;  // pairs (rows of `output`) in the call
  int hidden, inter;
  int block_begin, block_count; // the 128-output blocks this launch computes (a launch may take a part of them)
  int *bad;
  // Expert-parallel down projection: the rows do not go to `output` but straight back to the ranks that sent them,
  // into their exchange blocks over NVLink (pair index = source*cap + k -> row from[source] + k of that rank's
  // `returned` area); the CTA that finishes last announces them with the epoch flag.
  int return_to_peers;
  PeerBlocks peers;
  ExchangeLayout layout;
  int rank, world, cap;
  unsigned epoch;
};

__device__ __forceinline__ unsigned SmemAddress(const void *p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void BarrierInit(unsigned long long *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddress(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void BarrierArrive(unsigned long long *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddress(bar)) : "memory");
}
// Bounded wait for the phase of parity `parity`; false if it did not complete in time or the CTA is aborting.
// `backoff` (nanoseconds of sleep after a failed poll) keeps warps with long waits off the issue slots the producers
// need; the MMA thread polls without sleeping.
__device__ __forceinline__ bool BarrierWait(unsigned long long *bar, unsigned parity, const volatile int *abort, unsigned backoff) {
  const unsigned addr = SmemAddress(bar);
  unsigned long long started = 0;
  for (unsigned spins = 0;; ++spins) {
    unsigned done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(addr), "r"(parity)
                 : "memory");
    if (done)
      return true;
    if ((spins & 63u) == 63u) {
      if (*abort)
        return false;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (!started)
        started = now;
      else if (now - started > kWaitLimitNs)
        return false;
    }
    if (backoff)
      __nanosleep(backoff);
  }
}
// K-major with 128-byte swizzle: rows of 128 bytes, eight-row groups 1024 bytes apart; a K16 step inside the 64-input row
// is selected by moving the start address 32 bytes on.  Bits: [0,14) address>>4, [16,30) leading offset>>4 (unused
// here), [32,46) distance between eight-row groups>>4, [46,48) descriptor version 1 (sm_100), [61,64) layout 2 =
// SWIZZLE_128B.
__device__ __forceinline__ unsigned long long SwizzledOperandDescriptor(unsigned smem_address) {
  return static_cast<unsigned long long>((smem_address & 0x3ffffu) >> 4) | (1ull << 16) | (static_cast<unsigned long long>(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// One tile of the 2-D tensor behind `map` (inner coordinate x in elements, a multiple of 8; outer coordinate y) into
// shared memory; its bytes are counted on `bar`.  The CTA is the only reader of the tile.
__device__ __forceinline__ void TensorTileLoad(void *smem, const CUtensorMap *map, int x, int y, unsigned long long *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   SmemAddress(smem)),
               "l"(map), "r"(x), "r"(y), "r"(SmemAddress(bar))
               : "memory");
}
__device__ __forceinline__ void BarrierExpect(unsigned long long *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddress(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ unsigned InstructionDescriptor(int n) {
  // kind::f16: FP32 accumulate (bits 4-5 = 1), A and B FP16 (0), both K-major (0), N>>3 at [17,23), M>>4 at [24,29)
  return (1u << 4) | (static_cast<unsigned>(n >> 3) << 17) | (static_cast<unsigned>(128 >> 4) << 24);
}
__device__ __forceinline__ void MmaSS(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc, bool accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u)
               : "memory");
}
__device__ __forceinline__ void MmaCommit(unsigned long long *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(SmemAddress(bar)) : "memory");
}
// 32 lanes x 32 columns: thread i of the warp gets columns [column, column+32) of its own lane
__device__ __forceinline__ void TmemLoad32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                 "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                 "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                 "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i)
    v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void TmemStore32(unsigned taddr, const float (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
               "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
               "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
               "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
               "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
               "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
               "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
               "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
               "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
               : "memory");
}
// four pieces x 8 columns: v[q][j] = column 32*q + j of the thread's lane, counted from `taddr`
__device__ __forceinline__ void TmemLoad4x8(unsigned taddr, float (&v)[4][8]) {
  unsigned r[4][8];
#pragma unroll
  for (int q = 0; q < 4; ++q)
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[q][0]), "=r"(r[q][1]), "=r"(r[q][2]), "=r"(r[q][3]), "=r"(r[q][4]), "=r"(r[q][5]), "=r"(r[q][6]), "=r"(r[q][7])
                 : "r"(taddr + 32 * q)
                 : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int q = 0; q < 4; ++q)
#pragma unroll
    for (int j = 0; j < 8; ++j)
      v[q][j] = __uint_as_float(r[q][j]);
}


// return_to_peers: every CTA fences its peer stores and draws a ticket; the last one tells the sources that their
// rows have come back.  All threads of the CTA call it.
__device__ __forceinline__ void AnnounceReturn(const PrefillArgs &a, int *last) {
  if (!a.return_to_peers)
    return;
  __threadfence_system();
  __syncthreads();
  unsigned *ticket = reinterpret_cast<unsigned *>(a.peers.base[a.rank] + a.layout.tickets) + 1;
  if (!threadIdx.x)
    *last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (*last && threadIdx.x < a.world) {
    __threadfence_system();
    StoreFlagSystem(reinterpret_cast<unsigned *>(a.peers.base[threadIdx.x] + a.layout.came_back) + a.rank, a.epoch);
    if (!threadIdx.x)
      *ticket = 0;
  }
}

// Item `sequence` of this CTA: tiles sorted by size are dealt out forwards and backwards in turn.
__device__ __forceinline__ int ItemIndex(int sequence) {
  const int g = gridDim.x, c = blockIdx.x;
  return sequence * g + ((sequence & 1) ? g - 1 - c : c);
}

template <int Rate>
__global__ void __launch_bounds__(kPrefillThreads, 1) PrefillGemmKernel(PrefillArgs a, const __grid_constant__ CUtensorMap activations,
                                                                        const __grid_constant__ CUtensorMap activations_second) {
  using L = codec::Lane<Rate>;
  extern __shared__ __align__(16) unsigned char raw_smem[];
  // swizzled tiles want 1024-byte alignment: the launch provides 1024 spare bytes and the struct starts at the next boundary
  PrefillSmem &sm = *reinterpret_cast<PrefillSmem *>(raw_smem + ((1024u - (SmemAddress(raw_smem) & 1023u)) & 1023u));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rows = a.part == 2 ? a.hidden : a.inter, cols = a.part == 2 ? a.inter : a.hidden;
  const int pairs_total = a.pairs_total;
  const int row_blocks = (a.block_count + kItemBlocks - 1) / kItemBlocks; // items per token tile: pairs of output blocks
  const int stages = cols / kStageK;

  // ---- the tile list: every CTA builds the same one ----
  if (tid == 0) {
    sm.abort = *a.bad != 0;
    sm.tiles = 0;
    asm volatile("prefetch.tensormap [%0];" ::"l"(&activations) : "memory");
    if (a.parts == 2)
      asm volatile("prefetch.tensormap [%0];" ::"l"(&activations_second) : "memory");
  }
  if (a.return_to_peers && tid < a.world) {
    const int4 meta = reinterpret_cast<const int4 *>(a.peers.base[a.rank] + a.layout.meta)[tid];
    sm.from[tid] = meta.y;
    if (meta.x < 0 || meta.x > a.cap || meta.y < 0 || meta.y + meta.x > a.cap) {
      Raise(a.bad);
      sm.from[tid] = 0; // stays inside the source's area; the rows are garbage and the flag says so
    }
  }
  __syncthreads();
  int my_count = 0, my_tiles = 0, tile_prefix = 0, pair_prefix = 0;
  if (tid < kExperts) {
    my_count = a.counts[tid];
    if (my_count < 0 || my_count > a.group_stride) {
      Raise(a.bad);
      sm.abort = 1;
      my_count = 0;
    }
    my_tiles = (my_count + kMaxTileN - 1) / kMaxTileN;
    if (my_count) {
      for (int p = 0; p < a.parts; ++p) {
        const Matrix &m = a.matrices[(static_cast<size_t>(a.layer) * kExperts + tid) * 3 + a.part + p];
        if (m.format != FormatOfRate(Rate) || m.rows != rows || m.cols != cols || (cols % 128) || (rows % kTileM) || !m.data || !m.svh || !m.suh) {
          Raise(a.bad);
          sm.abort = 1;
        }
      }
    }
    tile_prefix = my_tiles, pair_prefix = my_count; // inclusive scans inside the warp
#pragma unroll
    for (int d = 1; d < 32; d *= 2) {
      const int t = __shfl_up_sync(0xffffffffu, tile_prefix, d), p = __shfl_up_sync(0xffffffffu, pair_prefix, d);
      if (lane >= d)
        tile_prefix += t, pair_prefix += p;
    }
    if (lane == 31)
      sm.scan[2 * warp] = tile_prefix, sm.scan[2 * warp + 1] = pair_prefix;
  }
  __syncthreads();
  if (tid < kExperts) {
    if (warp == 1)
      tile_prefix += sm.scan[0], pair_prefix += sm.scan[1];
    if (tid == kExperts - 1) {
      sm.tiles = tile_prefix < kMaxTiles ? tile_prefix : kMaxTiles;
      if (pair_prefix > pairs_total || pair_prefix > kMaxPairs || tile_prefix > kMaxTiles) {
        Raise(a.bad);
        sm.abort = 1;
      }
    }
    const int first_tile = tile_prefix - my_tiles, first_pair = pair_prefix - my_count;
    for (int j = 0; j < my_tiles && first_tile + j < kMaxTiles; ++j) { // more tiles only with counts that are rejected above
      TileInfo t;
      t.expert = tid, t.begin = j * kMaxTileN;
      t.valid = my_count - t.begin < kMaxTileN ? my_count - t.begin : kMaxTileN;
      t.row_base = first_pair + t.begin;
      sm.unsorted[first_tile + j] = t;
    }
  }
  __syncthreads();
  const int tiles = sm.tiles;
  if (tid < tiles) { // rank sort, largest tiles first
    const TileInfo mine = sm.unsorted[tid];
    int rank = 0;
    for (int t = 0; t < tiles; ++t) {
      const int v = sm.unsorted[t].valid;
      rank += (v > mine.valid) || (v == mine.valid && t < tid);
    }
    sm.tile[rank] = mine;
  }
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      BarrierInit(&sm.full[s], kProducerSets * kWarpsPerSet + 1); // one arrival per producer warp + the activation copy's
      BarrierInit(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      BarrierInit(&sm.accumulator_ready[b], 1);
      BarrierInit(&sm.accumulator_free[b], kEpilogueWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // item index -> (second part?, token tile, pair of output blocks): the parts' item lists follow one another
  const int items_per_part = tiles * row_blocks, items = items_per_part * a.parts;
  auto second_part = [&](int index) { return index >= items_per_part; };
  auto tile_of = [&](int index) { return (index >= items_per_part ? index - items_per_part : index) / row_blocks; };
  auto block_item_of = [&](int index) { return (index >= items_per_part ? index - items_per_part : index) % row_blocks; };
  if (sm.abort || ItemIndex(0) >= items) { // nothing allocated yet
    AnnounceReturn(a, &sm.last);
    return;
  }
  if (warp == kMmaWarp) { // one warp allocates the accumulator columns and gives the permit back
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddress(&sm.tmem_base)), "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = sm.tmem_base;
  const volatile int *abort = &sm.abort;

  if (warp == kCopyWarp) {
    // =============================== activation copies ===============================
    // One thread runs ahead of everybody by as many stages as the ring has: as soon as a stage's buffers are free it
    // asks for the stage's 128 rows x 64 inputs with one tensor copy, whose bytes complete the stage's `full` barrier.
    if (lane == 0) {
      bool alive = true;
      unsigned q = 0;
      for (int sequence = 0; alive; ++sequence, q += stages) {
        const int index = ItemIndex(sequence);
        if (index >= items)
          break;
        const int row_base = sm.tile[tile_of(index)].row_base;
        const CUtensorMap *map = second_part(index) ? &activations_second : &activations;
        for (int i = 0; i < stages && alive; ++i) {
          const int s = (q + i) % kStages;
          alive = BarrierWait(&sm.empty[s], (((q + i) / kStages) & 1) ^ 1, abort, 64);
          if (!alive)
            break;
          BarrierExpect(&sm.full[s], kStageBBytes);
          // rows past the expert's group are the next group's, or zero past the end of the tensor: they only reach
          // accumulator rows nobody reads
          TensorTileLoad(sm.b[s], map, i * kStageK, row_base, &sm.full[s]);
        }
      }
    }
    __syncwarp();
  } else if (warp >= kFirstProducerWarp) {
    // =============================== producers ===============================
    const int set = (warp - kFirstProducerWarp) / kWarpsPerSet;   // output block of the item this warp decodes
    const int column = (warp - kFirstProducerWarp) % kWarpsPerSet; // 16-output tile column inside the 128-output block
    const int ptid = tid - kFirstProducerWarp * 32; // 0..511
    const int g = lane & 7, kstep = lane >> 3; // row pair, K16 step inside the stage
    const size_t tiles_per_kstep = rows / 16;
    const size_t stage_bytes = static_cast<size_t>(4) * tiles_per_kstep * L::kTileBytes;
    // address of this lane's packed words for stage 0 of an item
    auto lane_base_of = [&](int index) -> const unsigned char * {
      const TileInfo t = sm.tile[tile_of(index)];
      const unsigned char *data = a.matrices[(static_cast<size_t>(a.layer) * kExperts + t.expert) * 3 + a.part + second_part(index)].data;
      int block = a.block_begin + block_item_of(index) * kItemBlocks + set;
      if (block >= a.block_begin + a.block_count)
        block = a.block_begin + a.block_count - 1; // odd block count: the last item has one block, this set idles there
      return data + (static_cast<size_t>(kstep) * tiles_per_kstep + block * 8 + column) * L::kTileBytes + g * L::kBytes;
    };
    // The look-ahead runs through the same (item, stage) sequence as the loop below, kAhead own stages in front of
    // it, across item boundaries; the matrix address of the item after the cursor's is fetched one item early.
    int ahead_sequence = 0, ahead_stage = 0;
    const unsigned char *ahead_base = lane_base_of(ItemIndex(0));
    const unsigned char *ahead_next = ItemIndex(1) < items ? lane_base_of(ItemIndex(1)) : nullptr;
    auto fetch = [&](uint32_t(&into)[Rate]) {
      if (ahead_base)
        codec::LoadWords<Rate>(ahead_base + static_cast<size_t>(ahead_stage) * stage_bytes, into);
      ahead_stage += 1;
      if (ahead_stage >= stages) {
        ahead_stage -= stages;
        ++ahead_sequence;
        ahead_base = ahead_next;
        const int following = ItemIndex(ahead_sequence + 1);
        ahead_next = ahead_base && following < items ? lane_base_of(following) : nullptr;
      }
    };
    uint32_t ahead[kAhead][Rate] = {};
#pragma unroll
    for (int d = 0; d < kAhead; ++d)
      fetch(ahead[d]);
    // where this lane's four 16-byte pieces go inside a weight stage (see the stores below): the same for every stage
    unsigned store_offset[4];
#pragma unroll
    for (int f = 0; f < 4; ++f)
      store_offset[f] = (set * 128 + column * 16 + (f & 1) * 8 + g) * 128 + (((2 * kstep + (f >> 1)) ^ g) << 4);
    bool alive = true;
    unsigned q = 0;        // stages this CTA has been through before the current item
    for (int sequence = 0; alive; ++sequence, q += stages) {
      const int index = ItemIndex(sequence);
      if (index >= items)
        break;
      const bool decodes = block_item_of(index) * kItemBlocks + set < a.block_count; // false: single-block last item
      for (int i = 0; i < stages; ++i) {
        const int s = (q + i) % kStages;
        uint32_t words[Rate];
#pragma unroll
        for (int w = 0; w < Rate; ++w) {
          words[w] = ahead[0][w];
#pragma unroll
          for (int d = 0; d + 1 < kAhead; ++d)
            ahead[d][w] = ahead[d + 1][w];
        }
        fetch(ahead[kAhead - 1]);
        // the stage's buffers are free once the MMAs that read them four stages ago have completed: normally long ago.
        // ONE lane asks (thirty-two lanes polling one barrier word are served one after the other, and that was a third of
        // the stage's time); the warp-wide exchange of its answer also orders the other lanes' stores behind the wait.
        if (lane == 0)
          alive = BarrierWait(&sm.empty[s], (((q + i) / kStages) & 1) ^ 1, abort, 32);
        alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
        if (!alive)
          break;
        if (ptid == 0)
          PF_TRACE(q + i, 0);
        const uint32_t previous = __shfl_sync(0xffffffffu, words[Rate - 1], (lane & 24) | ((lane + 7) & 7));
        uint32_t frag[4][4];
        codec::Decode32<Rate>(words, previous, frag);
        if (ptid == 0)
          PF_TRACE(q + i, 1);
        // weights: this lane's four 16-byte pieces (fragment f: K half f>>1, output row g + 8*(f&1) of the warp's tile
        // column), into the same layout the tensor copies produce: one 128-byte row of 64 inputs per output, eight-row
        // groups of 1024 bytes, the 16-byte piece index XORed with the row's low three bits.  The eight lanes of a quarter
        // warp (g = 0..7, one K16 step) hit eight different pieces: no bank conflicts, for these stores or for the MMA.
        unsigned char *a_stage = sm.a[s];
        if (decodes) {
#pragma unroll
          for (int f = 0; f < 4; ++f) // output row set*128 + column*16 + (f&1)*8 + g of the stage's 256
            *reinterpret_cast<uint4 *>(a_stage + store_offset[f]) = make_uint4(frag[0][f], frag[1][f], frag[2][f], frag[3][f]);
        }
        // publish at once (release); the MMA thread orders these generic-proxy writes before its tensor-core reads
        // with a proxy fence after its wait, so nobody waits here for the copies
        __syncwarp();
        if (lane == 0)
          BarrierArrive(&sm.full[s]);
        if (ptid == 0)
          PF_TRACE(q + i, 2);
      }
    }
  } else if (warp == kMmaWarp) {
    // =============================== MMA issue ===============================
    if (lane == 0) {
      bool alive = true;
      unsigned q = 0;
      for (int sequence = 0; alive; ++sequence, q += stages) {
        const int index = ItemIndex(sequence);
        if (index >= items)
          break;
        const int left = a.block_count - block_item_of(index) * kItemBlocks;
        const unsigned idesc = InstructionDescriptor((left < kItemBlocks ? left : kItemBlocks) * kTileM);
        const int buffer = sequence & 1;
        // the accumulator must have been drained by the epilogue of the item two before
        alive = BarrierWait(&sm.accumulator_free[buffer], ((sequence >> 1) & 1) ^ 1, abort, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int i = 0; i < stages && alive; ++i) {
          const int s = (q + i) % kStages;
          PF_TRACE(q + i, 3);
          alive = BarrierWait(&sm.full[s], ((q + i) / kStages) & 1, abort, 0);
          if (!alive)
            break;
          PF_TRACE(q + i, 4);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // producers' stores and copies -> tensor-core reads
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned w_base = SmemAddress(sm.a[s]), x_base = SmemAddress(sm.b[s]);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const unsigned long long x_desc = SwizzledOperandDescriptor(x_base + ks * 32);
            const unsigned long long w_desc = SwizzledOperandDescriptor(w_base + ks * 32);
            MmaSS(tmem + buffer * kBufferColumns, x_desc, w_desc, idesc, i > 0 || ks > 0);
          }
          MmaCommit(&sm.empty[s]); // arrives when the MMAs above have finished reading the stage
          PF_TRACE(q + i, 5);
        }
        if (alive)
          MmaCommit(&sm.accumulator_ready[buffer]);
      }
      if (!alive) {
        sm.abort = 1;
        Raise(a.bad);
      }
    }
    __syncwarp();
  } else {
    // =============================== epilogue ===============================
    const int o = warp * 32 + lane; // tensor-memory lane of this thread = token row inside a token tile
    for (int sequence = 0;; ++sequence) {
      const int index = ItemIndex(sequence);
      if (index >= items)
        break;
      const TileInfo t = sm.tile[tile_of(index)];
      const int first_block = a.block_begin + block_item_of(index) * kItemBlocks, valid = t.valid, buffer = sequence & 1;
      const int left = a.block_begin + a.block_count - first_block, item_blocks = left < kItemBlocks ? left : kItemBlocks;
      const Matrix &m = a.matrices[(static_cast<size_t>(a.layer) * kExperts + t.expert) * 3 + a.part + second_part(index)];
      unsigned short *const item_output = second_part(index) ? a.output_second : a.output;
      for (int b = 0; b < item_blocks; ++b)
        sm.scale[buffer][b * kTileM + o] = HalfBitsToFloat(m.svh[(first_block + b) * kTileM + o]);
      int *pairs = sm.pairs[buffer];
      for (int n = o; n < valid; n += kEpilogueWarps * 32) {
        const int pair = a.groups[static_cast<size_t>(t.expert) * a.group_stride + t.begin + n];
        pairs[n] = pair;
        if (pair < 0 || pair >= pairs_total) {
          Raise(a.bad);
          sm.abort = 1;
        }
      }
      unsigned failed = 0, any_failed;
      if (!BarrierWait(&sm.accumulator_ready[buffer], (sequence >> 1) & 1, abort, 200)) {
        sm.abort = 1;
        Raise(a.bad);
        failed = 1;
      }
      // pairs[] and scale[] complete, and ONE decision for all four warps
      asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(any_failed)
                   : "r"(failed | static_cast<unsigned>(*abort))
                   : "memory");
      if (any_failed)
        break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // one token row per thread; the item's output blocks are separate 128-point transforms of that row
      for (int b = 0; b < item_blocks && warp * 32 < valid; ++b) { // warp-uniform
        const int n = o, block = first_block + b;
        const float *scale = sm.scale[buffer] + b * kTileM;
        const unsigned lane_address = tmem + buffer * kBufferColumns + b * kTileM + (static_cast<unsigned>(warp * 32) << 16);
        // output Hadamard over the 128 outputs of the row, stages in ascending order like the reference
        // (src/cuda/expert_exl3.cuh:102-109).  Stages d = 1..16 stay inside a 32-column piece:
#pragma unroll 1
        for (int piece = 0; piece < 4; ++piece) {
          float v[32];
          TmemLoad32(lane_address + 32 * piece, v);
#pragma unroll
          for (int d = 1; d < 32; d *= 2)
#pragma unroll
            for (int c = 0; c < 32; ++c)
              if (!(c & d)) {
                const float lower = v[c], upper = v[c + d];
                v[c] = __fadd_rn(lower, upper);
                v[c + d] = __fsub_rn(lower, upper);
              }
          TmemStore32(lane_address + 32 * piece, v);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        // stages d = 32 and 64 combine the four pieces column by column
        unsigned short *out;
        if (a.return_to_peers) {
          const int pair = n < valid ? pairs[n] : 0, source = pair / a.cap;
          out = reinterpret_cast<unsigned short *>(a.peers.base[source] + a.layout.returned) +
                static_cast<size_t>(sm.from[source] + (pair - source * a.cap)) * rows + block * kTileM;
        } else {
          out = item_output + (n < valid ? static_cast<size_t>(pairs[n]) : 0) * rows + block * kTileM;
        }
#pragma unroll 1
        for (int c0 = 0; c0 < 32; c0 += 8) {
          float v[4][8];
          TmemLoad4x8(lane_address + c0, v);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float a0 = __fadd_rn(v[0][j], v[1][j]), a1 = __fsub_rn(v[0][j], v[1][j]);
            const float a2 = __fadd_rn(v[2][j], v[3][j]), a3 = __fsub_rn(v[2][j], v[3][j]);
            v[0][j] = __fadd_rn(a0, a2), v[2][j] = __fsub_rn(a0, a2);
            v[1][j] = __fadd_rn(a1, a3), v[3][j] = __fsub_rn(a1, a3);
          }
          if (n < valid) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              unsigned packed[4], exponents = 0;
#pragma unroll
              for (int j = 0; j < 8; j += 2) {
                // two outputs rounded to BF16 by one conversion; a BF16 with all exponent bits set is not finite
                const __nv_bfloat162 pair = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(v[q][j], kHadamardScale), scale[32 * q + c0 + j]),
                                                                  __fmul_rn(__fmul_rn(v[q][j + 1], kHadamardScale), scale[32 * q + c0 + j + 1]));
                packed[j >> 1] = *reinterpret_cast<const unsigned *>(&pair);
                exponents |= ((packed[j >> 1] & 0x7f80u) == 0x7f80u) | ((packed[j >> 1] & 0x7f800000u) == 0x7f800000u);
              }
              if (exponents)
                Raise(a.bad);
              *reinterpret_cast<uint4 *>(out + 32 * q + c0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
          }
        }
      }
      // hand the accumulator back to the MMA thread
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0)
        BarrierArrive(&sm.accumulator_free[buffer]);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
  }
  AnnounceReturn(a, &sm.last);
}

// x~ rows in expert-grouped order: row (offset of expert e) + i holds the transform of the i-th pair routed to e.
// Parts 0/1: x~ = fp16(B(H128(x[token] * suh)))  (reference: src/cuda/expert_exl3_prefill_warp.cuh:14-57);
// part 2: x = SwiGLU(gate[pair], up[pair]) first (expert_exl3_prefill_packed_activations.cuh:17-73).
// second_offset != 0: the launch transforms the rows for parts `first_part` and `first_part + 1` (gate and up: the same
// input, read once, each part's own signs), the second part's rows `second_offset` halves behind the first's.
__global__ void __launch_bounds__(256) PrefillInputKernel(const Matrix *matrices, int layer, int first_part, const int *groups,
                                                          const int *counts, const float *input, const unsigned short *gate,
                                                          const unsigned short *up, const unsigned short *pair_rows,
                                                          const unsigned short *table, __half *transformed, size_t second_offset,
                                                          int group_stride, int pairs, int hidden, int inter, int format, int *bad) {
  const int part = first_part, parts = second_offset ? 2 : 1;
  __shared__ int s_offset[kExperts + 1], s_half;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cols = part == 2 ? inter : hidden, blocks = cols / 128;
  if (threadIdx.x < kExperts) { // exclusive prefix sum of the 64 group sizes: two warp scans
    int n = counts[threadIdx.x];
    n = (n < 0 || n > group_stride) ? 0 : n;
    int inclusive = n;
#pragma unroll
    for (int d = 1; d < 32; d *= 2) {
      const int other = __shfl_up_sync(0xffffffffu, inclusive, d);
      if (lane >= d)
        inclusive += other;
    }
    if (threadIdx.x == 31)
      s_half = inclusive;
    asm volatile("bar.sync 1, 64;" ::: "memory");
    const int base = warp ? s_half : 0;
    s_offset[threadIdx.x] = base + inclusive - n;
    if (threadIdx.x == kExperts - 1)
      s_offset[kExperts] = base + inclusive;
  }
  __syncthreads();
  if (*bad)
    return;
  // one warp per grouped row: the row's expert, pair and sidecar address are looked up once for all its blocks
  const int grouped_rows = s_offset[kExperts] < kMaxPairs ? s_offset[kExperts] : kMaxPairs; // the workspace holds no more
  for (int row = blockIdx.x * 8 + warp; row < grouped_rows; row += gridDim.x * 8) {
  int expert = 0; // the expert whose group holds grouped row `row`
  for (int step = 32; step; step >>= 1)
    if (expert + step < kExperts && s_offset[expert + step] <= row)
      expert += step;
  const int pair = groups[static_cast<size_t>(expert) * group_stride + (row - s_offset[expert])];
  if (pair < 0 || pair >= pairs) {
    if (!lane)
      Raise(bad);
    continue;
  }
  // the descriptor is checked before anything is read through it: a table of another rate or shape, or a missing
  // sidecar, raises the flag and the row is skipped
  const uint16_t *suh[2] = {nullptr, nullptr};
  bool fits = true;
  for (int p = 0; p < parts; ++p) {
    const Matrix &dm = matrices[(static_cast<size_t>(layer) * kExperts + expert) * 3 + part + p];
    suh[p] = dm.suh;
    fits = fits && dm.format == format && dm.cols == cols && dm.rows == (part == 2 ? hidden : inter) && suh[p] && dm.data;
  }
  if (!fits) {
    if (!lane)
      Raise(bad);
    continue;
  }
#pragma unroll 4
  for (int h = 0; h < blocks; ++h) {
  const int k = h * 128 + lane * 4;
  float src[4];
  if (part == 2) {
    const uint2 gb = *reinterpret_cast<const uint2 *>(gate + static_cast<size_t>(pair) * cols + k);
    const uint2 ub = *reinterpret_cast<const uint2 *>(up + static_cast<size_t>(pair) * cols + k);
    const unsigned short gs[4] = {static_cast<unsigned short>(gb.x & 0xffffu), static_cast<unsigned short>(gb.x >> 16),
                                  static_cast<unsigned short>(gb.y & 0xffffu), static_cast<unsigned short>(gb.y >> 16)};
    const unsigned short us[4] = {static_cast<unsigned short>(ub.x & 0xffffu), static_cast<unsigned short>(ub.x >> 16),
                                  static_cast<unsigned short>(ub.y & 0xffffu), static_cast<unsigned short>(ub.y >> 16)};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gv = FromBF16Bits(gs[j]), uv = FromBF16Bits(us[j]);
      if (!isfinite(gv) || !isfinite(uv)) {
        Raise(bad);
        src[j] = 0.f;
      } else {
        src[j] = RoundBF16(__fmul_rn(FromBF16Bits(__ldg(table + gs[j])), uv));
        if (!isfinite(src[j]))
          Raise(bad);
      }
    }
  } else if (pair_rows) { // one BF16 row per pair (rows received from other ranks)
    const uint2 xb = *reinterpret_cast<const uint2 *>(pair_rows + static_cast<size_t>(pair) * cols + k);
    src[0] = FromBF16Bits(xb.x & 0xffffu), src[1] = FromBF16Bits(xb.x >> 16);
    src[2] = FromBF16Bits(xb.y & 0xffffu), src[3] = FromBF16Bits(xb.y >> 16);
  } else {
    const float4 x = *reinterpret_cast<const float4 *>(input + static_cast<size_t>(pair >> 3) * cols + k);
    src[0] = x.x, src[1] = x.y, src[2] = x.z, src[3] = x.w;
  }
  for (int p = 0; p < parts; ++p) {
    const uint2 sign = __ldg(reinterpret_cast<const uint2 *>(suh[p] + k));
    float v[4] = {__fmul_rn(src[0], HalfBitsToFloat(sign.x & 0xffffu)), __fmul_rn(src[1], HalfBitsToFloat(sign.x >> 16)),
                  __fmul_rn(src[2], HalfBitsToFloat(sign.y & 0xffffu)), __fmul_rn(src[3], HalfBitsToFloat(sign.y >> 16))};
    WarpHadamard128(v);
    __half hv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float r = RoundBF16(v[j]);
      hv[j] = __float2half_rn(r);
      if (!isfinite(r) || (__half_as_ushort(hv[j]) & 0x7c00) == 0x7c00)
        Raise(bad);
    }
    uint2 packed;
    packed.x = static_cast<unsigned>(__half_as_ushort(hv[0])) | (static_cast<unsigned>(__half_as_ushort(hv[1])) << 16);
    packed.y = static_cast<unsigned>(__half_as_ushort(hv[2])) | (static_cast<unsigned>(__half_as_ushort(hv[3])) << 16);
    *reinterpret_cast<uint2 *>(transformed + p * second_offset + static_cast<size_t>(row) * cols + k) = packed;
  }
  }
  }
}

// The tensor map of the transformed activation rows [rows][cols] FP16: tiles of 128 rows x 64 inputs, 128-byte swizzle,
// zeros past the end.  The encoder is a driver entry point, looked up through the runtime (no link against the driver).
int MakeActivationMap(CUtensorMap *map, const void *transformed, int rows, int cols) {
  using Encode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                              const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  void *entry = nullptr;
  cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found) != cudaSuccess || found != cudaDriverEntryPointSuccess ||
      !entry)
    return PADRA_INTERNAL;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * sizeof(__half)};
  const cuuint32_t box[2] = {kStageK, kMaxTileN}, element_strides[2] = {1, 1};
  const CUresult status = reinterpret_cast<Encode>(entry)(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(transformed), dims, strides, box,
                                                          element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return status == CUDA_SUCCESS ? PADRA_OK : PADRA_INTERNAL;
}

template <int Rate> int LaunchGemm(const PrefillArgs &a, const CUtensorMap &map, const CUtensorMap &map_second, dim3 grid, cudaStream_t stream) {
  const size_t smem = sizeof(PrefillSmem) + 1024; // room to start the struct on a 1024-byte boundary
  // set on every launch: the attribute belongs to the current device, and the call is cheap
  if (cudaFuncSetAttribute(PrefillGemmKernel<Rate>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return PADRA_RESOURCE_EXHAUSTED;
  PrefillGemmKernel<Rate><<<grid, kPrefillThreads, smem, stream>>>(a, map, map_second);
  return CudaStatus(cudaGetLastError());
}

} // namespace


// `pair_rows` null: the reference's layout, pairs = tokens*8 and input row pair/8.  Otherwise one BF16 input row per
// pair, any number of pairs per expert up to group_stride (rows that other ranks routed to this rank's experts).
static std::atomic<int> g_reserved_sms{0};
int SetPrefillReservedSms(int sms) {
  if (sms < 0 || sms > 64)
    return PADRA_INVALID_ARGUMENT;
  g_reserved_sms.store(sms, std::memory_order_relaxed);
  return PADRA_OK;
}

struct ReturnSpec {
  const unsigned long long *bases;
  int rank, world, cap;
  unsigned epoch;
};

static int LaunchPrefillGemm(const Matrix *matrices, int layer, int part, const int *groups, const int *counts, const float *input,
                             const unsigned short *pair_rows, unsigned short *output, const unsigned short *gate,
                             const unsigned short *up, const unsigned short *table, void *transformed, int group_stride, int pairs,
                             int *bad, cudaStream_t stream, int rate, int hidden, int inter, const ReturnSpec *ret = nullptr,
                             int block_begin = 0, int block_count = 0, unsigned short *output_second = nullptr) {
  // output_second: gate (part 0) and up (part 1) as ONE list of work items: `transformed` then holds both parts'
  // rows, the second part's behind the first's
  if (output_second && (part != 0 || ret || reinterpret_cast<uintptr_t>(output_second) % 16))
    return PADRA_INVALID_ARGUMENT;
  if (pairs < 1 || pairs > kMaxPairIndex || group_stride < 1 || group_stride > kMaxPairs || !transformed)
    return PADRA_INVALID_ARGUMENT;
  if ((!ret && (!output || reinterpret_cast<uintptr_t>(output) % 16)) || reinterpret_cast<uintptr_t>(transformed) % 16)
    return PADRA_INVALID_ARGUMENT;
  const int all_blocks = (part == 2 ? hidden : inter) / kTileM;
  if (block_count == 0)
    block_begin = 0, block_count = all_blocks;
  if (block_begin < 0 || block_count < 1 || block_begin + block_count > all_blocks)
    return PADRA_INVALID_ARGUMENT;
  // a launch that starts at a later block continues a call whose first launch has filled `transformed` already
  const int cols = part == 2 ? inter : hidden, map_rows = pairs < kMaxPairs ? pairs : kMaxPairs;
  __half *const transformed_second = static_cast<__half *>(transformed) + static_cast<size_t>(map_rows) * cols;
  if (block_begin == 0) {
    PrefillInputKernel<<<(map_rows + 7) / 8, 256, 0, stream>>>(
        matrices, layer, part, groups, counts, input, gate, up, pair_rows, table, static_cast<__half *>(transformed),
        output_second ? static_cast<size_t>(map_rows) * cols : 0, group_stride, pairs, hidden, inter, FormatOfRate(rate), bad);
    if (cudaGetLastError() != cudaSuccess)
      return PADRA_INTERNAL;
  }
  PrefillArgs a{};
  a.matrices = matrices, a.layer = layer, a.part = part, a.groups = groups, a.counts = counts;
  a.transformed = static_cast<const __half *>(transformed), a.output = output, a.group_stride = group_stride;
  a.pairs_total = pairs, a.hidden = hidden, a.inter = inter, a.bad = bad;
  a.block_begin = block_begin, a.block_count = block_count;
  a.parts = output_second ? 2 : 1, a.output_second = output_second;
  if (ret) {
    if (part != 2 || ret->world < 1 || ret->world > kMaxRanks || ret->rank < 0 || ret->rank >= ret->world || ret->cap < 1 ||
        static_cast<long long>(ret->world) * ret->cap != pairs || !ret->bases)
      return PADRA_INVALID_ARGUMENT;
    for (int r = 0; r < kMaxRanks; ++r) {
      a.peers.base[r] = r < ret->world ? reinterpret_cast<unsigned char *>(static_cast<uintptr_t>(ret->bases[r])) : nullptr;
      if (r < ret->world && (!a.peers.base[r] || ret->bases[r] % 256))
        return PADRA_INVALID_ARGUMENT;
    }
    a.return_to_peers = 1, a.layout = MakeExchangeLayout(ret->world, ret->cap, hidden);
    a.rank = ret->rank, a.world = ret->world, a.cap = ret->cap, a.epoch = ret->epoch;
  }
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 1)
    return PADRA_INTERNAL;
  const int reserved = g_reserved_sms.load(std::memory_order_relaxed);
  const dim3 grid(sms - reserved > 0 ? sms - reserved : 1); // persistent: one CTA per SM, less the SMs left to other streams
  CUtensorMap map, map_second;
  if (const int status = MakeActivationMap(&map, transformed, map_rows, cols); status != PADRA_OK)
    return status;
  if (const int status = MakeActivationMap(&map_second, output_second ? transformed_second : transformed, map_rows, cols); status != PADRA_OK)
    return status;
  switch (rate) {
  case 3:
    return LaunchGemm<3>(a, map, map_second, grid, stream);
  case 4:
    return LaunchGemm<4>(a, map, map_second, grid, stream);
  case 6:
    return LaunchGemm<6>(a, map, map_second, grid, stream);
  default:
    return PADRA_UNSUPPORTED;
  }
}

int LaunchPrefillTensorMemory(const Matrix *matrices, int layer, int part, const int *groups, const int *counts, const float *input,
                              unsigned short *output, const unsigned short *gate, const unsigned short *up,
                              const unsigned short *table, void *transformed, int tokens, int *bad, cudaStream_t stream, int rate,
                              int hidden, int inter) {
  if (tokens < 1 || tokens > kMaxTokensPrefill)
    return PADRA_INVALID_ARGUMENT;
  return LaunchPrefillGemm(matrices, layer, part, groups, counts, input, nullptr, output, gate, up, table, transformed, tokens,
                           tokens * kTopK, bad, stream, rate, hidden, inter);
}

int LaunchPrefillGateUp(const Matrix *matrices, int layer, const int *groups, const int *counts, const float *input,
                        unsigned short *gate_output, unsigned short *up_output, void *transformed, int tokens, int *bad, cudaStream_t stream,
                        int rate, int hidden, int inter) {
  if (tokens < 1 || tokens > kMaxTokensPrefill || !up_output)
    return PADRA_INVALID_ARGUMENT;
  return LaunchPrefillGemm(matrices, layer, 0, groups, counts, input, nullptr, gate_output, nullptr, nullptr, nullptr, transformed, tokens,
                           tokens * kTopK, bad, stream, rate, hidden, inter, nullptr, 0, 0, up_output);
}

int LaunchPrefillRowsGateUp(const Matrix *matrices, int layer, const int *groups, const int *counts, int group_stride, int rows,
                            const unsigned short *input_rows, unsigned short *gate_output, unsigned short *up_output, void *transformed,
                            int *bad, cudaStream_t stream, int rate, int hidden, int inter) {
  if (!input_rows || !up_output)
    return PADRA_INVALID_ARGUMENT;
  return LaunchPrefillGemm(matrices, layer, 0, groups, counts, nullptr, input_rows, gate_output, nullptr, nullptr, nullptr, transformed,
                           group_stride, rows, bad, stream, rate, hidden, inter, nullptr, 0, 0, up_output);
}

int LaunchPrefillRows(const Matrix *matrices, int layer, int part, const int *groups, const int *counts, int group_stride, int rows,
                      const unsigned short *input_rows, unsigned short *output, const unsigned short *gate,
                      const unsigned short *up, const unsigned short *table, void *transformed, int *bad, cudaStream_t stream,
                      int rate, int hidden, int inter, int block_begin, int block_count) {
  if (part != 2 && !input_rows)
    return PADRA_INVALID_ARGUMENT;
  return LaunchPrefillGemm(matrices, layer, part, groups, counts, nullptr, input_rows, output, gate, up, table, transformed,
                           group_stride, rows, bad, stream, rate, hidden, inter, nullptr, block_begin, block_count);
}

// The down projection of received rows with its results stored straight into the source ranks' exchange blocks.
int LaunchPrefillDownReturn(const Matrix *matrices, int layer, const int *groups, const int *counts, int group_stride,
                            const unsigned short *gate, const unsigned short *up, const unsigned short *table, void *transformed,
                            const unsigned long long *bases, int rank, int world, int cap, unsigned epoch, int *bad, cudaStream_t stream,
                            int rate, int hidden, int inter) {
  if (world < 1 || cap < 1)
    return PADRA_INVALID_ARGUMENT;
  const ReturnSpec ret{bases, rank, world, cap, epoch};
  return LaunchPrefillGemm(matrices, layer, 2, groups, counts, nullptr, nullptr, nullptr, gate, up, table, transformed, group_stride,
                           world * cap, bad, stream, rate, hidden, inter, &ret);
}

} // namespace padra

#ifdef PADRA_PREFILL_TRACE
extern "C" __attribute__((visibility("default"))) int padra_debug_set_prefill_trace(unsigned long long *buffer) {
  return static_cast<int>(cudaMemcpyToSymbol(padra::g_prefill_trace, &buffer, sizeof(buffer)));
}
#endif
