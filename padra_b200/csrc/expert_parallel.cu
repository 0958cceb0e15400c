// Expert-parallel prefill: the device-side pieces around the all-to-all exchange.
//
// With the 64 experts of a layer spread over N GPUs, a rank (1) packs the activation row of every (token, slot) pair
// into BF16 rows ordered by destination rank, (2) exchanges them (NCCL all-to-all, host side), (3) groups the rows
// it received by expert and runs the grouped projections on them (prefill.cu, one input row per pair), (4) sends the
// down rows back, and (5) combines them with the routing weights, reading each pair's row through an index map so
// that no un-permute pass over the rows is needed.  Arithmetic is that of the single-GPU path: rows cross the wire as
// BF16, which is exactly what the projections' inputs and outputs hold.
//
// Two forms of the exchange exist.  The host can run it (all_to_all_single of packed rows), or the GPUs do it
// themselves over NVLink peer memory: every rank owns an exchange block that all ranks have mapped, the dispatch
// kernel converts a pair's activation row to BF16 and stores it straight into the owner rank's block (into the region
// reserved for this source rank, so no offsets have to be agreed first), and the return kernel stores the down rows
// straight back into the source's block at the rows it sent them from.  Arrival is announced with one flag per
// (source, destination) that carries the call's epoch, written after a system-scope fence by the last CTA of the
// sending kernel; a one-CTA wait kernel on the receiving side polls its own flags, bounded in time.  Nothing in this
// form touches the host: row counts stay on the device, next to the flags.
#include <atomic>

#include "common.cuh"
#include "exchange.cuh"
#include "kernels.cuh"

namespace padra {
namespace {

constexpr int kMaxRows = 4096 * kTopK; // rows one grouped-projection call takes (received rows may exceed a rank's own)

// Expert-major row lists for rows that carry their expert id (received rows): one CTA per expert; thread t owns the
// consecutive rows [t*per, (t+1)*per), counts its matches, one scan over the CTA gives every thread its first position,
// then it writes -- lists are stable in row order.  `ids` are expert ids 0..63 per row; experts this rank does not own
// simply get no rows.  (The same form as GroupKernel in schedule.cu and GroupRegionsKernel below.)
__global__ void __launch_bounds__(256) GroupRowsKernel(const int *ids, int *groups, int *counts, int rows, int stride, int *bad) {
  const int expert = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __shared__ int warp_counts[8], warp_offsets[8], total;
  const int per = (rows + 255) / 256, first = threadIdx.x * per, last = first + per < rows ? first + per : rows;
  int mine = 0;
  for (int row = first; row < last; ++row) {
    const int id = ids[row];
    if ((id < 0 || id >= kExperts) && expert == 0)
      Raise(bad);
    mine += id == expert;
  }
  int inclusive = mine;
#pragma unroll
  for (int d = 1; d < 32; d *= 2) {
    const int other = __shfl_up_sync(0xffffffffu, inclusive, d);
    if (lane >= d)
      inclusive += other;
  }
  if (lane == 31)
    warp_counts[warp] = inclusive;
  __syncthreads();
  if (!threadIdx.x) {
    int n = 0;
    for (int w = 0; w < 8; ++w) {
      warp_offsets[w] = n;
      n += warp_counts[w];
    }
    total = n;
  }
  __syncthreads();
  int at = warp_offsets[warp] + inclusive - mine;
  for (int row = first; row < last && mine; ++row)
    if (ids[row] == expert) {
      if (at < stride)
        groups[static_cast<size_t>(expert) * stride + at] = row;
      ++at;
    }
  if (!threadIdx.x) {
    if (total > stride)
      Raise(bad);
    counts[expert] = total < stride ? total : stride;
  }
}

// The send plan of one rank, one CTA: a stable counting sort of the pairs by destination rank owner[ids[pair]].
// An owner entry may name two ranks (rank | (1 + second rank) << 8) for an expert whose weights two ranks hold: the
// pairs of even tokens go to the first, those of odd tokens to the second, which halves the load of a very popular expert.
//   order[j]      pair that travels as row j          position[pair]  row at which the pair's result comes back
//   send_ids[j]   expert id of row j                  send_counts[r]  rows for rank r (64-bit, as the host API wants)
// Thread t owns the 16 consecutive pairs from 16*t on; a scan over (destination, thread) keeps the order stable.
__global__ void __launch_bounds__(1024) PlanKernel(const int *ids, const int *owner, int *order, int *position, int *send_ids,
                                                   long long *send_counts, int pairs, int world, int *bad) {
  __shared__ int s_owner[kExperts], s_warp_total[kMaxRanks][32], s_base[kMaxRanks + 1];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5, per = (pairs + 1023) / 1024, first = t * per;
  if (t < kExperts)
    s_owner[t] = owner[t];
  __syncthreads();
  // the thread's pairs: at most 16 (2048 tokens), fetched up front so that the loads overlap
  constexpr int kPer = 16;
  int dest[kPer], expert[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int pair = first + i;
    expert[i] = (i < per && pair < pairs) ? ids[pair] : -1;
  }
  int mine[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    mine[r] = 0;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = expert[i];
    int r = (e >= 0 && e < kExperts) ? s_owner[e] : -1;
    if (r >= 0) { // low byte: the expert's rank; next byte: 1 + the rank of a second copy, which takes the odd tokens' pairs
      const int second = (r >> 8) & 0xff;
      r = (second && (((first + i) >> 3) & 1)) ? second - 1 : (r & 0xff);
    }
    if ((i < per && first + i < pairs) && (r < 0 || r >= world)) {
      Raise(bad);
      r = -1;
    }
    dest[i] = r;
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q)
      mine[q] += (q == r);
  }
  // exclusive scan over the 1024 threads, all destinations at once: inside the warp with shuffles, across the warps
  // through the warps' totals
  int before[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r) {
    int inclusive = mine[r];
#pragma unroll
    for (int d = 1; d < 32; d *= 2) {
      const int other = __shfl_up_sync(0xffffffffu, inclusive, d);
      if (lane >= d)
        inclusive += other;
    }
    before[r] = inclusive - mine[r];
    if (lane == 31)
      s_warp_total[r][warp] = inclusive;
  }
  __syncthreads();
  if (warp < kMaxRanks) { // warp r turns the 32 warp totals of destination r into exclusive prefixes
    const int total = s_warp_total[warp][lane];
    int inclusive = total;
#pragma unroll
    for (int d = 1; d < 32; d *= 2) {
      const int other = __shfl_up_sync(0xffffffffu, inclusive, d);
      if (lane >= d)
        inclusive += other;
    }
    s_warp_total[warp][lane] = inclusive - total;
    if (lane == 31)
      s_base[warp] = inclusive; // rows for destination `warp`, turned into first rows below
  }
  __syncthreads();
  if (t == 0) {
    int sum = 0;
    for (int r = 0; r < kMaxRanks; ++r) {
      const int n = r < world ? s_base[r] : 0;
      if (r < world)
        send_counts[r] = n;
      s_base[r] = sum;
      sum += n;
    }
    s_base[kMaxRanks] = sum;
  }
  __syncthreads();
  int cursor[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    cursor[r] = s_base[r] + s_warp_total[r][warp] + before[r];
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int pair = first + i, r = dest[i];
    if (i < per && pair < pairs) {
      int at = 0;
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q)
        if (q == r)
          at = cursor[q]++;
      if (r >= 0)
        order[at] = pair, send_ids[at] = expert[i];
      position[pair] = r >= 0 ? at : 0;
    }
  }
}

// packed[j] = BF16 bits of activations[order[j] / 8]: order[j] is the (token*8+slot) pair that travels as row j.
__global__ void __launch_bounds__(256) PackRowsKernel(const float *activations, const int *order, unsigned short *packed, int rows,
                                                      int hidden, int *bad) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const int pair = order[row];
    if (pair < 0 || pair >= rows) {
      if (!lane)
        Raise(bad);
      continue;
    }
    const float *from = activations + static_cast<size_t>(pair >> 3) * hidden;
    unsigned short *to = packed + static_cast<size_t>(row) * hidden;
    for (int k = lane * 4; k < hidden; k += 128) {
      const float4 v = *reinterpret_cast<const float4 *>(from + k);
      uint2 bits;
      bits.x = static_cast<unsigned>(BF16Bits(v.x)) | (static_cast<unsigned>(BF16Bits(v.y)) << 16);
      bits.y = static_cast<unsigned>(BF16Bits(v.z)) | (static_cast<unsigned>(BF16Bits(v.w)) << 16);
      *reinterpret_cast<uint2 *>(to + k) = bits;
    }
  }
}

// The combine of src/cuda/expert_exl3_prefill_packed_activations.cuh:86-103 with the down row of pair p found at
// down_rows[position[p]]: x[t] = B(x[t] + sum), sum = B(sum + B(down * w)) over the eight slots in order.
__global__ void __launch_bounds__(128) CombineIndexedKernel(float *x, const unsigned short *down_rows, const int *position,
                                                            const float *weights, int tokens, int hidden, int *bad, bool residual) {
  const int token = blockIdx.y, col = (blockIdx.x * blockDim.x + threadIdx.x) * 4; // four columns per thread
  if (token >= tokens || col >= hidden)
    return;
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < kTopK; ++s) {
    const int at = position[token * kTopK + s];
    if (at < 0 || at >= tokens * kTopK) {
      Raise(bad);
      return;
    }
    const uint2 bits = *reinterpret_cast<const uint2 *>(down_rows + static_cast<size_t>(at) * hidden + col);
    const float w = weights[token * kTopK + s];
    const float d[4] = {FromBF16Bits(bits.x & 0xffffu), FromBF16Bits(bits.x >> 16), FromBF16Bits(bits.y & 0xffffu),
                        FromBF16Bits(bits.y >> 16)};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      sum[j] = RoundBF16(__fadd_rn(sum[j], RoundBF16(__fmul_rn(d[j], w))));
  }
  float4 *target = reinterpret_cast<float4 *>(x + static_cast<size_t>(token) * hidden + col);
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

// ---- the exchange over peer memory (block layout and flag helpers: exchange.cuh) ------------------------------
// Fused pack + dispatch: send row j (pair order[j]) goes to rank d = the destination whose range of the send order
// holds j, as row rank*cap + (j - first row for d) of d's block.
__global__ void __launch_bounds__(256) DispatchKernel(const float *activations, const int *order, const int *send_ids,
                                                      const long long *send_counts, PeerBlocks peers, ExchangeLayout layout, int rank,
                                                      int world, int cap, int pairs, int hidden, unsigned epoch, int *bad) {
  __shared__ int s_first[kMaxRanks + 1], s_ok, s_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (!threadIdx.x) {
    int sum = 0, ok = 1;
    for (int d = 0; d < world; ++d) {
      const long long c = send_counts[d];
      s_first[d] = sum;
      if (c < 0 || c > cap)
        ok = 0;
      else
        sum += static_cast<int>(c);
    }
    s_first[world] = sum;
    s_ok = ok && sum == pairs;
    if (!s_ok)
      Raise(bad);
  }
  __syncthreads();
  if (s_ok) {
    // every rank starts with the rows of its right-hand neighbour and walks round the ring, so that the ranks do not
    // all store into the same destination at the same time
    const int start = s_first[(rank + 1) % world];
    for (int turn = blockIdx.x * 8 + warp; turn < pairs; turn += gridDim.x * 8) {
      const int row = turn + start < pairs ? turn + start : turn + start - pairs;
      int d = 0;
      while (d + 1 < world && s_first[d + 1] <= row)
        ++d;
      const int pair = order[row];
      if (pair < 0 || pair >= pairs) {
        if (!lane)
          Raise(bad);
        continue;
      }
      const size_t slot = static_cast<size_t>(rank) * cap + (row - s_first[d]);
      const float *from = activations + static_cast<size_t>(pair >> 3) * hidden;
      unsigned short *to = reinterpret_cast<unsigned short *>(peers.base[d] + layout.rows) + slot * hidden;
      for (int k0 = lane * 8; k0 < hidden; k0 += 1024) { // four 16-byte pieces per lane in flight
        float4 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int k = k0 + 256 * u;
          if (k < hidden)
            a[u] = *reinterpret_cast<const float4 *>(from + k), b[u] = *reinterpret_cast<const float4 *>(from + k + 4);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int k = k0 + 256 * u;
          if (k < hidden) {
            uint4 bits;
            bits.x = static_cast<unsigned>(BF16Bits(a[u].x)) | (static_cast<unsigned>(BF16Bits(a[u].y)) << 16);
            bits.y = static_cast<unsigned>(BF16Bits(a[u].z)) | (static_cast<unsigned>(BF16Bits(a[u].w)) << 16);
            bits.z = static_cast<unsigned>(BF16Bits(b[u].x)) | (static_cast<unsigned>(BF16Bits(b[u].y)) << 16);
            bits.w = static_cast<unsigned>(BF16Bits(b[u].z)) | (static_cast<unsigned>(BF16Bits(b[u].w)) << 16);
            *reinterpret_cast<uint4 *>(to + k) = bits;
          }
        }
      }
      if (!lane)
        reinterpret_cast<int *>(peers.base[d] + layout.ids)[slot] = send_ids[row];
    }
  }
  // every CTA's stores are fenced before its ticket; the CTA that draws the last ticket announces the rows
  __threadfence_system();
  __syncthreads();
  unsigned *ticket = reinterpret_cast<unsigned *>(peers.base[rank] + layout.tickets);
  if (!threadIdx.x)
    s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last && threadIdx.x < world) {
    const int d = threadIdx.x;
    int4 meta;
    meta.x = s_ok ? s_first[d + 1] - s_first[d] : 0, meta.y = s_first[d], meta.z = 0, meta.w = 0;
    *reinterpret_cast<int4 *>(peers.base[d] + layout.meta + static_cast<size_t>(rank) * 16) = meta;
    __threadfence_system();
    StoreFlagSystem(reinterpret_cast<unsigned *>(peers.base[d] + layout.arrived) + rank, epoch);
    if (!d)
      *ticket = 0;
  }
}

// Poll `world` flags of this rank's own block until each carries `epoch`; give up after limit_ns (the kernel then raises the
// error flag and returns: the stream goes on, the context stays usable).
__global__ void WaitFlagsKernel(const unsigned *flags, int world, unsigned epoch, int *bad, unsigned long long limit_ns) {
  if (threadIdx.x >= world)
    return;
  unsigned long long started;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(started));
  while (LoadFlagSystem(flags + threadIdx.x) != epoch) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - started > limit_ns) {
      Raise(bad);
      break;
    }
    __nanosleep(200);
  }
}

// GroupRowsKernel over the regions of the exchange block: region s holds meta[s].x rows.
__global__ void __launch_bounds__(256) GroupRegionsKernel(const int *ids, const int4 *meta, int world, int cap, int *groups, int *counts,
                                                          int stride, int *bad) {
  const int expert = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __shared__ int s_first[kMaxRanks + 1], warp_counts[8], warp_offsets[8], total;
  if (!threadIdx.x) {
    int sum = 0;
    for (int s = 0; s < world; ++s) {
      int n = meta[s].x;
      if (n < 0 || n > cap) {
        if (!expert)
          Raise(bad);
        n = 0;
      }
      s_first[s] = sum;
      sum += n;
    }
    s_first[world] = sum;
  }
  __syncthreads();
  // the valid rows of all regions, in region order, form one list; thread t owns a contiguous piece of it
  const int valid = s_first[world], per = (valid + 255) / 256;
  const int first = threadIdx.x * per, last = first + per < valid ? first + per : valid;
  int region = 0;
  while (region + 1 < world && s_first[region + 1] <= first)
    ++region;
  int mine = 0;
  for (int v = first, s = region; v < last; ++v) {
    while (s + 1 < world && s_first[s + 1] <= v)
      ++s;
    const int id = ids[s * cap + (v - s_first[s])];
    if ((id < 0 || id >= kExperts) && !expert)
      Raise(bad);
    mine += id == expert;
  }
  int inclusive = mine;
#pragma unroll
  for (int d = 1; d < 32; d *= 2) {
    const int other = __shfl_up_sync(0xffffffffu, inclusive, d);
    if (lane >= d)
      inclusive += other;
  }
  if (lane == 31)
    warp_counts[warp] = inclusive;
  __syncthreads();
  if (!threadIdx.x) {
    int n = 0;
    for (int w = 0; w < 8; ++w) {
      warp_offsets[w] = n;
      n += warp_counts[w];
    }
    total = n;
  }
  __syncthreads();
  int at = warp_offsets[warp] + inclusive - mine;
  for (int v = first, s = region; v < last && mine; ++v) {
    while (s + 1 < world && s_first[s + 1] <= v)
      ++s;
    const int row = s * cap + (v - s_first[s]);
    if (ids[row] == expert) {
      if (at < stride)
        groups[static_cast<size_t>(expert) * stride + at] = row;
      ++at;
    }
  }
  if (!threadIdx.x) {
    if (total > stride)
      Raise(bad);
    counts[expert] = total < stride ? total : stride;
  }
}

// The down rows of region s go back to rank s, to the send rows they came from.
__global__ void __launch_bounds__(256) ReturnKernel(const unsigned short *down, PeerBlocks peers, ExchangeLayout layout, int rank, int world,
                                                    int cap, int hidden, unsigned epoch, int *bad, int column_begin, int column_count,
                                                    int announce) {
  __shared__ int s_first[kMaxRanks + 1], s_from[kMaxRanks], s_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (!threadIdx.x) {
    const int4 *meta = reinterpret_cast<const int4 *>(peers.base[rank] + layout.meta);
    int sum = 0;
    for (int s = 0; s < world; ++s) {
      int n = meta[s].x;
      if (n < 0 || n > cap || meta[s].y < 0 || meta[s].y + n > cap) {
        Raise(bad);
        n = 0;
      }
      s_first[s] = sum, s_from[s] = meta[s].y;
      sum += n;
    }
    s_first[world] = sum;
  }
  __syncthreads();
  const int total = s_first[world], start = s_first[(rank + 1) % world]; // ring order, like the dispatch
  for (int turn = blockIdx.x * 8 + warp; turn < total; turn += gridDim.x * 8) {
    const int item = turn + start < total ? turn + start : turn + start - total;
    int s = 0;
    while (s + 1 < world && s_first[s + 1] <= item)
      ++s;
    const int k = item - s_first[s];
    const uint4 *from = reinterpret_cast<const uint4 *>(down + (static_cast<size_t>(s) * cap + k) * hidden + column_begin);
    uint4 *to = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned short *>(peers.base[s] + layout.returned) +
                                          static_cast<size_t>(s_from[s] + k) * hidden + column_begin);
    for (int c0 = lane; c0 < column_count / 8; c0 += 128) { // four 16-byte pieces per lane in flight
      uint4 piece[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + 32 * u < column_count / 8)
          piece[u] = from[c0 + 32 * u];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c0 + 32 * u < column_count / 8)
          to[c0 + 32 * u] = piece[u];
    }
  }
  if (!announce) // a later launch on the same stream sends the rest of the columns and raises the flags
    return;
  __threadfence_system();
  __syncthreads();
  unsigned *ticket = reinterpret_cast<unsigned *>(peers.base[rank] + layout.tickets) + 1;
  if (!threadIdx.x)
    s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last && threadIdx.x < world) {
    StoreFlagSystem(reinterpret_cast<unsigned *>(peers.base[threadIdx.x] + layout.came_back) + rank, epoch);
    if (!threadIdx.x)
      *ticket = 0;
  }
}

bool FillPeers(PeerBlocks &peers, const unsigned long long *bases, int world) {
  for (int r = 0; r < kMaxRanks; ++r) {
    peers.base[r] = r < world ? reinterpret_cast<unsigned char *>(static_cast<uintptr_t>(bases[r])) : nullptr;
    if (r < world && (!peers.base[r] || bases[r] % 256))
      return false;
  }
  return true;
}

} // namespace

// How long padra_ep_wait's kernel polls before it gives up (host setting, default kFlagWaitNs).
static std::atomic<unsigned long long> g_flag_wait_ns{kFlagWaitNs};
int SetExchangeWaitLimit(int milliseconds) {
  if (milliseconds < 1 || milliseconds > 60000)
    return PADRA_INVALID_ARGUMENT;
  g_flag_wait_ns.store(static_cast<unsigned long long>(milliseconds) * 1000000ull);
  return PADRA_OK;
}

// SMs of the current device (asked every time: a process may drive several devices).
static int SmCount() {
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 1)
    return 132; // a floor that any part this library runs on exceeds
  return sms;
}

size_t ExchangeBytes(int world, int cap, int hidden, size_t *offsets) {
  if (world < 1 || world > kMaxRanks || cap < 8 || cap > 2048 * kTopK || hidden < 128 || (hidden % 128))
    return 0;
  const ExchangeLayout l = MakeExchangeLayout(world, cap, hidden);
  if (offsets)
    offsets[0] = l.rows, offsets[1] = l.ids, offsets[2] = l.meta, offsets[3] = l.returned, offsets[4] = l.arrived, offsets[5] = l.came_back;
  return l.total;
}

int LaunchDispatch(const float *activations, const int *order, const int *send_ids, const long long *send_counts,
                   const unsigned long long *bases, int rank, int world, int cap, int pairs, int hidden, unsigned epoch, int *bad,
                   cudaStream_t stream) {
  PeerBlocks peers;
  if (!activations || !order || !send_ids || !send_counts || !bases || !bad || rank < 0 || rank >= world || pairs < 8 ||
      pairs > cap || !ExchangeBytes(world, cap, hidden, nullptr) || !FillPeers(peers, bases, world) ||
      reinterpret_cast<uintptr_t>(activations) % 16)
    return PADRA_INVALID_ARGUMENT;
  const int blocks = (pairs + 7) / 8;
  DispatchKernel<<<blocks < SmCount() * 4 ? blocks : SmCount() * 4, 256, 0, stream>>>(activations, order, send_ids, send_counts, peers,
                                                                          MakeExchangeLayout(world, cap, hidden), rank, world, cap, pairs,
                                                                          hidden, epoch, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchWaitFlags(const void *block, int which, int world, int cap, int hidden, unsigned epoch, int *bad, cudaStream_t stream) {
  if (!block || !bad || (which != 0 && which != 1) || !ExchangeBytes(world, cap, hidden, nullptr))
    return PADRA_INVALID_ARGUMENT;
  const ExchangeLayout l = MakeExchangeLayout(world, cap, hidden);
  WaitFlagsKernel<<<1, 32, 0, stream>>>(
      reinterpret_cast<const unsigned *>(static_cast<const unsigned char *>(block) + (which ? l.came_back : l.arrived)), world, epoch, bad,
      g_flag_wait_ns.load());
  return CudaStatus(cudaGetLastError());
}

int LaunchGroupRegions(const void *block, int world, int cap, int hidden, int *groups, int *counts, int group_stride, int *bad,
                       cudaStream_t stream) {
  if (!block || !groups || !counts || !bad || group_stride < 1 || !ExchangeBytes(world, cap, hidden, nullptr))
    return PADRA_INVALID_ARGUMENT;
  const ExchangeLayout l = MakeExchangeLayout(world, cap, hidden);
  const unsigned char *base = static_cast<const unsigned char *>(block);
  GroupRegionsKernel<<<kExperts, 256, 0, stream>>>(reinterpret_cast<const int *>(base + l.ids), reinterpret_cast<const int4 *>(base + l.meta),
                                                   world, cap, groups, counts, group_stride, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchReturn(const unsigned short *down, const unsigned long long *bases, int rank, int world, int cap, int hidden, unsigned epoch,
                 int *bad, cudaStream_t stream, int column_begin, int column_count, int announce) {
  PeerBlocks peers;
  if (column_count == 0)
    column_begin = 0, column_count = hidden;
  if (!down || !bases || !bad || rank < 0 || rank >= world || !ExchangeBytes(world, cap, hidden, nullptr) ||
      !FillPeers(peers, bases, world) || reinterpret_cast<uintptr_t>(down) % 16 || column_begin < 0 || column_count < 8 ||
      (column_begin % 8) || (column_count % 8) || column_begin + column_count > hidden)
    return PADRA_INVALID_ARGUMENT;
  ReturnKernel<<<SmCount() * 4, 256, 0, stream>>>(down, peers, MakeExchangeLayout(world, cap, hidden), rank, world, cap, hidden, epoch, bad,
                                            column_begin, column_count, announce);
  return CudaStatus(cudaGetLastError());
}

int LaunchGroupRows(const int *ids, int *groups, int *counts, int rows, int group_stride, int *bad, cudaStream_t stream) {
  if (!ids || !groups || !counts || !bad || rows < 1 || rows > kMaxRows || group_stride < 1 || group_stride > rows)
    return PADRA_INVALID_ARGUMENT;
  GroupRowsKernel<<<kExperts, 256, 0, stream>>>(ids, groups, counts, rows, group_stride, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchPlan(const int *ids, const int *owner, int *order, int *position, int *send_ids, long long *send_counts, int pairs,
               int world, int *bad, cudaStream_t stream) {
  if (!ids || !owner || !order || !position || !send_ids || !send_counts || !bad || pairs < 1 || pairs > 16 * 1024 ||
      world < 1 || world > kMaxRanks)
    return PADRA_INVALID_ARGUMENT;
  PlanKernel<<<1, 1024, 0, stream>>>(ids, owner, order, position, send_ids, send_counts, pairs, world, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchPackRows(const float *activations, const int *order, unsigned short *packed, int rows, int hidden, int *bad,
                   cudaStream_t stream) {
  if (!activations || !order || !packed || !bad || rows < 8 || (rows % kTopK) || hidden < 128 || (hidden % 128) ||
      reinterpret_cast<uintptr_t>(activations) % 16 || reinterpret_cast<uintptr_t>(packed) % 8)
    return PADRA_INVALID_ARGUMENT;
  const int blocks = (rows + 7) / 8;
  PackRowsKernel<<<blocks < SmCount() * 16 ? blocks : SmCount() * 16, 256, 0, stream>>>(activations, order, packed, rows, hidden, bad);
  return CudaStatus(cudaGetLastError());
}

int LaunchCombineIndexed(float *x, const unsigned short *down_rows, const int *position, const float *weights, int tokens,
                         int *bad, int residual, int hidden, cudaStream_t stream) {
  if (!x || !down_rows || !position || !weights || !bad || tokens < 1 || hidden < 4 || (hidden % 4) ||
      reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(down_rows) % 8)
    return PADRA_INVALID_ARGUMENT;
  CombineIndexedKernel<<<dim3((hidden / 4 + 127) / 128, tokens), 128, 0, stream>>>(x, down_rows, position, weights, tokens, hidden, bad,
                                                                                residual != 0);
  return CudaStatus(cudaGetLastError());
}

} // namespace padra
