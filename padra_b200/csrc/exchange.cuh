// The exchange block of expert-parallel prefill: layout, peer table and the system-scope flag accesses, shared by the
// exchange kernels (expert_parallel.cu) and the grouped GEMM, whose down projection can store its rows straight into the
// source ranks' blocks (prefill.cu).
#pragma once
#include "common.cuh"

namespace padra {

constexpr int kMaxRanks = 8;

struct ExchangeLayout {
  size_t rows, ids, meta, returned, arrived, came_back, tickets, total;
};
// One block per rank: rows/ids = what others sent me, region s (cap rows) for source rank s; meta[s] = {rows source s
// sent me, the send row its first row came from}; returned = the down rows of MY pairs, in my send order;
// arrived[s] / came_back[d] = epoch flags written by peers; tickets = two CTA counters of my own kernels.
__host__ __device__ inline ExchangeLayout MakeExchangeLayout(int world, int cap, int hidden) {
  ExchangeLayout l{};
  size_t at = 0;
#define PADRA_ALIGN_256(n) (((n) + 255) & ~static_cast<size_t>(255))
  l.rows = at, at += PADRA_ALIGN_256(static_cast<size_t>(world) * cap * hidden * 2);
  l.ids = at, at += PADRA_ALIGN_256(static_cast<size_t>(world) * cap * 4);
  l.meta = at, at += PADRA_ALIGN_256(static_cast<size_t>(world) * 16);
  l.returned = at, at += PADRA_ALIGN_256(static_cast<size_t>(cap) * hidden * 2);
  l.arrived = at, at += PADRA_ALIGN_256(static_cast<size_t>(world) * 4);
  l.came_back = at, at += PADRA_ALIGN_256(static_cast<size_t>(world) * 4);
#undef PADRA_ALIGN_256
  l.tickets = at, at += 256;
  l.total = at;
  return l;
}

struct PeerBlocks {
  unsigned char *base[kMaxRanks];
};

constexpr unsigned long long kFlagWaitNs = 2000000000ull;

__device__ __forceinline__ void StoreFlagSystem(unsigned *flag, unsigned value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}
__device__ __forceinline__ unsigned LoadFlagSystem(const unsigned *flag) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  return v;
}


} // namespace padra
