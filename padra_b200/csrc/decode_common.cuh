// Pieces shared by the decode-layer kernels (decode_layer.cu: several tokens; decode_single.cu: one token).
#pragma once
#include <cstdlib>

#include "codec.cuh"
#include "common.cuh"
#include "kernels.cuh"

namespace padra {
namespace decode {

constexpr int kThreads = 256;
constexpr int kMaxSlices = 8;
constexpr int kMaxBlocks = 64; // 128-wide blocks per dimension the ticket area provides for

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
__device__ __forceinline__ void LetSuccessorLaunch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void WaitForPredecessor() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
// A hint: fetch `bytes` (a multiple of 16, from a 16-byte aligned address) into L2.  Nothing waits for it.
__device__ __forceinline__ void PrefetchL2(const void *p, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ int LoadFlag(const int *p) { // never from a stale L1 line
  return __ldcg(p);
}

// Place of element k of a row (k counted from the start of the row or slice) in the order the B fragments are read:
// inside every K16 step, input i sits at codec::PermutedInput(i).
__device__ __forceinline__ int PermutedPlace(int k) {
  return (k & ~15) + codec::PermutedInput(k & 15);
}


// A timeline for scratch builds (-DPADRA_DECODE_TRACE): thread 0 of every CTA records %globaltimer at numbered points.
#ifdef PADRA_DECODE_TRACE
extern unsigned long long *g_trace;
extern int g_trace_launch;
#define PADRA_TRACE(trace, slot)                                                                                       \
  do {                                                                                                                 \
    if ((trace) && threadIdx.x == 0) {                                                                                 \
      unsigned long long now;                                                                                          \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));                                                          \
      (trace)[((static_cast<size_t>(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + (slot)] = now; \
    }                                                                                                                  \
  } while (0)
#define PADRA_TRACE_SM(trace)                                                                                          \
  do {                                                                                                                 \
    if ((trace) && threadIdx.x == 0) {                                                                                 \
      unsigned sm;                                                                                                     \
      asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));                                                                  \
      (trace)[((static_cast<size_t>(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + 15] = sm + 1; \
    }                                                                                                                  \
  } while (0)
#else
#define PADRA_TRACE(trace, slot)
#define PADRA_TRACE_SM(trace)
#endif

// K-slices: enough CTAs to fill the machine several deep, slices of whole 128-input blocks.
// PADRA_DECODE_SLICES (read once per process) overrides the default of four: a tuning aid, not part of the interface.
inline int SliceOverride() {
  static const int value = [] {
    const char *text = std::getenv("PADRA_DECODE_SLICES");
    return text ? std::atoi(text) : 0;
  }();
  return value;
}
inline int PickSlices(int cols, int base_ctas) {
  int slices = SliceOverride() > 0 ? SliceOverride() : 4;
  if (slices > kMaxSlices)
    slices = kMaxSlices;
  while (slices > 1 && ((cols / 128) % slices != 0 || base_ctas * slices > 1024))
    slices /= 2;
  return slices;
}

struct LayerWorkspace {
  size_t tickets_gateup, tickets_down, gateup, xdown, down, svh, sidecars, total;
  int slices_gateup, slices_down;
  LayerWorkspace(int tokens, int hidden, int inter) {
    const size_t pairs = static_cast<size_t>(tokens) * kTopK;
    const int units = pairs < kExperts ? static_cast<int>(pairs) : kExperts;
    slices_gateup = PickSlices(hidden, (inter / 128) * units * 2);
    slices_down = PickSlices(inter, (hidden / 128) * units);
    auto align = [](size_t n) { return (n + 255) & ~static_cast<size_t>(255); };
    size_t at = 0;
    // the ticket area has one size for every shape, so that a workspace (or the built-in array) that serves calls of
    // different shapes never has one shape's partial sums where another shape keeps its counters
    tickets_gateup = at, at += align(static_cast<size_t>(kExperts) * kMaxBlocks * sizeof(unsigned));
    tickets_down = at, at += align(static_cast<size_t>(kMaxDecodeRows) * kMaxBlocks * sizeof(unsigned));
    gateup = at, at += align(pairs * 2 * slices_gateup * inter * sizeof(float));
    xdown = at, at += align(pairs * inter * sizeof(__half));
    down = at, at += align(pairs * slices_down * hidden * sizeof(float));
    svh = at, at += align(pairs * hidden * sizeof(__half));
    sidecars = at, at += align(pairs * 2 * inter * sizeof(__half)); // svh of gate and up beside their partial sums
    total = at;
  }
};

template <typename... KernelArgs, typename... Args>
inline int LaunchProgrammatic(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  // PADRA_DECODE_NO_OVERLAP (read once per process) launches in plain stream order: a diagnostic that takes the
  // overlap of consecutive launches out of a timing; results are the same either way
  static const int allowed = std::getenv("PADRA_DECODE_NO_OVERLAP") ? 0 : 1;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = allowed;
  cudaLaunchConfig_t config{};
  config.gridDim = grid, config.blockDim = block, config.dynamicSmemBytes = smem, config.stream = stream;
  config.attrs = &attribute, config.numAttrs = 1;
  return CudaStatus(cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...));
}


} // namespace decode

// One token: decode_single.cu.  workspace has the layout of decode::LayerWorkspace(1, hidden, inter).
int LaunchSingleTokenLayer(const Matrix *matrices, int layer, const int *ids, const float *routing, const float *normalized, float *x,
                           int rate, int hidden, int inter, const unsigned short *table, void *workspace, int *bad, cudaStream_t stream,
                           unsigned launches);
} // namespace padra
