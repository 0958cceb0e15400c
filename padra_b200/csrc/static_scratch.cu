// The decode-layer call for callers that may not allocate device memory.
//
// Who that is: an inference server that hands every free byte of the device to its own arena at start-up (KV cache,
// activation pools) has nothing left for cudaMalloc to return; a plugin loaded into such a server is usually told
// not to touch the allocator at all; and code on a latency-critical path avoids cudaMalloc/cudaFree because they
// synchronise the whole device.  The regular entry point (padra_exl3_moe_decode_layer) leaves the allocation of
// its workspace to the caller; this one brings its own, a fixed array that is part of the loaded module, so the
// call itself allocates nothing: no cudaMalloc, no cudaFree, no allocating library routine.
//
// The price: the array has a fixed size (kStaticScratchBytes), requests that need more are refused, and there is ONE
// array per device, shared by every call in the process.  Calls that can overlap on the GPU (different streams, or
// different host threads without ordering between their streams) would race on it -- they would mix each other's
// partial sums and ticket counts and give wrong results, not an error; callers must order them.  The array keeps
// whatever the last call left there.  The only part that has to start at zero is the pipeline's ticket counters at
// its beginning: the module loader zero-fills the array, and every call leaves the counters at zero again (the CTA that
// takes a counter's last ticket clears it, on error paths too), so nothing has to be cleared between calls.
#include <mutex>

#include "common.cuh"
#include "kernels.cuh"

namespace padra {
namespace {

constexpr size_t kStaticScratchBytes = PADRA_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the runtime's symbol calls, never an address the GPU understands.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void *g_scratch_address[kMaxDevices]; // device address of the array on each device, filled on first use

// The array's address on the current device.  Looked up once per device, with that device current.
int ScratchAddress(void **address) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return PADRA_INTERNAL;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_address[device]) {
    void *found = nullptr;
    if (cudaGetSymbolAddress(&found, g_static_scratch) != cudaSuccess || !found) {
      cudaGetLastError(); // leave no stale error behind for the caller's next runtime call
      return PADRA_INTERNAL;
    }
    g_scratch_address[device] = found;
  }
  *address = g_scratch_address[device];
  return PADRA_OK;
}

} // namespace
} // namespace padra

extern "C" PADRA_API int padra_exl3_moe_decode_layer_static(const padra_matrix *matrices, int layer, const int *ids,
                                                             const float *routing, const float *normalized, float *x,
                                                             int tokens, int rate, int hidden, int inter,
                                                             const unsigned short *table, int *bad, padra_stream stream) {
  using namespace padra;
  if (rate != 3 && rate != 4 && rate != 6)
    return PADRA_UNSUPPORTED;
  if (!matrices || !ids || !routing || !normalized || !x || !table || !bad || tokens < 1 || tokens > 16 || layer < 0 ||
      hidden < 128 || inter < 128 || hidden % 128 || inter % 128)
    return PADRA_INVALID_ARGUMENT;
  if (DecodeLayerWorkspaceBytes(tokens, hidden, inter) > kStaticScratchBytes)
    return PADRA_RESOURCE_EXHAUSTED; // more scratch than the built-in array holds: use the caller-workspace entry point
  void *scratch = nullptr;
  const int status = ScratchAddress(&scratch);
  if (status != PADRA_OK)
    return status;
  return LaunchDecodeLayer(reinterpret_cast<const Matrix *>(matrices), layer, ids, routing, normalized, x, tokens, rate,
                                hidden, inter, table, scratch, kStaticScratchBytes, bad, static_cast<cudaStream_t>(stream));
}
