// Harness prologue for compiling the reference's own EXL3 expert kernels for sm_100a, unmodified, from
// where they lie in the reference checkout.  TEST INFRASTRUCTURE ONLY: the resulting library
// (oracle/_ref/libref_kernels.so) is the GPU-side parity oracle and the "reference kernels on this GPU"
// timing arm.  The reference keeps these kernels in the anonymous namespace of one translation unit
// (src/cuda/inference.cu:46-47); the Makefile splices the helper functions they expect (B, ExpRN,
// Accumulate, Finite, Route, Activate, Combine) out of that file's text between this prologue and the
// epilogue, then includes the kernel headers.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <type_traits>
#include "runtime/exl3_masked_schedule.h"
namespace mellum16 {
inline constexpr int kW4A8FMaxPrefillChunk = 2048; // src/runtime/inference.h:13
// Field order and size of src/cuda/device_matrix.cuh:6-13 (its binder needs the model loader, which
// the kernels do not).
struct DeviceMatrix {
  const unsigned char *data = nullptr;
  const unsigned char *scales = nullptr;
  const float *divisor = nullptr;
  int rows = 0, cols = 0, format = 0;
  const std::uint16_t *suh = nullptr;
  const std::uint16_t *svh = nullptr;
};
static_assert(sizeof(DeviceMatrix) == 56);
namespace {
