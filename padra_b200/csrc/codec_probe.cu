// Two utilities around the trellis codec that are not on the timed path:
//
//   * CodecCeilingKernel: the codec's inner loop on registers alone (no memory traffic after the first instruction),
//     in both of its forms (byte sums by dp4a on the integer pipe, or by an integer mma on the tensor cores), with or
//     without the FP16 mma that consumes the decoded fragments.  Timed by the benchmark, it gives the rate at which an
//     SM can decode weights at all: the instruction-issue ceiling that stands beside the HBM roofline of the decode
//     kernels (a K4 layer step decodes 50.3 M weights for 25.3 MB of packed words).
//   * DecodeWeightsTensorKernel: full FP16 dump of one matrix through the tensor-core form of the codec, so that the
//     form the decode kernels use is checked bit for bit against the reference decoder
//     (src/cuda/expert_exl3.cuh:8-22), like DecodeWeightsKernel does for the dp4a form.
#include "codec.cuh"
#include "common.cuh"
#include "kernels.cuh"

namespace padra {
namespace {

__device__ __forceinline__ void MmaF16(const uint32_t (&a)[4], uint32_t b0, uint32_t b1, float (&d)[4]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int Rate, bool Tensor, bool WithMma>
__global__ void __launch_bounds__(256) CodecCeilingKernel(unsigned *sink, int iterations, unsigned seed) {
  const int lane = threadIdx.x & 31;
  const unsigned id = blockIdx.x * blockDim.x + threadIdx.x;
  uint32_t words[Rate];
#pragma unroll
  for (int i = 0; i < Rate; ++i)
    words[i] = (id + 1u) * 0x9E3779B9u + seed * (2u * i + 1u);
  const codec::ByteSumSelector sel = codec::MakeByteSumSelector(lane);
  const uint32_t b0 = 0x3c003c00u ^ (seed & 0x00010001u), b1 = 0x38003800u; // FP16 ones and halves
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  uint32_t fold = 0;
  for (int it = 0; it < iterations; ++it) {
    const uint32_t previous = __shfl_sync(0xffffffffu, words[Rate - 1], (lane + 28) & 31);
    uint32_t frag[4][4];
    if constexpr (Tensor)
      codec::Decode32Tensor<Rate>(words, previous, sel, frag);
    else
      codec::Decode32<Rate>(words, previous, frag);
    if constexpr (WithMma) {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        MmaF16(frag[c], b0, b1, acc);
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) // three-input exclusive-or: two instructions per four registers
        fold ^= (frag[c][0] ^ frag[c][1]) ^ (frag[c][2] ^ frag[c][3]);
    }
    // the next iteration decodes other words: nothing can be hoisted out of the loop
#pragma unroll
    for (int i = 0; i < Rate; ++i)
      words[i] += 0x632BE5ABu;
  }
  sink[id] = fold ^ __float_as_uint(acc[0] + acc[1] + acc[2] + acc[3]);
}

template <int Rate, bool Tensor, bool WithMma> int LaunchCeiling(unsigned *sink, int iterations, int blocks, unsigned seed, cudaStream_t s) {
  CodecCeilingKernel<Rate, Tensor, WithMma><<<blocks, 256, 0, s>>>(sink, iterations, seed);
  return CudaStatus(cudaGetLastError());
}
template <int Rate> int DispatchCeiling(int form, unsigned *sink, int iterations, int blocks, unsigned seed, cudaStream_t s) {
  switch (form) {
  case 0:
    return LaunchCeiling<Rate, false, false>(sink, iterations, blocks, seed, s);
  case 1:
    return LaunchCeiling<Rate, true, false>(sink, iterations, blocks, seed, s);
  case 2:
    return LaunchCeiling<Rate, false, true>(sink, iterations, blocks, seed, s);
  default:
    return LaunchCeiling<Rate, true, true>(sink, iterations, blocks, seed, s);
  }
}

template <int Rate>
__global__ void DecodeWeightsTensorKernel(const Matrix *matrix, unsigned short *out, int rows, int cols, int *bad) {
  using L = codec::Lane<Rate>;
  const Matrix m = *matrix;
  if (m.format != FormatOfRate(Rate) || m.rows != rows || m.cols != cols || (rows % 16) || (cols % 64) || !m.data) {
    if (!threadIdx.x && !blockIdx.x)
      Raise(bad);
    return;
  }
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const codec::ByteSumSelector sel = codec::MakeByteSumSelector(lane);
  const int tiles_per_kstep = rows / 16, rounds = cols / 64;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  // whole warps only: the loop bound is the same for every lane of a warp
  for (int item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < rounds * tiles_per_kstep; item += warps) {
    const int round = item / tiles_per_kstep, column = item % tiles_per_kstep;
    uint32_t words[Rate];
    codec::LoadWords<Rate>(m.data + (static_cast<size_t>(round * 4 + t) * tiles_per_kstep + column) * L::kTileBytes + g * L::kBytes,
                           words);
    const uint32_t previous = __shfl_sync(0xffffffffu, words[Rate - 1], (lane + 28) & 31);
    uint32_t frag[4][4];
    codec::Decode32Tensor<Rate>(words, previous, sel, frag);
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int o = column * 16 + g + ((f & 1) ? 8 : 0);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int k = 2 * t + e + ((f & 2) ? 8 : 0); // logical input of mma number c
          const int i = (round * 4 + (k & 3)) * 16 + codec::TensorInput(c, k >> 2);
          out[static_cast<size_t>(i) * rows + o] = static_cast<unsigned short>(e ? frag[c][f] >> 16 : frag[c][f] & 0xffffu);
        }
      }
  }
}

} // namespace

int LaunchCodecCeiling(int rate, int form, int iterations, int blocks, unsigned *sink, cudaStream_t stream) {
  if (!sink || iterations < 1 || blocks < 1 || form < 0 || form > 3)
    return PADRA_INVALID_ARGUMENT;
  switch (rate) {
  case 3:
    return DispatchCeiling<3>(form, sink, iterations, blocks, 17u, stream);
  case 4:
    return DispatchCeiling<4>(form, sink, iterations, blocks, 17u, stream);
  case 6:
    return DispatchCeiling<6>(form, sink, iterations, blocks, 17u, stream);
  default:
    return PADRA_UNSUPPORTED;
  }
}

int LaunchDecodeWeightsTensor(const Matrix *matrix, unsigned short *out, int rows, int cols, int rate, int *bad, cudaStream_t stream) {
  if (!matrix || !out || !bad || rows < 16 || cols < 64 || (rows % 16) || (cols % 64))
    return PADRA_INVALID_ARGUMENT;
  const int items = (cols / 64) * (rows / 16);
  const int blocks = (items + 7) / 8 < 1184 ? (items + 7) / 8 : 1184;
  switch (rate) {
  case 3:
    DecodeWeightsTensorKernel<3><<<blocks, 256, 0, stream>>>(matrix, out, rows, cols, bad);
    break;
  case 4:
    DecodeWeightsTensorKernel<4><<<blocks, 256, 0, stream>>>(matrix, out, rows, cols, bad);
    break;
  case 6:
    DecodeWeightsTensorKernel<6><<<blocks, 256, 0, stream>>>(matrix, out, rows, cols, bad);
    break;
  default:
    return PADRA_UNSUPPORTED;
  }
  return CudaStatus(cudaGetLastError());
}

} // namespace padra
