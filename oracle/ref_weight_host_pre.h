// Host stand-ins for the few CUDA intrinsics the reference's scalar trellis decoder uses, so that the
// reference's own Index/Weight source text can be compiled for the host cores and used to pin the
// oracle.  TEST INFRASTRUCTURE ONLY.  The FP16 fused multiply-add here is written independently of the
// oracle's integer formulation (frexp/nearbyint instead of bit arithmetic) on purpose.

#include <cmath>
#include <cstdint>
#include <cstring>
#define __device__
struct __half {
  std::uint16_t bits;
};
static inline __half __ushort_as_half(unsigned v) {
  return {static_cast<std::uint16_t>(v)};
}
static inline double HalfToDouble(__half h) {
  const int sign = h.bits >> 15, exp = (h.bits >> 10) & 31, man = h.bits & 1023;
  double v;
  if (exp == 31)
    v = man ? NAN : INFINITY;
  else if (exp == 0)
    v = std::ldexp(double(man), -24);
  else
    v = std::ldexp(double(1024 + man), exp - 25);
  return sign ? -v : v;
}
static inline __half DoubleToHalf(double v) { // round to nearest even, default FP environment
  if (std::isnan(v))
    return {0x7fff};
  const std::uint16_t sign = std::signbit(v) ? 0x8000 : 0;
  double a = std::fabs(v);
  if (a == 0)
    return {sign};
  int e;
  std::frexp(a, &e); // a = f * 2^e, f in [0.5, 1)
  int unit = e - 11; // 11 significant bits
  if (unit < -24)
    unit = -24; // subnormal spacing
  const double q = std::nearbyint(std::ldexp(a, -unit));
  a = std::ldexp(q, unit);
  if (a >= 65536.0)
    return {static_cast<std::uint16_t>(sign | 0x7c00)};
  if (a == 0)
    return {sign};
  std::frexp(a, &e);
  if (e - 1 < -14)
    return {static_cast<std::uint16_t>(sign | static_cast<std::uint16_t>(std::ldexp(a, 24)))};
  const int man = static_cast<int>(std::ldexp(a, 11 - e)) - 1024;
  return {static_cast<std::uint16_t>(sign | ((e - 1 + 15) << 10) | man)};
}
static inline __half __hfma(__half a, __half b, __half c) {
  // product of two 11-bit significands is exact in double; std::fma rounds the sum once to double,
  // which is exact for the magnitudes the codebook produces (and far finer than FP16 otherwise).
  return DoubleToHalf(std::fma(HalfToDouble(a), HalfToDouble(b), HalfToDouble(c)));
}
static inline float __half2float(__half h) {
  return static_cast<float>(HalfToDouble(h));
}
static inline unsigned __funnelshift_r(unsigned lo, unsigned hi, unsigned shift) {
  return static_cast<unsigned>(((static_cast<std::uint64_t>(hi) << 32) | lo) >> (shift & 31));
}
// Same field order as the reference descriptor (src/cuda/device_matrix.cuh:6-13).
struct DeviceMatrix {
  const unsigned char *data = nullptr;
  const unsigned char *scales = nullptr;
  const float *divisor = nullptr;
  int rows = 0, cols = 0, format = 0;
  const std::uint16_t *suh = nullptr;
  const std::uint16_t *svh = nullptr;
};
namespace ref_host {
