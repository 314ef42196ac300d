// Device self-checks exported for the GPU test-suite.
#include "common.cuh"

namespace pb {
namespace {

__device__ __forceinline__ uint32_t mix(uint64_t v) {
  v ^= v >> 33; v *= 0xff51afd7ed558ccdull; v ^= v >> 33; v *= 0xc4ceb9fe1a85ec53ull; v ^= v >> 33;
  return (uint32_t)v;
}

// Compares the hoisted-reciprocal division used by the quantizers with IEEE
// division on pseudo-random operands drawn like the quantizer's: a divisor D with a
// random mantissa and exponent in [2^-30, 2^96], and x = D * t with t in (0, 256]
// (random mantissa, random exponent) plus a random perturbation of the low bits.
__global__ void division_check_kernel(uint64_t n, uint64_t seed, unsigned long long* mismatches) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  unsigned long long bad = 0;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const uint32_t r0 = mix(seed + 3 * i), r1 = mix(seed + 3 * i + 1), r2 = mix(seed + 3 * i + 2);
    const uint32_t d_exp = 97 + (r0 >> 23) % 127;                  // biased 97..223
    const float D = __uint_as_float((d_exp << 23) | (r0 & 0x7fffffu));
    const uint32_t t_exp = 135 - (r1 >> 23) % 40;                  // 2^8 down to 2^-31
    float t = __uint_as_float((t_exp << 23) | (r1 & 0x7fffffu));
    if (t > 256.0f) t = 256.0f;
    float x = __fmul_rn(D, t);
    x = __uint_as_float(__float_as_uint(x) ^ (r2 & 0xffu));        // break the exact-product structure
    if (r2 & 0x100u) x = -x;
    if ((r2 & 0xfffe00u) == 0) x = (r2 & 0x100u) ? -0.0f : 0.0f;   // occasional signed zeros
    const float want = __fdiv_rn(x, D);
    const float got = div_hoisted(x, D, __frcp_rn(D));
    if (__float_as_uint(want) != __float_as_uint(got)) ++bad;
  }
  if (bad) atomicAdd(mismatches, bad);
}

}  // namespace
}  // namespace pb

// Not part of the reference's surface: test hook.  Adds the number of operand pairs
// (out of n) on which the quantizer's division differs from IEEE division to *mismatches.
extern "C" PB_API int pb_debug_division_check(uint64_t n, uint64_t seed, unsigned long long* mismatches, void* stream) {
  if (!mismatches) return pb::fail(PB_ERR_NULL_POINTER, "pb_debug_division_check: mismatches must be non-null");
  pb::division_check_kernel<<<pb::sm_count() * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(n, seed, mismatches);
  PB_LAUNCH_CHECK("division_check_kernel");
  return PB_OK;
}
