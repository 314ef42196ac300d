// Shared host/device helpers of the pratchya_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <numeric>

#include "pratchya_b200.h"

namespace pb {

// ---- host-side error reporting -------------------------------------------------
char* error_buffer();            // thread-local, 512 bytes (defined in api.cu)
int fail(int status, const char* fmt, ...);

#define PB_CUDA_TRY(expr)                                                          \
  do {                                                                             \
    cudaError_t _e = (expr);                                                       \
    if (_e != cudaSuccess)                                                         \
      return ::pb::fail(PB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

#define PB_LAUNCH_CHECK(name)                                                      \
  do {                                                                             \
    cudaError_t _e = cudaGetLastError();                                           \
    if (_e != cudaSuccess)                                                         \
      return ::pb::fail(PB_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
  } while (0)

// Block / super-group geometry of one [rows, cols] slice on grid (a, b).
// Mirrors pratchya/_qualia/_qarr.py:474-480.
struct Geometry {
  int64_t rows, cols;
  int a, b;
  int64_t nbr, nbc;   // blocks per column / per row of the block grid
  int64_t Nb;         // blocks per slice
  int64_t K;          // blocks per super-group
  int64_t M;          // super-groups per slice
};

inline int make_geometry(int64_t rows, int64_t cols, int a, int b, Geometry* g) {
  if (rows <= 0 || cols <= 0) return fail(PB_ERR_BAD_SHAPE, "rows=%lld cols=%lld must be positive", (long long)rows, (long long)cols);
  if (a <= 0 || b <= 0) return fail(PB_ERR_BAD_GRID, "grid (%d,%d) must be positive", a, b);
  if (rows % a != 0 || cols % b != 0)
    return fail(PB_ERR_BAD_SHAPE, "shape (%lld,%lld) is not divisible by grid (%d,%d)", (long long)rows, (long long)cols, a, b);
  g->rows = rows; g->cols = cols; g->a = a; g->b = b;
  g->nbr = rows / a; g->nbc = cols / b;
  g->Nb = g->nbr * g->nbc;
  int64_t target = ((int64_t)a * b) / 16;
  if (target < 1) target = 1;
  g->K = std::gcd(target, g->Nb);
  g->M = g->Nb / g->K;
  return PB_OK;
}

int sm_count();   // SMs of the current device (cached per device)
void* tensor_map_encoder();   // cuTensorMapEncodeTiled from the driver (looked up once per process), or nullptr

// Tuning and diagnostic switches are read from the environment by the diagnostics build only
// (-DPB_DIAGNOSTICS); the product build always runs the defaults.
inline int env_switch(const char* name, int fallback) {
#ifdef PB_DIAGNOSTICS
  const char* e = getenv(name);
  return e ? atoi(e) : fallback;
#else
  (void)name;
  return fallback;
#endif
}

// Division of a 31-bit index by a run-time constant as multiply-high + shift
// (Granlund-Montgomery with N = 31: m = ceil(2^(31+l) / d), l = ceil(log2 d)).
struct FastDiv {
  uint32_t d, m, s;
  FastDiv() : d(1), m(0), s(0) {}
  explicit FastDiv(uint32_t div) : d(div), m(0), s(0) {
    if (div > 1) {
      uint32_t l = 0;
      while ((1ull << l) < div) ++l;
      m = (uint32_t)(((1ull << (31 + l)) + div - 1) / div);
      s = l - 1;
    }
  }
#ifdef __CUDACC__
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : (__umulhi(n, m) >> s); }
#endif
};

// Row-major [R, cols] view (R = batch*rows; rows % a == 0 makes the batch fold
// into the block-row index) cut into vectors of `vec` consecutive elements.
struct VecIndexer {
  FastDiv vecs_per_row, by_a, by_b;
  uint32_t vec, nbc;
  VecIndexer() : vec(1), nbc(1) {}
  VecIndexer(int64_t cols, int a, int b, int vec_)
      : vecs_per_row((uint32_t)(cols / vec_)), by_a((uint32_t)a), by_b((uint32_t)b), vec((uint32_t)vec_), nbc((uint32_t)(cols / b)) {}
#ifdef __CUDACC__
  // global block index of vector i
  __device__ __forceinline__ uint32_t block_of(uint32_t i) const {
    const uint32_t R = vecs_per_row.div(i);
    const uint32_t c = (i - R * vecs_per_row.d) * vec;
    return by_a.div(R) * nbc + by_b.div(c);
  }
#endif
};
constexpr int64_t kMaxIndexed = (1ll << 31) - 1;   // limit of the 31-bit index arithmetic

// ---- device-side arithmetic shared by the quantizers --------------------------
#ifdef __CUDACC__

__device__ __forceinline__ float e8m0_to_f32(uint32_t byte) { return __uint_as_float(byte << 23); }

// Per-block scale under the reference rule (_qarr.py:488-497):
//   S = m_i / safe(M_j); sb = biased exponent of S; S_eff = max(2^(sb-127) * M_j, 1e-7).
// Returns the divisor D = S_eff / 128 (exact: S_eff >= 1e-7 is far from the
// subnormal range), so that x / D == (x / S_eff) * 128 bit for bit.
__device__ __forceinline__ void block_scale(float m_i, float M_j, uint32_t& sb, float& D) {
  const float safe = (M_j == 0.0f) ? 1.0f : M_j;
  const float S = __fdiv_rn(m_i, safe);
  sb = (__float_as_uint(S) >> 23) & 0xffu;
  const float Sq = e8m0_to_f32(sb);
  const float S_eff = fmaxf(__fmul_rn(Sq, M_j), 1e-7f);
  D = __fmul_rn(S_eff, 0.0078125f);
}

// Correctly rounded x / D with the reciprocal r = RN(1/D) hoisted out of the
// per-element work: two Markstein refinement steps (q faithful after the first,
// correctly rounded after the second), then the sign of x is restored so that
// x = -0 gives -0 as IEEE division does.  Valid here because |x / D| <= 256 and
// D >= 7.8e-10, so no intermediate overflows and every quotient large enough to
// survive the fp8 cast is computed in the normal range.
__device__ __forceinline__ float div_hoisted_unsigned(float x, float D, float r) {
  float q = __fmul_rn(x, r);
  float e = __fmaf_rn(-q, D, x);
  q = __fmaf_rn(e, r, q);
  e = __fmaf_rn(-q, D, x);
  q = __fmaf_rn(e, r, q);
  return q;
}
// The same five operations on two elements at a time (packed f32x2 arithmetic of sm_100): r2 holds
// the reciprocal twice and nD2 the negated divisor twice; fma(q, -D, x) has the bits of fma(-q, D, x).
__device__ __forceinline__ float2 div_hoisted_unsigned2(float2 x, float2 nD2, float2 r2) {
  float2 q = __fmul2_rn(x, r2);
  float2 e = __ffma2_rn(q, nD2, x);
  q = __ffma2_rn(e, r2, q);
  e = __ffma2_rn(q, nD2, x);
  q = __ffma2_rn(e, r2, q);
  return q;
}
// (x0, x1) / D for f32 inputs, packed to bf16x2 with the inputs' signs (the quotient's own sign is
// lost only for x = -0): the bits of pack_bf16x2(div_hoisted(x0, D, r), div_hoisted(x1, D, r)).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi);
__device__ __forceinline__ uint32_t div_hoisted_pack2(float x0, float x1, float2 nD2, float2 r2) {
  const float2 q = div_hoisted_unsigned2(make_float2(x0, x1), nD2, r2);
  const uint32_t sign = ((__float_as_uint(x0) >> 16) & 0x8000u) | (__float_as_uint(x1) & 0x80000000u);
  return (pack_bf16x2(q.x, q.y) & 0x7fff7fffu) | sign;
}
__device__ __forceinline__ float div_hoisted(float x, float D, float r) {
  const float q = div_hoisted_unsigned(x, D, r);
  return __uint_as_float((__float_as_uint(q) & 0x7fffffffu) | (__float_as_uint(x) & 0x80000000u));
}

// f32 pair -> packed bf16x2 (round-to-nearest-even); `lo` lands in bits [0,16).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t p;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(hi), "f"(lo));
  return p;
}

// packed bf16x2 -> two fp8 bytes (round-to-nearest-even), low element in bits [0,8).
// The bf16 values are widened exactly to f32 first; |v| <= 256 so satfinite never clamps.
template <int FMT>
__device__ __forceinline__ uint32_t bf16x2_to_fp8x2(uint32_t p) {
  const float lo = __uint_as_float(p << 16);
  const float hi = __uint_as_float(p & 0xffff0000u);
  uint16_t o;
  if (FMT == PB_E4M3)
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(o) : "f"(hi), "f"(lo));
  else
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(o) : "f"(hi), "f"(lo));
  return o;
}

// two fp8 bytes -> two f32 (exact)
template <int FMT>
__device__ __forceinline__ float2 fp8x2_to_f32x2(uint16_t v) {
  uint32_t h2;
  if (FMT == PB_E4M3)
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(v));
  else
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(v));
  const __half2 h = *reinterpret_cast<const __half2*>(&h2);
  return __half22float2(h);
}

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

#endif  // __CUDACC__

}  // namespace pb
