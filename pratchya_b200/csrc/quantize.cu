// Block quantizers (sm_100a).  Replace quantize_impl, pratchya/_qualia/_qarr.py:458-506.
//
// Two implementations, identical results:
//   * row128: grid (1,128) with 8-block super-groups.  With a == 1 the row-major
//     block order is the memory order, so a super-group is 1024 contiguous
//     elements; one warp owns one super-group, keeps it in registers between the
//     amax pass and the cast, and touches HBM once (read x, write q + scales).
//     No scratch memory.
//   * generic: any grid.  Three small kernels around a scratch buffer
//     (per-block amax bits, then per-block divisors).
#include <mutex>

#include "common.cuh"

namespace pb {
namespace {

constexpr int kRowThreads = 256;
constexpr int kGroupElems = 1024;   // 8 blocks x 128

// ---------------------------------------------------------------------------------
// Butterfly max-reduction of N per-lane values (N a power of two).  After the call
// v[0] of a lane holds the maximum, over the 2^(log2 N + EXTRA) lanes that differ
// from it in those low lane bits, of the value with index bitrev(lane's low log2 N bits).
// Costs N-1+EXTRA shuffles instead of N*(log2 N + EXTRA).
template <int N, int EXTRA>
__device__ __forceinline__ void butterfly_max(float (&v)[N], int lane) {
  int mask = 1;
#pragma unroll
  for (int n = N; n > 1; n >>= 1, mask <<= 1) {
    const bool upper = (lane & mask) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float keep = upper ? v[i + n / 2] : v[i];
      const float send = upper ? v[i] : v[i + n / 2];
      v[i] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, mask));
    }
  }
#pragma unroll
  for (int s = 0; s < EXTRA; ++s, mask <<= 1) v[0] = fmaxf(v[0], __shfl_xor_sync(0xffffffffu, v[0], mask));
}

template <int BITS>
__device__ __forceinline__ int bitrev(int x) {
  int r = 0;
#pragma unroll
  for (int i = 0; i < BITS; ++i) r |= ((x >> i) & 1) << (BITS - 1 - i);
  return r;
}

// Optional second output of the row quantizer: the same scales in the layout the GEMM kernel
// consumes for its A operand (512-byte scale-factor atoms and one fp32 factor per row and
// 1024-deep chunk), so that a following pb_gemm_tn_ex need not re-tile them.  Needs whole
// super-groups per row (cols % 1024 == 0).
struct GemmPrepOut {
  uint8_t* sf;      // [kg][row tile of 128][512]; null: not requested
  float* f;         // [chunk][Mpad]
  uint32_t KB;      // 128-deep blocks per row
  uint32_t tiles;   // row tiles of 128 (atoms per kg)
  uint32_t Mpad;
};
__device__ __forceinline__ void write_gemm_prep(const GemmPrepOut& o, int64_t g, int blk, uint32_t sb, float Mj, bool write_byte, bool write_factor) {
  const uint32_t flat = (uint32_t)g * 8u;               // first block of this super-group
  const uint32_t row = flat / o.KB, kb0 = flat - row * o.KB;
  if (write_byte) {
    const uint32_t kb = kb0 + (uint32_t)blk;
    o.sf[((size_t)(kb >> 2) * o.tiles + (row >> 7)) * 512 + (row & 31u) * 16 + ((row & 127u) >> 5) * 4 + (kb & 3u)] = (uint8_t)sb;
  }
  if (write_factor) o.f[(size_t)(kb0 >> 3) * o.Mpad + row] = Mj * 0.0078125f;
}

// ---------------------------------------------------------------------------------
// bf16 input, 32-byte accesses: lane l, load j (0, 1) -> 16 elements at (j*32 + l)*16, which lie in
// block 4j + (l >> 3).  Two 256-bit loads and two 128-bit stores per lane and super-group (whole
// sectors per lane), eight lanes per block, and every lane forms the scales of its own two blocks,
// so nothing has to be handed round after the reductions.
__device__ __forceinline__ void ld_global_256(const void* p, uint32_t (&w)[8]) {
  asm volatile("ld.global.cs.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "l"(p));
}

template <int FMT, int MINB, bool PREP>
__global__ void __launch_bounds__(kRowThreads, MINB)
quantize_row128_bf16_wide_kernel(const uint8_t* __restrict__ x, uint4* __restrict__ q,
                                 uint8_t* __restrict__ sc8, float* __restrict__ sc32, int64_t n_groups, const GemmPrepOut prep) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * (kRowThreads / 32);
  for (int64_t g = (int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); g < n_groups; g += warps_total) {
    const uint8_t* src = x + g * (kGroupElems * 2);
    uint32_t w[2][8];
#pragma unroll
    for (int j = 0; j < 2; ++j) ld_global_256(src + (j * 32 + lane) * 32, w[j]);

    float m[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint32_t a = w[j][0] & 0x7fff7fffu;
      __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
      for (int k = 1; k < 8; ++k) {
        a = w[j][k] & 0x7fff7fffu;
        h = __hmax2(h, *reinterpret_cast<const __nv_bfloat162*>(&a));
      }
      const uint32_t hb = *reinterpret_cast<const uint32_t*>(&h);
      m[j] = fmaxf(__uint_as_float(hb << 16), __uint_as_float(hb & 0xffff0000u));
#pragma unroll
      for (int sft = 1; sft < 8; sft <<= 1) m[j] = fmaxf(m[j], __shfl_xor_sync(0xffffffffu, m[j], sft));      // the block's eight lanes
    }
    float Mj = fmaxf(m[0], m[1]);
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 8));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 16));
    if (lane == 0) sc32[g] = Mj;

    uint4* dst = q + g * (kGroupElems / 16);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint32_t sb; float D;
      block_scale(m[j], Mj, sb, D);
      const int blk = 4 * j + (lane >> 3);
      if ((lane & 7) == 0) sc8[g * 8 + blk] = (uint8_t)sb;
      if (PREP) write_gemm_prep(prep, g, blk, sb, Mj, (lane & 7) == 0, lane == 0 && j == 0);
      const float r = __frcp_rn(D);
      const float2 nD2 = make_float2(-D, -D), r2 = make_float2(r, r);
      uint32_t o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t in = w[j][k];
        const float2 v = div_hoisted_unsigned2(make_float2(__uint_as_float(in << 16), __uint_as_float(in & 0xffff0000u)), nD2, r2);
        const uint32_t p = (pack_bf16x2(v.x, v.y) & 0x7fff7fffu) | (in & 0x80008000u);      // the input's signs, also for -0
        o[k] = bf16x2_to_fp8x2<FMT>(p);
      }
      __stcs(dst + j * 32 + lane, make_uint4(o[0] | (o[1] << 16), o[2] | (o[3] << 16), o[4] | (o[5] << 16), o[6] | (o[7] << 16)));
    }
  }
}

// ---------------------------------------------------------------------------------
// bf16 input: lane l, load it -> 8 elements at (it*32 + l)*8; block = 2*it + (l >> 4).
template <int FMT, int MINB, bool PREP>
__global__ void __launch_bounds__(kRowThreads, MINB)
quantize_row128_bf16_kernel(const uint4* __restrict__ x, uint2* __restrict__ q,
                            uint8_t* __restrict__ sc8, float* __restrict__ sc32, int64_t n_groups, const GemmPrepOut prep) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * (kRowThreads / 32);
  for (int64_t g = (int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); g < n_groups; g += warps_total) {
    const uint4* src = x + g * (kGroupElems / 8);
    uint4 w[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) w[it] = __ldcs(src + it * 32 + lane);

    // per-load amax in the bf16 domain (exact), widened to f32
    float m[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const uint32_t a0 = w[it].x & 0x7fff7fffu, a1 = w[it].y & 0x7fff7fffu;
      const uint32_t a2 = w[it].z & 0x7fff7fffu, a3 = w[it].w & 0x7fff7fffu;
      __nv_bfloat162 h = __hmax2(__hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a0),
                                         *reinterpret_cast<const __nv_bfloat162*>(&a1)),
                                 __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a2),
                                         *reinterpret_cast<const __nv_bfloat162*>(&a3)));
      const uint32_t hb = *reinterpret_cast<const uint32_t*>(&h);
      m[it] = fmaxf(__uint_as_float(hb << 16), __uint_as_float(hb & 0xffff0000u));
    }
    butterfly_max<4, 2>(m, lane);                 // m[0]: amax of block (it_own, half)
    const int it_own = bitrev<2>(lane & 3);
    float Mj = m[0];
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 1));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 2));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 16));

    uint32_t sb; float D;
    block_scale(m[0], Mj, sb, D);
    const float r = __frcp_rn(D);
    if ((lane & 12) == 0) sc8[g * 8 + 2 * it_own + (lane >> 4)] = (uint8_t)sb;
    if (lane == 0) sc32[g] = Mj;
    if (PREP) write_gemm_prep(prep, g, 2 * it_own + (lane >> 4), sb, Mj, (lane & 12) == 0, lane == 0);

    uint2* dst = q + g * (kGroupElems / 8);
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int srcl = (lane & 16) | bitrev<2>(it);
      const float Di = __shfl_sync(0xffffffffu, D, srcl);
      const float ri = __shfl_sync(0xffffffffu, r, srcl);
      const uint32_t in[4] = {w[it].x, w[it].y, w[it].z, w[it].w};
      uint32_t o[4];
      const float2 nD2 = make_float2(-Di, -Di), r2 = make_float2(ri, ri);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 v = div_hoisted_unsigned2(make_float2(__uint_as_float(in[j] << 16), __uint_as_float(in[j] & 0xffff0000u)), nD2, r2);
        // sign of the input (also for -0) re-applied on the packed bf16 pair
        const uint32_t p = (pack_bf16x2(v.x, v.y) & 0x7fff7fffu) | (in[j] & 0x80008000u);
        o[j] = bf16x2_to_fp8x2<FMT>(p);
      }
      __stcs(dst + it * 32 + lane, make_uint2(o[0] | (o[1] << 16), o[2] | (o[3] << 16)));
    }
  }
}

// f32 input: lane l, load it -> 4 elements at (it*32 + l)*4; block = it.
template <int FMT, bool PREP>
__global__ void __launch_bounds__(kRowThreads)
quantize_row128_f32_kernel(const float4* __restrict__ x, uint32_t* __restrict__ q,
                           uint8_t* __restrict__ sc8, float* __restrict__ sc32, int64_t n_groups, const GemmPrepOut prep) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * (kRowThreads / 32);
  for (int64_t g = (int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); g < n_groups; g += warps_total) {
    const float4* src = x + g * (kGroupElems / 4);
    float4 w[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) w[it] = __ldcs(src + it * 32 + lane);
    float m[8];
#pragma unroll
    for (int it = 0; it < 8; ++it)
      m[it] = fmaxf(fmaxf(fabsf(w[it].x), fabsf(w[it].y)), fmaxf(fabsf(w[it].z), fabsf(w[it].w)));
    butterfly_max<8, 2>(m, lane);                 // m[0]: amax of block it_own over the warp
    const int it_own = bitrev<3>(lane & 7);
    float Mj = m[0];
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 1));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 2));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 4));

    uint32_t sb; float D;
    block_scale(m[0], Mj, sb, D);
    const float r = __frcp_rn(D);
    if (lane < 8) sc8[g * 8 + it_own] = (uint8_t)sb;
    if (lane == 0) sc32[g] = Mj;
    if (PREP) write_gemm_prep(prep, g, it_own, sb, Mj, lane < 8, lane == 0);

    uint32_t* dst = q + g * (kGroupElems / 4);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int srcl = bitrev<3>(it);
      const float Di = __shfl_sync(0xffffffffu, D, srcl);
      const float ri = __shfl_sync(0xffffffffu, r, srcl);
      const float2 nD2 = make_float2(-Di, -Di), r2 = make_float2(ri, ri);
      const uint32_t p0 = div_hoisted_pack2(w[it].x, w[it].y, nD2, r2);
      const uint32_t p1 = div_hoisted_pack2(w[it].z, w[it].w, nD2, r2);
      __stcs(dst + it * 32 + lane, bf16x2_to_fp8x2<FMT>(p0) | (bf16x2_to_fp8x2<FMT>(p1) << 16));
    }
  }
}

// The row quantizer (bf16 input) on 128-row x 1024-column tiles that also leaves the amax of every
// 128-row column block, for the transposed quantizer's second pass: Q(x,(1,128)) and the first
// half of Q(x^T,(1,128)) from one read of x.  A warp owns 16 rows of the tile; per row it is the
// kernel above, plus a running per-column maximum kept as packed bf16 pairs.
template <int FMT>
__global__ void __launch_bounds__(kRowThreads, 2)
quantize_row128_bf16_colmax_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, uint8_t* __restrict__ sc8,
                                   float* __restrict__ sc32, uint32_t* __restrict__ col_amax_bits, int rows, int cols) {
  __shared__ uint32_t red[kRowThreads / 32][512];          // per warp: 1024 column maxima as bf16 pairs
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int segs = cols >> 10;                              // super-groups per row
  const int seg = blockIdx.x, rb = blockIdx.y;
  const int64_t row0 = (int64_t)blockIdx.z * rows + (int64_t)rb * 128 + warp * 16;
  uint32_t cmax[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) cmax[i] = 0u;
  uint4 w[4], wn[4];
  {
    const uint4* src = x + (row0 * segs + seg) * (kGroupElems / 8);
#pragma unroll
    for (int it = 0; it < 4; ++it) wn[it] = __ldcs(src + it * 32 + lane);
  }
  for (int r = 0; r < 16; ++r) {
    const int64_t g = (row0 + r) * segs + seg;
#pragma unroll
    for (int it = 0; it < 4; ++it) w[it] = wn[it];
    if (r + 1 < 16) {
      const uint4* src = x + (g + segs) * (kGroupElems / 8);
#pragma unroll
      for (int it = 0; it < 4; ++it) wn[it] = __ldcs(src + it * 32 + lane);
    }
    float m[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const uint32_t a[4] = {w[it].x & 0x7fff7fffu, w[it].y & 0x7fff7fffu, w[it].z & 0x7fff7fffu, w[it].w & 0x7fff7fffu};
      __nv_bfloat162 h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        h[j] = *reinterpret_cast<const __nv_bfloat162*>(&a[j]);
        const __nv_bfloat162 c = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&cmax[it * 4 + j]), h[j]);
        cmax[it * 4 + j] = *reinterpret_cast<const uint32_t*>(&c);
      }
      const __nv_bfloat162 hm = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
      const uint32_t hb = *reinterpret_cast<const uint32_t*>(&hm);
      m[it] = fmaxf(__uint_as_float(hb << 16), __uint_as_float(hb & 0xffff0000u));
    }
    butterfly_max<4, 2>(m, lane);
    const int it_own = bitrev<2>(lane & 3);
    float Mj = m[0];
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 1));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 2));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 16));
    uint32_t sb; float D;
    block_scale(m[0], Mj, sb, D);
    const float rc = __frcp_rn(D);
    if ((lane & 12) == 0) sc8[g * 8 + 2 * it_own + (lane >> 4)] = (uint8_t)sb;
    if (lane == 0) sc32[g] = Mj;
    uint2* dst = q + g * (kGroupElems / 8);
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int srcl = (lane & 16) | bitrev<2>(it);
      const float Di = __shfl_sync(0xffffffffu, D, srcl);
      const float ri = __shfl_sync(0xffffffffu, rc, srcl);
      const uint32_t in[4] = {w[it].x, w[it].y, w[it].z, w[it].w};
      uint32_t o[4];
      const float2 nD2 = make_float2(-Di, -Di), r2 = make_float2(ri, ri);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 v = div_hoisted_unsigned2(make_float2(__uint_as_float(in[j] << 16), __uint_as_float(in[j] & 0xffff0000u)), nD2, r2);
        const uint32_t pk = (pack_bf16x2(v.x, v.y) & 0x7fff7fffu) | (in[j] & 0x80008000u);
        o[j] = bf16x2_to_fp8x2<FMT>(pk);
      }
      __stcs(dst + it * 32 + lane, make_uint2(o[0] | (o[1] << 16), o[2] | (o[3] << 16)));
    }
  }
  // column maxima of the 8 warps (16 rows each) -> one amax per column for this block row
#pragma unroll
  for (int it = 0; it < 4; ++it)
#pragma unroll
    for (int j = 0; j < 4; ++j) red[warp][(it * 32 + lane) * 4 + j] = cmax[it * 4 + j];
  __syncthreads();
  const int nrb = rows >> 7;
  for (int cp = threadIdx.x; cp < 512; cp += kRowThreads) {
    __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&red[0][cp]);
#pragma unroll
    for (int k = 1; k < kRowThreads / 32; ++k) v = __hmax2(v, *reinterpret_cast<const __nv_bfloat162*>(&red[k][cp]));
    const uint32_t vb = *reinterpret_cast<const uint32_t*>(&v);
    const size_t col = (size_t)blockIdx.z * cols + (size_t)seg * 1024 + 2 * cp;
    col_amax_bits[col * nrb + rb] = vb << 16;                    // f32 bits of the even column's amax
    col_amax_bits[(col + 1) * nrb + rb] = vb & 0xffff0000u;      // and of the odd one
  }
}

// Quantize and dequantize in one pass (f32 input, grid (1,128), 8-block super-groups): what
// `(x_q @ kernel).astype(dtype)` does to the f32 product in Linear.__call__
// (pratchya/_nnx_impl/_module.py:46-50 through QArrayImpl.__matmul__, _qarr.py:104-105, and
// astype/dequantize, :339-342, :46-59): out = dq(q(x)).  The arithmetic is the quantizer's above
// followed by the dequantizer's (fp8 -> f32 exactly, times f32(sc8<<23)*sc32, divided by 128,
// rounded to the output type), so the result has the bits of pb_quantize + pb_dequantize.
template <typename OutT> struct Out4;
template <> struct Out4<float> {
  using vec = float4;
  static __device__ __forceinline__ vec make(float a, float b, float c, float d) { return make_float4(a, b, c, d); }
};
template <> struct Out4<__nv_bfloat16> {
  using vec = uint2;
  static __device__ __forceinline__ vec make(float a, float b, float c, float d) { return make_uint2(pack_bf16x2(a, b), pack_bf16x2(c, d)); }
};

template <int FMT, typename OutT>
__global__ void __launch_bounds__(kRowThreads)
fake_quantize_row128_f32_kernel(const float4* __restrict__ x, typename Out4<OutT>::vec* __restrict__ out, int64_t n_groups) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * (kRowThreads / 32);
  for (int64_t g = (int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); g < n_groups; g += warps_total) {
    const float4* src = x + g * (kGroupElems / 4);
    float4 w[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) w[it] = __ldcs(src + it * 32 + lane);
    float m[8];
#pragma unroll
    for (int it = 0; it < 8; ++it)
      m[it] = fmaxf(fmaxf(fabsf(w[it].x), fabsf(w[it].y)), fmaxf(fabsf(w[it].z), fabsf(w[it].w)));
    butterfly_max<8, 2>(m, lane);                 // m[0]: amax of block it_own over the warp
    float Mj = m[0];
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 1));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 2));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 4));

    uint32_t sb; float D;
    block_scale(m[0], Mj, sb, D);
    const float r = __frcp_rn(D);
    const float x_sc = __fmul_rn(e8m0_to_f32(sb), Mj);       // the dequantizer's multiplier: raw amax, no floor

    typename Out4<OutT>::vec* dst = out + g * (kGroupElems / 4);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int srcl = bitrev<3>(it);
      const float Di = __shfl_sync(0xffffffffu, D, srcl);
      const float ri = __shfl_sync(0xffffffffu, r, srcl);
      const float si = __shfl_sync(0xffffffffu, x_sc, srcl);
      const float2 nD2 = make_float2(-Di, -Di), r2 = make_float2(ri, ri);
      const uint32_t p0 = div_hoisted_pack2(w[it].x, w[it].y, nD2, r2);
      const uint32_t p1 = div_hoisted_pack2(w[it].z, w[it].w, nD2, r2);
      const float2 a = fp8x2_to_f32x2<FMT>((uint16_t)bf16x2_to_fp8x2<FMT>(p0));
      const float2 b = fp8x2_to_f32x2<FMT>((uint16_t)bf16x2_to_fp8x2<FMT>(p1));
      const float k128 = 0.0078125f;
      __stcs(dst + it * 32 + lane, Out4<OutT>::make(__fmul_rn(__fmul_rn(a.x, si), k128), __fmul_rn(__fmul_rn(a.y, si), k128),
                                                    __fmul_rn(__fmul_rn(b.x, si), k128), __fmul_rn(__fmul_rn(b.y, si), k128)));
    }
  }
}

// The backward pass of a Linear starts from the cotangent g of its fake-quantized output: the output's dequantize rule
// scales it, g' = (g * x_sc) / 128 with x_sc = e8m0(y_sc8) * y_sc32 of the OUTPUT's (1,128) triple (dequantize_impl_bwd,
// _qarr.py:575-601), and g' is then quantized for the two products of the backward pass.  This is the row quantizer with that
// scaling as its prologue: the output's super-groups are the cotangent's, so a warp has its eight multipliers in lanes 0-7.
//
// RELU2 instead of the scaling: the value quantized is relu(g)^2, the activation between ChannelMix's two Linears
// (pratchya/_nnx_impl/_module.py:249) as the prologue of the second Linear's input quantizer.
template <int FMT, bool RELU2>
__global__ void __launch_bounds__(kRowThreads)
scaled_quantize_row128_f32_kernel(const float4* __restrict__ g, const uint8_t* __restrict__ y_sc8, const float* __restrict__ y_sc32,
                                  uint32_t* __restrict__ q, uint8_t* __restrict__ sc8, float* __restrict__ sc32, int64_t n_groups) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * (kRowThreads / 32);
  for (int64_t gi = (int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); gi < n_groups; gi += warps_total) {
    const float4* src = g + gi * (kGroupElems / 4);
    float4 w[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) w[it] = __ldcs(src + it * 32 + lane);
    float xs = 0.0f;
    if (!RELU2 && lane < 8) xs = __fmul_rn(e8m0_to_f32(__ldg(y_sc8 + gi * 8 + lane)), __ldg(y_sc32 + gi));
    float m[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) {        // load `it` holds elements of block `it`
      if (RELU2) {
        const float a = fmaxf(w[it].x, 0.f), b = fmaxf(w[it].y, 0.f), c = fmaxf(w[it].z, 0.f), d = fmaxf(w[it].w, 0.f);
        w[it] = make_float4(__fmul_rn(a, a), __fmul_rn(b, b), __fmul_rn(c, c), __fmul_rn(d, d));
      } else {
        const float x_sc = __shfl_sync(0xffffffffu, xs, it);
        const float k128 = 0.0078125f;
        w[it] = make_float4(__fmul_rn(__fmul_rn(w[it].x, x_sc), k128), __fmul_rn(__fmul_rn(w[it].y, x_sc), k128),
                            __fmul_rn(__fmul_rn(w[it].z, x_sc), k128), __fmul_rn(__fmul_rn(w[it].w, x_sc), k128));
      }
      m[it] = fmaxf(fmaxf(fabsf(w[it].x), fabsf(w[it].y)), fmaxf(fabsf(w[it].z), fabsf(w[it].w)));
    }
    butterfly_max<8, 2>(m, lane);                 // m[0]: amax of block it_own over the warp
    const int it_own = bitrev<3>(lane & 7);
    float Mj = m[0];
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 1));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 2));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 4));
    uint32_t sb; float D;
    block_scale(m[0], Mj, sb, D);
    const float r = __frcp_rn(D);
    if (lane < 8) sc8[gi * 8 + it_own] = (uint8_t)sb;
    if (lane == 0) sc32[gi] = Mj;
    uint32_t* dst = q + gi * (kGroupElems / 4);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int srcl = bitrev<3>(it);
      const float Di = __shfl_sync(0xffffffffu, D, srcl);
      const float ri = __shfl_sync(0xffffffffu, r, srcl);
      const float2 nD2 = make_float2(-Di, -Di), r2 = make_float2(ri, ri);
      const uint32_t p0 = div_hoisted_pack2(w[it].x, w[it].y, nD2, r2);
      const uint32_t p1 = div_hoisted_pack2(w[it].z, w[it].w, nD2, r2);
      __stcs(dst + it * 32 + lane, bf16x2_to_fp8x2<FMT>(p0) | (bf16x2_to_fp8x2<FMT>(p1) << 16));
    }
  }
}

// The head of TimeMix and of ChannelMix (pratchya/_nnx_impl/_module.py:126-134, 235-237) fused into the activation
// quantizers of the Linears that follow (Linear.__call__, :46-47): for mix k
//     v_k[r][c] = x[r][c] + (prev[r][c] - x[r][c]) * mu[k][c],   prev = the token before, the carried state for a first token,
// evaluated with the three roundings of the op-by-op form, and the kernel writes quantize_impl(v_k, (1,128)) for every k:
// x is read once (its previous row comes from the cache) and no v_k goes to memory.  A warp owns one super-group of 1024
// channels of one token and walks the mixes with x and prev - x in registers.
template <int FMT>
__global__ void __launch_bounds__(kRowThreads)
shift_lerp_quantize_row128_kernel(const float4* __restrict__ x, const float4* __restrict__ state, const float4* __restrict__ mu,
                                  uint32_t* __restrict__ q, uint8_t* __restrict__ sc8, float* __restrict__ sc32,
                                  int64_t n_groups, int segs, int steps, int n_mix) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * (kRowThreads / 32);
  for (int64_t g = (int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); g < n_groups; g += warps_total) {
    const int64_t row = g / segs;
    const int seg = (int)(g - row * segs);
    const int64_t seq = row / steps;
    const bool first = row - seq * steps == 0;
    const float4* src = x + g * (kGroupElems / 4);
    const float4* psrc = first ? (state ? state + (seq * segs + seg) * (kGroupElems / 4) : nullptr) : src - (int64_t)segs * (kGroupElems / 4);
    float4 w[8], d[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) w[it] = __ldg(src + it * 32 + lane);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const float4 pv = psrc ? __ldg(psrc + it * 32 + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
      d[it] = make_float4(__fsub_rn(pv.x, w[it].x), __fsub_rn(pv.y, w[it].y), __fsub_rn(pv.z, w[it].z), __fsub_rn(pv.w, w[it].w));
    }
    for (int k = 0; k < n_mix; ++k) {
      const float4* mk = mu + ((int64_t)k * segs + seg) * (kGroupElems / 4);
      const int64_t gk = (int64_t)k * n_groups + g;
      float4 v[8];
      float m[8];
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const float4 c = __ldg(mk + it * 32 + lane);
        v[it] = make_float4(__fadd_rn(w[it].x, __fmul_rn(d[it].x, c.x)), __fadd_rn(w[it].y, __fmul_rn(d[it].y, c.y)),
                            __fadd_rn(w[it].z, __fmul_rn(d[it].z, c.z)), __fadd_rn(w[it].w, __fmul_rn(d[it].w, c.w)));
        m[it] = fmaxf(fmaxf(fabsf(v[it].x), fabsf(v[it].y)), fmaxf(fabsf(v[it].z), fabsf(v[it].w)));
      }
      butterfly_max<8, 2>(m, lane);                 // m[0]: amax of block it_own over the warp
      const int it_own = bitrev<3>(lane & 7);
      float Mj = m[0];
      Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 1));
      Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 2));
      Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 4));
      uint32_t sb; float D;
      block_scale(m[0], Mj, sb, D);
      const float r = __frcp_rn(D);
      if (lane < 8) sc8[gk * 8 + it_own] = (uint8_t)sb;
      if (lane == 0) sc32[gk] = Mj;
      uint32_t* dst = q + gk * (kGroupElems / 4);
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int srcl = bitrev<3>(it);
        const float Di = __shfl_sync(0xffffffffu, D, srcl);
        const float ri = __shfl_sync(0xffffffffu, r, srcl);
        const float2 nD2 = make_float2(-Di, -Di), r2 = make_float2(ri, ri);
        const uint32_t p0 = div_hoisted_pack2(v[it].x, v[it].y, nD2, r2);
        const uint32_t p1 = div_hoisted_pack2(v[it].z, v[it].w, nD2, r2);
        __stcs(dst + it * 32 + lane, bf16x2_to_fp8x2<FMT>(p0) | (bf16x2_to_fp8x2<FMT>(p1) << 16));
      }
    }
  }
}

// The middle of ChannelMix (pratchya/_nnx_impl/_module.py:246-251) in one pass over the f32 product
// y of its first Linear:  k = dq(q(y, (1,128))) in f32 (what Linear.__call__ returns for an f32 input,
// :46-50), k = relu(k)^2 (:249), then the second Linear's own quantize_impl(k, (1,128)) (:46-47).  Both
// quantizations partition a row into the same 1024-element super-groups, so a warp keeps its
// super-group in registers across the three steps.  The bits are those of pb_fake_quantize, an f32
// relu and square, and pb_quantize.
template <int FMT, bool PREP>
__global__ void __launch_bounds__(kRowThreads)
relu2_requantize_row128_f32_kernel(const float4* __restrict__ y, uint32_t* __restrict__ q, uint8_t* __restrict__ sc8,
                                   float* __restrict__ sc32, int64_t n_groups, const GemmPrepOut prep) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * (kRowThreads / 32);
  for (int64_t g = (int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5); g < n_groups; g += warps_total) {
    const float4* src = y + g * (kGroupElems / 4);
    float4 w[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) w[it] = __ldcs(src + it * 32 + lane);
    float m[8];
    {   // ---- k = relu(dq(q(y)))^2, in place
#pragma unroll
      for (int it = 0; it < 8; ++it)
        m[it] = fmaxf(fmaxf(fabsf(w[it].x), fabsf(w[it].y)), fmaxf(fabsf(w[it].z), fabsf(w[it].w)));
      butterfly_max<8, 2>(m, lane);
      float Mj = m[0];
      Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 1));
      Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 2));
      Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 4));
      uint32_t sb; float D;
      block_scale(m[0], Mj, sb, D);
      const float r = __frcp_rn(D);
      const float x_sc = __fmul_rn(e8m0_to_f32(sb), Mj);
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int srcl = bitrev<3>(it);
        const float Di = __shfl_sync(0xffffffffu, D, srcl);
        const float ri = __shfl_sync(0xffffffffu, r, srcl);
        const float si = __shfl_sync(0xffffffffu, x_sc, srcl);
        const float2 nD2 = make_float2(-Di, -Di), r2 = make_float2(ri, ri);
        const uint32_t p0 = div_hoisted_pack2(w[it].x, w[it].y, nD2, r2);
        const uint32_t p1 = div_hoisted_pack2(w[it].z, w[it].w, nD2, r2);
        const float2 a = fp8x2_to_f32x2<FMT>((uint16_t)bf16x2_to_fp8x2<FMT>(p0));
        const float2 b = fp8x2_to_f32x2<FMT>((uint16_t)bf16x2_to_fp8x2<FMT>(p1));
        const float k128 = 0.0078125f;
        const float t0 = fmaxf(__fmul_rn(__fmul_rn(a.x, si), k128), 0.0f), t1 = fmaxf(__fmul_rn(__fmul_rn(a.y, si), k128), 0.0f);
        const float t2 = fmaxf(__fmul_rn(__fmul_rn(b.x, si), k128), 0.0f), t3 = fmaxf(__fmul_rn(__fmul_rn(b.y, si), k128), 0.0f);
        w[it] = make_float4(__fmul_rn(t0, t0), __fmul_rn(t1, t1), __fmul_rn(t2, t2), __fmul_rn(t3, t3));
      }
    }
    // ---- quantize_impl(k, (1,128)): the f32 row kernel on the values now in registers (all >= 0)
#pragma unroll
    for (int it = 0; it < 8; ++it) m[it] = fmaxf(fmaxf(w[it].x, w[it].y), fmaxf(w[it].z, w[it].w));
    butterfly_max<8, 2>(m, lane);
    const int it_own = bitrev<3>(lane & 7);
    float Mj = m[0];
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 1));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 2));
    Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, 4));
    uint32_t sb; float D;
    block_scale(m[0], Mj, sb, D);
    const float r = __frcp_rn(D);
    if (lane < 8) sc8[g * 8 + it_own] = (uint8_t)sb;
    if (lane == 0) sc32[g] = Mj;
    if (PREP) write_gemm_prep(prep, g, it_own, sb, Mj, lane < 8, lane == 0);
    uint32_t* dst = q + g * (kGroupElems / 4);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int srcl = bitrev<3>(it);
      const float Di = __shfl_sync(0xffffffffu, D, srcl);
      const float ri = __shfl_sync(0xffffffffu, r, srcl);
      const float2 nD2 = make_float2(-Di, -Di), r2 = make_float2(ri, ri);
      const uint32_t p0 = div_hoisted_pack2(w[it].x, w[it].y, nD2, r2);
      const uint32_t p1 = div_hoisted_pack2(w[it].z, w[it].w, nD2, r2);
      __stcs(dst + it * 32 + lane, bf16x2_to_fp8x2<FMT>(p0) | (bf16x2_to_fp8x2<FMT>(p1) << 16));
    }
  }
}

// ---------------------------------------------------------------------------------
// Generic path.  Scratch layout: uint32 amax_bits[batch*Nb] | float divisor[batch*Nb].
struct GenericDims {
  VecIndexer idx;
  uint32_t total_vecs;
};

template <typename InT, int VEC>
__device__ __forceinline__ void load_vec(const InT* p, float (&v)[VEC]) {
  if constexpr (VEC == 1) {
    v[0] = Elem<InT>::to_f32(p[0]);
  } else if constexpr (VEC == 16 && sizeof(InT) == 4) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 t = __ldcs(reinterpret_cast<const float4*>(p) + j);
      v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
    }
  } else if constexpr (VEC == 16) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint4 t = __ldcs(reinterpret_cast<const uint4*>(p) + j);
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) { v[8 * j + 2 * k] = __uint_as_float(w[k] << 16); v[8 * j + 2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u); }
    }
  } else if constexpr (sizeof(InT) == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
  }
}

template <typename InT, int VEC>
__global__ void __launch_bounds__(256)
generic_amax_kernel(const InT* __restrict__ x, uint32_t* __restrict__ amax_bits, GenericDims d) {
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; ; i += stride) {
    // whole warps leave together: lane 0 holds the warp's smallest index
    const bool active = i < d.total_vecs;
    if (__all_sync(0xffffffffu, !active)) break;
    uint32_t bits = 0;
    uint32_t blk = 0xffffffffu;
    if (active) {
      float v[VEC];
      load_vec<InT, VEC>(x + (size_t)i * VEC, v);
      float m = fabsf(v[0]);
#pragma unroll
      for (int j = 1; j < VEC; ++j) m = fmaxf(m, fabsf(v[j]));
      bits = __float_as_uint(m);          // non-negative floats order like unsigned ints
      blk = d.idx.block_of(i);
    }
    const uint32_t blk0 = __shfl_sync(0xffffffffu, blk, 0);
    if (__all_sync(0xffffffffu, blk == blk0)) {
      const uint32_t mx = __reduce_max_sync(0xffffffffu, bits);
      if ((threadIdx.x & 31) == 0) atomicMax(amax_bits + blk0, mx);
    } else if (active) {
      atomicMax(amax_bits + blk, bits);
    }
  }
}

// One warp per super-group when K >= 32, else one thread per super-group.
template <bool WARP_PER_GROUP>
__global__ void __launch_bounds__(256)
generic_scale_kernel(const uint32_t* __restrict__ amax_bits, float* __restrict__ divisor,
                     uint8_t* __restrict__ sc8, float* __restrict__ sc32, int64_t n_groups, int64_t K) {
  if constexpr (WARP_PER_GROUP) {
    const int lane = threadIdx.x & 31;
    const int64_t g = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (g >= n_groups) return;
    float Mj = 0.0f;
    for (int64_t k = lane; k < K; k += 32) Mj = fmaxf(Mj, __uint_as_float(amax_bits[g * K + k]));
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) Mj = fmaxf(Mj, __shfl_xor_sync(0xffffffffu, Mj, s));
    for (int64_t k = lane; k < K; k += 32) {
      uint32_t sb; float D;
      block_scale(__uint_as_float(amax_bits[g * K + k]), Mj, sb, D);
      sc8[g * K + k] = (uint8_t)sb;
      divisor[g * K + k] = D;
    }
    if (lane == 0) sc32[g] = Mj;
  } else {
    const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= n_groups) return;
    float Mj = 0.0f;
    for (int64_t k = 0; k < K; ++k) Mj = fmaxf(Mj, __uint_as_float(amax_bits[g * K + k]));
    for (int64_t k = 0; k < K; ++k) {
      uint32_t sb; float D;
      block_scale(__uint_as_float(amax_bits[g * K + k]), Mj, sb, D);
      sc8[g * K + k] = (uint8_t)sb;
      divisor[g * K + k] = D;
    }
    sc32[g] = Mj;
  }
}

}  // namespace

// Per-block amax bits -> e8m0 bytes, fp32 amax and per-block divisors (shared with the
// transposed quantizer).
int launch_group_scales(const uint32_t* amax_bits, float* divisor, uint8_t* sc8, float* sc32, int64_t n_groups, int64_t K, cudaStream_t st) {
  if (K >= 32) {
    generic_scale_kernel<true><<<(unsigned)((n_groups * 32 + 255) / 256), 256, 0, st>>>(amax_bits, divisor, sc8, sc32, n_groups, K);
  } else {
    generic_scale_kernel<false><<<(unsigned)((n_groups + 255) / 256), 256, 0, st>>>(amax_bits, divisor, sc8, sc32, n_groups, K);
  }
  PB_LAUNCH_CHECK("generic_scale_kernel");
  return PB_OK;
}

namespace {

template <typename InT, int VEC, int FMT>
__global__ void __launch_bounds__(256)
generic_apply_kernel(const InT* __restrict__ x, const float* __restrict__ divisor,
                     uint8_t* __restrict__ q, GenericDims d) {
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < d.total_vecs; i += stride) {
    float v[VEC];
    load_vec<InT, VEC>(x + (size_t)i * VEC, v);
    const float D = divisor[d.idx.block_of(i)];
    const float r = __frcp_rn(D);
    if constexpr (VEC == 1) {
      const uint32_t p = pack_bf16x2(div_hoisted(v[0], D, r), 0.0f);
      q[i] = (uint8_t)(bf16x2_to_fp8x2<FMT>(p) & 0xffu);
    } else if constexpr (VEC == 16) {
      const float2 nD2 = make_float2(-D, -D), r2 = make_float2(r, r);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = bf16x2_to_fp8x2<FMT>(div_hoisted_pack2(v[4 * j], v[4 * j + 1], nD2, r2)) |
               (bf16x2_to_fp8x2<FMT>(div_hoisted_pack2(v[4 * j + 2], v[4 * j + 3], nD2, r2)) << 16);
      __stcs(reinterpret_cast<uint4*>(q) + i, make_uint4(o[0], o[1], o[2], o[3]));
    } else {
      const uint32_t p0 = pack_bf16x2(div_hoisted(v[0], D, r), div_hoisted(v[1], D, r));
      const uint32_t p1 = pack_bf16x2(div_hoisted(v[2], D, r), div_hoisted(v[3], D, r));
      reinterpret_cast<uint32_t*>(q)[i] = bf16x2_to_fp8x2<FMT>(p0) | (bf16x2_to_fp8x2<FMT>(p1) << 16);
    }
  }
}

int grid_for(int64_t work_items, int threads, int ctas_per_sm) {
  const int64_t need = (work_items + threads - 1) / threads;
  const int64_t cap = (int64_t)sm_count() * ctas_per_sm;
  return (int)(need < cap ? (need > 0 ? need : 1) : cap);
}

template <typename InT, int VEC>
int launch_generic(const InT* x, const Geometry& g, int64_t batch, int fmt, uint8_t* q, uint8_t* sc8, float* sc32,
                   void* workspace, cudaStream_t st) {
  const int64_t nblk = batch * g.Nb;
  uint32_t* amax_bits = static_cast<uint32_t*>(workspace);
  float* divisor = reinterpret_cast<float*>(amax_bits + nblk);
  const int64_t total = batch * g.rows * g.cols;
  if (total / VEC > kMaxIndexed || batch * g.rows > kMaxIndexed)
    return fail(PB_ERR_UNSUPPORTED, "pb_quantize: %lld elements exceed the 31-bit index range of the generic kernels", (long long)total);
  GenericDims d{VecIndexer(g.cols, g.a, g.b, VEC), (uint32_t)(total / VEC)};
  PB_CUDA_TRY(cudaMemsetAsync(amax_bits, 0, nblk * sizeof(uint32_t), st));
  const int grid = grid_for(d.total_vecs, 256, 8);
  generic_amax_kernel<InT, VEC><<<grid, 256, 0, st>>>(x, amax_bits, d);
  PB_LAUNCH_CHECK("generic_amax_kernel");
  if (int s = launch_group_scales(amax_bits, divisor, sc8, sc32, batch * g.M, g.K, st)) return s;
  if (fmt == PB_E4M3) generic_apply_kernel<InT, VEC, PB_E4M3><<<grid, 256, 0, st>>>(x, divisor, q, d);
  else                generic_apply_kernel<InT, VEC, PB_E5M2><<<grid, 256, 0, st>>>(x, divisor, q, d);
  PB_LAUNCH_CHECK("generic_apply_kernel");
  return PB_OK;
}

bool row128_eligible(const Geometry& g) { return g.a == 1 && g.b == 128 && g.K == 8; }

}  // namespace

// First pass of pb_quantize_dual (transpose_quantize.cu): bf16 x[batch, rows, cols], rows % 128 == 0, cols % 1024 == 0.
int launch_row128_colmax(const void* x, int out_format, void* q, uint8_t* sc8, float* sc32, uint32_t* col_amax_bits,
                         int64_t batch, int64_t rows, int64_t cols, cudaStream_t st) {
  const dim3 grid((unsigned)(cols / 1024), (unsigned)(rows / 128), (unsigned)batch);
  if (out_format == PB_E4M3)
    quantize_row128_bf16_colmax_kernel<PB_E4M3><<<grid, kRowThreads, 0, st>>>((const uint4*)x, (uint2*)q, sc8, sc32, col_amax_bits, (int)rows, (int)cols);
  else
    quantize_row128_bf16_colmax_kernel<PB_E5M2><<<grid, kRowThreads, 0, st>>>((const uint4*)x, (uint2*)q, sc8, sc32, col_amax_bits, (int)rows, (int)cols);
  PB_LAUNCH_CHECK("quantize_row128_bf16_colmax_kernel");
  return PB_OK;
}
}  // namespace pb

using namespace pb;

extern "C" size_t pb_quantize_workspace_size(int64_t batch, int64_t rows, int64_t cols, int a, int b) {
  Geometry g;
  if (batch <= 0 || make_geometry(rows, cols, a, b, &g) != PB_OK) return 0;
  if (row128_eligible(g)) return 0;
  return (size_t)(batch * g.Nb) * 8;
}

namespace pb {
// defined in gemm_sm100.cu: where the A operand's prepared scales live inside a GEMM workspace
int gemm_a_prep_location(const pb_operand* a, const pb_operand* b, void* workspace, size_t workspace_bytes,
                         uint8_t** sf, float** f, uint32_t* tiles, uint32_t* Mpad, void* stream);
}

static int quantize_entry(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols,
                          int a, int b, int out_format, void* q, uint8_t* sc8, float* sc32,
                          void* workspace, size_t workspace_bytes, void* stream, const GemmPrepOut& prep) {
  if (!x || !q || !sc8 || !sc32) return fail(PB_ERR_NULL_POINTER, "pb_quantize: x, q, sc8 and sc32 must be non-null");
  if (batch <= 0) return fail(PB_ERR_BAD_SHAPE, "pb_quantize: batch=%lld must be positive", (long long)batch);
  if (x_dtype != PB_F32 && x_dtype != PB_BF16) return fail(PB_ERR_BAD_DTYPE, "pb_quantize: x_dtype %d is neither PB_F32 nor PB_BF16", x_dtype);
  if (out_format != PB_E4M3 && out_format != PB_E5M2) return fail(PB_ERR_BAD_DTYPE, "pb_quantize: out_format %d is neither PB_E4M3 nor PB_E5M2", out_format);
  Geometry g;
  if (int s = make_geometry(rows, cols, a, b, &g)) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  if (row128_eligible(g)) {
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7))
      return fail(PB_ERR_MISALIGNED, "pb_quantize: x must be 16-byte and q 8-byte aligned");
    const int64_t n_groups = batch * g.M;
    // 8 CTAs per SM, 16 once every warp then still gets three super-groups or more (measured: X[8192,2048] is
    // best at 8, X[32768,2048] and larger at 16); PB_QUANT_CTAS_PER_SM overrides
    static const int forced_ctas = [] { const int v = env_switch("PB_QUANT_CTAS_PER_SM", 0); return v > 0 ? v : 0; }();
    const int ctas_per_sm = forced_ctas ? forced_ctas : (n_groups >= (int64_t)sm_count() * 16 * (kRowThreads / 32) * 3 ? 16 : 8);
    const int grid = grid_for(n_groups * 32, kRowThreads, ctas_per_sm);
    // 40 registers per thread (6 CTAs of 256 threads per SM) measures the same as the compiler's
    // unconstrained 49; an unconstrained single CTA per SM (96 registers) is 15 % slower.
    const bool e4 = out_format == PB_E4M3;
#define PB_ROW128_LAUNCH(KERNEL, XT, QT) KERNEL<<<grid, kRowThreads, 0, st>>>((const XT*)x, (QT*)q, sc8, sc32, n_groups, prep)
    static const bool wide = env_switch("PB_QUANT_WIDE", 1) != 0;
    if (x_dtype == PB_BF16 && wide && (reinterpret_cast<uintptr_t>(x) & 31) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0) {
      if (prep.sf) {
        if (e4) PB_ROW128_LAUNCH((quantize_row128_bf16_wide_kernel<PB_E4M3, 6, true>), uint8_t, uint4);
        else    PB_ROW128_LAUNCH((quantize_row128_bf16_wide_kernel<PB_E5M2, 6, true>), uint8_t, uint4);
      } else {
        if (e4) PB_ROW128_LAUNCH((quantize_row128_bf16_wide_kernel<PB_E4M3, 6, false>), uint8_t, uint4);
        else    PB_ROW128_LAUNCH((quantize_row128_bf16_wide_kernel<PB_E5M2, 6, false>), uint8_t, uint4);
      }
    } else if (x_dtype == PB_BF16) {
      if (prep.sf) {
        if (e4) PB_ROW128_LAUNCH((quantize_row128_bf16_kernel<PB_E4M3, 6, true>), uint4, uint2);
        else    PB_ROW128_LAUNCH((quantize_row128_bf16_kernel<PB_E5M2, 6, true>), uint4, uint2);
      } else {
        if (e4) PB_ROW128_LAUNCH((quantize_row128_bf16_kernel<PB_E4M3, 6, false>), uint4, uint2);
        else    PB_ROW128_LAUNCH((quantize_row128_bf16_kernel<PB_E5M2, 6, false>), uint4, uint2);
      }
    } else {
      if (prep.sf) {
        if (e4) PB_ROW128_LAUNCH((quantize_row128_f32_kernel<PB_E4M3, true>), float4, uint32_t);
        else    PB_ROW128_LAUNCH((quantize_row128_f32_kernel<PB_E5M2, true>), float4, uint32_t);
      } else {
        if (e4) PB_ROW128_LAUNCH((quantize_row128_f32_kernel<PB_E4M3, false>), float4, uint32_t);
        else    PB_ROW128_LAUNCH((quantize_row128_f32_kernel<PB_E5M2, false>), float4, uint32_t);
      }
    }
#undef PB_ROW128_LAUNCH
    PB_LAUNCH_CHECK("quantize_row128_kernel");
    return PB_OK;
  }

  const size_t need = (size_t)(batch * g.Nb) * 8;
  if (!workspace || workspace_bytes < need)
    return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_quantize: grid (%d,%d) needs %zu bytes of workspace, got %zu", a, b, need, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 3) return fail(PB_ERR_MISALIGNED, "pb_quantize: workspace must be 4-byte aligned");
  const bool vec4 = (b % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(q) % 4 == 0);
  const bool vec16 = (b % 16 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(q) % 16 == 0);
  if (vec16) {      // 16 elements per thread: whole sectors in, one 16-byte store out
    if (x_dtype == PB_BF16) return launch_generic<__nv_bfloat16, 16>((const __nv_bfloat16*)x, g, batch, out_format, (uint8_t*)q, sc8, sc32, workspace, st);
    return launch_generic<float, 16>((const float*)x, g, batch, out_format, (uint8_t*)q, sc8, sc32, workspace, st);
  }
  if (x_dtype == PB_BF16) {
    return vec4 ? launch_generic<__nv_bfloat16, 4>((const __nv_bfloat16*)x, g, batch, out_format, (uint8_t*)q, sc8, sc32, workspace, st)
                : launch_generic<__nv_bfloat16, 1>((const __nv_bfloat16*)x, g, batch, out_format, (uint8_t*)q, sc8, sc32, workspace, st);
  }
  return vec4 ? launch_generic<float, 4>((const float*)x, g, batch, out_format, (uint8_t*)q, sc8, sc32, workspace, st)
              : launch_generic<float, 1>((const float*)x, g, batch, out_format, (uint8_t*)q, sc8, sc32, workspace, st);
}

extern "C" int pb_quantize(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols,
                           int a, int b, int out_format, void* q, uint8_t* sc8, float* sc32,
                           void* workspace, size_t workspace_bytes, void* stream) {
  return quantize_entry(x, x_dtype, batch, rows, cols, a, b, out_format, q, sc8, sc32, workspace, workspace_bytes, stream,
                        GemmPrepOut{nullptr, nullptr, 1, 1, 0});
}

extern "C" int pb_quantize_for_gemm(const void* x, int x_dtype, int64_t rows, int64_t cols, int out_format,
                                    void* q, uint8_t* sc8, float* sc32,
                                    const pb_operand* b, void* gemm_workspace, size_t gemm_workspace_bytes, void* stream) {
  if (cols <= 0 || cols % 1024 != 0)
    return fail(PB_ERR_BAD_SHAPE, "pb_quantize_for_gemm: cols=%lld must be a positive multiple of 1024", (long long)cols);
  GemmPrepOut prep{nullptr, nullptr, (uint32_t)(cols / 128), 0, 0};
  if (!x || !q || !sc8 || !sc32) return fail(PB_ERR_NULL_POINTER, "pb_quantize_for_gemm: x, q, sc8 and sc32 must be non-null");
  if (rows <= 0 || rows * (cols / 128) > kMaxIndexed) return fail(PB_ERR_UNSUPPORTED, "pb_quantize_for_gemm: rows=%lld is out of range", (long long)rows);
  pb_operand a_op;
  a_op.q = q; a_op.sc8 = sc8; a_op.sc32 = sc32; a_op.rows = rows; a_op.depth = cols;
  a_op.grid_a = 1; a_op.grid_b = 128; a_op.format = out_format; a_op.transposed_blocks = 0;
  if (int s = pb::gemm_a_prep_location(&a_op, b, gemm_workspace, gemm_workspace_bytes, &prep.sf, &prep.f, &prep.tiles, &prep.Mpad, stream)) return s;
  return quantize_entry(x, x_dtype, 1, rows, cols, 1, 128, out_format, q, sc8, sc32, nullptr, 0, stream, prep);
}

extern "C" int pb_relu2_requantize(const void* y, int64_t rows, int64_t cols, int out_format, void* q, uint8_t* sc8, float* sc32,
                                   const pb_operand* b, void* gemm_workspace, size_t gemm_workspace_bytes, void* stream) {
  if (!y || !q || !sc8 || !sc32) return fail(PB_ERR_NULL_POINTER, "pb_relu2_requantize: y, q, sc8 and sc32 must be non-null");
  if (out_format != PB_E4M3 && out_format != PB_E5M2) return fail(PB_ERR_BAD_DTYPE, "pb_relu2_requantize: out_format %d is neither PB_E4M3 nor PB_E5M2", out_format);
  if (rows <= 0 || cols <= 0 || cols % 1024 != 0)
    return fail(PB_ERR_UNSUPPORTED, "pb_relu2_requantize: [%lld, %lld]: cols must be a positive multiple of 1024 (whole super-groups per row)", (long long)rows, (long long)cols);
  if (rows * (cols / 128) > kMaxIndexed) return fail(PB_ERR_UNSUPPORTED, "pb_relu2_requantize: too many blocks");
  if ((reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(q) & 3))
    return fail(PB_ERR_MISALIGNED, "pb_relu2_requantize: y must be 16-byte and q 4-byte aligned");
  GemmPrepOut prep{nullptr, nullptr, (uint32_t)(cols / 128), 0, 0};
  if (b) {      // also lay the scales out for the GEMM against b, as pb_quantize_for_gemm does
    pb_operand a_op;
    a_op.q = q; a_op.sc8 = sc8; a_op.sc32 = sc32; a_op.rows = rows; a_op.depth = cols;
    a_op.grid_a = 1; a_op.grid_b = 128; a_op.format = out_format; a_op.transposed_blocks = 0;
    if (int s = pb::gemm_a_prep_location(&a_op, b, gemm_workspace, gemm_workspace_bytes, &prep.sf, &prep.f, &prep.tiles, &prep.Mpad, stream)) return s;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n_groups = rows * (cols / 1024);
  const int grid = grid_for(n_groups * 32, kRowThreads, 8);
  const bool e4 = out_format == PB_E4M3;
  if (prep.sf) {
    if (e4) relu2_requantize_row128_f32_kernel<PB_E4M3, true><<<grid, kRowThreads, 0, st>>>((const float4*)y, (uint32_t*)q, sc8, sc32, n_groups, prep);
    else    relu2_requantize_row128_f32_kernel<PB_E5M2, true><<<grid, kRowThreads, 0, st>>>((const float4*)y, (uint32_t*)q, sc8, sc32, n_groups, prep);
  } else {
    if (e4) relu2_requantize_row128_f32_kernel<PB_E4M3, false><<<grid, kRowThreads, 0, st>>>((const float4*)y, (uint32_t*)q, sc8, sc32, n_groups, prep);
    else    relu2_requantize_row128_f32_kernel<PB_E5M2, false><<<grid, kRowThreads, 0, st>>>((const float4*)y, (uint32_t*)q, sc8, sc32, n_groups, prep);
  }
  PB_LAUNCH_CHECK("relu2_requantize_row128_f32_kernel");
  return PB_OK;
}

namespace pb {   // transpose_quantize.cu
int launch_scaled_transposed(const float* g, const uint8_t* y_sc8, const float* y_sc32, int out_format, uint8_t* q_t, uint8_t* sc8, float* sc32,
                             int64_t rows, int64_t cols, cudaStream_t st);
}

extern "C" int pb_dequantize_bwd_quantize_dual(const float* g, const uint8_t* y_sc8, const float* y_sc32, int64_t rows, int64_t cols, int out_format,
                                               uint8_t* q, uint8_t* sc8, float* sc32, uint8_t* q_t, uint8_t* sc8_t, float* sc32_t, void* stream) {
  if (!g || !y_sc8 || !y_sc32 || !q || !sc8 || !sc32 || !q_t || !sc8_t || !sc32_t)
    return fail(PB_ERR_NULL_POINTER, "pb_dequantize_bwd_quantize_dual: null argument");
  if (out_format != PB_E4M3 && out_format != PB_E5M2) return fail(PB_ERR_BAD_DTYPE, "pb_dequantize_bwd_quantize_dual: out_format %d is neither PB_E4M3 nor PB_E5M2", out_format);
  if (rows <= 0 || cols <= 0 || cols % 1024 != 0 || rows % 1024 != 0)
    return fail(PB_ERR_UNSUPPORTED, "pb_dequantize_bwd_quantize_dual: [%lld, %lld]: rows and cols must be positive multiples of 1024", (long long)rows, (long long)cols);
  if (rows * (cols / 128) > kMaxIndexed) return fail(PB_ERR_UNSUPPORTED, "pb_dequantize_bwd_quantize_dual: too many blocks");
  if ((reinterpret_cast<uintptr_t>(g) & 15) || (reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(q_t) & 31))
    return fail(PB_ERR_MISALIGNED, "pb_dequantize_bwd_quantize_dual: g must be 16-byte, q 4-byte and q_t 32-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n_groups = rows * (cols / 1024);
  const int grid = grid_for(n_groups * 32, kRowThreads, 8);
  if (out_format == PB_E4M3)
    scaled_quantize_row128_f32_kernel<PB_E4M3, false><<<grid, kRowThreads, 0, st>>>(reinterpret_cast<const float4*>(g), y_sc8, y_sc32, reinterpret_cast<uint32_t*>(q), sc8, sc32, n_groups);
  else
    scaled_quantize_row128_f32_kernel<PB_E5M2, false><<<grid, kRowThreads, 0, st>>>(reinterpret_cast<const float4*>(g), y_sc8, y_sc32, reinterpret_cast<uint32_t*>(q), sc8, sc32, n_groups);
  PB_LAUNCH_CHECK("scaled_quantize_row128_f32_kernel");
  return pb::launch_scaled_transposed(g, y_sc8, y_sc32, out_format, q_t, sc8_t, sc32_t, rows, cols, st);
}

namespace pb {   // transpose_quantize.cu
int launch_relu2_transposed(const float* k, uint8_t* q_t, uint8_t* sc8, float* sc32, int64_t rows, int64_t cols, cudaStream_t st);
}

extern "C" int pb_relu2_quantize_dual(const float* k, int64_t rows, int64_t cols, uint8_t* q, uint8_t* sc8, float* sc32,
                                      uint8_t* q_t, uint8_t* sc8_t, float* sc32_t, void* stream) {
  if (!k || !q || !sc8 || !sc32 || !q_t || !sc8_t || !sc32_t) return fail(PB_ERR_NULL_POINTER, "pb_relu2_quantize_dual: null argument");
  if (rows <= 0 || cols <= 0 || cols % 1024 != 0 || rows % 1024 != 0)
    return fail(PB_ERR_UNSUPPORTED, "pb_relu2_quantize_dual: [%lld, %lld]: rows and cols must be positive multiples of 1024", (long long)rows, (long long)cols);
  if (rows * (cols / 128) > kMaxIndexed) return fail(PB_ERR_UNSUPPORTED, "pb_relu2_quantize_dual: too many blocks");
  if ((reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(q_t) & 31))
    return fail(PB_ERR_MISALIGNED, "pb_relu2_quantize_dual: k must be 16-byte, q 4-byte and q_t 32-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n_groups = rows * (cols / 1024);
  const int grid = grid_for(n_groups * 32, kRowThreads, 8);
  scaled_quantize_row128_f32_kernel<PB_E4M3, true><<<grid, kRowThreads, 0, st>>>(reinterpret_cast<const float4*>(k), nullptr, nullptr,
                                                                               reinterpret_cast<uint32_t*>(q), sc8, sc32, n_groups);
  PB_LAUNCH_CHECK("scaled_quantize_row128_f32_kernel");
  return pb::launch_relu2_transposed(k, q_t, sc8_t, sc32_t, rows, cols, st);
}

namespace pb {   // transpose_quantize.cu
int launch_shift_lerp_transposed(const float* x, const float* state, const float* mu, uint8_t* q_t, uint8_t* sc8, float* sc32,
                                 int64_t rows, int64_t steps, int64_t cols, cudaStream_t st);
}

extern "C" int pb_shift_lerp_quantize(const float* x, const float* state, const float* mu, int64_t batch, int64_t steps, int64_t channels,
                                      int n_mix, uint8_t* q, uint8_t* sc8, float* sc32, unsigned int transposed_mask,
                                      uint8_t* q_t, uint8_t* sc8_t, float* sc32_t, void* stream) {
  if (!x || !mu || !q || !sc8 || !sc32) return fail(PB_ERR_NULL_POINTER, "pb_shift_lerp_quantize: x, mu, q, sc8 and sc32 must be non-null");
  if (n_mix <= 0 || n_mix > 8) return fail(PB_ERR_UNSUPPORTED, "pb_shift_lerp_quantize: n_mix=%d (1..8)", n_mix);
  if (batch <= 0 || steps <= 0 || channels <= 0 || channels % 1024 != 0 || steps > 0x7fffffffll)
    return fail(PB_ERR_UNSUPPORTED, "pb_shift_lerp_quantize: batch=%lld steps=%lld channels=%lld: channels must be a positive multiple of 1024 "
                "(whole super-groups per token)", (long long)batch, (long long)steps, (long long)channels);
  const int64_t rows = batch * steps;
  if (rows * (channels / 128) * n_mix > kMaxIndexed) return fail(PB_ERR_UNSUPPORTED, "pb_shift_lerp_quantize: too many blocks");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(state) & 15) || (reinterpret_cast<uintptr_t>(mu) & 15) ||
      (reinterpret_cast<uintptr_t>(q) & 3))
    return fail(PB_ERR_MISALIGNED, "pb_shift_lerp_quantize: x, state and mu must be 16-byte and q 4-byte aligned");
  transposed_mask &= (1u << n_mix) - 1u;
  if (transposed_mask) {
    if (!q_t || !sc8_t || !sc32_t) return fail(PB_ERR_NULL_POINTER, "pb_shift_lerp_quantize: a transposed form was asked for without its outputs");
    if (steps % 1024 != 0)
      return fail(PB_ERR_UNSUPPORTED, "pb_shift_lerp_quantize: the transposed forms need steps %% 1024 == 0 (a 1024-token super-group inside one sequence), got %lld",
                  (long long)steps);
    if (reinterpret_cast<uintptr_t>(q_t) & 31) return fail(PB_ERR_MISALIGNED, "pb_shift_lerp_quantize: q_t must be 32-byte aligned");
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int segs = (int)(channels / 1024);
  const int64_t n_groups = rows * segs;
  const int grid = grid_for(n_groups * 32, kRowThreads, 4);
  shift_lerp_quantize_row128_kernel<PB_E4M3><<<grid, kRowThreads, 0, st>>>(
      reinterpret_cast<const float4*>(x), reinterpret_cast<const float4*>(state), reinterpret_cast<const float4*>(mu),
      reinterpret_cast<uint32_t*>(q), sc8, sc32, n_groups, segs, (int)steps, n_mix);
  PB_LAUNCH_CHECK("shift_lerp_quantize_row128_kernel");
  int slot = 0;
  for (int k = 0; k < n_mix; ++k) {
    if (!(transposed_mask >> k & 1u)) continue;
    const int64_t n = rows * channels;
    if (int s = pb::launch_shift_lerp_transposed(x, state, mu + (int64_t)k * channels, q_t + slot * n, sc8_t + slot * (n / 128), sc32_t + slot * (n / 1024),
                                                 rows, steps, channels, st))
      return s;
    ++slot;
  }
  return PB_OK;
}

extern "C" int pb_fake_quantize(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols, int a, int b,
                                int out_format, void* out, int out_dtype, void* stream) {
  if (!x || !out) return fail(PB_ERR_NULL_POINTER, "pb_fake_quantize: x and out must be non-null");
  if (batch <= 0) return fail(PB_ERR_BAD_SHAPE, "pb_fake_quantize: batch=%lld must be positive", (long long)batch);
  if (out_format != PB_E4M3 && out_format != PB_E5M2) return fail(PB_ERR_BAD_DTYPE, "pb_fake_quantize: out_format %d is neither PB_E4M3 nor PB_E5M2", out_format);
  if (out_dtype != PB_F32 && out_dtype != PB_BF16) return fail(PB_ERR_BAD_DTYPE, "pb_fake_quantize: out_dtype %d is neither PB_F32 nor PB_BF16", out_dtype);
  Geometry g;
  if (int s = make_geometry(rows, cols, a, b, &g)) return s;
  if (x_dtype != PB_F32 || !row128_eligible(g))
    return fail(PB_ERR_UNSUPPORTED, "pb_fake_quantize: only f32 input on the (1,128) grid with 8-block super-groups; use pb_quantize + pb_dequantize");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return fail(PB_ERR_MISALIGNED, "pb_fake_quantize: x and out must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n_groups = batch * g.M;
  const int grid = grid_for(n_groups * 32, kRowThreads, 8);
  const bool e4 = out_format == PB_E4M3;
  if (out_dtype == PB_F32) {
    if (e4) fake_quantize_row128_f32_kernel<PB_E4M3, float><<<grid, kRowThreads, 0, st>>>((const float4*)x, (float4*)out, n_groups);
    else    fake_quantize_row128_f32_kernel<PB_E5M2, float><<<grid, kRowThreads, 0, st>>>((const float4*)x, (float4*)out, n_groups);
  } else {
    if (e4) fake_quantize_row128_f32_kernel<PB_E4M3, __nv_bfloat16><<<grid, kRowThreads, 0, st>>>((const float4*)x, (uint2*)out, n_groups);
    else    fake_quantize_row128_f32_kernel<PB_E5M2, __nv_bfloat16><<<grid, kRowThreads, 0, st>>>((const float4*)x, (uint2*)out, n_groups);
  }
  PB_LAUNCH_CHECK("fake_quantize_row128_f32_kernel");
  return PB_OK;
}

// ---------------------------------------------------------------------------------------------
// Quantize without any caller-provided or library-allocated scratch.
//
// Some hosts of this library may not allocate device memory around a call: an XLA custom call
// that was registered without a scratch result, code running while a CUDA graph is being
// captured or replayed with fixed buffers, or a runtime whose allocator must not be re-entered
// from inside an op.  For them the scratch the generic quantizer needs (8 bytes per block: the
// block amax bits and the per-block divisors) lives in a fixed device array that is part of this
// library's image.  Every GPU that loads the library holds these 512 KiB until the process exits.
namespace pb {
namespace {

constexpr int64_t kStaticScratchBlocks = 65536;          // largest batch * Nb this entry point accepts
static __device__ __align__(256) unsigned char g_quantize_scratch[kStaticScratchBlocks * 8];

// Device address of g_quantize_scratch on the current device.  In host code the array's name
// is only a handle for the runtime, not an address a kernel can use; the real address is
// looked up once per device (with that device current) and cached.
int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* cached[64] = {nullptr};
  int dev = 0;
  PB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(PB_ERR_UNSUPPORTED, "pb_quantize_static: device ordinal %d is out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* p = nullptr;
    PB_CUDA_TRY(cudaGetSymbolAddress(&p, g_quantize_scratch));
    cached[dev] = p;
  }
  *out = cached[dev];
  return PB_OK;
}

}  // namespace
}  // namespace pb

extern "C" int pb_quantize_static(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols,
                                  int a, int b, int out_format, void* q, uint8_t* sc8, float* sc32, void* stream) {
  Geometry g;
  if (batch <= 0) return fail(PB_ERR_BAD_SHAPE, "pb_quantize_static: batch=%lld must be positive", (long long)batch);
  if (int s = make_geometry(rows, cols, a, b, &g)) return s;
  if (row128_eligible(g))      // this grid needs no scratch at all
    return pb_quantize(x, x_dtype, batch, rows, cols, a, b, out_format, q, sc8, sc32, nullptr, 0, stream);
  if (batch * g.Nb > kStaticScratchBlocks)
    return fail(PB_ERR_UNSUPPORTED,
                "pb_quantize_static: %lld blocks exceed the built-in scratch of %lld blocks; use pb_quantize with a caller workspace",
                (long long)(batch * g.Nb), (long long)kStaticScratchBlocks);
  void* scratch = nullptr;
  if (int s = static_scratch_address(&scratch)) return s;
  // pb_quantize clears the amax half of the scratch itself (cudaMemsetAsync on `stream`), so
  // whatever the previous call left behind is never read.
  return pb_quantize(x, x_dtype, batch, rows, cols, a, b, out_format, q, sc8, sc32, scratch,
                     (size_t)kStaticScratchBlocks * 8, stream);
}
