// Dequantizer and its cotangent (sm_100a).
// Replace dequantize_impl / dequantize_impl_bwd, pratchya/_qualia/_qarr.py:541-601:
//   out = f32(bf16(q)) * (f32(sc8 << 23) * sc32) / 128      (no 1e-7 floor on this side)
// Pure streaming: each thread converts 16 (or 1) consecutive elements of a row.
#include "common.cuh"

namespace pb {
namespace {

struct DqDims {
  VecIndexer idx;
  FastDiv by_K;
  uint32_t total_vecs;
};

__device__ __forceinline__ float block_multiplier(const DqDims& d, const uint8_t* __restrict__ sc8,
                                                  const float* __restrict__ sc32, uint32_t i) {
  const uint32_t blk = d.idx.block_of(i);
  // f32(sc8 << 23) * sc32, _qarr.py:562-563.  blk / K indexes sc32 across the batch because Nb = M*K.
  return __fmul_rn(e8m0_to_f32(__ldg(sc8 + blk)), __ldg(sc32 + d.by_K.div(blk)));
}

// (v * x_sc) / 128 with the reference's association, _qarr.py:564 and :597
__device__ __forceinline__ float apply_scale(float v, float x_sc) { return __fmul_rn(__fmul_rn(v, x_sc), 0.0078125f); }

template <typename OutT> __device__ __forceinline__ void store16(OutT* p, const float (&v)[16]);
template <> __device__ __forceinline__ void store16<float>(float* p, const float (&v)[16]) {
  if ((reinterpret_cast<uintptr_t>(p) & 31) == 0) {      // whole 32-byte sectors per store
#pragma unroll
    for (int j = 0; j < 2; ++j)
      asm volatile("st.global.cs.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                   ::"l"(p + 8 * j), "f"(v[8 * j]), "f"(v[8 * j + 1]), "f"(v[8 * j + 2]), "f"(v[8 * j + 3]),
                     "f"(v[8 * j + 4]), "f"(v[8 * j + 5]), "f"(v[8 * j + 6]), "f"(v[8 * j + 7]) : "memory");
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) __stcs(reinterpret_cast<float4*>(p) + j, make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
  }
}
template <> __device__ __forceinline__ void store16<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
  if ((reinterpret_cast<uintptr_t>(p) & 31) == 0) {      // one whole 32-byte sector per store
    asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
  } else {
    __stcs(reinterpret_cast<uint4*>(p), make_uint4(w[0], w[1], w[2], w[3]));
    __stcs(reinterpret_cast<uint4*>(p) + 1, make_uint4(w[4], w[5], w[6], w[7]));
  }
}

template <typename OutT, int FMT>
__device__ __forceinline__ void dequantize16(const uint4 w, float x_sc, OutT* dst) {
  const uint32_t in[4] = {w.x, w.y, w.z, w.w};
  float v[16];
  const float2 s2 = make_float2(x_sc, x_sc), k2 = make_float2(0.0078125f, 0.0078125f);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // (v * x_sc) / 128 on two elements at a time (packed f32x2 multiplies of sm_100): the bits of apply_scale
    const float2 lo = __fmul2_rn(__fmul2_rn(fp8x2_to_f32x2<FMT>((uint16_t)(in[j] & 0xffffu)), s2), k2);
    const float2 hi = __fmul2_rn(__fmul2_rn(fp8x2_to_f32x2<FMT>((uint16_t)(in[j] >> 16)), s2), k2);
    v[4 * j + 0] = lo.x; v[4 * j + 1] = lo.y;
    v[4 * j + 2] = hi.x; v[4 * j + 3] = hi.y;
  }
  store16<OutT>(dst, v);
}

template <typename OutT, int FMT, int VEC>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sc8, const float* __restrict__ sc32,
                  OutT* __restrict__ out, DqDims d) {
  const uint32_t stride = gridDim.x * blockDim.x;
  if constexpr (VEC == 16) {
    // two 16-byte vectors per iteration: both loads (and their scale lookups) are in flight together
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < d.total_vecs; i += 2 * stride) {
      const uint32_t i2 = i + stride;
      const uint4 w0 = __ldcs(reinterpret_cast<const uint4*>(q) + i);
      const uint4 w1 = __ldcs(reinterpret_cast<const uint4*>(q) + i2);
      const float s0 = block_multiplier(d, sc8, sc32, i);
      const float s1 = block_multiplier(d, sc8, sc32, i2);
      dequantize16<OutT, FMT>(w0, s0, out + (size_t)i * 16);
      dequantize16<OutT, FMT>(w1, s1, out + (size_t)i2 * 16);
    }
    if (i < d.total_vecs) {
      const uint4 w0 = __ldcs(reinterpret_cast<const uint4*>(q) + i);
      dequantize16<OutT, FMT>(w0, block_multiplier(d, sc8, sc32, i), out + (size_t)i * 16);
    }
  } else {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < d.total_vecs; i += stride) {
      const float x_sc = block_multiplier(d, sc8, sc32, i);
      const float2 f = fp8x2_to_f32x2<FMT>((uint16_t)q[i]);
      out[i] = Elem<OutT>::from_f32(apply_scale(f.x, x_sc));
    }
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
dequantize_bwd_kernel(const T* __restrict__ g, const uint8_t* __restrict__ sc8, const float* __restrict__ sc32,
                      T* __restrict__ out, DqDims d) {
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < d.total_vecs; i += stride) {
    const float x_sc = block_multiplier(d, sc8, sc32, i);
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      out[(size_t)i * VEC + j] = Elem<T>::from_f32(apply_scale(Elem<T>::to_f32(g[(size_t)i * VEC + j]), x_sc));
  }
}

// Grid (1,128) with 8-block super-groups: a super-group is 1024 consecutive bytes with eight e8m0
// bytes and one fp32 amax, so a warp takes a super-group per step (two in flight): lanes 0-7 form the
// eight block multipliers, every lane converts two 16-byte vectors and no index arithmetic is left.
template <typename OutT, int FMT>
__global__ void __launch_bounds__(256)
dequantize_row128_kernel(const uint4* __restrict__ q, const uint8_t* __restrict__ sc8, const float* __restrict__ sc32,
                         OutT* __restrict__ out, int64_t n_groups) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (int64_t)gridDim.x * 8;
  int64_t g = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  for (; g + warps_total < n_groups; g += 2 * warps_total) {
    const int64_t g2 = g + warps_total;
    const uint4 a0 = __ldcs(q + g * 64 + lane), a1 = __ldcs(q + g * 64 + 32 + lane);
    const uint4 b0 = __ldcs(q + g2 * 64 + lane), b1 = __ldcs(q + g2 * 64 + 32 + lane);
    float sa = 0.0f, sb = 0.0f;
    if (lane < 8) {
      sa = __fmul_rn(e8m0_to_f32(__ldg(sc8 + g * 8 + lane)), __ldg(sc32 + g));
      sb = __fmul_rn(e8m0_to_f32(__ldg(sc8 + g2 * 8 + lane)), __ldg(sc32 + g2));
    }
    // vector (it*32 + lane) holds elements of block it*4 + lane/8
    dequantize16<OutT, FMT>(a0, __shfl_sync(0xffffffffu, sa, lane >> 3), out + (g * 64 + lane) * 16);
    dequantize16<OutT, FMT>(a1, __shfl_sync(0xffffffffu, sa, 4 + (lane >> 3)), out + (g * 64 + 32 + lane) * 16);
    dequantize16<OutT, FMT>(b0, __shfl_sync(0xffffffffu, sb, lane >> 3), out + (g2 * 64 + lane) * 16);
    dequantize16<OutT, FMT>(b1, __shfl_sync(0xffffffffu, sb, 4 + (lane >> 3)), out + (g2 * 64 + 32 + lane) * 16);
  }
  if (g < n_groups) {
    const uint4 a0 = __ldcs(q + g * 64 + lane), a1 = __ldcs(q + g * 64 + 32 + lane);
    float sa = 0.0f;
    if (lane < 8) sa = __fmul_rn(e8m0_to_f32(__ldg(sc8 + g * 8 + lane)), __ldg(sc32 + g));
    dequantize16<OutT, FMT>(a0, __shfl_sync(0xffffffffu, sa, lane >> 3), out + (g * 64 + lane) * 16);
    dequantize16<OutT, FMT>(a1, __shfl_sync(0xffffffffu, sa, 4 + (lane >> 3)), out + (g * 64 + 32 + lane) * 16);
  }
}

// Both operands of an elementwise op dequantized and combined in one pass (same shape, same grid):
// out = op(dq(x), dq(y)) in f32, the forward of make_elementwise_impl (_qarr.py:715-720).
enum { kOpAdd = 0, kOpSub = 1, kOpMul = 2, kOpDiv = 3 };

template <int OP> __device__ __forceinline__ float combine(float a, float b) {
  if (OP == kOpAdd) return __fadd_rn(a, b);
  if (OP == kOpSub) return __fsub_rn(a, b);
  if (OP == kOpMul) return __fmul_rn(a, b);
  return __fdiv_rn(a, b);
}

template <int OP, int FX, int FY, int VEC>
__global__ void __launch_bounds__(256)
elementwise_kernel(const uint8_t* __restrict__ xq, const uint8_t* __restrict__ xs8, const float* __restrict__ xs32,
                   const uint8_t* __restrict__ yq, const uint8_t* __restrict__ ys8, const float* __restrict__ ys32,
                   float* __restrict__ out, DqDims d) {
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < d.total_vecs; i += stride) {
    const float sx = block_multiplier(d, xs8, xs32, i), sy = block_multiplier(d, ys8, ys32, i);
    if constexpr (VEC == 16) {
      const uint4 wx = __ldcs(reinterpret_cast<const uint4*>(xq) + i), wy = __ldcs(reinterpret_cast<const uint4*>(yq) + i);
      const uint32_t ax[4] = {wx.x, wx.y, wx.z, wx.w}, ay[4] = {wy.x, wy.y, wy.z, wy.w};
      float v[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xl = fp8x2_to_f32x2<FX>((uint16_t)(ax[j] & 0xffffu)), xh = fp8x2_to_f32x2<FX>((uint16_t)(ax[j] >> 16));
        const float2 yl = fp8x2_to_f32x2<FY>((uint16_t)(ay[j] & 0xffffu)), yh = fp8x2_to_f32x2<FY>((uint16_t)(ay[j] >> 16));
        v[4 * j + 0] = combine<OP>(apply_scale(xl.x, sx), apply_scale(yl.x, sy));
        v[4 * j + 1] = combine<OP>(apply_scale(xl.y, sx), apply_scale(yl.y, sy));
        v[4 * j + 2] = combine<OP>(apply_scale(xh.x, sx), apply_scale(yh.x, sy));
        v[4 * j + 3] = combine<OP>(apply_scale(xh.y, sx), apply_scale(yh.y, sy));
      }
      store16<float>(out + (size_t)i * 16, v);
    } else {
      const float a = apply_scale(fp8x2_to_f32x2<FX>((uint16_t)xq[i]).x, sx);
      const float b = apply_scale(fp8x2_to_f32x2<FY>((uint16_t)yq[i]).x, sy);
      out[i] = combine<OP>(a, b);
    }
  }
}

int dq_grid(int64_t vecs) {
  const int64_t need = (vecs + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  return (int)(need < cap ? (need > 0 ? need : 1) : cap);
}

template <typename OutT, int FMT>
int launch_dq(const uint8_t* q, const uint8_t* sc8, const float* sc32, OutT* out, const Geometry& g, int64_t batch, cudaStream_t st) {
  const int64_t total = batch * g.rows * g.cols;
  const bool vec16 = (g.b % 16 == 0) && (reinterpret_cast<uintptr_t>(q) % 16 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0);
  if (vec16 && g.a == 1 && g.b == 128 && g.K == 8) {
    const int64_t n_groups = batch * g.M;
    const int64_t need = (n_groups + 7) / 8, cap = (int64_t)sm_count() * 16;
    dequantize_row128_kernel<OutT, FMT><<<(int)(need < cap ? need : cap), 256, 0, st>>>((const uint4*)q, sc8, sc32, out, n_groups);
    PB_LAUNCH_CHECK("dequantize_row128_kernel");
    return PB_OK;
  }
  const int vec = vec16 ? 16 : 1;
  if (total / vec > kMaxIndexed || batch * g.rows > kMaxIndexed)
    return fail(PB_ERR_UNSUPPORTED, "pb_dequantize: %lld elements exceed the 31-bit index range of this kernel", (long long)total);
  DqDims d{VecIndexer(g.cols, g.a, g.b, vec), FastDiv((uint32_t)g.K), (uint32_t)(total / vec)};
  if (vec16) dequantize_kernel<OutT, FMT, 16><<<dq_grid(d.total_vecs), 256, 0, st>>>(q, sc8, sc32, out, d);
  else       dequantize_kernel<OutT, FMT, 1><<<dq_grid(d.total_vecs), 256, 0, st>>>(q, sc8, sc32, out, d);
  PB_LAUNCH_CHECK("dequantize_kernel");
  return PB_OK;
}

template <int OP, int FX, int FY>
int launch_elementwise(const uint8_t* xq, const uint8_t* xs8, const float* xs32, const uint8_t* yq, const uint8_t* ys8, const float* ys32,
                       float* out, const Geometry& g, int64_t batch, cudaStream_t st) {
  const int64_t total = batch * g.rows * g.cols;
  const bool vec16 = (g.b % 16 == 0) && ((reinterpret_cast<uintptr_t>(xq) | reinterpret_cast<uintptr_t>(yq) | reinterpret_cast<uintptr_t>(out)) % 16 == 0);
  const int vec = vec16 ? 16 : 1;
  if (total / vec > kMaxIndexed || batch * g.rows > kMaxIndexed)
    return fail(PB_ERR_UNSUPPORTED, "pb_elementwise: %lld elements exceed the 31-bit index range of this kernel", (long long)total);
  DqDims d{VecIndexer(g.cols, g.a, g.b, vec), FastDiv((uint32_t)g.K), (uint32_t)(total / vec)};
  if (vec16) elementwise_kernel<OP, FX, FY, 16><<<dq_grid(d.total_vecs), 256, 0, st>>>(xq, xs8, xs32, yq, ys8, ys32, out, d);
  else       elementwise_kernel<OP, FX, FY, 1><<<dq_grid(d.total_vecs), 256, 0, st>>>(xq, xs8, xs32, yq, ys8, ys32, out, d);
  PB_LAUNCH_CHECK("elementwise_kernel");
  return PB_OK;
}

template <int OP>
int launch_elementwise_fmt(int fx, int fy, const uint8_t* xq, const uint8_t* xs8, const float* xs32, const uint8_t* yq, const uint8_t* ys8,
                           const float* ys32, float* out, const Geometry& g, int64_t batch, cudaStream_t st) {
  if (fx == PB_E4M3 && fy == PB_E4M3) return launch_elementwise<OP, PB_E4M3, PB_E4M3>(xq, xs8, xs32, yq, ys8, ys32, out, g, batch, st);
  if (fx == PB_E4M3) return launch_elementwise<OP, PB_E4M3, PB_E5M2>(xq, xs8, xs32, yq, ys8, ys32, out, g, batch, st);
  if (fy == PB_E4M3) return launch_elementwise<OP, PB_E5M2, PB_E4M3>(xq, xs8, xs32, yq, ys8, ys32, out, g, batch, st);
  return launch_elementwise<OP, PB_E5M2, PB_E5M2>(xq, xs8, xs32, yq, ys8, ys32, out, g, batch, st);
}

}  // namespace
}  // namespace pb

using namespace pb;

extern "C" int pb_elementwise(int op, const void* xq, int x_format, const uint8_t* xs8, const float* xs32,
                              const void* yq, int y_format, const uint8_t* ys8, const float* ys32,
                              int64_t batch, int64_t rows, int64_t cols, int a, int b, float* out, void* stream) {
  if (!xq || !xs8 || !xs32 || !yq || !ys8 || !ys32 || !out) return fail(PB_ERR_NULL_POINTER, "pb_elementwise: operands and out must be non-null");
  if (batch <= 0) return fail(PB_ERR_BAD_SHAPE, "pb_elementwise: batch=%lld must be positive", (long long)batch);
  if ((x_format != PB_E4M3 && x_format != PB_E5M2) || (y_format != PB_E4M3 && y_format != PB_E5M2))
    return fail(PB_ERR_BAD_DTYPE, "pb_elementwise: formats %d, %d", x_format, y_format);
  Geometry g;
  if (int s = make_geometry(rows, cols, a, b, &g)) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* x8 = static_cast<const uint8_t*>(xq);
  const uint8_t* y8 = static_cast<const uint8_t*>(yq);
  switch (op) {
    case PB_OP_ADD: return launch_elementwise_fmt<kOpAdd>(x_format, y_format, x8, xs8, xs32, y8, ys8, ys32, out, g, batch, st);
    case PB_OP_SUB: return launch_elementwise_fmt<kOpSub>(x_format, y_format, x8, xs8, xs32, y8, ys8, ys32, out, g, batch, st);
    case PB_OP_MUL: return launch_elementwise_fmt<kOpMul>(x_format, y_format, x8, xs8, xs32, y8, ys8, ys32, out, g, batch, st);
    case PB_OP_DIV: return launch_elementwise_fmt<kOpDiv>(x_format, y_format, x8, xs8, xs32, y8, ys8, ys32, out, g, batch, st);
    default: return fail(PB_ERR_UNSUPPORTED, "pb_elementwise: op %d (add, sub, mul and div only; floor_divide, mod and pow go through pb_dequantize)", op);
  }
}

extern "C" int pb_dequantize(const void* q, int q_format, const uint8_t* sc8, const float* sc32,
                             int64_t batch, int64_t rows, int64_t cols, int a, int b,
                             int out_dtype, void* out, void* stream) {
  if (!q || !sc8 || !sc32 || !out) return fail(PB_ERR_NULL_POINTER, "pb_dequantize: q, sc8, sc32 and out must be non-null");
  if (batch <= 0) return fail(PB_ERR_BAD_SHAPE, "pb_dequantize: batch=%lld must be positive", (long long)batch);
  if (q_format != PB_E4M3 && q_format != PB_E5M2) return fail(PB_ERR_BAD_DTYPE, "pb_dequantize: q_format %d is neither PB_E4M3 nor PB_E5M2", q_format);
  if (out_dtype != PB_F32 && out_dtype != PB_BF16) return fail(PB_ERR_BAD_DTYPE, "pb_dequantize: out_dtype %d is neither PB_F32 nor PB_BF16", out_dtype);
  Geometry g;
  if (int s = make_geometry(rows, cols, a, b, &g)) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* qb = static_cast<const uint8_t*>(q);
  if (out_dtype == PB_F32)
    return q_format == PB_E4M3 ? launch_dq<float, PB_E4M3>(qb, sc8, sc32, (float*)out, g, batch, st)
                               : launch_dq<float, PB_E5M2>(qb, sc8, sc32, (float*)out, g, batch, st);
  return q_format == PB_E4M3 ? launch_dq<__nv_bfloat16, PB_E4M3>(qb, sc8, sc32, (__nv_bfloat16*)out, g, batch, st)
                             : launch_dq<__nv_bfloat16, PB_E5M2>(qb, sc8, sc32, (__nv_bfloat16*)out, g, batch, st);
}

extern "C" int pb_dequantize_bwd(const void* gin, int dtype, const uint8_t* sc8, const float* sc32,
                                 int64_t batch, int64_t rows, int64_t cols, int a, int b,
                                 void* out, void* stream) {
  if (!gin || !sc8 || !sc32 || !out) return fail(PB_ERR_NULL_POINTER, "pb_dequantize_bwd: g, sc8, sc32 and out must be non-null");
  if (batch <= 0) return fail(PB_ERR_BAD_SHAPE, "pb_dequantize_bwd: batch=%lld must be positive", (long long)batch);
  if (dtype != PB_F32 && dtype != PB_BF16) return fail(PB_ERR_BAD_DTYPE, "pb_dequantize_bwd: dtype %d is neither PB_F32 nor PB_BF16", dtype);
  Geometry g;
  if (int s = make_geometry(rows, cols, a, b, &g)) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t total = batch * rows * cols;
  const bool vec4 = (b % 4 == 0);
  const int vec = vec4 ? 4 : 1;
  if (total / vec > kMaxIndexed || batch * g.rows > kMaxIndexed)
    return fail(PB_ERR_UNSUPPORTED, "pb_dequantize_bwd: %lld elements exceed the 31-bit index range of this kernel", (long long)total);
  DqDims d{VecIndexer(g.cols, g.a, g.b, vec), FastDiv((uint32_t)g.K), (uint32_t)(total / vec)};
  const int grid = dq_grid(d.total_vecs);
  if (dtype == PB_F32) {
    if (vec4) dequantize_bwd_kernel<float, 4><<<grid, 256, 0, st>>>((const float*)gin, sc8, sc32, (float*)out, d);
    else      dequantize_bwd_kernel<float, 1><<<grid, 256, 0, st>>>((const float*)gin, sc8, sc32, (float*)out, d);
  } else {
    if (vec4) dequantize_bwd_kernel<__nv_bfloat16, 4><<<grid, 256, 0, st>>>((const __nv_bfloat16*)gin, sc8, sc32, (__nv_bfloat16*)out, d);
    else      dequantize_bwd_kernel<__nv_bfloat16, 1><<<grid, 256, 0, st>>>((const __nv_bfloat16*)gin, sc8, sc32, (__nv_bfloat16*)out, d);
  }
  PB_LAUNCH_CHECK("dequantize_bwd_kernel");
  return PB_OK;
}
