// Momentum step of the reference's optimizer on quantized arrays (sm_100a).
//
// For a QArrayImpl parameter the reference (pratchya/_nnx_impl/_optimizer.py:171-205) dequantizes
// the gradient g and the momentum m to f32, forms
//     c     = beta1 * m + (1 - beta1) * g        (what sign() or Newton-Schulz is then applied to)
//     new_m = beta2 * m + (1 - beta2) * g        and stores QArrayImpl(new_m, tgrid),
// which in jax.numpy is two dequantizations, four scaled-array temporaries and a quantization.
// Here: one pass reads the bytes of g and m, writes c and takes the block amaxes of new_m; the
// shared scale kernel turns them into e8m0 bytes and divisors; a second pass re-reads the bytes of
// g and m (2 B/element, not a 4 B/element temporary), recomputes new_m and writes its fp8 bytes.
// Arithmetic: f32 multiplies and one add per value, no FMA contraction, in the reference's order.
//
// Stacked (3-D) parameters take the reference's scanned branch (:108-160) instead: per leading index
// the same step on bfloat16 values -- g and m dequantized to bf16, the blend in bf16 with the scalars
// as bf16 and every product and sum rounded to bf16, c returned in bf16 -- and new_m quantized again.
// The kernels below are templated on that (BF): the passes and their traffic are the same, c is half
// the bytes.
#include "common.cuh"

namespace pb {

// defined in quantize.cu
int launch_group_scales(const uint32_t* amax_bits, float* divisor, uint8_t* sc8, float* sc32, int64_t n_groups, int64_t K, cudaStream_t st);

namespace {

struct MomentumParams {
  const uint8_t* gq; const uint8_t* g_sc8; const float* g_sc32;
  const uint8_t* mq; const uint8_t* m_sc8; const float* m_sc32;
  float b1, c1, b2, c2;       // beta1, 1 - beta1, beta2, 1 - beta2 (each rounded to f32 by the caller, as JAX does with Python scalars)
  VecIndexer idx;
  FastDiv by_K;
  uint32_t total_vecs;
};

__device__ __forceinline__ float multiplier(const MomentumParams& p, const uint8_t* sc8, const float* sc32, uint32_t blk) {
  return __fmul_rn(e8m0_to_f32(__ldg(sc8 + blk)), __ldg(sc32 + p.by_K.div(blk)));       // _qarr.py:562-563
}
__device__ __forceinline__ float dq(float v, float x_sc) { return __fmul_rn(__fmul_rn(v, x_sc), 0.0078125f); }     // :564

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// 16 (or 1) consecutive elements of g and m, dequantized (BF: and rounded to bf16, the reference's astype)
template <int FG, int FM, int VEC, bool BF = false>
__device__ __forceinline__ void load_pair(const MomentumParams& p, uint32_t i, uint32_t blk, float (&g)[VEC], float (&m)[VEC]) {
  const float sg = multiplier(p, p.g_sc8, p.g_sc32, blk), sm = multiplier(p, p.m_sc8, p.m_sc32, blk);
  if constexpr (VEC == 16) {
    const uint4 wg = __ldg(reinterpret_cast<const uint4*>(p.gq) + i), wm = __ldg(reinterpret_cast<const uint4*>(p.mq) + i);
    const uint32_t ag[4] = {wg.x, wg.y, wg.z, wg.w}, am[4] = {wm.x, wm.y, wm.z, wm.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gl = fp8x2_to_f32x2<FG>((uint16_t)(ag[j] & 0xffffu)), gh = fp8x2_to_f32x2<FG>((uint16_t)(ag[j] >> 16));
      const float2 ml = fp8x2_to_f32x2<FM>((uint16_t)(am[j] & 0xffffu)), mh = fp8x2_to_f32x2<FM>((uint16_t)(am[j] >> 16));
      g[4 * j] = dq(gl.x, sg); g[4 * j + 1] = dq(gl.y, sg); g[4 * j + 2] = dq(gh.x, sg); g[4 * j + 3] = dq(gh.y, sg);
      m[4 * j] = dq(ml.x, sm); m[4 * j + 1] = dq(ml.y, sm); m[4 * j + 2] = dq(mh.x, sm); m[4 * j + 3] = dq(mh.y, sm);
    }
  } else {
    g[0] = dq(fp8x2_to_f32x2<FG>((uint16_t)p.gq[i]).x, sg);
    m[0] = dq(fp8x2_to_f32x2<FM>((uint16_t)p.mq[i]).x, sm);
  }
  if constexpr (BF) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) { g[j] = round_bf16(g[j]); m[j] = round_bf16(m[j]); }
  }
}

// beta_m * m + beta_g * g.  BF: on bf16 values (held widened in f32): a product of two bf16 numbers is exact in
// f32, so rounding it once gives the bf16 product; the sum is formed in f32 and rounded to bf16, as a
// bf16 add that computes in f32 does.
template <bool BF = false>
__device__ __forceinline__ float blend(float bm, float m, float bg, float g) {
  if constexpr (BF) return round_bf16(__fadd_rn(round_bf16(__fmul_rn(bm, m)), round_bf16(__fmul_rn(bg, g))));
  else return __fadd_rn(__fmul_rn(bm, m), __fmul_rn(bg, g));
}

// pass 1: c out, block amax of new_m (atomicMax on the f32 bits, one per warp where a warp sits in one block)
template <int FG, int FM, int VEC, bool BF>
__global__ void __launch_bounds__(256)
momentum_first_pass_kernel(MomentumParams p, void* __restrict__ c_out_v, uint32_t* __restrict__ amax_bits) {
  float* c_out = static_cast<float*>(c_out_v);                          // BF == false
  __nv_bfloat16* c_out_bf = static_cast<__nv_bfloat16*>(c_out_v);       // BF == true
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; ; i += stride) {
    const bool active = i < p.total_vecs;
    if (__all_sync(0xffffffffu, !active)) break;
    uint32_t bits = 0, blk = 0xffffffffu;
    if (active) {
      blk = p.idx.block_of(i);
      float g[VEC], m[VEC], c[VEC];
      load_pair<FG, FM, VEC, BF>(p, i, blk, g, m);
      float mx = 0.0f;
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        c[j] = blend<BF>(p.b1, m[j], p.c1, g[j]);
        mx = fmaxf(mx, fabsf(blend<BF>(p.b2, m[j], p.c2, g[j])));
      }
      if constexpr (BF) {
        if constexpr (VEC == 16) {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) w[j] = pack_bf16x2(c[2 * j], c[2 * j + 1]);      // exact: the values are bf16 already
          uint4* dst = reinterpret_cast<uint4*>(c_out_bf + (size_t)i * 16);
          __stcs(dst, make_uint4(w[0], w[1], w[2], w[3]));
          __stcs(dst + 1, make_uint4(w[4], w[5], w[6], w[7]));
        } else {
          c_out_bf[i] = __float2bfloat16_rn(c[0]);
        }
      } else if constexpr (VEC == 16) {
        float* dst = c_out + (size_t)i * 16;
        if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {      // whole 32-byte sectors per store
#pragma unroll
          for (int j = 0; j < 2; ++j)
            asm volatile("st.global.cs.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                         ::"l"(dst + 8 * j), "f"(c[8 * j]), "f"(c[8 * j + 1]), "f"(c[8 * j + 2]), "f"(c[8 * j + 3]),
                           "f"(c[8 * j + 4]), "f"(c[8 * j + 5]), "f"(c[8 * j + 6]), "f"(c[8 * j + 7]) : "memory");
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) __stcs(reinterpret_cast<float4*>(dst) + j, make_float4(c[4 * j], c[4 * j + 1], c[4 * j + 2], c[4 * j + 3]));
        }
      } else {
        c_out[i] = c[0];
      }
      bits = __float_as_uint(mx);
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

// pass 2: new_m recomputed from the bytes of g and m, divided by its block's divisor, to fp8
template <int FG, int FM, int FOUT, int VEC, bool BF>
__global__ void __launch_bounds__(256)
momentum_second_pass_kernel(MomentumParams p, const float* __restrict__ divisor, uint8_t* __restrict__ new_mq) {
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < p.total_vecs; i += stride) {
    const uint32_t blk = p.idx.block_of(i);
    float g[VEC], m[VEC];
    load_pair<FG, FM, VEC, BF>(p, i, blk, g, m);
    const float D = divisor[blk], r = __frcp_rn(D);
    const float2 nD2 = make_float2(-D, -D), r2 = make_float2(r, r);
    if constexpr (VEC == 16) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = blend<BF>(p.b2, m[4 * j + k], p.c2, g[4 * j + k]);
        o[j] = bf16x2_to_fp8x2<FOUT>(div_hoisted_pack2(v[0], v[1], nD2, r2)) | (bf16x2_to_fp8x2<FOUT>(div_hoisted_pack2(v[2], v[3], nD2, r2)) << 16);
      }
      __stcs(reinterpret_cast<uint4*>(new_mq) + i, make_uint4(o[0], o[1], o[2], o[3]));
    } else {
      const float v = blend<BF>(p.b2, m[0], p.c2, g[0]);
      new_mq[i] = (uint8_t)(bf16x2_to_fp8x2<FOUT>(div_hoisted_pack2(v, 0.0f, nD2, r2)) & 0xffu);
    }
  }
}

int grid_of(uint32_t vecs) {
  const int64_t need = ((int64_t)vecs + 255) / 256, cap = (int64_t)sm_count() * 8;
  return (int)(need < cap ? (need > 0 ? need : 1) : cap);
}

template <int VEC, bool BF>
int launch_momentum(const MomentumParams& p, void* c_out, uint32_t* amax_bits, float* divisor, uint8_t* new_mq, uint8_t* sc8,
                    float* sc32, int64_t n_groups, int64_t K, cudaStream_t st) {
  const int grid = grid_of(p.total_vecs);
  momentum_first_pass_kernel<PB_E4M3, PB_E4M3, VEC, BF><<<grid, 256, 0, st>>>(p, c_out, amax_bits);
  PB_LAUNCH_CHECK("momentum_first_pass_kernel");
  if (int s = launch_group_scales(amax_bits, divisor, sc8, sc32, n_groups, K, st)) return s;
  momentum_second_pass_kernel<PB_E4M3, PB_E4M3, PB_E4M3, VEC, BF><<<grid, 256, 0, st>>>(p, divisor, new_mq);
  PB_LAUNCH_CHECK("momentum_second_pass_kernel");
  return PB_OK;
}

int momentum_update(const char* name, bool bf, const void* gq, const uint8_t* g_sc8, const float* g_sc32,
                    const void* mq, const uint8_t* m_sc8, const float* m_sc32,
                    int64_t batch, int64_t rows, int64_t cols, int a, int b,
                    float beta1, float one_minus_beta1, float beta2, float one_minus_beta2,
                    void* c_out, void* new_mq, uint8_t* new_m_sc8, float* new_m_sc32,
                    void* workspace, size_t workspace_bytes, void* stream) {
  if (!gq || !g_sc8 || !g_sc32 || !mq || !m_sc8 || !m_sc32 || !c_out || !new_mq || !new_m_sc8 || !new_m_sc32)
    return fail(PB_ERR_NULL_POINTER, "%s: the two triples and the four outputs must be non-null", name);
  if (batch <= 0) return fail(PB_ERR_BAD_SHAPE, "%s: batch=%lld must be positive", name, (long long)batch);
  Geometry g;
  if (int s = make_geometry(rows, cols, a, b, &g)) return s;
  const int64_t nblk = batch * g.Nb, total = batch * rows * cols;
  const size_t need = (size_t)nblk * 8;
  if (!workspace || workspace_bytes < need)
    return fail(PB_ERR_WORKSPACE_TOO_SMALL, "%s: needs %zu bytes of workspace, got %zu", name, need, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 3) return fail(PB_ERR_MISALIGNED, "%s: workspace must be 4-byte aligned", name);
  const bool vec16 = (b % 16 == 0) && ((reinterpret_cast<uintptr_t>(gq) | reinterpret_cast<uintptr_t>(mq) | reinterpret_cast<uintptr_t>(new_mq) |
                                         reinterpret_cast<uintptr_t>(c_out)) % 16 == 0);
  const int vec = vec16 ? 16 : 1;
  if (total / vec > kMaxIndexed || batch * rows > kMaxIndexed)
    return fail(PB_ERR_UNSUPPORTED, "%s: %lld elements exceed the 31-bit index range of this kernel", name, (long long)total);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* amax_bits = static_cast<uint32_t*>(workspace);
  float* divisor = reinterpret_cast<float*>(amax_bits + nblk);
  PB_CUDA_TRY(cudaMemsetAsync(amax_bits, 0, (size_t)nblk * sizeof(uint32_t), st));
  MomentumParams p{static_cast<const uint8_t*>(gq), g_sc8, g_sc32, static_cast<const uint8_t*>(mq), m_sc8, m_sc32,
                   beta1, one_minus_beta1, beta2, one_minus_beta2, VecIndexer(cols, a, b, vec), FastDiv((uint32_t)g.K), (uint32_t)(total / vec)};
  uint8_t* out = static_cast<uint8_t*>(new_mq);
  const int64_t n_groups = batch * g.M;
  if (bf) return vec16 ? launch_momentum<16, true>(p, c_out, amax_bits, divisor, out, new_m_sc8, new_m_sc32, n_groups, g.K, st)
                       : launch_momentum<1, true>(p, c_out, amax_bits, divisor, out, new_m_sc8, new_m_sc32, n_groups, g.K, st);
  return vec16 ? launch_momentum<16, false>(p, c_out, amax_bits, divisor, out, new_m_sc8, new_m_sc32, n_groups, g.K, st)
               : launch_momentum<1, false>(p, c_out, amax_bits, divisor, out, new_m_sc8, new_m_sc32, n_groups, g.K, st);
}

}  // namespace
}  // namespace pb

using namespace pb;

extern "C" size_t pb_momentum_workspace_size(int64_t batch, int64_t rows, int64_t cols, int a, int b) {
  Geometry g;
  if (batch <= 0 || make_geometry(rows, cols, a, b, &g) != PB_OK) return 0;
  return (size_t)(batch * g.Nb) * 8;
}

extern "C" int pb_momentum_update(const void* gq, const uint8_t* g_sc8, const float* g_sc32,
                                  const void* mq, const uint8_t* m_sc8, const float* m_sc32,
                                  int64_t batch, int64_t rows, int64_t cols, int a, int b,
                                  float beta1, float one_minus_beta1, float beta2, float one_minus_beta2,
                                  float* c_out, void* new_mq, uint8_t* new_m_sc8, float* new_m_sc32,
                                  void* workspace, size_t workspace_bytes, void* stream) {
  return momentum_update("pb_momentum_update", false, gq, g_sc8, g_sc32, mq, m_sc8, m_sc32, batch, rows, cols, a, b,
                         beta1, one_minus_beta1, beta2, one_minus_beta2, c_out, new_mq, new_m_sc8, new_m_sc32,
                         workspace, workspace_bytes, stream);
}

extern "C" int pb_momentum_update_stacked(const void* gq, const uint8_t* g_sc8, const float* g_sc32,
                                          const void* mq, const uint8_t* m_sc8, const float* m_sc32,
                                          int64_t layers, int64_t rows, int64_t cols, int a, int b,
                                          float beta1, float one_minus_beta1, float beta2, float one_minus_beta2,
                                          void* c_out_bf16, void* new_mq, uint8_t* new_m_sc8, float* new_m_sc32,
                                          void* workspace, size_t workspace_bytes, void* stream) {
  return momentum_update("pb_momentum_update_stacked", true, gq, g_sc8, g_sc32, mq, m_sc8, m_sc32, layers, rows, cols, a, b,
                         beta1, one_minus_beta1, beta2, one_minus_beta2, c_out_bf16, new_mq, new_m_sc8, new_m_sc32,
                         workspace, workspace_bytes, stream);
}
