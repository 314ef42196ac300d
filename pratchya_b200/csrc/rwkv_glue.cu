// The f32 element-wise work around the FP8 linears and the WKV-7 scan in the modified RWKV-7 block
// (pratchya/_nnx_impl/_module.py:129-258), as a few HBM-bound kernels instead of a chain of framework
// operations that each read and write the whole [tokens, channels] activation:
//
//   token shift + lerps (:137-151 TimeMix, six mixes; :240-247 ChannelMix, one)      pb_token_shift_lerp(_bwd)
//   everything between TimeMix's linears and its scan (:157-184): rotary embedding of r and k, sigmoid of
//   iclr and nu, v lerp, decay = exp(-exp(d)), removal_k = normalized(k * m), replacement_k            pb_wkv_prepare(_bwd)
//
// Arithmetic follows the reference's order of operations with unfused multiplies and adds (a lerp is
// i + (j - i) * w, two roundings), so forward values match an op-by-op f32 evaluation to the last bit except
// for the order of the 64-term sum in `normalized`.  Sums over tokens for parameter gradients are formed per
// tile of tokens and then added in tile order by reduce_partials_kernel: no atomics, same bits every run.
#include "common.cuh"

namespace pb {
namespace {

constexpr int kGlueThreads = 256;
constexpr int kGlueH = 64;               // head size of the rotary / normalisation kernels
constexpr int kLerpTileRows = 64;        // tokens per CTA of the lerp backward kernel
constexpr int kPrepTileRows = 32;        // tokens per warp of the prepare backward kernel
constexpr int kMaxMix = 8;

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
// i + (j - i) * w with the three roundings of the op-by-op evaluation
__device__ __forceinline__ float lerp_rn(float i, float j, float w) { return __fadd_rn(i, __fmul_rn(__fsub_rn(j, i), w)); }
__device__ __forceinline__ float sigmoid_rn(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
// for the backward kernels, which are compared with autograd to 2e-5 and not bit for bit: hardware exp2 and reciprocal
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// out[k][r][c] = x[r][c] + (prev[r][c] - x[r][c]) * mu[k][c], prev = the token before (the carried state for the first)
struct ShiftLerpParams {
  const float* x; const float* state; const float* mu; float* out;
  int64_t R; int T, C, n_mix;
};

__global__ void __launch_bounds__(kGlueThreads) shift_lerp_fwd_kernel(const ShiftLerpParams p) {
  const int C4 = p.C >> 2;
  const int64_t total = p.R * C4, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int64_t r = idx / C4;
    const int c = (int)(idx - r * C4) << 2;
    const int t = (int)(r % p.T);
    const float4 x = ld4(p.x + r * p.C + c);
    float4 prev;
    if (t > 0) prev = ld4(p.x + (r - 1) * p.C + c);
    else prev = p.state ? ld4(p.state + (r / p.T) * p.C + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < p.n_mix; ++k) {
      const float4 m = __ldg(reinterpret_cast<const float4*>(p.mu + (size_t)k * p.C + c));
      st4(p.out + ((size_t)k * p.R + r) * p.C + c,
          make_float4(lerp_rn(x.x, prev.x, m.x), lerp_rn(x.y, prev.y, m.y), lerp_rn(x.z, prev.z, m.z), lerp_rn(x.w, prev.w, m.w)));
    }
  }
}

// Backward: with s_r = sum_k g_k[r] * mu_k,
//   dx[r] = sum_k g_k[r] - s_r + (s_{r+1} if r+1 is in the same sequence), dstate[b] = s of the sequence's first token,
//   dmu_k[c] = sum_r g_k[r][c] * (prev[r][c] - x[r][c]).
// A CTA walks kLerpTileRows tokens of 1024 channels (four per thread), carrying x[r-1] and the unfinished dx[r-1].
struct ShiftLerpBwdParams {
  const float* g[kMaxMix];                         // cotangent of each mix, [R][C]
  const float* x; const float* state; const float* mu;
  float* dx; float* dstate; float* partial;        // partial [tiles][n_mix][C]
  int64_t R; int T, C, n_mix;
};

template <int NMIX>
__global__ void __launch_bounds__(kGlueThreads) shift_lerp_bwd_kernel(const ShiftLerpBwdParams p) {
  const int c = (blockIdx.x * kGlueThreads + threadIdx.x) << 2;
  if (c >= p.C) return;
  const int64_t r0 = (int64_t)blockIdx.y * kLerpTileRows, r1 = min(p.R, r0 + kLerpTileRows);
  float4 mu[NMIX], acc[NMIX];
#pragma unroll
  for (int k = 0; k < NMIX; ++k) { mu[k] = __ldg(reinterpret_cast<const float4*>(p.mu + (size_t)k * p.C + c)); acc[k] = make_float4(0.f, 0.f, 0.f, 0.f); }
  float4 xprev = make_float4(0.f, 0.f, 0.f, 0.f), open = xprev;       // x[r-1]; dx[r-1] without the term of token r
  if (r0 % p.T != 0) xprev = ld4(p.x + (r0 - 1) * p.C + c);
  auto weighted = [&](int64_t r, float4& gsum, float4& s, float4 d, bool accumulate) {
#pragma unroll
    for (int k = 0; k < NMIX; ++k) {
      const float4 g = ld4(p.g[k] + (size_t)r * p.C + c);
      gsum.x += g.x; gsum.y += g.y; gsum.z += g.z; gsum.w += g.w;
      s.x = fmaf(g.x, mu[k].x, s.x); s.y = fmaf(g.y, mu[k].y, s.y); s.z = fmaf(g.z, mu[k].z, s.z); s.w = fmaf(g.w, mu[k].w, s.w);
      if (accumulate) {
        acc[k].x = fmaf(g.x, d.x, acc[k].x); acc[k].y = fmaf(g.y, d.y, acc[k].y);
        acc[k].z = fmaf(g.z, d.z, acc[k].z); acc[k].w = fmaf(g.w, d.w, acc[k].w);
      }
    }
  };
  for (int64_t r = r0; r < r1; ++r) {
    const int t = (int)(r % p.T);
    const float4 x = ld4(p.x + r * p.C + c);
    float4 prev = xprev;
    if (t == 0) prev = p.state ? ld4(p.state + (r / p.T) * p.C + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 d = make_float4(prev.x - x.x, prev.y - x.y, prev.z - x.z, prev.w - x.w);
    float4 gsum = make_float4(0.f, 0.f, 0.f, 0.f), s = gsum;
    weighted(r, gsum, s, d, true);
    if (t == 0) {
      if (p.dstate) st4(p.dstate + (r / p.T) * p.C + c, s);
      if (r > r0) st4(p.dx + (r - 1) * p.C + c, open);
    } else if (r > r0) {
      st4(p.dx + (r - 1) * p.C + c, make_float4(open.x + s.x, open.y + s.y, open.z + s.z, open.w + s.w));
    }
    open = make_float4(gsum.x - s.x, gsum.y - s.y, gsum.z - s.z, gsum.w - s.w);
    xprev = x;
  }
  // the tile's last token: its successor, if it has one in the same sequence, belongs to the next tile
  if (r1 < p.R && r1 % p.T != 0) {
    float4 gsum = make_float4(0.f, 0.f, 0.f, 0.f), s = gsum;
    weighted(r1, gsum, s, gsum, false);
    open = make_float4(open.x + s.x, open.y + s.y, open.z + s.z, open.w + s.w);
  }
  st4(p.dx + (r1 - 1) * p.C + c, open);
#pragma unroll
  for (int k = 0; k < NMIX; ++k) st4(p.partial + ((size_t)blockIdx.y * NMIX + k) * p.C + c, acc[k]);
}

// out[j] = sum over tiles of partial[tile][j]: eight partial sums per column (tiles g, g + 8, ...), added in a fixed order.
// A block takes 32 columns; out may be the first tile's slot of partial (a column is read and written by its block only).
__global__ void __launch_bounds__(kGlueThreads) reduce_partials_kernel(const float* partial, float* out, int tiles, int64_t n) {
  __shared__ float red[kGlueThreads / 32][32];
  const int cx = threadIdx.x & 31, gy = threadIdx.x >> 5;
  const int64_t j = (int64_t)blockIdx.x * 32 + cx;
  float s = 0.0f;
  if (j < n)
    for (int t = gy; t < tiles; t += kGlueThreads / 32) s += partial[(size_t)t * n + j];
  red[gy][cx] = s;
  __syncthreads();
  if (gy == 0 && j < n) {
    float r = red[0][cx];
#pragma unroll
    for (int g = 1; g < kGlueThreads / 32; ++g) r += red[g][cx];
    out[j] = r;
  }
}

// ---- TimeMix between its linears and the scan ----------------------------------------------------------------
// One warp per (token, head); lane l holds channels l and l + 32 of the head: the two halves that the rotary
// embedding pairs (_module.py:275-283: x * cos + cat(-x2, x1) * sin, the same angle for both halves).
struct PrepareParams {
  const float* r_raw; const float* k_raw; const float* d; const float* iclr_raw; const float* v_prime;
  const float* v0; const float* nu_raw;                      // null in the first layer (v = v_prime)
  const float* cos_tab; const float* sin_tab;                // [T][32]
  const float* rk_mult; const float* mix_amt;                // [C], already read through their quantization
  float* decay; float* iclr; float* removal_k; float* replacement_k; float* v; float* r; float* k;
  int64_t R; int T, N;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(kGlueThreads) wkv_prepare_fwd_kernel(const PrepareParams p) {
  const int lane = threadIdx.x & 31;
  const int C = p.N * kGlueH;
  const int64_t warps = (int64_t)gridDim.x * (kGlueThreads / 32), total = p.R * p.N;
  for (int64_t w = (int64_t)blockIdx.x * (kGlueThreads / 32) + (threadIdx.x >> 5); w < total; w += warps) {
    const int64_t row = w / p.N;
    const int n = (int)(w - row * p.N), t = (int)(row % p.T);
    const int c1 = n * kGlueH + lane, c2 = c1 + 32;
    const size_t i1 = (size_t)row * C + c1, i2 = i1 + 32;
    const float cs = __ldg(p.cos_tab + t * 32 + lane), sn = __ldg(p.sin_tab + t * 32 + lane);
    const float ra = p.r_raw[i1], rb = p.r_raw[i2], ka = p.k_raw[i1], kb = p.k_raw[i2];
    const float r1 = __fadd_rn(__fmul_rn(ra, cs), __fmul_rn(-rb, sn)), r2 = __fadd_rn(__fmul_rn(rb, cs), __fmul_rn(ra, sn));
    const float k1 = __fadd_rn(__fmul_rn(ka, cs), __fmul_rn(-kb, sn)), k2 = __fadd_rn(__fmul_rn(kb, cs), __fmul_rn(ka, sn));
    const float a1 = sigmoid_rn(p.iclr_raw[i1]), a2 = sigmoid_rn(p.iclr_raw[i2]);
    float v1 = p.v_prime[i1], v2 = p.v_prime[i2];
    if (p.v0) {
      v1 = lerp_rn(v1, p.v0[i1], sigmoid_rn(p.nu_raw[i1]));
      v2 = lerp_rn(v2, p.v0[i2], sigmoid_rn(p.nu_raw[i2]));
    }
    const float u1 = __fmul_rn(k1, __ldg(p.rk_mult + c1)), u2 = __fmul_rn(k2, __ldg(p.rk_mult + c2));
    const float nrm = sqrtf(__fadd_rn(warp_sum(__fadd_rn(__fmul_rn(u1, u1), __fmul_rn(u2, u2))), 1e-12f));
    p.decay[i1] = expf(-expf(p.d[i1])); p.decay[i2] = expf(-expf(p.d[i2]));
    p.iclr[i1] = a1; p.iclr[i2] = a2;
    p.removal_k[i1] = __fdiv_rn(u1, nrm); p.removal_k[i2] = __fdiv_rn(u2, nrm);
    p.replacement_k[i1] = lerp_rn(k1, __fmul_rn(k1, a1), __ldg(p.mix_amt + c1));
    p.replacement_k[i2] = lerp_rn(k2, __fmul_rn(k2, a2), __ldg(p.mix_amt + c2));
    p.v[i1] = v1; p.v[i2] = v2;
    p.r[i1] = r1; p.r[i2] = r2;
    p.k[i1] = k1; p.k[i2] = k2;
  }
}

// Backward of the above from the cotangents of its seven outputs.  A warp walks kPrepTileRows tokens of one head,
// so each lane adds up its two channels' share of d(rk_mult) and d(mix_amt) in registers.
struct PrepareBwdParams {
  PrepareParams f;                       // the forward inputs (outputs unused)
  const float* g_decay; const float* g_iclr; const float* g_removal_k; const float* g_replacement_k;
  const float* g_v; const float* g_r; const float* g_k;
  float* d_r_raw; float* d_k_raw; float* d_d; float* d_iclr_raw; float* d_v_prime; float* d_v0; float* d_nu_raw;
  float* partial;                        // [tiles][2][C]: rk_mult, mix_amt
};

__global__ void __launch_bounds__(kGlueThreads) wkv_prepare_bwd_kernel(const PrepareBwdParams p) {
  const PrepareParams& f = p.f;
  const int lane = threadIdx.x & 31;
  const int C = f.N * kGlueH;
  const int tiles = (int)((f.R + kPrepTileRows - 1) / kPrepTileRows);
  const int64_t w = (int64_t)blockIdx.x * (kGlueThreads / 32) + (threadIdx.x >> 5);
  if (w >= (int64_t)tiles * f.N) return;
  const int tile = (int)(w / f.N), n = (int)(w - (int64_t)tile * f.N);
  const int c1 = n * kGlueH + lane, c2 = c1 + 32;
  const float m1 = __ldg(f.rk_mult + c1), m2 = __ldg(f.rk_mult + c2), x1 = __ldg(f.mix_amt + c1), x2 = __ldg(f.mix_amt + c2);
  float dm1 = 0.f, dm2 = 0.f, dx1 = 0.f, dx2 = 0.f;
  const int64_t row_end = min(f.R, (int64_t)(tile + 1) * kPrepTileRows);
  for (int64_t row = (int64_t)tile * kPrepTileRows; row < row_end; ++row) {
    const int t = (int)(row % f.T);
    const size_t i1 = (size_t)row * C + c1, i2 = i1 + 32;
    const float cs = __ldg(f.cos_tab + t * 32 + lane), sn = __ldg(f.sin_tab + t * 32 + lane);
    const float ka = f.k_raw[i1], kb = f.k_raw[i2];
    const float k1 = __fadd_rn(__fmul_rn(ka, cs), __fmul_rn(-kb, sn)), k2 = __fadd_rn(__fmul_rn(kb, cs), __fmul_rn(ka, sn));
    const float a1 = sigmoid_fast(f.iclr_raw[i1]), a2 = sigmoid_fast(f.iclr_raw[i2]);
    // removal_k = u / nrm, u = k * m: d_u = (g - removal_k * sum(g * removal_k)) / nrm
    const float u1 = __fmul_rn(k1, m1), u2 = __fmul_rn(k2, m2);
    const float inv_nrm = rsqrtf(warp_sum(u1 * u1 + u2 * u2) + 1e-12f);
    const float q1 = u1 * inv_nrm, q2 = u2 * inv_nrm;
    const float gq1 = p.g_removal_k[i1], gq2 = p.g_removal_k[i2];
    const float dot = warp_sum(gq1 * q1 + gq2 * q2);
    const float du1 = (gq1 - q1 * dot) * inv_nrm, du2 = (gq2 - q2 * dot) * inv_nrm;
    dm1 = fmaf(du1, k1, dm1); dm2 = fmaf(du2, k2, dm2);
    // replacement_k = k + (k * a - k) * x
    const float gp1 = p.g_replacement_k[i1], gp2 = p.g_replacement_k[i2];
    dx1 = fmaf(gp1, k1 * a1 - k1, dx1); dx2 = fmaf(gp2, k2 * a2 - k2, dx2);
    const float dk1 = p.g_k[i1] + du1 * m1 + gp1 * (1.0f + (a1 - 1.0f) * x1);
    const float dk2 = p.g_k[i2] + du2 * m2 + gp2 * (1.0f + (a2 - 1.0f) * x2);
    const float da1 = p.g_iclr[i1] + gp1 * k1 * x1, da2 = p.g_iclr[i2] + gp2 * k2 * x2;
    p.d_iclr_raw[i1] = da1 * a1 * (1.0f - a1); p.d_iclr_raw[i2] = da2 * a2 * (1.0f - a2);
    // rotary: out1 = x1 cos - x2 sin, out2 = x2 cos + x1 sin
    p.d_k_raw[i1] = dk1 * cs + dk2 * sn; p.d_k_raw[i2] = dk2 * cs - dk1 * sn;
    const float gr1 = p.g_r[i1], gr2 = p.g_r[i2];
    p.d_r_raw[i1] = gr1 * cs + gr2 * sn; p.d_r_raw[i2] = gr2 * cs - gr1 * sn;
    // decay = exp(-e), e = exp(d)
    const float e1 = __expf(f.d[i1]), e2 = __expf(f.d[i2]);
    p.d_d[i1] = -p.g_decay[i1] * __expf(-e1) * e1; p.d_d[i2] = -p.g_decay[i2] * __expf(-e2) * e2;
    const float gv1 = p.g_v[i1], gv2 = p.g_v[i2];
    if (f.v0) {
      const float nu1 = sigmoid_fast(f.nu_raw[i1]), nu2 = sigmoid_fast(f.nu_raw[i2]);
      p.d_v_prime[i1] = gv1 - gv1 * nu1; p.d_v_prime[i2] = gv2 - gv2 * nu2;
      p.d_v0[i1] = gv1 * nu1; p.d_v0[i2] = gv2 * nu2;
      p.d_nu_raw[i1] = gv1 * (f.v0[i1] - f.v_prime[i1]) * nu1 * (1.0f - nu1);
      p.d_nu_raw[i2] = gv2 * (f.v0[i2] - f.v_prime[i2]) * nu2 * (1.0f - nu2);
    } else {
      p.d_v_prime[i1] = gv1; p.d_v_prime[i2] = gv2;
    }
  }
  float* part = p.partial + (size_t)tile * 2 * C;
  part[c1] = dm1; part[c2] = dm2;
  part[C + c1] = dx1; part[C + c2] = dx2;
}

int grid_stride_blocks(int64_t items_per_thread_unit) {
  const int64_t want = (items_per_thread_unit + kGlueThreads - 1) / kGlueThreads;
  const int64_t cap = (int64_t)sm_count() * 16;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

bool misaligned(std::initializer_list<const void*> ptrs) {
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return true;
  return false;
}

}  // namespace
}  // namespace pb

using namespace pb;

extern "C" int pb_token_shift_lerp(const float* x, const float* state, const float* mu, int64_t batch, int64_t steps, int64_t channels,
                                   int n_mix, float* out, void* stream) {
  if (!x || !mu || !out) return fail(PB_ERR_NULL_POINTER, "pb_token_shift_lerp: x, mu and out must be non-null");
  if (batch <= 0 || steps <= 0 || channels <= 0 || channels % 4 != 0 || steps > 0x7fffffffll || channels > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "pb_token_shift_lerp: batch=%lld steps=%lld channels=%lld (channels must be a multiple of 4)",
                (long long)batch, (long long)steps, (long long)channels);
  if (n_mix <= 0 || n_mix > kMaxMix) return fail(PB_ERR_UNSUPPORTED, "pb_token_shift_lerp: n_mix=%d (1..%d)", n_mix, kMaxMix);
  if (misaligned({x, state, mu, out})) return fail(PB_ERR_MISALIGNED, "pb_token_shift_lerp: every array must be 16-byte aligned");
  ShiftLerpParams p{x, state, mu, out, batch * steps, (int)steps, (int)channels, n_mix};
  shift_lerp_fwd_kernel<<<grid_stride_blocks(p.R * (channels / 4)), kGlueThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PB_LAUNCH_CHECK("shift_lerp_fwd_kernel");
  return PB_OK;
}

extern "C" size_t pb_token_shift_lerp_bwd_workspace_size(int64_t batch, int64_t steps, int64_t channels, int n_mix) {
  if (batch <= 0 || steps <= 0 || channels <= 0 || n_mix <= 0) return 0;
  const int64_t tiles = (batch * steps + kLerpTileRows - 1) / kLerpTileRows;
  return (size_t)tiles * n_mix * channels * sizeof(float);
}

extern "C" int pb_token_shift_lerp_bwd(const float* const* g, const float* x, const float* state, const float* mu,
                                       int64_t batch, int64_t steps, int64_t channels, int n_mix,
                                       float* dx, float* dstate, float* dmu, void* workspace, size_t workspace_bytes, void* stream) {
  if (!g || !x || !mu || !dx || !dmu) return fail(PB_ERR_NULL_POINTER, "pb_token_shift_lerp_bwd: g, x, mu, dx and dmu must be non-null");
  if (batch <= 0 || steps <= 0 || channels <= 0 || channels % 4 != 0 || steps > 0x7fffffffll || channels > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "pb_token_shift_lerp_bwd: batch=%lld steps=%lld channels=%lld", (long long)batch, (long long)steps, (long long)channels);
  if (n_mix != 1 && n_mix != 6) return fail(PB_ERR_UNSUPPORTED, "pb_token_shift_lerp_bwd: n_mix=%d (built for 1 and 6)", n_mix);
  const size_t need = pb_token_shift_lerp_bwd_workspace_size(batch, steps, channels, n_mix);
  if (!workspace || workspace_bytes < need)
    return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_token_shift_lerp_bwd: needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  if (misaligned({x, state, mu, dx, dstate, dmu, workspace})) return fail(PB_ERR_MISALIGNED, "pb_token_shift_lerp_bwd: every array must be 16-byte aligned");
  for (int k = 0; k < n_mix; ++k)
    if (!g[k] || (reinterpret_cast<uintptr_t>(g[k]) & 15)) return fail(PB_ERR_MISALIGNED, "pb_token_shift_lerp_bwd: g[%d] must be non-null and 16-byte aligned", k);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t R = batch * steps;
  const int tiles = (int)((R + kLerpTileRows - 1) / kLerpTileRows);
  ShiftLerpBwdParams p{{}, x, state, mu, dx, dstate, static_cast<float*>(workspace), R, (int)steps, (int)channels, n_mix};
  for (int k = 0; k < n_mix; ++k) p.g[k] = g[k];
  const dim3 grid((unsigned)((channels / 4 + kGlueThreads - 1) / kGlueThreads), (unsigned)tiles);
  if (n_mix == 6) shift_lerp_bwd_kernel<6><<<grid, kGlueThreads, 0, st>>>(p);
  else shift_lerp_bwd_kernel<1><<<grid, kGlueThreads, 0, st>>>(p);
  PB_LAUNCH_CHECK("shift_lerp_bwd_kernel");
  const int64_t n = (int64_t)n_mix * channels;
  reduce_partials_kernel<<<(unsigned)((n + 31) / 32), kGlueThreads, 0, st>>>(p.partial, dmu, tiles, n);
  PB_LAUNCH_CHECK("reduce_partials_kernel");
  return PB_OK;
}

static int check_prepare(const char* who, int64_t batch, int64_t steps, int64_t heads, int head_dim) {
  if (head_dim != kGlueH) return fail(PB_ERR_UNSUPPORTED, "%s: head size %d (this kernel is built for %d)", who, head_dim, kGlueH);
  if (batch <= 0 || steps <= 0 || heads <= 0 || steps > 0x7fffffffll || heads > 0x7fffffll)
    return fail(PB_ERR_BAD_SHAPE, "%s: batch=%lld steps=%lld heads=%lld", who, (long long)batch, (long long)steps, (long long)heads);
  return PB_OK;
}

extern "C" int pb_wkv_prepare(const float* r_raw, const float* k_raw, const float* d, const float* iclr_raw, const float* v_prime,
                              const float* v0, const float* nu_raw, const float* cos_tab, const float* sin_tab,
                              const float* rk_mult, const float* mix_amt, int64_t batch, int64_t steps, int64_t heads, int head_dim,
                              float* decay, float* iclr, float* removal_k, float* replacement_k, float* v, float* r, float* k, void* stream) {
  if (int s = check_prepare("pb_wkv_prepare", batch, steps, heads, head_dim)) return s;
  if (!r_raw || !k_raw || !d || !iclr_raw || !v_prime || !cos_tab || !sin_tab || !rk_mult || !mix_amt || !decay || !iclr || !removal_k ||
      !replacement_k || !v || !r || !k)
    return fail(PB_ERR_NULL_POINTER, "pb_wkv_prepare: only v0 and nu_raw may be null");
  if ((v0 == nullptr) != (nu_raw == nullptr)) return fail(PB_ERR_NULL_POINTER, "pb_wkv_prepare: v0 and nu_raw come together");
  PrepareParams p{r_raw, k_raw, d, iclr_raw, v_prime, v0, nu_raw, cos_tab, sin_tab, rk_mult, mix_amt,
                  decay, iclr, removal_k, replacement_k, v, r, k, batch * steps, (int)steps, (int)heads};
  wkv_prepare_fwd_kernel<<<grid_stride_blocks(p.R * heads * 32), kGlueThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PB_LAUNCH_CHECK("wkv_prepare_fwd_kernel");
  return PB_OK;
}

extern "C" size_t pb_wkv_prepare_bwd_workspace_size(int64_t batch, int64_t steps, int64_t heads, int head_dim) {
  if (batch <= 0 || steps <= 0 || heads <= 0 || head_dim != kGlueH) return 0;
  const int64_t tiles = (batch * steps + kPrepTileRows - 1) / kPrepTileRows;
  return (size_t)tiles * 2 * heads * kGlueH * sizeof(float);
}

extern "C" int pb_wkv_prepare_bwd(const float* r_raw, const float* k_raw, const float* d, const float* iclr_raw, const float* v_prime,
                                  const float* v0, const float* nu_raw, const float* cos_tab, const float* sin_tab,
                                  const float* rk_mult, const float* mix_amt, int64_t batch, int64_t steps, int64_t heads, int head_dim,
                                  const float* g_decay, const float* g_iclr, const float* g_removal_k, const float* g_replacement_k,
                                  const float* g_v, const float* g_r, const float* g_k,
                                  float* d_r_raw, float* d_k_raw, float* d_d, float* d_iclr_raw, float* d_v_prime, float* d_v0, float* d_nu_raw,
                                  float* d_rk_mult, float* d_mix_amt, void* workspace, size_t workspace_bytes, void* stream) {
  if (int s = check_prepare("pb_wkv_prepare_bwd", batch, steps, heads, head_dim)) return s;
  if (!r_raw || !k_raw || !d || !iclr_raw || !v_prime || !cos_tab || !sin_tab || !rk_mult || !mix_amt || !g_decay || !g_iclr ||
      !g_removal_k || !g_replacement_k || !g_v || !g_r || !g_k || !d_r_raw || !d_k_raw || !d_d || !d_iclr_raw || !d_v_prime ||
      !d_rk_mult || !d_mix_amt)
    return fail(PB_ERR_NULL_POINTER, "pb_wkv_prepare_bwd: only v0, nu_raw, d_v0 and d_nu_raw may be null");
  if ((v0 == nullptr) != (nu_raw == nullptr) || (v0 != nullptr && (!d_v0 || !d_nu_raw)))
    return fail(PB_ERR_NULL_POINTER, "pb_wkv_prepare_bwd: v0, nu_raw, d_v0 and d_nu_raw come together");
  const size_t need = pb_wkv_prepare_bwd_workspace_size(batch, steps, heads, head_dim);
  if (!workspace || workspace_bytes < need)
    return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_wkv_prepare_bwd: needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t R = batch * steps;
  const int tiles = (int)((R + kPrepTileRows - 1) / kPrepTileRows);
  const int64_t C = heads * kGlueH;
  PrepareBwdParams p{{r_raw, k_raw, d, iclr_raw, v_prime, v0, nu_raw, cos_tab, sin_tab, rk_mult, mix_amt,
                      nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, R, (int)steps, (int)heads},
                     g_decay, g_iclr, g_removal_k, g_replacement_k, g_v, g_r, g_k,
                     d_r_raw, d_k_raw, d_d, d_iclr_raw, d_v_prime, d_v0, d_nu_raw, static_cast<float*>(workspace)};
  const int64_t warps = (int64_t)tiles * heads;
  wkv_prepare_bwd_kernel<<<(unsigned)((warps + kGlueThreads / 32 - 1) / (kGlueThreads / 32)), kGlueThreads, 0, st>>>(p);
  PB_LAUNCH_CHECK("wkv_prepare_bwd_kernel");
  // partial is [tiles][2][C]: the two parameters' sums come out as one [2][C] array, split below
  float* sums = static_cast<float*>(workspace);      // reduced in place into the first tile's slot after the reduction reads it
  reduce_partials_kernel<<<(unsigned)((2 * C + 31) / 32), kGlueThreads, 0, st>>>(p.partial, sums, tiles, 2 * C);
  PB_LAUNCH_CHECK("reduce_partials_kernel");
  PB_CUDA_TRY(cudaMemcpyAsync(d_rk_mult, sums, (size_t)C * sizeof(float), cudaMemcpyDeviceToDevice, st));
  PB_CUDA_TRY(cudaMemcpyAsync(d_mix_amt, sums + C, (size_t)C * sizeof(float), cudaMemcpyDeviceToDevice, st));
  return PB_OK;
}
