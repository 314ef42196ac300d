// More of the f32 element-wise work of the modified RWKV-7 block (pratchya/_nnx_impl/_module.py), fused:
//
//   RMSNorm (:61-72)                                                              pb_rms_norm(_bwd)
//   relu(k)^2 between ChannelMix's linears (:249)                                 pb_relu2(_bwd)
//   TimeMix after its scan (:208-216): GroupNorm over (timesteps x head channels) per batch element and head,
//   the bonus term sum_c(r k m) * v over all channels of a token, and the gate    pb_wkv_finish(_bwd)
//
// Forward values follow the reference's order of operations ((x * inv_rms) * scale; ((y - mean) * rstd) * scale +
// bias; (gn + dot * v) * gate); sums (mean of squares, group statistics, the bonus dot product) are formed in
// this file's own order.  Sums over tokens for parameter gradients go through per-tile partials added in tile
// order: no atomics, the same bits every run.
#include "common.cuh"

namespace pb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kH = 64;
constexpr int kTileRows = 32;             // tokens per CTA / per warp where a parameter gradient is summed over tokens
constexpr int kStatTileSteps = 256;       // timesteps per CTA of the group statistics

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// out[j] = sum over tiles of partial[tile][j]: eight partial sums per column (tiles g, g + 8, ...), added in a fixed order.
// A block takes 32 columns; out may be the first tile's slot of partial (a column is read and written by its block only).
__global__ void __launch_bounds__(kThreads) reduce_tiles_kernel(const float* partial, float* out, int tiles, int64_t n) {
  __shared__ float red[kWarps][32];
  const int cx = threadIdx.x & 31, gy = threadIdx.x >> 5;
  const int64_t j = (int64_t)blockIdx.x * 32 + cx;
  float s = 0.0f;
  if (j < n)
    for (int t = gy; t < tiles; t += kWarps) s += partial[(size_t)t * n + j];
  red[gy][cx] = s;
  __syncthreads();
  if (gy == 0 && j < n) {
    float r = red[0][cx];
#pragma unroll
    for (int g = 1; g < kWarps; ++g) r += red[g][cx];
    out[j] = r;
  }
}

// ---- RMSNorm: y = (x * rsqrt(mean(x^2) + eps)) * scale, one warp per row --------------------------------------
__global__ void __launch_bounds__(kThreads) rms_norm_fwd_kernel(const float* x, const float* scale, float* y, float* inv_rms,
                                                               int64_t R, int C, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  for (int64_t row = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); row < R; row += warps) {
    const float* xr = x + row * C;
    float ss = 0.0f;
    for (int c = lane * 4; c < C; c += 128) {
      const float4 v = ld4(xr + c);
      ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    }
    const float inv = rsqrtf(__fadd_rn(__fdiv_rn(warp_sum(ss), (float)C), eps));
    if (lane == 0) inv_rms[row] = inv;
    for (int c = lane * 4; c < C; c += 128) {
      const float4 v = ld4(xr + c);
      const float4 s = __ldg(reinterpret_cast<const float4*>(scale + c));
      st4(y + row * C + c, make_float4(__fmul_rn(__fmul_rn(v.x, inv), s.x), __fmul_rn(__fmul_rn(v.y, inv), s.y),
                                       __fmul_rn(__fmul_rn(v.z, inv), s.z), __fmul_rn(__fmul_rn(v.w, inv), s.w)));
    }
  }
}

// dx = inv * (dy * scale) - x * (inv^3 * sum_c(dy * scale * x) / C)
__global__ void __launch_bounds__(kThreads) rms_norm_bwd_dx_kernel(const float* dy, const float* x, const float* scale, const float* inv_rms,
                                                                  float* dx, int64_t R, int C) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  for (int64_t row = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); row < R; row += warps) {
    const float* xr = x + row * C;
    const float* gr = dy + row * C;
    float dot = 0.0f;
    for (int c = lane * 4; c < C; c += 128) {
      const float4 v = ld4(xr + c), g = ld4(gr + c);
      const float4 s = __ldg(reinterpret_cast<const float4*>(scale + c));
      dot += (g.x * s.x * v.x + g.y * s.y * v.y) + (g.z * s.z * v.z + g.w * s.w * v.w);
    }
    const float inv = inv_rms[row];
    const float k = inv * inv * inv * warp_sum(dot) / (float)C;
    for (int c = lane * 4; c < C; c += 128) {
      const float4 v = ld4(xr + c), g = ld4(gr + c);
      const float4 s = __ldg(reinterpret_cast<const float4*>(scale + c));
      st4(dx + row * C + c, make_float4(inv * (g.x * s.x) - v.x * k, inv * (g.y * s.y) - v.y * k, inv * (g.z * s.z) - v.z * k, inv * (g.w * s.w) - v.w * k));
    }
  }
}

// partial[tile][c] = sum over the tile's rows of dy * x * inv_rms
__global__ void __launch_bounds__(kThreads) rms_norm_bwd_dscale_kernel(const float* dy, const float* x, const float* inv_rms, float* partial,
                                                                      int64_t R, int C) {
  const int c = (blockIdx.x * kThreads + threadIdx.x) << 2;
  if (c >= C) return;
  const int64_t r0 = (int64_t)blockIdx.y * kTileRows, r1 = min(R, r0 + kTileRows);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int64_t r = r0; r < r1; ++r) {
    const float4 v = ld4(x + r * C + c), g = ld4(dy + r * C + c);
    const float inv = __ldg(inv_rms + r);
    acc.x = fmaf(g.x * v.x, inv, acc.x); acc.y = fmaf(g.y * v.y, inv, acc.y);
    acc.z = fmaf(g.z * v.z, inv, acc.z); acc.w = fmaf(g.w * v.w, inv, acc.w);
  }
  st4(partial + (size_t)blockIdx.y * C + c, acc);
}

// ---- relu(x)^2 -----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) relu2_fwd_kernel(const float4* x, float4* y, int64_t n4) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = x[i];
    const float a = fmaxf(v.x, 0.f), b = fmaxf(v.y, 0.f), c = fmaxf(v.z, 0.f), d = fmaxf(v.w, 0.f);
    y[i] = make_float4(a * a, b * b, c * c, d * d);
  }
}
__global__ void __launch_bounds__(kThreads) relu2_bwd_kernel(const float4* g, const float4* x, float4* dx, int64_t n4) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = x[i], gg = g[i];
    dx[i] = make_float4(gg.x * (2.0f * fmaxf(v.x, 0.f)), gg.y * (2.0f * fmaxf(v.y, 0.f)), gg.z * (2.0f * fmaxf(v.z, 0.f)), gg.w * (2.0f * fmaxf(v.w, 0.f)));
  }
}

// ---- TimeMix after the scan ------------------------------------------------------------------------------------
// GroupNorm as flax builds it on [B, T, C] with one group per head (_module.py:118-123): per (batch element, head)
// the mean and the variance E[x^2] - E[x]^2 (clamped at 0) over the T x 64 values.
// group_sums_kernel: partial[b][n][tile][2] = (sum, sum of squares) over a tile of kStatTileSteps timesteps.
__global__ void __launch_bounds__(kThreads) group_sums_kernel(const float* y, float* partial, int T, int N, int tiles) {
  __shared__ float red[kWarps][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int bn = blockIdx.x, tile = blockIdx.y;
  const int b = bn / N, n = bn - b * N;
  const int C = N * kH;
  const int t1 = min(T, (tile + 1) * kStatTileSteps);
  float s = 0.f, q = 0.f;
  for (int t = tile * kStatTileSteps + warp; t < t1; t += kWarps) {
    const float* p = y + ((size_t)b * T + t) * C + n * kH + lane;
    const float a = p[0], c = p[32];
    s += a + c; q += a * a + c * c;
  }
  s = warp_sum(s); q = warp_sum(q);
  if (lane == 0) { red[warp][0] = s; red[warp][1] = q; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float ts = 0.f, tq = 0.f;
    for (int w = 0; w < kWarps; ++w) { ts += red[w][0]; tq += red[w][1]; }
    partial[((size_t)bn * tiles + tile) * 2] = ts;
    partial[((size_t)bn * tiles + tile) * 2 + 1] = tq;
  }
}
// stats[bn] = (mean, rstd)
__global__ void group_stats_kernel(const float* partial, float* stats, int groups, int tiles, float count, float eps) {
  const int bn = blockIdx.x * blockDim.x + threadIdx.x;
  if (bn >= groups) return;
  float s = 0.f, q = 0.f;
  for (int t = 0; t < tiles; ++t) { s += partial[((size_t)bn * tiles + t) * 2]; q += partial[((size_t)bn * tiles + t) * 2 + 1]; }
  const float mean = s / count;
  const float var = fmaxf(q / count - mean * mean, 0.0f);
  stats[2 * bn] = mean;
  stats[2 * bn + 1] = rsqrtf(var + eps);
}

struct FinishParams {
  const float* y; const float* r; const float* k; const float* v; const float* gate;
  const float* gn_scale; const float* gn_bias; const float* bonus_mult;     // [C]
  const float* stats;                                                       // [B * N][2]
  float* out;
  int64_t R; int T, N;
};

// One warp per token: first the bonus dot product over all channels, then the output head by head.
__global__ void __launch_bounds__(kThreads) wkv_finish_fwd_kernel(const FinishParams p) {
  const int lane = threadIdx.x & 31;
  const int C = p.N * kH;
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  for (int64_t row = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); row < p.R; row += warps) {
    const size_t base = (size_t)row * C;
    float dot = 0.0f;
    for (int c = lane; c < C; c += 32) dot = fmaf(__fmul_rn(p.r[base + c], p.k[base + c]), __ldg(p.bonus_mult + c), dot);
    dot = warp_sum(dot);
    const int b = (int)(row / p.T);
    for (int n = 0; n < p.N; ++n) {
      const float mean = __ldg(p.stats + 2 * (b * p.N + n)), rstd = __ldg(p.stats + 2 * (b * p.N + n) + 1);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = n * kH + lane + 32 * h;
        const float gn = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(p.y[base + c], mean), rstd), __ldg(p.gn_scale + c)), __ldg(p.gn_bias + c));
        p.out[base + c] = __fmul_rn(__fadd_rn(gn, __fmul_rn(dot, p.v[base + c])), p.gate[base + c]);
      }
    }
  }
}

// Backward, first pass (one warp per token): the token's dot = sum_c r k m and d_dot = sum_c g gate v, and per head
// the token's share of sum(dxhat) and sum(dxhat * xhat), dxhat = g * gate * gn_scale.
struct FinishBwdParams {
  FinishParams f;
  const float* g;                      // cotangent of out
  float* token_scalars;                // [R][2]: dot, d_dot
  float* head_sums;                    // [R][N][2]
  const float* group_terms;            // [B * N][2]: mean over the group of dxhat and of dxhat * xhat
  float* d_y; float* d_r; float* d_k; float* d_v; float* d_gate;
  float* partial;                      // [tiles][3][C]: gn_scale, gn_bias, bonus_mult
};

__global__ void __launch_bounds__(kThreads) wkv_finish_bwd_scalars_kernel(const FinishBwdParams p) {
  const FinishParams& f = p.f;
  const int lane = threadIdx.x & 31;
  const int C = f.N * kH;
  const int64_t warps = (int64_t)gridDim.x * kWarps;
  for (int64_t row = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); row < f.R; row += warps) {
    const size_t base = (size_t)row * C;
    const int b = (int)(row / f.T);
    float dot = 0.f, ddot = 0.f;
    for (int n = 0; n < f.N; ++n) {
      const float mean = __ldg(f.stats + 2 * (b * f.N + n)), rstd = __ldg(f.stats + 2 * (b * f.N + n) + 1);
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = n * kH + lane + 32 * h;
        const float dpre = p.g[base + c] * f.gate[base + c];
        dot = fmaf(__fmul_rn(f.r[base + c], f.k[base + c]), __ldg(f.bonus_mult + c), dot);
        ddot = fmaf(dpre, f.v[base + c], ddot);
        const float dxhat = dpre * __ldg(f.gn_scale + c);
        s1 += dxhat;
        s2 = fmaf(dxhat, (f.y[base + c] - mean) * rstd, s2);
      }
      s1 = warp_sum(s1); s2 = warp_sum(s2);
      if (lane == 0) { p.head_sums[((size_t)row * f.N + n) * 2] = s1; p.head_sums[((size_t)row * f.N + n) * 2 + 1] = s2; }
    }
    dot = warp_sum(dot); ddot = warp_sum(ddot);
    if (lane == 0) { p.token_scalars[2 * row] = dot; p.token_scalars[2 * row + 1] = ddot; }
  }
}

// group_terms[bn] = (sum_t head_sums[b, t, n, 0], sum_t head_sums[b, t, n, 1]) / (T * 64); one CTA per (b, n)
__global__ void __launch_bounds__(kThreads) group_terms_kernel(const float* head_sums, float* group_terms, int T, int N) {
  __shared__ float red[kWarps][2];
  const int bn = blockIdx.x, b = bn / N, n = bn - b * N;
  float s1 = 0.f, s2 = 0.f;
  for (int t = threadIdx.x; t < T; t += kThreads) {
    const float* p = head_sums + (((size_t)b * T + t) * N + n) * 2;
    s1 += p[0]; s2 += p[1];
  }
  s1 = warp_sum(s1); s2 = warp_sum(s2);
  if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5][0] = s1; red[threadIdx.x >> 5][1] = s2; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, c = 0.f;
    for (int w = 0; w < kWarps; ++w) { a += red[w][0]; c += red[w][1]; }
    const float count = (float)T * (float)kH;
    group_terms[2 * bn] = a / count;
    group_terms[2 * bn + 1] = c / count;
  }
}

// Backward, second pass: one warp per (head, tile of tokens); lane l holds channels l and l + 32 of the head and
// adds up their share of the three parameter gradients over the tile's tokens.
__global__ void __launch_bounds__(kThreads) wkv_finish_bwd_main_kernel(const FinishBwdParams p) {
  const FinishParams& f = p.f;
  const int lane = threadIdx.x & 31;
  const int C = f.N * kH;
  const int tiles = (int)((f.R + kTileRows - 1) / kTileRows);
  const int64_t w = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (w >= (int64_t)tiles * f.N) return;
  const int tile = (int)(w / f.N), n = (int)(w - (int64_t)tile * f.N);
  float dgs[2] = {0.f, 0.f}, dgb[2] = {0.f, 0.f}, dbm[2] = {0.f, 0.f};
  float gs[2], gb[2], bm[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int c = n * kH + lane + 32 * h;
    gs[h] = __ldg(f.gn_scale + c); gb[h] = __ldg(f.gn_bias + c); bm[h] = __ldg(f.bonus_mult + c);
  }
  const int64_t row_end = min(f.R, (int64_t)(tile + 1) * kTileRows);
  for (int64_t row = (int64_t)tile * kTileRows; row < row_end; ++row) {
    const int b = (int)(row / f.T);
    const float mean = __ldg(f.stats + 2 * (b * f.N + n)), rstd = __ldg(f.stats + 2 * (b * f.N + n) + 1);
    const float m1 = __ldg(p.group_terms + 2 * (b * f.N + n)), m2 = __ldg(p.group_terms + 2 * (b * f.N + n) + 1);
    const float dot = __ldg(p.token_scalars + 2 * row), ddot = __ldg(p.token_scalars + 2 * row + 1);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const size_t i = (size_t)row * C + n * kH + lane + 32 * h;
      const float g = p.g[i], gate = f.gate[i], v = f.v[i], r = f.r[i], k = f.k[i];
      const float xhat = (f.y[i] - mean) * rstd;
      const float gn = xhat * gs[h] + gb[h];
      const float dpre = g * gate;
      p.d_gate[i] = g * (gn + dot * v);
      p.d_v[i] = dpre * dot;
      p.d_r[i] = ddot * k * bm[h];
      p.d_k[i] = ddot * r * bm[h];
      dbm[h] = fmaf(ddot, r * k, dbm[h]);
      dgb[h] += dpre;
      dgs[h] = fmaf(dpre, xhat, dgs[h]);
      const float dxhat = dpre * gs[h];
      p.d_y[i] = rstd * (dxhat - m1 - xhat * m2);
    }
  }
  float* part = p.partial + (size_t)tile * 3 * C;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int c = n * kH + lane + 32 * h;
    part[c] = dgs[h]; part[C + c] = dgb[h]; part[2 * C + c] = dbm[h];
  }
}

int blocks_for(int64_t units, int per_block) {
  const int64_t want = (units + per_block - 1) / per_block;
  const int64_t cap = (int64_t)sm_count() * 16;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

bool any_misaligned(std::initializer_list<const void*> ptrs) {
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return true;
  return false;
}

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace
}  // namespace pb

using namespace pb;

extern "C" int pb_rms_norm(const float* x, const float* scale, int64_t rows, int64_t channels, float eps, float* y, float* inv_rms, void* stream) {
  if (!x || !scale || !y || !inv_rms) return fail(PB_ERR_NULL_POINTER, "pb_rms_norm: x, scale, y and inv_rms must be non-null");
  if (rows <= 0 || channels <= 0 || channels % 128 != 0 || channels > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "pb_rms_norm: rows=%lld channels=%lld (channels must be a multiple of 128)", (long long)rows, (long long)channels);
  if (any_misaligned({x, scale, y})) return fail(PB_ERR_MISALIGNED, "pb_rms_norm: x, scale and y must be 16-byte aligned");
  rms_norm_fwd_kernel<<<blocks_for(rows, kWarps), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, scale, y, inv_rms, rows, (int)channels, eps);
  PB_LAUNCH_CHECK("rms_norm_fwd_kernel");
  return PB_OK;
}

extern "C" size_t pb_rms_norm_bwd_workspace_size(int64_t rows, int64_t channels) {
  if (rows <= 0 || channels <= 0) return 0;
  return (size_t)((rows + kTileRows - 1) / kTileRows) * channels * sizeof(float);
}

extern "C" int pb_rms_norm_bwd(const float* dy, const float* x, const float* scale, const float* inv_rms, int64_t rows, int64_t channels,
                               float* dx, float* dscale, void* workspace, size_t workspace_bytes, void* stream) {
  if (!dy || !x || !scale || !inv_rms || !dx || !dscale) return fail(PB_ERR_NULL_POINTER, "pb_rms_norm_bwd: null argument");
  if (rows <= 0 || channels <= 0 || channels % 128 != 0 || channels > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "pb_rms_norm_bwd: rows=%lld channels=%lld", (long long)rows, (long long)channels);
  const size_t need = pb_rms_norm_bwd_workspace_size(rows, channels);
  if (!workspace || workspace_bytes < need) return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_rms_norm_bwd: needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  if (any_misaligned({dy, x, scale, dx, workspace})) return fail(PB_ERR_MISALIGNED, "pb_rms_norm_bwd: arrays must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rms_norm_bwd_dx_kernel<<<blocks_for(rows, kWarps), kThreads, 0, st>>>(dy, x, scale, inv_rms, dx, rows, (int)channels);
  PB_LAUNCH_CHECK("rms_norm_bwd_dx_kernel");
  const int tiles = (int)((rows + kTileRows - 1) / kTileRows);
  const dim3 grid((unsigned)((channels / 4 + kThreads - 1) / kThreads), (unsigned)tiles);
  rms_norm_bwd_dscale_kernel<<<grid, kThreads, 0, st>>>(dy, x, inv_rms, static_cast<float*>(workspace), rows, (int)channels);
  PB_LAUNCH_CHECK("rms_norm_bwd_dscale_kernel");
  reduce_tiles_kernel<<<(unsigned)((channels + 31) / 32), kThreads, 0, st>>>(static_cast<const float*>(workspace), dscale, tiles, channels);
  PB_LAUNCH_CHECK("reduce_tiles_kernel");
  return PB_OK;
}

extern "C" int pb_relu2(const float* x, int64_t n, float* y, void* stream) {
  if (!x || !y) return fail(PB_ERR_NULL_POINTER, "pb_relu2: x and y must be non-null");
  if (n <= 0 || n % 4 != 0) return fail(PB_ERR_BAD_SHAPE, "pb_relu2: n=%lld must be a positive multiple of 4", (long long)n);
  if (any_misaligned({x, y})) return fail(PB_ERR_MISALIGNED, "pb_relu2: x and y must be 16-byte aligned");
  relu2_fwd_kernel<<<blocks_for(n / 4, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), n / 4);
  PB_LAUNCH_CHECK("relu2_fwd_kernel");
  return PB_OK;
}

extern "C" int pb_relu2_bwd(const float* g, const float* x, int64_t n, float* dx, void* stream) {
  if (!g || !x || !dx) return fail(PB_ERR_NULL_POINTER, "pb_relu2_bwd: g, x and dx must be non-null");
  if (n <= 0 || n % 4 != 0) return fail(PB_ERR_BAD_SHAPE, "pb_relu2_bwd: n=%lld must be a positive multiple of 4", (long long)n);
  if (any_misaligned({g, x, dx})) return fail(PB_ERR_MISALIGNED, "pb_relu2_bwd: g, x and dx must be 16-byte aligned");
  relu2_bwd_kernel<<<blocks_for(n / 4, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(g), reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(dx), n / 4);
  PB_LAUNCH_CHECK("relu2_bwd_kernel");
  return PB_OK;
}

static int check_finish(const char* who, int64_t batch, int64_t steps, int64_t heads, int head_dim) {
  if (head_dim != kH) return fail(PB_ERR_UNSUPPORTED, "%s: head size %d (this kernel is built for %d)", who, head_dim, kH);
  if (batch <= 0 || steps <= 0 || heads <= 0 || steps > 0x7fffffffll || heads > 0xffffll || batch * heads > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "%s: batch=%lld steps=%lld heads=%lld", who, (long long)batch, (long long)steps, (long long)heads);
  return PB_OK;
}

// workspace of the forward call: the per-tile sums of the group statistics
extern "C" size_t pb_wkv_finish_workspace_size(int64_t batch, int64_t steps, int64_t heads, int head_dim) {
  if (batch <= 0 || steps <= 0 || heads <= 0 || head_dim != kH) return 0;
  return (size_t)batch * heads * ((steps + kStatTileSteps - 1) / kStatTileSteps) * 2 * sizeof(float);
}

extern "C" int pb_wkv_finish(const float* y, const float* r, const float* k, const float* v, const float* gate,
                             const float* gn_scale, const float* gn_bias, const float* bonus_mult, float eps,
                             int64_t batch, int64_t steps, int64_t heads, int head_dim,
                             float* out, float* stats, void* workspace, size_t workspace_bytes, void* stream) {
  if (int s = check_finish("pb_wkv_finish", batch, steps, heads, head_dim)) return s;
  if (!y || !r || !k || !v || !gate || !gn_scale || !gn_bias || !bonus_mult || !out || !stats)
    return fail(PB_ERR_NULL_POINTER, "pb_wkv_finish: null argument");
  const size_t need = pb_wkv_finish_workspace_size(batch, steps, heads, head_dim);
  if (!workspace || workspace_bytes < need) return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_wkv_finish: needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int tiles = (int)((steps + kStatTileSteps - 1) / kStatTileSteps);
  const int groups = (int)(batch * heads);
  group_sums_kernel<<<dim3((unsigned)groups, (unsigned)tiles), kThreads, 0, st>>>(y, static_cast<float*>(workspace), (int)steps, (int)heads, tiles);
  PB_LAUNCH_CHECK("group_sums_kernel");
  group_stats_kernel<<<(groups + 127) / 128, 128, 0, st>>>(static_cast<const float*>(workspace), stats, groups, tiles, (float)steps * (float)kH, eps);
  PB_LAUNCH_CHECK("group_stats_kernel");
  FinishParams p{y, r, k, v, gate, gn_scale, gn_bias, bonus_mult, stats, out, batch * steps, (int)steps, (int)heads};
  wkv_finish_fwd_kernel<<<blocks_for(p.R, kWarps), kThreads, 0, st>>>(p);
  PB_LAUNCH_CHECK("wkv_finish_fwd_kernel");
  return PB_OK;
}

extern "C" size_t pb_wkv_finish_bwd_workspace_size(int64_t batch, int64_t steps, int64_t heads, int head_dim) {
  if (batch <= 0 || steps <= 0 || heads <= 0 || head_dim != kH) return 0;
  const int64_t R = batch * steps, C = heads * kH;
  const int64_t tiles = (R + kTileRows - 1) / kTileRows;
  return align256((size_t)R * 2 * 4) + align256((size_t)R * heads * 2 * 4) + align256((size_t)batch * heads * 2 * 4) + (size_t)tiles * 3 * C * 4;
}

extern "C" int pb_wkv_finish_bwd(const float* g, const float* y, const float* r, const float* k, const float* v, const float* gate,
                                 const float* gn_scale, const float* gn_bias, const float* bonus_mult, const float* stats,
                                 int64_t batch, int64_t steps, int64_t heads, int head_dim,
                                 float* d_y, float* d_r, float* d_k, float* d_v, float* d_gate,
                                 float* d_gn_scale, float* d_gn_bias, float* d_bonus_mult,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  if (int s = check_finish("pb_wkv_finish_bwd", batch, steps, heads, head_dim)) return s;
  if (!g || !y || !r || !k || !v || !gate || !gn_scale || !gn_bias || !bonus_mult || !stats || !d_y || !d_r || !d_k || !d_v || !d_gate ||
      !d_gn_scale || !d_gn_bias || !d_bonus_mult)
    return fail(PB_ERR_NULL_POINTER, "pb_wkv_finish_bwd: null argument");
  const size_t need = pb_wkv_finish_bwd_workspace_size(batch, steps, heads, head_dim);
  if (!workspace || workspace_bytes < need) return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_wkv_finish_bwd: needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(PB_ERR_MISALIGNED, "pb_wkv_finish_bwd: workspace must be 256-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t R = batch * steps, C = heads * kH;
  const int tiles = (int)((R + kTileRows - 1) / kTileRows);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* scalars = reinterpret_cast<float*>(ws);
  float* head_sums = reinterpret_cast<float*>(ws + align256((size_t)R * 2 * 4));
  float* group_terms = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(head_sums) + align256((size_t)R * heads * 2 * 4));
  float* partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(group_terms) + align256((size_t)batch * heads * 2 * 4));
  FinishBwdParams p{{y, r, k, v, gate, gn_scale, gn_bias, bonus_mult, stats, nullptr, R, (int)steps, (int)heads},
                    g, scalars, head_sums, group_terms, d_y, d_r, d_k, d_v, d_gate, partial};
  wkv_finish_bwd_scalars_kernel<<<blocks_for(R, kWarps), kThreads, 0, st>>>(p);
  PB_LAUNCH_CHECK("wkv_finish_bwd_scalars_kernel");
  group_terms_kernel<<<(unsigned)(batch * heads), kThreads, 0, st>>>(head_sums, group_terms, (int)steps, (int)heads);
  PB_LAUNCH_CHECK("group_terms_kernel");
  const int64_t warps = (int64_t)tiles * heads;
  wkv_finish_bwd_main_kernel<<<(unsigned)((warps + kWarps - 1) / kWarps), kThreads, 0, st>>>(p);
  PB_LAUNCH_CHECK("wkv_finish_bwd_main_kernel");
  reduce_tiles_kernel<<<(unsigned)((3 * C + 31) / 32), kThreads, 0, st>>>(partial, partial, tiles, 3 * C);
  PB_LAUNCH_CHECK("reduce_tiles_kernel");
  PB_CUDA_TRY(cudaMemcpyAsync(d_gn_scale, partial, (size_t)C * 4, cudaMemcpyDeviceToDevice, st));
  PB_CUDA_TRY(cudaMemcpyAsync(d_gn_bias, partial + C, (size_t)C * 4, cudaMemcpyDeviceToDevice, st));
  PB_CUDA_TRY(cudaMemcpyAsync(d_bonus_mult, partial + 2 * C, (size_t)C * 4, cudaMemcpyDeviceToDevice, st));
  return PB_OK;
}
