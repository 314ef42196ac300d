// The training loss of the reference, compute_loss (pratchya/_nnx_impl/_utils.py:7-13): softmax cross entropy against
// one-hot labels smoothed by alpha (optax.smooth_labels), mean over the positions that count.  Per row of logits z with
// target t:   loss_row = lse(z) - (1 - alpha) * z_t - alpha * mean_j(z_j)
// (the cross entropy against (1 - alpha) * onehot + alpha / V, written out), and its cotangent
//             dz_j = g_row * (exp(z_j - lse) - (1 - alpha) * [j == t] - alpha / V).
// As framework operations this is a log-softmax, a gather, a mean and their backward passes over an array of
// [tokens, vocabulary] f32 (8.6 GB at 32768 x 65536): six passes and three arrays of that size.  Here the forward kernel
// reads the logits once from HBM (one CTA per row; the second read of the row, for the sum of exponentials, comes from
// L2) and the backward kernel reads them once more and writes dz: HBM-bound, 4 + 8 bytes per logit.
#include "common.cuh"

namespace pb {
namespace {

constexpr int kLossThreads = 256;

__device__ __forceinline__ float block_reduce(float v, bool take_max, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = take_max ? fmaxf(v, other) : v + other;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
  for (int w = 1; w < kLossThreads / 32; ++w) r = take_max ? fmaxf(r, red[w]) : r + red[w];
  __syncthreads();
  return r;
}

// row_loss[r] = weight[r] * loss_row, lse[r] kept for the backward pass.  One CTA per row: the row's maximum and sum first,
// then the sum of exp(z - max) on a second read that comes from L2 (a row of 65536 logits is 256 KB).
__global__ void __launch_bounds__(kLossThreads) smoothed_xent_fwd_kernel(const float* logits, const int64_t* target, const float* weight,
                                                                        float* row_loss, float* lse, int64_t vocab, float alpha) {
  __shared__ float red[kLossThreads / 32];
  const int64_t row = blockIdx.x;
  const float* z = logits + row * vocab;
  float m = -INFINITY, zs = 0.0f;
  for (int64_t j = (int64_t)threadIdx.x * 4; j < vocab; j += kLossThreads * 4) {
    const float4 v = *reinterpret_cast<const float4*>(z + j);
    m = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    zs += (v.x + v.y) + (v.z + v.w);
  }
  m = block_reduce(m, true, red);
  zs = block_reduce(zs, false, red);
  float s = 0.0f;
  for (int64_t j = (int64_t)threadIdx.x * 4; j < vocab; j += kLossThreads * 4) {
    const float4 v = *reinterpret_cast<const float4*>(z + j);
    s += (expf(v.x - m) + expf(v.y - m)) + (expf(v.z - m) + expf(v.w - m));
  }
  s = block_reduce(s, false, red);
  if (threadIdx.x == 0) {
    const float l = m + logf(s);
    lse[row] = l;
    row_loss[row] = weight[row] * (l - (1.0f - alpha) * z[target[row]] - alpha * (zs / (float)vocab));
  }
}

// dz[r][j] = g[r] * (exp(z - lse) - (1 - alpha) * [j == t] - alpha / V), g[r] = upstream * weight[r] / denominator
__global__ void __launch_bounds__(kLossThreads) smoothed_xent_bwd_kernel(const float* logits, const int64_t* target, const float* weight,
                                                                        const float* lse, const float* upstream, float inv_denominator,
                                                                        float* dlogits, int64_t vocab, float alpha) {
  const int64_t row = blockIdx.x;
  const float* z = logits + row * vocab;
  float* dz = dlogits + row * vocab;
  const float g = upstream[0] * weight[row] * inv_denominator, l = lse[row];
  const int64_t t = target[row];
  const float smooth = alpha / (float)vocab;
  for (int64_t j = (int64_t)threadIdx.x * 4; j < vocab; j += kLossThreads * 4) {
    const float4 v = *reinterpret_cast<const float4*>(z + j);
    float4 d = make_float4(expf(v.x - l) - smooth, expf(v.y - l) - smooth, expf(v.z - l) - smooth, expf(v.w - l) - smooth);
    if (t >= j && t < j + 4) {
      const float hit = 1.0f - alpha;
      if (t == j) d.x -= hit; else if (t == j + 1) d.y -= hit; else if (t == j + 2) d.z -= hit; else d.w -= hit;
    }
    *reinterpret_cast<float4*>(dz + j) = make_float4(g * d.x, g * d.y, g * d.z, g * d.w);
  }
}

}  // namespace
}  // namespace pb

using namespace pb;

extern "C" int pb_smoothed_xent(const float* logits, const int64_t* target, const float* weight, int64_t rows, int64_t vocab, float alpha,
                                float* row_loss, float* lse, void* stream) {
  if (!logits || !target || !weight || !row_loss || !lse) return fail(PB_ERR_NULL_POINTER, "pb_smoothed_xent: null argument");
  if (rows <= 0 || vocab <= 0 || vocab % 4 != 0 || rows > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "pb_smoothed_xent: rows=%lld vocab=%lld (vocab must be a multiple of 4)", (long long)rows, (long long)vocab);
  if (reinterpret_cast<uintptr_t>(logits) & 15) return fail(PB_ERR_MISALIGNED, "pb_smoothed_xent: logits must be 16-byte aligned");
  smoothed_xent_fwd_kernel<<<(unsigned)rows, kLossThreads, 0, static_cast<cudaStream_t>(stream)>>>(logits, target, weight, row_loss, lse, vocab, alpha);
  PB_LAUNCH_CHECK("smoothed_xent_fwd_kernel");
  return PB_OK;
}

extern "C" int pb_smoothed_xent_bwd(const float* logits, const int64_t* target, const float* weight, const float* lse, const float* upstream,
                                    float denominator, int64_t rows, int64_t vocab, float alpha, float* dlogits, void* stream) {
  if (!logits || !target || !weight || !lse || !upstream || !dlogits) return fail(PB_ERR_NULL_POINTER, "pb_smoothed_xent_bwd: null argument");
  if (rows <= 0 || vocab <= 0 || vocab % 4 != 0 || rows > 0x7fffffffll || !(denominator > 0.0f))
    return fail(PB_ERR_BAD_SHAPE, "pb_smoothed_xent_bwd: rows=%lld vocab=%lld denominator=%g", (long long)rows, (long long)vocab, (double)denominator);
  if ((reinterpret_cast<uintptr_t>(logits) & 15) || (reinterpret_cast<uintptr_t>(dlogits) & 15))
    return fail(PB_ERR_MISALIGNED, "pb_smoothed_xent_bwd: logits and dlogits must be 16-byte aligned");
  smoothed_xent_bwd_kernel<<<(unsigned)rows, kLossThreads, 0, static_cast<cudaStream_t>(stream)>>>(logits, target, weight, lse, upstream,
                                                                                                1.0f / denominator, dlogits, vocab, alpha);
  PB_LAUNCH_CHECK("smoothed_xent_bwd_kernel");
  return PB_OK;
}
