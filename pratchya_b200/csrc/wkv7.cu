// WKV-7 state scan of the modified RWKV-7 TimeMix block (sm_100a): the per-timestep recurrence of
// pratchya/_nnx_impl/_module.py:187-207 as one kernel instead of a scan of T small matmuls.
//
// Per (batch b, head n) the state S is an H x H fp32 matrix (rows: value channel i, columns: key
// channel j).  With, at timestep t, w = decay, a = iclr, kap = removal_k, kt = replacement_k, v and r
// (each a vector of H channels of that head):
//     sa_i  = sum_j S[i][j] * kap_j                         (wkv_state @ removal_k_t, :197)
//     S[i][j] = S[i][j] * w_j - sa_i * (a_j * kap_j)        (:197)
//     S[i][j] += v_i * kt_j                                 (:198)
//     y_i   = sum_j S[i][j] * r_j                           (:199)
// All arithmetic is fp32, as in the reference (its inputs are cast to f32 before the scan).
//
// One CTA of 256 threads per (b, n), H = 64: thread (i, q) keeps columns 16q .. 16q+15 of row i in
// registers for the whole sequence; the two dot products are 16 FMAs per thread and two shuffles
// across the four threads of a row.  The six input vectors of a timestep (1.5 KB) are brought into a
// ring of shared-memory buffers by cp.async several steps ahead: the only serial dependence is S.
// HBM traffic is the algorithmic minimum: every input read once (6 x 4 B per channel and step), y
// written once (4 B), the state read and written once per sequence.
#include "common.cuh"

namespace pb {
namespace {

constexpr int kH = 64;            // head size
constexpr int kDepth = 8;         // timesteps of input in flight
constexpr int kVecs = 6;          // decay, iclr, removal_k, replacement_k, v, r

struct WkvParams {
  const float* in[kVecs];
  const float* state_in;          // [B, N, H, H] or null (zeros)
  float* y;                       // [B, T, C]
  float* state_out;               // [B, N, H, H] or null
  int T, N;                       // timesteps, heads
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(256)
wkv7_forward_kernel(const __grid_constant__ WkvParams p) {
  __shared__ __align__(16) float ring[kDepth][kVecs][kH];
  const int n = blockIdx.x % p.N, b = blockIdx.x / p.N;
  const int C = p.N * kH;
  const int tid = threadIdx.x, i = tid >> 2, q = tid & 3;
  const size_t head_base = (size_t)b * p.T * C + (size_t)n * kH;      // element (b, t = 0, channel n*H)

  // threads 0..95 each own one 16-byte chunk of one input vector
  const bool loader = tid < kVecs * (kH / 4);
  const int lvec = tid / (kH / 4), lchunk = tid % (kH / 4);
  const float* lsrc = loader ? p.in[lvec] + head_base + lchunk * 4 : nullptr;
  const uint32_t ldst = (uint32_t)__cvta_generic_to_shared(&ring[0][loader ? lvec : 0][loader ? lchunk * 4 : 0]);
  auto issue = [&](int t) {
    if (loader && t < p.T) cp_async16(ldst + (uint32_t)(t % kDepth) * (kVecs * kH * 4), lsrc + (size_t)t * C);
    cp_async_commit();            // every thread commits a (possibly empty) group per step: the counts stay aligned
  };

  float S[16];
  const size_t srow = (((size_t)b * p.N + n) * kH + i) * kH + q * 16;
  if (p.state_in) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.state_in + srow) + j);
      S[4 * j] = s4.x; S[4 * j + 1] = s4.y; S[4 * j + 2] = s4.z; S[4 * j + 3] = s4.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) S[j] = 0.0f;
  }

  for (int t = 0; t < kDepth - 1; ++t) issue(t);
  float* yp = p.y + head_base + i;
  for (int t = 0; t < p.T; ++t) {
    cp_async_wait<kDepth - 2>();      // this thread's copies for step t have landed
    __syncthreads();                  // ... and everyone's; every thread is also done with step t-1
    issue(t + kDepth - 1);            // into the buffer step t-1 used
    const float(*buf)[kH] = ring[t % kDepth];
    float w[16], kap[16], bk[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 w4 = *reinterpret_cast<const float4*>(&buf[0][q * 16 + 4 * j]);
      const float4 a4 = *reinterpret_cast<const float4*>(&buf[1][q * 16 + 4 * j]);
      const float4 k4 = *reinterpret_cast<const float4*>(&buf[2][q * 16 + 4 * j]);
      w[4 * j] = w4.x; w[4 * j + 1] = w4.y; w[4 * j + 2] = w4.z; w[4 * j + 3] = w4.w;
      kap[4 * j] = k4.x; kap[4 * j + 1] = k4.y; kap[4 * j + 2] = k4.z; kap[4 * j + 3] = k4.w;
      bk[4 * j] = a4.x * k4.x; bk[4 * j + 1] = a4.y * k4.y; bk[4 * j + 2] = a4.z * k4.z; bk[4 * j + 3] = a4.w * k4.w;
    }
    float sa0 = 0.0f, sa1 = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j += 2) { sa0 = fmaf(S[j], kap[j], sa0); sa1 = fmaf(S[j + 1], kap[j + 1], sa1); }
    float sa = sa0 + sa1;
    sa += __shfl_xor_sync(0xffffffffu, sa, 1);
    sa += __shfl_xor_sync(0xffffffffu, sa, 2);
    const float vi = buf[4][i];
    float y0 = 0.0f, y1 = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 kt4 = *reinterpret_cast<const float4*>(&buf[3][q * 16 + 4 * j]);
      const float4 r4 = *reinterpret_cast<const float4*>(&buf[5][q * 16 + 4 * j]);
      const float kt[4] = {kt4.x, kt4.y, kt4.z, kt4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = 4 * j + e;
        float s = fmaf(-sa, bk[c], S[c] * w[c]);
        s = fmaf(vi, kt[e], s);
        S[c] = s;
        if (e & 1) y1 = fmaf(s, rr[e], y1); else y0 = fmaf(s, rr[e], y0);
      }
    }
    float y = y0 + y1;
    y += __shfl_xor_sync(0xffffffffu, y, 1);
    y += __shfl_xor_sync(0xffffffffu, y, 2);
    if (q == 0) yp[(size_t)t * C] = y;
  }
  cp_async_wait<0>();
  if (p.state_out) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      reinterpret_cast<float4*>(p.state_out + srow)[j] = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
  }
}

}  // namespace
}  // namespace pb

using namespace pb;

extern "C" int pb_wkv7_forward(const float* decay, const float* iclr, const float* removal_k, const float* replacement_k,
                               const float* v, const float* r, const float* state_in,
                               int64_t batch, int64_t steps, int64_t heads, int head_dim,
                               float* y, float* state_out, void* stream) {
  if (!decay || !iclr || !removal_k || !replacement_k || !v || !r || !y)
    return fail(PB_ERR_NULL_POINTER, "pb_wkv7_forward: the six inputs and y must be non-null");
  if (head_dim != kH) return fail(PB_ERR_UNSUPPORTED, "pb_wkv7_forward: head size %d (this kernel is built for %d)", head_dim, kH);
  if (batch <= 0 || steps <= 0 || heads <= 0 || batch * heads > 0x7fffffffll || steps > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "pb_wkv7_forward: batch=%lld steps=%lld heads=%lld", (long long)batch, (long long)steps, (long long)heads);
  const void* ptrs[] = {decay, iclr, removal_k, replacement_k, v, r, state_in, state_out};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(PB_ERR_MISALIGNED, "pb_wkv7_forward: every array must be 16-byte aligned");
  WkvParams p{{decay, iclr, removal_k, replacement_k, v, r}, state_in, y, state_out, (int)steps, (int)heads};
  wkv7_forward_kernel<<<(unsigned)(batch * heads), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PB_LAUNCH_CHECK("wkv7_forward_kernel");
  return PB_OK;
}
