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
// One CTA of 64 threads per (b, n), H = 64: thread i keeps row i of S (64 floats, as 32 float2) in
// registers for the whole sequence, so both dot products run inside a thread (packed f32x2 FMAs, four
// independent partial sums) and need no shuffle, and every shared-memory read of an input vector is a
// 16-byte broadcast (all lanes read the same address: one pass, where distinct 16-byte reads take four).
// A first form with four threads per row was bound by exactly that shared-memory traffic.  The six
// input vectors of a timestep (1.5 KB) are brought into a ring of shared-memory buffers by cp.async
// eight steps ahead, two timesteps per block-wide barrier; a * kap is formed once per step by the
// block (one element per thread).  The only serial dependence is S.
// HBM traffic is the algorithmic minimum: every input read once (6 x 4 B per channel and step), y
// written once (4 B), the state read and written once per sequence.
#include "common.cuh"

namespace pb {
namespace {

constexpr int kH = 64;            // head size
constexpr int kPairs = 4;         // ring depth in pairs of timesteps: eight timesteps of input in flight
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

// One timestep for row i of S.  `buf` holds the step's decay, iclr, removal_k, replacement_k, v, r; `bk` = iclr * removal_k.
__device__ __forceinline__ float wkv_step(float2 (&S)[32], const float (*buf)[kH], const float* bk, int i) {
  // sa_i = sum_j S[i][j] * kap_j, four partial sums
  float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float4 k4 = *reinterpret_cast<const float4*>(&buf[2][4 * j]);
    acc[(2 * j) & 3] = __ffma2_rn(S[2 * j], make_float2(k4.x, k4.y), acc[(2 * j) & 3]);
    acc[(2 * j + 1) & 3] = __ffma2_rn(S[2 * j + 1], make_float2(k4.z, k4.w), acc[(2 * j + 1) & 3]);
  }
  const float sa = ((acc[0].x + acc[0].y) + (acc[1].x + acc[1].y)) + ((acc[2].x + acc[2].y) + (acc[3].x + acc[3].y));
  const float vi = buf[4][i];
  const float2 nsa2 = make_float2(-sa, -sa), vi2 = make_float2(vi, vi);
  float2 y[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float4 w4 = *reinterpret_cast<const float4*>(&buf[0][4 * j]);
    const float4 b4 = *reinterpret_cast<const float4*>(&bk[4 * j]);
    const float4 kt4 = *reinterpret_cast<const float4*>(&buf[3][4 * j]);
    const float4 r4 = *reinterpret_cast<const float4*>(&buf[5][4 * j]);
    float2 s0 = __ffma2_rn(nsa2, make_float2(b4.x, b4.y), __fmul2_rn(S[2 * j], make_float2(w4.x, w4.y)));
    float2 s1 = __ffma2_rn(nsa2, make_float2(b4.z, b4.w), __fmul2_rn(S[2 * j + 1], make_float2(w4.z, w4.w)));
    s0 = __ffma2_rn(vi2, make_float2(kt4.x, kt4.y), s0);
    s1 = __ffma2_rn(vi2, make_float2(kt4.z, kt4.w), s1);
    S[2 * j] = s0; S[2 * j + 1] = s1;
    y[(2 * j) & 3] = __ffma2_rn(s0, make_float2(r4.x, r4.y), y[(2 * j) & 3]);
    y[(2 * j + 1) & 3] = __ffma2_rn(s1, make_float2(r4.z, r4.w), y[(2 * j + 1) & 3]);
  }
  return ((y[0].x + y[0].y) + (y[1].x + y[1].y)) + ((y[2].x + y[2].y) + (y[3].x + y[3].y));
}

constexpr int kThreads = kH;      // one thread per state row

__global__ void __launch_bounds__(kThreads)
wkv7_forward_kernel(const __grid_constant__ WkvParams p) {
  __shared__ __align__(16) float ring[kPairs][2][kVecs][kH];      // [pair slot][step of the pair][vector][channel]
  __shared__ __align__(16) float bk[2][kH];                       // iclr * removal_k of the two steps of the current pair
  const int n = blockIdx.x % p.N, b = blockIdx.x / p.N;
  const int C = p.N * kH;
  const int i = threadIdx.x;
  const size_t head_base = (size_t)b * p.T * C + (size_t)n * kH;      // element (b, t = 0, channel n*H)

  // a pair of timesteps is 2 x 6 vectors x 16 chunks of 16 bytes = 192 chunks: three per thread
  auto issue = [&](int pair) {
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      const int id = c * kThreads + i;                         // 0 .. 191
      const int step = id / (kVecs * (kH / 4)), vec = (id / (kH / 4)) % kVecs, chunk = id % (kH / 4);
      const int t = 2 * pair + step;
      if (t < p.T)
        cp_async16((uint32_t)__cvta_generic_to_shared(&ring[pair % kPairs][step][vec][chunk * 4]),
                   p.in[vec] + head_base + (size_t)t * C + chunk * 4);
    }
    cp_async_commit();            // every thread commits a (possibly empty) group per pair: the counts stay aligned
  };

  float2 S[32];                   // row i of this head's state
  const size_t srow = (((size_t)b * p.N + n) * kH + i) * kH;
  if (p.state_in) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.state_in + srow) + j);
      S[2 * j] = make_float2(s4.x, s4.y); S[2 * j + 1] = make_float2(s4.z, s4.w);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) S[j] = make_float2(0.0f, 0.0f);
  }

  const int n_pairs = (p.T + 1) >> 1;
  for (int pr = 0; pr < kPairs - 1; ++pr) issue(pr);
  float* yp = p.y + head_base + i;
  for (int pr = 0; pr < n_pairs; ++pr) {
    cp_async_wait<kPairs - 2>();      // this thread's copies for this pair have landed
    __syncthreads();                  // ... and everyone's; every thread is also done with the previous pair (ring slot and bk)
    issue(pr + kPairs - 1);           // into the slot the previous pair used
    const float (*step0)[kH] = ring[pr % kPairs][0];
    const float (*step1)[kH] = ring[pr % kPairs][1];
    bk[0][i] = step0[1][i] * step0[2][i];
    bk[1][i] = step1[1][i] * step1[2][i];
    __syncthreads();
    const int t = 2 * pr;
    yp[(size_t)t * C] = wkv_step(S, step0, bk[0], i);
    if (t + 1 < p.T) yp[(size_t)(t + 1) * C] = wkv_step(S, step1, bk[1], i);
  }
  cp_async_wait<0>();
  if (p.state_out) {
#pragma unroll
    for (int j = 0; j < 16; ++j)
      reinterpret_cast<float4*>(p.state_out + srow)[j] = make_float4(S[2 * j].x, S[2 * j].y, S[2 * j + 1].x, S[2 * j + 1].y);
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
  wkv7_forward_kernel<<<(unsigned)(batch * heads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PB_LAUNCH_CHECK("wkv7_forward_kernel");
  return PB_OK;
}
