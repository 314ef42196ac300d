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
constexpr int kCk = 16;           // spacing of the state checkpoints the backward pass restarts from

struct WkvParams {
  const float* in[kVecs];
  const float* state_in;          // [B, N, H, H] or null (zeros)
  float* y;                       // [B, T, C]
  float* state_out;               // [B, N, H, H] or null
  float* ckpt;                    // [B, N, ceil(T / kCk), H, H] or null: the state before timesteps 0, kCk, 2*kCk, ...
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
    if (p.ckpt && (t & (kCk - 1)) == 0) {
      float4* dst = reinterpret_cast<float4*>(p.ckpt + ((((size_t)b * p.N + n) * ((p.T + kCk - 1) / kCk) + t / kCk) * kH + i) * kH);
#pragma unroll
      for (int j = 0; j < 16; ++j) dst[j] = make_float4(S[2 * j].x, S[2 * j].y, S[2 * j + 1].x, S[2 * j + 1].y);
    }
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

// ---- backward of the scan ------------------------------------------------------------------------------------
// With G_t = dS_t + dy_t r_t^T the gradient of the loss with respect to S_t (dS_t arriving from timestep t+1):
//     dr_t   = S_t^T dy_t                    dv_t  = G_t kt_t                 dkt_t = G_t^T v_t
//     dsa_t  = -G_t b_t   (b = a * kap)      db_t  = -G_t^T sa_t              dw_t  = sum_i G_t[i][:] * S_{t-1}[i][:]
//     dkap_t = S_{t-1}^T dsa_t + db_t * a_t  da_t  = db_t * kap_t             dS_{t-1} = G_t diag(w_t) + dsa_t kap_t^T
// Half of these are sums along a row of the state, half along a column, so a CTA of 128 threads keeps two
// copies of S_{t-1} and of dS in registers: threads 0..63 one row each, threads 64..127 one column each; the
// row threads publish sa and dsa (64 floats each) through shared memory, two block barriers per timestep.
// S_{t-1} is not stored by the forward pass for every t: it writes a checkpoint every kCk timesteps, and the
// backward pass recomputes the kCk states of a chunk from its checkpoint into a per-head scratch buffer
// (256 KB per head: it stays in L2), then walks the chunk backwards reading them from there.
struct WkvBwdParams {
  const float* in[kVecs];
  const float* dy;                // [B, T, C]
  const float* ckpt;              // [B, N, ceil(T / kCk), H, H]
  const float* dstate_out;        // [B, N, H, H] or null: gradient with respect to the final state
  float* din[kVecs];              // gradients of the six inputs, [B, T, C] each
  float* dstate_in;               // [B, N, H, H] or null: gradient with respect to the initial state
  float* scratch;                 // [B * N, kCk, H, H]
  int T, N;
};

__global__ void __launch_bounds__(2 * kH, 1)
wkv7_backward_kernel(const __grid_constant__ WkvBwdParams p) {
  __shared__ __align__(16) float vec[kCk][kVecs + 1][kH];       // the chunk's inputs and dy
  __shared__ __align__(16) float sa_s[kH], dsa_s[kH];
  const int n = blockIdx.x % p.N, b = blockIdx.x / p.N;
  const int C = p.N * kH;
  const int tid = threadIdx.x;
  const bool row_thread = tid < kH;
  const int idx = row_thread ? tid : tid - kH;                  // the row i, or the column j, this thread owns
  const size_t head_base = (size_t)b * p.T * C + (size_t)n * kH;
  const size_t head = (size_t)b * p.N + n;
  const int n_ck = (p.T + kCk - 1) / kCk;
  float* scratch = p.scratch + head * (size_t)kCk * kH * kH;

  float dS[kH];                   // row idx (row threads) or column idx (column threads) of dS
  if (p.dstate_out) {
#pragma unroll
    for (int e = 0; e < kH; ++e)
      dS[e] = row_thread ? p.dstate_out[(head * kH + idx) * kH + e] : p.dstate_out[(head * kH + e) * kH + idx];
  } else {
#pragma unroll
    for (int e = 0; e < kH; ++e) dS[e] = 0.0f;
  }

  for (int ck = n_ck - 1; ck >= 0; --ck) {
    const int t0 = ck * kCk, steps = min(kCk, p.T - t0);
    __syncthreads();              // everyone is done with the previous chunk's vectors and scratch
    for (int e = tid; e < steps * (kVecs + 1) * (kH / 4); e += 2 * kH) {
      const int s = e / ((kVecs + 1) * (kH / 4)), rem = e % ((kVecs + 1) * (kH / 4)), v = rem / (kH / 4), c4 = rem % (kH / 4);
      const float* src = (v < kVecs ? p.in[v] : p.dy) + head_base + (size_t)(t0 + s) * C + c4 * 4;
      *reinterpret_cast<float4*>(&vec[s][v][c4 * 4]) = __ldg(reinterpret_cast<const float4*>(src));
    }
    __syncthreads();
    if (row_thread) {
      // recompute the chunk's states forward from its checkpoint; the state BEFORE timestep t0 + s goes to scratch[s]
      float S[kH];
      const float4* c4p = reinterpret_cast<const float4*>(p.ckpt + ((head * n_ck + ck) * kH + idx) * kH);
#pragma unroll
      for (int j = 0; j < 16; ++j) { const float4 q = __ldg(c4p + j); S[4 * j] = q.x; S[4 * j + 1] = q.y; S[4 * j + 2] = q.z; S[4 * j + 3] = q.w; }
      for (int s = 0; s < steps; ++s) {
        float4* dst = reinterpret_cast<float4*>(scratch + ((size_t)s * kH + idx) * kH);
#pragma unroll
        for (int j = 0; j < 16; ++j) dst[j] = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
        if (s + 1 < steps) {      // the state after the chunk's last timestep is not needed
          float sa0 = 0.f, sa1 = 0.f, sa2 = 0.f, sa3 = 0.f;
#pragma unroll
          for (int j = 0; j < kH; j += 4) {
            sa0 = fmaf(S[j], vec[s][2][j], sa0); sa1 = fmaf(S[j + 1], vec[s][2][j + 1], sa1);
            sa2 = fmaf(S[j + 2], vec[s][2][j + 2], sa2); sa3 = fmaf(S[j + 3], vec[s][2][j + 3], sa3);
          }
          const float sa = (sa0 + sa1) + (sa2 + sa3), vi = vec[s][4][idx];
#pragma unroll
          for (int j = 0; j < kH; ++j)
            S[j] = fmaf(vi, vec[s][3][j], fmaf(-sa, vec[s][1][j] * vec[s][2][j], S[j] * vec[s][0][j]));
        }
      }
    }
    __syncthreads();              // the chunk's states are in scratch (written and read by this block only)

    for (int s = steps - 1; s >= 0; --s) {
      const size_t out = head_base + (size_t)(t0 + s) * C + idx;
      const float* w = vec[s][0]; const float* a = vec[s][1]; const float* kap = vec[s][2];
      const float* kt = vec[s][3]; const float* v = vec[s][4]; const float* r = vec[s][5]; const float* dy = vec[s][6];
      float Sp[kH];               // row / column idx of S_{t-1}
      if (row_thread) {
        const float4* src = reinterpret_cast<const float4*>(scratch + ((size_t)s * kH + idx) * kH);
#pragma unroll
        for (int j = 0; j < 16; ++j) { const float4 q = src[j]; Sp[4 * j] = q.x; Sp[4 * j + 1] = q.y; Sp[4 * j + 2] = q.z; Sp[4 * j + 3] = q.w; }
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
        for (int j = 0; j < kH; j += 4) {
          s0 = fmaf(Sp[j], kap[j], s0); s1 = fmaf(Sp[j + 1], kap[j + 1], s1);
          s2 = fmaf(Sp[j + 2], kap[j + 2], s2); s3 = fmaf(Sp[j + 3], kap[j + 3], s3);
        }
        sa_s[idx] = (s0 + s1) + (s2 + s3);
      } else {
#pragma unroll
        for (int i = 0; i < kH; ++i) Sp[i] = scratch[((size_t)s * kH + i) * kH + idx];
      }
      __syncthreads();            // sa is published
      float db_keep = 0.0f;
      if (row_thread) {
        const float dyi = dy[idx];
        float dv0 = 0.f, dv1 = 0.f, ds0 = 0.f, ds1 = 0.f;
#pragma unroll
        for (int j = 0; j < kH; j += 2) {
          const float g0 = fmaf(dyi, r[j], dS[j]), g1 = fmaf(dyi, r[j + 1], dS[j + 1]);
          dS[j] = g0; dS[j + 1] = g1;
          dv0 = fmaf(g0, kt[j], dv0); dv1 = fmaf(g1, kt[j + 1], dv1);
          ds0 = fmaf(g0, a[j] * kap[j], ds0); ds1 = fmaf(g1, a[j + 1] * kap[j + 1], ds1);
        }
        const float dsa = -(ds0 + ds1);
        dsa_s[idx] = dsa;
        p.din[4][out] = dv0 + dv1;
#pragma unroll
        for (int j = 0; j < kH; ++j) dS[j] = fmaf(dsa, kap[j], dS[j] * w[j]);
      } else {
        const float wj = w[idx], bj = a[idx] * kap[idx], ktj = kt[idx], rj = r[idx];
        float dr0 = 0.f, dr1 = 0.f, dkt0 = 0.f, dkt1 = 0.f, db0 = 0.f, db1 = 0.f, dw0 = 0.f, dw1 = 0.f;
#pragma unroll
        for (int i = 0; i < kH; i += 2) {
          const float st0 = fmaf(v[i], ktj, fmaf(-sa_s[i], bj, Sp[i] * wj));
          const float st1 = fmaf(v[i + 1], ktj, fmaf(-sa_s[i + 1], bj, Sp[i + 1] * wj));
          const float g0 = fmaf(dy[i], rj, dS[i]), g1 = fmaf(dy[i + 1], rj, dS[i + 1]);
          dS[i] = g0; dS[i + 1] = g1;
          dr0 = fmaf(st0, dy[i], dr0); dr1 = fmaf(st1, dy[i + 1], dr1);
          dkt0 = fmaf(g0, v[i], dkt0); dkt1 = fmaf(g1, v[i + 1], dkt1);
          db0 = fmaf(g0, sa_s[i], db0); db1 = fmaf(g1, sa_s[i + 1], db1);
          dw0 = fmaf(g0, Sp[i], dw0); dw1 = fmaf(g1, Sp[i + 1], dw1);
        }
        db_keep = -(db0 + db1);
        p.din[5][out] = dr0 + dr1;
        p.din[3][out] = dkt0 + dkt1;
        p.din[0][out] = dw0 + dw1;
      }
      __syncthreads();            // dsa is published
      if (!row_thread) {
        const float db = db_keep, wj = w[idx];
        const float kapj = kap[idx];
        float dk0 = 0.f, dk1 = 0.f;
#pragma unroll
        for (int i = 0; i < kH; i += 2) {
          dk0 = fmaf(Sp[i], dsa_s[i], dk0); dk1 = fmaf(Sp[i + 1], dsa_s[i + 1], dk1);
          dS[i] = fmaf(dsa_s[i], kapj, dS[i] * wj);
          dS[i + 1] = fmaf(dsa_s[i + 1], kapj, dS[i + 1] * wj);
        }
        p.din[2][out] = (dk0 + dk1) + db * a[idx];
        p.din[1][out] = db * kapj;
      }
      __syncthreads();            // sa_s / dsa_s may be overwritten by the next timestep
    }
  }
  if (p.dstate_in && row_thread) {
#pragma unroll
    for (int j = 0; j < 16; ++j)
      reinterpret_cast<float4*>(p.dstate_in + (head * kH + idx) * kH)[j] = make_float4(dS[4 * j], dS[4 * j + 1], dS[4 * j + 2], dS[4 * j + 3]);
  }
}

}  // namespace
}  // namespace pb

using namespace pb;

extern "C" int pb_wkv7_forward(const float* decay, const float* iclr, const float* removal_k, const float* replacement_k,
                               const float* v, const float* r, const float* state_in,
                               int64_t batch, int64_t steps, int64_t heads, int head_dim,
                               float* y, float* state_out, float* checkpoints, void* stream) {
  if (!decay || !iclr || !removal_k || !replacement_k || !v || !r || !y)
    return fail(PB_ERR_NULL_POINTER, "pb_wkv7_forward: the six inputs and y must be non-null");
  if (head_dim != kH) return fail(PB_ERR_UNSUPPORTED, "pb_wkv7_forward: head size %d (this kernel is built for %d)", head_dim, kH);
  if (batch <= 0 || steps <= 0 || heads <= 0 || batch * heads > 0x7fffffffll || steps > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "pb_wkv7_forward: batch=%lld steps=%lld heads=%lld", (long long)batch, (long long)steps, (long long)heads);
  const void* ptrs[] = {decay, iclr, removal_k, replacement_k, v, r, state_in, state_out, checkpoints};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(PB_ERR_MISALIGNED, "pb_wkv7_forward: every array must be 16-byte aligned");
  WkvParams p{{decay, iclr, removal_k, replacement_k, v, r}, state_in, y, state_out, checkpoints, (int)steps, (int)heads};
  wkv7_forward_kernel<<<(unsigned)(batch * heads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PB_LAUNCH_CHECK("wkv7_forward_kernel");
  return PB_OK;
}

extern "C" size_t pb_wkv7_checkpoint_floats(int64_t batch, int64_t steps, int64_t heads, int head_dim) {
  if (batch <= 0 || steps <= 0 || heads <= 0 || head_dim != kH) return 0;
  return (size_t)batch * heads * ((steps + kCk - 1) / kCk) * kH * kH;
}

extern "C" size_t pb_wkv7_backward_workspace_size(int64_t batch, int64_t heads, int head_dim) {
  if (batch <= 0 || heads <= 0 || head_dim != kH) return 0;
  return (size_t)batch * heads * kCk * kH * kH * sizeof(float);
}

extern "C" int pb_wkv7_backward(const float* decay, const float* iclr, const float* removal_k, const float* replacement_k,
                                const float* v, const float* r, const float* checkpoints, const float* dy, const float* dstate_out,
                                int64_t batch, int64_t steps, int64_t heads, int head_dim,
                                float* d_decay, float* d_iclr, float* d_removal_k, float* d_replacement_k, float* d_v, float* d_r,
                                float* dstate_in, void* workspace, size_t workspace_bytes, void* stream) {
  if (!decay || !iclr || !removal_k || !replacement_k || !v || !r || !checkpoints || !dy || !d_decay || !d_iclr || !d_removal_k ||
      !d_replacement_k || !d_v || !d_r)
    return fail(PB_ERR_NULL_POINTER, "pb_wkv7_backward: the six inputs, the checkpoints, dy and the six gradients must be non-null");
  if (head_dim != kH) return fail(PB_ERR_UNSUPPORTED, "pb_wkv7_backward: head size %d (this kernel is built for %d)", head_dim, kH);
  if (batch <= 0 || steps <= 0 || heads <= 0 || batch * heads > 0x7fffffffll || steps > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "pb_wkv7_backward: batch=%lld steps=%lld heads=%lld", (long long)batch, (long long)steps, (long long)heads);
  const size_t need = pb_wkv7_backward_workspace_size(batch, heads, head_dim);
  if (!workspace || workspace_bytes < need)
    return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_wkv7_backward: needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  const void* ptrs[] = {decay, iclr, removal_k, replacement_k, v, r, checkpoints, dy, dstate_out, dstate_in, workspace};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(PB_ERR_MISALIGNED, "pb_wkv7_backward: every array must be 16-byte aligned");
  WkvBwdParams p{{decay, iclr, removal_k, replacement_k, v, r}, dy, checkpoints, dstate_out,
                 {d_decay, d_iclr, d_removal_k, d_replacement_k, d_v, d_r}, dstate_in, static_cast<float*>(workspace), (int)steps, (int)heads};
  wkv7_backward_kernel<<<(unsigned)(batch * heads), 2 * kH, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PB_LAUNCH_CHECK("wkv7_backward_kernel");
  return PB_OK;
}
