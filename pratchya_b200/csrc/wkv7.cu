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
constexpr int kCk = 8;            // spacing of the state checkpoints the backward pass restarts from

struct WkvParams {
  const float* in[kVecs];
  const float* state_in;          // [B, N, H, H] or null (zeros)
  float* y;                       // [B, T, C]
  float* state_out;               // [B, N, H, H] or null
  float* ckpt;                    // [B, N, ceil(T / kCk), H, H] or null: the state before timesteps 0, kCk, 2*kCk, ...
  float* sa;                      // [B, T, C] or null: sa of every timestep (S before the step, times removal_k), for the backward pass
  int T, N;                       // timesteps, heads
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One timestep for row i of S.  `buf` holds the step's decay, iclr, removal_k, replacement_k, v, r; `bk` = iclr * removal_k.
__device__ __forceinline__ float wkv_step(float2 (&S)[32], const float (*buf)[kH], const float* bk, int i, float& sa_out) {
  // sa_i = sum_j S[i][j] * kap_j, four partial sums
  float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float4 k4 = *reinterpret_cast<const float4*>(&buf[2][4 * j]);
    acc[(2 * j) & 3] = __ffma2_rn(S[2 * j], make_float2(k4.x, k4.y), acc[(2 * j) & 3]);
    acc[(2 * j + 1) & 3] = __ffma2_rn(S[2 * j + 1], make_float2(k4.z, k4.w), acc[(2 * j + 1) & 3]);
  }
  const float sa = ((acc[0].x + acc[0].y) + (acc[1].x + acc[1].y)) + ((acc[2].x + acc[2].y) + (acc[3].x + acc[3].y));
  sa_out = sa;
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
    float sa0, sa1;
    yp[(size_t)t * C] = wkv_step(S, step0, bk[0], i, sa0);
    if (p.sa) p.sa[head_base + (size_t)t * C + i] = sa0;
    if (t + 1 < p.T) {
      yp[(size_t)(t + 1) * C] = wkv_step(S, step1, bk[1], i, sa1);
      if (p.sa) p.sa[head_base + (size_t)(t + 1) * C + i] = sa1;
    }
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
// Half of these are sums along a row of the state, half along a column, so a CTA keeps dS twice: 128 row
// threads (row i, one half of its columns each) and 128 column threads (column j, one half of its rows each).
// The halves of a row or column sit in different warps, so a warp still reads every input vector at one
// address per instruction (a broadcast), and the two partial sums meet in shared memory.
//
// S_{t-1} is needed for every t and is not stored by the forward pass, which writes a checkpoint every
// kCk = 8 timesteps and sa_t = S_{t-1} kap_t (64 floats) for every t.  With sa_t known the recurrence is
// element-wise, so per chunk the row threads recompute the states from the checkpoint without any sum: first
// the states before the chunk's last four timesteps into four shared-memory slots, those four timesteps run
// backwards, then the states before the first four into the same slots, and those run backwards.  A slot is
// H x H floats with the 16-byte groups of row i stored at group ^ (i & 15): the row threads' 16-byte row stores
// and the column threads' 4-byte column loads are both free of bank conflicts.
// One block barrier per timestep: before it the row threads publish the halves of dv and of -dsa, after it
// everyone forms dsa.  The column threads' five sums are published as halves too and added one timestep later
// (three buffers in rotation).  The chunk's eight vectors per timestep arrive by cp.async one chunk ahead, and
// the checkpoint the next recomputation starts from is loaded into the row threads' registers before the
// timesteps that precede it.
constexpr int kSub = 4;                  // timesteps whose states are kept at once
constexpr int kBwdThreads = 4 * kH;
constexpr int kBwdVecs = kVecs + 2;      // the six inputs, dy and sa

struct WkvBwdParams {
  const float* in[kVecs];
  const float* dy;                // [B, T, C]
  const float* sa;                // [B, T, C]: S_{t-1} kap_t, from the forward pass
  const float* ckpt;              // [B, N, ceil(T / kCk), H, H]
  const float* dstate_out;        // [B, N, H, H] or null: gradient with respect to the final state
  float* din[kVecs];              // gradients of the six inputs, [B, T, C] each
  float* dstate_in;               // [B, N, H, H] or null: gradient with respect to the initial state
  int T, N;
};

struct WkvBwdSmem {
  float slot[kSub][kH * kH];                // recomputed states, swizzled
  float vec[2][kCk][kBwdVecs][kH];          // the chunk's vectors, two chunks
  float bk[kCk][kH];                        // iclr * removal_k
  float ds_part[2][2][kH];                  // [parity of t][column half][row]: halves of sum_j G b
  float dv_part[2][2][kH];                  // ... of sum_j G kt
  float col_part[3][2][5][kH];              // [t mod 3][row half][dr, dkt, sum G sa, dw, S^T dsa][column]
};

__device__ __forceinline__ float sum4(const float2 a, const float2 b) { return (a.x + a.y) + (b.x + b.y); }

__global__ void __launch_bounds__(kBwdThreads, 2)
wkv7_backward_kernel(const __grid_constant__ WkvBwdParams p) {
  extern __shared__ __align__(16) unsigned char wkv_bwd_smem[];
  WkvBwdSmem& sm = *reinterpret_cast<WkvBwdSmem*>(wkv_bwd_smem);
  const int n = blockIdx.x % p.N, b = blockIdx.x / p.N;
  const int C = p.N * kH;
  const int tid = threadIdx.x;
  const bool row_thread = tid < 2 * kH;
  const int half = (tid >> 6) & 1;             // row threads: which 32 columns; column threads: which 32 rows
  const int idx = tid & (kH - 1);              // the row i, or the column j
  const int h0 = 32 * half;
  const size_t head_base = (size_t)b * p.T * C + (size_t)n * kH;
  const size_t head = (size_t)b * p.N + n;
  const int n_ck = (p.T + kCk - 1) / kCk;

  // element (h0 + e, idx) of a slot, for a column thread: (h0 + e) * kH + joff[e & 15]
  int joff[16];
#pragma unroll
  for (int c = 0; c < 16; ++c) joff[c] = ((((idx >> 2) ^ c) << 2) | (idx & 3));

  float2 dS[16];                  // row threads: dS[idx][h0 + 2e, +1]; column threads: dS[h0 + 2e, +1][idx]
  if (p.dstate_out) {
    if (row_thread) {
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(p.dstate_out + (head * kH + idx) * kH + h0) + g);
        dS[2 * g] = make_float2(q.x, q.y); dS[2 * g + 1] = make_float2(q.z, q.w);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 16; ++e)
        dS[e] = make_float2(__ldg(p.dstate_out + (head * kH + h0 + 2 * e) * kH + idx), __ldg(p.dstate_out + (head * kH + h0 + 2 * e + 1) * kH + idx));
    }
  } else {
#pragma unroll
    for (int e = 0; e < 16; ++e) dS[e] = make_float2(0.0f, 0.0f);
  }

  // the eight vectors of every timestep of chunk ck -> vec[ck & 1]; every thread commits one group per call
  auto issue_vec = [&](int ck) {
    if (ck >= 0) {
      const int t0 = ck * kCk, steps = min(kCk, p.T - t0);
      for (int e = tid; e < steps * kBwdVecs * (kH / 4); e += kBwdThreads) {
        const int s = e / (kBwdVecs * (kH / 4)), rem = e % (kBwdVecs * (kH / 4)), v = rem / (kH / 4), c4 = rem % (kH / 4);
        const float* src = (v < kVecs ? p.in[v] : (v == kVecs ? p.dy : p.sa)) + head_base + (size_t)(t0 + s) * C + c4 * 4;
        cp_async16((uint32_t)__cvta_generic_to_shared(&sm.vec[ck & 1][s][v][c4 * 4]), src);
      }
    }
    cp_async_commit();
  };

  // row threads: their half of the row of the state being recomputed (in flight from the checkpoint while
  // timesteps run backwards); column threads: their half of column idx of S_{t-1} within a timestep.
  float2 S[16];
  auto load_ckpt = [&](int ck) {
    const float4* c4p = reinterpret_cast<const float4*>(p.ckpt + ((head * n_ck + ck) * kH + idx) * kH + h0);
#pragma unroll
    for (int g = 0; g < 8; ++g) { const float4 q = __ldg(c4p + g); S[2 * g] = make_float2(q.x, q.y); S[2 * g + 1] = make_float2(q.z, q.w); }
  };
  auto store_slot = [&](float* slot) {
#pragma unroll
    for (int g = 0; g < 8; ++g)
      *reinterpret_cast<float4*>(&slot[idx * kH + (((8 * half + g) ^ (idx & 15)) << 2)]) = make_float4(S[2 * g].x, S[2 * g].y, S[2 * g + 1].x, S[2 * g + 1].y);
  };
  // S[idx][h0..] <- S * w - sa_idx * b + v_idx * kt
  auto update = [&](const float (*buf)[kH], const float* bk) {
    const float sa = buf[kVecs + 1][idx], vi = buf[4][idx];
    const float2 nsa2 = make_float2(-sa, -sa), vi2 = make_float2(vi, vi);
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const float4 w4 = *reinterpret_cast<const float4*>(&buf[0][h0 + 4 * g]);
      const float4 b4 = *reinterpret_cast<const float4*>(&bk[h0 + 4 * g]);
      const float4 kt4 = *reinterpret_cast<const float4*>(&buf[3][h0 + 4 * g]);
      const float2 s0 = __ffma2_rn(nsa2, make_float2(b4.x, b4.y), __fmul2_rn(S[2 * g], make_float2(w4.x, w4.y)));
      const float2 s1 = __ffma2_rn(nsa2, make_float2(b4.z, b4.w), __fmul2_rn(S[2 * g + 1], make_float2(w4.z, w4.w)));
      S[2 * g] = __ffma2_rn(vi2, make_float2(kt4.x, kt4.y), s0);
      S[2 * g + 1] = __ffma2_rn(vi2, make_float2(kt4.z, kt4.w), s1);
    }
  };

  // the column sums of the timestep before this one in the walk: their halves are complete once a barrier has passed
  int pend_buf = -1;
  size_t pend_out = 0;
  float pend_kap = 0.f, pend_a = 0.f;
  auto finish_pending = [&]() {
    if (pend_buf >= 0 && !row_thread && half == 0) {
      const float (*c0)[kH] = sm.col_part[pend_buf][0];
      const float (*c1)[kH] = sm.col_part[pend_buf][1];
      const float db = -(c0[2][idx] + c1[2][idx]);
      p.din[5][pend_out] = c0[0][idx] + c1[0][idx];
      p.din[3][pend_out] = c0[1][idx] + c1[1][idx];
      p.din[0][pend_out] = c0[3][idx] + c1[3][idx];
      p.din[1][pend_out] = db * pend_kap;
      p.din[2][pend_out] = (c0[4][idx] + c1[4][idx]) + db * pend_a;
    }
    pend_buf = -1;
  };

  int buf3 = 0;                   // rotates over the three col_part buffers, one per timestep
  // timesteps hi-1 .. lo of the chunk at t0 backwards; the state before local timestep s is in slot[s - lo]
  auto run_backwards = [&](const float (*V)[kBwdVecs][kH], int t0, int lo, int hi) {
    for (int s = hi - 1; s >= lo; --s) {
      const int par = s & 1;      // chunks start at multiples of 8: the parity of the timestep
      const size_t out = head_base + (size_t)(t0 + s) * C + idx;
      const float* w = V[s][0]; const float* a = V[s][1]; const float* kap = V[s][2];
      const float* kt = V[s][3]; const float* v = V[s][4]; const float* r = V[s][5]; const float* dy = V[s][6];
      const float* sa = V[s][7];
      const float* bk = sm.bk[s];
      if (row_thread) {
        const float dyi = dy[idx];
        const float2 dy2 = make_float2(dyi, dyi);
        float2 dv0 = make_float2(0.f, 0.f), dv1 = dv0, ds0 = dv0, ds1 = dv0;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 r4 = *reinterpret_cast<const float4*>(&r[h0 + 4 * g]);
          const float4 kt4 = *reinterpret_cast<const float4*>(&kt[h0 + 4 * g]);
          const float4 b4 = *reinterpret_cast<const float4*>(&bk[h0 + 4 * g]);
          const float2 g0 = __ffma2_rn(dy2, make_float2(r4.x, r4.y), dS[2 * g]);
          const float2 g1 = __ffma2_rn(dy2, make_float2(r4.z, r4.w), dS[2 * g + 1]);
          dS[2 * g] = g0; dS[2 * g + 1] = g1;
          dv0 = __ffma2_rn(g0, make_float2(kt4.x, kt4.y), dv0); dv1 = __ffma2_rn(g1, make_float2(kt4.z, kt4.w), dv1);
          ds0 = __ffma2_rn(g0, make_float2(b4.x, b4.y), ds0); ds1 = __ffma2_rn(g1, make_float2(b4.z, b4.w), ds1);
        }
        sm.ds_part[par][half][idx] = sum4(ds0, ds1);
        sm.dv_part[par][half][idx] = sum4(dv0, dv1);
      } else {
        const float* slot = sm.slot[s - lo];
#pragma unroll
        for (int e = 0; e < 16; ++e)
          S[e] = make_float2(slot[(h0 + 2 * e) * kH + joff[(2 * e) & 15]], slot[(h0 + 2 * e + 1) * kH + joff[(2 * e + 1) & 15]]);
        const float wj = w[idx], ktj = kt[idx], rj = r[idx], bj = bk[idx];
        const float2 wj2 = make_float2(wj, wj), nbj2 = make_float2(-bj, -bj), ktj2 = make_float2(ktj, ktj), rj2 = make_float2(rj, rj);
        float2 dr0 = make_float2(0.f, 0.f), dr1 = dr0, dkt0 = dr0, dkt1 = dr0, db0 = dr0, db1 = dr0, dw0 = dr0, dw1 = dr0;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 sa4 = *reinterpret_cast<const float4*>(&sa[h0 + 4 * g]);
          const float4 v4 = *reinterpret_cast<const float4*>(&v[h0 + 4 * g]);
          const float4 dy4 = *reinterpret_cast<const float4*>(&dy[h0 + 4 * g]);
          const float2 sa_a = make_float2(sa4.x, sa4.y), sa_b = make_float2(sa4.z, sa4.w);
          const float2 v_a = make_float2(v4.x, v4.y), v_b = make_float2(v4.z, v4.w);
          const float2 dy_a = make_float2(dy4.x, dy4.y), dy_b = make_float2(dy4.z, dy4.w);
          const float2 st_a = __ffma2_rn(v_a, ktj2, __ffma2_rn(sa_a, nbj2, __fmul2_rn(S[2 * g], wj2)));
          const float2 st_b = __ffma2_rn(v_b, ktj2, __ffma2_rn(sa_b, nbj2, __fmul2_rn(S[2 * g + 1], wj2)));
          const float2 g_a = __ffma2_rn(dy_a, rj2, dS[2 * g]), g_b = __ffma2_rn(dy_b, rj2, dS[2 * g + 1]);
          dS[2 * g] = g_a; dS[2 * g + 1] = g_b;
          dr0 = __ffma2_rn(st_a, dy_a, dr0); dr1 = __ffma2_rn(st_b, dy_b, dr1);
          dkt0 = __ffma2_rn(g_a, v_a, dkt0); dkt1 = __ffma2_rn(g_b, v_b, dkt1);
          db0 = __ffma2_rn(g_a, sa_a, db0); db1 = __ffma2_rn(g_b, sa_b, db1);
          dw0 = __ffma2_rn(g_a, S[2 * g], dw0); dw1 = __ffma2_rn(g_b, S[2 * g + 1], dw1);
        }
        float (*cp)[kH] = sm.col_part[buf3][half];
        cp[0][idx] = sum4(dr0, dr1);
        cp[1][idx] = sum4(dkt0, dkt1);
        cp[2][idx] = sum4(db0, db1);
        cp[3][idx] = sum4(dw0, dw1);
      }
      __syncthreads();            // the halves of this timestep's dv and -dsa, and all of the previous timestep's column sums, are published
      finish_pending();
      if (row_thread) {
        const float dsa = -(sm.ds_part[par][0][idx] + sm.ds_part[par][1][idx]);
        if (half == 0) p.din[4][out] = sm.dv_part[par][0][idx] + sm.dv_part[par][1][idx];
        const float2 dsa2 = make_float2(dsa, dsa);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 w4 = *reinterpret_cast<const float4*>(&w[h0 + 4 * g]);
          const float4 k4 = *reinterpret_cast<const float4*>(&kap[h0 + 4 * g]);
          dS[2 * g] = __ffma2_rn(dsa2, make_float2(k4.x, k4.y), __fmul2_rn(dS[2 * g], make_float2(w4.x, w4.y)));
          dS[2 * g + 1] = __ffma2_rn(dsa2, make_float2(k4.z, k4.w), __fmul2_rn(dS[2 * g + 1], make_float2(w4.z, w4.w)));
        }
      } else {
        const float wj = w[idx], kapj = kap[idx];
        const float2 wj2 = make_float2(wj, wj), kapj2 = make_float2(kapj, kapj);
        float2 dk0 = make_float2(0.f, 0.f), dk1 = dk0;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 p0 = *reinterpret_cast<const float4*>(&sm.ds_part[par][0][h0 + 4 * g]);
          const float4 p1 = *reinterpret_cast<const float4*>(&sm.ds_part[par][1][h0 + 4 * g]);
          const float2 d_a = make_float2(-(p0.x + p1.x), -(p0.y + p1.y)), d_b = make_float2(-(p0.z + p1.z), -(p0.w + p1.w));
          dk0 = __ffma2_rn(S[2 * g], d_a, dk0); dk1 = __ffma2_rn(S[2 * g + 1], d_b, dk1);
          dS[2 * g] = __ffma2_rn(d_a, kapj2, __fmul2_rn(dS[2 * g], wj2));
          dS[2 * g + 1] = __ffma2_rn(d_b, kapj2, __fmul2_rn(dS[2 * g + 1], wj2));
        }
        sm.col_part[buf3][half][4][idx] = sum4(dk0, dk1);
        pend_kap = kapj; pend_a = a[idx];
      }
      pend_buf = buf3; pend_out = out;
      buf3 = buf3 == 2 ? 0 : buf3 + 1;
    }
  };

  issue_vec(n_ck - 1);
  if (row_thread) load_ckpt(n_ck - 1);
  for (int ck = n_ck - 1; ck >= 0; --ck) {
    const int t0 = ck * kCk, steps = min(kCk, p.T - t0);
    const int lo = steps > kSub ? kSub : 0;      // the chunk runs as [lo, steps) and then, if lo > 0, [0, lo)
    __syncthreads();              // everyone is done with the chunk after this one: its vectors, bk and slots
    finish_pending();             // (reads col_part only)
    issue_vec(ck - 1);            // into the buffer that chunk used
    cp_async_wait<1>();           // this thread's copies of chunk ck have landed
    __syncthreads();              // ... and everyone's
    const float (*V)[kBwdVecs][kH] = sm.vec[ck & 1];
    for (int e = tid; e < steps * kH; e += kBwdThreads) sm.bk[e / kH][e % kH] = V[e / kH][1][e % kH] * V[e / kH][2][e % kH];
    __syncthreads();
    if (row_thread) {             // the states before timesteps lo .. steps-1
      for (int s = 0; s < steps; ++s) {
        if (s >= lo) store_slot(sm.slot[s - lo]);
        if (s + 1 < steps) update(V[s], sm.bk[s]);
      }
      if (lo > 0) load_ckpt(ck); else if (ck > 0) load_ckpt(ck - 1);
    }
    __syncthreads();
    run_backwards(V, t0, lo, steps);
    if (lo > 0) {
      __syncthreads();            // the column threads are done with the slots
      finish_pending();
      if (row_thread) {           // the states before timesteps 0 .. lo-1
        for (int s = 0; s < lo; ++s) {
          store_slot(sm.slot[s]);
          if (s + 1 < lo) update(V[s], sm.bk[s]);
        }
        if (ck > 0) load_ckpt(ck - 1);
      }
      __syncthreads();
      run_backwards(V, t0, 0, lo);
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  finish_pending();
  if (p.dstate_in && row_thread) {
#pragma unroll
    for (int g = 0; g < 8; ++g)
      reinterpret_cast<float4*>(p.dstate_in + (head * kH + idx) * kH + h0)[g] = make_float4(dS[2 * g].x, dS[2 * g].y, dS[2 * g + 1].x, dS[2 * g + 1].y);
  }
}

}  // namespace
}  // namespace pb

using namespace pb;

extern "C" int pb_wkv7_forward(const float* decay, const float* iclr, const float* removal_k, const float* replacement_k,
                               const float* v, const float* r, const float* state_in,
                               int64_t batch, int64_t steps, int64_t heads, int head_dim,
                               float* y, float* state_out, float* checkpoints, float* sa, void* stream) {
  if (!decay || !iclr || !removal_k || !replacement_k || !v || !r || !y)
    return fail(PB_ERR_NULL_POINTER, "pb_wkv7_forward: the six inputs and y must be non-null");
  if (head_dim != kH) return fail(PB_ERR_UNSUPPORTED, "pb_wkv7_forward: head size %d (this kernel is built for %d)", head_dim, kH);
  if (batch <= 0 || steps <= 0 || heads <= 0 || batch * heads > 0x7fffffffll || steps > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "pb_wkv7_forward: batch=%lld steps=%lld heads=%lld", (long long)batch, (long long)steps, (long long)heads);
  const void* ptrs[] = {decay, iclr, removal_k, replacement_k, v, r, state_in, state_out, checkpoints, sa};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(PB_ERR_MISALIGNED, "pb_wkv7_forward: every array must be 16-byte aligned");
  WkvParams p{{decay, iclr, removal_k, replacement_k, v, r}, state_in, y, state_out, checkpoints, sa, (int)steps, (int)heads};
  wkv7_forward_kernel<<<(unsigned)(batch * heads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PB_LAUNCH_CHECK("wkv7_forward_kernel");
  return PB_OK;
}

extern "C" size_t pb_wkv7_checkpoint_floats(int64_t batch, int64_t steps, int64_t heads, int head_dim) {
  if (batch <= 0 || steps <= 0 || heads <= 0 || head_dim != kH) return 0;
  return (size_t)batch * heads * ((steps + kCk - 1) / kCk) * kH * kH;
}

extern "C" int pb_wkv7_backward(const float* decay, const float* iclr, const float* removal_k, const float* replacement_k,
                                const float* v, const float* r, const float* checkpoints, const float* sa, const float* dy, const float* dstate_out,
                                int64_t batch, int64_t steps, int64_t heads, int head_dim,
                                float* d_decay, float* d_iclr, float* d_removal_k, float* d_replacement_k, float* d_v, float* d_r,
                                float* dstate_in, void* stream) {
  if (!decay || !iclr || !removal_k || !replacement_k || !v || !r || !checkpoints || !sa || !dy || !d_decay || !d_iclr || !d_removal_k ||
      !d_replacement_k || !d_v || !d_r)
    return fail(PB_ERR_NULL_POINTER, "pb_wkv7_backward: the six inputs, the checkpoints, sa, dy and the six gradients must be non-null");
  if (head_dim != kH) return fail(PB_ERR_UNSUPPORTED, "pb_wkv7_backward: head size %d (this kernel is built for %d)", head_dim, kH);
  if (batch <= 0 || steps <= 0 || heads <= 0 || batch * heads > 0x7fffffffll || steps > 0x7fffffffll)
    return fail(PB_ERR_BAD_SHAPE, "pb_wkv7_backward: batch=%lld steps=%lld heads=%lld", (long long)batch, (long long)steps, (long long)heads);
  const void* ptrs[] = {decay, iclr, removal_k, replacement_k, v, r, checkpoints, sa, dy, dstate_out, dstate_in};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(PB_ERR_MISALIGNED, "pb_wkv7_backward: every array must be 16-byte aligned");
  WkvBwdParams p{{decay, iclr, removal_k, replacement_k, v, r}, dy, sa, checkpoints, dstate_out,
                 {d_decay, d_iclr, d_removal_k, d_replacement_k, d_v, d_r}, dstate_in, (int)steps, (int)heads};
  PB_CUDA_TRY(cudaFuncSetAttribute(wkv7_backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(WkvBwdSmem)));   // per device
  wkv7_backward_kernel<<<(unsigned)(batch * heads), kBwdThreads, sizeof(WkvBwdSmem), static_cast<cudaStream_t>(stream)>>>(p);
  PB_LAUNCH_CHECK("wkv7_backward_kernel");
  return PB_OK;
}
