// WKV-7 state scan of the modified RWKV-7 TimeMix block (sm_100a): the per-timestep recurrence of
// pratchya/_nnx_impl/_module.py:187-207 as one kernel instead of a scan of T small matmuls, and its
// cotangents (what jax.grad derives from that scan) as a second kernel.
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
// Two layouts of the state over the threads of a CTA (one CTA per (b, n), H = 64).
// Forward: one row per thread (64 threads).  Both dot products of a timestep run inside the thread, so the recurrence
// holds no shuffle; the price is that every thread reads every input vector in full, and although those reads are
// same-address broadcasts a 16-byte load still returns 512 bytes per warp to the registers: at 128 bytes per clock
// and SM that traffic is what bounds the kernel.
// Backward: 2-D tiles (128 threads).  Warp q owns rows 16q .. 16q+15; its 32 lanes form a 4 x 8 grid (ti, tj) and
// lane (ti, tj) keeps the 4 x 8 tile of rows 16q + 4ti .. +3 and columns 4tj .. +3 and 32 + 4tj .. +3 (as float2 pairs
// along the columns).  A lane reads 8 elements of each vector per timestep, not 64, which the backward pass needs:
// kept per row and per column it moved four times the forward pass's vector bytes.  Sums along a row end with three
// xor-shuffles across tj and never leave the warp; sums along a column are outputs, not part of the recurrence: two
// butterfly shuffle levels across ti, then the warps' parts meet in shared memory.
// The input vectors of a timestep arrive by cp.async ahead of time.  HBM traffic is the algorithmic minimum: every
// input read once, every output written once, the state once per sequence, plus what the backward pass needs when
// one follows (below).
#include "common.cuh"

namespace pb {
namespace {

constexpr int kH = 64;            // head size
constexpr int kR = 4;             // rows of a lane's tile (measured: 4 beats 8 and 2 on batch 8 x 32 heads x 4096 timesteps)
constexpr int kWarps = 16 / kR;   // a warp owns 4 * kR rows
constexpr int kThreads = 32 * kWarps;      // per head
constexpr int kPairs = 4;         // forward ring depth in pairs of timesteps: eight timesteps of input in flight
constexpr int kVecs = 6;          // decay, iclr, removal_k, replacement_k, v, r
constexpr int kCk = 8;            // spacing of the state checkpoints the backward pass restarts from
#ifndef PB_WKV_FWD_ROWS
#define PB_WKV_FWD_ROWS 1
#endif
// State rows per thread of the forward kernel (64 / kFwdRows threads per head).  Two rows per thread halve the vector bytes a
// timestep pulls from shared memory, but the one warp left per head then runs twice the arithmetic in sequence: measured 2.67 ms
// against 1.88 ms for one row per thread (batch 8 x 32 heads x 4096 timesteps).
constexpr int kFwdRows = PB_WKV_FWD_ROWS;
constexpr int kSub = 4;           // timesteps whose recomputed states the backward pass keeps at once
constexpr int kBwdVecs = kVecs + 2;      // the six inputs, dy and sa
constexpr int kTileQuads = kH * kH / 4;  // float4 per state

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float2 dup(float x) { return make_float2(x, x); }

// a lane's eight columns of a shared-memory vector (four at p, four at p + 32) as four float2
__device__ __forceinline__ void ld8(const float* p, float2 (&out)[4]) {
  const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 32);
  out[0] = make_float2(lo.x, lo.y); out[1] = make_float2(lo.z, lo.w); out[2] = make_float2(hi.x, hi.y); out[3] = make_float2(hi.z, hi.w);
}
// kR consecutive floats
__device__ __forceinline__ void ldr(const float* p, float (&out)[kR]) {
  if constexpr (kR == 8) {
    const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
    out[0] = lo.x; out[1] = lo.y; out[2] = lo.z; out[3] = lo.w; out[4] = hi.x; out[5] = hi.y; out[6] = hi.z; out[7] = hi.w;
  } else if constexpr (kR == 4) {
    const float4 lo = *reinterpret_cast<const float4*>(p);
    out[0] = lo.x; out[1] = lo.y; out[2] = lo.z; out[3] = lo.w;
  } else {
    const float2 lo = *reinterpret_cast<const float2*>(p);
    out[0] = lo.x; out[1] = lo.y;
  }
}

// every lane's v[a] becomes the sum over the eight lanes that share ti (lane bits 0..2)
__device__ __forceinline__ void row_allreduce(float (&v)[kR]) {
#pragma unroll
  for (int m = 1; m < 8; m <<= 1) {
#pragma unroll
    for (int a = 0; a < kR; ++a) v[a] += __shfl_xor_sync(0xffffffffu, v[a], m);
  }
}
// four column sums over the four lanes that share tj (lane bits 3, 4): lane ti ends up with column ti of the four
__device__ __forceinline__ float col_reduce_scatter(const float2 (&v)[2], int ti) {
  bool up = ti & 2;
  const float2 keep = up ? v[1] : v[0], send = up ? v[0] : v[1];
  const float2 w2 = make_float2(keep.x + __shfl_xor_sync(0xffffffffu, send.x, 16), keep.y + __shfl_xor_sync(0xffffffffu, send.y, 16));
  up = ti & 1;
  return (up ? w2.y : w2.x) + __shfl_xor_sync(0xffffffffu, up ? w2.x : w2.y, 8);
}
__device__ __forceinline__ float pick(const float (&v)[kR], int a) {
  float r = v[0];
#pragma unroll
  for (int k = 1; k < kR; ++k) r = a == k ? v[k] : r;
  return r;
}

// Where lane (ti, tj) of warp q sits: rows row0 .. row0 + kR - 1, columns col0 .. col0+3 and 32 + col0 .. +3 (so that the
// eight lanes of a tile row read 128 contiguous bytes of a vector with each 16-byte load: no bank conflicts).
struct Tile {
  int tid, ti, tj, row0, col0;
  __device__ Tile() {
    tid = threadIdx.x;
    const int lane = tid & 31;
    ti = lane >> 3; tj = lane & 7;
    row0 = 4 * kR * (tid >> 5) + kR * ti; col0 = 4 * tj;
  }
};

// the 8 x 8 tile of a row-major H x H matrix in global memory
__device__ __forceinline__ void load_tile_rowmajor(const float* m, const Tile& tl, float2 (&S)[kR][4]) {
#pragma unroll
  for (int a = 0; a < kR; ++a) {
    const float4 lo = __ldg(reinterpret_cast<const float4*>(m + (tl.row0 + a) * kH + tl.col0));
    const float4 hi = __ldg(reinterpret_cast<const float4*>(m + (tl.row0 + a) * kH + tl.col0 + 32));
    S[a][0] = make_float2(lo.x, lo.y); S[a][1] = make_float2(lo.z, lo.w); S[a][2] = make_float2(hi.x, hi.y); S[a][3] = make_float2(hi.z, hi.w);
  }
}
__device__ __forceinline__ void store_tile_rowmajor(float* m, const Tile& tl, const float2 (&S)[kR][4]) {
#pragma unroll
  for (int a = 0; a < kR; ++a) {
    *reinterpret_cast<float4*>(m + (tl.row0 + a) * kH + tl.col0) = make_float4(S[a][0].x, S[a][0].y, S[a][1].x, S[a][1].y);
    *reinterpret_cast<float4*>(m + (tl.row0 + a) * kH + tl.col0 + 32) = make_float4(S[a][2].x, S[a][2].y, S[a][3].x, S[a][3].y);
  }
}
// The tile in the kernels' own layout, [2 kR quarters][threads] float4: consecutive threads, consecutive 16 bytes
// (checkpoints in global memory, recomputed states in shared memory).
template <typename Ptr>
__device__ __forceinline__ void store_tile_private(Ptr base, const Tile& tl, const float2 (&S)[kR][4]) {
#pragma unroll
  for (int a = 0; a < kR; ++a) {
    base[(2 * a) * kThreads + tl.tid] = make_float4(S[a][0].x, S[a][0].y, S[a][1].x, S[a][1].y);
    base[(2 * a + 1) * kThreads + tl.tid] = make_float4(S[a][2].x, S[a][2].y, S[a][3].x, S[a][3].y);
  }
}
template <typename Ptr>
__device__ __forceinline__ void load_tile_private(Ptr base, const Tile& tl, float2 (&S)[kR][4]) {
#pragma unroll
  for (int a = 0; a < kR; ++a) {
    const float4 lo = base[(2 * a) * kThreads + tl.tid], hi = base[(2 * a + 1) * kThreads + tl.tid];
    S[a][0] = make_float2(lo.x, lo.y); S[a][1] = make_float2(lo.z, lo.w); S[a][2] = make_float2(hi.x, hi.y); S[a][3] = make_float2(hi.z, hi.w);
  }
}

// ---- forward ---------------------------------------------------------------------------------------------------
// The forward pass keeps one state ROW per thread (64 threads per head): both dot products of a timestep run inside the
// thread on four independent partial sums, with no shuffle anywhere in the recurrence, and every vector is read as a
// same-address broadcast.  That makes it bound by the bytes those reads return to the registers (80 16-byte loads per
// thread and timestep), and still a fifth faster than a forward pass on the backward pass's tiles (measured: 1.66 ms
// against 2.04 ms on batch 8 x 32 heads x 4096 timesteps), whose three shuffle levels sit inside the recurrence.
struct WkvParams {
  const float* in[kVecs];
  const float* state_in;          // [B, N, H, H] or null (zeros)
  float* y;                       // [B, T, C]
  float* state_out;               // [B, N, H, H] or null
  float4* ckpt;                   // [B, N, ceil(T / kCk)][kTileQuads] float4 or null: the state before timesteps 0, kCk, 2*kCk, ... (tile layout)
  float* sa;                      // [B, T, C] or null: sa of every timestep, for the backward pass
  int T, N;                       // timesteps, heads
};

// One timestep for ROWS rows of S (rows i, i + kH / ROWS, ...): every vector load serves all of the thread's rows.
// `buf` holds the step's decay, iclr, removal_k, replacement_k, v, r; `bk` = iclr * removal_k.
template <int ROWS>
__device__ __forceinline__ void wkv_step(float2 (&S)[ROWS][32], const float (*buf)[kH], const float* bk, int i, float (&y_out)[ROWS], float (&sa_out)[ROWS]) {
  // sa_i = sum_j S[i][j] * kap_j, four partial sums per row
  float2 acc[ROWS][4];
#pragma unroll
  for (int a = 0; a < ROWS; ++a)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[a][q] = make_float2(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float4 k4 = *reinterpret_cast<const float4*>(&buf[2][4 * j]);
#pragma unroll
    for (int a = 0; a < ROWS; ++a) {
      acc[a][(2 * j) & 3] = __ffma2_rn(S[a][2 * j], make_float2(k4.x, k4.y), acc[a][(2 * j) & 3]);
      acc[a][(2 * j + 1) & 3] = __ffma2_rn(S[a][2 * j + 1], make_float2(k4.z, k4.w), acc[a][(2 * j + 1) & 3]);
    }
  }
  float2 nsa2[ROWS], vi2[ROWS], y[ROWS][4];
#pragma unroll
  for (int a = 0; a < ROWS; ++a) {
    const float sa = ((acc[a][0].x + acc[a][0].y) + (acc[a][1].x + acc[a][1].y)) + ((acc[a][2].x + acc[a][2].y) + (acc[a][3].x + acc[a][3].y));
    sa_out[a] = sa;
    const float vi = buf[4][i + a * (kH / ROWS)];
    nsa2[a] = make_float2(-sa, -sa); vi2[a] = make_float2(vi, vi);
#pragma unroll
    for (int q = 0; q < 4; ++q) y[a][q] = make_float2(0.f, 0.f);
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float4 w4 = *reinterpret_cast<const float4*>(&buf[0][4 * j]);
    const float4 b4 = *reinterpret_cast<const float4*>(&bk[4 * j]);
    const float4 kt4 = *reinterpret_cast<const float4*>(&buf[3][4 * j]);
    const float4 r4 = *reinterpret_cast<const float4*>(&buf[5][4 * j]);
#pragma unroll
    for (int a = 0; a < ROWS; ++a) {
      float2 s0 = __ffma2_rn(nsa2[a], make_float2(b4.x, b4.y), __fmul2_rn(S[a][2 * j], make_float2(w4.x, w4.y)));
      float2 s1 = __ffma2_rn(nsa2[a], make_float2(b4.z, b4.w), __fmul2_rn(S[a][2 * j + 1], make_float2(w4.z, w4.w)));
      s0 = __ffma2_rn(vi2[a], make_float2(kt4.x, kt4.y), s0);
      s1 = __ffma2_rn(vi2[a], make_float2(kt4.z, kt4.w), s1);
      S[a][2 * j] = s0; S[a][2 * j + 1] = s1;
      y[a][(2 * j) & 3] = __ffma2_rn(s0, make_float2(r4.x, r4.y), y[a][(2 * j) & 3]);
      y[a][(2 * j + 1) & 3] = __ffma2_rn(s1, make_float2(r4.z, r4.w), y[a][(2 * j + 1) & 3]);
    }
  }
#pragma unroll
  for (int a = 0; a < ROWS; ++a)
    y_out[a] = ((y[a][0].x + y[a][0].y) + (y[a][1].x + y[a][1].y)) + ((y[a][2].x + y[a][2].y) + (y[a][3].x + y[a][3].y));
}

template <int ROWS>
__global__ void __launch_bounds__(kH / ROWS)
wkv7_forward_kernel(const __grid_constant__ WkvParams p) {
  constexpr int kFwdThreads = kH / ROWS;
  __shared__ __align__(16) float ring[kPairs][2][kVecs][kH];      // [pair slot][step of the pair][vector][channel]
  __shared__ __align__(16) float bk[2][kH];                       // iclr * removal_k of the two steps of the current pair
  __shared__ __align__(16) float stage[kH * kH];                  // a checkpoint on its way out
  const int n = blockIdx.x % p.N, b = blockIdx.x / p.N;
  const int C = p.N * kH;
  const int i = threadIdx.x;                                      // this thread's rows: i + a * kFwdThreads
  const size_t head_base = (size_t)b * p.T * C + (size_t)n * kH;      // element (b, t = 0, channel n*H)

  // a pair of timesteps is 2 x 6 vectors x 16 chunks of 16 bytes = 192 chunks: 3 * ROWS per thread
  auto issue = [&](int pair) {
#pragma unroll
    for (int c = 0; c < 3 * ROWS; ++c) {
      const int id = c * kFwdThreads + i;                // 0 .. 191
      const int step = id / (kVecs * (kH / 4)), vec = (id / (kH / 4)) % kVecs, chunk = id % (kH / 4);
      const int t = 2 * pair + step;
      if (t < p.T)
        cp_async16((uint32_t)__cvta_generic_to_shared(&ring[pair % kPairs][step][vec][chunk * 4]),
                   p.in[vec] + head_base + (size_t)t * C + chunk * 4);
    }
    cp_async_commit();            // every thread commits a (possibly empty) group per pair: the counts stay aligned
  };

  float2 S[ROWS][32];             // this thread's rows of the head's state
  const size_t shead = ((size_t)b * p.N + n) * kH * kH;
#pragma unroll
  for (int a = 0; a < ROWS; ++a) {
    if (p.state_in) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.state_in + shead + (size_t)(i + a * kFwdThreads) * kH) + j);
        S[a][2 * j] = make_float2(s4.x, s4.y); S[a][2 * j + 1] = make_float2(s4.z, s4.w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) S[a][j] = make_float2(0.0f, 0.0f);
    }
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
#pragma unroll
    for (int a = 0; a < ROWS; ++a) {
      const int r = i + a * kFwdThreads;
      bk[0][r] = step0[1][r] * step0[2][r];
      bk[1][r] = step1[1][r] * step1[2][r];
    }
    __syncthreads();
    const int t = 2 * pr;
    if (p.ckpt && (t & (kCk - 1)) == 0) {
      // the state before timestep t, in the backward kernel's tile layout.  A row would store 16 bytes every 2 KB; the rows
      // go through shared memory (16-byte groups of row i at group ^ (i & 15): conflict-free) and leave in the layout's
      // order, consecutive threads consecutive 16 bytes.
#pragma unroll
      for (int a = 0; a < ROWS; ++a) {
        const int r = i + a * kFwdThreads;
#pragma unroll
        for (int g = 0; g < 16; ++g)
          *reinterpret_cast<float4*>(&stage[r * kH + ((g ^ (r & 15)) << 2)]) = make_float4(S[a][2 * g].x, S[a][2 * g].y, S[a][2 * g + 1].x, S[a][2 * g + 1].y);
      }
      __syncthreads();
      float4* dst = p.ckpt + (((size_t)b * p.N + n) * ((p.T + kCk - 1) / kCk) + t / kCk) * kTileQuads;
#pragma unroll
      for (int k = 0; k < kTileQuads / kFwdThreads; ++k) {
        const int d = k * kFwdThreads + i;              // quarter q of backward thread bt
        const int q = d / kThreads, bt = d % kThreads;
        const int row = 4 * kR * (bt >> 5) + kR * ((bt & 31) >> 3) + (q >> 1);
        const int g = (bt & 7) + 8 * (q & 1);
        dst[d] = *reinterpret_cast<const float4*>(&stage[row * kH + ((g ^ (row & 15)) << 2)]);
      }
      // the next write of `stage` is eight timesteps and several barriers away
    }
    float y0[ROWS], sa0[ROWS];
    wkv_step<ROWS>(S, step0, bk[0], i, y0, sa0);
#pragma unroll
    for (int a = 0; a < ROWS; ++a) {
      yp[(size_t)t * C + a * kFwdThreads] = y0[a];
      if (p.sa) p.sa[head_base + (size_t)t * C + i + a * kFwdThreads] = sa0[a];
    }
    if (t + 1 < p.T) {
      wkv_step<ROWS>(S, step1, bk[1], i, y0, sa0);
#pragma unroll
      for (int a = 0; a < ROWS; ++a) {
        yp[(size_t)(t + 1) * C + a * kFwdThreads] = y0[a];
        if (p.sa) p.sa[head_base + (size_t)(t + 1) * C + i + a * kFwdThreads] = sa0[a];
      }
    }
  }
  cp_async_wait<0>();
  if (p.state_out) {
#pragma unroll
    for (int a = 0; a < ROWS; ++a)
#pragma unroll
      for (int j = 0; j < 16; ++j)
        reinterpret_cast<float4*>(p.state_out + shead + (size_t)(i + a * kFwdThreads) * kH)[j] =
            make_float4(S[a][2 * j].x, S[a][2 * j].y, S[a][2 * j + 1].x, S[a][2 * j + 1].y);
  }
}

// ---- backward of the scan ------------------------------------------------------------------------------------
// With G_t = dS_t + dy_t r_t^T the gradient of the loss with respect to S_t (dS_t arriving from timestep t+1):
//     dr_t   = S_t^T dy_t                    dv_t  = G_t kt_t                 dkt_t = G_t^T v_t
//     dsa_t  = -G_t b_t   (b = a * kap)      db_t  = -G_t^T sa_t              dw_t  = sum_i G_t[i][:] * S_{t-1}[i][:]
//     dkap_t = S_{t-1}^T dsa_t + db_t * a_t  da_t  = db_t * kap_t             dS_{t-1} = G_t diag(w_t) + dsa_t kap_t^T
// Each lane keeps its tile of dS and, within a timestep, of S_{t-1}.  dsa is a row sum (needed at once: three
// xor-shuffles); dv a row sum that is only written out; the other five are column sums that are only written out:
// two shuffle levels inside the warp, then the warps' parts go to shared memory and are added after the
// timestep's one block barrier (two buffers, by the parity of t).
//
// S_{t-1} is needed for every t and is not stored by the forward pass; inverting the recurrence would divide by the
// decay, which the reference lets go to zero.  The forward pass writes a checkpoint every kCk = 8 timesteps and
// sa_t for every t; with sa_t known the recurrence is element-wise, so every lane recomputes its own tile of the
// states from the checkpoint with no sums and no exchange: first the states before the chunk's last four
// timesteps into four shared-memory slots (the lane's private 64 floats of each), those four timesteps run
// backwards, then the states before the first four into the same slots, and those run backwards.  The chunk's
// eight vectors per timestep arrive by cp.async one chunk ahead, and the checkpoint that the next recomputation
// starts from by cp.async into the first slot that the timesteps before it have emptied.
struct WkvBwdParams {
  const float* in[kVecs];
  const float* dy;                // [B, T, C]
  const float* sa;                // [B, T, C]: S_{t-1} kap_t, from the forward pass
  const float4* ckpt;             // as the forward pass wrote it
  const float* dstate_out;        // [B, N, H, H] or null: gradient with respect to the final state
  float* din[kVecs];              // gradients of the six inputs, [B, T, C] each
  float* dstate_in;               // [B, N, H, H] or null: gradient with respect to the initial state
  int T, N;
};

struct WkvBwdSmem {
  float4 slot[kSub][kTileQuads];            // recomputed states, every lane its own tile
  float vec[2][kCk][kBwdVecs][kH];          // the chunk's vectors, two chunks
  float col_part[2][kWarps][5][kH];         // [parity of t][warp][dr, dkt, sum G sa, dw, S^T dsa][column]
};

__global__ void __launch_bounds__(kThreads)
wkv7_backward_kernel(const __grid_constant__ WkvBwdParams p) {
  extern __shared__ __align__(16) unsigned char wkv_bwd_smem[];
  WkvBwdSmem& sm = *reinterpret_cast<WkvBwdSmem*>(wkv_bwd_smem);
  const Tile tl;
  const int warp = tl.tid >> 5;
  const int n = blockIdx.x % p.N, b = blockIdx.x / p.N;
  const int C = p.N * kH;
  const size_t head_base = (size_t)b * p.T * C + (size_t)n * kH;
  const size_t head = (size_t)b * p.N + n;
  const int n_ck = (p.T + kCk - 1) / kCk;

  float2 dS[kR][4];
  if (p.dstate_out) {
    load_tile_rowmajor(p.dstate_out + head * kH * kH, tl, dS);
  } else {
#pragma unroll
    for (int a = 0; a < kR; ++a)
#pragma unroll
      for (int k = 0; k < 4; ++k) dS[a][k] = make_float2(0.0f, 0.0f);
  }

  // the eight vectors of every timestep of chunk ck -> vec[ck & 1]; every thread commits one group per call
  auto issue_vec = [&](int ck) {
    if (ck >= 0) {
      const int t0 = ck * kCk, steps = min(kCk, p.T - t0);
      for (int e = tl.tid; e < steps * kBwdVecs * (kH / 4); e += kThreads) {
        const int s = e / (kBwdVecs * (kH / 4)), rem = e % (kBwdVecs * (kH / 4)), v = rem / (kH / 4), c4 = rem % (kH / 4);
        const float* src = (v < kVecs ? p.in[v] : (v == kVecs ? p.dy : p.sa)) + head_base + (size_t)(t0 + s) * C + c4 * 4;
        cp_async16((uint32_t)__cvta_generic_to_shared(&sm.vec[ck & 1][s][v][c4 * 4]), src);
      }
    }
    cp_async_commit();
  };

  float2 S[kR][4];                // the tile being recomputed, or S_{t-1} within a timestep
  // The checkpoint a recomputation starts from is copied (this thread's 16 quarters of it) into a slot the walk has
  // just emptied, well before it is needed; the thread that copies is the thread that reads, so its own
  // cp.async wait is all the ordering this needs.
  auto prefetch_ckpt = [&](int ck, int slot) {
    if (ck >= 0) {
      const float4* src = p.ckpt + (head * n_ck + ck) * kTileQuads;
#pragma unroll
      for (int q = 0; q < 2 * kR; ++q)
        cp_async16((uint32_t)__cvta_generic_to_shared(&sm.slot[slot][q * kThreads + tl.tid]), src + q * kThreads + tl.tid);
    }
    cp_async_commit();
  };
  // S <- S * w - sa b^T + v kt^T on the tile
  auto update = [&](const float (*buf)[kH]) {
    float2 kap[4], w[4], bb[4], kt[4];
    float v[kR], sa[kR];
    ld8(buf[2] + tl.col0, kap); ld8(buf[1] + tl.col0, bb); ld8(buf[0] + tl.col0, w); ld8(buf[3] + tl.col0, kt);
    ldr(buf[4] + tl.row0, v); ldr(buf[kVecs + 1] + tl.row0, sa);
#pragma unroll
    for (int k = 0; k < 4; ++k) bb[k] = __fmul2_rn(bb[k], kap[k]);
#pragma unroll
    for (int a = 0; a < kR; ++a) {
      const float2 nsa2 = dup(-sa[a]), v2 = dup(v[a]);
#pragma unroll
      for (int k = 0; k < 4; ++k) S[a][k] = __ffma2_rn(v2, kt[k], __ffma2_rn(nsa2, bb[k], __fmul2_rn(S[a][k], w[k])));
    }
  };

  // Timesteps hi-1 .. lo of the chunk at t0 backwards; the state before local timestep s is in slot (s - lo + shift) & 3.
  // The slot of the first timestep is free as soon as its tile is in registers: checkpoint `next_ck` goes there.
  auto run_backwards = [&](const float (*V)[kBwdVecs][kH], int t0, int lo, int hi, int shift, int next_ck) {
    for (int s = hi - 1; s >= lo; --s) {
      const float (*buf)[kH] = V[s];
      const int slot = (s - lo + shift) & (kSub - 1);
      load_tile_private(sm.slot[slot], tl, S);
      if (s == hi - 1) prefetch_ckpt(next_ck, slot);
      float dy[kR], v[kR], sa[kR];
      ldr(buf[kVecs] + tl.row0, dy); ldr(buf[4] + tl.row0, v); ldr(buf[kVecs + 1] + tl.row0, sa);
      float dvp[kR], dsp[kR];
#pragma unroll
      for (int a = 0; a < kR; ++a) { dvp[a] = 0.f; dsp[a] = 0.f; }
      const int par = (t0 + s) & 1;
      float (*cp)[kH] = sm.col_part[par][warp];
      // first pass over the tile, four columns at a time: G, the row sums' parts, four of the five column sums
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        float2 w[2], bb[2], kap[2], kt[2], r[2];
        {
          const int c = tl.col0 + 32 * hc;
          const float4 w4 = *reinterpret_cast<const float4*>(buf[0] + c), a4 = *reinterpret_cast<const float4*>(buf[1] + c);
          const float4 k4 = *reinterpret_cast<const float4*>(buf[2] + c), kt4 = *reinterpret_cast<const float4*>(buf[3] + c);
          const float4 r4 = *reinterpret_cast<const float4*>(buf[5] + c);
          w[0] = make_float2(w4.x, w4.y); w[1] = make_float2(w4.z, w4.w);
          kap[0] = make_float2(k4.x, k4.y); kap[1] = make_float2(k4.z, k4.w);
          bb[0] = __fmul2_rn(make_float2(a4.x, a4.y), kap[0]); bb[1] = __fmul2_rn(make_float2(a4.z, a4.w), kap[1]);
          kt[0] = make_float2(kt4.x, kt4.y); kt[1] = make_float2(kt4.z, kt4.w);
          r[0] = make_float2(r4.x, r4.y); r[1] = make_float2(r4.z, r4.w);
        }
        float2 dr[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)}, dkt[2] = {dr[0], dr[0]}, db[2] = {dr[0], dr[0]}, dw[2] = {dr[0], dr[0]};
#pragma unroll
        for (int a = 0; a < kR; ++a) {
          const float2 dy2 = dup(dy[a]), v2 = dup(v[a]), sa2 = dup(sa[a]), nsa2 = dup(-sa[a]);
          float2 rdv = make_float2(0.f, 0.f), rds = rdv;
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const float2 sp = S[a][2 * hc + k];
            const float2 g = __ffma2_rn(dy2, r[k], dS[a][2 * hc + k]);
            dS[a][2 * hc + k] = g;
            rdv = __ffma2_rn(g, kt[k], rdv);
            rds = __ffma2_rn(g, bb[k], rds);
            const float2 st = __ffma2_rn(v2, kt[k], __ffma2_rn(nsa2, bb[k], __fmul2_rn(sp, w[k])));
            dr[k] = __ffma2_rn(st, dy2, dr[k]);
            dkt[k] = __ffma2_rn(g, v2, dkt[k]);
            db[k] = __ffma2_rn(g, sa2, db[k]);
            dw[k] = __ffma2_rn(g, sp, dw[k]);
          }
          dvp[a] += rdv.x + rdv.y;
          dsp[a] += rds.x + rds.y;
        }
        const int col = tl.col0 + 32 * hc + tl.ti;
        cp[0][col] = col_reduce_scatter(dr, tl.ti);
        cp[1][col] = col_reduce_scatter(dkt, tl.ti);
        cp[2][col] = col_reduce_scatter(db, tl.ti);
        cp[3][col] = col_reduce_scatter(dw, tl.ti);
      }
      row_allreduce(dsp);         // dsp[a] = sum_j G b of row row0 + a; dsa = -dsp
      const size_t out = head_base + (size_t)(t0 + s) * C;
      row_allreduce(dvp);
      if (tl.tj < kR) p.din[4][out + tl.row0 + tl.tj] = pick(dvp, tl.tj);
      // second pass: S_{t-1}^T dsa and dS_{t-1}
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        const int c = tl.col0 + 32 * hc;
        const float4 w4 = *reinterpret_cast<const float4*>(buf[0] + c), k4 = *reinterpret_cast<const float4*>(buf[2] + c);
        const float2 w[2] = {make_float2(w4.x, w4.y), make_float2(w4.z, w4.w)};
        const float2 kap[2] = {make_float2(k4.x, k4.y), make_float2(k4.z, k4.w)};
        float2 dk[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int a = 0; a < kR; ++a) {
          const float2 dsa2 = dup(-dsp[a]);
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            dk[k] = __ffma2_rn(S[a][2 * hc + k], dsa2, dk[k]);
            dS[a][2 * hc + k] = __ffma2_rn(dsa2, kap[k], __fmul2_rn(dS[a][2 * hc + k], w[k]));
          }
        }
        cp[4][c + tl.ti] = col_reduce_scatter(dk, tl.ti);
      }
      // the five column sums of this timestep: each warp's half is in shared memory after the barrier; thread j adds column j.
      // (The buffer of the other parity is written by the next timestep, and this one again only after the next barrier.)
      const int j = tl.tid & (kH - 1);
      const float kap_j = buf[2][j], a_j = buf[1][j];
      __syncthreads();
      if (tl.tid < kH) {
        float sum[5];
#pragma unroll
        for (int q = 0; q < 5; ++q) {
          sum[q] = sm.col_part[par][0][q][j];
#pragma unroll
          for (int w = 1; w < kWarps; ++w) sum[q] += sm.col_part[par][w][q][j];
        }
        p.din[5][out + j] = sum[0];
        p.din[3][out + j] = sum[1];
        p.din[0][out + j] = sum[3];
        p.din[1][out + j] = -sum[2] * kap_j;
        p.din[2][out + j] = sum[4] - sum[2] * a_j;
      }
    }
  };

  issue_vec(n_ck - 1);
  int pre_slot = 0;               // the slot that holds the checkpoint the next recomputation starts from
  prefetch_ckpt(n_ck - 1, pre_slot);
  for (int ck = n_ck - 1; ck >= 0; --ck) {
    const int t0 = ck * kCk, steps = min(kCk, p.T - t0);
    const int lo = steps > kSub ? kSub : 0;      // the chunk runs as [lo, steps) and then, if lo > 0, [0, lo)
    __syncthreads();              // everyone is done with the vectors of the chunk after this one
    issue_vec(ck - 1);            // into the buffer that chunk used
    cp_async_wait<1>();           // this thread's copies of chunk ck, and of its checkpoint, have landed
    __syncthreads();              // ... and everyone's vectors
    const float (*V)[kBwdVecs][kH] = sm.vec[ck & 1];
    load_tile_private(sm.slot[pre_slot], tl, S);
    for (int s = 0; s < steps; ++s) {            // the states before timesteps lo .. steps-1 -> slots 0 ..
      if (s >= lo) store_tile_private(sm.slot[s - lo], tl, S);
      if (s + 1 < steps) update(V[s]);
    }
    if (lo > 0) {
      run_backwards(V, t0, lo, steps, 0, ck);    // its first timestep empties slot steps-1-lo: this chunk's checkpoint goes there again
      pre_slot = steps - 1 - lo;
      cp_async_wait<0>();
      load_tile_private(sm.slot[pre_slot], tl, S);
      // the states before timesteps 0 .. lo-1 -> slots pre_slot, pre_slot+1, ... (mod 4): the first is there already
      for (int s = 0; s + 1 < lo; ++s) {
        update(V[s]);
        store_tile_private(sm.slot[(s + 1 + pre_slot) & (kSub - 1)], tl, S);
      }
      run_backwards(V, t0, 0, lo, pre_slot, ck - 1);
      pre_slot = (lo - 1 + pre_slot) & (kSub - 1);
    } else {
      run_backwards(V, t0, 0, steps, 0, ck - 1);
      pre_slot = steps - 1;
    }
  }
  cp_async_wait<0>();
  if (p.dstate_in) store_tile_rowmajor(p.dstate_in + head * kH * kH, tl, dS);
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
  WkvParams p{{decay, iclr, removal_k, replacement_k, v, r}, state_in, y, state_out, reinterpret_cast<float4*>(checkpoints), sa, (int)steps, (int)heads};
  wkv7_forward_kernel<kFwdRows><<<(unsigned)(batch * heads), kH / kFwdRows, 0, static_cast<cudaStream_t>(stream)>>>(p);
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
  WkvBwdParams p{{decay, iclr, removal_k, replacement_k, v, r}, dy, sa, reinterpret_cast<const float4*>(checkpoints), dstate_out,
                 {d_decay, d_iclr, d_removal_k, d_replacement_k, d_v, d_r}, dstate_in, (int)steps, (int)heads};
  PB_CUDA_TRY(cudaFuncSetAttribute(wkv7_backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(WkvBwdSmem)));   // per device
  wkv7_backward_kernel<<<(unsigned)(batch * heads), kThreads, sizeof(WkvBwdSmem), static_cast<cudaStream_t>(stream)>>>(p);
  PB_LAUNCH_CHECK("wkv7_backward_kernel");
  return PB_OK;
}
