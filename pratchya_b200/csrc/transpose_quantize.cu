// Quantizer of the transpose, and a plain byte transpose (sm_100a).
//
// pb_quantize_transposed produces the triple of quantize_impl(swapaxes(x,-1,-2), (1, b))
// (the operands fp8_matmul_bwd builds from x^T and g, pratchya/_qualia/_qarr.py:784-789)
// directly from x[rows, cols], without writing the transposed dense matrix:
//   1. column-block amax: m[c][rb] = max |x[rb*b .. rb*b+b-1, c]|   (scratch, the block order of x^T)
//   2. the shared per-super-group scale kernel (divisors into scratch, sc8 / sc32 out)
//   3. tile transpose through shared memory, dividing on the way, coalesced byte rows out.
#include <cuda.h>

#include "common.cuh"

#include <mutex>

namespace pb {

// defined in quantize.cu
int launch_group_scales(const uint32_t* amax_bits, float* divisor, uint8_t* sc8, float* sc32, int64_t n_groups, int64_t K, cudaStream_t st);
int launch_row128_colmax(const void* x, int out_format, void* q, uint8_t* sc8, float* sc32, uint32_t* col_amax_bits,
                         int64_t batch, int64_t rows, int64_t cols, cudaStream_t st);

namespace {

constexpr int kTile = 64;

// grid: (cols/2 per 128 threads, row blocks, batch).  Each thread owns two adjacent columns.
template <typename InT>
__global__ void __launch_bounds__(128)
column_amax_kernel(const InT* __restrict__ x, uint32_t* __restrict__ amax_bits, int rows, int cols, int b) {
  const int c = (blockIdx.x * 128 + threadIdx.x) * 2;
  const int rb = blockIdx.y;
  const int nrb = rows / b;
  const InT* src = x + ((size_t)blockIdx.z * rows + (size_t)rb * b) * cols;
  if (c >= cols) return;
  float m0 = 0.0f, m1 = 0.0f;
  const bool pair = (c + 1 < cols) && ((cols & 1) == 0);
  for (int r = 0; r < b; ++r) {
    if (pair) {
      if constexpr (sizeof(InT) == 2) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(src + (size_t)r * cols + c);
        m0 = fmaxf(m0, fabsf(__uint_as_float(w << 16)));
        m1 = fmaxf(m1, fabsf(__uint_as_float(w & 0xffff0000u)));
      } else {
        const float2 w = *reinterpret_cast<const float2*>(src + (size_t)r * cols + c);
        m0 = fmaxf(m0, fabsf(w.x));
        m1 = fmaxf(m1, fabsf(w.y));
      }
    } else {
      m0 = fmaxf(m0, fabsf(Elem<InT>::to_f32(src[(size_t)r * cols + c])));
      if (c + 1 < cols) m1 = fmaxf(m1, fabsf(Elem<InT>::to_f32(src[(size_t)r * cols + c + 1])));
    }
  }
  uint32_t* dst = amax_bits + ((size_t)blockIdx.z * cols + c) * nrb + rb;
  dst[0] = __float_as_uint(m0);
  if (c + 1 < cols) dst[nrb] = __float_as_uint(m1);
}

// grid: (ceil(cols/64), ceil(rows/64), batch), 256 threads.  Reads a 64x64 tile of x row-wise,
// writes 64 rows (columns of x) of 64 quantized bytes each.
template <typename InT, int FMT>
__global__ void __launch_bounds__(256)
transpose_apply_kernel(const InT* __restrict__ x, const float* __restrict__ divisor, uint8_t* __restrict__ q_t,
                       int rows, int cols, int b) {
  __shared__ float tile[kTile][kTile + 1];
  const int r0 = blockIdx.y * kTile, c0 = blockIdx.x * kTile;
  const InT* src = x + (size_t)blockIdx.z * rows * cols;
  for (int i = threadIdx.x; i < kTile * kTile; i += 256) {
    const int r = i / kTile, c = i % kTile;
    tile[r][c] = (r0 + r < rows && c0 + c < cols) ? Elem<InT>::to_f32(src[(size_t)(r0 + r) * cols + c0 + c]) : 0.0f;
  }
  __syncthreads();
  const int nrb = rows / b;
  uint8_t* dst = q_t + (size_t)blockIdx.z * rows * cols;
  const float* div = divisor + (size_t)blockIdx.z * cols * nrb;
  // thread -> (output row = column c of x, 16 consecutive source rows)
  const int c = threadIdx.x / 4, seg = threadIdx.x % 4;
  if (c0 + c >= cols) return;
  uint32_t out[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    uint32_t packed = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = seg * 16 + w * 4 + h * 2;
      float v0 = 0.0f, v1 = 0.0f;
      if (r0 + r < rows) {
        const float D = div[(size_t)(c0 + c) * nrb + (r0 + r) / b];
        v0 = div_hoisted(tile[r][c], D, __frcp_rn(D));
      }
      if (r0 + r + 1 < rows) {
        const float D = div[(size_t)(c0 + c) * nrb + (r0 + r + 1) / b];
        v1 = div_hoisted(tile[r + 1][c], D, __frcp_rn(D));
      }
      packed |= bf16x2_to_fp8x2<FMT>(pack_bf16x2(v0, v1)) << (16 * h);
    }
    out[w] = packed;
  }
  uint8_t* o = dst + (size_t)(c0 + c) * rows + r0 + seg * 16;
  if (r0 + seg * 16 + 16 <= rows && (rows & 15) == 0 && (reinterpret_cast<uintptr_t>(q_t) & 15) == 0) {
    *reinterpret_cast<uint4*>(o) = make_uint4(out[0], out[1], out[2], out[3]);
  } else {
    for (int j = 0; j < 16; ++j)
      if (r0 + seg * 16 + j < rows) o[j] = (uint8_t)(out[j >> 2] >> (8 * (j & 3)));
  }
}


// ---- vectorised variants (cols a multiple of the tile width, 16-byte aligned rows) -------------
// Column-block amax: a CTA owns one 128-row block of kAmaxCols channels.  Each lane keeps VEC
// channels, each warp 16 of the 128 rows (16 independent 128-bit loads per lane), then the eight
// warps are reduced through shared memory.
template <typename InT> struct Vec16 { static constexpr int n = 16 / (int)sizeof(InT); };

template <typename InT>
__global__ void __launch_bounds__(256)
column_amax128_kernel(const InT* __restrict__ x, uint32_t* __restrict__ amax_bits, int rows, int cols) {
  constexpr int VEC = Vec16<InT>::n;
  constexpr int kCols = 32 * VEC;
  __shared__ float red[8][kCols];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = blockIdx.x * kCols + lane * VEC;
  const int rb = blockIdx.y, nrb = rows / 128;
  const InT* src = x + ((size_t)blockIdx.z * rows + (size_t)rb * 128 + warp * 16) * cols + c0;
  float m[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) m[j] = 0.0f;
  uint4 w[16];
#pragma unroll
  for (int r = 0; r < 16; ++r) w[r] = __ldcs(reinterpret_cast<const uint4*>(src + (size_t)r * cols));
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const uint32_t in[4] = {w[r].x, w[r].y, w[r].z, w[r].w};
    if constexpr (sizeof(InT) == 2) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        m[2 * j] = fmaxf(m[2 * j], fabsf(__uint_as_float(in[j] << 16)));
        m[2 * j + 1] = fmaxf(m[2 * j + 1], fabsf(__uint_as_float(in[j] & 0xffff0000u)));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) m[j] = fmaxf(m[j], fabsf(__uint_as_float(in[j])));
    }
  }
#pragma unroll
  for (int j = 0; j < VEC; ++j) red[warp][lane * VEC + j] = m[j];
  __syncthreads();
  for (int c = threadIdx.x; c < kCols; c += 256) {
    float v = red[0][c];
#pragma unroll
    for (int k = 1; k < 8; ++k) v = fmaxf(v, red[k][c]);
    amax_bits[((size_t)blockIdx.z * cols + blockIdx.x * kCols + c) * nrb + rb] = __float_as_uint(v);
  }
}

// Apply + transpose: a CTA owns 128 rows (one block row) x 64 channels.  The tile is loaded with
// 128-bit loads into shared memory; then thread (channel, segment) walks 32 rows down its channel
// (consecutive lanes = consecutive channels: conflict-free), quantizes with the block's divisor and
// writes one whole 32-byte sector of the transposed output.
template <typename InT, int FMT>
__global__ void __launch_bounds__(256)
transpose_apply128_kernel(const InT* __restrict__ x, const float* __restrict__ divisor, uint8_t* __restrict__ q_t,
                          int rows, int cols) {
  constexpr int VEC = Vec16<InT>::n;
  constexpr int kPitch = 64 + VEC;                   // elements per tile row, padded
  __shared__ __align__(16) InT tile[128 * kPitch];
  const int r0 = blockIdx.y * 128, c0 = blockIdx.x * 64;
  const InT* src = x + (size_t)blockIdx.z * rows * cols + (size_t)r0 * cols + c0;
  constexpr int kThreadsPerRow = 64 / VEC;           // 8 (bf16) or 16 (f32)
  constexpr int kRowsPerPass = 256 / kThreadsPerRow;
  const int lr = threadIdx.x / kThreadsPerRow, lc = (threadIdx.x % kThreadsPerRow) * VEC;
#pragma unroll
  for (int p = 0; p < 128 / kRowsPerPass; ++p) {
    const int r = p * kRowsPerPass + lr;
    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(src + (size_t)r * cols + lc));
    *reinterpret_cast<uint4*>(&tile[r * kPitch + lc]) = v;
  }
  __syncthreads();
  const int c = threadIdx.x & 63, seg = threadIdx.x >> 6;      // 4 segments of 32 rows
  const int nrb = rows / 128;
  const float D = divisor[((size_t)blockIdx.z * cols + c0 + c) * nrb + blockIdx.y];
  const float rcp = __frcp_rn(D);
  uint32_t out[8];
  const float2 nD2 = make_float2(-D, -D), r2 = make_float2(rcp, rcp);
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = Elem<InT>::to_f32(tile[(seg * 32 + w * 4 + j) * kPitch + c]);
    out[w] = bf16x2_to_fp8x2<FMT>(div_hoisted_pack2(v[0], v[1], nD2, r2)) | (bf16x2_to_fp8x2<FMT>(div_hoisted_pack2(v[2], v[3], nD2, r2)) << 16);
  }
  uint8_t* o = q_t + (size_t)blockIdx.z * rows * cols + (size_t)(c0 + c) * rows + r0 + seg * 32;
  asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(o), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]), "r"(out[4]), "r"(out[5]), "r"(out[6]), "r"(out[7]) : "memory");
}

// Single pass for b = 128 when rows % 1024 == 0: then a super-group of x^T (eight blocks of 128) is
// 1024 consecutive rows of one column of x, so a CTA that holds a 1024-row x kCols-column tile of x
// in shared memory (64 KB) has everything its part of the output needs: x is read once and nothing
// goes through scratch.  Thread (column c, block blk): amax of its 128 rows, the column's amax over the
// eight blocks, the block's scale, then its 128 output bytes as four 32-byte stores along x^T's row.
template <typename InT> struct OnePass {
  static constexpr int kCols = 64 / (int)sizeof(InT);        // 32 (bf16) or 16 (f32): 64-byte row segments
  static constexpr int kThreads = kCols * 8;
  static constexpr int kSmem = 1024 * 64;
};

template <typename InT, int FMT>
__global__ void __launch_bounds__(OnePass<InT>::kThreads)
transpose_quantize1024_kernel(const InT* __restrict__ x, uint8_t* __restrict__ q_t, uint8_t* __restrict__ sc8,
                              float* __restrict__ sc32, int rows, int cols) {
  constexpr int kCols = OnePass<InT>::kCols, kThreads = OnePass<InT>::kThreads;
  extern __shared__ __align__(16) uint8_t tile_raw[];
  InT* tile = reinterpret_cast<InT*>(tile_raw);                // [1024][kCols]
  __shared__ float col_amax[8][kCols];
  const int c0 = blockIdx.x * kCols, r0 = blockIdx.y * 1024;
  const InT* src = x + ((size_t)blockIdx.z * rows + r0) * cols + c0;
  // load: 4 threads per 64-byte row segment
  // sixteen loads in flight per thread before the first one is stored
#pragma unroll 1
  for (int base = 0; base < 1024 * 4; base += 16 * kThreads) {
    uint4 w[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const int v = base + k * kThreads + threadIdx.x, r = v >> 2, part = v & 3;
      w[k] = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(src + (size_t)r * cols) + part * 16));
    }
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const int v = base + k * kThreads + threadIdx.x;
      *reinterpret_cast<uint4*>(tile_raw + (v >> 2) * 64 + (v & 3) * 16) = w[k];
    }
  }
  __syncthreads();
  const int c = threadIdx.x % kCols, blk = threadIdx.x / kCols;
  const InT* colp = tile + (blk * 128) * kCols + c;
  float m = 0.0f;
#pragma unroll 16
  for (int i = 0; i < 128; ++i) m = fmaxf(m, fabsf(Elem<InT>::to_f32(colp[i * kCols])));
  col_amax[blk][c] = m;
  __syncthreads();
  float Mj = col_amax[0][c];
#pragma unroll
  for (int k = 1; k < 8; ++k) Mj = fmaxf(Mj, col_amax[k][c]);
  uint32_t sb; float D;
  block_scale(m, Mj, sb, D);
  const int nsg = rows >> 10;                                  // super-groups per column of x
  const size_t grp = ((size_t)blockIdx.z * cols + c0 + c) * nsg + blockIdx.y;
  sc8[grp * 8 + blk] = (uint8_t)sb;
  if (blk == 0) sc32[grp] = Mj;
  const float rcp = __frcp_rn(D);
  const float2 nD2 = make_float2(-D, -D), r2 = make_float2(rcp, rcp);
  uint8_t* o = q_t + ((size_t)blockIdx.z * cols + c0 + c) * rows + r0 + blk * 128;
#pragma unroll
  for (int seg = 0; seg < 4; ++seg) {
    uint32_t out[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = Elem<InT>::to_f32(colp[(seg * 32 + w * 4 + j) * kCols]);
      out[w] = bf16x2_to_fp8x2<FMT>(div_hoisted_pack2(v[0], v[1], nD2, r2)) | (bf16x2_to_fp8x2<FMT>(div_hoisted_pack2(v[2], v[3], nD2, r2)) << 16);
    }
    asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(o + seg * 32), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]), "r"(out[4]), "r"(out[5]), "r"(out[6]), "r"(out[7]) : "memory");
  }
}

// bf16 version of the single pass: 512 threads, thread (column pair, block, quarter) keeps its 32 rows x
// 2 columns (32 words) in registers between the amax and the quantization, works on packed bf16 pairs
// like the row quantizer (a byte permute regroups two rows of a column pair into one pair per
// column), and writes one 32-byte store per column.  Rows of odd blocks are stored with their
// 64-byte halves swapped in pairs (row ^ 1 ... as a bank-half swizzle), so that the two rows a warp
// reads at once, 128 rows apart, fall into different halves of the banks.
template <int FMT>
__global__ void __launch_bounds__(512, 2)
transpose_quantize1024_bf16_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q_t, uint8_t* __restrict__ sc8,
                                   float* __restrict__ sc32, int rows, int cols) {
  extern __shared__ __align__(16) uint8_t tile_raw[];              // [1024 rows][64 bytes]
  __shared__ uint32_t part_amax[32][16];                            // [block*4 + quarter][column pair], bf16 pairs
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 1024;
  const __nv_bfloat16* src = x + ((size_t)blockIdx.z * rows + r0) * cols + c0;
  auto row_offset = [](int r) { return (uint32_t)(r * 64) ^ (uint32_t)(((r >> 7) & 1) << 6); };
  {
    uint4 w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int v = k * 512 + threadIdx.x, r = v >> 2, part = v & 3;
      w[k] = __ldcs(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(src + (size_t)r * cols) + part * 16));
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int v = k * 512 + threadIdx.x;
      *reinterpret_cast<uint4*>(tile_raw + row_offset(v >> 2) + (v & 3) * 16) = w[k];
    }
  }
  __syncthreads();
  const int cp = threadIdx.x & 15, blk = (threadIdx.x >> 4) & 7, quarter = threadIdx.x >> 7;
  const int row_first = blk * 128 + quarter * 32;
  uint32_t w[32];
  uint32_t cm = 0u;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    w[i] = *reinterpret_cast<const uint32_t*>(tile_raw + row_offset(row_first + i) + cp * 4);
    const uint32_t a = w[i] & 0x7fff7fffu;
    const __nv_bfloat162 h = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&cm), *reinterpret_cast<const __nv_bfloat162*>(&a));
    cm = *reinterpret_cast<const uint32_t*>(&h);
  }
  part_amax[blk * 4 + quarter][cp] = cm;
  __syncthreads();
  uint32_t mb = 0u, mg = 0u;           // block amax and super-group amax of the two columns, packed
#pragma unroll
  for (int k = 0; k < 32; ++k) {
    const uint32_t v = part_amax[k][cp];
    const __nv_bfloat162 g = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&mg), *reinterpret_cast<const __nv_bfloat162*>(&v));
    mg = *reinterpret_cast<const uint32_t*>(&g);
    if ((k >> 2) == blk) {
      const __nv_bfloat162 b2 = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&mb), *reinterpret_cast<const __nv_bfloat162*>(&v));
      mb = *reinterpret_cast<const uint32_t*>(&b2);
    }
  }
  const int nsg = rows >> 10;
  uint32_t sbv[2]; float D[2];
  block_scale(__uint_as_float(mb << 16), __uint_as_float(mg << 16), sbv[0], D[0]);
  block_scale(__uint_as_float(mb & 0xffff0000u), __uint_as_float(mg & 0xffff0000u), sbv[1], D[1]);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const size_t col = (size_t)blockIdx.z * cols + c0 + 2 * cp + j;
    const size_t grp = col * nsg + blockIdx.y;
    if (quarter == 0) {
      sc8[grp * 8 + blk] = (uint8_t)sbv[j];
      if (blk == 0) sc32[grp] = j == 0 ? __uint_as_float(mg << 16) : __uint_as_float(mg & 0xffff0000u);
    }
    const float rcp = __frcp_rn(D[j]);
    const float2 nD2 = make_float2(-D[j], -D[j]), r2 = make_float2(rcp, rcp);
    uint32_t out[8];
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      uint32_t o2[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // rows i+2h and i+2h+1 of column j as one packed bf16 pair
        const uint32_t pr = __byte_perm(w[i + 2 * h], w[i + 2 * h + 1], j == 0 ? 0x5410 : 0x7632);
        const float2 v = div_hoisted_unsigned2(make_float2(__uint_as_float(pr << 16), __uint_as_float(pr & 0xffff0000u)), nD2, r2);
        const uint32_t pk = (pack_bf16x2(v.x, v.y) & 0x7fff7fffu) | (pr & 0x80008000u);
        o2[h] = bf16x2_to_fp8x2<FMT>(pk);
      }
      out[i >> 2] = o2[0] | (o2[1] << 16);
    }
    uint8_t* o = q_t + col * rows + r0 + row_first;
    asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(o), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]), "r"(out[4]), "r"(out[5]), "r"(out[6]), "r"(out[7]) : "memory");
  }
}

template <int FMT>
int launch_one_pass_bf16(const void* x, uint8_t* q_t, uint8_t* sc8, float* sc32, int64_t batch, int64_t rows, int64_t cols, cudaStream_t st) {
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  PB_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      PB_CUDA_TRY(cudaFuncSetAttribute(transpose_quantize1024_bf16_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 1024 * 64));
      configured[dev] = true;
    }
  }
  const dim3 grid((unsigned)(cols / 32), (unsigned)(rows / 1024), (unsigned)batch);
  transpose_quantize1024_bf16_kernel<FMT><<<grid, 512, 1024 * 64, st>>>((const __nv_bfloat16*)x, q_t, sc8, sc32, (int)rows, (int)cols);
  PB_LAUNCH_CHECK("transpose_quantize1024_bf16_kernel");
  return PB_OK;
}

// ---- persistent form of the bf16 single pass: TMA-staged tiles, copy and arithmetic overlapped ----------
// The kernel above holds one tile per CTA and alternates between filling it and working on it, so with two
// CTAs per SM the memory system idles while both compute (58 us for X[32768,2048]: the sum of the two phases,
// not their maximum).  Here one CTA per SM stays resident and walks over its tiles: three 64 KB tile buffers
// are filled by TMA (four boxes of 256 rows x 64 bytes per tile, one mbarrier per buffer), two groups of 512
// threads take the tiles in turn with the arithmetic of the kernel above, and the group that has just moved a
// tile into its registers refills that buffer with the tile three ahead.  A tile buffer is plain row-major
// (64-byte rows): the two half-warps of a warp read rows 128 apart, which would share banks, so the upper
// half-warp walks its rows in swapped pairs (row i ^ 1) and swaps them back in the byte permute that pairs rows.
constexpr int kRingBufs = 3;
constexpr int kRingTileBytes = 1024 * 64;
constexpr int kRingPartBytes = 2 * 2 * 32 * 16 * 4;      // part_amax[group][parity][block * 4 + quarter][column pair]
constexpr int kRingBlockBytes = 2 * 2 * 8 * 16 * 4;      // block_amax[group][parity][block][column pair]
constexpr int kRingSmem = kRingBufs * kRingTileBytes + kRingPartBytes + kRingBlockBytes + 64 + 1024;   // tiles, maxima, barriers, alignment slack
constexpr uint32_t kRingWaitPolls = 1u << 21;      // bounded wait: at most ~4 s of 2 us polls, then the kernel gives up

__device__ unsigned int g_tq_status;               // 0, or PB_ERR_DEVICE_TIMEOUT once a bounded wait ran out

__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .u32 n;\n\t"
      "mov.u32 n, 0;\n"
      "WAIT_%=:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 2000;\n\t"
      "@p bra DONE_%=;\n\t"
      "add.u32 n, n, 1;\n\t"
      "setp.lt.u32 p, n, %3;\n\t"
      "@p bra WAIT_%=;\n\t"
      "setp.ne.u32 p, n, n;\n"
      "DONE_%=:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(kRingWaitPolls) : "memory");
  return ok != 0;
}

// Waits for fill number `fill` (0, 1, 2, ... of this buffer) to land.  The two groups take a buffer's fills in turn, so the
// group that waits here did not consume the buffer's previous fill and may arrive before that one has even landed; a
// parity wait alone would then take the phase BEFORE the previous fill's (same parity as the awaited one, and over) for
// the awaited one, read a tile that is still arriving and arm the barrier a second time within one phase.  So the
// thread that arms a fill publishes its number in shared memory afterwards (release), and a waiter first sees that
// number (acquire): from then on the barrier is in the awaited fill's own phase and the parity wait means what it says.
// Both waits are bounded.
__device__ __noinline__ bool ring_wait_armed(uint32_t armed_addr, uint32_t fill) {      // the rare case: the fill is not armed yet
  for (uint32_t n = 0; n < kRingWaitPolls; ++n) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(armed_addr) : "memory");
    if (v > fill) return true;
  }
  return false;
}
__device__ __forceinline__ bool ring_wait_tile(uint32_t bar, uint32_t armed_addr, uint32_t fill) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(armed_addr) : "memory");
  if (v <= fill && !ring_wait_armed(armed_addr, fill)) return false;
  return ring_wait(bar, fill & 1u);
}
__device__ __forceinline__ void ring_publish_fill(uint32_t armed_addr, uint32_t fill) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(armed_addr), "r"(fill + 1u) : "memory");
}

template <int FMT>
__global__ void __launch_bounds__(1024, 1)
transpose_quantize1024_bf16_ring_kernel(const __grid_constant__ CUtensorMap map_x, uint8_t* __restrict__ q_t, uint8_t* __restrict__ sc8,
                                        float* __restrict__ sc32, int rows, int cols, int tiles_x, int tiles_y, int n_tiles) {
  extern __shared__ uint8_t ring_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ring_raw) + 1023) & ~(uintptr_t)1023);
  uint32_t (*part_amax)[32][16] = reinterpret_cast<uint32_t (*)[32][16]>(smem + kRingBufs * kRingTileBytes);   // [group * 2 + parity]
  uint32_t (*block_amax)[8][16] = reinterpret_cast<uint32_t (*)[8][16]>(smem + kRingBufs * kRingTileBytes + kRingPartBytes);
  const uint32_t s_tiles = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t s_bar = s_tiles + kRingBufs * kRingTileBytes + kRingPartBytes + kRingBlockBytes;
  const int tid = threadIdx.x, grp = tid >> 9, gt = tid & 511;

  if (tid == 0) {
    for (int b = 0; b < kRingBufs; ++b) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_bar + 8u * b));
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(s_bar + 32u + 4u * b), "r"(0u) : "memory");      // fills armed so far
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // tile `seq` of this CTA: global tile blockIdx.x + seq * gridDim.x, column tiles fastest (neighbouring CTAs read
  // neighbouring 64-byte segments of the same rows)
  auto issue = [&](int seq) {
    const int tl = blockIdx.x + seq * gridDim.x;
    if (tl >= n_tiles) return;
    const int cx = tl % tiles_x, rest = tl / tiles_x, ry = rest % tiles_y, z = rest / tiles_y;
    const uint32_t bar = s_bar + 8u * (seq % kRingBufs), dst = s_tiles + (uint32_t)(seq % kRingBufs) * kRingTileBytes;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)kRingTileBytes) : "memory");
#pragma unroll
    for (int j = 0; j < 4; ++j)
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                   ::"r"(dst + j * 16384u), "l"(&map_x), "r"(cx * 32), "r"(z * rows + ry * 1024 + j * 256), "r"(bar) : "memory");
    ring_publish_fill(s_bar + 32u + 4u * (seq % kRingBufs), (uint32_t)(seq / kRingBufs));
  };
  if (tid == 0) { issue(0); issue(1); issue(2); }

  const int cp = gt & 15, blk = (gt >> 4) & 7, quarter = gt >> 7;
  const int row_first = blk * 128 + quarter * 32;
  const int swap = (gt >> 4) & 1;                 // upper half-warp: rows in swapped pairs
  const uint32_t sel0 = swap ? 0x1054u : 0x5410u, sel1 = swap ? 0x3276u : 0x7632u;
  const int nsg = rows >> 10;
  int local = 0;
  for (int seq = grp; blockIdx.x + seq * (int)gridDim.x < n_tiles; seq += 2, ++local) {
    const int tl = blockIdx.x + seq * gridDim.x;
    const int cx = tl % tiles_x, rest = tl / tiles_x, ry = rest % tiles_y, z = rest / tiles_y;
    const int c0 = cx * 32, r0 = ry * 1024;
    const bool landed = ring_wait_tile(s_bar + 8u * (seq % kRingBufs), s_bar + 32u + 4u * (seq % kRingBufs), (uint32_t)(seq / kRingBufs));
    if (!landed) atomicExch(&g_tq_status, (unsigned int)PB_ERR_DEVICE_TIMEOUT);
    const uint8_t* tile = smem + (size_t)(seq % kRingBufs) * kRingTileBytes;
    uint32_t w[32];
    uint32_t cm = 0u;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      w[i] = *reinterpret_cast<const uint32_t*>(tile + (row_first + (i ^ swap)) * 64 + cp * 4);
      const uint32_t a = w[i] & 0x7fff7fffu;
      const __nv_bfloat162 h = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&cm), *reinterpret_cast<const __nv_bfloat162*>(&a));
      cm = *reinterpret_cast<const uint32_t*>(&h);
    }
    uint32_t (*pa)[16] = part_amax[grp * 2 + (local & 1)];
    pa[blk * 4 + quarter][cp] = cm;
    // every thread of the group has moved its part of the tile into registers and published its maxima; the vote
    // makes the whole group leave together if any of its threads gave up waiting
    int give_up;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbarrier.cta.red.or.pred q, %2, 512, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(give_up) : "r"(landed ? 0 : 1), "r"(grp + 1) : "memory");
    if (give_up) break;
    if (gt == 0) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the group's reads of the buffer come before the copy that refills it
      issue(seq + kRingBufs);
    }
    // two levels: the block's amax from its four quarters, then the super-group's from the eight block maxima
    // (12 shared-memory reads per thread instead of 32: the kernel is bound by its integer instructions)
    auto hmax_u32 = [](uint32_t a, uint32_t b) {
      const __nv_bfloat162 h = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
      return *reinterpret_cast<const uint32_t*>(&h);
    };
    const uint32_t mb = hmax_u32(hmax_u32(pa[blk * 4][cp], pa[blk * 4 + 1][cp]), hmax_u32(pa[blk * 4 + 2][cp], pa[blk * 4 + 3][cp]));
    uint32_t (*pb)[16] = block_amax[grp * 2 + (local & 1)];
    if (quarter == 0) pb[blk][cp] = mb;
    asm volatile("barrier.cta.sync %0, 512;" ::"r"(grp + 1) : "memory");
    uint32_t mg = hmax_u32(hmax_u32(pb[0][cp], pb[1][cp]), hmax_u32(pb[2][cp], pb[3][cp]));
    mg = hmax_u32(mg, hmax_u32(hmax_u32(pb[4][cp], pb[5][cp]), hmax_u32(pb[6][cp], pb[7][cp])));
    uint32_t sbv[2]; float D[2];
    block_scale(__uint_as_float(mb << 16), __uint_as_float(mg << 16), sbv[0], D[0]);
    block_scale(__uint_as_float(mb & 0xffff0000u), __uint_as_float(mg & 0xffff0000u), sbv[1], D[1]);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const size_t col = (size_t)z * cols + c0 + 2 * cp + j;
      const size_t grpi = col * nsg + ry;
      if (quarter == 0) {
        sc8[grpi * 8 + blk] = (uint8_t)sbv[j];
        if (blk == 0) sc32[grpi] = j == 0 ? __uint_as_float(mg << 16) : __uint_as_float(mg & 0xffff0000u);
      }
      const float rcp = __frcp_rn(D[j]);
      const float2 nD2 = make_float2(-D[j], -D[j]), r2 = make_float2(rcp, rcp);
      uint32_t out[8];
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        uint32_t o2[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          // rows i+2h and i+2h+1 of column j as one packed bf16 pair (the registers of the upper half-warp hold them swapped)
          const uint32_t pr = __byte_perm(w[i + 2 * h], w[i + 2 * h + 1], j == 0 ? sel0 : sel1);
          const float2 v = div_hoisted_unsigned2(make_float2(__uint_as_float(pr << 16), __uint_as_float(pr & 0xffff0000u)), nD2, r2);
          const uint32_t pk = (pack_bf16x2(v.x, v.y) & 0x7fff7fffu) | (pr & 0x80008000u);
          o2[h] = bf16x2_to_fp8x2<FMT>(pk);
        }
        out[i >> 2] = o2[0] | (o2[1] << 16);
      }
      uint8_t* o = q_t + col * rows + r0 + row_first;
      asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                   ::"l"(o), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]), "r"(out[4]), "r"(out[5]), "r"(out[6]), "r"(out[7]) : "memory");
    }
  }
}

// The same persistent kernel for f32 input (what the reference's model quantizes: its activations are f32).  A tile is
// still 1024 rows of 64 bytes, now 16 f32 columns: a thread keeps 32 rows of ONE column, its maximum is an f32
// maximum, and pairs of rows go through the f32 division straight to a bf16 pair.  Everything else (three TMA-filled
// buffers, two groups of 512 threads, the swapped row pairs of the upper half-warp, the two-level maxima) is as above.
//
// LERP: the token-shift lerp of TimeMix / ChannelMix as a prologue (pratchya/_nnx_impl/_module.py:126-134, 235-237): the
// value quantized is v[r][c] = x[r][c] + (prev[r][c] - x[r][c]) * mu[c] with prev the row before (the carried state for the
// first row of a sequence; sequences are whole tiles long), three roundings as in the op-by-op form.  The row before a
// thread's first row is in the tile, except for the tile's first row, which sixteen threads fetch with a plain load.
//
// RELU2 (LERP == 3): relu(x)^2 on the way to the registers.  SCALE (LERP == 2): the cotangent rule of a (1,128) dequantize as a prologue (dequantize_impl_bwd, _qarr.py:575-601): the value
// quantized is (x[r][c] * x_sc(r, c / 128)) / 128 with x_sc = e8m0(y_sc8) * y_sc32 of another array's (1,128) triple (the forward
// output whose cotangent x is).  A tile's 16 columns lie in one block, so it needs one multiplier per row: the group's
// threads form the 1024 of them in shared memory (rows 128 apart one bank apart) before they read the tile.
struct LerpPrologue {
  const float* x; const float* state; const float* mu; int steps;
  const uint8_t* y_sc8; const float* y_sc32;
};
constexpr int kRingScaleFloats = 1024 + 8;             // one multiplier per tile row, index r + (r >> 7)
constexpr int kRingScaleBytes = 2 * kRingScaleFloats * 4;   // per group

template <int FMT, int LERP>
__global__ void __launch_bounds__(1024, 1)
transpose_quantize1024_f32_ring_kernel(const __grid_constant__ CUtensorMap map_x, uint8_t* __restrict__ q_t, uint8_t* __restrict__ sc8,
                                       float* __restrict__ sc32, int rows, int cols, int tiles_x, int tiles_y, int n_tiles,
                                       const LerpPrologue lerp) {
  extern __shared__ uint8_t ring_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ring_raw) + 1023) & ~(uintptr_t)1023);
  float (*part_amax)[32][16] = reinterpret_cast<float (*)[32][16]>(smem + kRingBufs * kRingTileBytes);   // [group * 2 + parity]
  float (*block_amax)[8][16] = reinterpret_cast<float (*)[8][16]>(smem + kRingBufs * kRingTileBytes + kRingPartBytes);
  const uint32_t s_tiles = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t s_bar = s_tiles + kRingBufs * kRingTileBytes + kRingPartBytes + kRingBlockBytes;
  const int tid = threadIdx.x, grp = tid >> 9, gt = tid & 511;

  if (tid == 0) {
    for (int b = 0; b < kRingBufs; ++b) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_bar + 8u * b));
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(s_bar + 32u + 4u * b), "r"(0u) : "memory");      // fills armed so far
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](int seq) {
    const int tl = blockIdx.x + seq * gridDim.x;
    if (tl >= n_tiles) return;
    const int cx = tl % tiles_x, rest = tl / tiles_x, ry = rest % tiles_y, z = rest / tiles_y;
    const uint32_t bar = s_bar + 8u * (seq % kRingBufs), dst = s_tiles + (uint32_t)(seq % kRingBufs) * kRingTileBytes;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)kRingTileBytes) : "memory");
#pragma unroll
    for (int j = 0; j < 4; ++j)
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                   ::"r"(dst + j * 16384u), "l"(&map_x), "r"(cx * 16), "r"(z * rows + ry * 1024 + j * 256), "r"(bar) : "memory");
    ring_publish_fill(s_bar + 32u + 4u * (seq % kRingBufs), (uint32_t)(seq / kRingBufs));
  };
  if (tid == 0) { issue(0); issue(1); issue(2); }

  const int cp = gt & 15, blk = (gt >> 4) & 7, quarter = gt >> 7;        // cp: the column of the tile this thread owns
  const int row_first = blk * 128 + quarter * 32;
  const int swap = (gt >> 4) & 1;                 // upper half-warp: rows in swapped pairs
  const int nsg = rows >> 10;
  int local = 0;
  uint32_t nb0 = 0, nb1 = 0;                      // SCALE: the e8m0 bytes and fp32 factors of rows gt and gt + 512 of the group's next tile
  float nf0 = 0.0f, nf1 = 0.0f;
  auto fetch_scales = [&](int tile_index) {
    const int cx = tile_index % tiles_x, rest = tile_index / tiles_x, ry = rest % tiles_y, z = rest / tiles_y;
    const int64_t row = (int64_t)z * rows + ry * 1024 + gt;
    const int c0 = cx * 16;
    nb0 = __ldg(lerp.y_sc8 + row * (cols >> 7) + (c0 >> 7));
    nf0 = __ldg(lerp.y_sc32 + row * (cols >> 10) + (c0 >> 10));
    nb1 = __ldg(lerp.y_sc8 + (row + 512) * (cols >> 7) + (c0 >> 7));
    nf1 = __ldg(lerp.y_sc32 + (row + 512) * (cols >> 10) + (c0 >> 10));
  };
  for (int seq = grp; blockIdx.x + seq * (int)gridDim.x < n_tiles; seq += 2, ++local) {
    const int tl = blockIdx.x + seq * gridDim.x;
    const int cx = tl % tiles_x, rest = tl / tiles_x, ry = rest % tiles_y, z = rest / tiles_y;
    const int c0 = cx * 16, r0 = ry * 1024;
    float before = 0.0f, mu_c = 0.0f;             // LERP: the row before the tile's first row (threads of rows 0..31), mu of the column
    float* xs = reinterpret_cast<float*>(smem + kRingBufs * kRingTileBytes + kRingPartBytes + kRingBlockBytes + 64) + grp * kRingScaleFloats;
    if (LERP == 2) {
      // This thread's two multipliers of the tile (rows gt and gt + 512) were fetched while the group's previous tile was being
      // worked on; every thread of the group is past both barriers of that tile, so nobody still reads the old table.
      if (local == 0) fetch_scales(tl);
      xs[gt + (gt >> 7)] = __fmul_rn(e8m0_to_f32(nb0), nf0);
      xs[gt + 512 + ((gt + 512) >> 7)] = __fmul_rn(e8m0_to_f32(nb1), nf1);
      asm volatile("barrier.cta.sync %0, 512;" ::"r"(grp + 1) : "memory");
      const int next = blockIdx.x + (seq + 2) * gridDim.x;
      if (next < n_tiles) fetch_scales(next);       // in flight under this tile's arithmetic
    }
    if (LERP == 1) {
      mu_c = __ldg(lerp.mu + c0 + cp);
      if (row_first == 0) {
        const int64_t row = (int64_t)z * rows + r0;
        if (row % lerp.steps != 0) before = __ldg(lerp.x + (row - 1) * cols + c0 + cp);
        else if (lerp.state) before = __ldg(lerp.state + (row / lerp.steps) * cols + c0 + cp);
      }
    }
    const bool landed = ring_wait_tile(s_bar + 8u * (seq % kRingBufs), s_bar + 32u + 4u * (seq % kRingBufs), (uint32_t)(seq / kRingBufs));
    if (!landed) atomicExch(&g_tq_status, (unsigned int)PB_ERR_DEVICE_TIMEOUT);
    const uint8_t* tile = smem + (size_t)(seq % kRingBufs) * kRingTileBytes;
    float w[32];
    float cm = 0.0f;
    if (LERP == 3) {                              // RELU2: relu(x)^2, ChannelMix's activation, on the way to the registers
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float a = fmaxf(*reinterpret_cast<const float*>(tile + (row_first + (i ^ swap)) * 64 + cp * 4), 0.0f);
        w[i] = __fmul_rn(a, a);
        cm = fmaxf(cm, w[i]);
      }
    } else if (LERP == 2) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int r = row_first + (i ^ swap);
        w[i] = __fmul_rn(__fmul_rn(*reinterpret_cast<const float*>(tile + r * 64 + cp * 4), xs[r + (r >> 7)]), 0.0078125f);
        cm = fmaxf(cm, fabsf(w[i]));
      }
    } else if (LERP == 1) {
      if (row_first != 0) before = *reinterpret_cast<const float*>(tile + (row_first - 1) * 64 + cp * 4);
#pragma unroll
      for (int i = 0; i < 32; i += 2) {           // the two loads of a pair in the half-warp's own order, then rows in their natural order
        const float first = *reinterpret_cast<const float*>(tile + (row_first + (i ^ swap)) * 64 + cp * 4);
        const float second = *reinterpret_cast<const float*>(tile + (row_first + ((i + 1) ^ swap)) * 64 + cp * 4);
        w[i] = swap ? second : first;
        w[i + 1] = swap ? first : second;
      }
#pragma unroll
      for (int i = 31; i > 0; --i) w[i] = __fadd_rn(w[i], __fmul_rn(__fsub_rn(w[i - 1], w[i]), mu_c));
      w[0] = __fadd_rn(w[0], __fmul_rn(__fsub_rn(before, w[0]), mu_c));
#pragma unroll
      for (int i = 0; i < 32; ++i) cm = fmaxf(cm, fabsf(w[i]));
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        w[i] = *reinterpret_cast<const float*>(tile + (row_first + (i ^ swap)) * 64 + cp * 4);
        cm = fmaxf(cm, fabsf(w[i]));
      }
    }
    const int qswap = LERP == 1 ? 0 : swap;       // the lerp prologue leaves the registers in row order
    float (*pa)[16] = part_amax[grp * 2 + (local & 1)];
    pa[blk * 4 + quarter][cp] = cm;
    int give_up;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbarrier.cta.red.or.pred q, %2, 512, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(give_up) : "r"(landed ? 0 : 1), "r"(grp + 1) : "memory");
    if (give_up) break;
    if (gt == 0) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the group's reads of the buffer come before the copy that refills it
      issue(seq + kRingBufs);
    }
    const float mb = fmaxf(fmaxf(pa[blk * 4][cp], pa[blk * 4 + 1][cp]), fmaxf(pa[blk * 4 + 2][cp], pa[blk * 4 + 3][cp]));
    float (*pb)[16] = block_amax[grp * 2 + (local & 1)];
    if (quarter == 0) pb[blk][cp] = mb;
    asm volatile("barrier.cta.sync %0, 512;" ::"r"(grp + 1) : "memory");
    float mg = fmaxf(fmaxf(pb[0][cp], pb[1][cp]), fmaxf(pb[2][cp], pb[3][cp]));
    mg = fmaxf(mg, fmaxf(fmaxf(pb[4][cp], pb[5][cp]), fmaxf(pb[6][cp], pb[7][cp])));
    uint32_t sbv; float D;
    block_scale(mb, mg, sbv, D);
    const size_t col = (size_t)z * cols + c0 + cp;
    const size_t grpi = col * nsg + ry;
    if (quarter == 0) {
      sc8[grpi * 8 + blk] = (uint8_t)sbv;
      if (blk == 0) sc32[grpi] = mg;
    }
    const float rcp = __frcp_rn(D);
    const float2 nD2 = make_float2(-D, -D), r2 = make_float2(rcp, rcp);
    uint32_t out[8];
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      // rows i..i+3 of the column; the registers of the upper half-warp hold each pair of rows swapped
      const uint32_t p0 = div_hoisted_pack2(qswap ? w[i + 1] : w[i], qswap ? w[i] : w[i + 1], nD2, r2);
      const uint32_t p1 = div_hoisted_pack2(qswap ? w[i + 3] : w[i + 2], qswap ? w[i + 2] : w[i + 3], nD2, r2);
      out[i >> 2] = bf16x2_to_fp8x2<FMT>(p0) | (bf16x2_to_fp8x2<FMT>(p1) << 16);
    }
    uint8_t* o = q_t + col * rows + r0 + row_first;
    asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(o), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]), "r"(out[4]), "r"(out[5]), "r"(out[6]), "r"(out[7]) : "memory");
  }
}

template <int FMT, int LERP>
int launch_one_pass_f32_ring(const void* x, uint8_t* q_t, uint8_t* sc8, float* sc32, int64_t batch, int64_t rows, int64_t cols, cudaStream_t st,
                             const LerpPrologue lerp = LerpPrologue{nullptr, nullptr, nullptr, 1, nullptr, nullptr}) {
  using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  EncodeFn encode = reinterpret_cast<EncodeFn>(tensor_map_encoder());
  if (!encode) return fail(PB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)(batch * rows)};
  const cuuint64_t strides[1] = {(cuuint64_t)(cols * 4)};
  const cuuint32_t box[2] = {16, 256};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(x), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PB_ERR_CUDA, "cuTensorMapEncodeTiled (transposed quantizer, f32) failed with CUresult %d", (int)r);
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  PB_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      PB_CUDA_TRY(cudaFuncSetAttribute(transpose_quantize1024_f32_ring_kernel<FMT, LERP>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingSmem + kRingScaleBytes));
      configured[dev] = true;
    }
  }
  const int tiles_x = (int)(cols / 16), tiles_y = (int)(rows / 1024);
  const int64_t n_tiles = (int64_t)tiles_x * tiles_y * batch;
  const int grid = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
  transpose_quantize1024_f32_ring_kernel<FMT, LERP><<<grid, 1024, kRingSmem + kRingScaleBytes, st>>>(map, q_t, sc8, sc32, (int)rows, (int)cols, tiles_x, tiles_y, (int)n_tiles, lerp);
  PB_LAUNCH_CHECK("transpose_quantize1024_f32_ring_kernel");
  return PB_OK;
}

template <int FMT>
int launch_one_pass_bf16_ring(const void* x, uint8_t* q_t, uint8_t* sc8, float* sc32, int64_t batch, int64_t rows, int64_t cols, cudaStream_t st) {
  using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  EncodeFn encode = reinterpret_cast<EncodeFn>(tensor_map_encoder());
  if (!encode) return fail(PB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)(batch * rows)};
  const cuuint64_t strides[1] = {(cuuint64_t)(cols * 2)};
  const cuuint32_t box[2] = {32, 256};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PB_ERR_CUDA, "cuTensorMapEncodeTiled (transposed quantizer) failed with CUresult %d", (int)r);
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  PB_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      PB_CUDA_TRY(cudaFuncSetAttribute(transpose_quantize1024_bf16_ring_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingSmem));
      configured[dev] = true;
    }
  }
  const int tiles_x = (int)(cols / 32), tiles_y = (int)(rows / 1024);
  const int64_t n_tiles = (int64_t)tiles_x * tiles_y * batch;
  const int grid = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
  transpose_quantize1024_bf16_ring_kernel<FMT><<<grid, 1024, kRingSmem, st>>>(map, q_t, sc8, sc32, (int)rows, (int)cols, tiles_x, tiles_y, (int)n_tiles);
  PB_LAUNCH_CHECK("transpose_quantize1024_bf16_ring_kernel");
  return PB_OK;
}

template <typename InT, int FMT>
int launch_one_pass(const void* x, uint8_t* q_t, uint8_t* sc8, float* sc32, int64_t batch, int64_t rows, int64_t cols, cudaStream_t st) {
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  PB_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      PB_CUDA_TRY(cudaFuncSetAttribute(transpose_quantize1024_kernel<InT, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, OnePass<InT>::kSmem));
      configured[dev] = true;
    }
  }
  const dim3 grid((unsigned)(cols / OnePass<InT>::kCols), (unsigned)(rows / 1024), (unsigned)batch);
  transpose_quantize1024_kernel<InT, FMT><<<grid, OnePass<InT>::kThreads, OnePass<InT>::kSmem, st>>>((const InT*)x, q_t, sc8, sc32, (int)rows, (int)cols);
  PB_LAUNCH_CHECK("transpose_quantize1024_kernel");
  return PB_OK;
}

__global__ void __launch_bounds__(256)
transpose_bytes_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int rows, int cols) {
  __shared__ uint8_t tile[kTile][kTile + 4];
  const int r0 = blockIdx.y * kTile, c0 = blockIdx.x * kTile;
  for (int i = threadIdx.x; i < kTile * kTile; i += 256) {
    const int r = i / kTile, c = i % kTile;
    tile[r][c] = (r0 + r < rows && c0 + c < cols) ? src[(size_t)(r0 + r) * cols + c0 + c] : 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kTile * kTile; i += 256) {
    const int c = i / kTile, r = i % kTile;
    if (r0 + r < rows && c0 + c < cols) dst[(size_t)(c0 + c) * rows + r0 + r] = tile[r][c];
  }
}

}  // namespace

// quantize_impl(v^T, (1,128)) of one mix v = x + (prev - x) * mu of the token-shift lerp, straight from x [rows, cols] f32
// (rows and steps multiples of 1024, cols of 16): the persistent f32 kernel with the lerp as its prologue.
int launch_shift_lerp_transposed(const float* x, const float* state, const float* mu, uint8_t* q_t, uint8_t* sc8, float* sc32,
                                 int64_t rows, int64_t steps, int64_t cols, cudaStream_t st) {
  if (rows % 1024 != 0 || steps % 1024 != 0 || cols % 16 != 0 || rows >= (1ll << 31) || (cols / 16) * (rows / 1024) >= (1ll << 31))
    return fail(PB_ERR_UNSUPPORTED, "shift-lerp transposed quantizer: rows=%lld steps=%lld cols=%lld", (long long)rows, (long long)steps, (long long)cols);
  return launch_one_pass_f32_ring<PB_E4M3, 1>(x, q_t, sc8, sc32, 1, rows, cols, st, LerpPrologue{x, state, mu, (int)steps, nullptr, nullptr});
}

// quantize_impl((relu(k)^2)^T, (1,128)) from k [rows, cols] f32 (rows and cols multiples of 1024)
int launch_relu2_transposed(const float* k, uint8_t* q_t, uint8_t* sc8, float* sc32, int64_t rows, int64_t cols, cudaStream_t st) {
  if (rows % 1024 != 0 || cols % 16 != 0 || rows >= (1ll << 31) || (cols / 16) * (rows / 1024) >= (1ll << 31))
    return fail(PB_ERR_UNSUPPORTED, "relu^2 transposed quantizer: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  return launch_one_pass_f32_ring<PB_E4M3, 3>(k, q_t, sc8, sc32, 1, rows, cols, st);
}

// quantize_impl(g'^T, (1,128)) of g' = (g * x_sc) / 128, x_sc from the (1,128) triple (y_sc8, y_sc32) of an array of g's shape
// [rows, cols] (rows a multiple of 1024, cols of 128): the persistent f32 kernel with that scaling as its prologue.
int launch_scaled_transposed(const float* g, const uint8_t* y_sc8, const float* y_sc32, int out_format, uint8_t* q_t, uint8_t* sc8, float* sc32,
                             int64_t rows, int64_t cols, cudaStream_t st) {
  if (rows % 1024 != 0 || cols % 1024 != 0 || rows >= (1ll << 31) || (cols / 16) * (rows / 1024) >= (1ll << 31))
    return fail(PB_ERR_UNSUPPORTED, "scaled transposed quantizer: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  const LerpPrologue pro{nullptr, nullptr, nullptr, 1, y_sc8, y_sc32};
  return out_format == PB_E4M3 ? launch_one_pass_f32_ring<PB_E4M3, 2>(g, q_t, sc8, sc32, 1, rows, cols, st, pro)
                               : launch_one_pass_f32_ring<PB_E5M2, 2>(g, q_t, sc8, sc32, 1, rows, cols, st, pro);
}

// Reads and clears the transposed quantizer's device status word (see pb_gemm_check).
int transposed_status_fetch(unsigned int* out) {
  unsigned int zero = 0;
  PB_CUDA_TRY(cudaMemcpyFromSymbol(out, g_tq_status, sizeof(*out)));
  if (*out != 0) PB_CUDA_TRY(cudaMemcpyToSymbol(g_tq_status, &zero, sizeof(zero)));
  return PB_OK;
}
}  // namespace pb

using namespace pb;

extern "C" size_t pb_quantize_transposed_workspace_size(int64_t batch, int64_t rows, int64_t cols, int b) {
  Geometry g;
  if (batch <= 0 || make_geometry(cols, rows, 1, b, &g) != PB_OK) return 0;
  return (size_t)(batch * g.Nb) * 8;
}

extern "C" int pb_quantize_transposed(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols,
                                      int b, int out_format, void* q_t, uint8_t* sc8, float* sc32,
                                      void* workspace, size_t workspace_bytes, void* stream) {
  if (!x || !q_t || !sc8 || !sc32) return fail(PB_ERR_NULL_POINTER, "pb_quantize_transposed: x, q_t, sc8 and sc32 must be non-null");
  if (batch <= 0) return fail(PB_ERR_BAD_SHAPE, "pb_quantize_transposed: batch=%lld must be positive", (long long)batch);
  if (x_dtype != PB_F32 && x_dtype != PB_BF16) return fail(PB_ERR_BAD_DTYPE, "pb_quantize_transposed: x_dtype %d is neither PB_F32 nor PB_BF16", x_dtype);
  if (out_format != PB_E4M3 && out_format != PB_E5M2) return fail(PB_ERR_BAD_DTYPE, "pb_quantize_transposed: out_format %d is neither PB_E4M3 nor PB_E5M2", out_format);
  Geometry g;   // geometry of x^T: [cols, rows] on (1, b)
  if (int s = make_geometry(cols, rows, 1, b, &g)) return s;
  if (rows > kMaxIndexed || cols > kMaxIndexed || batch > 65535 || rows / b > 65535 || (rows + kTile - 1) / kTile > 65535)
    return fail(PB_ERR_UNSUPPORTED, "pb_quantize_transposed: shape [%lld, %lld, %lld] exceeds the launch limits", (long long)batch, (long long)rows, (long long)cols);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {   // one read of x, no scratch: whole super-groups of x^T inside 1024-row tiles
    const int esz = x_dtype == PB_BF16 ? 2 : 4;
    const int tile_cols = 64 / esz;
    if (b == 128 && rows % 1024 == 0 && cols % tile_cols == 0 && g.K == 8 && rows / 1024 <= 65535 &&
        (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (cols * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(q_t) & 31) == 0) {
      uint8_t* o = static_cast<uint8_t*>(q_t);
      if (x_dtype == PB_BF16) {
        // the persistent TMA-staged form needs every tile's rows inside one slice's 2^31 row range and enough tiles to fill the SMs
        const bool ring = batch * rows < (1ll << 31) && (cols / 32) * (rows / 1024) * batch >= 2 * sm_count() && env_switch("PB_TQ_RING", 1) != 0;
        if (ring)
          return out_format == PB_E4M3 ? launch_one_pass_bf16_ring<PB_E4M3>(x, o, sc8, sc32, batch, rows, cols, st)
                                       : launch_one_pass_bf16_ring<PB_E5M2>(x, o, sc8, sc32, batch, rows, cols, st);
        return out_format == PB_E4M3 ? launch_one_pass_bf16<PB_E4M3>(x, o, sc8, sc32, batch, rows, cols, st)
                                     : launch_one_pass_bf16<PB_E5M2>(x, o, sc8, sc32, batch, rows, cols, st);
      }
      const bool ring32 = batch * rows < (1ll << 31) && (cols / 16) * (rows / 1024) * batch >= 2 * sm_count() && env_switch("PB_TQ_RING", 1) != 0;
      if (ring32)
        return out_format == PB_E4M3 ? launch_one_pass_f32_ring<PB_E4M3, 0>(x, o, sc8, sc32, batch, rows, cols, st)
                                     : launch_one_pass_f32_ring<PB_E5M2, 0>(x, o, sc8, sc32, batch, rows, cols, st);
      return out_format == PB_E4M3 ? launch_one_pass<float, PB_E4M3>(x, o, sc8, sc32, batch, rows, cols, st)
                                   : launch_one_pass<float, PB_E5M2>(x, o, sc8, sc32, batch, rows, cols, st);
    }
  }
  const size_t need = (size_t)(batch * g.Nb) * 8;
  if (!workspace || workspace_bytes < need)
    return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_quantize_transposed: needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 3) return fail(PB_ERR_MISALIGNED, "pb_quantize_transposed: workspace must be 4-byte aligned");
  if (reinterpret_cast<uintptr_t>(x) & 7) return fail(PB_ERR_MISALIGNED, "pb_quantize_transposed: x must be 8-byte aligned");
  uint32_t* amax_bits = static_cast<uint32_t*>(workspace);
  float* divisor = reinterpret_cast<float*>(amax_bits + batch * g.Nb);

  uint8_t* out = static_cast<uint8_t*>(q_t);
  const int vec = x_dtype == PB_BF16 ? 8 : 4;
  const bool fast = b == 128 && cols % (32 * vec) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(q_t) & 31) == 0 && rows % 32 == 0 && cols / 64 <= 65535;
  if (fast) {
    const dim3 ga((unsigned)(cols / (32 * vec)), (unsigned)(rows / 128), (unsigned)batch);
    if (x_dtype == PB_BF16) column_amax128_kernel<__nv_bfloat16><<<ga, 256, 0, st>>>((const __nv_bfloat16*)x, amax_bits, (int)rows, (int)cols);
    else                    column_amax128_kernel<float><<<ga, 256, 0, st>>>((const float*)x, amax_bits, (int)rows, (int)cols);
    PB_LAUNCH_CHECK("column_amax128_kernel");
    if (int s = launch_group_scales(amax_bits, divisor, sc8, sc32, batch * g.M, g.K, st)) return s;
    const dim3 gc((unsigned)(cols / 64), (unsigned)(rows / 128), (unsigned)batch);
    if (x_dtype == PB_BF16) {
      if (out_format == PB_E4M3) transpose_apply128_kernel<__nv_bfloat16, PB_E4M3><<<gc, 256, 0, st>>>((const __nv_bfloat16*)x, divisor, out, (int)rows, (int)cols);
      else                       transpose_apply128_kernel<__nv_bfloat16, PB_E5M2><<<gc, 256, 0, st>>>((const __nv_bfloat16*)x, divisor, out, (int)rows, (int)cols);
    } else {
      if (out_format == PB_E4M3) transpose_apply128_kernel<float, PB_E4M3><<<gc, 256, 0, st>>>((const float*)x, divisor, out, (int)rows, (int)cols);
      else                       transpose_apply128_kernel<float, PB_E5M2><<<gc, 256, 0, st>>>((const float*)x, divisor, out, (int)rows, (int)cols);
    }
    PB_LAUNCH_CHECK("transpose_apply128_kernel");
    return PB_OK;
  }

  const dim3 grid1((unsigned)((cols + 255) / 256), (unsigned)(rows / b), (unsigned)batch);
  if (x_dtype == PB_BF16) column_amax_kernel<__nv_bfloat16><<<grid1, 128, 0, st>>>((const __nv_bfloat16*)x, amax_bits, (int)rows, (int)cols, b);
  else                    column_amax_kernel<float><<<grid1, 128, 0, st>>>((const float*)x, amax_bits, (int)rows, (int)cols, b);
  PB_LAUNCH_CHECK("column_amax_kernel");
  if (int s = launch_group_scales(amax_bits, divisor, sc8, sc32, batch * g.M, g.K, st)) return s;

  const dim3 grid3((unsigned)((cols + kTile - 1) / kTile), (unsigned)((rows + kTile - 1) / kTile), (unsigned)batch);
  if (x_dtype == PB_BF16) {
    if (out_format == PB_E4M3) transpose_apply_kernel<__nv_bfloat16, PB_E4M3><<<grid3, 256, 0, st>>>((const __nv_bfloat16*)x, divisor, out, (int)rows, (int)cols, b);
    else                       transpose_apply_kernel<__nv_bfloat16, PB_E5M2><<<grid3, 256, 0, st>>>((const __nv_bfloat16*)x, divisor, out, (int)rows, (int)cols, b);
  } else {
    if (out_format == PB_E4M3) transpose_apply_kernel<float, PB_E4M3><<<grid3, 256, 0, st>>>((const float*)x, divisor, out, (int)rows, (int)cols, b);
    else                       transpose_apply_kernel<float, PB_E5M2><<<grid3, 256, 0, st>>>((const float*)x, divisor, out, (int)rows, (int)cols, b);
  }
  PB_LAUNCH_CHECK("transpose_apply_kernel");
  return PB_OK;
}

extern "C" int pb_quantize_dual(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols, int out_format,
                                void* q, uint8_t* sc8, float* sc32, void* q_t, uint8_t* sc8_t, float* sc32_t,
                                void* workspace, size_t workspace_bytes, void* stream) {
  if (!x || !q || !sc8 || !sc32 || !q_t || !sc8_t || !sc32_t) return fail(PB_ERR_NULL_POINTER, "pb_quantize_dual: x and the six outputs must be non-null");
  if (batch <= 0) return fail(PB_ERR_BAD_SHAPE, "pb_quantize_dual: batch=%lld must be positive", (long long)batch);
  if (out_format != PB_E4M3 && out_format != PB_E5M2) return fail(PB_ERR_BAD_DTYPE, "pb_quantize_dual: out_format %d is neither PB_E4M3 nor PB_E5M2", out_format);
  if (x_dtype != PB_BF16 && x_dtype != PB_F32) return fail(PB_ERR_BAD_DTYPE, "pb_quantize_dual: x_dtype %d is neither PB_F32 nor PB_BF16", x_dtype);
  Geometry gr, gt;      // x on (1,128) and x^T on (1,128)
  if (int s = make_geometry(rows, cols, 1, 128, &gr)) return s;
  if (int s = make_geometry(cols, rows, 1, 128, &gt)) return s;
  if (x_dtype != PB_BF16 || cols % 1024 != 0 || rows % 128 != 0 || gr.K != 8 || batch > 65535 || rows / 128 > 65535 ||
      rows > kMaxIndexed || cols > kMaxIndexed)
    return fail(PB_ERR_UNSUPPORTED, "pb_quantize_dual: needs bf16 x with rows %% 128 == 0 and cols %% 1024 == 0; use pb_quantize and pb_quantize_transposed");
  if (rows % 1024 == 0 && gt.K == 8) {
    // whole super-groups of x^T inside 1024-row tiles: the transposed side is a single pass of its own
    // (measured a little faster than sharing the row quantizer's pass), and the row side is the plain row quantizer
    if (int s = pb_quantize(x, x_dtype, batch, rows, cols, 1, 128, out_format, q, sc8, sc32, nullptr, 0, stream)) return s;
    return pb_quantize_transposed(x, x_dtype, batch, rows, cols, 128, out_format, q_t, sc8_t, sc32_t, workspace, workspace_bytes, stream);
  }
  const size_t need = (size_t)(batch * gt.Nb) * 8;
  if (!workspace || workspace_bytes < need)
    return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_quantize_dual: needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 3) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7) ||
      (reinterpret_cast<uintptr_t>(q_t) & 31))
    return fail(PB_ERR_MISALIGNED, "pb_quantize_dual: x must be 16-byte, q 8-byte, q_t 32-byte and the workspace 4-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* amax_bits = static_cast<uint32_t*>(workspace);
  float* divisor = reinterpret_cast<float*>(amax_bits + batch * gt.Nb);
  if (int s = launch_row128_colmax(x, out_format, q, sc8, sc32, amax_bits, batch, rows, cols, st)) return s;
  if (int s = launch_group_scales(amax_bits, divisor, sc8_t, sc32_t, batch * gt.M, gt.K, st)) return s;
  const dim3 gc((unsigned)(cols / 64), (unsigned)(rows / 128), (unsigned)batch);
  uint8_t* out = static_cast<uint8_t*>(q_t);
  if (out_format == PB_E4M3) transpose_apply128_kernel<__nv_bfloat16, PB_E4M3><<<gc, 256, 0, st>>>((const __nv_bfloat16*)x, divisor, out, (int)rows, (int)cols);
  else                       transpose_apply128_kernel<__nv_bfloat16, PB_E5M2><<<gc, 256, 0, st>>>((const __nv_bfloat16*)x, divisor, out, (int)rows, (int)cols);
  PB_LAUNCH_CHECK("transpose_apply128_kernel");
  return PB_OK;
}

extern "C" int pb_transpose_bytes(const void* src, int64_t rows, int64_t cols, void* dst, void* stream) {
  if (!src || !dst) return fail(PB_ERR_NULL_POINTER, "pb_transpose_bytes: src and dst must be non-null");
  if (rows <= 0 || cols <= 0 || rows > kMaxIndexed || cols > kMaxIndexed || (rows + kTile - 1) / kTile > 65535)
    return fail(PB_ERR_BAD_SHAPE, "pb_transpose_bytes: bad shape [%lld, %lld]", (long long)rows, (long long)cols);
  const dim3 grid((unsigned)((cols + kTile - 1) / kTile), (unsigned)((rows + kTile - 1) / kTile));
  transpose_bytes_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>((const uint8_t*)src, (uint8_t*)dst, (int)rows, (int)cols);
  PB_LAUNCH_CHECK("transpose_bytes_kernel");
  return PB_OK;
}
