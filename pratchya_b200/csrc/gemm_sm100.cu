// Block-scaled FP8 matmul for sm_100a: tcgen05.mma (kind::mxf8f6f4, block_scale) with TMEM
// accumulators, operands staged by TMA, scale factors staged by bulk copies + tcgen05.cp.
// Replaces the dequantize-then-f32-dot of matmul_impl / matmul_impl_bwd / fp8_matmul_bwd,
// pratchya/_qualia/_qarr.py:605-642, :780-791.
//
// Scale algebra.  A quantized element is q * 2^(e-127) * M / 128 with e the block's e8m0
// byte and M the fp32 amax of its super-group (_qarr.py:562-564).  The power-of-two part is
// exactly what the tensor core's block scaling applies (one ue8m0 factor per row and 32-deep
// K step; the byte of a 128-deep block is simply reused for its four K steps).  The fp32 part
// is constant over aligned runs of P <= 8 k-blocks ("chunks") for every row of both
// operands, so a chunk is accumulated in TMEM by the tensor core and then promoted into fp32
// registers:  acc[m,n] += partial[m,n] * fA[m,chunk] * fB[n,chunk].
//
// One CTA per SM, persistent over output tiles, warp-specialised:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocator + MMA issuer (one elected lane)
//   warps 4..   epilogue warpgroups: TMEM -> registers, chunk promotion, store of D
// (warps 2-3 only fill warpgroup 0, which gives most of its registers to the epilogue.)
// Every wait on an mbarrier is bounded; on expiry the kernel records PB_ERR_DEVICE_TIMEOUT in
// a device status word, all roles leave their loops, TMEM is released and the kernel returns.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

#include "common.cuh"

// The cycle counters, the timing experiments that skip loads or stores, and the fault injection
// of the abort-path test exist only in the diagnostics build (-DPB_DIAGNOSTICS, a second library
// that the tests load by name).  The product library has none of them and reads no switch that
// could change its results.
#ifdef PB_DIAGNOSTICS
#define PB_EPI_SKIP_DRAIN (PROF && p.profile == 3)
#define PB_EPI_SKIP_STORE (PROF && p.profile >= 2)
#else
#define PB_EPI_SKIP_DRAIN false
#define PB_EPI_SKIP_STORE false
#endif

namespace pb {
namespace {

constexpr int BM = 128;        // rows of A per tile (TMEM lanes)
constexpr int BK = 128;        // depth of one pipeline stage = one 128-byte swizzle row
constexpr int UMMA_K = 32;     // depth of one tcgen05.mma for 8-bit operands
constexpr int kMaxChunk = 8;   // k-blocks per promotion at most (1024-deep)
constexpr uint32_t kTmemCols = 512;

// Tile widths.  224 is the default: two 224-column accumulators plus the scale-factor columns fit
// the 512 TMEM columns (two 256-column ones do not), so the epilogue drains one chunk while the
// tensor core fills the next, and a 44 KB stage leaves room for five pipeline stages.
template <int BN>
struct Cfg {
  static_assert(BN == 128 || BN == 224 || BN == 256, "tile width");
  static constexpr int kStages = BN == 128 ? 5 : (BN == 224 ? 4 : 3);
  static constexpr int kAccBufs = BN == 256 ? 1 : 2;
  static constexpr int kEpiWarps = BN == 128 ? 4 : 8;
  static constexpr int kThreads = 128 + 32 * kEpiWarps;   // warpgroup 0: producer, MMA, two idle warps; then the epilogue warpgroups
  static constexpr int kABytes = BM * BK;
  static constexpr int kBBytes = BN * BK;
  static constexpr int kSfbAtoms = (BN + 127) / 128;             // 512-byte scale-factor atoms per B tile
  static constexpr int kSfaBytes = 512;
  static constexpr int kSfbBytes = 512 * kSfbAtoms;
  static constexpr int kSfSlot = kSfaBytes + kSfbBytes;          // one slot holds the atoms of 4 k-blocks
  // Scale-factor slots in shared memory and sets in TMEM, both taken in turn by every fill.  A fill may follow the last one
  // after a single k-block (a 128-deep product has one per tile), and what the producer knows when it refills a slot, and
  // the MMA thread when it overwrites a set, is that the k-blocks kStages and more before have completed: so kStages of each.
  static constexpr int kSfSlots = kStages > 4 ? 8 : 4;
  static constexpr int kSfCols = 12;                             // TMEM columns of one scale-factor set (4 for A, up to 8 for B)
  static constexpr int kSfColBase = kAccBufs * BN;
  static_assert(kSfSlots >= kStages && kSfColBase + kSfSlots * kSfCols <= 512, "scale-factor slots and TMEM budget");
  static constexpr int kOffB = kStages * kABytes;
  static constexpr int kOffSf = kOffB + kStages * kBBytes;
  static constexpr int kOffStore = ((kOffSf + kSfSlots * kSfSlot + 1023) / 1024) * 1024;   // epilogue staging, 4 KB per warp
  static constexpr int kOffBar = kOffStore + kEpiWarps * 4096;
  static constexpr int kNumBars = 2 * kStages + 2 * kAccBufs;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16 + 1024;   // +1024: manual alignment slack
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

__device__ unsigned int g_gemm_status;   // 0, or PB_ERR_DEVICE_TIMEOUT once any bounded wait ran out
// Cycle counters summed over CTAs when GemmParams::profile is set (diagnostics only):
// 0 producer waits for a free stage, 1 MMA waits for a full stage, 2 MMA waits for a drained
// accumulator, 3 epilogue (first warp) waits for an accumulated chunk, 4 epilogue busy,
// 5 CTA lifetime, 6 MMA issue (non-wait), 7 CTAs counted
__device__ unsigned long long g_gemm_prof[16];

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// The same test, letting the hardware park the warp for up to `ns` nanoseconds (it resumes when
// the phase completes): a parked warp does not compete for issue slots with the MMA warp.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the abort flag) when the poll budget ran out.  The
// budget (GemmParams::wait_polls) is a poll count, not a clock: a poll parks the warp for up to
// 2 us, so the default of 2^21 polls gives up after about four seconds at most (tens of
// milliseconds if the hardware never parks the warp), while a healthy wait in this kernel lasts
// microseconds.  Counting keeps the slow path to a handful of registers, which matters in the
// MMA-issuing thread.
constexpr uint32_t kDefaultWaitPolls = 1u << 21;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t polls) {
  // The whole poll loop is one PTX block: the compiler sees a single opaque instruction, so the
  // loops that wait (the MMA issue loop above all) keep their state in registers.
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
      "setp.ne.u32 p, n, n;\n"          // budget exhausted: p = false
      "DONE_%=:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(polls) : "memory");
  if (ok) return true;
  *abort_flag = 1;
  atomicExch(&g_gemm_status, (unsigned int)PB_ERR_DEVICE_TIMEOUT);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_block_scaled(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// the same load, written straight into 32 consecutive floats of an accumulator array
template <int OFF>
__device__ __forceinline__ void tc_ld32f(uint32_t taddr, float (&a)[128]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=f"(a[OFF + 0]), "=f"(a[OFF + 1]), "=f"(a[OFF + 2]), "=f"(a[OFF + 3]), "=f"(a[OFF + 4]), "=f"(a[OFF + 5]), "=f"(a[OFF + 6]), "=f"(a[OFF + 7]),
        "=f"(a[OFF + 8]), "=f"(a[OFF + 9]), "=f"(a[OFF + 10]), "=f"(a[OFF + 11]), "=f"(a[OFF + 12]), "=f"(a[OFF + 13]), "=f"(a[OFF + 14]), "=f"(a[OFF + 15]),
        "=f"(a[OFF + 16]), "=f"(a[OFF + 17]), "=f"(a[OFF + 18]), "=f"(a[OFF + 19]), "=f"(a[OFF + 20]), "=f"(a[OFF + 21]), "=f"(a[OFF + 22]), "=f"(a[OFF + 23]),
        "=f"(a[OFF + 24]), "=f"(a[OFF + 25]), "=f"(a[OFF + 26]), "=f"(a[OFF + 27]), "=f"(a[OFF + 28]), "=f"(a[OFF + 29]), "=f"(a[OFF + 30]), "=f"(a[OFF + 31])
      : "r"(taddr) : "memory");
}
// Four per-column factors through the read-only path, as a volatile instruction: the compiler keeps it
// where it is written.  As a plain load it hoisted every factor of a chunk (up to 128 registers) to the
// top of the drain, on top of the 128 accumulators, and the epilogue spilled.
__device__ __forceinline__ float4 ld_factors(const float* p) {
  float4 v;
  asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
// acc[off .. off+15] += r * fa * fb[column]; `off` is a constant after unrolling.  `uniform`: 1 = one factor for the
// whole tile (s_uni = fa * fb), 2 = one factor per eight adjacent columns, lane l of the warp holding that of the
// warp's column group l in fb8 (a weight on the (128,1) grid), 0 = a factor per column, read from fbp.
__device__ __forceinline__ void promote16(float (&acc)[128], int off, const uint32_t (&r)[16], float fa, float s_uni, const float* fbp, int uniform,
                                          float fb8 = 0.0f) {
  if (uniform == 2) {
    const float s0 = fa * __shfl_sync(0xffffffffu, fb8, off >> 3), s1 = fa * __shfl_sync(0xffffffffu, fb8, (off >> 3) + 1);
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      const float sj = j < 8 ? s0 : s1;
      const float2 v = __ffma2_rn(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), make_float2(sj, sj), make_float2(acc[off + j], acc[off + j + 1]));
      acc[off + j] = v.x; acc[off + j + 1] = v.y;
    }
  } else if (uniform) {
    const float2 s2 = make_float2(s_uni, s_uni);
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      const float2 v = __ffma2_rn(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), s2, make_float2(acc[off + j], acc[off + j + 1]));
      acc[off + j] = v.x; acc[off + j + 1] = v.y;
    }
  } else {
    const float2 fa2 = make_float2(fa, fa);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 fb = ld_factors(fbp + off + 4 * j);
      const float2 t0 = __fmul2_rn(make_float2(__uint_as_float(r[4 * j + 0]), __uint_as_float(r[4 * j + 1])), fa2);
      const float2 t1 = __fmul2_rn(make_float2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])), fa2);
      const float2 v0 = __ffma2_rn(t0, make_float2(fb.x, fb.y), make_float2(acc[off + 4 * j + 0], acc[off + 4 * j + 1]));
      const float2 v1 = __ffma2_rn(t1, make_float2(fb.z, fb.w), make_float2(acc[off + 4 * j + 2], acc[off + 4 * j + 3]));
      acc[off + 4 * j + 0] = v0.x; acc[off + 4 * j + 1] = v0.y; acc[off + 4 * j + 2] = v1.x; acc[off + 4 * j + 3] = v1.y;
    }
  }
}
// A later chunk of a tile: 16-column parts through two alternating 16-register buffers, the load of
// part i+1 in flight under the arithmetic of part i.  128 accumulators + 32 staging registers leave the
// epilogue's 216-register budget with room to spare (with two 32-register buffers the kernel spilled).
// `release` hands the TMEM buffer back as soon as the last load has landed.
template <typename Release>
__device__ __forceinline__ void drain_later_chunk(float (&acc)[128], uint32_t t_addr, bool four_parts, float fa, float s_uni,
                                                  const float* fbp, int uniform, Release&& release, float fb8 = 0.0f) {
  uint32_t r[2][16];
  tc_ld16(t_addr, r[0]);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (j < 6 || four_parts) {
      tc_wait_ld();
      const bool more = j + 1 < 6 || (four_parts && j + 1 < 8);
      if (more) tc_ld16(t_addr + 16 * (j + 1), r[(j + 1) & 1]);
      else release();
      promote16(acc, 16 * j, r[j & 1], fa, s_uni, fbp, uniform, fb8);
    }
  }
}

// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes, 8-row groups
// 1024 bytes apart.  Fields: start >> 4 at [0,14), LBO >> 4 at [16,30) (unused for swizzled
// K-major, set to 1), SBO >> 4 at [32,46), descriptor version 1 at [46,48), layout 2 at [61,64).
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3ffffu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Scale-factor atom: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3ffffu) >> 4) | ((uint64_t)(128 >> 4) << 32) | (1ull << 46);
}
// Instruction descriptor of kind::mxf8f6f4.block_scale: b_sf_id [4,6), a/b format [7,10)/[10,13)
// (0 = e4m3, 1 = e5m2), both operands K-major (bits 15, 16 clear), N >> 3 at [17,23),
// ue8m0 scales (bit 23), M >> 4 at [24,29), a_sf_id [29,31).
__device__ __forceinline__ uint32_t instr_desc(int bn, int a_fmt, int b_fmt, uint32_t sf_id) {
  return (sf_id << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(bn >> 3) << 17) | (1u << 23) |
         ((uint32_t)(BM >> 4) << 24) | (sf_id << 29);
}

// 32-bit forms for the MMA-issuing thread: the upper descriptor word never changes, so only the
// low word (address >> 4, plus the LBO field) is carried and advanced.
constexpr uint32_t kOperandDescHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);   // SBO, version 1, 128-byte swizzle
constexpr uint32_t kSfDescHi = (uint32_t)(128 >> 4) | (1u << 14);                      // SBO, version 1, no swizzle
__device__ __forceinline__ uint32_t operand_desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3ffffu) >> 4) | (1u << 16); }
__device__ __forceinline__ uint32_t sf_desc_lo(uint32_t smem_addr) { return (smem_addr & 0x3ffffu) >> 4; }
__device__ __forceinline__ void tc_cp_sf_lo(uint32_t taddr, uint32_t desc_lo) {
  asm volatile("{\n\t.reg .b64 d;\n\tmov.b64 d, {%1, %2};\n\ttcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n\t}"
               ::"r"(taddr), "r"(desc_lo), "r"(kSfDescHi));
}
__device__ __forceinline__ void tc_mma_block_scaled_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                       uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %7};\n\tmov.b64 db, {%2, %7};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], da, db, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(kOperandDescHi));
}

struct GemmParams {
  const uint8_t* sfa;     // [KG][Mpad/128][512]
  const uint8_t* sfb;     // [KG][Npad/128][512]
  const float* fa;        // [nchunks][Mpad]
  const float* fb;        // [nchunks][Npad]
  void* d;
  int64_t ldd;
  int M, N, KB, P, nchunks;
  int Mpad, Npad;
  int tiles_m, tiles_n;
  int a_fmt, b_fmt;
  int d_dtype;
  int diag;         // diagnostics build only (PB_DIAGNOSTICS), pair kernel: 1 skips the loads of B, 2 those of A, 4 those of the scale
                    // factors (timing experiments); 8 leaves the first pipeline slot unfilled and unarmed, so that every bounded
                    // wait of the launch runs out (the test of the abort path).  Always 0 in the product build.
  int splitk;       // pair kernel: 1, or 2 = each tile's chunks are shared by two work units that add into a zeroed f32 D
  int band;         // pair kernel: tile rows per band; a band's tiles are visited column by column before the next band
  int fb_uniform;   // B's fp32 factor is the same for all rows of B within a chunk (selects the kernel instantiation)
  int fb_groups8;   // ... or the same within aligned runs of eight rows of B (a weight on the (128,1) grid)
  int tma_store;    // D is written through shared memory and TMA stores (needs 16-byte aligned rows)
  int profile;      // diagnostics build only: 1 per-role cycle counters, 2 also no stores of D, 3 also no TMEM reads.  0 in the product build.
  uint32_t wait_polls;   // poll budget of every bounded mbarrier wait
};


// TMA store of a [32 rows x 32 columns] box from shared memory, tracked by this thread's bulk group
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// the same box added to what global memory holds (f32 only)
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N> __device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Stages 32 columns (OFF .. OFF+31) of this lane's row into the warp's staging buffer and lets lane 0
// hand the 32 x 32 box to the TMA.  The buffer is swizzled the way the store's tensor map expects
// (64-byte rows for bf16, 128-byte rows for f32), which also keeps the 16-byte writes of the 32
// lanes on distinct banks.  bf16 alternates between two 2 KB halves; f32 uses the whole 4 KB.
template <int OFF>
__device__ __forceinline__ void stage_and_store(const CUtensorMap* map, const float (&acc)[128], uint32_t stage, int lane,
                                                int d_dtype, int col0, int row0, uint32_t& stores, bool add = false) {
  if (d_dtype == PB_BF16) {
    const uint32_t buf = stage + (stores++ & 1u) * 2048;     // halves alternate over the warp's whole run of stores
    if (lane == 0) tma_store_wait_read<1>();      // the store that last read this half has finished reading
    __syncwarp();
    const uint32_t sw = ((uint32_t)lane >> 1) & 3u;
#pragma unroll
    for (int c = 0; c < 4; ++c)
      st_shared_v4(buf + lane * 64 + (((uint32_t)c ^ sw) << 4),
                   pack_bf16x2(acc[OFF + 8 * c], acc[OFF + 8 * c + 1]), pack_bf16x2(acc[OFF + 8 * c + 2], acc[OFF + 8 * c + 3]),
                   pack_bf16x2(acc[OFF + 8 * c + 4], acc[OFF + 8 * c + 5]), pack_bf16x2(acc[OFF + 8 * c + 6], acc[OFF + 8 * c + 7]));
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) tma_store_2d(map, buf, col0 + OFF, row0);
  } else {
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
    const uint32_t sw = (uint32_t)lane & 7u;
#pragma unroll
    for (int c = 0; c < 8; ++c)
      st_shared_v4(stage + lane * 128 + (((uint32_t)c ^ sw) << 4), __float_as_uint(acc[OFF + 4 * c]), __float_as_uint(acc[OFF + 4 * c + 1]),
                   __float_as_uint(acc[OFF + 4 * c + 2]), __float_as_uint(acc[OFF + 4 * c + 3]));
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      if (add) tma_reduce_add_2d(map, stage, col0 + OFF, row0);
      else tma_store_2d(map, stage, col0 + OFF, row0);
    }
  }
}

__device__ __forceinline__ void st_global_stream_256(void* ptr, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                                     uint32_t e, uint32_t f, uint32_t g, uint32_t h) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(ptr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(e), "r"(f), "r"(g), "r"(h) : "memory");
}

// One thread stores its row segment of `ncols` (96 or 128) output columns (bf16 or f32), clipped to [M, N].
__device__ __forceinline__ void store_row_segment(const GemmParams& p, const float (&acc)[128], int row, int n0, int ncols = 128) {
  if (row >= p.M) return;
  if (p.d_dtype == PB_BF16) {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.d) + (size_t)row * p.ldd + n0;
    const bool vec = ((p.ldd & 15) == 0) && (n0 + ncols <= p.N) && ((reinterpret_cast<uintptr_t>(p.d) & 31) == 0);
    if (vec) {
      // 256-bit streaming stores: every instruction writes whole 32-byte sectors, and the output
      // (larger than L2 for the benchmark shapes) is marked evict-first so that it does not push the
      // operand tiles, which every CTA re-reads, out of L2.
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (16 * j < ncols)
          st_global_stream_256(dst + 16 * j,
                               pack_bf16x2(acc[16 * j], acc[16 * j + 1]), pack_bf16x2(acc[16 * j + 2], acc[16 * j + 3]),
                               pack_bf16x2(acc[16 * j + 4], acc[16 * j + 5]), pack_bf16x2(acc[16 * j + 6], acc[16 * j + 7]),
                               pack_bf16x2(acc[16 * j + 8], acc[16 * j + 9]), pack_bf16x2(acc[16 * j + 10], acc[16 * j + 11]),
                               pack_bf16x2(acc[16 * j + 12], acc[16 * j + 13]), pack_bf16x2(acc[16 * j + 14], acc[16 * j + 15]));
    } else {
#pragma unroll
      for (int j = 0; j < 128; ++j)
        if (j < ncols && n0 + j < p.N) dst[j] = __float2bfloat16_rn(acc[j]);
    }
  } else {
    float* dst = static_cast<float*>(p.d) + (size_t)row * p.ldd + n0;
    const bool vec = ((p.ldd & 7) == 0) && (n0 + ncols <= p.N) && ((reinterpret_cast<uintptr_t>(p.d) & 31) == 0);
    if (vec) {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (8 * j < ncols)
          st_global_stream_256(dst + 8 * j, __float_as_uint(acc[8 * j]), __float_as_uint(acc[8 * j + 1]), __float_as_uint(acc[8 * j + 2]),
                               __float_as_uint(acc[8 * j + 3]), __float_as_uint(acc[8 * j + 4]), __float_as_uint(acc[8 * j + 5]),
                               __float_as_uint(acc[8 * j + 6]), __float_as_uint(acc[8 * j + 7]));
    } else {
#pragma unroll
      for (int j = 0; j < 128; ++j)
        if (j < ncols && n0 + j < p.N) dst[j] = acc[j];
    }
  }
}

template <int BN, bool PROF, bool UNI>
__global__ void __launch_bounds__(Cfg<BN>::kThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_d, const __grid_constant__ GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t s_a = s_base, s_b = s_base + C::kOffB, s_sf = s_base + C::kOffSf, s_bar = s_base + C::kOffBar;
  auto bar_full = [&](int s) { return s_bar + 8u * s; };
  auto bar_empty = [&](int s) { return s_bar + 8u * (C::kStages + s); };
  auto bar_acc_full = [&](int b) { return s_bar + 8u * (2 * C::kStages + b); };
  auto bar_acc_empty = [&](int b) { return s_bar + 8u * (2 * C::kStages + C::kAccBufs + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::kOffBar + C::kNumBars * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int b = 0; b < C::kAccBufs; ++b) { mbar_init(bar_acc_full(b), 1); mbar_init(bar_acc_empty(b), C::kEpiWarps); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const long long t_cta0 = PROF ? clock64() : 0;
  // With eight epilogue warps 384 threads start with 168 registers each; the epilogue needs ~220
  // (128 accumulators + two 32-register load buffers), warpgroup 0 almost none.
  if (warp < 4) {
    if (C::kEpiWarps == 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------- TMA producer
      uint32_t it = 0;   // running stage counter across tiles
      uint32_t sf_fills = 0;
      long long waited = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
        for (int kb = 0; kb < p.KB; ++kb, ++it) {
          const int s = it % C::kStages;
          const long long t0 = PROF ? clock64() : 0;
          if (!mbar_wait(bar_empty(s), ((it / C::kStages) & 1u) ^ 1u, abort_flag, p.wait_polls)) { ok = false; break; }
          if (PROF) waited += clock64() - t0;
          // the scale-factor atom of a stage covers 4 k-blocks: only the first of them carries it
          const bool with_sf = (kb & 3) == 0;
          mbar_arrive_expect_tx(bar_full(s), C::kABytes + C::kBBytes + (with_sf ? C::kSfSlot : 0));
          tma_load_2d(s_a + s * C::kABytes, &map_a, kb * BK, m0, bar_full(s));
          tma_load_2d(s_b + s * C::kBBytes, &map_b, kb * BK, n0, bar_full(s));
          if (with_sf) {
            // The slots are taken in turn.  A slot is rewritten kSfSlots fills, so at least kSfSlots >= kStages k-blocks,
            // after the copy that read it was issued; this fill waited for the commit of k-block it - kStages, which
            // completes only after every earlier tcgen05 operation, that copy included.
            const int kg = kb >> 2;
            const uint32_t slot = s_sf + (sf_fills % C::kSfSlots) * C::kSfSlot;
            ++sf_fills;
            bulk_load(slot, p.sfa + ((size_t)kg * p.tiles_m + tile % p.tiles_m) * 512, C::kSfaBytes, bar_full(s));
            bulk_load(slot + C::kSfaBytes, p.sfb + ((size_t)kg * p.tiles_n + tile / p.tiles_m) * C::kSfbBytes, C::kSfbBytes, bar_full(s));
          }
        }
      }
      // Leave only when every copy this thread started has landed (bounded): the last
      // kStages fills are the ones that can still be in flight.
      const uint32_t issued = it;
      for (uint32_t j = (issued > (uint32_t)C::kStages ? issued - C::kStages : 0); j < issued; ++j)
        (void)mbar_wait(bar_full(j % C::kStages), (j / C::kStages) & 1u, abort_flag, p.wait_polls);
      if (PROF) atomicAdd(&g_gemm_prof[0], (unsigned long long)waited);
    } else if (warp == 1 && lane == 0) {
      // ------------------------------------------------------------- MMA issuer
      // This one thread is the kernel's critical resource.  It runs alone on its scheduler, so
      // every dependent instruction costs its full latency, and a tcgen05.mma takes ~75 cycles to
      // issue: the four of a k-block leave ~200 of the tensor core's 512 cycles for everything
      // else.  Hence: no divisions, 32-bit descriptor arithmetic, incremental stage state.
      const int KB = p.KB, P = p.P, nchunks = p.nchunks;
      const uint32_t idesc0 = instr_desc(BN, p.a_fmt, p.b_fmt, 0u);
      const uint32_t a_lo0 = operand_desc_lo(s_a), b_lo0 = operand_desc_lo(s_b);
      const uint32_t sf_tmem0 = tmem_base + C::kSfColBase;
      uint32_t s = 0, phase = 0;                 // pipeline stage and the parity of its current fill
      uint32_t a_lo = a_lo0, b_lo = b_lo0, full = bar_full(0), empty = bar_empty(0);
      const uint32_t sf_lo0 = sf_desc_lo(s_sf);
      uint32_t sf_reads = 0, sf_col = sf_tmem0;  // scale-factor slots consumed so far; the TMEM set of the current group of four k-blocks
      uint32_t g = 0;                            // chunk counter
      long long wait_full = 0, wait_acc = 0;
      const long long t_begin = PROF ? clock64() : 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int c = 0; c < nchunks && ok; ++c, ++g) {
          const int buf = g % C::kAccBufs;
          long long t0 = PROF ? clock64() : 0;
          if (!mbar_wait(bar_acc_empty(buf), ((g / C::kAccBufs) & 1u) ^ 1u, abort_flag, p.wait_polls)) { ok = false; break; }
          if (PROF) wait_acc += clock64() - t0;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          const int kb_end = min(KB, (c + 1) * P);
          uint32_t accumulate = 0;
          for (int kb = c * P; kb < kb_end; ++kb) {
            if (PROF) t0 = clock64();
            if (!mbar_wait(full, phase, abort_flag, p.wait_polls)) { ok = false; break; }
            if (PROF) wait_full += clock64() - t0;
            // the scale factors of k-blocks 4j..4j+3 go to the TMEM set of their fill; the MMAs that read that set's
            // last contents were kSfSlots fills ago: k-blocks whose commits this stage's producer has waited for
            if ((kb & 3) == 0) {
              const uint32_t turn = sf_reads % C::kSfSlots;
              const uint32_t sf_lo = sf_lo0 + turn * (C::kSfSlot >> 4);
              sf_col = sf_tmem0 + turn * C::kSfCols;
              ++sf_reads;
              tc_cp_sf_lo(sf_col, sf_lo);
#pragma unroll
              for (int j = 0; j < C::kSfbAtoms; ++j) tc_cp_sf_lo(sf_col + 4 + 4 * j, sf_lo + ((C::kSfaBytes + 512 * j) >> 4));
            }
            const uint32_t idesc = idesc0 + ((uint32_t)kb & 3u) * ((1u << 4) | (1u << 29));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              tc_mma_block_scaled_lo(d_tmem, a_lo + (k * UMMA_K >> 4), b_lo + (k * UMMA_K >> 4), idesc, sf_col, sf_col + 4, accumulate);
              accumulate = 1;
            }
            tc_commit(empty);          // frees the stage once these MMAs have read it
            ++s; a_lo += C::kABytes >> 4; b_lo += C::kBBytes >> 4; full += 8; empty += 8;
            if (s == C::kStages) {
              s = 0; phase ^= 1u;
              a_lo = a_lo0; b_lo = b_lo0; full = bar_full(0); empty = bar_empty(0);
            }
          }
          if (ok) tc_commit(bar_acc_full(buf));   // chunk accumulated
        }
      }
      if (PROF) {
        atomicAdd(&g_gemm_prof[1], (unsigned long long)wait_full);
        atomicAdd(&g_gemm_prof[2], (unsigned long long)wait_acc);
        atomicAdd(&g_gemm_prof[6], (unsigned long long)(clock64() - t_begin - wait_full - wait_acc));
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue
    if (C::kEpiWarps == 8) asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int ew = warp - 4;
    const int quarter = warp & 3;             // TMEM lanes this warp may touch
    const int col_half = ew >> 2;             // which column slice of the tile: [0,128) or [128,BN)
    const int ncols = col_half == 0 ? (BN < 128 ? BN : 128) : BN - 128;      // 128, or 96 for the 224-wide tile
    const bool four_parts = ncols == 128;     // 32-column parts this warp drains per chunk (else three)
    const int row_in_tile = quarter * 32 + lane;
    uint32_t g = 0, stores = 0;
    bool ok = true;
    long long wait_chunk = 0;
    const long long t_begin = PROF ? clock64() : 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN + col_half * 128;
      float acc[128];
      for (int c = 0; c < p.nchunks; ++c, ++g) {
        const int buf = g % C::kAccBufs;
        // the chunk's fp32 factors do not depend on the MMAs: fetch them before waiting
        const float fa = __ldg(p.fa + (size_t)c * p.Mpad + m0 + row_in_tile);
        const float* fbp = p.fb + (size_t)c * p.Npad + n0;
        const float s_uni = fa * __ldg(fbp);      // the whole factor when B's fp32 factor does not vary over the tile
        const long long t0 = PROF ? clock64() : 0;
        if (!mbar_wait(bar_acc_full(buf), (g / C::kAccBufs) & 1u, abort_flag, p.wait_polls)) { ok = false; break; }
        if (PROF) wait_chunk += clock64() - t0;
        tc_fence_after();
        const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + col_half * 128;
        auto release = [&]() {
          // all of this warp's reads of the buffer are done: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_acc_empty(buf));
        };
        if (PB_EPI_SKIP_DRAIN) { release(); continue; }      // diagnostics build: handshake only
        if (c == 0) {
          // First chunk of a tile: straight into the accumulator registers, so the buffer goes
          // back to the MMA warp before any arithmetic.
          tc_ld32f<0>(t_addr, acc); tc_ld32f<32>(t_addr + 32, acc); tc_ld32f<64>(t_addr + 64, acc);
          if (four_parts) tc_ld32f<96>(t_addr + 96, acc);
          tc_wait_ld();
          release();
          if (UNI) {
#pragma unroll
            for (int j = 0; j < 128; ++j) acc[j] *= s_uni;
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < 24 || four_parts) {
                const float4 fb = ld_factors(fbp + 4 * j);
                acc[4 * j + 0] = acc[4 * j + 0] * fa * fb.x; acc[4 * j + 1] = acc[4 * j + 1] * fa * fb.y;
                acc[4 * j + 2] = acc[4 * j + 2] * fa * fb.z; acc[4 * j + 3] = acc[4 * j + 3] * fa * fb.w;
              }
            }
          }
        } else {
          drain_later_chunk(acc, t_addr, four_parts, fa, s_uni, fbp, UNI, release);
        }
      }
      if (!ok) break;
      if (PB_EPI_SKIP_STORE) continue;       // diagnostics build: no stores of D
      if (p.tma_store) {
        const uint32_t stage = s_base + C::kOffStore + ew * 4096;
        const int row0 = m0 + quarter * 32;
        stage_and_store<0>(&map_d, acc, stage, lane, p.d_dtype, n0, row0, stores);
        stage_and_store<32>(&map_d, acc, stage, lane, p.d_dtype, n0, row0, stores);
        stage_and_store<64>(&map_d, acc, stage, lane, p.d_dtype, n0, row0, stores);
        if (four_parts) stage_and_store<96>(&map_d, acc, stage, lane, p.d_dtype, n0, row0, stores);
      } else {
        store_row_segment(p, acc, m0 + row_in_tile, n0, ncols);
      }
    }
    if (lane == 0) tma_store_wait_all();          // this thread's stores have left shared memory and are complete
    if (PROF && warp == 4 && lane == 0) {
      atomicAdd(&g_gemm_prof[3], (unsigned long long)wait_chunk);
      atomicAdd(&g_gemm_prof[4], (unsigned long long)(clock64() - t_begin - wait_chunk));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (PROF && threadIdx.x == 0) {
    atomicAdd(&g_gemm_prof[5], (unsigned long long)(clock64() - t_cta0));
    atomicAdd(&g_gemm_prof[7], 1ull);
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ==============================================================================================
// CTA-pair variant: tcgen05.mma.cta_group::2 on 256 x 224 output tiles.  Each CTA of a 2-CTA
// cluster owns 128 rows of the tile (its own TMEM accumulators) and stages its own 128 rows of A
// and its own 112 of the tile's 224 rows of B, so a k-block moves 30 KB from L2 into each SM
// instead of 44 KB: the single-CTA kernel is bound by that L2-to-SM traffic (about 9 TB/s summed
// over the chip at 2.1 PFLOP/s).  The leader CTA (cluster rank 0) issues every MMA and
// scale-factor copy for the pair; all TMA loads of both CTAs complete on the leader's barrier.
struct Cfg2 {
  static constexpr int BN = 224;
  static constexpr int kStages = 6;
  static constexpr int kSlots = kStages / 2;         // the pipeline moves in pairs of stages
  static constexpr int kAccBufs = 2;
  static constexpr int kEpiWarps = 8;
  static constexpr int kThreads = 128 + 32 * kEpiWarps;
  static constexpr int kABytes = BM * BK;            // this CTA's 128 rows of A
  static constexpr int kBBytes = (BN / 2) * BK;      // this CTA's half of the tile's B rows
  static constexpr int kSfaBytes = 512;              // scale factors of this CTA's A rows
  static constexpr int kSfbBytes = 1024;             // scale factors of all 224 B rows (each CTA needs them all)
  static constexpr int kSfSlot = kSfaBytes + kSfbBytes;
  static constexpr int kSfSlots = 4;                 // slots in shared memory and sets in TMEM, taken in turn by every fill (>= kSlots)
  static constexpr int kSfCols = 12;
  static constexpr int kSfColBase = kAccBufs * BN;
  static constexpr int kOffB = kStages * kABytes;
  static constexpr int kOffSf = kOffB + kStages * kBBytes;
  static constexpr int kOffStore = ((kOffSf + kSfSlots * kSfSlot + 1023) / 1024) * 1024;
  static constexpr int kOffBar = kOffStore + kEpiWarps * 4096;
  static constexpr int kNumBars = 2 * kStages + 2 * kAccBufs;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16 + 1024;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
  static_assert(kSfSlots >= kSlots && kSfColBase + kSfSlots * kSfCols <= 512, "scale-factor slots and TMEM budget");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion is signalled on a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc2_commit(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
// one commit that arrives on the barrier at this shared-memory offset in both CTAs of the pair
__device__ __forceinline__ void tc2_commit_both(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc2_cp_sf_lo(uint32_t taddr, uint32_t desc_lo) {
  asm volatile("{\n\t.reg .b64 d;\n\tmov.b64 d, {%1, %2};\n\ttcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d;\n\t}"
               ::"r"(taddr), "r"(desc_lo), "r"(kSfDescHi));
}
__device__ __forceinline__ void tc2_mma_block_scaled_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                        uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %7};\n\tmov.b64 db, {%2, %7};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], da, db, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(kOperandDescHi));
}
// as instr_desc, for the pair: M = 256
__device__ __forceinline__ uint32_t instr_desc_pair(int bn, int a_fmt, int b_fmt, uint32_t sf_id) {
  return (sf_id << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(bn >> 3) << 17) | (1u << 23) |
         ((uint32_t)(256 >> 4) << 24) | (sf_id << 29);
}

// Tile order of the pair kernel.  Tiles are numbered band by band: a band is `p.band` tile rows,
// walked down its tile rows first and then across the tile columns, so that the band's rows of A
// and all of B stay in L2 while the band is worked through (with one band spanning all of M, a
// 32768-row A is evicted between two columns and read from DRAM once per tile column).
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& tm, int& tn) {
  const int per_band = p.band * p.tiles_n;
  const int b = tile / per_band, within = tile - b * per_band;
  const int rows = min(p.band, p.tiles_m - b * p.band);
  tn = within / rows;
  tm = b * p.band + (within - tn * rows);
}

// UNI: how B's fp32 factor varies over a tile's columns within a chunk: 1 = not at all, 2 = in runs of eight adjacent
// columns (a weight on the (128,1) grid, whose chunks are single k-blocks: its drain runs once per k-block, so the
// factors of the next chunk are fetched a chunk ahead and nothing in the drain waits on memory), 0 = per column.
template <bool PROF, int UNI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg2::kThreads, 1)
gemm_tn_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                    const __grid_constant__ CUtensorMap map_d, const __grid_constant__ GemmParams p) {
  using C = Cfg2;
  constexpr int BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t s_a = s_base, s_b = s_base + C::kOffB, s_sf = s_base + C::kOffSf, s_bar = s_base + C::kOffBar;
  auto bar_full = [&](int s) { return s_bar + 8u * s; };                                    // used in the leader only
  auto bar_empty = [&](int s) { return s_bar + 8u * (C::kStages + s); };                    // one set per CTA
  auto bar_acc_full = [&](int b) { return s_bar + 8u * (2 * C::kStages + b); };             // one set per CTA
  auto bar_acc_empty = [&](int b) { return s_bar + 8u * (2 * C::kStages + C::kAccBufs + b); };   // used in the leader only
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::kOffBar + C::kNumBars * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int b = 0; b < C::kAccBufs; ++b) { mbar_init(bar_acc_full(b), 1); mbar_init(bar_acc_empty(b), 2 * C::kEpiWarps); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers are initialised before any remote signal
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;          // 256 x 224 tiles
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  // Work units: a tile, or with p.splitk == 2 one half of a tile's chunks (units 2t and 2t+1 of tile t).
  const int num_units = num_tiles * p.splitk;
  auto unit_chunks = [&](int unit, int& tile, int& c_begin, int& c_end) {
    if (p.splitk == 2) {
      tile = unit >> 1;
      const int half = (p.nchunks + 1) >> 1;
      c_begin = (unit & 1) ? half : 0;
      c_end = (unit & 1) ? p.nchunks : half;
    } else {
      tile = unit; c_begin = 0; c_end = p.nchunks;
    }
  };
  long long life_c0 = 0; unsigned long long life_n0 = 0;
  if (PROF && threadIdx.x == 96) { life_c0 = clock64(); asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(life_n0)); }

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------- TMA producer (both CTAs)
      // The pipeline moves in steps of two k-blocks (one inside a chunk's odd tail): slot q is the
      // stage pair (2q, 2q+1) with one full and one empty barrier.  Half as many waits and commits
      // in the MMA thread, the same bytes in flight.
      uint32_t it = 0, sf_fills = 0;
      bool ok = true;
      long long prod_wait = 0;
      const long long prod_begin = PROF ? clock64() : 0;
      for (int unit = cluster_id; unit < num_units && ok; unit += num_clusters) {
        int tile, c_begin, c_end, tm, tn;
        unit_chunks(unit, tile, c_begin, c_end);
        tile_coords(p, tile, tm, tn);
        const int m0 = tm * 256 + (int)rank * 128;          // this CTA's rows of A and D
        const int nb0 = tn * BN + (int)rank * (BN / 2);     // this CTA's half of the tile's B rows
        for (int c = c_begin; c < c_end && ok; ++c) {
          const int kb_end = min(p.KB, (c + 1) * p.P);
          for (int kb = c * p.P; kb < kb_end; kb += 2, ++it) {
            const int q = it % C::kSlots;
            const long long tw = PROF ? clock64() : 0;
            if (!mbar_wait(bar_empty(q), ((it / C::kSlots) & 1u) ^ 1u, abort_flag, p.wait_polls)) { ok = false; break; }
            if (PROF) prod_wait += clock64() - tw;
            const bool two = kb + 1 < kb_end;
            // a step of two starts at an even k-block: only its first can open a group of four; a unit that starts inside
            // a group (the second half of a split tile) fetches that group's atom too
            const bool with_sf = (kb & 3) == 0 || kb == c_begin * p.P;
            const uint32_t full = map_to_cta(bar_full(q), 0);
            // diagnostics build: the very first slot of the launch is neither armed nor filled, so its barrier
            // never completes, nothing is in flight for it, and every role's bounded wait runs out
            const bool unarmed = PROF && (p.diag & 8) && it == 0;
            const bool ld_a = !(PROF && (p.diag & 2)) && !unarmed, ld_b = !(PROF && (p.diag & 1)) && !unarmed, ld_sf = !(PROF && (p.diag & 4)) && !unarmed;
            if (leader && !unarmed) mbar_arrive_expect_tx(bar_full(q), 2 * ((two ? 2 : 1) * ((ld_a ? C::kABytes : 0) + (ld_b ? C::kBBytes : 0)) + (with_sf && ld_sf ? C::kSfSlot : 0)));
            const int s = 2 * q;
            if (ld_a) tma_load_2d_pair(s_a + s * C::kABytes, &map_a, kb * BK, m0, full);
            if (ld_b) tma_load_2d_pair(s_b + s * C::kBBytes, &map_b, kb * BK, nb0, full);
            if (with_sf && ld_sf) {
              // The slots are taken in turn.  A slot is rewritten kSfSlots fills, so at least kSfSlots >= kSlots steps,
              // after the copy that read it was issued (a 128- or 256-deep product fills at every step); this fill
              // waited for the commit of the step kSlots before this one, which came after that copy in the MMA
              // thread and completes only after every earlier tcgen05 operation of that thread.
              const int kg = kb >> 2;
              const uint32_t slot = s_sf + (sf_fills % C::kSfSlots) * C::kSfSlot;
              ++sf_fills;
              tma_load_2d_pair(slot, &map_sfa, 0, kg * (2 * p.tiles_m) + 2 * tm + (int)rank, full);
              tma_load_2d_pair(slot + C::kSfaBytes, &map_sfb, 0, (kg * p.tiles_n + tn) * 2, full);
            }
            if (two) {
              if (ld_a) tma_load_2d_pair(s_a + (s + 1) * C::kABytes, &map_a, (kb + 1) * BK, m0, full);
              if (ld_b) tma_load_2d_pair(s_b + (s + 1) * C::kBBytes, &map_b, (kb + 1) * BK, nb0, full);
            }
          }
        }
      }
      if (PROF && leader) {      // slots 0 and 3: the producer's time waiting for a free slot, and the rest of its time
        atomicAdd(&g_gemm_prof[0], (unsigned long long)prod_wait);
        atomicAdd(&g_gemm_prof[3], (unsigned long long)(clock64() - prod_begin - prod_wait));
      }
    } else if (warp == 1 && lane == 0 && leader) {
      // ------------------------------------------------------------- MMA issuer (leader CTA only)
      // Issuing is what bounds this kernel: an MMA takes the thread ~72 cycles to issue and the
      // tensor core 112 to run, but a barrier wait costs ~130, a commit ~65 and the three
      // scale-factor copies ~350, during which a short MMA queue runs dry.  Eight MMAs per wait and
      // commit keep enough work queued to cover them.
      const int KB = p.KB, P = p.P, nchunks = p.nchunks;
      const uint32_t idesc0 = instr_desc_pair(BN, p.a_fmt, p.b_fmt, 0u);
      const uint32_t a_lo0 = operand_desc_lo(s_a), b_lo0 = operand_desc_lo(s_b);
      const uint32_t sf_tmem0 = tmem_base + C::kSfColBase;
      const uint32_t sf_lo0 = sf_desc_lo(s_sf);
      uint32_t q = 0, phase = 0, sf_reads = 0, g = 0, sf_col = sf_tmem0;
      uint32_t a_lo = a_lo0, b_lo = b_lo0, full = bar_full(0), empty = bar_empty(0);
      long long wait_full = 0, wait_acc = 0;
      const long long t_begin = PROF ? clock64() : 0;
      bool ok = true;
      for (int unit = cluster_id; unit < num_units && ok; unit += num_clusters) {
        int tile, c_begin, c_end;
        unit_chunks(unit, tile, c_begin, c_end);
        for (int c = c_begin; c < c_end && ok; ++c, ++g) {
          const int buf = g % C::kAccBufs;
          long long t0 = PROF ? clock64() : 0;
          if (!mbar_wait(bar_acc_empty(buf), ((g / C::kAccBufs) & 1u) ^ 1u, abort_flag, p.wait_polls)) { ok = false; break; }
          if (PROF) wait_acc += clock64() - t0;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          const int kb_end = min(KB, (c + 1) * P);
          uint32_t accumulate = 0;
          for (int kb = c * P; kb < kb_end; kb += 2) {
            if (PROF) t0 = clock64();
            if (!mbar_wait(full, phase, abort_flag, p.wait_polls)) { ok = false; break; }
            if (PROF) wait_full += clock64() - t0;
            // A new group of four k-blocks: its scale factors go to the next TMEM set in turn.  The MMAs that read that
            // set's last contents ran kSfSlots fills ago, in steps whose commits this step's producer has waited for
            // (nothing orders a copy behind an earlier MMA by itself).
            if ((kb & 3) == 0 || kb == c_begin * P) {
              const uint32_t turn = sf_reads % C::kSfSlots;
              const uint32_t sf_lo = sf_lo0 + turn * (C::kSfSlot >> 4);
              sf_col = sf_tmem0 + turn * C::kSfCols;
              ++sf_reads;
              tc2_cp_sf_lo(sf_col, sf_lo);
              tc2_cp_sf_lo(sf_col + 4, sf_lo + (C::kSfaBytes >> 4));
              tc2_cp_sf_lo(sf_col + 8, sf_lo + ((C::kSfaBytes + 512) >> 4));
            }
            const uint32_t idesc = idesc0 + ((uint32_t)kb & 3u) * ((1u << 4) | (1u << 29));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              tc2_mma_block_scaled_lo(d_tmem, a_lo + (k * UMMA_K >> 4), b_lo + (k * UMMA_K >> 4), idesc, sf_col, sf_col + 4, accumulate);
              accumulate = 1;
            }
            if (kb + 1 < kb_end) {
              const uint32_t idesc1 = idesc + ((1u << 4) | (1u << 29));
              const uint32_t a1 = a_lo + (C::kABytes >> 4), b1 = b_lo + (C::kBBytes >> 4);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k)
                tc2_mma_block_scaled_lo(d_tmem, a1 + (k * UMMA_K >> 4), b1 + (k * UMMA_K >> 4), idesc1, sf_col, sf_col + 4, 1u);
            }
            tc2_commit_both(empty);     // free the stage pair in both CTAs once these MMAs have read it
            ++q; a_lo += 2 * (C::kABytes >> 4); b_lo += 2 * (C::kBBytes >> 4); full += 8; empty += 8;
            if (q == C::kSlots) {
              q = 0; phase ^= 1u;
              a_lo = a_lo0; b_lo = b_lo0; full = bar_full(0); empty = bar_empty(0);
            }
          }
          if (ok) {
            tc2_commit_both(bar_acc_full(buf));
          }
        }
      }
      if (PROF) {
        atomicAdd(&g_gemm_prof[1], (unsigned long long)wait_full);
        atomicAdd(&g_gemm_prof[2], (unsigned long long)wait_acc);
        atomicAdd(&g_gemm_prof[6], (unsigned long long)(clock64() - t_begin - wait_full - wait_acc));
        atomicAdd(&g_gemm_prof[7], 1ull);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int ew = warp - 4;
    const int quarter = warp & 3;
    const int col_half = ew >> 2;
    const int ncols = col_half == 0 ? 128 : BN - 128;
    const bool four_parts = ncols == 128;
    const int row_in_tile = quarter * 32 + lane;
    uint32_t g = 0, stores = 0;
    bool ok = true;
    const bool add = p.splitk == 2;
    for (int unit = cluster_id; unit < num_units && ok; unit += num_clusters) {
      int tile, c_begin, c_end, tm, tn;
      unit_chunks(unit, tile, c_begin, c_end);
      tile_coords(p, tile, tm, tn);
      const int m0 = tm * 256 + (int)rank * 128, n0 = tn * BN + col_half * 128;
      float acc[128];
      float fa_next = 0.0f, fb8_next = 0.0f, fb8 = 0.0f;
      auto fetch = [&](int c) {       // UNI == 2: this row's factor and this lane's column group's, a chunk ahead
        fa_next = __ldg(p.fa + (size_t)c * p.Mpad + m0 + row_in_tile);
        fb8_next = lane * 8 < ncols ? __ldg(p.fb + (size_t)c * p.Npad + n0 + lane * 8) : 0.0f;
      };
      if (UNI == 2) fetch(c_begin);
      for (int c = c_begin; c < c_end; ++c, ++g) {
        const int buf = g % C::kAccBufs;
        float fa, s_uni = 0.0f;
        const float* fbp = p.fb + (size_t)c * p.Npad + n0;
        if (UNI == 2) {
          fa = fa_next; fb8 = fb8_next;
          if (c + 1 < c_end) fetch(c + 1);
        } else {
          fa = __ldg(p.fa + (size_t)c * p.Mpad + m0 + row_in_tile);
          s_uni = fa * __ldg(fbp);
        }
        // per-column factors of this chunk: new lines every chunk, so ask for them now; the chunk's MMAs
        // are still running and an L2 round trip per 32 columns would otherwise sit inside the drain
        if (UNI == 0 && lane * 32 < ncols) asm volatile("prefetch.global.L1 [%0];" ::"l"(fbp + lane * 32));
        if (!mbar_wait(bar_acc_full(buf), (g / C::kAccBufs) & 1u, abort_flag, p.wait_polls)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + col_half * 128;
        const uint32_t acc_empty_leader = map_to_cta(bar_acc_empty(buf), 0);
        auto release = [&]() {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
        };
        if (PB_EPI_SKIP_DRAIN) { release(); continue; }      // diagnostics build: handshake only
        if (c == c_begin) {
          tc_ld32f<0>(t_addr, acc); tc_ld32f<32>(t_addr + 32, acc); tc_ld32f<64>(t_addr + 64, acc);
          if (four_parts) tc_ld32f<96>(t_addr + 96, acc);
          tc_wait_ld();
          release();
          if (UNI == 2) {
#pragma unroll
            for (int j8 = 0; j8 < 16; ++j8) {
              const float sj = fa * __shfl_sync(0xffffffffu, fb8, j8);
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[8 * j8 + j] *= sj;
            }
          } else if (UNI) {
#pragma unroll
            for (int j = 0; j < 128; ++j) acc[j] *= s_uni;
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < 24 || four_parts) {
                const float4 fb = ld_factors(fbp + 4 * j);
                acc[4 * j + 0] = acc[4 * j + 0] * fa * fb.x; acc[4 * j + 1] = acc[4 * j + 1] * fa * fb.y;
                acc[4 * j + 2] = acc[4 * j + 2] * fa * fb.z; acc[4 * j + 3] = acc[4 * j + 3] * fa * fb.w;
              }
            }
          }
        } else {
          drain_later_chunk(acc, t_addr, four_parts, fa, s_uni, fbp, UNI, release, fb8);
        }
      }
      if (!ok) break;
      if (PB_EPI_SKIP_STORE) continue;       // diagnostics build: no stores of D
      if (p.tma_store) {
        const uint32_t stage = s_base + C::kOffStore + ew * 4096;
        const int row0 = m0 + quarter * 32;
        stage_and_store<0>(&map_d, acc, stage, lane, p.d_dtype, n0, row0, stores, add);
        stage_and_store<32>(&map_d, acc, stage, lane, p.d_dtype, n0, row0, stores, add);
        stage_and_store<64>(&map_d, acc, stage, lane, p.d_dtype, n0, row0, stores, add);
        if (four_parts) stage_and_store<96>(&map_d, acc, stage, lane, p.d_dtype, n0, row0, stores, add);
      } else {
        store_row_segment(p, acc, m0 + row_in_tile, n0, ncols);
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  // Neither CTA may leave (or free TMEM) while its partner can still signal its barriers, read
  // its shared memory or write its TMEM.
  tc_fence_before();
  __syncthreads();
  if (PROF && threadIdx.x == 96 && leader) {       // slots 13-15: this CTA's life in SM cycles and in nanoseconds
    unsigned long long n1; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(n1));
    atomicAdd(&g_gemm_prof[13], (unsigned long long)(clock64() - life_c0));
    atomicAdd(&g_gemm_prof[14], n1 - life_n0);
    atomicAdd(&g_gemm_prof[15], 1ull);
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- scale preparation -----------------------------------------------------------------------
// Rewrites one operand's (sc8, sc32) into what the main kernel consumes:
//   sf[kg][tile][atom][ (r%32)*16 + (r/32)*4 + kb%4 ]   e8m0 byte of (row, kb); kg = kb/4, the row is
//        tile*tile_rows + atom*128 + r with r in [0,128): atoms are relative to the tile's first row
//        (a 224-row tile of B has two atoms, the second one three quarters full)
//   f[chunk][row] = sc32[group of (row, chunk*P)] / 128
struct PrepParams {
  const uint8_t* sc8;
  const float* sc32;
  uint8_t* sf;
  float* f;
  int rows, rows_pad, KB, KG, P, nchunks;
  int tile_rows, tiles, atoms_per_tile;
  int grid_a;        // 1 or 128: rows per block
  int transposed;    // blocks numbered on the [depth, rows] view
  int64_t Ksg;       // blocks per super-group
};

__device__ __forceinline__ int64_t flat_block(const PrepParams& q, int r, int kb) {
  return q.transposed ? (int64_t)kb * (q.rows / q.grid_a) + r / q.grid_a : (int64_t)(r / q.grid_a) * q.KB + kb;
}

__global__ void __launch_bounds__(256) gemm_prep_kernel(PrepParams q) {
  const int atoms_per_kg = q.tiles * q.atoms_per_tile;
  const int64_t n_sf = (int64_t)q.KG * atoms_per_kg * 512;
  const int64_t n_f = (int64_t)q.rows_pad * q.nchunks;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_sf + n_f; i += stride) {
    if (i < n_sf) {
      // i enumerates the destination bytes in order: kg, tile, atom, then the 512 bytes of the atom
      const int within = (int)(i & 511);
      const int64_t atom_global = i >> 9;
      const int kg = (int)(atom_global / atoms_per_kg), rem = (int)(atom_global % atoms_per_kg);
      const int tile = rem / q.atoms_per_tile, atom = rem % q.atoms_per_tile;
      const int local = atom * 128 + ((within >> 2) & 3) * 32 + (within >> 4);
      const int r = tile * q.tile_rows + local;
      const int kb = kg * 4 + (within & 3);
      uint8_t v = 0;
      if (local < q.tile_rows && r < q.rows && kb < q.KB) v = q.sc8[flat_block(q, r, kb)];
      q.sf[i] = v;
    } else {
      const int64_t j = i - n_sf;
      const int r = (int)(j % q.rows_pad), c = (int)(j / q.rows_pad);
      float v = 0.0f;
      if (r < q.rows) v = q.sc32[flat_block(q, r, c * q.P) / q.Ksg] * 0.0078125f;
      q.f[j] = v;
    }
  }
}

// ---- host side -------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() { return reinterpret_cast<EncodeTiledFn>(tensor_map_encoder()); }

// A tensor map is a pure function of its arguments, and a layer calls with the same few (pointer, shape)
// sets step after step: each host thread keeps the last sixteen maps it encoded instead of asking the driver
// for five of them on every launch.
struct MapKey {
  const void* base; cuuint64_t d0, d1, stride; cuuint32_t b0, b1; int type, swizzle, promotion;
  bool operator==(const MapKey& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && stride == o.stride && b0 == o.b0 && b1 == o.b1 && type == o.type &&
           swizzle == o.swizzle && promotion == o.promotion;
  }
};
CUresult encode_cached(EncodeTiledFn fn, CUtensorMap* map, CUtensorMapDataType type, const void* base, const cuuint64_t* dims,
                       const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promotion) {
  struct Entry { MapKey key; CUtensorMap map; bool used; };
  static thread_local Entry cache[16] = {};
  static thread_local int next = 0;
  const MapKey key{base, dims[0], dims[1], strides[0], box[0], box[1], (int)type, (int)swizzle, (int)promotion};
  for (const Entry& e : cache)
    if (e.used && e.key == key) { *map = e.map; return CUDA_SUCCESS; }
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promotion,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) { cache[next] = Entry{key, *map, true}; next = (next + 1) & 15; }
  return r;
}

int make_operand_map(CUtensorMap* map, const void* q, int64_t rows, int64_t depth, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return fail(PB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {(cuuint64_t)depth, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)depth};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const CUresult r = encode_cached(fn, map, CU_TENSOR_MAP_DATA_TYPE_UINT8, q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  if (r != CUDA_SUCCESS) return fail(PB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return PB_OK;
}

// D as a 2-D tensor [M, N] for the epilogue's TMA stores: boxes of 32 rows x 32 columns, swizzled
// like the staging buffers (64-byte rows for bf16, 128-byte rows for f32).
int make_store_map(CUtensorMap* map, void* d, int d_dtype, int64_t M, int64_t N, int64_t ldd) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return fail(PB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const int es = d_dtype == PB_BF16 ? 2 : 4;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)(ldd * es)};
  const cuuint32_t box[2] = {32, 32};
  const CUresult r = encode_cached(fn, map, d_dtype == PB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, d, dims,
                                   strides, box, d_dtype == PB_BF16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_NONE);
  if (r != CUDA_SUCCESS) return fail(PB_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
  return PB_OK;
}

// Scale-factor atoms as a 2-D tensor of 32-bit words: [atoms, 128 words]; a box is `atoms_per_box` atoms.
int make_sf_map(CUtensorMap* map, const void* sf, int64_t atoms, int atoms_per_box) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return fail(PB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {128, (cuuint64_t)atoms};
  const cuuint64_t strides[1] = {512};
  const cuuint32_t box[2] = {128, (cuuint32_t)atoms_per_box};
  const CUresult r = encode_cached(fn, map, CU_TENSOR_MAP_DATA_TYPE_UINT32, sf, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE,
                                   CU_TENSOR_MAP_L2_PROMOTION_NONE);
  if (r != CUDA_SUCCESS) return fail(PB_ERR_CUDA, "cuTensorMapEncodeTiled (scale factors) failed with CUresult %d", (int)r);
  return PB_OK;
}

struct OperandPlan {
  int64_t Ksg, Mgroups;
  int P;      // largest run of k-blocks with a constant fp32 factor for every row
  bool row_uniform;   // the fp32 factor of a chunk is the same for every row of the operand
  bool row_groups8;   // ... or for aligned runs of eight rows: blocks of one row each, eight to a super-group (a (128,1) weight)
};

int plan_operand(const pb_operand* o, const char* name, OperandPlan* plan) {
  if (!o->q || !o->sc8 || !o->sc32) return fail(PB_ERR_NULL_POINTER, "pb_gemm_tn: operand %s has a null pointer", name);
  if (o->rows <= 0 || o->depth <= 0 || o->depth % BK != 0)
    return fail(PB_ERR_BAD_SHAPE, "pb_gemm_tn: operand %s is [%lld, %lld]; depth must be a positive multiple of 128", name,
                (long long)o->rows, (long long)o->depth);
  if (!((o->grid_a == 1 || o->grid_a == 128) && o->grid_b == 128))
    return fail(PB_ERR_BAD_GRID, "pb_gemm_tn: operand %s grid (%d,%d) is neither (1,128) nor (128,128)", name, o->grid_a, o->grid_b);
  if (o->format != PB_E4M3 && o->format != PB_E5M2) return fail(PB_ERR_BAD_DTYPE, "pb_gemm_tn: operand %s format %d", name, o->format);
  if (o->grid_a == 128 && o->rows % 128 != 0)
    return fail(PB_ERR_BAD_SHAPE, "pb_gemm_tn: operand %s rows=%lld not divisible by its 128-row blocks", name, (long long)o->rows);
  if (reinterpret_cast<uintptr_t>(o->q) & 15) return fail(PB_ERR_MISALIGNED, "pb_gemm_tn: operand %s bytes must be 16-byte aligned", name);
  if (o->rows > (1ll << 30) || o->depth > (1ll << 30)) return fail(PB_ERR_UNSUPPORTED, "pb_gemm_tn: operand %s is too large", name);
  Geometry g;
  // the scales were produced on the [rows, depth] view, or on its transpose [depth, rows], where the same blocks
  // are (128, grid_a): a (128,128) weight, or a (128,1) weight (one scale per column and 128-deep block)
  const int s = o->transposed_blocks ? make_geometry(o->depth, o->rows, 128, o->grid_a, &g) : make_geometry(o->rows, o->depth, o->grid_a, 128, &g);
  if (s) return s;
  plan->Ksg = g.K;
  plan->Mgroups = g.M;
  const int64_t KB = o->depth / BK;
  int P = kMaxChunk;
  if (g.M > 1) {
    if (!o->transposed_blocks) {
      P = (int)std::gcd((int64_t)kMaxChunk, std::gcd(g.K, KB));
    } else {
      const int64_t nbc = o->rows / o->grid_a;
      P = 1;
      for (int c = kMaxChunk; c > 1; c >>= 1)
        if (g.K % (c * nbc) == 0) { P = c; break; }
    }
  }
  plan->P = P;
  // one super-group in all, or blocks numbered along the rows first with whole block-rows per
  // super-group: every row then sees the same fp32 amax in a given k-block
  plan->row_uniform = (g.M == 1) || (o->transposed_blocks && g.K % (o->rows / o->grid_a) == 0);
  plan->row_groups8 = !plan->row_uniform && o->transposed_blocks && o->grid_a == 1 && g.K == 8 && o->rows % 8 == 0;
  return PB_OK;
}

struct GemmPlan {
  OperandPlan pa, pb;
  int P, KB, KG, nchunks, Mpad, Npad, BN;
  int tiles_m, tiles_n, atoms_b;      // A tiles of 128 rows, B tiles of BN rows, scale-factor atoms per B tile
  bool pair;      // CTA-pair kernel (256 x 256 tiles) instead of the single-CTA one
  size_t off_sfa, off_sfb, off_fa, off_fb, total;
};

bool pick_pair() {      // the CTA-pair kernel is the default; PB_GEMM_SINGLE=1 selects the single-CTA one
  static const bool pair = env_switch("PB_GEMM_SINGLE", 0) == 0;
  return pair;
}

int pick_bn() {      // PB_GEMM_BN=128|224|256: tile width of the single-CTA kernel
  static const int bn = [] { const int v = env_switch("PB_GEMM_BN", 224); return (v == 128 || v == 256) ? v : 224; }();
  return bn;
}

#ifdef PB_DIAGNOSTICS
std::atomic<int> g_diag_bits{-1};                       // -1: take PB_GEMM_DIAG from the environment
std::atomic<uint32_t> g_wait_polls{kDefaultWaitPolls};
int profile_level() {   // 0 off, 1 per-role cycle counters; 2 also skips the stores of D, 3 also the TMEM reads (timing only)
  static const int level = env_switch("PB_GEMM_PROFILE", 0);
  return level;
}
int diag_bits() {
  const int forced = g_diag_bits.load();
  if (forced >= 0) return forced;
  static const int env = env_switch("PB_GEMM_DIAG", 0);
  return env;
}
uint32_t wait_polls() { return g_wait_polls.load(); }
#else
constexpr int profile_level() { return 0; }
constexpr int diag_bits() { return 0; }
constexpr uint32_t wait_polls() { return kDefaultWaitPolls; }
#endif

int make_plan(const pb_operand* a, const pb_operand* b, GemmPlan* gp) {
  if (!a || !b) return fail(PB_ERR_NULL_POINTER, "pb_gemm_tn: operands must be non-null");
  if (int s = plan_operand(a, "A", &gp->pa)) return s;
  if (int s = plan_operand(b, "B", &gp->pb)) return s;
  if (a->depth != b->depth)
    return fail(PB_ERR_BAD_SHAPE, "pb_gemm_tn: contraction lengths differ (%lld vs %lld)", (long long)a->depth, (long long)b->depth);
  gp->pair = pick_pair() && a->rows > 128;
  gp->BN = gp->pair ? Cfg2::BN : pick_bn();
  gp->P = gp->pa.P < gp->pb.P ? gp->pa.P : gp->pb.P;
  gp->KB = (int)(a->depth / BK);
  if (gp->P > gp->KB) gp->P = gp->KB;
  gp->KG = (gp->KB + 3) / 4;
  gp->nchunks = (gp->KB + gp->P - 1) / gp->P;
  gp->Mpad = (int)((a->rows + 255) / 256 * 256);
  gp->tiles_m = gp->Mpad / 128;
  gp->tiles_n = (int)((b->rows + gp->BN - 1) / gp->BN);
  gp->atoms_b = (gp->BN + 127) / 128;
  gp->Npad = (gp->tiles_n * gp->BN + 255) / 256 * 256;
  auto align = [](size_t v) { return (v + 255) & ~(size_t)255; };
  size_t off = 0;
  gp->off_sfa = off; off = align(off + (size_t)gp->KG * gp->tiles_m * 512);
  gp->off_sfb = off; off = align(off + (size_t)gp->KG * gp->tiles_n * gp->atoms_b * 512);
  gp->off_fa = off;  off = align(off + (size_t)gp->nchunks * gp->Mpad * 4);
  gp->off_fb = off;  off = align(off + (size_t)gp->nchunks * gp->Npad * 4);
  gp->total = off;
  return PB_OK;
}

int launch_prep(const pb_operand* o, const OperandPlan& op, const GemmPlan& gp, int rows_pad, int tile_rows, int tiles, int atoms_per_tile,
                uint8_t* sf, float* f, cudaStream_t st) {
  PrepParams q{o->sc8, o->sc32, sf, f, (int)o->rows, rows_pad, gp.KB, gp.KG, gp.P, gp.nchunks, tile_rows, tiles, atoms_per_tile,
               o->grid_a, o->transposed_blocks, op.Ksg};
  const int64_t items = (int64_t)gp.KG * tiles * atoms_per_tile * 512 + (int64_t)rows_pad * gp.nchunks;
  const int64_t need = (items + 255) / 256;
  const int grid = (int)(need < (int64_t)sm_count() * 8 ? need : (int64_t)sm_count() * 8);
  gemm_prep_kernel<<<grid, 256, 0, st>>>(q);
  PB_LAUNCH_CHECK("gemm_prep_kernel");
  return PB_OK;
}

template <int BN, bool PROF, bool UNI>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, const GemmParams& p, cudaStream_t st) {
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  PB_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      PB_CUDA_TRY(cudaFuncSetAttribute(gemm_tn_kernel<BN, PROF, UNI>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmemBytes));
      configured[dev] = true;
    }
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_tn_kernel<BN, PROF, UNI><<<grid, Cfg<BN>::kThreads, Cfg<BN>::kSmemBytes, st>>>(ma, mb, md, p);
  PB_LAUNCH_CHECK("gemm_tn_kernel");
  return PB_OK;
}
template <int BN, bool PROF>
int launch_gemm_uni(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, const GemmParams& p, cudaStream_t st) {
  return p.fb_uniform ? launch_gemm<BN, PROF, true>(ma, mb, md, p, st) : launch_gemm<BN, PROF, false>(ma, mb, md, p, st);
}

template <bool PROF, int UNI>
int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& msfa, const CUtensorMap& msfb,
                     const CUtensorMap& md, const GemmParams& p, cudaStream_t st) {
  static std::mutex mu;
  static bool configured[64] = {false};
  int dev = 0;
  PB_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      PB_CUDA_TRY(cudaFuncSetAttribute(gemm_tn_pair_kernel<PROF, UNI>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg2::kSmemBytes));
      configured[dev] = true;
    }
  }
  const int tiles = p.tiles_m * p.tiles_n * p.splitk;
  const int pairs = sm_count() / 2;
  const int grid = 2 * (tiles < pairs ? tiles : pairs);
  gemm_tn_pair_kernel<PROF, UNI><<<grid, Cfg2::kThreads, Cfg2::kSmemBytes, st>>>(ma, mb, msfa, msfb, md, p);
  PB_LAUNCH_CHECK("gemm_tn_pair_kernel");
  return PB_OK;
}
template <bool PROF>
int launch_gemm_pair_uni(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& msfa, const CUtensorMap& msfb,
                         const CUtensorMap& md, const GemmParams& p, cudaStream_t st) {
  if (p.fb_uniform) return launch_gemm_pair<PROF, 1>(ma, mb, msfa, msfb, md, p, st);
  return p.fb_groups8 ? launch_gemm_pair<PROF, 2>(ma, mb, msfa, msfb, md, p, st) : launch_gemm_pair<PROF, 0>(ma, mb, msfa, msfb, md, p, st);
}

}  // namespace

// Where the A operand's prepared scales live inside the workspace of the GEMM (a x b): used by
// the row quantizer that writes them directly.  The quantizer covers one super-group of eight
// k-blocks per warp, so the plan must promote in chunks of eight.
int gemm_a_prep_location(const pb_operand* a, const pb_operand* b, void* workspace, size_t workspace_bytes,
                         uint8_t** sf, float** f, uint32_t* tiles, uint32_t* Mpad, void* stream) {
  GemmPlan gp;
  if (int s = make_plan(a, b, &gp)) return s;
  if (gp.P != kMaxChunk)
    return fail(PB_ERR_UNSUPPORTED, "pb_quantize_for_gemm: this operand pair promotes every %d k-blocks, the fused preparation needs %d", gp.P, kMaxChunk);
  if (!workspace || workspace_bytes < gp.total)
    return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_quantize_for_gemm: needs %zu bytes of GEMM workspace, got %zu", gp.total, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(PB_ERR_MISALIGNED, "pb_quantize_for_gemm: workspace must be 256-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  if (gp.Mpad != a->rows) {      // rows of padding are never written by the quantizer: give them zeros
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PB_CUDA_TRY(cudaMemsetAsync(ws + gp.off_sfa, 0, (size_t)gp.KG * gp.tiles_m * 512, st));
    PB_CUDA_TRY(cudaMemsetAsync(ws + gp.off_fa, 0, (size_t)gp.nchunks * gp.Mpad * 4, st));
  }
  *sf = ws + gp.off_sfa;
  *f = reinterpret_cast<float*>(ws + gp.off_fa);
  *tiles = (uint32_t)gp.tiles_m;
  *Mpad = (uint32_t)gp.Mpad;
  return PB_OK;
}
}  // namespace pb

using namespace pb;

extern "C" size_t pb_gemm_workspace_size(const pb_operand* a, const pb_operand* b) {
  GemmPlan gp;
  if (make_plan(a, b, &gp) != PB_OK) return 0;
  return gp.total;
}

extern "C" int pb_gemm_tn(const pb_operand* a, const pb_operand* b, void* d, int d_dtype, int64_t ldd,
                          void* workspace, size_t workspace_bytes, void* stream) {
  return pb_gemm_tn_ex(a, b, d, d_dtype, ldd, workspace, workspace_bytes, 0u, stream);
}

extern "C" int pb_gemm_tn_ex(const pb_operand* a, const pb_operand* b, void* d, int d_dtype, int64_t ldd,
                             void* workspace, size_t workspace_bytes, unsigned int flags, void* stream) {
  GemmPlan gp;
  if (int s = make_plan(a, b, &gp)) return s;
  if (flags & ~(unsigned)(PB_GEMM_A_PREPARED | PB_GEMM_B_PREPARED))
    return fail(PB_ERR_UNSUPPORTED, "pb_gemm_tn_ex: unknown flag bits 0x%x", flags);
  if ((flags & PB_GEMM_A_PREPARED) && gp.P != kMaxChunk)
    return fail(PB_ERR_UNSUPPORTED, "pb_gemm_tn_ex: PB_GEMM_A_PREPARED needs a plan that promotes every %d k-blocks (this one: %d)", kMaxChunk, gp.P);
  if (!d) return fail(PB_ERR_NULL_POINTER, "pb_gemm_tn: d must be non-null");
  if (d_dtype != PB_F32 && d_dtype != PB_BF16) return fail(PB_ERR_BAD_DTYPE, "pb_gemm_tn: d_dtype %d is neither PB_F32 nor PB_BF16", d_dtype);
  if (ldd < b->rows) return fail(PB_ERR_BAD_SHAPE, "pb_gemm_tn: ldd=%lld is smaller than N=%lld", (long long)ldd, (long long)b->rows);
  if (!workspace || workspace_bytes < gp.total)
    return fail(PB_ERR_WORKSPACE_TOO_SMALL, "pb_gemm_tn: needs %zu bytes of workspace, got %zu", gp.total, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(PB_ERR_MISALIGNED, "pb_gemm_tn: workspace must be 256-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);

  if (!(flags & PB_GEMM_A_PREPARED))
    if (int s = launch_prep(a, gp.pa, gp, gp.Mpad, 128, gp.tiles_m, 1, ws + gp.off_sfa, reinterpret_cast<float*>(ws + gp.off_fa), st)) return s;
  if (!(flags & PB_GEMM_B_PREPARED))
    if (int s = launch_prep(b, gp.pb, gp, gp.Npad, gp.BN, gp.tiles_n, gp.atoms_b, ws + gp.off_sfb, reinterpret_cast<float*>(ws + gp.off_fb), st)) return s;

  CUtensorMap ma, mb;
  if (int s = make_operand_map(&ma, a->q, a->rows, a->depth, BM)) return s;
  if (int s = make_operand_map(&mb, b->q, b->rows, b->depth, gp.pair ? Cfg2::BN / 2 : gp.BN)) return s;

  GemmParams p;
  p.sfa = ws + gp.off_sfa; p.sfb = ws + gp.off_sfb;
  p.fa = reinterpret_cast<const float*>(ws + gp.off_fa); p.fb = reinterpret_cast<const float*>(ws + gp.off_fb);
  p.d = d; p.ldd = ldd;
  p.M = (int)a->rows; p.N = (int)b->rows; p.KB = gp.KB; p.P = gp.P; p.nchunks = gp.nchunks;
  p.Mpad = gp.Mpad; p.Npad = gp.Npad;
  p.tiles_m = gp.pair ? gp.Mpad / 256 : gp.tiles_m; p.tiles_n = gp.tiles_n;
  p.a_fmt = a->format; p.b_fmt = b->format; p.d_dtype = d_dtype;
  p.fb_uniform = gp.pb.row_uniform ? 1 : 0;
  p.fb_groups8 = gp.pb.row_groups8 ? 1 : 0;
  {
    // band height: about 16 MB of A rows (they and B, at most a few tens of MB, then share the 126 MB L2 with the stream of D)
    static const int forced = env_switch("PB_GEMM_BAND", 0);
    int band = (int)((16ll << 20) / (256 * a->depth));
    if (forced > 0) band = forced;
    if (band < 4) band = 4;
    if (band > p.tiles_m) band = p.tiles_m;
    p.band = band;
  }
  p.tma_store = 0;
  p.splitk = 1;
  p.profile = profile_level();
  p.diag = diag_bits();
  p.wait_polls = wait_polls();
  // D goes out through TMA stores when its rows are 16-byte aligned; otherwise by direct stores
  CUtensorMap md = ma;
  const int es = d_dtype == PB_BF16 ? 2 : 4;
  p.tma_store = ((reinterpret_cast<uintptr_t>(d) & 15) == 0 && (ldd * es) % 16 == 0) ? 1 : 0;
  if (p.tma_store) {
    if (int s = make_store_map(&md, d, d_dtype, a->rows, b->rows, ldd)) return s;
  }
  if (gp.pair) {
    // Few tiles for the 74 CTA pairs (a 2048 x 2048 weight gradient is 80): give each tile's chunks to
    // two work units that add their halves into D.  Needs f32 output through TMA (the reduction is
    // an f32 TMA add into zeros, so the two orders give the same bits) and at least two chunks a half.
    static const int split_env = env_switch("PB_GEMM_SPLITK", 0);
    const int pairs = sm_count() / 2, tiles = p.tiles_m * p.tiles_n;
    auto efficiency = [&](int units) { return (double)units / (double)(((units + pairs - 1) / pairs) * pairs); };
    bool split = d_dtype == PB_F32 && p.tma_store && gp.nchunks >= 4 && efficiency(tiles) < 0.8 && efficiency(2 * tiles) > efficiency(tiles) + 0.1;
    if (split_env == 1) split = false;
    if (split_env == 2) split = d_dtype == PB_F32 && p.tma_store && gp.nchunks >= 2;
    if (split) {
      p.splitk = 2;
      PB_CUDA_TRY(cudaMemset2DAsync(d, (size_t)ldd * 4, 0, (size_t)b->rows * 4, (size_t)a->rows, st));
    }
    CUtensorMap msfa, msfb;
    if (int s = make_sf_map(&msfa, ws + gp.off_sfa, (int64_t)gp.KG * gp.tiles_m, 1)) return s;
    if (int s = make_sf_map(&msfb, ws + gp.off_sfb, (int64_t)gp.KG * gp.tiles_n * 2, 2)) return s;
#ifdef PB_DIAGNOSTICS
    if (p.profile || p.diag) return launch_gemm_pair_uni<true>(ma, mb, msfa, msfb, md, p, st);
#endif
    return launch_gemm_pair_uni<false>(ma, mb, msfa, msfb, md, p, st);
  }
#ifdef PB_DIAGNOSTICS
  if (p.profile) {
    if (gp.BN == 224) return launch_gemm_uni<224, true>(ma, mb, md, p, st);
    return gp.BN == 256 ? launch_gemm_uni<256, true>(ma, mb, md, p, st) : launch_gemm_uni<128, true>(ma, mb, md, p, st);
  }
  if (gp.BN == 256) return launch_gemm_uni<256, false>(ma, mb, md, p, st);
  if (gp.BN == 128) return launch_gemm_uni<128, false>(ma, mb, md, p, st);
#endif
  return launch_gemm_uni<224, false>(ma, mb, md, p, st);
}

namespace pb { int transposed_status_fetch(unsigned int* out); }   // transpose_quantize.cu

extern "C" int pb_gemm_check(void* stream) {
  PB_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  unsigned int v = 0, zero = 0;
  PB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(v)));
  if (v != 0) {
    PB_CUDA_TRY(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(zero)));
    return fail((int)v, "a bounded device-side wait in the GEMM kernel ran out");
  }
  if (int s = transposed_status_fetch(&v)) return s;
  if (v != 0) return fail((int)v, "a bounded device-side wait in the transposed quantizer ran out");
  return PB_OK;
}

#ifdef PB_DIAGNOSTICS
// Diagnostics build only (not part of the reference's surface, not in the product library).
// Copies (and clears) the sixteen cycle counters the GEMM kernels accumulate under PB_GEMM_PROFILE=1.
extern "C" PB_API int pb_debug_gemm_profile(unsigned long long* out16, void* stream) {
  if (!out16) return fail(PB_ERR_NULL_POINTER, "pb_debug_gemm_profile: out16 must be non-null");
  PB_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  unsigned long long zero[16] = {0};
  PB_CUDA_TRY(cudaMemcpyFromSymbol(out16, g_gemm_prof, sizeof(zero)));
  PB_CUDA_TRY(cudaMemcpyToSymbol(g_gemm_prof, zero, sizeof(zero)));
  return PB_OK;
}
// Sets the poll budget of the bounded waits (0 restores the default) and the diagnostic bits of
// GemmParams::diag (-1 hands them back to the environment) for the launches that follow.
extern "C" PB_API int pb_debug_gemm_control(unsigned int polls, int diag) {
  g_wait_polls.store(polls ? polls : kDefaultWaitPolls);
  g_diag_bits.store(diag);
  return PB_OK;
}
#endif
