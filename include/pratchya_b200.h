/*
 * pratchya_b200 -- C ABI of the sm_100a implementation of pratchya's FP8
 * block-quantization path (quantize / dequantize / block-scaled FP8 matmul).
 *
 * The reference has no FFI: its ops are jitted Python functions in
 * pratchya/_qualia/_qarr.py.  Each entry point below names the reference
 * function it replaces; a JAX host binds them as jax.ffi custom calls, the
 * bundled Python host binds them with ctypes.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller unless stated;
 *   - `stream` is a cudaStream_t passed as void*; calls are asynchronous on it,
 *     never synchronise the host and never touch the default stream;
 *   - the library allocates nothing: scratch memory is a caller buffer whose
 *     size the matching *_workspace_size() call returns;
 *   - every function returns a pb_status; pb_last_error() gives the text of
 *     the calling thread's last failure.  No C++ exception crosses this ABI.
 *
 * Quantized triple of an array x[batch, rows, cols] on grid (a, b)
 * (identical to the reference's (value, sc_fp8, sc_fp32), _qarr.py:500-506):
 *   q    : uint8  [batch, rows, cols]   fp8 bytes (e4m3fn, or e5m2 extension)
 *   sc8  : uint8  [batch, M, K]         float8_e8m0fnu bytes, one per block
 *   sc32 : float  [batch, M]            fp32 amax, one per super-group
 * with Nb = rows*cols/(a*b) blocks numbered row-major, K = gcd(max(1,a*b/16), Nb),
 * M = Nb/K.  `batch` is the reference's per-leading-index scan (_qarr.py:38-42).
 */
#ifndef PRATCHYA_B200_H_
#define PRATCHYA_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define PB_API __attribute__((visibility("default")))
#else
#define PB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pb_status {
  PB_OK = 0,
  PB_ERR_NULL_POINTER = 1,
  PB_ERR_BAD_SHAPE = 2,        /* non-positive, or rows % a / cols % b != 0 (the reference's reshape fails too) */
  PB_ERR_BAD_GRID = 3,
  PB_ERR_BAD_DTYPE = 4,
  PB_ERR_WORKSPACE_TOO_SMALL = 5,
  PB_ERR_CUDA = 6,             /* a CUDA runtime/driver call failed; text in pb_last_error() */
  PB_ERR_DEVICE_TIMEOUT = 7,   /* a bounded device-side wait ran out (read back via pb_gemm_check) */
  PB_ERR_UNSUPPORTED = 8,
  PB_ERR_MISALIGNED = 9
} pb_status;

/* element types of dense (unquantized) arrays */
enum { PB_F32 = 0, PB_BF16 = 1 };
/* fp8 storage formats.  E4M3 is the reference's; E5M2 swaps only the final cast. */
enum { PB_E4M3 = 0, PB_E5M2 = 1 };

PB_API int pb_version(void);
PB_API const char* pb_last_error(void);
PB_API const char* pb_status_string(int status);

/* (M, K) of the scale arrays for one [rows, cols] slice.  _qarr.py:474-480. */
PB_API int pb_group_geometry(int64_t rows, int64_t cols, int a, int b, int64_t* M, int64_t* K);

/* ---- quantize: replaces quantize_impl(x, tgrid), _qarr.py:458-506 (and the
 *      per-leading-index scan of QArrayImpl.__quantize, :34-44, via `batch`).
 *      x is [batch, rows, cols] of x_dtype (PB_F32 | PB_BF16), row-major, 16-byte aligned.
 *      Non-finite inputs are where this library knowingly departs from the reference: jnp.max propagates a
 *      NaN, so one NaN makes the reference's whole super-group (its fp32 amax, every scale and byte) NaN; the
 *      amax reductions here drop NaNs (fmaxf / __hmax2 / integer max on the bits), so only the NaN element
 *      itself becomes the fp8 NaN byte and its neighbours keep finite scales.  An Inf input gives an Inf amax
 *      in both.  Finite inputs are bit-exact. */
PB_API size_t pb_quantize_workspace_size(int64_t batch, int64_t rows, int64_t cols, int a, int b);
PB_API int pb_quantize(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols,
                int a, int b, int out_format,
                void* q, uint8_t* sc8, float* sc32,
                void* workspace, size_t workspace_bytes, void* stream);

/* ---- quantize for callers that can neither pass nor allocate scratch memory.  It has no
 *      counterpart in the reference.  Same arguments and results as pb_quantize, minus the
 *      workspace: the scratch is a 512 KiB device array built into the library (held by every
 *      GPU that loads it until the process exits), so batch * (rows*cols/(a*b)) must not exceed
 *      65536 blocks; larger inputs return PB_ERR_UNSUPPORTED.  The call allocates nothing
 *      (no cudaMalloc/cudaFree, no allocating library routine).  The first call on each device
 *      looks up the array's device address (cudaGetSymbolAddress) and caches it: make that
 *      first call outside any stream capture.  All calls share the one array, which keeps what
 *      the last call wrote; each call clears what it reads before use, but two calls that
 *      overlap on the GPU (different streams) race on it. */
PB_API int pb_quantize_static(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols,
                       int a, int b, int out_format,
                       void* q, uint8_t* sc8, float* sc32, void* stream);

/* ---- quantize of the transpose without materialising it: the triple of
 *      quantize_impl(swapaxes(x,-1,-2), (1, b)) as used by fp8_matmul_bwd,
 *      _qarr.py:784-789.  x is [batch, rows, cols]; q is [batch, cols, rows]. */
PB_API size_t pb_quantize_transposed_workspace_size(int64_t batch, int64_t rows, int64_t cols, int b);
PB_API int pb_quantize_transposed(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols,
                           int b, int out_format,
                           void* q_t, uint8_t* sc8, float* sc32,
                           void* workspace, size_t workspace_bytes, void* stream);

/* ---- dequantize: replaces dequantize_impl(x_fp8, sc_fp8, sc_fp32, dtype, tgrid),
 *      _qarr.py:541-569.  out is [batch, rows, cols] of out_dtype. */
PB_API int pb_dequantize(const void* q, int q_format, const uint8_t* sc8, const float* sc32,
                  int64_t batch, int64_t rows, int64_t cols, int a, int b,
                  int out_dtype, void* out, void* stream);

/* ---- cotangent of dequantize: g * x_sc / 128, dequantize_impl_bwd, _qarr.py:575-601.
 *      g and out are [batch, rows, cols] of `dtype`. */
PB_API int pb_dequantize_bwd(const void* g, int dtype, const uint8_t* sc8, const float* sc32,
                      int64_t batch, int64_t rows, int64_t cols, int a, int b,
                      void* out, void* stream);

/* out = op(dq(x), dq(y)) in f32 for two quantized arrays of the same shape on the same grid: the
 * forward of make_elementwise_impl (pratchya/_qualia/_qarr.py:715-720; add_impl, sub_impl, mul_impl,
 * truediv_impl :757-760) in one pass instead of two dequantizations and an op.  IEEE f32 arithmetic,
 * so the bits are those of the three steps.  floordiv, mod and pow (:761-763) are not offered here. */
#define PB_OP_ADD 0
#define PB_OP_SUB 1
#define PB_OP_MUL 2
#define PB_OP_DIV 3
PB_API int pb_elementwise(int op, const void* xq, int x_format, const uint8_t* x_sc8, const float* x_sc32,
                   const void* yq, int y_format, const uint8_t* y_sc8, const float* y_sc32,
                   int64_t batch, int64_t rows, int64_t cols, int a, int b, float* out, void* stream);

/* Momentum step of the reference's optimizer for a quantized parameter
 * (pratchya/_nnx_impl/_optimizer.py:171-205): with g and m the gradient and momentum triples on the
 * parameter's grid (a,b),
 *     c     = beta1 * dq(m) + (1 - beta1) * dq(g)     f32, written to c_out (input of sign() / Newton-Schulz)
 *     new_m = beta2 * dq(m) + (1 - beta2) * dq(g)     written as the triple quantize_impl(new_m, (a,b))
 * in two passes over the bytes of g and m instead of two dequantizations, four scaled temporaries
 * and a quantization.  The four scalars are passed as the f32 values JAX would use (beta and
 * 1 - beta, each computed in double and rounded once).  e4m3 triples; workspace:
 * pb_momentum_workspace_size (8 bytes per block). */
PB_API size_t pb_momentum_workspace_size(int64_t batch, int64_t rows, int64_t cols, int a, int b);
PB_API int pb_momentum_update(const void* gq, const uint8_t* g_sc8, const float* g_sc32,
                       const void* mq, const uint8_t* m_sc8, const float* m_sc32,
                       int64_t batch, int64_t rows, int64_t cols, int a, int b,
                       float beta1, float one_minus_beta1, float beta2, float one_minus_beta2,
                       float* c_out, void* new_mq, uint8_t* new_m_sc8, float* new_m_sc32,
                       void* workspace, size_t workspace_bytes, void* stream);

/* The same step for a stacked parameter [layers, rows, cols], the scanned branch of the reference's optimizer
 * (pratchya/_nnx_impl/_optimizer.py:108-160), which every parameter of the model's scanned blocks takes: per layer
 * g and m are dequantized to bfloat16 (:113-114), c and new_m are blended in bfloat16 (:123-124; the scalars
 * become bfloat16, every product and sum rounds to bfloat16) and new_m is quantized again on (a,b) (:134).
 * c_out_bf16 is bfloat16 [layers, rows, cols].  The four scalars are passed as f32 holding the bfloat16 values of
 * beta and 1 - beta.  Super-groups never cross a layer.  Workspace: pb_momentum_workspace_size(layers, ...). */
PB_API int pb_momentum_update_stacked(const void* gq, const uint8_t* g_sc8, const float* g_sc32,
                               const void* mq, const uint8_t* m_sc8, const float* m_sc32,
                               int64_t layers, int64_t rows, int64_t cols, int a, int b,
                               float beta1, float one_minus_beta1, float beta2, float one_minus_beta2,
                               void* c_out_bf16, void* new_mq, uint8_t* new_m_sc8, float* new_m_sc32,
                               void* workspace, size_t workspace_bytes, void* stream);

/* ---- block-scaled FP8 matmul.
 * A GEMM operand is a K-major quantized matrix: bytes [rows, depth] (depth = the
 * contraction length, contiguous), one e8m0 byte per (row-block, 128-deep block)
 * and one fp32 factor per super-group, exactly as pb_quantize lays them out for
 * the grids (1,128) (per-row scales) and (128,128) (per-tile scales).
 *
 *   D[m, n] = sum_k dq(A)[m, k] * dq(B)[n, k]        fp32 accumulate
 *
 * pb_gemm_tn covers all three matmuls of the reference's training triple:
 *   forward  matmul_impl, _qarr.py:605-608 : A = Q(x,(1,128)),   B = the weight's bytes transposed
 *   dgrad    matmul_impl_bwd g @ W^T, :621  : A = Q(g,(1,128)),   B = the weight as stored [K,N] (N is the depth)
 *   wgrad    fp8_matmul_bwd x^T @ g, :789   : A = Q(x^T,(1,128)), B = Q(g^T,(1,128))
 */
typedef struct pb_operand {
  const void* q;          /* fp8 bytes [rows, depth], row pitch = depth, 16-byte aligned */
  const uint8_t* sc8;     /* e8m0 bytes [M, K] as produced by pb_quantize on `grid` */
  const float* sc32;      /* fp32 [M] */
  int64_t rows;           /* M for operand A, N for operand B */
  int64_t depth;          /* contraction length, multiple of 128 */
  int grid_a, grid_b;     /* (1,128) or (128,128); blocks are counted on the [rows, depth] view */
  int format;             /* PB_E4M3 | PB_E5M2 */
  int transposed_blocks;  /* 1: sc8/sc32 were produced on the [depth, rows] view of the same bytes' transpose, where the
                             blocks are (128, grid_a): a weight stored [K, N] and quantized on (128,128) (grid_a = 128)
                             or on (128,1) (grid_a = 1: the reference's gate, lm_head and LoRA weights,
                             pratchya/_nnx_impl/_module.py:82-84, 326), used without re-quantizing; 0 otherwise */
} pb_operand;

PB_API size_t pb_gemm_workspace_size(const pb_operand* a, const pb_operand* b);
PB_API int pb_gemm_tn(const pb_operand* a, const pb_operand* b,
               void* d, int d_dtype, int64_t ldd,
               void* workspace, size_t workspace_bytes, void* stream);
/* pb_gemm_tn with the re-tiling of the scales skipped for operands whose prepared scales are
 * already in `workspace` (no counterpart in the reference: it saves the two small launches that
 * pb_gemm_tn spends on them in a step like Linear.__call__, pratchya/_nnx_impl/_module.py:46-50,
 * where the weight's scales do not change between calls).
 *   PB_GEMM_A_PREPARED  A's scales were written by pb_quantize_for_gemm into this workspace.
 *   PB_GEMM_B_PREPARED  an earlier pb_gemm_tn / pb_gemm_tn_ex with the same B (bytes may differ, sc8
 *                       and sc32 may not), the same A shape and grid and this workspace has run, and
 *                       nothing else has written the workspace since.
 * flags = 0 is pb_gemm_tn. PB_GEMM_A_PREPARED on an operand pair whose fp32 factors do not hold
 * for eight k-blocks at a time returns PB_ERR_UNSUPPORTED. */
#define PB_GEMM_A_PREPARED 1u
#define PB_GEMM_B_PREPARED 2u
PB_API int pb_gemm_tn_ex(const pb_operand* a, const pb_operand* b,
                  void* d, int d_dtype, int64_t ldd,
                  void* workspace, size_t workspace_bytes, unsigned int flags, void* stream);
/* quantize_impl (pratchya/_qualia/_qarr.py:458-506) on the (1,128) grid for an activation
 * x[rows, cols] that is about to be operand A of pb_gemm_tn_ex against `b`: the same q, sc8 and
 * sc32 as pb_quantize, and in the same pass A's scales in the layout the GEMM kernel reads, written
 * into `gemm_workspace` (size from pb_gemm_workspace_size(a, b)).  cols must be a multiple of
 * 1024 (whole super-groups of eight blocks per row); PB_ERR_UNSUPPORTED when b's scales do not
 * allow promotion every eight k-blocks.  Follow it with pb_gemm_tn_ex(..., PB_GEMM_A_PREPARED ...). */
PB_API int pb_quantize_for_gemm(const void* x, int x_dtype, int64_t rows, int64_t cols, int out_format,
                         void* q, uint8_t* sc8, float* sc32,
                         const pb_operand* b, void* gemm_workspace, size_t gemm_workspace_bytes, void* stream);
/* out = dequantize(quantize(x)) in one pass: what Linear.__call__ does to its f32 product,
 * `(x_q @ kernel).astype(x.dtype)` (pratchya/_nnx_impl/_module.py:46-50; the product is wrapped as
 * QArrayImpl(out, (1, b)), pratchya/_qualia/_qarr.py:104-105, and read back by astype, :339-342).
 * Same bits as pb_quantize followed by pb_dequantize.  f32 input on the (1,128) grid with whole
 * super-groups of eight blocks only; anything else returns PB_ERR_UNSUPPORTED (use the two calls). */
PB_API int pb_fake_quantize(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols, int a, int b,
                     int out_format, void* out, int out_dtype, void* stream);
/* Reads (and clears) the device status words of the kernels that wait on mbarriers (the GEMM kernels and the
 * persistent transposed quantizer) launched on this device; synchronises `stream`.  Every such wait is bounded
 * (a few seconds at most); a wait that runs out makes its kernel return early and is reported here:
 * PB_OK or PB_ERR_DEVICE_TIMEOUT. */
PB_API int pb_gemm_check(void* stream);

/* The middle of ChannelMix (pratchya/_nnx_impl/_module.py:246-251) on the f32 product y[rows, cols] of
 * its first Linear, in one pass: k = dq(q(y, (1,128))) as Linear.__call__ returns it for an f32
 * input (:46-50), k = relu(k)^2 (:249), then quantize_impl(k, (1,128)) for the second Linear (:46-47).
 * Outputs the triple of k; the bits are those of pb_fake_quantize (f32 out), an f32 relu and square
 * and pb_quantize.  With a non-null `b` it also writes k's scales for pb_gemm_tn_ex(...,
 * PB_GEMM_A_PREPARED ...) against b into gemm_workspace, as pb_quantize_for_gemm does.
 * cols must be a multiple of 1024, otherwise PB_ERR_UNSUPPORTED. */
PB_API int pb_relu2_requantize(const void* y, int64_t rows, int64_t cols, int out_format,
                        void* q, uint8_t* sc8, float* sc32,
                        const pb_operand* b, void* gemm_workspace, size_t gemm_workspace_bytes, void* stream);
/* Both quantized forms of an activation (or gradient) that a training step needs, from one
 * call: Q(x, (1,128)) for the forward / dgrad product and Q(x^T, (1,128)) for wgrad (the
 * operands of fp8_matmul_bwd, pratchya/_qualia/_qarr.py:784-789).  The same bits as pb_quantize
 * on (1,128) and pb_quantize_transposed with b = 128; x is read twice instead of three times
 * (the row quantizer's pass also takes the column-block maxima).  bf16 x with rows % 128 == 0 and
 * cols % 1024 == 0, otherwise PB_ERR_UNSUPPORTED (use the two calls).  Workspace:
 * pb_quantize_transposed_workspace_size(batch, rows, cols, 128). */
PB_API int pb_quantize_dual(const void* x, int x_dtype, int64_t batch, int64_t rows, int64_t cols, int out_format,
                     void* q, uint8_t* sc8, float* sc32, void* q_t, uint8_t* sc8_t, float* sc32_t,
                     void* workspace, size_t workspace_bytes, void* stream);
/* ---- WKV-7 state scan of the TimeMix block: replaces the per-timestep nnx.scan `wkv_state_scan`,
 *      pratchya/_nnx_impl/_module.py:187-207.  The six inputs (decay, iclr, removal_k, replacement_k, v, r)
 *      are f32 [batch, steps, heads*head_dim]; state_in / state_out are f32 [batch, heads, head_dim, head_dim]
 *      (state_in may be null for a zero state, state_out may be null); y is f32 [batch, steps, heads*head_dim],
 *      the order the reference has after its transpose (:210).  head_dim must be 64.  16-byte aligned arrays.
 *      `checkpoints` (may be null) receives the state before timesteps 0, 8, 16, ... as f32
 *      [batch, heads, ceil(steps/8), head_dim, head_dim] (pb_wkv7_checkpoint_floats elements): what
 *      pb_wkv7_backward restarts from.  `sa` (may be null) receives, for every timestep, the state before the step times
 *      removal_k (f32 [batch, steps, heads*head_dim]): with it the backward pass recomputes the states element-wise. */
PB_API int pb_wkv7_forward(const float* decay, const float* iclr, const float* removal_k, const float* replacement_k,
                    const float* v, const float* r, const float* state_in,
                    int64_t batch, int64_t steps, int64_t heads, int head_dim,
                    float* y, float* state_out, float* checkpoints, float* sa, void* stream);
PB_API size_t pb_wkv7_checkpoint_floats(int64_t batch, int64_t steps, int64_t heads, int head_dim);
/* Cotangents of the scan: what jax.grad derives from `wkv_state_scan` (pratchya/_nnx_impl/_module.py:187-207) for the
 * six inputs and the initial state, given dy [batch, steps, heads*head_dim] and (optionally) the cotangent of the final
 * state.  The states the derivatives need are recomputed eight timesteps at a time from the forward pass's checkpoints
 * and its `sa` array, and stay in shared memory: the call needs no workspace.  All arrays f32. */
PB_API int pb_wkv7_backward(const float* decay, const float* iclr, const float* removal_k, const float* replacement_k,
                     const float* v, const float* r, const float* checkpoints, const float* sa, const float* dy, const float* dstate_out,
                     int64_t batch, int64_t steps, int64_t heads, int head_dim,
                     float* d_decay, float* d_iclr, float* d_removal_k, float* d_replacement_k, float* d_v, float* d_r,
                     float* dstate_in, void* stream);

/* ---- the f32 element-wise work of the modified RWKV-7 block around its linears and its scan
 *      (pratchya/_nnx_impl/_module.py:129-258), fused.  All arrays f32, 16-byte aligned where stated.
 *
 * Token shift and lerps (TimeMix :137-151 with six mixes, ChannelMix :240-247 with one):
 *   out[k][b][t][c] = x[b][t][c] + (prev - x[b][t][c]) * mu[k][c],  prev = x[b][t-1][c], or state[b][c] for t = 0
 * (state may be null: zeros).  out is [n_mix, batch, steps, channels]; channels a multiple of 4; n_mix <= 8. */
PB_API int pb_token_shift_lerp(const float* x, const float* state, const float* mu, int64_t batch, int64_t steps, int64_t channels,
                        int n_mix, float* out, void* stream);
/* Its cotangents from g[k] [batch, steps, channels], k < n_mix (a host array of n_mix device pointers): dx, dstate [batch, channels] (may be null) and
 * dmu [n_mix, channels] (summed over tokens per tile and then in tile order: deterministic).  n_mix is 1 or 6. */
PB_API size_t pb_token_shift_lerp_bwd_workspace_size(int64_t batch, int64_t steps, int64_t channels, int n_mix);
PB_API int pb_token_shift_lerp_bwd(const float* const* g, const float* x, const float* state, const float* mu,
                            int64_t batch, int64_t steps, int64_t channels, int n_mix,
                            float* dx, float* dstate, float* dmu, void* workspace, size_t workspace_bytes, void* stream);
/* relu(k)^2 (ChannelMix's activation, pratchya/_nnx_impl/_module.py:249) as the prologue of the second Linear's two input
 * quantizers: from k [rows, cols] f32 the triples of quantize_impl(relu(k)^2, (1,128)) (q, sc8, sc32) and of its transpose
 * (q_t [cols, rows], sc8_t, sc32_t), e4m3, without writing relu(k)^2.  The bytes are those of pb_relu2 followed by pb_quantize
 * and pb_quantize_transposed.  rows and cols multiples of 1024; k 16-byte, q_t 32-byte aligned. */
PB_API int pb_relu2_quantize_dual(const float* k, int64_t rows, int64_t cols, uint8_t* q, uint8_t* sc8, float* sc32,
                           uint8_t* q_t, uint8_t* sc8_t, float* sc32_t, void* stream);
/* The first step of a Linear's backward pass in one call (pratchya/_qualia/_qarr.py:575-601 followed by the quantizations of
 * :784-789): the cotangent g [rows, cols] f32 of the layer's fake-quantized output is scaled by the cotangent rule of that
 * output's dequantize, g' = (g * x_sc) / 128 with x_sc = e8m0(y_sc8) * y_sc32 of the OUTPUT's (1,128) triple (what pb_dequantize_bwd
 * computes), and g' leaves as the triple of quantize_impl(g', (1,128)) (q, sc8, sc32: the dgrad operand) and as the triple of
 * quantize_impl(g'^T, (1,128)) (q_t [cols, rows], sc8_t, sc32_t: the wgrad operand).  g' itself is not written.  The bytes are
 * those of pb_dequantize_bwd followed by pb_quantize and pb_quantize_transposed.  rows and cols multiples of 1024; g 16-byte,
 * q_t 32-byte aligned; out_format PB_E4M3 or PB_E5M2. */
PB_API int pb_dequantize_bwd_quantize_dual(const float* g, const uint8_t* y_sc8, const float* y_sc32, int64_t rows, int64_t cols, int out_format,
                                    uint8_t* q, uint8_t* sc8, float* sc32, uint8_t* q_t, uint8_t* sc8_t, float* sc32_t, void* stream);
/* Token shift and lerps fused into the activation quantizers of the Linears that consume the mixes
 * (Linear.__call__, pratchya/_nnx_impl/_module.py:46-47, applied to the mixes of :137-151 and :240-247): with
 * v_k = x + (prev - x) * mu[k] as above, every mix k < n_mix leaves as the triple of quantize_impl(v_k, (1,128)),
 *   q [n_mix][batch*steps][channels] e4m3, sc8 [n_mix][batch*steps*channels/128], sc32 [n_mix][batch*steps*channels/1024],
 * and every mix whose bit is set in transposed_mask also as the triple of quantize_impl(v_k^T, (1,128)) (what
 * pb_quantize_transposed gives for v_k), stacked in the order of the set bits:
 *   q_t [n_t][channels][batch*steps], sc8_t [n_t][channels*batch*steps/128], sc32_t [n_t][channels*batch*steps/1024].
 * No v_k is written.  The bytes are those of pb_token_shift_lerp followed by pb_quantize / pb_quantize_transposed.
 * channels a multiple of 1024; with a transposed form steps a multiple of 1024 and q_t 32-byte aligned. */
PB_API int pb_shift_lerp_quantize(const float* x, const float* state, const float* mu, int64_t batch, int64_t steps, int64_t channels,
                           int n_mix, uint8_t* q, uint8_t* sc8, float* sc32, unsigned int transposed_mask,
                           uint8_t* q_t, uint8_t* sc8_t, float* sc32_t, void* stream);
/* TimeMix between its linears and its scan (:157-184), per token and head of 64 channels:
 *   r, k    = rotary embedding of r_raw, k_raw with the angle tables cos_tab / sin_tab [steps, 32] (:275-283)
 *   iclr    = sigmoid(iclr_raw);  decay = exp(-exp(d))
 *   v       = v_prime, or v_prime + (v0 - v_prime) * sigmoid(nu_raw) when v0 / nu_raw are given (not the first layer)
 *   removal_k     = normalized(k * rk_mult) over the head's channels (eps 1e-12, :15-18)
 *   replacement_k = k + (k * iclr - k) * mix_amt
 * rk_mult and mix_amt are [channels] (the parameters as read through their quantization). */
PB_API int pb_wkv_prepare(const float* r_raw, const float* k_raw, const float* d, const float* iclr_raw, const float* v_prime,
                   const float* v0, const float* nu_raw, const float* cos_tab, const float* sin_tab,
                   const float* rk_mult, const float* mix_amt, int64_t batch, int64_t steps, int64_t heads, int head_dim,
                   float* decay, float* iclr, float* removal_k, float* replacement_k, float* v, float* r, float* k, void* stream);
/* Cotangents of pb_wkv_prepare's seven inputs and two parameters from those of its seven outputs. */
PB_API size_t pb_wkv_prepare_bwd_workspace_size(int64_t batch, int64_t steps, int64_t heads, int head_dim);
PB_API int pb_wkv_prepare_bwd(const float* r_raw, const float* k_raw, const float* d, const float* iclr_raw, const float* v_prime,
                       const float* v0, const float* nu_raw, const float* cos_tab, const float* sin_tab,
                       const float* rk_mult, const float* mix_amt, int64_t batch, int64_t steps, int64_t heads, int head_dim,
                       const float* g_decay, const float* g_iclr, const float* g_removal_k, const float* g_replacement_k,
                       const float* g_v, const float* g_r, const float* g_k,
                       float* d_r_raw, float* d_k_raw, float* d_d, float* d_iclr_raw, float* d_v_prime, float* d_v0, float* d_nu_raw,
                       float* d_rk_mult, float* d_mix_amt, void* workspace, size_t workspace_bytes, void* stream);

/* RMSNorm (pratchya/_nnx_impl/_module.py:61-72): y = (x * rsqrt(mean(x^2) + eps)) * scale over the last dimension of
 * x [rows, channels]; scale [channels] as read through its quantization; inv_rms [rows] is kept for the backward call.
 * channels a multiple of 128. */
PB_API int pb_rms_norm(const float* x, const float* scale, int64_t rows, int64_t channels, float eps, float* y, float* inv_rms, void* stream);
PB_API size_t pb_rms_norm_bwd_workspace_size(int64_t rows, int64_t channels);
PB_API int pb_rms_norm_bwd(const float* dy, const float* x, const float* scale, const float* inv_rms, int64_t rows, int64_t channels,
                    float* dx, float* dscale, void* workspace, size_t workspace_bytes, void* stream);
/* relu(x)^2 (ChannelMix between its linears, :249) and its cotangent g * 2 * relu(x); n elements, a multiple of 4. */
PB_API int pb_relu2(const float* x, int64_t n, float* y, void* stream);
PB_API int pb_relu2_bwd(const float* g, const float* x, int64_t n, float* dx, void* stream);
/* TimeMix after its scan (:208-216): out = (GroupNorm(y) + sum_c(r k bonus_mult) * v) * gate, GroupNorm as flax builds
 * it with one group per head (:118-123): per batch element and head, mean and variance (E[x^2] - E[x]^2, clamped at 0)
 * over the steps x 64 values, then gn_scale and gn_bias per channel.  stats [batch * heads][2] receives (mean, rstd)
 * for the backward call. */
PB_API size_t pb_wkv_finish_workspace_size(int64_t batch, int64_t steps, int64_t heads, int head_dim);
PB_API int pb_wkv_finish(const float* y, const float* r, const float* k, const float* v, const float* gate,
                  const float* gn_scale, const float* gn_bias, const float* bonus_mult, float eps,
                  int64_t batch, int64_t steps, int64_t heads, int head_dim,
                  float* out, float* stats, void* workspace, size_t workspace_bytes, void* stream);
PB_API size_t pb_wkv_finish_bwd_workspace_size(int64_t batch, int64_t steps, int64_t heads, int head_dim);
PB_API int pb_wkv_finish_bwd(const float* g, const float* y, const float* r, const float* k, const float* v, const float* gate,
                      const float* gn_scale, const float* gn_bias, const float* bonus_mult, const float* stats,
                      int64_t batch, int64_t steps, int64_t heads, int head_dim,
                      float* d_y, float* d_r, float* d_k, float* d_v, float* d_gate,
                      float* d_gn_scale, float* d_gn_bias, float* d_bonus_mult,
                      void* workspace, size_t workspace_bytes, void* stream);

/* The training loss, compute_loss (pratchya/_nnx_impl/_utils.py:7-13): softmax cross entropy of logits [rows, vocab] (f32)
 * against one-hot targets smoothed by alpha (optax.smooth_labels).  row_loss[r] = weight[r] * (lse_r - (1 - alpha) * z[r][target[r]]
 * - alpha * mean_j z[r][j]); the caller sums the rows and divides by the number of positions that count (weight 0 leaves a
 * row out: the last position of every sequence has no next token).  lse [rows] is kept for the backward call, which writes
 * dlogits = upstream[0] * weight[r] / denominator * (softmax - (1 - alpha) * onehot - alpha / vocab).  vocab a multiple of 4. */
PB_API int pb_smoothed_xent(const float* logits, const int64_t* target, const float* weight, int64_t rows, int64_t vocab, float alpha,
                     float* row_loss, float* lse, void* stream);
PB_API int pb_smoothed_xent_bwd(const float* logits, const int64_t* target, const float* weight, const float* lse, const float* upstream,
                         float denominator, int64_t rows, int64_t vocab, float alpha, float* dlogits, void* stream);

/* byte transpose [rows, cols] -> [cols, rows] of an fp8 matrix (weight prepared for the forward GEMM) */
PB_API int pb_transpose_bytes(const void* src, int64_t rows, int64_t cols, void* dst, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PRATCHYA_B200_H_ */
