// XLA FFI handlers around the C ABI of libpratchya_b200.so, for a JAX host.
//
// NOT BUILT OR RUN WHERE THIS LIBRARY IS TESTED: neither jax nor the XLA FFI headers are installed
// there.  It is the binding the C ABI was shaped for; build it next to a JAX installation with
//
//   g++ -std=c++17 -shared -fPIC xla_ffi_shim.cc -I../../include \
//       -I"$(python -c 'import jax; print(jax.ffi.include_dir())')" -I"$CUDA_HOME/include" \
//       -L. -lpratchya_b200 -Wl,-rpath,'$ORIGIN' -o libpratchya_b200_xla.so
//
// and register the symbols below with jax.ffi.register_ffi_target (see pratchya_b200/jax_ffi.py).
//
// One handler per function of the reference that the library replaces
// (pratchya/_qualia/_qarr.py): quantize_impl :458-506, dequantize_impl :541-569 and the forward
// product of Linear, matmul_impl :605-608 for a (1,128) activation against a (128,128) weight.
// Shapes follow the reference: x[..., R, C]; sc_fp8[..., M, K]; sc_fp32[..., M, 1, 1].  Scratch
// comes from XLA as an extra result buffer, so the handlers allocate nothing.
#include <cuda_runtime_api.h>

#include <cstdint>

#include "pratchya_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error status_to_error(int status) {
  if (status == PB_OK) return ffi::Error::Success();
  const ffi::ErrorCode code = (status == PB_ERR_CUDA || status == PB_ERR_DEVICE_TIMEOUT) ? ffi::ErrorCode::kInternal
                                                                                         : ffi::ErrorCode::kInvalidArgument;
  return ffi::Error(code, pb_last_error());
}

// PB_F32 / PB_BF16 for a dense buffer; -1 for anything else
int dense_code(ffi::DataType t) {
  if (t == ffi::DataType::F32) return PB_F32;
  if (t == ffi::DataType::BF16) return PB_BF16;
  return -1;
}

// PB_E4M3 / PB_E5M2 for a quantized buffer; -1 for anything else
int fp8_code(ffi::DataType t) {
  if (t == ffi::DataType::F8E4M3FN) return PB_E4M3;
  if (t == ffi::DataType::F8E5M2) return PB_E5M2;
  return -1;
}

// [..., R, C] -> (batch, R, C); a 1-D array is [1, n] and a 0-D one [1, 1], as in _qarr.py:461-464
void split_dims(ffi::AnyBuffer::Dimensions dims, int64_t* batch, int64_t* rows, int64_t* cols) {
  const size_t n = dims.size();
  *cols = n >= 1 ? dims[n - 1] : 1;
  *rows = n >= 2 ? dims[n - 2] : 1;
  *batch = 1;
  for (size_t i = 0; i + 2 < n; ++i) *batch *= dims[i];
}

ffi::Error QuantizeImpl(cudaStream_t stream, ffi::AnyBuffer x, int64_t a, int64_t b,
                        ffi::Result<ffi::AnyBuffer> q, ffi::Result<ffi::AnyBuffer> sc8, ffi::Result<ffi::AnyBuffer> sc32,
                        ffi::Result<ffi::AnyBuffer> scratch) {
  int64_t batch, rows, cols;
  split_dims(x.dimensions(), &batch, &rows, &cols);
  const int in = dense_code(x.element_type()), out = fp8_code(q->element_type());
  if (in < 0 || out < 0) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "pb_quantize: x must be f32 or bf16 and q an fp8 type");
  return status_to_error(pb_quantize(x.untyped_data(), in, batch, rows, cols, (int)a, (int)b, out, q->untyped_data(),
                                     static_cast<uint8_t*>(sc8->untyped_data()), static_cast<float*>(sc32->untyped_data()),
                                     scratch->untyped_data(), scratch->size_bytes(), stream));
}

ffi::Error DequantizeImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer sc8, ffi::AnyBuffer sc32, int64_t a, int64_t b,
                          ffi::Result<ffi::AnyBuffer> out) {
  int64_t batch, rows, cols;
  split_dims(q.dimensions(), &batch, &rows, &cols);
  const int in = fp8_code(q.element_type()), dt = dense_code(out->element_type());
  if (in < 0 || dt < 0) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "pb_dequantize: q must be an fp8 type and out f32 or bf16");
  return status_to_error(pb_dequantize(q.untyped_data(), in, static_cast<const uint8_t*>(sc8.untyped_data()),
                                       static_cast<const float*>(sc32.untyped_data()), batch, rows, cols, (int)a, (int)b, dt,
                                       out->untyped_data(), stream));
}

// x_q[..., M, K] on (1,128) times a weight given K-major: w_t[N, K] = the fp8 bytes of the stored
// [K, N] weight transposed once with pb_transpose_bytes, with the weight's own (128,128) scales.
// Leading dims of x stack into rows (their super-groups are eight blocks of one row each).
ffi::Error MatmulImpl(cudaStream_t stream, ffi::AnyBuffer xq, ffi::AnyBuffer x_sc8, ffi::AnyBuffer x_sc32, ffi::AnyBuffer w_t,
                      ffi::AnyBuffer w_sc8, ffi::AnyBuffer w_sc32, ffi::Result<ffi::AnyBuffer> y, ffi::Result<ffi::AnyBuffer> scratch) {
  int64_t batch, rows, depth;
  split_dims(xq.dimensions(), &batch, &rows, &depth);
  const auto wd = w_t.dimensions();
  if (wd.size() != 2 || wd[1] != depth) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "pb_gemm_tn: w_t must be [N, K] with K = x's last dim");
  const int fa = fp8_code(xq.element_type()), fb = fp8_code(w_t.element_type()), dt = dense_code(y->element_type());
  if (fa < 0 || fb < 0 || dt < 0) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "pb_gemm_tn: operands must be fp8 and y f32 or bf16");
  // The stacked rows are declared as one (1,128) operand, which is only the layout the scales were written with
  // when every slice's super-groups are eight blocks of one row: check the scale arrays against that.
  const auto sd = x_sc8.dimensions();
  if (sd.empty() || sd.back() != 8 || (rows * depth / 128) % 8 != 0)
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "pb_gemm_tn: x's super-groups must be eight 128-wide blocks (x_sc8[..., M, 8])");
  int64_t wm = 0, wk = 0;
  if (pb_group_geometry(depth, wd[0], 128, 128, &wm, &wk) != PB_OK) return ffi::Error(ffi::ErrorCode::kInvalidArgument, pb_last_error());
  if ((int64_t)x_sc8.element_count() != batch * rows * depth / 128 || (int64_t)x_sc32.element_count() != batch * rows * depth / 1024 ||
      (int64_t)w_sc8.element_count() != wm * wk || (int64_t)w_sc32.element_count() != wm)
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "pb_gemm_tn: scale arrays do not match the operands' block geometry");
  // A bounded device-side wait that runs out is recorded in a device status word, not returned here (the call is
  // asynchronous): the host polls pb_gemm_check between steps.
  pb_operand a, b;
  a.q = xq.untyped_data(); a.sc8 = static_cast<const uint8_t*>(x_sc8.untyped_data()); a.sc32 = static_cast<const float*>(x_sc32.untyped_data());
  a.rows = batch * rows; a.depth = depth; a.grid_a = 1; a.grid_b = 128; a.format = fa; a.transposed_blocks = 0;
  b.q = w_t.untyped_data(); b.sc8 = static_cast<const uint8_t*>(w_sc8.untyped_data()); b.sc32 = static_cast<const float*>(w_sc32.untyped_data());
  b.rows = wd[0]; b.depth = depth; b.grid_a = 128; b.grid_b = 128; b.format = fb; b.transposed_blocks = 1;
  const size_t need = pb_gemm_workspace_size(&a, &b);
  if (need == 0) return ffi::Error(ffi::ErrorCode::kInvalidArgument, pb_last_error());
  if (scratch->size_bytes() < need) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "pb_gemm_tn: scratch result is smaller than pb_gemm_workspace_size");
  return status_to_error(pb_gemm_tn(&a, &b, y->untyped_data(), dt, wd[0], scratch->untyped_data(), scratch->size_bytes(), stream));
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(pb_quantize_ffi, QuantizeImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Attr<int64_t>("a")
                                  .Attr<int64_t>("b")
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(pb_dequantize_ffi, DequantizeImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Attr<int64_t>("a")
                                  .Attr<int64_t>("b")
                                  .Ret<ffi::AnyBuffer>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(pb_matmul_ffi, MatmulImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>());
