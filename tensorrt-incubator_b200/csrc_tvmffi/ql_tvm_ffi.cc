// The library's kernels as TVM-FFI functions, the reference's second plug-in boundary:
// `executor.plugin` / `executor.call_plugin` load a shared object, resolve `__tvm_ffi_<name>` and call
//   int safe_call(void *self, const TVMFFIAny *args, int32_t num_args, TVMFFIAny *result)
// with DLTensor arguments, outputs passed as arguments, and the CUDA stream taken from the
// TVM-FFI environment (mlir-tensorrt/executor/lib/Runtime/FFI/FFI.cpp:69-97; StableHLO spelling
// `custom_call @name {plugin = "lib.so", func = "sym", arg_spec = "args.0;args.1;rets.0"}`,
// compiler/test/Passes/0_Frontend/StablehloToPlan/plugins.mlir:6-31).
//
// Exported functions (argument order):
//   ql_quantize(input, scale, output[, axis = -1[, fp8_mode = 0]])
//   ql_dequantize(input, scale, output[, axis = -1])
//   ql_linear_w8a16(x, w, scale, y)        ql_linear_w4a16(x, w_packed_u8[N, K/2], scale, y)
//   ql_gemm_fp8(xq, wq, sx, sw, y)         ql_gemm_i8(xq, wq, sx, sw, y)         ql_gemm_16(x, w, sw | None, y)
//   ql_linear(x, w, sx | None, sw | None, bias | None, y)                         ql_matmul(a, b, c)
//   ql_dynamic_quantize(input, double_quant_scale, data_u8[..., K/2], scales[, axis = -1[, block = 16]])
//   ql_dequantize_nvfp4(data_u8, scales, double_quant_scale, output)
//   ql_gemm_nvfp4(a_u8, a_scales, a_global | None, b_u8, b_scales, b_global | None, y)
//   ql_rmsnorm_quant_fp8(x, eps, q, scale)    ql_gemm_fp8_swiglu(xq, wq, sx, sw, act, row_amax)
//   ql_quantize_rows_fp8(act, row_amax, q, scale)
// uint8 tensors are raw bytes: e4m3 bit patterns, or two int4 / e2m1 values per byte where the signature says so.
// Errors become a raised TVM-FFI error (non-zero return), never an abort.
#include <dlpack/dlpack.h>
#include <tvm/ffi/c_api.h>
#include <tvm/ffi/extra/c_env_api.h>

#include <cstdio>
#include <cstring>

#include "qlinear_b200.h"

namespace {

int fail(const char *msg) {
  TVMFFIErrorSetRaisedFromCStr("ValueError", msg);
  return -1;
}

const DLTensor *tensor_arg(const TVMFFIAny &a) {
  if (a.type_index == kTVMFFIDLTensorPtr) return static_cast<const DLTensor *>(a.v_ptr);
  if (a.type_index == kTVMFFITensor) return TVMFFITensorGetDLTensorPtr(a.v_obj);
  return nullptr;
}

bool int_arg(const TVMFFIAny &a, int64_t *out) {
  if (a.type_index == kTVMFFIInt || a.type_index == kTVMFFIBool) {
    *out = a.v_int64;
    return true;
  }
  return false;
}

// DLTensor -> ql_tensor.  `packed` reinterprets a uint8 [..., K/2] tensor as int4 (1) or e2m1 (2) [..., K].
bool to_ql(const DLTensor *t, ql_tensor *out, int packed, char *why, size_t why_len) {
  if (!t) {
    snprintf(why, why_len, "expected a tensor argument");
    return false;
  }
  if (t->device.device_type != kDLCUDA) {
    snprintf(why, why_len, "tensors must live in CUDA device memory (there is no CPU path)");
    return false;
  }
  if (t->ndim > QL_MAX_RANK) {
    snprintf(why, why_len, "rank %d exceeds %d", t->ndim, QL_MAX_RANK);
    return false;
  }
  int64_t expect = 1;
  for (int i = t->ndim - 1; i >= 0; i--) {
    if (t->strides && t->shape[i] > 1 && t->strides[i] != expect) {
      snprintf(why, why_len, "tensors must be dense row-major");
      return false;
    }
    expect *= t->shape[i];
  }
  const DLDataType d = t->dtype;
  int q = -1;
  if (d.lanes == 1) {
    if (d.code == kDLFloat && d.bits == 32) q = QL_F32;
    else if (d.code == kDLFloat && d.bits == 16) q = QL_F16;
    else if (d.code == kDLBfloat && d.bits == 16) q = QL_BF16;
    else if (d.code == kDLInt && d.bits == 8) q = QL_I8;
    else if (d.code == kDLInt && d.bits == 4) q = QL_I4;
    else if (d.code == kDLFloat8_e4m3fn && d.bits == 8) q = QL_F8E4M3;
    else if (d.code == kDLUInt && d.bits == 8) q = packed == 1 ? QL_I4 : packed == 2 ? QL_F4E2M1 : QL_F8E4M3; // raw bytes
  }
  if (q < 0) {
    snprintf(why, why_len, "unsupported tensor dtype (code %d, %d bits)", (int)d.code, (int)d.bits);
    return false;
  }
  out->data = static_cast<char *>(t->data) + t->byte_offset;
  out->dtype = q;
  out->rank = t->ndim;
  for (int i = 0; i < t->ndim; i++) out->shape[i] = t->shape[i];
  if (packed && d.code == kDLUInt && t->ndim >= 1) out->shape[t->ndim - 1] *= 2;
  return true;
}

void *stream_of(const DLTensor *t) { return TVMFFIEnvGetStream(t->device.device_type, t->device.device_id); }

int finish(int rc) {
  if (rc == QL_OK) return 0;
  return fail(ql_last_error());
}

#define QL_TENSOR(idx, name, packed)                                                                \
  ql_tensor name;                                                                                  \
  const DLTensor *name##_dl = (idx) < n ? tensor_arg(args[idx]) : nullptr;                         \
  if (!to_ql(name##_dl, &name, packed, why, sizeof(why))) return fail(why);
// an argument that may be None: name##_p is null then
#define QL_OPTIONAL(idx, name)                                                                     \
  ql_tensor name;                                                                                  \
  const ql_tensor *name##_p = nullptr;                                                             \
  if ((idx) < n && args[idx].type_index != kTVMFFINone) {                                          \
    if (!to_ql(tensor_arg(args[idx]), &name, 0, why, sizeof(why))) return fail(why);               \
    name##_p = &name;                                                                              \
  }

int qdq(const TVMFFIAny *args, int32_t n, bool quantize) {
  char why[160];
  if (n < 3) return fail("expected (input, scale, output[, axis[, fp8_mode]])");
  QL_TENSOR(0, in, 0)
  QL_TENSOR(1, scale, 0)
  QL_TENSOR(2, out, 0)
  ql_qdq_attrs at = {0, 0, QL_FP8_DIRECT};
  int64_t v;
  if (n > 3 && int_arg(args[3], &v) && v >= 0) {
    at.has_axis = 1;
    at.axis = (int32_t)v;
  }
  if (n > 4 && int_arg(args[4], &v)) at.fp8_mode = (int32_t)v;
  void *st = stream_of(in_dl);
  return finish(quantize ? ql_quantize(&in, &scale, &out, &at, st) : ql_dequantize(&in, &scale, &out, &at, st));
}

} // namespace

extern "C" {

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_quantize(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) { return qdq(args, n, true); }
TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_dequantize(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) { return qdq(args, n, false); }

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_linear_w8a16(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 4) return fail("expected (x, w, scale, y)");
  QL_TENSOR(0, x, 0)
  QL_TENSOR(1, w, 0)
  QL_TENSOR(2, scale, 0)
  QL_TENSOR(3, y, 0)
  return finish(ql_linear_w8a16(&x, &w, &scale, &y, stream_of(x_dl)));
}

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_linear_w4a16(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 4) return fail("expected (x, w_packed, scale, y)");
  QL_TENSOR(0, x, 0)
  QL_TENSOR(1, w, 1)
  QL_TENSOR(2, scale, 0)
  QL_TENSOR(3, y, 0)
  return finish(ql_linear_w4a16(&x, &w, &scale, &y, stream_of(x_dl)));
}

static int gemm8(const TVMFFIAny *args, int32_t n, bool fp8) {
  char why[160];
  if (n != 5) return fail("expected (xq, wq, sx, sw, y)");
  QL_TENSOR(0, x, 0)
  QL_TENSOR(1, w, 0)
  QL_TENSOR(2, sx, 0)
  QL_TENSOR(3, sw, 0)
  QL_TENSOR(4, y, 0)
  void *st = stream_of(x_dl);
  return finish(fp8 ? ql_gemm_fp8(&x, &w, &sx, &sw, &y, st) : ql_gemm_i8(&x, &w, &sx, &sw, &y, st));
}
TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_gemm_fp8(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) { return gemm8(args, n, true); }
TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_gemm_i8(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) { return gemm8(args, n, false); }

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_gemm_16(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 4) return fail("expected (x, w, sw | None, y)");
  QL_TENSOR(0, x, 0)
  QL_TENSOR(1, w, 0)
  QL_OPTIONAL(2, sw)
  QL_TENSOR(3, y, 0)
  return finish(ql_gemm_16(&x, &w, sw_p, &y, stream_of(x_dl)));
}

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_linear(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 6) return fail("expected (x, w, sx | None, sw | None, bias | None, y)");
  QL_TENSOR(0, x, 0)
  QL_TENSOR(1, w, 0)
  QL_OPTIONAL(2, sx)
  QL_OPTIONAL(3, sw)
  QL_OPTIONAL(4, bias)
  QL_TENSOR(5, y, 0)
  return finish(ql_linear(&x, &w, sx_p, sw_p, bias_p, &y, stream_of(x_dl)));
}

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_matmul(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 3) return fail("expected (a, b, c)");
  QL_TENSOR(0, a, 0)
  QL_TENSOR(1, b, 0)
  QL_TENSOR(2, c, 0)
  return finish(ql_matmul(&a, &b, &c, stream_of(a_dl)));
}

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_dynamic_quantize(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n < 4) return fail("expected (input, double_quant_scale, data, scales[, axis[, block_size]])");
  QL_TENSOR(0, in, 0)
  QL_TENSOR(1, gs, 0)
  QL_TENSOR(2, data, 2)
  QL_TENSOR(3, scales, 0)
  int64_t axis = -1, block = 16, v;
  if (n > 4 && int_arg(args[4], &v)) axis = v;
  if (n > 5 && int_arg(args[5], &v)) block = v;
  if (axis < 0) axis += in.rank;
  return finish(ql_dynamic_quantize(&in, &gs, (int32_t)axis, (int32_t)block, &data, &scales, stream_of(in_dl)));
}

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_dequantize_nvfp4(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 4) return fail("expected (data, scales, double_quant_scale, output)");
  QL_TENSOR(0, data, 2)
  QL_TENSOR(1, scales, 0)
  QL_TENSOR(2, gs, 0)
  QL_TENSOR(3, out, 0)
  return finish(ql_dequantize_nvfp4(&data, &scales, &gs, &out, stream_of(data_dl)));
}

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_gemm_nvfp4(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 7) return fail("expected (a, a_scales, a_global | None, b, b_scales, b_global | None, y)");
  QL_TENSOR(0, a, 2)
  QL_TENSOR(1, sa, 0)
  QL_OPTIONAL(2, ga)
  QL_TENSOR(3, b, 2)
  QL_TENSOR(4, sb, 0)
  QL_OPTIONAL(5, gb)
  QL_TENSOR(6, y, 0)
  return finish(ql_gemm_nvfp4(&a, &sa, ga_p, &b, &sb, gb_p, &y, stream_of(a_dl)));
}

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_rmsnorm_quant_fp8(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 4) return fail("expected (x, eps, q, scale)");
  QL_TENSOR(0, x, 0)
  double eps;
  if (args[1].type_index == kTVMFFIFloat) eps = args[1].v_float64;
  else if (args[1].type_index == kTVMFFIInt) eps = (double)args[1].v_int64;
  else return fail("eps must be a number");
  QL_TENSOR(2, q, 0)
  QL_TENSOR(3, scale, 0)
  return finish(ql_rmsnorm_quant_fp8(&x, (float)eps, &q, &scale, stream_of(x_dl)));
}

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_gemm_fp8_swiglu(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 6) return fail("expected (xq, wq, sx, sw, act, row_amax)");
  QL_TENSOR(0, x, 0)
  QL_TENSOR(1, w, 0)
  QL_TENSOR(2, sx, 0)
  QL_TENSOR(3, sw, 0)
  QL_TENSOR(4, act, 0)
  QL_TENSOR(5, amax, 0)
  return finish(ql_gemm_fp8_swiglu(&x, &w, &sx, &sw, &act, &amax, stream_of(x_dl)));
}

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_quantize_rows_fp8(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 4) return fail("expected (act, row_amax, q, scale)");
  QL_TENSOR(0, a, 0)
  QL_TENSOR(1, amax, 0)
  QL_TENSOR(2, q, 0)
  QL_TENSOR(3, scale, 0)
  return finish(ql_quantize_rows_fp8(&a, &amax, &q, &scale, stream_of(a_dl)));
}
}
