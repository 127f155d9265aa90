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
//   ql_gemm_fp8(xq, wq, sx, sw, y)         ql_gemm_i8(xq, wq, sx, sw, y)
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

// DLTensor -> ql_tensor.  `as_int4` reinterprets a uint8 [N, K/2] tensor as int4 [N, K].
bool to_ql(const DLTensor *t, ql_tensor *out, bool as_int4, char *why, size_t why_len) {
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
    else if (d.code == kDLUInt && d.bits == 8) q = as_int4 ? QL_I4 : QL_F8E4M3; // raw bytes: packed int4 or e4m3 bits
  }
  if (q < 0) {
    snprintf(why, why_len, "unsupported tensor dtype (code %d, %d bits)", (int)d.code, (int)d.bits);
    return false;
  }
  out->data = static_cast<char *>(t->data) + t->byte_offset;
  out->dtype = q;
  out->rank = t->ndim;
  for (int i = 0; i < t->ndim; i++) out->shape[i] = t->shape[i];
  if (as_int4 && d.code == kDLUInt && t->ndim >= 1) out->shape[t->ndim - 1] *= 2;
  return true;
}

void *stream_of(const DLTensor *t) { return TVMFFIEnvGetStream(t->device.device_type, t->device.device_id); }

int finish(int rc) {
  if (rc == QL_OK) return 0;
  return fail(ql_last_error());
}

#define QL_TENSOR(idx, name, int4)                                                                  \
  ql_tensor name;                                                                                  \
  const DLTensor *name##_dl = (idx) < n ? tensor_arg(args[idx]) : nullptr;                         \
  if (!to_ql(name##_dl, &name, int4, why, sizeof(why))) return fail(why);

int qdq(const TVMFFIAny *args, int32_t n, bool quantize) {
  char why[160];
  if (n < 3) return fail("expected (input, scale, output[, axis[, fp8_mode]])");
  QL_TENSOR(0, in, false)
  QL_TENSOR(1, scale, false)
  QL_TENSOR(2, out, false)
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
  QL_TENSOR(0, x, false)
  QL_TENSOR(1, w, false)
  QL_TENSOR(2, scale, false)
  QL_TENSOR(3, y, false)
  return finish(ql_linear_w8a16(&x, &w, &scale, &y, stream_of(x_dl)));
}

TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_linear_w4a16(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) {
  char why[160];
  if (n != 4) return fail("expected (x, w_packed, scale, y)");
  QL_TENSOR(0, x, false)
  QL_TENSOR(1, w, true)
  QL_TENSOR(2, scale, false)
  QL_TENSOR(3, y, false)
  return finish(ql_linear_w4a16(&x, &w, &scale, &y, stream_of(x_dl)));
}

static int gemm8(const TVMFFIAny *args, int32_t n, bool fp8) {
  char why[160];
  if (n != 5) return fail("expected (xq, wq, sx, sw, y)");
  QL_TENSOR(0, x, false)
  QL_TENSOR(1, w, false)
  QL_TENSOR(2, sx, false)
  QL_TENSOR(3, sw, false)
  QL_TENSOR(4, y, false)
  void *st = stream_of(x_dl);
  return finish(fp8 ? ql_gemm_fp8(&x, &w, &sx, &sw, &y, st) : ql_gemm_i8(&x, &w, &sx, &sw, &y, st));
}
TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_gemm_fp8(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) { return gemm8(args, n, true); }
TVM_FFI_DLL_EXPORT int __tvm_ffi_ql_gemm_i8(void *, const TVMFFIAny *args, int32_t n, TVMFFIAny *) { return gemm8(args, n, false); }
}
