// Tensor-core GEMM entry points (placeholder until the tcgen05 kernels land in this file).
#include "ql_common.cuh"

using namespace ql;

extern "C" {

int ql_gemm_fp8(const ql_tensor *, const ql_tensor *, const ql_tensor *, const ql_tensor *, ql_tensor *, void *) {
  return set_error(QL_ERR_UNSUPPORTED, "gemm_fp8: not built yet");
}
int ql_gemm_i8(const ql_tensor *, const ql_tensor *, const ql_tensor *, const ql_tensor *, ql_tensor *, void *) {
  return set_error(QL_ERR_UNSUPPORTED, "gemm_i8: not built yet");
}
int ql_gemm_16(const ql_tensor *, const ql_tensor *, const ql_tensor *, ql_tensor *, void *) {
  return set_error(QL_ERR_UNSUPPORTED, "gemm_16: not built yet");
}
}
