// General matrix product on the CUDA cores, for every shape and alignment the tensor-core kernels refuse:
//     Y[b][m,n] = (sum_k A[b][m,k] * B[b][k,n]) * sa[m] * sb[n] + bias[n]
// with f32 accumulation (s32 for int8), operands f32 / f16 / bf16 / e4m3 / int8 addressed through
// element strides (so B may be stored [N,K] as Linear holds its weight, or [K,N] as `a @ b` passes it, and a
// leading batch dimension may be broadcast with stride 0), result f32 / f16 / bf16.
//
// It is what makes the operator layer a drop-in at the points the reference pins with known answers:
// tp.Linear defaults to float32 (tripy/nvtripy/frontend/module/linear.py:65) and its tests use in_features = 4
// (tripy/tests/integration/test_linear.py:52-150); the int4 dequantize -> matmul answer uses K = 2
// (mlir-tensorrt/compiler/test/python/IntegrationTests/test_tensorrt10_data_type_support.py:218-246).  It is also
// tensorrt.matrix_multiply (TensorRTOps.td:1986-2080) / tp.matmul (tripy/nvtripy/frontend/ops/matmul.py:29-108)
// for float32 operands.  64 x 64 output tile per block, 16-deep k slices through shared memory, 4 x 4 outputs per
// thread; loads are scalar and bounds-checked, so nothing is assumed about K, strides or pointers.
#include "ql_common.cuh"

namespace ql {
namespace {

constexpr int TM = 64, TN = 64, TK = 16, kSimtThreads = 256;

struct SimtArgs {
  const void *A, *B;
  void *Y;
  const float *sa; // null, one value (sa_n == 1) or one per row
  const float *sb; // null, one value (sb_n == 1) or one per column
  const void *bias; // null or one value per column, of type bias_dtype
  int bias_dtype, y_dtype;
  int sa_n, sb_n;
  int M, N, K;
  int64_t a_m, a_k, b_k, b_n, ldy; // element strides
  int64_t a_batch, b_batch, y_batch;
};

template <typename T> struct Elem;
template <> struct Elem<float> { using Acc = float; __device__ static float get(const float *p, int64_t i) { return p[i]; } };
template <> struct Elem<__half> { using Acc = float; __device__ static float get(const __half *p, int64_t i) { return __half2float(p[i]); } };
template <> struct Elem<__nv_bfloat16> { using Acc = float; __device__ static float get(const __nv_bfloat16 *p, int64_t i) { return __bfloat162float(p[i]); } };
template <> struct Elem<__nv_fp8_e4m3> {
  using Acc = float;
  __device__ static float get(const __nv_fp8_e4m3 *p, int64_t i) { return e4m3x2_to_f32x2(reinterpret_cast<const uint8_t *>(p)[i]).x; }
};
template <> struct Elem<int8_t> { using Acc = int; __device__ static int get(const int8_t *p, int64_t i) { return (int)p[i]; } };

template <typename T>
__global__ void __launch_bounds__(kSimtThreads) gemm_simt_kernel(const SimtArgs a) {
  using Acc = typename Elem<T>::Acc;
  __shared__ Acc As[TK][TM + 4];
  __shared__ Acc Bs[TK][TN + 4];
  const int b = blockIdx.z;
  const T *A = static_cast<const T *>(a.A) + (int64_t)b * a.a_batch;
  const T *B = static_cast<const T *>(a.B) + (int64_t)b * a.b_batch;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  Acc acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0;

  for (int k0 = 0; k0 < a.K; k0 += TK) {
    // 64 x 16 elements of each operand, four per thread; k runs fastest over threads
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int e = threadIdx.x + i * kSimtThreads;
      const int kk = e & 15, r = e >> 4;
      const int k = k0 + kk, m = m0 + r, n = n0 + r;
      As[kk][r] = (m < a.M && k < a.K) ? Elem<T>::get(A, (int64_t)m * a.a_m + (int64_t)k * a.a_k) : Acc(0);
      Bs[kk][r] = (n < a.N && k < a.K) ? Elem<T>::get(B, (int64_t)k * a.b_k + (int64_t)n * a.b_n) : Acc(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk++) {
      Acc av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += av[i] * bv[j]; // one fused multiply-add per product, k rising
    }
    __syncthreads();
  }

  const float sb1 = (a.sb && a.sb_n == 1) ? a.sb[0] : 1.f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= a.M) continue;
    const float sa = a.sa ? (a.sa_n == 1 ? a.sa[0] : a.sa[m]) : 1.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n >= a.N) continue;
      const float sb = (a.sb && a.sb_n != 1) ? a.sb[n] : sb1;
      float v = (float)acc[i][j];
      if (a.sa || a.sb) v *= sa * sb;
      if (a.bias) v += load_scale(a.bias, a.bias_dtype, n);
      const int64_t o = (int64_t)b * a.y_batch + (int64_t)m * a.ldy + n;
      if (a.y_dtype == QL_F32) static_cast<float *>(a.Y)[o] = v;
      else if (a.y_dtype == QL_F16) static_cast<__half *>(a.Y)[o] = __float2half_rn(v);
      else static_cast<__nv_bfloat16 *>(a.Y)[o] = __float2bfloat16_rn(v);
    }
  }
}

} // namespace

// Launches the general product.  `dtype` is the operands' type; strides are in elements.
int launch_gemm_simt(int dtype, const void *A, const void *B, const float *sa, int sa_n, const float *sb, int sb_n, const void *bias,
                     int bias_dtype, void *Y, int y_dtype, int batch, int M, int N, int K, int64_t a_m, int64_t a_k, int64_t b_k,
                     int64_t b_n, int64_t ldy, int64_t a_batch, int64_t b_batch, int64_t y_batch, cudaStream_t st) {
  if (batch <= 0 || M <= 0 || N <= 0) return QL_OK;
  if (batch > 65535) return set_error(QL_ERR_UNSUPPORTED, "matmul: more than 65535 matrices in a batch");
  SimtArgs a;
  a.A = A; a.B = B; a.Y = Y; a.sa = sa; a.sb = sb; a.bias = bias;
  a.bias_dtype = bias_dtype; a.y_dtype = y_dtype; a.sa_n = sa_n; a.sb_n = sb_n;
  a.M = M; a.N = N; a.K = K;
  a.a_m = a_m; a.a_k = a_k; a.b_k = b_k; a.b_n = b_n; a.ldy = ldy;
  a.a_batch = a_batch; a.b_batch = b_batch; a.y_batch = y_batch;
  const dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, batch);
  if (grid.y > 65535) return set_error(QL_ERR_UNSUPPORTED, "matmul: M too large for the general kernel");
  switch (dtype) {
  case QL_F32: gemm_simt_kernel<float><<<grid, kSimtThreads, 0, st>>>(a); break;
  case QL_F16: gemm_simt_kernel<__half><<<grid, kSimtThreads, 0, st>>>(a); break;
  case QL_BF16: gemm_simt_kernel<__nv_bfloat16><<<grid, kSimtThreads, 0, st>>>(a); break;
  case QL_F8E4M3: gemm_simt_kernel<__nv_fp8_e4m3><<<grid, kSimtThreads, 0, st>>>(a); break;
  case QL_I8: gemm_simt_kernel<int8_t><<<grid, kSimtThreads, 0, st>>>(a); break;
  default: return set_error(QL_ERR_INVALID_ARGUMENT, "matmul: operands must be f32, f16, bf16, e4m3 or int8");
  }
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

} // namespace ql
