// Row kernels of the quantized Llama-style MLP block (benchmark config 5): RMSNorm fused with the
// dynamic per-token e4m3 quantization of the activations, and SwiGLU fused with the per-token
// re-quantization that feeds the down projection.  Neither is a reference operator; they are the
// compositions reduce/rsqrt/multiply -> tensorrt.quantize and logistic/multiply ->
// tensorrt.quantize that a StableHLO program for the block would contain, with the quantize step
// keeping the reference's arithmetic (f32 division by the scale, saturating e4m3 conversion).
// Both stream each row once from HBM (the second pass over a row hits L1/L2) and are bounded by
// HBM bandwidth.
#include "ql_common.cuh"

namespace ql {
namespace {

constexpr int kRowThreads = 256;

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One block per token.  r = x * rsqrt(mean(x^2) + eps); s = max|r| / 448; q = e4m3(r / s).
// mean(x^2) is accumulated in f64 so that the result does not depend on how the row is split
// over threads (up to the last bit of the f64 sum).
template <typename XT>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_quant_fp8_kernel(const XT *__restrict__ X, uint8_t *__restrict__ Q, float *__restrict__ S, int H, float eps) {
  constexpr int kPer16 = 16 / sizeof(XT);
  const int64_t row = blockIdx.x;
  const XT *x = X + row * H;
  uint8_t *q = Q + row * H;
  const int n_words = H / kPer16; // H % 16 == 0 is checked by the host
  double ss = 0.0;
  float amax = 0.f;
  for (int w = threadIdx.x; w < n_words; w += kRowThreads) {
    float v[kPer16];
    load_vec_f32<XT, kPer16>(x + w * kPer16, v);
#pragma unroll
    for (int j = 0; j < kPer16; j++) {
      ss += (double)v[j] * (double)v[j];
      amax = fmaxf(amax, fabsf(v[j]));
    }
  }
  __shared__ double part_ss[kRowThreads / 32];
  __shared__ float part_mx[kRowThreads / 32];
  __shared__ float s_rinv, s_scale;
  ss = warp_sum_f64(ss);
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) {
    part_ss[threadIdx.x >> 5] = ss;
    part_mx[threadIdx.x >> 5] = amax;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    float m = 0.f;
    for (int i = 0; i < kRowThreads / 32; i++) {
      t += part_ss[i];
      m = fmaxf(m, part_mx[i]);
    }
    const float rinv = (float)(1.0 / sqrt(t / (double)H + (double)eps));
    // rounding is monotonic, so max|x * rinv| over the row is |x|max * rinv rounded once
    float s = __fdiv_rn(__fmul_rn(m, rinv), 448.f);
    if (s == 0.f) s = 1.f;
    s_rinv = rinv;
    s_scale = s;
    S[row] = s;
  }
  __syncthreads();
  const float rinv = s_rinv;
  const SharedDivisor by_s(s_scale);
  // second pass: the row is still in L1/L2; 16 values -> one 16-byte store
  const int n_chunks = H / 16;
  for (int c = threadIdx.x; c < n_chunks; c += kRowThreads) {
    float v[16];
    load_vec_f32<XT, 16>(x + c * 16, v);
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = __fmul_rn(v[j], rinv);
    by_s.divide(v);
#pragma unroll
    for (int j = 0; j < 16; j += 2) w[j >> 2] |= (f32x2_to_e4m3x2(v[j], v[j + 1]) & 0xFFFFu) << (8 * (j & 3));
    __stcs(reinterpret_cast<uint4 *>(q) + c, make_uint4(w[0], w[1], w[2], w[3]));
  }
}

// The same for rows of at most 16 * P * 256 values, read from HBM once: every thread keeps its P groups of 16 values
// (two 16-byte words of 16-bit data) in registers between the reduction and the quantize pass, and all of its loads
// are in flight together.
template <typename XT, int P>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_quant_fp8_regs_kernel(const XT *__restrict__ X, uint8_t *__restrict__ Q, float *__restrict__ S, int H, float eps) {
  static_assert(sizeof(XT) == 2, "two 16-byte words per group of 16 values");
  const int64_t row = blockIdx.x;
  const uint4 *x = reinterpret_cast<const uint4 *>(X + row * H);
  uint4 *q = reinterpret_cast<uint4 *>(Q + row * H);
  const int n_groups = H / 16;
  uint4 raw[P][2];
#pragma unroll
  for (int i = 0; i < P; i++) {
    const int g = threadIdx.x + i * kRowThreads;
    if (g < n_groups) {
      raw[i][0] = __ldcs(x + 2 * g);
      raw[i][1] = __ldcs(x + 2 * g + 1);
    } else {
      raw[i][0] = raw[i][1] = make_uint4(0, 0, 0, 0);
    }
  }
  double ss = 0.0;
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < P; i++) {
    const XT *e = reinterpret_cast<const XT *>(&raw[i][0]);
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const float v = FloatIO<XT>::to_f32(e[j]);
      ss += (double)v * (double)v;
      amax = fmaxf(amax, fabsf(v));
    }
  }
  __shared__ double part_ss[kRowThreads / 32];
  __shared__ float part_mx[kRowThreads / 32];
  __shared__ float s_rinv, s_scale;
  ss = warp_sum_f64(ss);
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) {
    part_ss[threadIdx.x >> 5] = ss;
    part_mx[threadIdx.x >> 5] = amax;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    float m = 0.f;
    for (int i = 0; i < kRowThreads / 32; i++) {
      t += part_ss[i];
      m = fmaxf(m, part_mx[i]);
    }
    const float rinv = (float)(1.0 / sqrt(t / (double)H + (double)eps));
    float s = __fdiv_rn(__fmul_rn(m, rinv), 448.f);
    if (s == 0.f) s = 1.f;
    s_rinv = rinv;
    s_scale = s;
    S[row] = s;
  }
  __syncthreads();
  const float rinv = s_rinv;
  const SharedDivisor by_s(s_scale);
#pragma unroll
  for (int i = 0; i < P; i++) {
    const int g = threadIdx.x + i * kRowThreads;
    if (g >= n_groups) break;
    const XT *e = reinterpret_cast<const XT *>(&raw[i][0]);
    uint32_t w[4] = {0, 0, 0, 0};
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = __fmul_rn(FloatIO<XT>::to_f32(e[j]), rinv);
    by_s.divide(v);
#pragma unroll
    for (int j = 0; j < 16; j += 2) w[j >> 2] |= (f32x2_to_e4m3x2(v[j], v[j + 1]) & 0xFFFFu) << (8 * (j & 3));
    __stcs(q + g, make_uint4(w[0], w[1], w[2], w[3]));
  }
}

// One block per token.  GU holds [gate | up] (I columns each); a = silu(gate) * up in f32;
// s = max|a| / 448; q = e4m3(a / s).  The f32 products of the first pass are parked in shared
// memory (kCache) so that expf runs once per element; rows too long for that are recomputed.
template <typename XT, bool kCache>
__global__ void __launch_bounds__(kRowThreads)
swiglu_quant_fp8_kernel(const XT *__restrict__ GU, uint8_t *__restrict__ Q, float *__restrict__ S, int I) {
  extern __shared__ __align__(16) float a_cache[];
  const int64_t row = blockIdx.x;
  const XT *g = GU + row * 2 * I, *u = g + I;
  uint8_t *q = Q + row * I;
  const int n_chunks = I / 16;
  float amax = 0.f;
  for (int c = threadIdx.x; c < n_chunks; c += kRowThreads) {
    float gv[16], uv[16];
    load_vec_f32<XT, 16>(g + c * 16, gv);
    load_vec_f32<XT, 16>(u + c * 16, uv);
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const float a = silu_mul(gv[j], uv[j]);
      amax = fmaxf(amax, fabsf(a));
      gv[j] = a;
    }
    if constexpr (kCache) {
#pragma unroll
      for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4 *>(a_cache + c * 16 + j) = make_float4(gv[j], gv[j + 1], gv[j + 2], gv[j + 3]);
    }
  }
  __shared__ float part[kRowThreads / 32];
  __shared__ float s_scale;
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < kRowThreads / 32; i++) m = fmaxf(m, part[i]);
    float s = __fdiv_rn(m, 448.f);
    if (s == 0.f) s = 1.f;
    s_scale = s;
    S[row] = s;
  }
  __syncthreads();
  const SharedDivisor by_s(s_scale);
  for (int c = threadIdx.x; c < n_chunks; c += kRowThreads) {
    float av[16];
    if constexpr (kCache) {
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        const float4 t = *reinterpret_cast<const float4 *>(a_cache + c * 16 + j);
        av[j] = t.x; av[j + 1] = t.y; av[j + 2] = t.z; av[j + 3] = t.w;
      }
    } else {
      float gv[16], uv[16];
      load_vec_f32<XT, 16>(g + c * 16, gv);
      load_vec_f32<XT, 16>(u + c * 16, uv);
#pragma unroll
      for (int j = 0; j < 16; j++) av[j] = silu_mul(gv[j], uv[j]);
    }
    by_s.divide(av);
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; j += 2)
      w[j >> 2] |= (f32x2_to_e4m3x2(av[j], av[j + 1]) & 0xFFFFu) << (8 * (j & 3));
    __stcs(reinterpret_cast<uint4 *>(q) + c, make_uint4(w[0], w[1], w[2], w[3]));
  }
}

// q[t, :] = e4m3(a[t, :] / s[t]) with s[t] = amax[t] / 448 (1 where the row is all zero): tensorrt.quantize per
// channel along axis 0 with the scale formed on the fly from row maxima that an earlier kernel left in `amax`
// (the SwiGLU epilogue of the gate/up projection).  16 values per thread: 32 bytes in, 16 bytes out.
template <typename XT>
__global__ void __launch_bounds__(256) quantize_rows_fp8_kernel(const XT *__restrict__ A, const float *__restrict__ amax, uint8_t *__restrict__ Q,
                                                                float *__restrict__ S, int64_t n_chunks, int chunks_per_row) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks; c += stride) {
    const int64_t row = c / chunks_per_row;
    float s = __fdiv_rn(__ldg(amax + row), 448.f);
    if (s == 0.f) s = 1.f;
    if (c - row * chunks_per_row == 0) S[row] = s;
    float v[16];
    load_vec_f32<XT, 16>(A + c * 16, v);
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; j += 2)
      w[j >> 2] |= (f32x2_to_e4m3x2(__fdiv_rn(v[j], s), __fdiv_rn(v[j + 1], s)) & 0xFFFFu) << (8 * (j & 3));
    __stcs(reinterpret_cast<uint4 *>(Q) + c, make_uint4(w[0], w[1], w[2], w[3]));
  }
}

// The same for long rows.  A work item is a segment of at most 256 * kQU chunks of one row, so the scale is formed once
// per thread and item and no index is divided per chunk; the blocks stay resident and walk the items with the grid's
// stride, and in every item a thread issues all of its loads before it reads the row maximum, so that the latency of
// that dependent load is hidden behind them.  Two chunks per thread and five blocks per SM measured best (64 us on
// 4096 x 28672; four chunks and three blocks: 80 us; one chunk and six blocks: 73 us).
constexpr int kQU = 2;
template <typename XT>
__global__ void __launch_bounds__(256, 5) quantize_rows_fp8_seg_kernel(const XT *__restrict__ A, const float *__restrict__ amax, uint8_t *__restrict__ Q,
                                                                    float *__restrict__ S, int chunks_per_row, int segs, int per_seg, int n_items) {
  static_assert(sizeof(XT) == 2, "two 16-byte words per chunk of 16 values");
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int row = item / segs, seg = item - row * segs;
    const int c_end = min(chunks_per_row, (seg + 1) * per_seg); // per_seg <= 256 * kQU: one trip per item
    const int c0 = seg * per_seg + threadIdx.x;
    const uint4 *a = reinterpret_cast<const uint4 *>(A) + (int64_t)row * chunks_per_row * 2;
    uint4 *q = reinterpret_cast<uint4 *>(Q) + (int64_t)row * chunks_per_row;
    uint4 raw[kQU][2];
#pragma unroll
    for (int u = 0; u < kQU; u++) {
      const int c = c0 + u * 256;
      if (c < c_end) {
        raw[u][0] = __ldcs(a + 2 * c);
        raw[u][1] = __ldcs(a + 2 * c + 1);
      }
    }
    float s = __fdiv_rn(__ldg(amax + row), 448.f);
    if (s == 0.f) s = 1.f;
    if (seg == 0 && threadIdx.x == 0) S[row] = s;
    const SharedDivisor by_s(s);
#pragma unroll
    for (int u = 0; u < kQU; u++) {
      const int c = c0 + u * 256;
      if (c >= c_end) break;
      const XT *e = reinterpret_cast<const XT *>(&raw[u][0]);
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; j++) v[j] = FloatIO<XT>::to_f32(e[j]);
      by_s.divide(v);
      uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
      for (int j = 0; j < 16; j += 2) w[j >> 2] |= (f32x2_to_e4m3x2(v[j], v[j + 1]) & 0xFFFFu) << (8 * (j & 3));
      __stcs(q + c, make_uint4(w[0], w[1], w[2], w[3]));
    }
  }
}

template <typename XT>
int launch_swiglu(const void *gu, void *q, void *s, int64_t T, int64_t I, cudaStream_t st) {
  const size_t cache_bytes = (size_t)I * sizeof(float);
  const XT *g = static_cast<const XT *>(gu);
  if (cache_bytes <= 200 * 1024) {
    auto kern = swiglu_quant_fp8_kernel<XT, true>;
    static bool configured[64] = {false};
    int dev = 0;
    QL_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      QL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      configured[dev] = true;
    }
    kern<<<(unsigned)T, kRowThreads, cache_bytes, st>>>(g, static_cast<uint8_t *>(q), static_cast<float *>(s), (int)I);
  } else {
    swiglu_quant_fp8_kernel<XT, false><<<(unsigned)T, kRowThreads, 0, st>>>(g, static_cast<uint8_t *>(q), static_cast<float *>(s), (int)I);
  }
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

int check_rows(const char *op, const ql_tensor *x, const ql_tensor *q, const ql_tensor *s, int64_t cols_in, int64_t cols_out) {
  if (!x || !q || !s) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  if (x->rank != 2 || q->rank != 2 || s->rank != 1) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: expected x [T,C], q [T,C'], scale [T]", op);
  if (!(x->dtype == QL_BF16 || x->dtype == QL_F16)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: x must be bf16 or f16", op);
  if (q->dtype != QL_F8E4M3 || s->dtype != QL_F32) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: q must be e4m3 and scale f32", op);
  if (x->shape[1] != cols_in || q->shape[1] != cols_out || q->shape[0] != x->shape[0] || s->shape[0] != x->shape[0])
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: shapes do not agree", op);
  if (cols_out % 16 != 0) return set_error(QL_ERR_UNSUPPORTED, "%s: the row length must be a multiple of 16 (got %lld)", op, (long long)cols_out);
  if (!aligned16(x->data) || !aligned16(q->data)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: x and q must be 16-byte aligned", op);
  if (x->shape[0] > INT32_MAX || cols_in > INT32_MAX) return set_error(QL_ERR_UNSUPPORTED, "%s: dimension too large", op);
  return QL_OK;
}

} // namespace
} // namespace ql

using namespace ql;

extern "C" {

int ql_rmsnorm_quant_fp8(const ql_tensor *x, float eps, ql_tensor *q, ql_tensor *scale, void *stream) {
  const char *op = "rmsnorm_quant_fp8";
  if (!x) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  int rc = check_rows(op, x, q, scale, x->rank == 2 ? x->shape[1] : 0, x->rank == 2 ? x->shape[1] : 0);
  if (rc != QL_OK) return rc;
  const int64_t T = x->shape[0], H = x->shape[1];
  if (T == 0) return QL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t *qp = static_cast<uint8_t *>(q->data);
  float *sp = static_cast<float *>(scale->data);
  const int groups = (int)(H / 16);
#define QL_RMS(XT)                                                                                                             \
  do {                                                                                                                         \
    const XT *xp = static_cast<const XT *>(x->data);                                                                           \
    if (groups <= kRowThreads) rmsnorm_quant_fp8_regs_kernel<XT, 1><<<(unsigned)T, kRowThreads, 0, st>>>(xp, qp, sp, (int)H, eps); \
    else if (groups <= 2 * kRowThreads) rmsnorm_quant_fp8_regs_kernel<XT, 2><<<(unsigned)T, kRowThreads, 0, st>>>(xp, qp, sp, (int)H, eps); \
    else rmsnorm_quant_fp8_kernel<XT><<<(unsigned)T, kRowThreads, 0, st>>>(xp, qp, sp, (int)H, eps);                            \
  } while (0)
  if (x->dtype == QL_BF16) QL_RMS(__nv_bfloat16);
  else QL_RMS(__half);
#undef QL_RMS
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

int ql_quantize_rows_fp8(const ql_tensor *a, const ql_tensor *row_amax, ql_tensor *q, ql_tensor *scale, void *stream) {
  const char *op = "quantize_rows_fp8";
  if (!a || !row_amax) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  int rc = check_rows(op, a, q, scale, a->rank == 2 ? a->shape[1] : 0, a->rank == 2 ? a->shape[1] : 0);
  if (rc != QL_OK) return rc;
  if (row_amax->dtype != QL_F32 || row_amax->rank != 1 || row_amax->shape[0] != a->shape[0] || (!row_amax->data && a->shape[0] > 0))
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: row_amax must be f32 [T]", op);
  const int64_t T = a->shape[0], I = a->shape[1];
  if (T == 0 || I == 0) return QL_OK;
  const int64_t n_chunks = T * (I / 16);
  cudaStream_t st = (cudaStream_t)stream;
  const float *am = static_cast<const float *>(row_amax->data);
  uint8_t *qp = static_cast<uint8_t *>(q->data);
  float *sp = static_cast<float *>(scale->data);
  const int cpr = (int)(I / 16);
  if (cpr >= 256 && T * ((cpr + 256 * kQU - 1) / (256 * kQU)) <= INT32_MAX) {
    // long rows: work items of one row segment of at most 256 * kQU chunks, walked by a resident grid
    const int segs = (cpr + 256 * kQU - 1) / (256 * kQU), per_seg = (cpr + segs - 1) / segs;
    const int n_items = (int)(T * segs);
    const int grid = n_items < sm_count() * 5 ? n_items : sm_count() * 5;
    if (a->dtype == QL_BF16)
      quantize_rows_fp8_seg_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(a->data), am, qp, sp, cpr, segs, per_seg, n_items);
    else
      quantize_rows_fp8_seg_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half *>(a->data), am, qp, sp, cpr, segs, per_seg, n_items);
  } else {
    int64_t blocks = (n_chunks + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (a->dtype == QL_BF16)
      quantize_rows_fp8_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(a->data), am, qp, sp, n_chunks, cpr);
    else
      quantize_rows_fp8_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __half *>(a->data), am, qp, sp, n_chunks, cpr);
  }
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

int ql_swiglu_quant_fp8(const ql_tensor *gate_up, ql_tensor *q, ql_tensor *scale, void *stream) {
  const char *op = "swiglu_quant_fp8";
  if (!gate_up || !q) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  int rc = check_rows(op, gate_up, q, scale, q->rank == 2 ? 2 * q->shape[1] : 0, q->rank == 2 ? q->shape[1] : 0);
  if (rc != QL_OK) return rc;
  const int64_t T = gate_up->shape[0], I = q->shape[1];
  if (T == 0) return QL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (gate_up->dtype == QL_BF16) return launch_swiglu<__nv_bfloat16>(gate_up->data, q->data, scale->data, T, I, st);
  return launch_swiglu<__half>(gate_up->data, q->data, scale->data, T, I, st);
}
}
