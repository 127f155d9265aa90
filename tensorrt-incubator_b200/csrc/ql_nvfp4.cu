// NVFP4: tensorrt.dynamic_quantize and its inverse
// (tensorrt/include/mlir-tensorrt-dialect/TensorRT/IR/TensorRTOps.td:3279-3358, verifier
// tensorrt/lib/TensorRT/IR/Verification.cpp:1270-1290).  Blocks of 16 values along the last axis share one e4m3
// scale = (max|x| / 6) / double_quant_scale; the data are x / (scale * double_quant_scale) in e2m1, two per byte
// with the first element in the low nibble.  Conversions are the PTX ones the reference's kernel backend emits
// (cvt.rn.satfinite.e2m1x2.f32, kernel/lib/Kernel/Transforms/LowerToNVVM.cpp:339-392; cvt.rn.f16x2.e2m1x2, :466-527).
// One thread owns one block: 64 (f32) or 32 (16-bit) contiguous input bytes in, 8 data bytes and 1 scale byte out,
// so a warp reads 1-2 KiB contiguous.  HBM-bound: 4.5625 (f32) or 2.5625 (16-bit) bytes per element.
#include "ql_common.cuh"

namespace ql {
namespace {

constexpr int kThreadsF4 = 256;

// (lo, hi) -> one byte holding two e2m1 values, lo in the low nibble
__device__ __forceinline__ uint32_t f32x2_to_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %2, %1;\n\tcvt.u32.u8 %0, t;\n\t}" : "=r"(r) : "f"(lo), "f"(hi));
  return r;
}

// one byte of two e2m1 values -> (lo, hi) as f32
__device__ __forceinline__ float2 e2m1x2_to_f32x2(uint32_t byte) {
  uint32_t h2;
  asm("{\n\t.reg .b8 t;\n\tcvt.u8.u32 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(h2) : "r"(byte));
  return __half22float2(*reinterpret_cast<__half2 *>(&h2));
}

constexpr int kUnrollF4 = 4; // blocks whose loads one thread has in flight at once

// (Keeping several blocks' loads in flight per thread, as the dequantize kernel does, was measured slower here:
// 64 more live registers for 75 us against 47 us.)
template <typename InT>
__global__ void __launch_bounds__(kThreadsF4)
nvfp4_quantize_kernel(const InT *__restrict__ x, const void *__restrict__ gs, int gsdt, uint8_t *__restrict__ q,
                      uint8_t *__restrict__ scales, int64_t nblocks) {
  const float g = load_scale(gs, gsdt, 0);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += stride) {
    float v[16];
    load_vec_f32<InT, 16>(x + b * 16, v);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(v[i]));
    const uint32_t sq = f32x2_to_e4m3x2(__fdiv_rn(__fdiv_rn(amax, 6.f), g), 0.f) & 0xFFu;
    const float s = e4m3x2_to_f32x2(sq).x * g;
    uint32_t w[2] = {0u, 0u};
    if (s != 0.f) { // a block whose scale rounds to zero quantizes to zeros
      const SharedDivisor by_s(s);
      by_s.divide(v);
#pragma unroll
      for (int i = 0; i < 16; i += 2) w[i >> 3] |= f32x2_to_e2m1x2(v[i], v[i + 1]) << (4 * (i & 7));
    }
    *reinterpret_cast<uint2 *>(q + b * 8) = make_uint2(w[0], w[1]);
    scales[b] = (uint8_t)sq;
  }
}

template <typename OutT>
__global__ void __launch_bounds__(kThreadsF4)
nvfp4_dequantize_kernel(const uint8_t *__restrict__ q, const uint8_t *__restrict__ scales, const void *__restrict__ gs, int gsdt,
                        OutT *__restrict__ y, int64_t nblocks) {
  const float g = load_scale(gs, gsdt, 0);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t b0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b0 < nblocks; b0 += stride * kUnrollF4) {
    uint2 w[kUnrollF4];
    uint32_t sq[kUnrollF4];
#pragma unroll
    for (int u = 0; u < kUnrollF4; u++) {
      const int64_t b = b0 + u * stride;
      if (b < nblocks) {
        w[u] = __ldcs(reinterpret_cast<const uint2 *>(q + b * 8));
        sq[u] = scales[b];
      }
    }
#pragma unroll
    for (int u = 0; u < kUnrollF4; u++) {
      const int64_t b = b0 + u * stride;
      if (b >= nblocks) break;
      const float s = e4m3x2_to_f32x2(sq[u]).x * g;
      const uint32_t ww[2] = {w[u].x, w[u].y};
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        const float2 f = e2m1x2_to_f32x2((ww[i >> 3] >> (4 * (i & 7))) & 0xFFu);
        v[i] = f.x * s;
        v[i + 1] = f.y * s;
      }
      store_vec_f32<OutT, 16>(y + b * 16, v);
    }
  }
}

// tensorrt.dequantize of e2m1 data with floating-point block scales along the last axis (the second step of the
// operator's documented use: the scales are themselves the result of dequantizing the e4m3 block scales).
// One thread per 16 values; `block` (a multiple of 16) values share one scale.
template <typename OutT>
__global__ void __launch_bounds__(kThreadsF4)
f4_block_dequantize_kernel(const uint8_t *__restrict__ q, const void *__restrict__ scale, int sdt, OutT *__restrict__ y, int64_t n16,
                           int chunks_per_scale) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < n16; b += stride) {
    const uint2 w = __ldcs(reinterpret_cast<const uint2 *>(q + b * 8));
    const float s = load_scale(scale, sdt, b / chunks_per_scale);
    const uint32_t ww[2] = {w.x, w.y};
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const float2 f = e2m1x2_to_f32x2((ww[i >> 3] >> (4 * (i & 7))) & 0xFFu);
      v[i] = f.x * s;
      v[i + 1] = f.y * s;
    }
    store_vec_f32<OutT, 16>(y + b * 16, v);
  }
}

int64_t numel_of(const ql_tensor *t) {
  int64_t n = 1;
  for (int i = 0; i < t->rank; i++) n *= t->shape[i];
  return n;
}

// shared argument rules; `x` is the floating-point side ([..., K]), `q` the e2m1 side, `s` the e4m3 block scales
int check_nvfp4(const char *op, const ql_tensor *x, const ql_tensor *gs, const ql_tensor *q, const ql_tensor *s) {
  if (!x || !gs || !q || !s) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  if (!(x->dtype == QL_F32 || x->dtype == QL_F16 || x->dtype == QL_BF16))
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: the floating-point tensor must be f32, f16 or bf16", op);
  if (!(gs->dtype == QL_F32 || gs->dtype == QL_F16 || gs->dtype == QL_BF16) || gs->rank != 0)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: double_quant_scale must be a rank-0 f32, f16 or bf16 tensor", op);
  if (q->dtype != QL_F4E2M1 || s->dtype != QL_F8E4M3) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: data must be f4E2M1FN and scales f8E4M3FN", op);
  if (x->rank < 1 || x->rank > QL_MAX_RANK || q->rank != x->rank || s->rank != x->rank)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: input, result and scales must have the same rank", op);
  for (int i = 0; i < x->rank; i++) {
    if (q->shape[i] != x->shape[i]) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: data and floating-point tensor differ in shape", op);
    const int64_t want = (i == x->rank - 1) ? x->shape[i] / 16 : x->shape[i];
    if (s->shape[i] != want) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: scales must have one entry per block of 16 along the last axis", op);
  }
  if (numel_of(x) > 0 && (!x->data || !q->data || !s->data || !gs->data)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: tensor without data", op);
  if (!aligned16(x->data) || (reinterpret_cast<uintptr_t>(q->data) & 7)) return set_error(QL_ERR_UNSUPPORTED, "%s: buffers must be 16-byte (data: 8-byte) aligned", op);
  return QL_OK;
}

unsigned grid_for(int64_t nblocks, int per_thread) {
  int64_t blocks = (nblocks + kThreadsF4 * per_thread - 1) / (kThreadsF4 * per_thread);
  const int64_t cap = (int64_t)sm_count() * 8;
  return (unsigned)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

} // namespace

// q: e2m1 [..., K]; scale: f32 | f16 | bf16 [..., K / block], block % 16 == 0; y: [..., K].  Called by ql_dequantize.
int launch_f4_block_dequantize(const ql_tensor *q, const ql_tensor *scale, ql_tensor *y, cudaStream_t st) {
  const char *op = "tensorrt.dequantize";
  if (q->rank < 1 || scale->rank != q->rank)
    return set_error(QL_ERR_UNSUPPORTED, "%s: f4E2M1FN input is dequantized with block scales of the input's rank", op);
  for (int i = 0; i + 1 < q->rank; i++)
    if (scale->shape[i] != q->shape[i]) return set_error(QL_ERR_UNSUPPORTED, "%s: f4E2M1FN blocks must run along the last axis", op);
  const int64_t K = q->shape[q->rank - 1], nb = scale->shape[q->rank - 1];
  if (nb <= 0 || K % nb != 0 || (K / nb) % 16 != 0)
    return set_error(QL_ERR_UNSUPPORTED, "%s: f4E2M1FN block size must be a multiple of 16 (last axis %lld, %lld scales)", op, (long long)K, (long long)nb);
  const int64_t n16 = numel_of(q) / 16;
  if (n16 == 0) return QL_OK;
  if (!aligned16(y->data) || (reinterpret_cast<uintptr_t>(q->data) & 7)) return set_error(QL_ERR_UNSUPPORTED, "%s: buffers must be 16-byte (data: 8-byte) aligned", op);
  const int cps = (int)((K / nb) / 16);
  const uint8_t *qp = static_cast<const uint8_t *>(q->data);
  const unsigned grid = grid_for(n16, 1);
  if (y->dtype == QL_F32) f4_block_dequantize_kernel<float><<<grid, kThreadsF4, 0, st>>>(qp, scale->data, scale->dtype, static_cast<float *>(y->data), n16, cps);
  else if (y->dtype == QL_F16) f4_block_dequantize_kernel<__half><<<grid, kThreadsF4, 0, st>>>(qp, scale->data, scale->dtype, static_cast<__half *>(y->data), n16, cps);
  else f4_block_dequantize_kernel<__nv_bfloat16><<<grid, kThreadsF4, 0, st>>>(qp, scale->data, scale->dtype, static_cast<__nv_bfloat16 *>(y->data), n16, cps);
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

} // namespace ql

using namespace ql;

extern "C" {

int ql_dynamic_quantize(const ql_tensor *input, const ql_tensor *double_quant_scale, int32_t axis, int32_t block_size,
                        ql_tensor *result, ql_tensor *scales, void *stream) {
  const char *op = "tensorrt.dynamic_quantize";
  if (!input) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  // the verifier's three checks, in its order and words
  if (block_size != 16) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: currently only block size of 16 is supported!", op);
  if (input->rank < 0 || input->rank > QL_MAX_RANK) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: input has rank %d (0..%d supported)", op, input->rank, QL_MAX_RANK);
  if (axis < 0 || axis < input->rank - 2 || axis >= input->rank)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: invalid axis! Axis can be either last or second last dimension of the input.", op);
  if (input->shape[axis] % 16 != 0) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: shape(input)[axis] must be divisible by 16.", op);
  if (axis != input->rank - 1) return set_error(QL_ERR_UNSUPPORTED, "%s: blocks along the second last dimension are not built", op);
  int rc = check_nvfp4(op, input, double_quant_scale, result, scales);
  if (rc != QL_OK) return rc;
  const int64_t nblocks = numel_of(input) / 16;
  if (nblocks == 0) return QL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t *q = static_cast<uint8_t *>(result->data), *s = static_cast<uint8_t *>(scales->data);
  const void *gs = double_quant_scale->data;
  const int gsdt = double_quant_scale->dtype;
  if (input->dtype == QL_F32) nvfp4_quantize_kernel<float><<<grid_for(nblocks, 1), kThreadsF4, 0, st>>>(static_cast<const float *>(input->data), gs, gsdt, q, s, nblocks);
  else if (input->dtype == QL_F16) nvfp4_quantize_kernel<__half><<<grid_for(nblocks, 1), kThreadsF4, 0, st>>>(static_cast<const __half *>(input->data), gs, gsdt, q, s, nblocks);
  else nvfp4_quantize_kernel<__nv_bfloat16><<<grid_for(nblocks, 1), kThreadsF4, 0, st>>>(static_cast<const __nv_bfloat16 *>(input->data), gs, gsdt, q, s, nblocks);
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

int ql_dequantize_nvfp4(const ql_tensor *data, const ql_tensor *scales, const ql_tensor *double_quant_scale, ql_tensor *output,
                        void *stream) {
  const char *op = "dequantize_nvfp4";
  if (!output) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  if (output->rank >= 1 && output->shape[output->rank - 1] % 16 != 0)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: the last dimension must be divisible by 16.", op);
  int rc = check_nvfp4(op, output, double_quant_scale, data, scales);
  if (rc != QL_OK) return rc;
  const int64_t nblocks = numel_of(output) / 16;
  if (nblocks == 0) return QL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const uint8_t *q = static_cast<const uint8_t *>(data->data), *s = static_cast<const uint8_t *>(scales->data);
  const void *gs = double_quant_scale->data;
  const int gsdt = double_quant_scale->dtype;
  if (output->dtype == QL_F32) nvfp4_dequantize_kernel<float><<<grid_for(nblocks, kUnrollF4), kThreadsF4, 0, st>>>(q, s, gs, gsdt, static_cast<float *>(output->data), nblocks);
  else if (output->dtype == QL_F16) nvfp4_dequantize_kernel<__half><<<grid_for(nblocks, kUnrollF4), kThreadsF4, 0, st>>>(q, s, gs, gsdt, static_cast<__half *>(output->data), nblocks);
  else nvfp4_dequantize_kernel<__nv_bfloat16><<<grid_for(nblocks, kUnrollF4), kThreadsF4, 0, st>>>(q, s, gs, gsdt, static_cast<__nv_bfloat16 *>(output->data), nblocks);
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}
}
