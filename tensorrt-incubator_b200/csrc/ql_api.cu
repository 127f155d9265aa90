// C ABI of qlinear_b200: argument validation (the reference verifier's rules and wording) and
// dispatch to the sm_100a kernels.  There is no CPU path: without a usable device every compute
// entry returns QL_ERR_NO_DEVICE / QL_ERR_CUDA.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>

#include "ql_common.cuh"

namespace ql {

static thread_local char g_error[512] = "";

int set_error(int status, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return status;
}

int cuda_error(cudaError_t e, const char *what) {
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver)
    return set_error(QL_ERR_NO_DEVICE, "%s: %s", what, cudaGetErrorString(e));
  return set_error(QL_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

static std::atomic<uint64_t> g_launches{0};
void count_launches(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

// The stream-ordered allocator gives scratch memory back to the driver at every synchronisation
// unless told otherwise; keep it cached so that scratch users pay for it once.
void keep_scratch_pool_warm() {
  static bool done[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || done[dev]) return;
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
    uint64_t keep = UINT64_MAX;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
  }
  done[dev] = true;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int *device_status_word() {
  // one word per device, allocated on first use and kept for the life of the process
  static int *words[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!words[dev]) {
    if (cudaMalloc(&words[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(words[dev], 0, sizeof(int));
  }
  return words[dev];
}

// kernels (ql_qdq.cu)
int launch_quantize(const ql_tensor *in, const ql_tensor *scale, ql_tensor *q, ql_tensor *y, const QdqPlan &p,
                    int fp8_mode, cudaStream_t st);
int launch_dequantize(const ql_tensor *q, const ql_tensor *scale, ql_tensor *y, const QdqPlan &p, cudaStream_t st);
int launch_amax(const ql_tensor *in, float *amax, const QdqPlan &p, cudaStream_t st);
int launch_scale_from_amax(const float *amax, void *scale, int sdt, int64_t n, float maxbound, cudaStream_t st);

// ql_wo_linear.cu
int launch_wo_linear(int wbits, int xdt, const void *X, const void *W, const void *scale, int sdt, void *Y, int M,
                     int N, int K, int block, bool weights_constant, cudaStream_t st);

// ql_gemm_w8a16.cu
int launch_w8a16_fused(int xdt, const void *X, const void *W, const void *scale, int sdt, void *Y, int M, int N, int K,
                       cudaStream_t st);
int launch_w8a16_widen(int xdt, const void *X, const void *W, const void *scale, int sdt, void *Y, int M, int N, int K,
                       cudaStream_t st);
// Above this many rows the product is compute-bound and the separate widening pass is the cheaper route.
constexpr int kFusedWidenMaxRows = 256;
// ql_gemm_tc.cu
int gemm16_device(int dtype, const void *X, const void *W, const float *sb, int sb_n, void *Y, int M, int N, int K,
                  cudaStream_t st);

// ql_nvfp4.cu
int launch_f4_block_dequantize(const ql_tensor *q, const ql_tensor *scale, ql_tensor *y, cudaStream_t st);

// Above this many rows of X the weight-only layers leave the streaming kernel for the tcgen05 GEMM.  The int8
// layer has a tcgen05 kernel that widens the weights itself and takes over earlier: the streaming kernel walks
// batches in slices of 32 rows (58 us for 64 rows of config 2 against 35 us for 128 rows on the tensor cores).
constexpr int kWeightOnlyMaxRows = 64;
constexpr int kWeightOnlyMaxRowsInt8 = 32;

static bool same_shape(const ql_tensor *a, const ql_tensor *b) {
  if (a->rank != b->rank) return false;
  for (int i = 0; i < a->rank; i++)
    if (a->shape[i] != b->shape[i]) return false;
  return true;
}

static int check_tensor(const ql_tensor *t, const char *op, const char *name) {
  if (!t) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: %s is null", op, name);
  if (t->rank < 0 || t->rank > QL_MAX_RANK)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: %s has rank %d (0..%d supported)", op, name, t->rank, QL_MAX_RANK);
  for (int i = 0; i < t->rank; i++)
    if (t->shape[i] < 0) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: %s has a negative dimension", op, name);
  if (numel(t) > 0 && !t->data) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: %s has no data pointer", op, name);
  return QL_OK;
}

// Messages follow tensorrt/lib/TensorRT/IR/Verification.cpp:1182-1265 (quantize) and :1296-1380
// (dequantize) of the reference, which word the two operators alike.
int plan_qdq(const ql_tensor *data, const ql_tensor *scale, const ql_qdq_attrs *attrs, int qdt, const char *op,
             QdqPlan *plan) {
  const int R = data->rank;
  const bool has_axis = attrs && attrs->has_axis;
  const int axis = attrs ? attrs->axis : 0;
  if (!is_float_dtype(scale->dtype))
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: scale must be f32, f16 or bf16", op);
  if (!(scale->rank == 0 || scale->rank == 1 || scale->rank == R))
    return set_error(QL_ERR_INVALID_ARGUMENT,
                     "%s: Scale value must be scalar for per-tensor quantization, 1D for per-channel "
                     "quantization, and same rank as the input for block quantization.", op);
  plan->n = numel(data);
  plan->uniform_run = 0;
  plan->contig_run = 0;
  if (scale->rank == 0) {
    if (has_axis)
      return set_error(QL_ERR_INVALID_ARGUMENT,
                       "%s: When scale value is scalar, quantization is per-tensor and thus axis value "
                       "shouldn't be provided.", op);
    plan->mode = 0;
    plan->g = ScaleGeom{1, 1, 0, 1, 1};
    plan->n_scales = 1;
    plan->uniform_run = plan->n;
    return QL_OK;
  }
  if (scale->rank == 1) {
    if (!has_axis)
      return set_error(QL_ERR_INVALID_ARGUMENT,
                       "%s: When scale is 1D tensor, quantization is per-channel and thus axis value must be "
                       "provided.", op);
    if (axis >= R || axis < 0)
      return set_error(QL_ERR_INVALID_ARGUMENT, "%s: expected axis to be non-negative and less than %d", op, R);
    if (data->shape[axis] != scale->shape[0])
      return set_error(QL_ERR_INVALID_ARGUMENT,
                       "%s: For per-channel quantization, expected the scales tensor dimension to match the "
                       "quantization axis dimension of input tensor", op);
    int64_t inner = 1;
    for (int i = axis + 1; i < R; i++) inner *= data->shape[i];
    int64_t C = data->shape[axis];
    plan->mode = 1;
    plan->g = ScaleGeom{inner, C > 0 ? C : 1, 1, 1, 1};
    plan->n_scales = C;
    if (inner > 1) plan->uniform_run = inner;
    else plan->contig_run = C;
    return QL_OK;
  }
  // block quantization: scale has the input's rank
  if (has_axis)
    return set_error(QL_ERR_INVALID_ARGUMENT,
                     "%s: Scale has same rank as that of input, thus this is block quantization. Axis is not "
                     "valid in this case.", op);
  if (!(qdt == QL_I4 || qdt == QL_F8E4M3))
    return set_error(QL_ERR_INVALID_ARGUMENT,
                     "%s: Block quantization is supported only for int4, fp4 or fp8 output types.", op);
  int bdim = -1;
  for (int i = 0; i < R; i++) {
    if (data->shape[i] == scale->shape[i]) continue;
    if (bdim == -1) { bdim = i; continue; }
    return set_error(QL_ERR_INVALID_ARGUMENT,
                     "%s: For block quantization, all input and scale dimensions match except a single "
                     "blocking dimension : %d", op, bdim);
  }
  if (bdim != -1 && bdim < R - 2)
    return set_error(QL_ERR_INVALID_ARGUMENT,
                     "%s: For block quantization, blocking dimension should be either last or second last.", op);
  int64_t cols = R >= 1 ? data->shape[R - 1] : 1;
  int64_t B = 1;
  if (bdim != -1) {
    if (scale->shape[bdim] <= 0 || data->shape[bdim] % scale->shape[bdim] != 0)
      return set_error(QL_ERR_INVALID_ARGUMENT,
                       "%s: block quantization needs input.shape[%d] to be a multiple of scale.shape[%d]", op, bdim, bdim);
    B = data->shape[bdim] / scale->shape[bdim];
  }
  plan->mode = 2;
  plan->n_scales = numel(scale);
  if (cols <= 0) cols = 1;
  if (bdim == -1 || bdim == R - 1) {
    // scale[r, c / B]
    int64_t rows = plan->n / cols;
    plan->g = ScaleGeom{cols, rows > 0 ? rows : 1, cols / B, cols, B};
    plan->uniform_run = B;
  } else {
    // scale[r / B, c] with r running over every leading dimension
    int64_t rows = plan->n / cols;
    plan->g = ScaleGeom{cols * B, rows / B > 0 ? rows / B : 1, cols, cols, 1};
    plan->contig_run = cols;
  }
  return QL_OK;
}

static int check_qdq_common(const ql_tensor *fl, const ql_tensor *scale, const ql_tensor *qt, const char *op) {
  int rc;
  if ((rc = check_tensor(fl, op, "floating-point tensor")) != QL_OK) return rc;
  if ((rc = check_tensor(scale, op, "scale")) != QL_OK) return rc;
  if ((rc = check_tensor(qt, op, "quantized tensor")) != QL_OK) return rc;
  if (!is_float_dtype(fl->dtype))
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: valid conversions are (f32 | f16 | bf16) <-> (int8 | f8E4M3FN | int4)", op);
  if (!is_quant_dtype(qt->dtype))
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: valid conversions are (f32 | f16 | bf16) <-> (int8 | f8E4M3FN | int4)", op);
  if (!same_shape(fl, qt)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: input and output shapes differ", op);
  return QL_OK;
}

} // namespace ql

using namespace ql;

extern "C" {

int ql_version(void) { return 100; }

const char *ql_last_error(void) { return g_error; }

uint64_t ql_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int ql_device_info(int32_t *sms, int32_t *cc) {
  int dev = 0;
  QL_CUDA_TRY(cudaGetDevice(&dev));
  int n = 0, major = 0, minor = 0;
  QL_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
  QL_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  QL_CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
  if (sms) *sms = n;
  if (cc) *cc = major * 10 + minor;
  return QL_OK;
}

int ql_quantize(const ql_tensor *input, const ql_tensor *scale, ql_tensor *output, const ql_qdq_attrs *attrs,
                void *stream) {
  int rc = check_qdq_common(input, scale, output, "tensorrt.quantize");
  if (rc != QL_OK) return rc;
  QdqPlan plan;
  if ((rc = plan_qdq(input, scale, attrs, output->dtype, "tensorrt.quantize", &plan)) != QL_OK) return rc;
  int fp8_mode = attrs ? attrs->fp8_mode : QL_FP8_DIRECT;
  if (fp8_mode < 0 || fp8_mode > QL_FP8_STABLEHLO)
    return set_error(QL_ERR_INVALID_ARGUMENT, "tensorrt.quantize: unknown fp8 mode %d", fp8_mode);
  return launch_quantize(input, scale, output, nullptr, plan, fp8_mode, (cudaStream_t)stream);
}

int ql_dequantize(const ql_tensor *input, const ql_tensor *scale, ql_tensor *output, const ql_qdq_attrs *attrs,
                  void *stream) {
  if (input && input->dtype == QL_F4E2M1) { // NVFP4 data: block scales along the last axis (ql_nvfp4.cu)
    int rc;
    if ((rc = check_tensor(input, "tensorrt.dequantize", "quantized tensor")) != QL_OK) return rc;
    if ((rc = check_tensor(output, "tensorrt.dequantize", "floating-point tensor")) != QL_OK) return rc;
    if ((rc = check_tensor(scale, "tensorrt.dequantize", "scale")) != QL_OK) return rc;
    if (!is_float_dtype(output->dtype) || !is_float_dtype(scale->dtype))
      return set_error(QL_ERR_INVALID_ARGUMENT, "tensorrt.dequantize: f4E2M1FN dequantizes to f32, f16 or bf16 with scales of one of those types");
    if (!same_shape(output, input)) return set_error(QL_ERR_INVALID_ARGUMENT, "tensorrt.dequantize: input and output shapes differ");
    return launch_f4_block_dequantize(input, scale, output, (cudaStream_t)stream);
  }
  int rc = check_qdq_common(output, scale, input, "tensorrt.dequantize");
  if (rc != QL_OK) return rc;
  QdqPlan plan;
  if ((rc = plan_qdq(input, scale, attrs, input->dtype, "tensorrt.dequantize", &plan)) != QL_OK) return rc;
  return launch_dequantize(input, scale, output, plan, (cudaStream_t)stream);
}

int ql_quantize_dequantize(const ql_tensor *input, const ql_tensor *scale, ql_tensor *quantized,
                           ql_tensor *dequantized, const ql_qdq_attrs *attrs, void *stream) {
  int rc = check_qdq_common(input, scale, quantized, "quantize_dequantize");
  if (rc != QL_OK) return rc;
  if ((rc = check_tensor(dequantized, "quantize_dequantize", "dequantized")) != QL_OK) return rc;
  if (dequantized->dtype != input->dtype || !same_shape(input, dequantized))
    return set_error(QL_ERR_INVALID_ARGUMENT, "quantize_dequantize: dequantized must have the input's type and shape");
  QdqPlan plan;
  if ((rc = plan_qdq(input, scale, attrs, quantized->dtype, "quantize_dequantize", &plan)) != QL_OK) return rc;
  int fp8_mode = attrs ? attrs->fp8_mode : QL_FP8_DIRECT;
  if (fp8_mode < 0 || fp8_mode > QL_FP8_STABLEHLO)
    return set_error(QL_ERR_INVALID_ARGUMENT, "quantize_dequantize: unknown fp8 mode %d", fp8_mode);
  return launch_quantize(input, scale, quantized, dequantized, plan, fp8_mode, (cudaStream_t)stream);
}

int ql_amax_scale(const ql_tensor *input, ql_tensor *scale, const ql_qdq_attrs *attrs, float maxbound, void *stream) {
  int rc;
  if ((rc = check_tensor(input, "amax_scale", "input")) != QL_OK) return rc;
  if ((rc = check_tensor(scale, "amax_scale", "scale")) != QL_OK) return rc;
  if (!is_float_dtype(input->dtype)) return set_error(QL_ERR_INVALID_ARGUMENT, "amax_scale: input must be f32, f16 or bf16");
  if (!(maxbound > 0.f)) return set_error(QL_ERR_INVALID_ARGUMENT, "amax_scale: maxbound must be positive");
  QdqPlan plan;
  // block groupings are legal for every quantized type here: only the grouping is used
  if ((rc = plan_qdq(input, scale, attrs, QL_I4, "amax_scale", &plan)) != QL_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (plan.n_scales == 0) return QL_OK;
  if (scale->dtype == QL_F32) {
    // accumulate max|x| in the output itself, then divide in place
    float *acc = static_cast<float *>(scale->data);
    if ((rc = launch_amax(input, acc, plan, st)) != QL_OK) return rc;
    return launch_scale_from_amax(acc, scale->data, QL_F32, plan.n_scales, maxbound, st);
  }
  // 16-bit scales: f32 accumulators in stream-ordered scratch memory
  float *acc = nullptr;
  keep_scratch_pool_warm();
  QL_CUDA_TRY(cudaMallocAsync(&acc, sizeof(float) * (size_t)plan.n_scales, st));
  rc = launch_amax(input, acc, plan, st);
  if (rc == QL_OK) rc = launch_scale_from_amax(acc, scale->data, scale->dtype, plan.n_scales, maxbound, st);
  cudaError_t fe = cudaFreeAsync(acc, st);
  if (rc == QL_OK && fe != cudaSuccess) return cuda_error(fe, "cudaFreeAsync");
  return rc;
}


static int check_linear_io(const char *op, const ql_tensor *x, const ql_tensor *w, const ql_tensor *scale,
                           const ql_tensor *y, int wdtype) {
  int rc;
  if ((rc = check_tensor(x, op, "x")) != QL_OK) return rc;
  if ((rc = check_tensor(w, op, "w")) != QL_OK) return rc;
  if ((rc = check_tensor(scale, op, "scale")) != QL_OK) return rc;
  if ((rc = check_tensor(y, op, "y")) != QL_OK) return rc;
  if (x->rank != 2 || w->rank != 2 || y->rank != 2)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: x, w and y must be 2-D ([M,K], [N,K], [M,N])", op);
  if (!(x->dtype == QL_F16 || x->dtype == QL_BF16) || y->dtype != x->dtype)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: x and y must both be f16 or both be bf16", op);
  if (w->dtype != wdtype) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: unexpected weight type %d", op, w->dtype);
  if (!is_float_dtype(scale->dtype)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: scale must be f32, f16 or bf16", op);
  if (w->shape[1] != x->shape[1])
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: x is [M,%lld] but w is [N,%lld]", op, (long long)x->shape[1], (long long)w->shape[1]);
  if (y->shape[0] != x->shape[0] || y->shape[1] != w->shape[0])
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: y must be [M,N] = [%lld,%lld]", op, (long long)x->shape[0], (long long)w->shape[0]);
  if (!aligned16(x->data) || !aligned16(w->data) || !aligned16(y->data))
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: x, w and y must be 16-byte aligned", op);
  if (x->shape[0] > INT32_MAX || w->shape[0] > INT32_MAX || x->shape[1] > INT32_MAX)
    return set_error(QL_ERR_UNSUPPORTED, "%s: dimension too large", op);
  return QL_OK;
}

static int linear_w8a16_impl(const ql_tensor *x, const ql_tensor *w, const ql_tensor *scale, ql_tensor *y, uint32_t flags, void *stream) {
  const char *op = "linear_w8a16";
  int rc = check_linear_io(op, x, w, scale, y, QL_I8);
  if (rc != QL_OK) return rc;
  const int64_t M = x->shape[0], K = x->shape[1], N = w->shape[0];
  if (scale->rank != 1 || scale->shape[0] != N)
    return set_error(QL_ERR_INVALID_ARGUMENT,
                     "%s: For per-channel quantization, expected the scales tensor dimension to match the "
                     "quantization axis dimension of input tensor", op);
  if (K % 64 != 0) return set_error(QL_ERR_UNSUPPORTED, "%s: K must be a multiple of 64 (got %lld)", op, (long long)K);
  static const int fused_max = [] { // tuning aid, read once per process
    const char *e = getenv("QL_W8_FUSED_MAX_M");
    return e ? atoi(e) : kFusedWidenMaxRows;
  }();
  if (M > fused_max)
    return launch_w8a16_widen(x->dtype, x->data, w->data, scale->data, scale->dtype, y->data, (int)M, (int)N, (int)K,
                              (cudaStream_t)stream);
  if (M > kWeightOnlyMaxRowsInt8)
    return launch_w8a16_fused(x->dtype, x->data, w->data, scale->data, scale->dtype, y->data, (int)M, (int)N, (int)K,
                              (cudaStream_t)stream);
  return launch_wo_linear(8, x->dtype, x->data, w->data, scale->data, scale->dtype, y->data, (int)M, (int)N, (int)K, 0,
                          (flags & QL_WEIGHTS_CONSTANT) != 0, (cudaStream_t)stream);
}

static int linear_w4a16_impl(const ql_tensor *x, const ql_tensor *w, const ql_tensor *scale, ql_tensor *y, uint32_t flags, void *stream) {
  const char *op = "linear_w4a16";
  int rc = check_linear_io(op, x, w, scale, y, QL_I4);
  if (rc != QL_OK) return rc;
  const int64_t M = x->shape[0], K = x->shape[1], N = w->shape[0];
  if (scale->rank != 2 || scale->shape[0] != N || scale->shape[1] <= 0 || K % scale->shape[1] != 0)
    return set_error(QL_ERR_INVALID_ARGUMENT,
                     "%s: For block quantization, all input and scale dimensions match except a single blocking "
                     "dimension : 1", op);
  const int64_t block = K / scale->shape[1];
  if (K % 128 != 0 || block % 128 != 0)
    return set_error(QL_ERR_UNSUPPORTED, "%s: K and the block size must be multiples of 128 (K=%lld, block=%lld)", op,
                     (long long)K, (long long)block);
  if (M > kWeightOnlyMaxRows) {
    // dequantize to the activation type in scratch memory (the reference's dequantize), then the 16-bit GEMM
    cudaStream_t st = (cudaStream_t)stream;
    void *wide = nullptr;
    keep_scratch_pool_warm();
    QL_CUDA_TRY(cudaMallocAsync(&wide, (size_t)N * K * 2, st));
    ql_tensor wd{wide, x->dtype, 2, {N, K}};
    QdqPlan plan;
    rc = plan_qdq(w, scale, nullptr, QL_I4, op, &plan);
    if (rc == QL_OK) rc = launch_dequantize(w, scale, &wd, plan, st);
    if (rc == QL_OK) rc = gemm16_device(x->dtype, x->data, wide, nullptr, 0, y->data, (int)M, (int)N, (int)K, st);
    cudaError_t fe = cudaFreeAsync(wide, st);
    if (rc == QL_OK && fe != cudaSuccess) return cuda_error(fe, "cudaFreeAsync");
    return rc;
  }
  return launch_wo_linear(4, x->dtype, x->data, w->data, scale->data, scale->dtype, y->data, (int)M, (int)N, (int)K,
                          (int)block, (flags & QL_WEIGHTS_CONSTANT) != 0, (cudaStream_t)stream);
}

int ql_linear_w8a16(const ql_tensor *x, const ql_tensor *w, const ql_tensor *scale, ql_tensor *y, void *stream) {
  return linear_w8a16_impl(x, w, scale, y, 0, stream);
}

int ql_linear_w4a16(const ql_tensor *x, const ql_tensor *w, const ql_tensor *scale, ql_tensor *y, void *stream) {
  return linear_w4a16_impl(x, w, scale, y, 0, stream);
}

int ql_linear_weight_only(const ql_tensor *x, const ql_tensor *w, const ql_tensor *scale, ql_tensor *y, uint32_t flags, void *stream) {
  if (!w) return set_error(QL_ERR_INVALID_ARGUMENT, "linear_weight_only: w is null");
  if (flags & ~(uint32_t)QL_WEIGHTS_CONSTANT) return set_error(QL_ERR_INVALID_ARGUMENT, "linear_weight_only: unknown flags 0x%x", flags);
  if (w->dtype == QL_I8) return linear_w8a16_impl(x, w, scale, y, flags, stream);
  if (w->dtype == QL_I4) return linear_w4a16_impl(x, w, scale, y, flags, stream);
  return set_error(QL_ERR_INVALID_ARGUMENT, "linear_weight_only: weights must be int8 or int4");
}

} // extern "C"
