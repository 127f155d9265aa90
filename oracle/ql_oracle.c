/*
 * CPU oracle for the quantized-linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic that the reference
 * (NVIDIA/TensorRT-Incubator) specifies for tensorrt.quantize /
 * tensorrt.dequantize and for the matmul that consumes dequantized weights.
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may link or
 * load it; the shipped library never does.
 *
 * Parity status: the conversions below are pinned against the reference's own
 * software types (executor/lib/Runtime/Backend/Common/DataTypes.cpp, compiled
 * unmodified into oracle/_ref by oracle/Makefile) and against the golden
 * vectors of the reference's tests (tests/golden/reference_kat.json).  The
 * reference tests pin neither round-half-even ties nor saturation for
 * quantize; there the oracle follows the operator's specification text
 * (tensorrt/include/mlir-tensorrt-dialect/TensorRT/IR/TensorRTOps.td:3133-3194
 * for Q, :3408-3445 for DQ).
 *
 * Build: gcc -O2 -std=c11 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* element types (values shared with the tests, not with the product headers) */
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2, ORC_I8 = 3, ORC_I4 = 4, ORC_F8E4M3 = 5 };
/* quantization modes: scale rank 0 / 1 / same-as-input
 * (tensorrt/lib/TensorRT/IR/Verification.cpp:1182-1265) */
enum { ORC_PER_TENSOR = 0, ORC_PER_CHANNEL = 1, ORC_BLOCK = 2 };
/* the three fp8 quantize semantics that exist in the reference tree */
enum {
  ORC_FP8_DIRECT = 0,   /* e4m3_rne_satfinite(f32 quotient): TensorRTOps.td:3138-3153, DataTypes.cpp:43-122 */
  ORC_FP8_VIA_F16 = 1,  /* f32 -> f16 -> e4m3: kernel/lib/Kernel/Transforms/NormalizeQuantizedConversions.cpp:43-80 */
  ORC_FP8_STABLEHLO = 2 /* divide, round to integer, clamp +-448, convert, all in the input type:
                           compiler/test/Dialect/StableHloExt/raise-qdq-per-tensor-quantize.mlir:84-97 */
};

/* ------------------------------------------------------------------------ */
/* scalar conversions                                                        */
/* ------------------------------------------------------------------------ */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* IEEE binary16 -> binary32 (exact). Same value mapping as Float16::operator float,
 * DataTypes.cpp:308-360. */
float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t man = h & 0x3FF;
  if (exp == 0x1F) return bits_f32(sign | 0x7F800000u | (man << 13));
  if (exp == 0) {
    if (man == 0) return bits_f32(sign);
    float v = ldexpf((float)man, -24);
    return (sign ? -v : v);
  }
  return bits_f32(sign | ((exp + 112) << 23) | (man << 13));
}

/* binary32 -> binary16, round-to-nearest-even, overflow to infinity
 * (Float16::Float16(float), DataTypes.cpp:226-306). */
uint16_t orc_f32_to_f16(float f) {
  uint32_t u = f32_bits(f);
  uint16_t sign = (uint16_t)((u >> 16) & 0x8000);
  uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00 | ((a >> 13) & 0x3FF)); /* NaN */
  if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00); /* >= 65520 rounds to inf */
  if (a < 0x33000001u) return sign;                        /* <= 2^-25 rounds to 0 */
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
  int shift = (e < -14) ? (13 + (-14 - e)) : 13; /* bits dropped from the 24-bit significand */
  uint32_t kept = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (kept & 1))) kept++;
  if (e < -14) return (uint16_t)(sign | kept); /* subnormal (kept may carry into exp=1) */
  /* normal: kept has the hidden bit at position 10 (or 11 after carry) */
  uint32_t bits = ((uint32_t)(e + 15) << 10) + (kept - 0x400u);
  return (uint16_t)(sign | bits);
}

float orc_bf16_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

/* binary32 -> bfloat16, round-to-nearest-even (BFloat16::BFloat16(float), DataTypes.cpp:411-435). */
uint16_t orc_f32_to_bf16(float f) {
  uint32_t u = f32_bits(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40); /* quiet NaN */
  uint32_t lsb = (u >> 16) & 1;
  u += 0x7FFFu + lsb;
  return (uint16_t)(u >> 16);
}

/* e4m3fn -> binary32 (exact); 0x7F / 0xFF are NaN (F8E4M3FN::operator float, DataTypes.cpp:124-174). */
float orc_f8e4m3_to_f32(uint8_t b) {
  int sign = b >> 7;
  int exp = (b >> 3) & 0xF;
  int man = b & 7;
  float v;
  if (exp == 0xF && man == 7) return bits_f32(0x7FC00000u | ((uint32_t)sign << 31));
  if (exp == 0) v = ldexpf((float)man, -9);
  else v = ldexpf((float)(8 + man), exp - 10);
  return sign ? -v : v;
}

/* binary32 -> e4m3fn, round-to-nearest-even, saturate-to-finite: |x| above the largest finite
 * value (448), +-inf included, gives +-448 (0x7E / 0xFE); NaN gives 0x7F.  This is the
 * conversion the operator specification implies and that PTX cvt.rn.satfinite.e4m3x2.f32
 * performs.  The reference's software type (DataTypes.cpp:43-98) agrees except for three
 * documented defects of that file (see tests/test_oracle_vs_reference.py). */
uint8_t orc_f32_to_f8e4m3(float f) {
  uint32_t u = f32_bits(f);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80);
  uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return 0x7F;
  float x = bits_f32(a);
  if (x >= 448.0f) return (uint8_t)(sign | 0x7E);
  if (x < 0.015625f) { /* below 2^-6: subnormal grid of 2^-9 */
    float q = nearbyintf(x * 512.0f); /* exact scaling, ties-to-even */
    return (uint8_t)(sign | (uint8_t)q); /* q == 8 encodes the smallest normal */
  }
  int e = (int)(a >> 23) - 127; /* -6 .. 8 */
  uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
  uint32_t kept = m >> 20, rem = m & 0xFFFFFu;
  if (rem > 0x80000u || (rem == 0x80000u && (kept & 1))) kept++;
  if (kept == 16) { kept = 8; e++; }
  uint32_t bits = ((uint32_t)(e + 7) << 3) | (kept - 8);
  if (bits > 0x7E) bits = 0x7E;
  return (uint8_t)(sign | bits);
}

static inline float load_as_f32(const void *p, int dtype, int64_t i) {
  switch (dtype) {
  case ORC_F32: return ((const float *)p)[i];
  case ORC_F16: return orc_f16_to_f32(((const uint16_t *)p)[i]);
  case ORC_BF16: return orc_bf16_to_f32(((const uint16_t *)p)[i]);
  default: return 0.0f;
  }
}

static inline void store_from_f32(void *p, int dtype, int64_t i, float v) {
  switch (dtype) {
  case ORC_F32: ((float *)p)[i] = v; break;
  case ORC_F16: ((uint16_t *)p)[i] = orc_f32_to_f16(v); break;
  case ORC_BF16: ((uint16_t *)p)[i] = orc_f32_to_bf16(v); break;
  default: break;
  }
}

/* round a binary32 value to the given float type and back (identity for f32) */
static inline float round_to(float v, int dtype) {
  if (dtype == ORC_F16) return orc_f16_to_f32(orc_f32_to_f16(v));
  if (dtype == ORC_BF16) return orc_bf16_to_f32(orc_f32_to_bf16(v));
  return v;
}

/* int4 storage: two values per byte, first element in the low nibble
 * (tensorrt/lib/Target/TensorRTEncodingOpInterface/NetworkEncoder.cpp:552-570). */
static inline void store_i4(uint8_t *p, int64_t i, int v) {
  uint8_t nib = (uint8_t)(v & 0xF);
  if (i & 1) p[i >> 1] = (uint8_t)((p[i >> 1] & 0x0F) | (nib << 4));
  else p[i >> 1] = (uint8_t)((p[i >> 1] & 0xF0) | nib);
}
static inline int load_i4(const uint8_t *p, int64_t i) {
  int nib = (i & 1) ? (p[i >> 1] >> 4) : (p[i >> 1] & 0xF);
  return (nib ^ 8) - 8; /* sign-extend */
}

/* ------------------------------------------------------------------------ */
/* quantize / dequantize                                                     */
/* ------------------------------------------------------------------------ */

/* Geometry shared by Q and DQ.  The tensor is seen as [outer, C, inner], row-major.
 *   per-tensor : C = 1 (scale has one element)
 *   per-channel: scale[c], c the index along the quantization axis
 *   block      : the tensor is 2-D [outer=rows, ... ] -- rows = outer, cols = C*inner is not
 *                used; instead rows/cols are passed as outer/C with inner = 1 and
 *                block_dim selects which of the two dims is blocked by `block`:
 *                  block_dim 0: scale[(r / block) * cols + c]   (scale shape [rows/block, cols])
 *                  block_dim 1: scale[r * (cols / block) + c / block]
 */
static inline int64_t scale_index(int mode, int64_t i, int64_t C, int64_t inner, int block_dim,
                                  int64_t block) {
  if (mode == ORC_PER_TENSOR) return 0;
  if (mode == ORC_PER_CHANNEL) return (i / inner) % C;
  int64_t cols = C, r = i / cols, c = i % cols;
  if (block_dim == 0) return (r / block) * cols + c;
  return r * (cols / block) + c / block;
}

/* integer quantize core: clamp(round_half_even(x / (f32)scale), lo, hi); NaN -> 0 */
static inline int quant_int(float x, float s, float lo, float hi, int x_dtype, int fp8_mode) {
  float q = x / s;
  /* the StableHLO pattern divides in the input's element type */
  if (fp8_mode == ORC_FP8_STABLEHLO) q = round_to(q, x_dtype);
  if (q != q) return 0;
  float r = nearbyintf(q); /* FE_TONEAREST: ties to even */
  if (r < lo) r = lo;
  if (r > hi) r = hi;
  return (int)r;
}

int orc_quantize(const void *x, int x_dtype, const void *scale, int s_dtype, void *q, int q_dtype,
                 int mode, int64_t outer, int64_t C, int64_t inner, int block_dim, int64_t block,
                 int fp8_mode) {
  int64_t n = outer * C * inner;
  if (q_dtype == ORC_I4) memset(q, 0, (size_t)((n + 1) / 2));
  for (int64_t i = 0; i < n; i++) {
    float xv = load_as_f32(x, x_dtype, i);
    float sv = load_as_f32(scale, s_dtype, scale_index(mode, i, C, inner, block_dim, block));
    if (q_dtype == ORC_I8) {
      ((int8_t *)q)[i] = (int8_t)quant_int(xv, sv, -128.0f, 127.0f, x_dtype, fp8_mode);
    } else if (q_dtype == ORC_I4) {
      store_i4((uint8_t *)q, i, quant_int(xv, sv, -8.0f, 7.0f, x_dtype, fp8_mode));
    } else if (q_dtype == ORC_F8E4M3) {
      float quo = xv / sv;
      uint8_t b;
      if (fp8_mode == ORC_FP8_DIRECT) {
        b = orc_f32_to_f8e4m3(quo);
      } else if (fp8_mode == ORC_FP8_VIA_F16) {
        b = orc_f32_to_f8e4m3(orc_f16_to_f32(orc_f32_to_f16(quo)));
      } else {
        /* every op in the input element type; a correctly rounded f32 quotient rounded again
         * to f16/bf16 equals the correctly rounded f16/bf16 quotient */
        float d = round_to(quo, x_dtype);
        float r = nearbyintf(d);
        if (r < -448.0f) r = -448.0f;
        if (r > 448.0f) r = 448.0f;
        b = orc_f32_to_f8e4m3(r);
      }
      ((uint8_t *)q)[i] = b;
    } else {
      return -1;
    }
  }
  return 0;
}

int orc_dequantize(const void *q, int q_dtype, const void *scale, int s_dtype, void *y, int y_dtype,
                   int mode, int64_t outer, int64_t C, int64_t inner, int block_dim,
                   int64_t block) {
  int64_t n = outer * C * inner;
  for (int64_t i = 0; i < n; i++) {
    float sv = load_as_f32(scale, s_dtype, scale_index(mode, i, C, inner, block_dim, block));
    float qv;
    if (q_dtype == ORC_I8) qv = (float)((const int8_t *)q)[i];
    else if (q_dtype == ORC_I4) qv = (float)load_i4((const uint8_t *)q, i);
    else if (q_dtype == ORC_F8E4M3) qv = orc_f8e4m3_to_f32(((const uint8_t *)q)[i]);
    else return -1;
    store_from_f32(y, y_dtype, i, qv * sv); /* one f32 multiply, then one rounding to y_dtype */
  }
  return 0;
}

/* max |x| over groups, as binary32.  Layout as above: per-tensor -> 1 value, per-channel -> C
 * values, block -> one per scale element.  NaN inputs are ignored (fmaxf semantics). */
int orc_amax(const void *x, int x_dtype, float *amax, int mode, int64_t outer, int64_t C,
             int64_t inner, int block_dim, int64_t block) {
  int64_t n = outer * C * inner;
  int64_t ns = 1;
  if (mode == ORC_PER_CHANNEL) ns = C;
  else if (mode == ORC_BLOCK) ns = (block_dim == 0) ? (outer / block) * C : outer * (C / block);
  for (int64_t j = 0; j < ns; j++) amax[j] = 0.0f;
  for (int64_t i = 0; i < n; i++) {
    float a = fabsf(load_as_f32(x, x_dtype, i));
    int64_t j = scale_index(mode, i, C, inner, block_dim, block);
    amax[j] = fmaxf(amax[j], a);
  }
  return 0;
}

/* scale = amax / maxbound in f32, then rounded to s_dtype
 * (tripy/docs/pre0_user_guides/02-quantization.md:104-112). */
int orc_scale_from_amax(const float *amax, int64_t n, float maxbound, void *scale, int s_dtype) {
  for (int64_t i = 0; i < n; i++) store_from_f32(scale, s_dtype, i, amax[i] / maxbound);
  return 0;
}

/* ------------------------------------------------------------------------ */
/* linear layers that consume dequantized weights                           */
/* (tripy/nvtripy/frontend/module/linear.py:127-151: out = x @ transpose(dq(W)))  */
/* ------------------------------------------------------------------------ */

/* Y[M,N] = X[M,K] . (Wq[N,K] * scale[n])^T, weights int8 per output channel.
 * acc64 != 0: products and sums in double (a tight reference); else f32 sums in k order,
 * the loop nest Linalg-to-loops gives on the reference's host path.  */
int orc_linear_w8(const void *X, int x_dtype, const int8_t *Wq, const void *scale, int s_dtype,
                  int64_t M, int64_t N, int64_t K, void *Y, int y_dtype, int acc64) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    float sv = load_as_f32(scale, s_dtype, n);
    for (int64_t m = 0; m < M; m++) {
      if (acc64) {
        double acc = 0.0;
        for (int64_t k = 0; k < K; k++)
          acc += (double)load_as_f32(X, x_dtype, m * K + k) * ((double)Wq[n * K + k] * (double)sv);
        store_from_f32(Y, y_dtype, m * N + n, (float)acc);
      } else {
        float acc = 0.0f;
        for (int64_t k = 0; k < K; k++)
          acc += load_as_f32(X, x_dtype, m * K + k) * ((float)Wq[n * K + k] * sv);
        store_from_f32(Y, y_dtype, m * N + n, acc);
      }
    }
  }
  return 0;
}

/* Y[M,N] = X[M,K] . dq(W)^T, W packed int4 [N, K/2], scale[N, K/block] (blocks along K). */
int orc_linear_w4(const void *X, int x_dtype, const uint8_t *Wp, const void *scale, int s_dtype,
                  int64_t M, int64_t N, int64_t K, int64_t block, void *Y, int y_dtype,
                  int acc64) {
  int64_t nb = K / block;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    for (int64_t m = 0; m < M; m++) {
      double acc = 0.0;
      float accf = 0.0f;
      for (int64_t k = 0; k < K; k++) {
        float sv = load_as_f32(scale, s_dtype, n * nb + k / block);
        int w = load_i4(Wp, n * K + k);
        float xv = load_as_f32(X, x_dtype, m * K + k);
        if (acc64) acc += (double)xv * ((double)w * (double)sv);
        else accf += xv * ((float)w * sv);
      }
      store_from_f32(Y, y_dtype, m * N + n, acc64 ? (float)acc : accf);
    }
  }
  return 0;
}

/* C[b] = A[b] @ B[b] for operands of one float type: tensorrt.matrix_multiply with both operands kNONE
 * (tensorrt/include/mlir-tensorrt-dialect/TensorRT/IR/TensorRTOps.td:1986-2080), which is what tp.matmul emits
 * (tripy/nvtripy/frontend/ops/matmul.py:29-108).  Strides are in elements, so that x @ transpose(W)
 * (tripy/nvtripy/frontend/module/linear.py:148) is the same loop with b_k = 1, b_n = K; a batch stride of 0
 * broadcasts an operand.  f32 sums in k order (double when acc64), one rounding to the result type; `bias`
 * (same type, one value per column, may be null) is then added and the sum rounded again, as the reference's
 * separate add does (linear.py:149-150). */
int orc_matmul(const void *A, const void *B, const void *bias, int dtype, int64_t batch, int64_t M, int64_t N, int64_t K,
               int64_t a_m, int64_t a_k, int64_t b_k, int64_t b_n, int64_t a_batch, int64_t b_batch, void *C, int acc64) {
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t b = 0; b < batch; b++) {
    for (int64_t m = 0; m < M; m++) {
      for (int64_t n = 0; n < N; n++) {
        double acc = 0.0;
        float accf = 0.0f;
        for (int64_t k = 0; k < K; k++) {
          float av = load_as_f32(A, dtype, b * a_batch + m * a_m + k * a_k);
          float bv = load_as_f32(B, dtype, b * b_batch + k * b_k + n * b_n);
          if (acc64) acc += (double)av * (double)bv;
          else accf += av * bv;
        }
        float v = round_to(acc64 ? (float)acc : accf, dtype);
        if (bias) v = v + load_as_f32(bias, dtype, n);
        store_from_f32(C, dtype, (b * M + m) * N + n, v);
      }
    }
  }
  return 0;
}

/* Y[M,N] = (Xq[M,K] . Wq[N,K]^T) * sx[m or 0] * sw[n or 0]; e4m3 operands, f32 scales.
 * sx_n / sw_n give the scale counts (1 = per-tensor, M / N = per-row / per-channel). */
int orc_gemm_fp8(const uint8_t *Xq, const uint8_t *Wq, const float *sx, int64_t sx_n,
                 const float *sw, int64_t sw_n, int64_t M, int64_t N, int64_t K, void *Y,
                 int y_dtype, int acc64) {
  float lut[256];
  for (int i = 0; i < 256; i++) lut[i] = orc_f8e4m3_to_f32((uint8_t)i);
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++) {
    for (int64_t n = 0; n < N; n++) {
      float s = sx[sx_n == 1 ? 0 : m] * sw[sw_n == 1 ? 0 : n];
      if (acc64) {
        double acc = 0.0;
        for (int64_t k = 0; k < K; k++) acc += (double)lut[Xq[m * K + k]] * (double)lut[Wq[n * K + k]];
        store_from_f32(Y, y_dtype, m * N + n, (float)(acc * (double)s));
      } else {
        float acc = 0.0f;
        for (int64_t k = 0; k < K; k++) acc += lut[Xq[m * K + k]] * lut[Wq[n * K + k]];
        store_from_f32(Y, y_dtype, m * N + n, acc * s);
      }
    }
  }
  return 0;
}

/* Y[M,N] = (Xq[M,K] . Wq[N,K]^T in int32) * sx * sw[n]; int8 operands. */
int orc_gemm_i8(const int8_t *Xq, const int8_t *Wq, const float *sx, int64_t sx_n, const float *sw,
                int64_t sw_n, int64_t M, int64_t N, int64_t K, void *Y, int y_dtype) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++) {
    for (int64_t n = 0; n < N; n++) {
      int32_t acc = 0;
      for (int64_t k = 0; k < K; k++) acc += (int32_t)Xq[m * K + k] * (int32_t)Wq[n * K + k];
      float s = sx[sx_n == 1 ? 0 : m] * sw[sw_n == 1 ? 0 : n];
      store_from_f32(Y, y_dtype, m * N + n, (float)acc * s);
    }
  }
  return 0;
}

/* RMSNorm (weight 1) followed by per-token e4m3 quantization:
 *   r = x * rsqrt(mean(x^2) + eps);  s_m = max|r_m| / 448;  q = e4m3(r / s_m)
 * Not a reference operator: the benchmark configuration defines it.  Math in f32 with the mean
 * accumulated in double so that the result does not depend on summation order. */
int orc_rmsnorm_quant_fp8(const void *X, int x_dtype, int64_t M, int64_t H, float eps, uint8_t *Q,
                          float *scale) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++) {
    double ss = 0.0;
    for (int64_t h = 0; h < H; h++) {
      double v = load_as_f32(X, x_dtype, m * H + h);
      ss += v * v;
    }
    float rinv = (float)(1.0 / sqrt(ss / (double)H + (double)eps));
    float amax = 0.0f;
    for (int64_t h = 0; h < H; h++) amax = fmaxf(amax, fabsf(load_as_f32(X, x_dtype, m * H + h) * rinv));
    float s = amax / 448.0f;
    if (s == 0.0f) s = 1.0f;
    scale[m] = s;
    for (int64_t h = 0; h < H; h++)
      Q[m * H + h] = orc_f32_to_f8e4m3((load_as_f32(X, x_dtype, m * H + h) * rinv) / s);
  }
  return 0;
}

/* SwiGLU: a = silu(g) * u with g, u given as f32 */
float orc_silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

/* SwiGLU then per-token e4m3 quantization: a = silu(g) * u (f32), s_m = max|a_m| / 448, q = e4m3(a / s_m).
 * GU is [M, 2I] = [gate | up].  Defined by the benchmark configuration, not by a reference operator. */
int orc_swiglu_quant_fp8(const void *GU, int x_dtype, int64_t M, int64_t I, uint8_t *Q, float *scale) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++) {
    float amax = 0.0f;
    for (int64_t i = 0; i < I; i++) {
      float a = orc_silu_mul(load_as_f32(GU, x_dtype, m * 2 * I + i), load_as_f32(GU, x_dtype, m * 2 * I + I + i));
      amax = fmaxf(amax, fabsf(a));
    }
    float s = amax / 448.0f;
    if (s == 0.0f) s = 1.0f;
    scale[m] = s;
    for (int64_t i = 0; i < I; i++) {
      float a = orc_silu_mul(load_as_f32(GU, x_dtype, m * 2 * I + i), load_as_f32(GU, x_dtype, m * 2 * I + I + i));
      Q[m * I + i] = orc_f32_to_f8e4m3(a / s);
    }
  }
  return 0;
}

/* SwiGLU over a gate/up projection whose columns are interleaved in groups of 32 (columns [64b, 64b+32) = gate
 * channels [32b, 32b+32), columns [64b+32, 64b+64) = the up channels of the same indices), as the fused epilogue of
 * the gate/up GEMM sees them: act[m, i] = silu(g) * u from the unrounded f32 projection, rounded once to y_dtype;
 * row_amax[m] = max_i |act[m, i]| over the rounded values.  (Not a reference operator: the composition
 * logistic / multiply of a StableHLO program for the block.) */
int orc_swiglu_interleaved(const float *GU, int64_t M, int64_t N, void *act, int y_dtype, float *row_amax) {
  const int64_t I = N / 2;
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++) {
    float mx = 0.0f;
    for (int64_t i = 0; i < I; i++) {
      const int64_t col = (i / 32) * 64 + (i % 32);
      const float a = round_to(orc_silu_mul(GU[m * N + col], GU[m * N + col + 32]), y_dtype);
      store_from_f32(act, y_dtype, m * I + i, a);
      if (fabsf(a) > mx) mx = fabsf(a);
    }
    row_amax[m] = mx;
  }
  return 0;
}

/* ---- NVFP4 (tensorrt.dynamic_quantize, tensorrt/include/mlir-tensorrt-dialect/TensorRT/IR/TensorRTOps.td:3279-3358):
 * blocks of 16 along the last axis; block scale = max|x| / 6 divided by the per-tensor "double quantization" scale
 * and rounded to e4m3; data = x / (e4m3 scale * double_quant_scale) rounded to e2m1 (values 0, 0.5, 1, 1.5, 2, 3, 4, 6
 * and their negatives; round to nearest even, saturating, as PTX cvt.rn.satfinite.e2m1x2.f32 which the reference's
 * kernel backend uses, kernel/lib/Kernel/Transforms/LowerToNVVM.cpp:339-392).  Pinned by the known answer of
 * compiler/test/python/IntegrationTests/test_tensorrt_fp4.py.  A block whose scale rounds to zero quantizes to
 * zeros (this implementation's choice; the reference has no test there). */
static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

float orc_f4e2m1_to_f32(uint8_t nibble) {
  float v = kE2M1[nibble & 7];
  return (nibble & 8) ? -v : v;
}

uint8_t orc_f32_to_f4e2m1(float f) {
  if (f != f) return 0x7; /* satfinite: NaN becomes the largest positive value */
  uint8_t sign = (f < 0.0f || (f == 0.0f && 1.0f / f < 0.0f)) ? 8 : 0;
  float a = fabsf(f);
  if (a >= 6.0f) return sign | 7;
  /* nearest representable value; a tie goes to the one with an even mantissa bit (even index here, because
   * the codes alternate mantissa 0 / 1) */
  int best = 0;
  for (int i = 1; i < 8; i++) {
    float dlo = fabsf(a - kE2M1[best]), dhi = fabsf(kE2M1[i] - a);
    if (dhi < dlo || (dhi == dlo && (i & 1) == 0)) best = i;
  }
  return sign | (uint8_t)best;
}

/* x: [rows, K] (K % 16 == 0) of x_dtype; q: rows*K/2 bytes, first element in the low nibble; scales: [rows, K/16] e4m3 */
int orc_dynamic_quantize_nvfp4(const void *x, int x_dtype, int64_t rows, int64_t K, float double_quant_scale, uint8_t *q,
                               uint8_t *scales) {
  if (K % 16 != 0) return -1;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++) {
    for (int64_t b = 0; b < K / 16; b++) {
      const int64_t base = r * K + b * 16;
      float amax = 0.0f;
      for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(load_as_f32(x, x_dtype, base + i)));
      const uint8_t sq = orc_f32_to_f8e4m3((amax / 6.0f) / double_quant_scale);
      scales[r * (K / 16) + b] = sq;
      const float s = orc_f8e4m3_to_f32(sq) * double_quant_scale;
      for (int i = 0; i < 16; i += 2) {
        uint8_t lo = 0, hi = 0;
        if (s != 0.0f) {
          lo = orc_f32_to_f4e2m1(load_as_f32(x, x_dtype, base + i) / s);
          hi = orc_f32_to_f4e2m1(load_as_f32(x, x_dtype, base + i + 1) / s);
        }
        q[(base + i) / 2] = (uint8_t)(lo | (hi << 4));
      }
    }
  }
  return 0;
}

/* y = e2m1 value * (e4m3 block scale * double_quant_scale): the two tensorrt.dequantize steps of the operator's
 * documented use, each one f32 multiply, the last rounded to y_dtype */
int orc_dequantize_nvfp4(const uint8_t *q, const uint8_t *scales, float double_quant_scale, int64_t rows, int64_t K, void *y,
                         int y_dtype) {
  if (K % 16 != 0) return -1;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++)
    for (int64_t k = 0; k < K; k++) {
      const int64_t i = r * K + k;
      const float s = orc_f8e4m3_to_f32(scales[r * (K / 16) + k / 16]) * double_quant_scale;
      const uint8_t nib = (i & 1) ? (q[i / 2] >> 4) : (q[i / 2] & 0xF);
      store_from_f32(y, y_dtype, i, orc_f4e2m1_to_f32(nib) * s);
    }
  return 0;
}

int orc_num_threads(void) {
  int n = 1;
#ifdef _OPENMP
#pragma omp parallel
  {
#pragma omp single
    n = omp_get_num_threads();
  }
#endif
  return n;
}
