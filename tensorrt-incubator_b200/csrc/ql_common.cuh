// Shared device/host helpers of the qlinear_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "qlinear_b200.h"

namespace ql {

// ---------------------------------------------------------------------------------------------
// error plumbing (host)
// ---------------------------------------------------------------------------------------------
int set_error(int status, const char *fmt, ...);
int cuda_error(cudaError_t e, const char *what);
#define QL_CUDA_TRY(expr)                                                                         \
  do {                                                                                            \
    cudaError_t _e = (expr);                                                                      \
    if (_e != cudaSuccess) return ::ql::cuda_error(_e, #expr);                                    \
  } while (0)

int sm_count();
void count_launches(int n); // bumps the counter ql_launch_count() reports
// One int per device in global memory where kernels record that a bounded wait ran out (0 = none).
int *device_status_word();
void keep_scratch_pool_warm(); // call before cudaMallocAsync

static inline int64_t numel(const ql_tensor *t) {
  int64_t n = 1;
  for (int i = 0; i < t->rank; i++) n *= t->shape[i];
  return n;
}
static inline bool is_float_dtype(int d) { return d == QL_F32 || d == QL_F16 || d == QL_BF16; }
static inline bool is_quant_dtype(int d) { return d == QL_I8 || d == QL_I4 || d == QL_F8E4M3; }
static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Where the scale of element i lives:  idx(i) = ((i / a) % b) * c + (i % d) / e
//   per-tensor            a=1 b=1 c=0 d=1 e=1
//   per-channel           a=inner b=C c=1 d=1 e=1          (tensor seen as [outer, C, inner])
//   block along dim 0     a=cols*B b=rows/B c=cols d=cols e=1   (scale [rows/B, cols])
//   block along dim 1     a=cols b=rows c=cols/B d=cols e=B     (scale [rows, cols/B])
struct ScaleGeom {
  int64_t a, b, c, d, e;
};

// How one thread's chunk of V consecutive elements finds its scales.
enum ScaleFetch {
  SF_TENSOR = 0,  // one scale for the whole tensor
  SF_UNIFORM = 1, // one scale per chunk, idx(first element)
  SF_CONTIG = 2,  // V consecutive scales starting at idx(first element)
  SF_GENERIC = 3  // idx(i) per element
};

struct QdqPlan {
  int mode;        // 0 per-tensor, 1 per-channel, 2 block
  ScaleGeom g;
  int64_t n;       // elements
  int64_t n_scales;
  int64_t uniform_run; // consecutive elements (from a multiple of it) that share one scale, or 0
  int64_t contig_run;  // consecutive elements (from a multiple of it) with consecutive scales, or 0
};

// Validates (input, scale, attrs) against the reference verifier's rules and fills the plan.
int plan_qdq(const ql_tensor *data, const ql_tensor *scale, const ql_qdq_attrs *attrs,
             int quantized_dtype, const char *opname, QdqPlan *plan);

#ifdef __CUDACC__
// ---------------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------------
template <typename IdxT>
__device__ __forceinline__ IdxT scale_idx(const ScaleGeom &g, IdxT i) {
  return ((i / (IdxT)g.a) % (IdxT)g.b) * (IdxT)g.c + (i % (IdxT)g.d) / (IdxT)g.e;
}

// Plain loads on purpose: the 16-bit overloads of __ldg are non-volatile inline assembly, which the compiler may
// hoist above a null check of `p` (it did, in a GEMM epilogue called without scales: an illegal address).
__device__ __forceinline__ float load_scale(const void *p, int dtype, int64_t i) {
  if (dtype == QL_F32) return reinterpret_cast<const float *>(p)[i];
  if (dtype == QL_F16) return __half2float(reinterpret_cast<const __half *>(p)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
}

template <typename T> struct FloatIO;
template <> struct FloatIO<float> {
  static constexpr int kDtype = QL_F32;
  __device__ static __forceinline__ float to_f32(float v) { return v; }
  __device__ static __forceinline__ float from_f32(float v) { return v; }
};
template <> struct FloatIO<__half> {
  static constexpr int kDtype = QL_F16;
  __device__ static __forceinline__ float to_f32(__half v) { return __half2float(v); }
  __device__ static __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct FloatIO<__nv_bfloat16> {
  static constexpr int kDtype = QL_BF16;
  __device__ static __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

// Load N consecutive elements (N*sizeof(T) a multiple of 16, pointer 16-byte aligned) as f32.
template <typename T, int N>
__device__ __forceinline__ void load_vec_f32(const T *__restrict__ p, float (&v)[N]) {
  constexpr int kPer16 = 16 / sizeof(T);
  static_assert(N % kPer16 == 0, "whole 16-byte words");
#pragma unroll
  for (int w = 0; w < N / kPer16; w++) {
    uint4 raw = __ldcs(reinterpret_cast<const uint4 *>(p) + w); // streamed once: evict first
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int j = 0; j < kPer16; j++) v[w * kPer16 + j] = FloatIO<T>::to_f32(e[j]);
  }
}

template <typename T, int N>
__device__ __forceinline__ void store_vec_f32(T *__restrict__ p, const float (&v)[N]) {
  constexpr int kPer16 = 16 / sizeof(T);
  static_assert(N % kPer16 == 0, "whole 16-byte words");
#pragma unroll
  for (int w = 0; w < N / kPer16; w++) {
    uint4 raw;
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int j = 0; j < kPer16; j++) e[j] = FloatIO<T>::from_f32(v[w * kPer16 + j]);
    __stcs(reinterpret_cast<uint4 *>(p) + w, raw);
  }
}

// clamp(round_half_even(q), -128, 127) with NaN -> 0, in one instruction
__device__ __forceinline__ int quant_i8(float q) {
  int r;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(q));
  return r;
}
__device__ __forceinline__ int quant_i4(float q) {
  int r = __float2int_rn(q); // saturating, NaN -> 0
  return max(-8, min(7, r));
}

// two f32 -> two e4m3 bytes (low byte = first), round-to-nearest-even, saturate to +-448
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2_via_f16(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return (uint32_t)__nv_cvt_halfraw2_to_fp8x2(*reinterpret_cast<__half2_raw *>(&h), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint32_t two) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two & 0xFFFF), __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2 *>(&r));
}

template <typename InT>
__device__ __forceinline__ float round_through(float v) {
  return FloatIO<InT>::to_f32(FloatIO<InT>::from_f32(v));
}

// Division by a divisor that many numerators share, with the result of the IEEE division (round to nearest even)
// wherever a quantize step can tell the difference.  y = RN(1/s) once; per numerator q0 = RN(v y), then twice
// r = v - s q (exact in an FMA), q = RN(q + r y).  After the first correction q is within an ulp of v/s, and for
// such a q and a correctly rounded reciprocal the second correction returns RN(v/s) (Markstein's theorem on
// FMA-based division): five instructions and a branch-free select against about a dozen, with a call, for the
// general division.  The corrected value is taken where 2^-50 <= |q0| < inf; elsewhere q0 itself is returned: a
// signed zero, a quotient below 2^-50 (its residuals could underflow; every quantized type rounds it to a zero of
// that sign, as it does the exact quotient), an infinity (v infinite or v/s beyond the largest float: saturates
// either way) or a NaN.  A divisor outside [2^-40, 2^40], or NaN, takes the general division throughout.
struct SharedDivisor {
  float s, y;
  bool fast;
  __device__ __forceinline__ explicit SharedDivisor(float s_) {
    s = s_;
    y = __frcp_rn(s_);
    const float a = fabsf(s_);
    fast = a >= 0x1p-40f && a <= 0x1p40f;
  }
  // requires `fast`
  __device__ __forceinline__ float quick(float v) const {
    const float q0 = __fmul_rn(v, y);
    float r = __fmaf_rn(-s, q0, v);
    float q = __fmaf_rn(r, y, q0);
    r = __fmaf_rn(-s, q, v);
    q = __fmaf_rn(r, y, q);
    const float a0 = fabsf(q0);
    return (a0 >= 0x1p-50f && a0 < __int_as_float(0x7f800000)) ? q : q0;
  }
  // The same for two numerators at once with Blackwell's packed f32x2 arithmetic (each half rounds as the scalar
  // instruction does): half the multiply / FMA instructions per value.
  __device__ __forceinline__ void quick2(float &a, float &b) const {
    uint64_t v, yy, ns, q0, r, q;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(a), "f"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(yy) : "f"(y));
    asm("mov.b64 %0, {%1, %1};" : "=l"(ns) : "f"(-s));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(q0) : "l"(v), "l"(yy));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(ns), "l"(q0), "l"(v));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(r), "l"(yy), "l"(q0));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(ns), "l"(q), "l"(v));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(r), "l"(yy), "l"(q));
    float qa, qb, za, zb;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(qa), "=f"(qb) : "l"(q));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(za), "=f"(zb) : "l"(q0));
    const float aa = fabsf(za), ab = fabsf(zb);
    a = (aa >= 0x1p-50f && aa < __int_as_float(0x7f800000)) ? qa : za;
    b = (ab >= 0x1p-50f && ab < __int_as_float(0x7f800000)) ? qb : zb;
  }
  __device__ __forceinline__ float operator()(float v) const { return fast ? quick(v) : __fdiv_rn(v, s); }
  // v[j] /= s for a group of values: one uniform branch for the group
  template <int N> __device__ __forceinline__ void divide(float (&v)[N]) const {
    if (fast) {
      if constexpr (N % 2 == 0) {
#pragma unroll
        for (int j = 0; j < N; j += 2) quick2(v[j], v[j + 1]);
      } else {
#pragma unroll
        for (int j = 0; j < N; j++) v[j] = quick(v[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < N; j++) v[j] = __fdiv_rn(v[j], s);
    }
  }
};

// The quotient an integer quantize rounds: the f32 quotient as the operator specifies it, or, under the StableHLO
// pattern's arithmetic (divide, round, clamp and convert all in the input's element type), that quotient rounded to
// the input type first.  An f32 quotient rounded again to f16/bf16 is the correctly rounded 16-bit quotient.
template <typename InT>
__device__ __forceinline__ float int_quotient(float q, int fp8_mode) {
  return fp8_mode == QL_FP8_STABLEHLO ? round_through<InT>(q) : q;
}

// fp8 quantize of a pair of quotients under the selected semantics
template <typename InT>
__device__ __forceinline__ uint32_t quant_f8_pair(float q0, float q1, int fp8_mode) {
  if (fp8_mode == QL_FP8_DIRECT) return f32x2_to_e4m3x2(q0, q1);
  if (fp8_mode == QL_FP8_VIA_F16) return f32x2_to_e4m3x2_via_f16(q0, q1);
  float r0 = fminf(fmaxf(rintf(round_through<InT>(q0)), -448.f), 448.f);
  float r1 = fminf(fmaxf(rintf(round_through<InT>(q1)), -448.f), 448.f);
  // fminf/fmaxf drop NaN; keep it so that NaN still encodes as 0x7F
  if (q0 != q0) r0 = q0;
  if (q1 != q1) r1 = q1;
  return f32x2_to_e4m3x2(r0, r1);
}

// silu(g) * u.  SiLU is not a reference operator and no rounding of it is specified, so it uses the hardware's fast
// exponential and reciprocal (a few ulp; the quantize step that follows is the exact one): the kernel is bound by
// instruction issue, and the exact expf + division cost three times as many instructions.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
#endif // __CUDACC__

} // namespace ql
