// Weight-only linear layers for small batches: Y[M,N] = X[M,K] . dequantize(W)[N,K]^T.
//
// The work is bounded by reading W once from HBM, so the kernel streams W with 16-byte loads
// straight into registers, dequantizes there (integer -> f16/bf16 is exact, so the scale can be
// applied to f32 partial sums instead of to every weight) and feeds the warp-level tensor-core
// MMA m16n8k16 with the weight tile as the 16-row operand and X as the 8-column operand.  A dot
// product does not care in which order k is visited, which is used twice: each lane's 16 bytes of
// one weight row are consumed as they lie in memory, and for int4 the value pairs that one mask
// extracts (elements e and e+4 of a word) are matched by permuting the X registers.
//
// One block owns 16 output channels.  A producer warp streams their weights into a shared-memory
// ring with TMA tile loads; 8 consumer warps split K and reduce through shared memory.
// Reference composition this implements: tripy/nvtripy/frontend/module/linear.py:140-151
// (quantize -> dequantize -> x @ transpose(w)) with the dequantize folded into the product.
#include <cuda/std/type_traits>

#include "ql_common.cuh"
#include "ql_tc_common.cuh"

namespace ql {
namespace {

constexpr int kWarps = 8;
constexpr int kThreadsWo = kWarps * 32;
constexpr int kRowsPerBlock = 16;

template <typename XT>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  if constexpr (cuda::std::is_same<XT, __half>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// bytes i and i+1 of `u` (int8 values with their sign bit already flipped, i.e. value + 128)
// -> packed pair of XT holding the exact integers
template <typename XT, int I>
__device__ __forceinline__ uint32_t int8_pair(uint32_t u) {
  if constexpr (cuda::std::is_same<XT, __half>::value) {
    // f16 0x6400 | b is 1024 + b; subtract 1024 + 128
    uint32_t v = __byte_perm(u, 0x64646464u, 0x4040 | I | ((I + 1) << 8));
    __half2 h = __hsub2(*reinterpret_cast<__half2 *>(&v), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<uint32_t *>(&h);
  } else {
    // f32 0x4B000000 | b is 2^23 + b; subtract 2^23 + 128, then round (exactly) to bf16
    float lo = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540 | I)) - 8388736.f;
    float hi = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540 | (I + 1))) - 8388736.f;
    __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&b);
  }
}

// nibbles E and E+4 of `w` (signed int4) -> packed pair of XT holding the exact integers
template <typename XT, int E>
__device__ __forceinline__ uint32_t int4_pair(uint32_t w) {
  uint32_t t = (w >> (4 * E)) & 0x000F000Fu;
  if constexpr (cuda::std::is_same<XT, __half>::value) {
    uint32_t v = t ^ 0x64086408u; // 1024 + (n ^ 8) = 1032 + value
    __half2 h = __hsub2(*reinterpret_cast<__half2 *>(&v), __half2half2(__ushort_as_half(0x6408)));
    return *reinterpret_cast<uint32_t *>(&h);
  } else {
    uint32_t v = t ^ 0x43084308u; // 128 + (n ^ 8) = 136 + value
    __nv_bfloat162 h = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&v), __bfloat162bfloat162(__ushort_as_bfloat16(0x4308)));
    return *reinterpret_cast<uint32_t *>(&h);
  }
}

template <int WBITS> struct WoTraits {
  static constexpr int kElemsPerLane = 128 / WBITS;       // elements in one 16-byte word
  static constexpr int kStep = 4 * kElemsPerLane;         // k covered by one warp iteration (64 bytes of a row)
};

// Shared-memory ring of weight slabs.  A stage holds kChunkBytes of each of the 16 rows, brought by
// one TMA tile request (a [16 x 1024 B] box; many small requests would be bound by the copy engine's
// per-request cost, not by HBM).
constexpr int kStagesWo = 4;
constexpr int kChunkBytes = 1024;
constexpr int kRowPitch = kChunkBytes;
constexpr int kStageBytesWo = kRowsPerBlock * kRowPitch;
constexpr int kItersPerStage = kChunkBytes / 64;
constexpr long long kWoWaitLimit = 1ll << 31;

__device__ __forceinline__ uint32_t wo_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool wo_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
               : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// bounded wait: false once the limit has run out (the caller records it and stops consuming)
__device__ __forceinline__ bool wo_wait(uint32_t bar, uint32_t parity) {
  if (wo_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!wo_try_wait(bar, parity))
    if (clock64() - t0 > kWoWaitLimit) return false;
  return true;
}

// NT = number of 8-row tiles of X handled at once (M <= 8 * NT).
// Warps 0..7 consume; warp 8 streams the block's 16 weight rows from HBM into the ring with one TMA
// tile request per stage, so HBM latency is hidden by the copy engine's queue instead of by registers.
template <typename XT, int WBITS, int NT>
__global__ void __launch_bounds__(kThreadsWo + 32)
wo_linear_kernel(const __grid_constant__ CUtensorMap map_w, const XT *__restrict__ X, const void *__restrict__ scale, int sdt,
                 XT *__restrict__ Y, int M, int N, int K, int block, int *status) {
  using T = WoTraits<WBITS>;
  extern __shared__ uint8_t wo_smem_raw[];
  uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(wo_smem_raw) + 127) & ~uintptr_t(127));
  float(*red)[kRowsPerBlock][NT * 8 + 1] = reinterpret_cast<float(*)[kRowsPerBlock][NT * 8 + 1]>(ring + kStagesWo * kStageBytesWo);
  __shared__ __align__(8) uint64_t bars[2 * kStagesWo];
  __shared__ int gave_up;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kRowsPerBlock;
  const int64_t row_bytes = (int64_t)K * WBITS / 8;
  const int n_iters = K / T::kStep;                                   // warp iterations over the whole K
  const int n_stages = (int)((row_bytes + kChunkBytes - 1) / kChunkBytes);
  const uint32_t bar0 = wo_smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStagesWo + s); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesWo; s++) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full_bar(s)), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty_bar(s)), "r"(kWarps) : "memory");
    }
    gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == kWarps) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      for (int st = 0; st < n_stages; st++) {
        const int slot = st % kStagesWo;
        if (st >= kStagesWo && !wo_wait(empty_bar(slot), ((st / kStagesWo) - 1) & 1)) {
          atomicCAS(status, 0, 11);
          break;
        }
        // out-of-range rows and bytes past the end of a row arrive as zeros; the whole box counts as bytes
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full_bar(slot)), "r"((uint32_t)kStageBytesWo) : "memory");
        tma_load_2d(wo_smem_u32(ring + slot * kStageBytesWo), &map_w, full_bar(slot), st * (kChunkBytes / 4), n0);
      }
    }
  } else {
    // ---------------------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;
    const int row_a = min(n0 + g, N - 1), row_b = min(n0 + g + 8, N - 1);
    const int nb = (WBITS == 4) ? K / block : 0;
    constexpr int XV = T::kElemsPerLane * 2 / 16; // 16-byte words of X per lane, row and iteration
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    // X does not depend on the weights arriving: the fragments of the next iteration are requested
    // before the current one is computed, so their L1/L2 latency hides behind the math
    auto load_x = [&](int it, uint4(&xb)[NT][XV]) {
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        const int m = nt * 8 + g;
        if (m < M) {
          const uint4 *xp = reinterpret_cast<const uint4 *>(X + (int64_t)m * K + it * T::kStep + t * T::kElemsPerLane);
#pragma unroll
          for (int v = 0; v < XV; v++) xb[nt][v] = __ldg(xp + v);
        } else {
#pragma unroll
          for (int v = 0; v < XV; v++) xb[nt][v] = make_uint4(0, 0, 0, 0);
        }
      }
    };
    constexpr bool kPrefetch = NT * XV <= 8; // beyond that the second buffer would spill
    uint4 xcur[NT][XV], xnext[kPrefetch ? NT : 1][XV];
    if (kPrefetch && warp < n_iters) load_x(warp, xcur);
    int cur_stage = -1;
    for (int it = warp; it < n_iters; it += kWarps) {
      const int st = it / kItersPerStage, slot = st % kStagesWo;
      const bool more = kPrefetch && it + kWarps < n_iters;
      if constexpr (kPrefetch) {
        if (more) load_x(it + kWarps, xnext);
      } else {
        load_x(it, xcur);
      }
      if (st != cur_stage) {
        if (cur_stage >= 0 && cur_stage + kStagesWo < n_stages) {
          // this warp is done with the previous slot: let the producer refill it
          __syncwarp();
          if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar(cur_stage % kStagesWo)) : "memory");
        }
        if (!wo_wait(full_bar(slot), (st / kStagesWo) & 1)) {
          if (lane == 0) { atomicCAS(status, 0, 12); gave_up = 1; }
          break;
        }
        cur_stage = st;
      }
      const uint8_t *stage = ring + slot * kStageBytesWo;
      const int it_in = it - st * kItersPerStage; // iteration inside the stage
      const int kb = it * T::kStep;
      const uint4 wa = *reinterpret_cast<const uint4 *>(stage + g * kRowPitch + it_in * 64 + t * 16);
      const uint4 wb = *reinterpret_cast<const uint4 *>(stage + (g + 8) * kRowPitch + it_in * 64 + t * 16);
      const uint32_t wav[4] = {wa.x, wa.y, wa.z, wa.w};
      const uint32_t wbv[4] = {wb.x, wb.y, wb.z, wb.w};

      if constexpr (WBITS == 8) {
        uint32_t a[4][4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          uint32_t ua = wav[j] ^ 0x80808080u, ub = wbv[j] ^ 0x80808080u;
          a[j][0] = int8_pair<XT, 0>(ua);
          a[j][1] = int8_pair<XT, 0>(ub);
          a[j][2] = int8_pair<XT, 2>(ua);
          a[j][3] = int8_pair<XT, 2>(ub);
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          const uint32_t xw[8] = {xcur[nt][0].x, xcur[nt][0].y, xcur[nt][0].z, xcur[nt][0].w,
                                  xcur[nt][1].x, xcur[nt][1].y, xcur[nt][1].z, xcur[nt][1].w};
#pragma unroll
          for (int j = 0; j < 4; j++) mma16816<XT>(acc[nt], a[j][0], a[j][1], a[j][2], a[j][3], xw[2 * j], xw[2 * j + 1]);
        }
      } else {
        // int4: one iteration (128 k) lies inside one scale block (block % 128 == 0)
        const float sa = load_scale(scale, sdt, (int64_t)row_a * nb + kb / block);
        const float sb = load_scale(scale, sdt, (int64_t)row_b * nb + kb / block);
        float part[NT][4];
#pragma unroll
        for (int i = 0; i < NT; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) part[i][j] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; j++) { // word j = elements 8j .. 8j+7 of this lane's 32
          uint32_t a_lo[4], a_hi[4];
          a_lo[0] = int4_pair<XT, 0>(wav[j]); a_lo[1] = int4_pair<XT, 0>(wbv[j]);
          a_lo[2] = int4_pair<XT, 1>(wav[j]); a_lo[3] = int4_pair<XT, 1>(wbv[j]);
          a_hi[0] = int4_pair<XT, 2>(wav[j]); a_hi[1] = int4_pair<XT, 2>(wbv[j]);
          a_hi[2] = int4_pair<XT, 3>(wav[j]); a_hi[3] = int4_pair<XT, 3>(wbv[j]);
#pragma unroll
          for (int nt = 0; nt < NT; nt++) {
            const uint4 xv = xcur[nt][j];
            // x pairs (0,4) (1,5) (2,6) (3,7) to line up with the weight pairs
            uint32_t p04 = __byte_perm(xv.x, xv.z, 0x5410), p15 = __byte_perm(xv.x, xv.z, 0x7632);
            uint32_t p26 = __byte_perm(xv.y, xv.w, 0x5410), p37 = __byte_perm(xv.y, xv.w, 0x7632);
            mma16816<XT>(part[nt], a_lo[0], a_lo[1], a_lo[2], a_lo[3], p04, p15);
            mma16816<XT>(part[nt], a_hi[0], a_hi[1], a_hi[2], a_hi[3], p26, p37);
          }
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          acc[nt][0] = fmaf(part[nt][0], sa, acc[nt][0]);
          acc[nt][1] = fmaf(part[nt][1], sa, acc[nt][1]);
          acc[nt][2] = fmaf(part[nt][2], sb, acc[nt][2]);
          acc[nt][3] = fmaf(part[nt][3], sb, acc[nt][3]);
        }
      }
      if constexpr (kPrefetch) {
        if (more) {
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int v = 0; v < XV; v++) xcur[nt][v] = xnext[nt][v];
        }
      }
    }

    // cross-warp reduction: red[warp][row][m]
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      red[warp][g][nt * 8 + 2 * t] = acc[nt][0];
      red[warp][g][nt * 8 + 2 * t + 1] = acc[nt][1];
      red[warp][g + 8][nt * 8 + 2 * t] = acc[nt][2];
      red[warp][g + 8][nt * 8 + 2 * t + 1] = acc[nt][3];
    }
  }
  __syncthreads();
  if (gave_up) return; // a copy never arrived: leave Y untouched, the status word says why
  for (int idx = threadIdx.x; idx < kRowsPerBlock * NT * 8; idx += kThreadsWo + 32) {
    const int r = idx % kRowsPerBlock, m = idx / kRowsPerBlock;
    const int n = n0 + r;
    if (m >= M || n >= N) continue;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; w++) s += red[w][r][m];
    if constexpr (WBITS == 8) s *= load_scale(scale, sdt, n);
    Y[(int64_t)m * N + n] = FloatIO<XT>::from_f32(s);
  }
}

template <int NT> constexpr int wo_dynamic_smem() { return 128 + kStagesWo * kStageBytesWo + kWarps * kRowsPerBlock * (NT * 8 + 1) * 4; }

template <typename XT, int WBITS, int NT>
int launch_wo_nt(const CUtensorMap &map_w, const XT *xp, const void *scale, int sdt, XT *yp, int mc, int N, int K, int block,
                 int *status, unsigned grid, cudaStream_t st) {
  auto kern = wo_linear_kernel<XT, WBITS, NT>;
  constexpr int smem = wo_dynamic_smem<NT>();
  static bool configured[64] = {false};
  int dev = 0;
  QL_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    QL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  }
  kern<<<grid, kThreadsWo + 32, smem, st>>>(map_w, xp, scale, sdt, yp, mc, N, K, block, status);
  count_launches(1);
  return QL_OK;
}

template <typename XT, int WBITS>
int launch_wo_t(const void *X, const void *W, const void *scale, int sdt, void *Y, int M, int N, int K, int block,
                cudaStream_t st) {
  const unsigned grid = (unsigned)((N + kRowsPerBlock - 1) / kRowsPerBlock);
  int *status = device_status_word();
  if (!status) return set_error(QL_ERR_CUDA, "weight-only linear: could not allocate the device status word");
  // the weights as a [N, row_bytes / 4] matrix of 32-bit words: one box = 16 rows x 1024 bytes
  CUtensorMap map_w;
  {
    EncodeTiledFn enc;
    int rc = get_encode_fn(&enc);
    if (rc != QL_OK) return rc;
    const int64_t row_bytes = (int64_t)K * WBITS / 8;
    cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 4), (cuuint64_t)N};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(kChunkBytes / 4), (cuuint32_t)kRowsPerBlock};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(W), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(QL_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  }
  // batches larger than 32 rows are walked in slices; the weights of the later slices come from L2
  for (int m0 = 0; m0 < M; m0 += 32) {
    const int mc = min(32, M - m0);
    const XT *xp = static_cast<const XT *>(X) + (int64_t)m0 * K;
    XT *yp = static_cast<XT *>(Y) + (int64_t)m0 * N;
    int rc;
    if (mc <= 8) rc = launch_wo_nt<XT, WBITS, 1>(map_w, xp, scale, sdt, yp, mc, N, K, block, status, grid, st);
    else if (mc <= 16) rc = launch_wo_nt<XT, WBITS, 2>(map_w, xp, scale, sdt, yp, mc, N, K, block, status, grid, st);
    else rc = launch_wo_nt<XT, WBITS, 4>(map_w, xp, scale, sdt, yp, mc, N, K, block, status, grid, st);
    if (rc != QL_OK) return rc;
  }
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

} // namespace

int launch_wo_linear(int wbits, int xdt, const void *X, const void *W, const void *scale, int sdt, void *Y, int M,
                     int N, int K, int block, cudaStream_t st) {
  if (M == 0 || N == 0) return QL_OK;
  if (wbits == 8) {
    if (xdt == QL_F16) return launch_wo_t<__half, 8>(X, W, scale, sdt, Y, M, N, K, block, st);
    return launch_wo_t<__nv_bfloat16, 8>(X, W, scale, sdt, Y, M, N, K, block, st);
  }
  if (xdt == QL_F16) return launch_wo_t<__half, 4>(X, W, scale, sdt, Y, M, N, K, block, st);
  return launch_wo_t<__nv_bfloat16, 4>(X, W, scale, sdt, Y, M, N, K, block, st);
}

} // namespace ql
