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
// One block owns 16 output channels; its 8 warps split K, keep several iterations' worth of 16-byte
// weight loads in flight in registers, and reduce through shared memory.  Where N / 16 blocks are too few to
// keep every SM's load queues full (N = 4096 gives 256 blocks for 148 SMs), K is also split across the CTAs of
// a thread-block cluster: each CTA takes a slice of K, writes its 16 x M partial sums into the leader's shared
// memory (distributed shared memory) and the leader adds them up in a fixed order.  (A shared-memory ring fed by
// TMA was measured slower here: blocks are short-lived, so the ring's set-up and the copy latency at the
// start of every block cost more than the deeper prefetch gained.)
// Reference composition this implements: tripy/nvtripy/frontend/module/linear.py:140-151
// (quantize -> dequantize -> x @ transpose(w)) with the dequantize folded into the product.
#include <cuda/std/type_traits>
#include <cstdlib>

#include "ql_common.cuh"

namespace ql {
namespace {

constexpr int kWarps = 8;
constexpr int kThreadsWo = kWarps * 32;
constexpr int kRowsPerBlock = 16;
constexpr int kMaxKSplit = 8; // CTAs of a cluster that share one block of output channels

__device__ __forceinline__ uint32_t wo_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void wo_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// f32 store into the same shared-memory variable of CTA `rank` of the cluster
__device__ __forceinline__ void wo_store_remote(float *local_addr, uint32_t rank, float v) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(local_addr), r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r), "f"(v) : "memory");
}

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

// bytes I and I+1 of `w` (two's-complement int8) -> packed pair of XT holding the exact integers
template <typename XT, int I>
__device__ __forceinline__ uint32_t int8_pair(uint32_t w) {
  if constexpr (cuda::std::is_same<XT, __half>::value) {
    // f16 0x6400 | b is 1024 + b with b = value + 128 after flipping the sign bit; subtract 1024 + 128
    uint32_t v = __byte_perm(w ^ 0x80808080u, 0x64646464u, 0x4040 | I | ((I + 1) << 8));
    __half2 h = __hsub2(*reinterpret_cast<__half2 *>(&v), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<uint32_t *>(&h);
  } else {
    // bf16 has 7 mantissa bits: 0x4300 | (b & 0x7F) is 128 + (b & 0x7F), which is value + 128 for value >= 0
    // and value + 256 for value < 0; subtract 128 or 256, chosen by the sign bit (0x4300 | 0x80 = 256.0)
    const uint32_t w16 = __byte_perm(w, 0u, 0x4140 + I * 0x0101); // bytes I, I+1 spread into the two 16-bit lanes
    uint32_t y = (w16 & 0x007F007Fu) | 0x43004300u;
    uint32_t c = (w16 & 0x00800080u) | 0x43004300u;
    __nv_bfloat162 d = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&y), *reinterpret_cast<__nv_bfloat162 *>(&c));
    return *reinterpret_cast<uint32_t *>(&d);
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
  static constexpr int kXWords = kElemsPerLane * 2 / 16;  // 16-byte words of X per lane, row and iteration
};

// NT = number of 8-row tiles of X handled at once (M <= 8 * NT); U = iterations whose loads are issued
// together before any of them is consumed.
template <typename XT, int WBITS, int NT, int U, int MINB>
__global__ void __launch_bounds__(kThreadsWo, MINB)
wo_linear_kernel(const XT *__restrict__ X, const uint8_t *__restrict__ W, const void *__restrict__ scale, int sdt,
                 XT *__restrict__ Y, int M, int N, int K, int block, int ksplit) {
  using T = WoTraits<WBITS>;
  constexpr int XV = T::kXWords;
  __shared__ float red[kWarps][kRowsPerBlock][NT * 8 + 1];
  __shared__ float part[kMaxKSplit][kRowsPerBlock * NT * 8]; // leader only: one slot per CTA of the cluster

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * kRowsPerBlock;
  const int row_a = min(n0 + g, N - 1), row_b = min(n0 + g + 8, N - 1);
  const int64_t row_bytes = (int64_t)K * WBITS / 8;
  const uint8_t *wa_ptr = W + (int64_t)row_a * row_bytes + t * 16;
  const uint8_t *wb_ptr = W + (int64_t)row_b * row_bytes + t * 16;
  // this CTA's slice of the k iterations (the cluster lies along grid.y)
  const int kslice = ksplit > 1 ? (int)wo_cluster_rank() : 0;
  const int all_iters = K / T::kStep, per_slice = (all_iters + ksplit - 1) / ksplit;
  const int it_begin = kslice * per_slice, n_iters = min(all_iters, it_begin + per_slice);
  const int nb = (WBITS == 4) ? K / block : 0;

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  // the kernel that follows on the stream may start being scheduled as this one's blocks retire
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  for (int it0 = it_begin + warp; it0 < n_iters; it0 += kWarps * U) {
    // ---- issue every load of this group of iterations: the weights first
    uint4 wa[U], wb[U], xv[U][NT][XV];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int it = it0 + u * kWarps;
      if (it < n_iters) {
        wa[u] = __ldcs(reinterpret_cast<const uint4 *>(wa_ptr + (int64_t)it * 64));
        wb[u] = __ldcs(reinterpret_cast<const uint4 *>(wb_ptr + (int64_t)it * 64));
      }
    }
    // The activations may be the result of the kernel that precedes this one on the stream.  When the launch was
    // allowed to start before that kernel has finished (see QL_WEIGHTS_CONSTANT), everything up to here overlapped
    // with its tail; this waits until it is complete and its writes are visible (no effect otherwise).
    if (it0 == it_begin + warp) asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int it = it0 + u * kWarps;
      if (it < n_iters) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          const int m = nt * 8 + g;
          if (m < M) {
            const uint4 *xp = reinterpret_cast<const uint4 *>(X + (int64_t)m * K + it * T::kStep + t * T::kElemsPerLane);
#pragma unroll
            for (int v = 0; v < XV; v++) xv[u][nt][v] = __ldg(xp + v);
          } else {
#pragma unroll
            for (int v = 0; v < XV; v++) xv[u][nt][v] = make_uint4(0, 0, 0, 0);
          }
        }
      }
    }
    // ---- consume them
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int it = it0 + u * kWarps;
      if (it >= n_iters) break;
      const int kb = it * T::kStep;
      const uint32_t wav[4] = {wa[u].x, wa[u].y, wa[u].z, wa[u].w};
      const uint32_t wbv[4] = {wb[u].x, wb[u].y, wb[u].z, wb[u].w};
      if constexpr (WBITS == 8) {
        uint32_t a[4][4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          a[j][0] = int8_pair<XT, 0>(wav[j]);
          a[j][1] = int8_pair<XT, 0>(wbv[j]);
          a[j][2] = int8_pair<XT, 2>(wav[j]);
          a[j][3] = int8_pair<XT, 2>(wbv[j]);
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          const uint32_t xw[8] = {xv[u][nt][0].x, xv[u][nt][0].y, xv[u][nt][0].z, xv[u][nt][0].w,
                                  xv[u][nt][1].x, xv[u][nt][1].y, xv[u][nt][1].z, xv[u][nt][1].w};
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
            const uint4 x8 = xv[u][nt][j];
            // x pairs (0,4) (1,5) (2,6) (3,7) to line up with the weight pairs
            uint32_t p04 = __byte_perm(x8.x, x8.z, 0x5410), p15 = __byte_perm(x8.x, x8.z, 0x7632);
            uint32_t p26 = __byte_perm(x8.y, x8.w, 0x5410), p37 = __byte_perm(x8.y, x8.w, 0x7632);
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
    }
  }

  asm volatile("griddepcontrol.wait;" ::: "memory"); // warps without a k step of their own; Y is written only after this
  // cross-warp reduction: red[warp][row][m]
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    red[warp][g][nt * 8 + 2 * t] = acc[nt][0];
    red[warp][g][nt * 8 + 2 * t + 1] = acc[nt][1];
    red[warp][g + 8][nt * 8 + 2 * t] = acc[nt][2];
    red[warp][g + 8][nt * 8 + 2 * t + 1] = acc[nt][3];
  }
  __syncthreads();
  if (ksplit > 1) {
    // every CTA hands its partial sums to the leader; the leader adds the slices in rank order
    for (int idx = threadIdx.x; idx < kRowsPerBlock * NT * 8; idx += kThreadsWo) {
      const int r = idx % kRowsPerBlock, m = idx / kRowsPerBlock;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; w++) s += red[w][r][m];
      wo_store_remote(&part[kslice][idx], 0, s);
    }
    wo_cluster_sync();
    if (kslice != 0) return;
  }
  for (int idx = threadIdx.x; idx < kRowsPerBlock * NT * 8; idx += kThreadsWo) {
    const int r = idx % kRowsPerBlock, m = idx / kRowsPerBlock;
    const int n = n0 + r;
    if (m >= M || n >= N) continue;
    float s = 0.f;
    if (ksplit > 1) {
      for (int c = 0; c < ksplit; c++) s += part[c][idx];
    } else {
#pragma unroll
      for (int w = 0; w < kWarps; w++) s += red[w][r][m];
    }
    if constexpr (WBITS == 8) s *= load_scale(scale, sdt, n);
    Y[(int64_t)m * N + n] = FloatIO<XT>::from_f32(s);
  }
}

// How many CTAs share one block of output channels.  Splitting pays while the blocks of an unsplit launch cannot
// fill the resident-block slots of the device a few times over; every slice keeps at least one k step per warp.
int read_forced_ksplit() {
  const char *e = getenv("QL_WO_KSPLIT"); // tuning aid
  return e ? atoi(e) : 0;
}
int g_forced_ksplit = read_forced_ksplit(); // read when the library is loaded and by ql_reload_tuning()

int pick_ksplit(unsigned row_blocks, int n_iters, int resident_per_sm) {
  const int forced = g_forced_ksplit;
  // Measured on B200 (N = 4096 and 11008, K = 4096, M = 1 .. 64): every doubling of the split costs 1.5 - 4 us
  // (cluster scheduling, the exchange and its barrier) and never pays for itself, so nothing is split unless asked.
  (void)row_blocks;
  (void)resident_per_sm;
  int ks = forced > 0 ? forced : 1;
  if (ks > kMaxKSplit) ks = kMaxKSplit;
  while (ks > 1 && n_iters / ks < 1) ks /= 2;
  return ks;
}

template <typename XT, int WBITS>
int launch_wo_t(const void *X, const void *W, const void *scale, int sdt, void *Y, int M, int N, int K, int block,
                bool weights_constant, cudaStream_t st) {
  const unsigned grid = (unsigned)((N + kRowsPerBlock - 1) / kRowsPerBlock);
  const uint8_t *wp = static_cast<const uint8_t *>(W);
  // batches larger than 32 rows are walked in slices; the weights of the later slices come from L2
  for (int m0 = 0; m0 < M; m0 += 32) {
    const int mc = min(32, M - m0);
    const XT *xp = static_cast<const XT *>(X) + (int64_t)m0 * K;
    XT *yp = static_cast<XT *>(Y) + (int64_t)m0 * N;
    // (k-steps in flight per warp, minimum resident blocks) per batch width, from timing on B200: many
    // resident blocks with one step in flight each beat fewer blocks with deeper unrolling
#define QL_WO_LAUNCH(NT_, U_, MB_)                                                                                        \
  do {                                                                                                                    \
    const int ks = pick_ksplit(grid, K / WoTraits<WBITS>::kStep, MB_);                                                    \
    cudaLaunchConfig_t cfg = {};                                                                                          \
    cfg.gridDim = dim3(grid, ks, 1);                                                                                      \
    cfg.blockDim = dim3(kThreadsWo, 1, 1);                                                                                \
    cfg.stream = st;                                                                                                      \
    cudaLaunchAttribute attr[2];                                                                                          \
    attr[0].id = cudaLaunchAttributeClusterDimension;                                                                     \
    attr[0].val.clusterDim.x = 1;                                                                                         \
    attr[0].val.clusterDim.y = ks;                                                                                        \
    attr[0].val.clusterDim.z = 1;                                                                                         \
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                                      \
    attr[1].val.programmaticStreamSerializationAllowed = 1;                                                               \
    cfg.attrs = attr;                                                                                                     \
    cfg.numAttrs = (early_start && ks == 1) ? 2 : 1;                                                                      \
    QL_CUDA_TRY(cudaLaunchKernelEx(&cfg, wo_linear_kernel<XT, WBITS, NT_, U_, MB_>, xp, wp, scale, sdt, yp, mc, N, K, block, ks)); \
  } while (0)
    // (int4 keeps four X words per row and step alive instead of two: the int8 settings would spill.)  When the
    // grid cannot fill the SMs several times over, occupancy is not what limits the bytes in flight, so each warp
    // issues all of its few steps at once instead.
    const bool few_blocks = grid < 3u * (unsigned)sm_count();
    // Starting before the preceding kernel has finished (only with constant weights, only for the first slice)
    // hides the launch gap and the first loads' latency: 6.8 -> 5.2 us at N = K = 4096 int4, M = 1.  With a grid
    // that fills the device and at most 8 rows the early blocks only get in the way (measured: 6 % slower).
    const bool early_start = weights_constant && m0 == 0 && (few_blocks || mc > 8);
    if (mc <= 8) {
      if (few_blocks) QL_WO_LAUNCH(1, 4, 2);
      else if constexpr (WBITS == 8) QL_WO_LAUNCH(1, 1, 6);
      else QL_WO_LAUNCH(1, 1, 4);
    } else if (mc <= 16) {
      if (few_blocks) QL_WO_LAUNCH(2, 2, 2);
      else if constexpr (WBITS == 8) QL_WO_LAUNCH(2, 2, 3);
      else QL_WO_LAUNCH(2, 1, 3);
    } else {
      QL_WO_LAUNCH(4, 1, 2);
    }
#undef QL_WO_LAUNCH
    count_launches(1);
  }
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

} // namespace

void wo_reload_tuning() { g_forced_ksplit = read_forced_ksplit(); }

// weights_constant: W and scale were written before the kernel preceding this launch on the stream started, so the
// kernel may begin fetching them while that kernel is still finishing.
int launch_wo_linear(int wbits, int xdt, const void *X, const void *W, const void *scale, int sdt, void *Y, int M,
                     int N, int K, int block, bool weights_constant, cudaStream_t st) {
  if (M == 0 || N == 0) return QL_OK;
  if (wbits == 8) {
    if (xdt == QL_F16) return launch_wo_t<__half, 8>(X, W, scale, sdt, Y, M, N, K, block, weights_constant, st);
    return launch_wo_t<__nv_bfloat16, 8>(X, W, scale, sdt, Y, M, N, K, block, weights_constant, st);
  }
  if (xdt == QL_F16) return launch_wo_t<__half, 4>(X, W, scale, sdt, Y, M, N, K, block, weights_constant, st);
  return launch_wo_t<__nv_bfloat16, 4>(X, W, scale, sdt, Y, M, N, K, block, weights_constant, st);
}

} // namespace ql
