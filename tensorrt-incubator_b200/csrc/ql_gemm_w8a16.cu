// W8A16 linear for large batches on the tcgen05 tensor cores, weights dequantized inside the kernel:
//     Y[M,N] = (X[M,K] . Wq[N,K]^T) * scale[n],  X bf16|f16, Wq int8, f32 accumulation in tensor memory.
// The int8 weights are read from HBM exactly once, as int8.  Per k-block TMA brings a
// [128 x 64] tile of X (128-byte swizzle) and the raw [BN x 64] int8 tile of W; eight converter warps
// widen the weights to the activation type (exact: |q| <= 128 fits the significand) and store them in
// the 128-byte-swizzled K-major layout the MMA's shared-memory descriptor expects, fence the writes
// for the async proxy and signal the MMA warp.  The per-channel scale is applied to the f32
// accumulator in the epilogue, which equals scaling every weight first up to f32 rounding
// (reference composition: quantize -> dequantize -> matmul, tripy/nvtripy/frontend/module/linear.py:140-151).
//
// Warps: 0 TMA producer (W), 1 TMEM owner + MMA issuer, 2-5 epilogue, 6-13 converters, 14 TMA producer (X).
// All waits bounded.
#include <cuda/std/type_traits>
#include <cstdlib>

#include "ql_common.cuh"
#include "ql_tc_common.cuh"

namespace ql {
namespace {

constexpr int kConvWarps = 8;
constexpr int kConvThreads = kConvWarps * 32;
constexpr int kW8Threads = (6 + kConvWarps + 1) * 32; // TMA(W), MMA, 4 epilogue, converters, TMA(X)
constexpr int kWarpXProducer = 6 + kConvWarps;
constexpr int BKE = 64; // k elements per stage: 128 bytes of X, 64 bytes of int8 W

// Three rings, so that each resource is held only as long as it is needed: the small raw int8 tiles
// sit in a deep ring (their HBM latency is the one to hide), X tiles in a 4-deep ring released by the
// MMA, and the widened tiles in a 2- or 3-deep ring between the converters and the MMA.
template <int BN> struct W8Smem {
  static constexpr int kA = BM * BK_BYTES;
  static constexpr int kConv = BN * BK_BYTES;
  static constexpr int kRaw = BN * BKE;
  static constexpr int NA = (BN <= 128) ? 6 : 4;
  static constexpr int NC = (BN >= 256) ? 2 : 3;
  static constexpr int kRawFit = (200 * 1024 - NA * kA - NC * kConv) / kRaw;
  static constexpr int NR = kRawFit > 16 ? 16 : kRawFit;
  static constexpr int kOffA = 0;
  static constexpr int kOffConv = NA * kA;
  static constexpr int kOffRaw = kOffConv + NC * kConv;
  static constexpr int kBarriers = kOffRaw + NR * kRaw; // raw_full[NR] raw_empty[NR] a_full[NA] a_empty[NA] conv_ready[NC] conv_empty[NC] tfull[2] tempty[2] drain
  static constexpr int kNumBarriers = 2 * NR + 2 * NA + 2 * NC + 5;
  static constexpr int kTmemPtr = kBarriers + kNumBarriers * 8;
  static constexpr int kAbort = kTmemPtr + 4;
  static constexpr int kTotal = kAbort + 4;
  static constexpr int kDynamic = kTotal + 1024;
  static_assert(NR >= 2, "raw ring too shallow");
};

struct W8Args {
  void *Y;
  const void *scale; // per output channel, f32 | f16 | bf16
  int sdt;
  int M, N, num_kb;
  int tiles_m, tiles_n, group_m;
  int *status;
};

__device__ __forceinline__ void w8_tile_coords(const W8Args &a, int tile, int *mt, int *nt) {
  const int per_group = a.group_m * a.tiles_n;
  const int grp = tile / per_group;
  const int first_m = grp * a.group_m;
  const int gsz = min(a.group_m, a.tiles_m - first_m);
  const int local = tile - grp * per_group;
  *mt = first_m + local % gsz;
  *nt = local / gsz;
}

// bytes I, I+1 of w (two's-complement int8) -> exact pair of XT (same tricks as the small-batch kernel)
template <typename XT, int I>
__device__ __forceinline__ uint32_t widen_pair(uint32_t w) {
  if constexpr (cuda::std::is_same<XT, __half>::value) {
    uint32_t v = __byte_perm(w ^ 0x80808080u, 0x64646464u, 0x4040 | I | ((I + 1) << 8));
    __half2 h = __hsub2(*reinterpret_cast<__half2 *>(&v), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<uint32_t *>(&h);
  } else {
    const uint32_t w16 = __byte_perm(w, 0u, 0x4140 + I * 0x0101);
    uint32_t y = (w16 & 0x007F007Fu) | 0x43004300u; // 128 + low seven bits
    uint32_t c = (w16 & 0x00800080u) | 0x43004300u; // 128, or 256 when the sign bit is set
    __nv_bfloat162 d = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&y), *reinterpret_cast<__nv_bfloat162 *>(&c));
    return *reinterpret_cast<uint32_t *>(&d);
  }
}

// Every CTA walks the k-blocks in the same cyclic order but starts at a different one, so that the CTAs
// which share an X tile (all of them, when M fits one row tile) do not ask L2 for the same lines at the
// same moment.  The sum over k does not depend on the order beyond f32 rounding.
__device__ __forceinline__ int rotated_kb(int kb, int num_kb) {
  const int v = kb + (int)((blockIdx.x * 7u) % (unsigned)num_kb);
  return v >= num_kb ? v - num_kb : v;
}

struct Ring {
  int stage = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int n) {
    if (++stage == n) { stage = 0; phase ^= 1; }
  }
};

template <typename XT, int BN>
__global__ void __launch_bounds__(kW8Threads, 1)
gemm_w8a16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const W8Args args) {
  using L = W8Smem<BN>;
  constexpr int NR = L::NR, NA = L::NA, NC = L::NC;
  constexpr int KIND = cuda::std::is_same<XT, __half>::value ? KIND_F16 : KIND_BF16;
  constexpr uint32_t kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarriers;
  auto raw_full = [&](int s) { return bar_base + 8u * s; };
  auto raw_empty = [&](int s) { return bar_base + 8u * (NR + s); };
  auto a_full = [&](int s) { return bar_base + 8u * (2 * NR + s); };
  auto a_empty = [&](int s) { return bar_base + 8u * (2 * NR + NA + s); };
  auto conv_ready = [&](int s) { return bar_base + 8u * (2 * NR + 2 * NA + s); };
  auto conv_empty = [&](int s) { return bar_base + 8u * (2 * NR + 2 * NA + NC + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * NR + 2 * NA + 2 * NC + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * NR + 2 * NA + 2 * NC + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * NR + 2 * NA + 2 * NC + 4);
  volatile uint32_t *tmem_ptr_smem = reinterpret_cast<volatile uint32_t *>(smem + L::kTmemPtr);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = args.tiles_m * args.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NR; s++) {
      mbar_init(raw_full(s), 1);
      mbar_init(raw_empty(s), kConvWarps);
    }
    for (int s = 0; s < NA; s++) {
      mbar_init(a_full(s), 1);
      mbar_init(a_empty(s), 1);
    }
    for (int s = 0; s < NC; s++) {
      mbar_init(conv_ready(s), kConvWarps);
      mbar_init(conv_empty(s), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_ptr_smem)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer, raw int8 weights
    if (lane == 0) {
      Ring r;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mt, nt;
        w8_tile_coords(args, tile, &mt, &nt);
        for (int kb = 0; kb < args.num_kb; kb++) {
          if (!mbar_wait(raw_empty(r.stage), r.phase ^ 1, abort_flag, args.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(raw_full(r.stage), L::kRaw);
          tma_load_2d(smem_base + L::kOffRaw + r.stage * L::kRaw, &map_w, raw_full(r.stage), rotated_kb(kb, args.num_kb) * BKE, nt * BN);
          r.advance(NR);
        }
      }
    }
  } else if (warp == kWarpXProducer) {
    // ------------------------------------------------------------------ TMA producer, X tiles
    if (lane == 0) {
      Ring r;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mt, nt;
        w8_tile_coords(args, tile, &mt, &nt);
        for (int kb = 0; kb < args.num_kb; kb++) {
          if (!mbar_wait(a_empty(r.stage), r.phase ^ 1, abort_flag, args.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(a_full(r.stage), L::kA);
          tma_load_2d(smem_base + L::kOffA + r.stage * L::kA, &map_x, a_full(r.stage), rotated_kb(kb, args.num_kb) * BKE, mt * BM);
          r.advance(NA);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc<KIND, BN>();
      Ring ra, rc;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, it++) {
        const int buf = it & 1;
        if (!mbar_wait(tempty_bar(buf), ((it >> 1) & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < args.num_kb; kb++) {
          if (!mbar_wait(a_full(ra.stage), ra.phase, abort_flag, args.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          if (!mbar_wait(conv_ready(rc.stage), rc.phase, abort_flag, args.status, ST_TIMEOUT_READY)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_base + L::kOffA + ra.stage * L::kA);
          const uint64_t bdesc = make_smem_desc(smem_base + L::kOffConv + rc.stage * L::kConv);
#pragma unroll
          for (int k = 0; k < BK_BYTES / 32; k++)
            tc_mma<KIND>(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(a_empty(ra.stage));
          tc_commit(conv_empty(rc.stage));
          ra.advance(NA);
          rc.advance(NC);
        }
        if (ok) tc_commit(tfull_bar(buf));
      }
      tc_commit(drain_bar);
      const long long t0 = clock64();
      while (!mbar_try_wait(drain_bar, 0)) {
        if (clock64() - t0 > kWaitLimitCycles) { atomicCAS(args.status, 0, ST_TIMEOUT_DRAIN); break; }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ converters
    const int ctid = threadIdx.x - 6 * 32;
    Ring rr, rc;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < args.num_kb; kb++) {
        if (!mbar_wait(raw_full(rr.stage), rr.phase, abort_flag, args.status, ST_TIMEOUT_FULL)) { ok = false; break; }
        if (!mbar_wait(conv_empty(rc.stage), rc.phase ^ 1, abort_flag, args.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
        const uint8_t *raw = smem + L::kOffRaw + rr.stage * L::kRaw;
        uint8_t *conv = smem + L::kOffConv + rc.stage * L::kConv;
#pragma unroll 2
        for (int idx = ctid; idx < BN * 4; idx += kConvThreads) {
          const int r = idx >> 2, c = idx & 3;
          const uint4 w = *reinterpret_cast<const uint4 *>(raw + r * BKE + c * 16);
          const uint4 lo = make_uint4(widen_pair<XT, 0>(w.x), widen_pair<XT, 2>(w.x), widen_pair<XT, 0>(w.y), widen_pair<XT, 2>(w.y));
          const uint4 hi = make_uint4(widen_pair<XT, 0>(w.z), widen_pair<XT, 2>(w.z), widen_pair<XT, 0>(w.w), widen_pair<XT, 2>(w.w));
          uint8_t *row = conv + r * BK_BYTES;
          const int sw = r & 7; // 128-byte swizzle: 16-byte chunk index XOR (row mod 8)
          *reinterpret_cast<uint4 *>(row + (((2 * c) ^ sw) << 4)) = lo;
          *reinterpret_cast<uint4 *>(row + (((2 * c + 1) ^ sw) << 4)) = hi;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(conv_ready(rc.stage));
          mbar_arrive(raw_empty(rr.stage));
        }
        rr.advance(NR);
        rc.advance(NC);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    XT *Y = static_cast<XT *>(args.Y);
    const bool vec_ok = (args.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, it++) {
      const int buf = it & 1;
      int mt, nt;
      w8_tile_coords(args, tile, &mt, &nt);
      const int m0 = mt * BM, n0 = nt * BN;
      if (!mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int m = m0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 16; c++) {
        uint32_t r[16];
        tmem_load_16(taddr + c * 16, r);
        const int n = n0 + c * 16;
        if (m < args.M && n < args.N) {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[j]) * ((n + j < args.N) ? load_scale(args.scale, args.sdt, n + j) : 0.f);
          XT *row = Y + (size_t)m * args.N + n;
          if (vec_ok && n + 16 <= args.N) {
            __stcs(reinterpret_cast<uint4 *>(row), make_uint4(pack2<XT>(v[0], v[1]), pack2<XT>(v[2], v[3]), pack2<XT>(v[4], v[5]), pack2<XT>(v[6], v[7])));
            __stcs(reinterpret_cast<uint4 *>(row + 8), make_uint4(pack2<XT>(v[8], v[9]), pack2<XT>(v[10], v[11]), pack2<XT>(v[12], v[13]), pack2<XT>(v[14], v[15])));
          } else {
            for (int j = 0; j < 16 && n + j < args.N; j++) row[j] = FloatIO<XT>::from_f32(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <typename XT, int BN>
int launch_w8_bn(const CUtensorMap &mx, const CUtensorMap &mw, W8Args args, cudaStream_t st) {
  using L = W8Smem<BN>;
  auto kern = gemm_w8a16_kernel<XT, BN>;
  static bool configured[64] = {false};
  int dev = 0;
  QL_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    QL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic));
    configured[dev] = true;
  }
  const int tiles = args.tiles_m * args.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kW8Threads, L::kDynamic, st>>>(mx, mw, args);
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

template <typename XT>
int launch_w8_t(const void *X, const void *W, const void *scale, int sdt, void *Y, int M, int N, int K, cudaStream_t st) {
  constexpr int KIND = cuda::std::is_same<XT, __half>::value ? KIND_F16 : KIND_BF16;
  W8Args args;
  args.Y = Y;
  args.scale = scale;
  args.sdt = sdt;
  args.M = M;
  args.N = N;
  args.num_kb = K / BKE;
  args.tiles_m = (M + BM - 1) / BM;
  args.status = device_status_word();
  if (!args.status) return set_error(QL_ERR_CUDA, "linear_w8a16: could not allocate the device status word");
  // pick the column-tile width: waves of tiles over the SMs times the bytes a tile pulls per k-block
  const int sms = sm_count();
  int best_bn = 256;
  long long best_cost = -1;
  for (int bn : {256, 128, 96, 80, 64, 48, 32}) {
    const long long tiles = (long long)args.tiles_m * ((N + bn - 1) / bn);
    const long long waves = (tiles + sms - 1) / sms;
    const long long cost = waves * (BM + bn);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_bn = bn; }
  }
  args.tiles_n = (N + best_bn - 1) / best_bn;
  {
    const long long band = (16ll << 20) / ((long long)BM * K * 2);
    args.group_m = (int)(band < 4 ? 4 : band);
    if (args.group_m > args.tiles_m) args.group_m = args.tiles_m;
  }
  CUtensorMap mx, mw;
  int rc;
  if ((rc = make_map(&mx, KIND, X, M, K, BM)) != QL_OK) return rc;
  if ((rc = make_map_bytes(&mw, W, N, K, BKE, best_bn)) != QL_OK) return rc;
  switch (best_bn) {
  case 256: return launch_w8_bn<XT, 256>(mx, mw, args, st);
  case 128: return launch_w8_bn<XT, 128>(mx, mw, args, st);
  case 96: return launch_w8_bn<XT, 96>(mx, mw, args, st);
  case 80: return launch_w8_bn<XT, 80>(mx, mw, args, st);
  case 64: return launch_w8_bn<XT, 64>(mx, mw, args, st);
  case 48: return launch_w8_bn<XT, 48>(mx, mw, args, st);
  default: return launch_w8_bn<XT, 32>(mx, mw, args, st);
  }
}

// int8 -> f16 / bf16, exact; 16 values per thread
template <typename XT>
__global__ void __launch_bounds__(256) widen_i8_kernel(const uint8_t *__restrict__ w, XT *__restrict__ out, int64_t n16) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n16) return;
  const uint4 raw = __ldcs(reinterpret_cast<const uint4 *>(w) + i);
  const uint32_t v[4] = {raw.x, raw.y, raw.z, raw.w};
  reinterpret_cast<uint4 *>(out)[2 * i] = make_uint4(widen_pair<XT, 0>(v[0]), widen_pair<XT, 2>(v[0]), widen_pair<XT, 0>(v[1]), widen_pair<XT, 2>(v[1]));
  reinterpret_cast<uint4 *>(out)[2 * i + 1] = make_uint4(widen_pair<XT, 0>(v[2]), widen_pair<XT, 2>(v[2]), widen_pair<XT, 0>(v[3]), widen_pair<XT, 2>(v[3]));
}

__global__ void __launch_bounds__(256) scale_to_f32_kernel(const void *__restrict__ s, int sdt, float *__restrict__ out, int n) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < n) out[i] = load_scale(s, sdt, i);
}

constexpr int kWidenCounters = 1024; // tile counters of the single-launch route (ceil(N / 256) + 1 are used)

} // namespace

int gemm16_device(int dtype, const void *X, const void *W, const float *sb, int sb_n, void *Y, int M, int N, int K,
                  cudaStream_t st);
int gemm16_widen_device(int dtype, const void *X, const void *Wraw, void *wide, int *counters, const void *scale, int sdt, void *Y,
                        int M, int N, int K, cudaStream_t st);

// Compute-bound batches: the weights are widened once per call into scratch (exact) and the 16-bit tcgen05 GEMM
// runs on the scratch with the per-channel scales in its epilogue.  (The per-tile conversion of the kernel above
// repeats the widening for every row tile and is bound by its converter warps once M grows.)  Where the CTA-pair
// kernel applies, the widening runs inside it, ahead of the tiles that need it; otherwise in a kernel of its own.
int launch_w8a16_widen(int xdt, const void *X, const void *W, const void *scale, int sdt, void *Y, int M, int N, int K,
                       cudaStream_t st) {
  // Scratch of this call alone, from the stream-ordered allocator: the 16-bit copy of the weights, f32 scales and the
  // tile counters.  Nothing is shared between calls, so calls on different streams may overlap, a later call with
  // larger weights cannot invalidate an address an earlier (or captured) call still uses, and inside a stream
  // capture the allocation becomes a node of the graph.
  const int64_t n = (int64_t)N * K;
  const size_t wide_bytes = (size_t)n * 2, scale_off = (wide_bytes + 255) & ~size_t(255);
  const size_t ctr_off = (scale_off + (size_t)N * sizeof(float) + 255) & ~size_t(255);
  uint8_t *scratch = nullptr;
  keep_scratch_pool_warm();
  QL_CUDA_TRY(cudaMallocAsync(&scratch, ctr_off + kWidenCounters * sizeof(int), st));
  float *sf = reinterpret_cast<float *>(scratch + scale_off);
  int rc = QL_ERR_UNSUPPORTED;
  if ((N + 255) / 256 + 1 <= kWidenCounters) {
    int *counters = reinterpret_cast<int *>(scratch + ctr_off);
    cudaError_t me = cudaMemsetAsync(counters, 0, kWidenCounters * sizeof(int), st);
    if (me != cudaSuccess) {
      cudaFreeAsync(scratch, st);
      return cuda_error(me, "cudaMemsetAsync");
    }
    rc = gemm16_widen_device(xdt, X, W, scratch, counters, scale, sdt, Y, M, N, K, st);
  }
  if (rc == QL_ERR_UNSUPPORTED) {
    const int64_t n16 = n / 16; // K % 64 == 0
    if (xdt == QL_F16) widen_i8_kernel<__half><<<(unsigned)((n16 + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t *>(W), reinterpret_cast<__half *>(scratch), n16);
    else widen_i8_kernel<__nv_bfloat16><<<(unsigned)((n16 + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t *>(W), reinterpret_cast<__nv_bfloat16 *>(scratch), n16);
    scale_to_f32_kernel<<<(N + 255) / 256, 256, 0, st>>>(scale, sdt, sf, N);
    count_launches(2);
    cudaError_t le = cudaGetLastError();
    rc = le != cudaSuccess ? cuda_error(le, "widen_i8_kernel") : gemm16_device(xdt, X, scratch, sf, N, Y, M, N, K, st);
  }
  cudaError_t fe = cudaFreeAsync(scratch, st);
  if (rc == QL_OK && fe != cudaSuccess) return cuda_error(fe, "cudaFreeAsync");
  return rc;
}

// Y = (X . Wq^T) * scale[n] with the int8 -> 16-bit conversion inside the kernel (K % 64 == 0).
int launch_w8a16_fused(int xdt, const void *X, const void *W, const void *scale, int sdt, void *Y, int M, int N, int K,
                       cudaStream_t st) {
  if (xdt == QL_F16) return launch_w8_t<__half>(X, W, scale, sdt, Y, M, N, K, st);
  return launch_w8_t<__nv_bfloat16>(X, W, scale, sdt, Y, M, N, K, st);
}

} // namespace ql
