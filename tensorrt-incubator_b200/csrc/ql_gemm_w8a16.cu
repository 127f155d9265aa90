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
//
// One row tile (M <= 128) is not bound by the tensor cores but by shared-memory bandwidth: per weight one raw byte
// is written and read and two widened bytes are written and read, and every CTA also stages all of X for its part
// of K (written by TMA, read by the MMA).  With one CTA per column tile and the whole of K the X traffic is as large
// as the weights' (2 MiB against 2 MiB per SM at 128 x 11008 x 4096).  The KS > 1 instantiations give a column tile
// KS times as wide to a cluster of KS CTAs that split K between them (each stages 1/KS of X) and add the KS partial
// accumulators through distributed shared memory: CTA r of the cluster owns columns [r BN/KS, (r+1) BN/KS) of the
// tile, gathers every CTA's partial sums for them in the (by then idle) pipeline buffers, adds them in rank order,
// scales and stores.  Measured at that shape: 31 us against 36 (the main loop 44 000 cycles against 59 000, which is
// the ratio of the shared-memory bytes, 3.0 MB against 4.0 MB per SM).
#include <cuda/std/type_traits>
#include <cstdlib>

#include "ql_common.cuh"
#include "ql_tc_common.cuh"

namespace ql {
namespace {

// Warp roles: TMA(W), MMA, 4 epilogue, converters, TMA(X).  The K-split kernels run twice the converter warps: one
// row tile leaves the tensor cores nearly idle and the widening, a chain of dependent integer operations per weight,
// is what bounds the main loop, so it needs the extra warps to overlap its latencies.
template <int KS> struct W8Warps {
  static constexpr int kConv = (KS > 1) ? 16 : 8;
  static constexpr int kConvThreads = kConv * 32;
  static constexpr int kThreads = (6 + kConv + 1) * 32;
  static constexpr int kXProducer = 6 + kConv;
};
constexpr int BKE = 64; // k elements per stage: 128 bytes of X, 64 bytes of int8 W

// Three rings, so that each resource is held only as long as it is needed: the small raw int8 tiles
// sit in a deep ring (their HBM latency is the one to hide), X tiles in a 4-deep ring released by the
// MMA, and the widened tiles in a 2- or 3-deep ring between the converters and the MMA.
template <int BN, int KS> struct W8Smem {
  static constexpr int kA = BM * BK_BYTES;
  static constexpr int kConv = BN * BK_BYTES;
  static constexpr int kRaw = BN * BKE;
  static constexpr int kBudget = (KS > 1 ? 216 : 200) * 1024;
  static constexpr int NA = (KS > 1) ? 3 : (BN <= 128) ? 6 : 4;
  static constexpr int NC = (BN >= 256) ? 2 : 3;
  static constexpr int kRawFit = (kBudget - NA * kA - NC * kConv) / kRaw;
  static constexpr int NR = kRawFit > 16 ? 16 : kRawFit;
  static constexpr int kOffA = 0;
  static constexpr int kOffConv = NA * kA;
  static constexpr int kOffRaw = kOffConv + NC * kConv;
  static constexpr int kBarriers = kOffRaw + NR * kRaw; // raw_full[NR] raw_empty[NR] a_full[NA] a_empty[NA] conv_ready[NC] conv_empty[NC] tfull[2] tempty[2] drain
  static constexpr int kNumBarriers = 2 * NR + 2 * NA + 2 * NC + 5;
  static constexpr int kTmemPtr = kBarriers + kNumBarriers * 8;
  static constexpr int kAbort = kTmemPtr + 4;
  static constexpr int kScales = (kAbort + 4 + 15) & ~15; // f32 scales of the columns this CTA stores (K split only), 16-byte aligned
  static constexpr int kTotal = kScales + ((KS > 1) ? (BN / KS) * 4 : 0);
  static constexpr int kDynamic = kTotal + 1024;
  // K split: columns owned by one CTA of the cluster, and the partial sums it gathers for them (one slot per CTA of
  // the cluster, its own included: [128 rows][kOwn f32], rows padded by 16 bytes against bank conflicts)
  static constexpr int kOwn = BN / KS;
  static constexpr int kSlotRow = kOwn * 4 + 16;
  static constexpr int kSlot = BM * kSlotRow;
  static_assert(NR >= 2, "raw ring too shallow");
  static_assert(KS == 1 || (kOwn % 16 == 0 && KS * kSlot <= kBarriers && kScales % 16 == 0), "partial sums must fit the idle rings");
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

// Every CTA walks its k-blocks in the same cyclic order but starts at a different one, so that the CTAs
// which share an X tile (all of them, when M fits one row tile) do not ask L2 for the same lines at the
// same moment.  The sum over k does not depend on the order beyond f32 rounding.
__device__ __forceinline__ int rotated_kb(int kb, int num_kb, int who) {
  const int v = kb + (int)(((unsigned)who * 7u) % (unsigned)num_kb);
  return v >= num_kb ? v - num_kb : v;
}

// 16 bytes into the shared memory of CTA `rank` of the cluster, at the address `local` has in this CTA
__device__ __forceinline__ void w8_store_remote(uint32_t local, uint32_t rank, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(map_to_cta(local, rank)), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

struct Ring {
  int stage = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int n) {
    if (++stage == n) { stage = 0; phase ^= 1; }
  }
};

template <typename XT, int BN, int KS>
__global__ void __launch_bounds__(W8Warps<KS>::kThreads, 1)
gemm_w8a16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const W8Args args) {
  using L = W8Smem<BN, KS>;
  constexpr int NR = L::NR, NA = L::NA, NC = L::NC;
  constexpr int kConvWarps = W8Warps<KS>::kConv, kConvThreads = W8Warps<KS>::kConvThreads, kWarpXProducer = W8Warps<KS>::kXProducer;
  constexpr int KIND = cuda::std::is_same<XT, __half>::value ? KIND_F16 : KIND_BF16;
  // a column tile wider than one MMA's N (256) is two MMAs per k-step over the halves of the widened tile
  constexpr int NMMA = BN > 256 ? 2 : 1;
  constexpr int BNM = BN / NMMA;
  constexpr int kAccCols = (KS > 1) ? BN : 2 * BN; // the K-split CTAs compute one tile each: a single accumulator
  constexpr uint32_t kTmemCols = (kAccCols <= 32) ? 32 : (kAccCols <= 64) ? 64 : (kAccCols <= 128) ? 128 : (kAccCols <= 256) ? 256 : 512;
  static_assert(BNM % 16 == 0 && BNM <= 256 && kAccCols <= 512, "tile shape");
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
  // K split: the cluster's CTAs share one tile and take consecutive ranges of the k-blocks; otherwise every CTA
  // walks the tiles with stride gridDim.x over the whole of K
  const int krank = (KS > 1) ? (int)cluster_ctarank() : 0;
  const int tile_begin = (KS > 1) ? (int)blockIdx.x / KS : (int)blockIdx.x;
  const int tile_step = (KS > 1) ? num_tiles : (int)gridDim.x;
  const int nkb = args.num_kb / KS, kb_first = krank * nkb;

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
      for (int tile = tile_begin; tile < num_tiles && ok; tile += tile_step) {
        int mt, nt;
        w8_tile_coords(args, tile, &mt, &nt);
        for (int kb = 0; kb < nkb; kb++) {
          if (!mbar_wait(raw_empty(r.stage), r.phase ^ 1, abort_flag, args.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(raw_full(r.stage), L::kRaw);
          const int k0 = (kb_first + rotated_kb(kb, nkb, tile)) * BKE;
#pragma unroll
          for (int h = 0; h < NMMA; h++)
            tma_load_2d(smem_base + L::kOffRaw + r.stage * L::kRaw + h * BNM * BKE, &map_w, raw_full(r.stage), k0, nt * BN + h * BNM);
          r.advance(NR);
        }
      }
    }
  } else if (warp == kWarpXProducer) {
    // ------------------------------------------------------------------ TMA producer, X tiles
    if (lane == 0) {
      Ring r;
      bool ok = true;
      for (int tile = tile_begin; tile < num_tiles && ok; tile += tile_step) {
        int mt, nt;
        w8_tile_coords(args, tile, &mt, &nt);
        for (int kb = 0; kb < nkb; kb++) {
          if (!mbar_wait(a_empty(r.stage), r.phase ^ 1, abort_flag, args.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(a_full(r.stage), L::kA);
          tma_load_2d(smem_base + L::kOffA + r.stage * L::kA, &map_x, a_full(r.stage), (kb_first + rotated_kb(kb, nkb, tile)) * BKE, mt * BM);
          r.advance(NA);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc<KIND, BNM>();
      Ring ra, rc;
      int it = 0;
      bool ok = true;
      for (int tile = tile_begin; tile < num_tiles && ok; tile += tile_step, it++) {
        const int buf = it & 1;
        if (!mbar_wait(tempty_bar(buf), ((it >> 1) & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < nkb; kb++) {
          if (!mbar_wait(a_full(ra.stage), ra.phase, abort_flag, args.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          if (!mbar_wait(conv_ready(rc.stage), rc.phase, abort_flag, args.status, ST_TIMEOUT_READY)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_base + L::kOffA + ra.stage * L::kA);
#pragma unroll
          for (int h = 0; h < NMMA; h++) {
            const uint64_t bdesc = make_smem_desc(smem_base + L::kOffConv + rc.stage * L::kConv + h * BNM * BK_BYTES);
#pragma unroll
            for (int k = 0; k < BK_BYTES / 32; k++)
              tc_mma<KIND>(tmem_d + (uint32_t)(h * BNM), adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
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
    for (int tile = tile_begin; tile < num_tiles && ok; tile += tile_step) {
      for (int kb = 0; kb < nkb; kb++) {
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
  } else if constexpr (KS == 1) {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    XT *Y = static_cast<XT *>(args.Y);
    const bool vec_ok = (args.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
    int it = 0;
    bool ok = true;
    for (int tile = tile_begin; tile < num_tiles && ok; tile += tile_step, it++) {
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

  if constexpr (KS > 1) {
    // ------------------------------------------------------------------ the cluster adds its partial sums
    // Every warp but the three single-thread roles (the epilogue warps and the converters, now idle): five warps for
    // each quadrant of the accumulator's 128 lanes, sharing the 16-column chunks between them.
    const bool worker = warp >= 2 && warp != kWarpXProducer;
    const int quad = warp & 3, share = (warp - 2) >> 2;
    constexpr int kShares = (4 + kConvWarps) / 4;
    constexpr int kChunks = L::kOwn / 16;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    float *sc = reinterpret_cast<float *>(smem + L::kScales);
    int mt, nt;
    w8_tile_coords(args, tile_begin, &mt, &nt);
    const int n_own = nt * BN + krank * L::kOwn; // first of the columns this CTA adds up and stores
    if (worker) {
      for (int j = threadIdx.x - 64; j < L::kOwn; j += (4 + kConvWarps) * 32) // (the X producer's threads sit past the end)
        sc[j] = (n_own + j < args.N) ? load_scale(args.scale, args.sdt, n_own + j) : 0.f;
      mbar_wait(tfull_bar(0), 0, abort_flag, args.status, ST_TIMEOUT_TMEM_FULL);
    }
    tc_fence_after();
    __syncthreads();
    // every CTA of the cluster has finished its k range (its MMAs are complete: the issuer waited for them), so the
    // pipeline buffers are idle everywhere and may take the partial sums
    cluster_sync_all();
    if (worker) {
      // slot `krank` of every owner (this CTA included) receives this CTA's partial sums for the owner's columns
      int item = 0;
      for (int o = 0; o < KS; o++) {
        const uint32_t owner = (uint32_t)((krank + o) % KS);
#pragma unroll 1
        for (int c = 0; c < kChunks; c++, item++) {
          if (item % kShares != share) continue;
          uint32_t r[16];
          tmem_load_16(lane_base + owner * L::kOwn + c * 16, r);
          const uint32_t dst = smem_base + krank * L::kSlot + row * L::kSlotRow + c * 64;
#pragma unroll
          for (int q = 0; q < 4; q++) w8_store_remote(dst + q * 16, owner, r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        }
      }
    }
    cluster_sync_all(); // release / acquire: the partial sums written into this CTA are visible
    if (worker) {
      // one item = eight adjacent columns of one row: added in rank order (whichever CTA does the adding), scaled,
      // rounded and stored as 16 bytes; consecutive threads take consecutive items, so a row's bytes leave together
      XT *Y = static_cast<XT *>(args.Y);
      const bool vec_ok = (args.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
      constexpr int kPerRow = L::kOwn / 8;
      const int wid = (warp < kWarpXProducer ? warp - 2 : warp - 3) * 32 + lane;
      for (int item = wid; item < BM * kPerRow; item += (4 + kConvWarps) * 32) {
        const int r = item / kPerRow, g8 = item % kPerRow;
        const int m = mt * BM + r, n = n_own + g8 * 8;
        if (m >= args.M || n >= args.N) continue;
        float v[8];
#pragma unroll
        for (int src = 0; src < KS; src++) {
          const float4 *sp = reinterpret_cast<const float4 *>(smem + src * L::kSlot + r * L::kSlotRow + g8 * 32);
          const float4 lo = sp[0], hi = sp[1];
          const float p[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
          for (int j = 0; j < 8; j++) v[j] = (src == 0) ? p[j] : v[j] + p[j];
        }
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] *= sc[g8 * 8 + j];
        XT *out = Y + (size_t)m * args.N + n;
        if (vec_ok && n + 8 <= args.N) {
          __stcs(reinterpret_cast<uint4 *>(out), make_uint4(pack2<XT>(v[0], v[1]), pack2<XT>(v[2], v[3]), pack2<XT>(v[4], v[5]), pack2<XT>(v[6], v[7])));
        } else {
          for (int j = 0; j < 8 && n + j < args.N; j++) out[j] = FloatIO<XT>::from_f32(v[j]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <typename XT, int BN, int KS>
int configure_w8(int *max_clusters) {
  using L = W8Smem<BN, KS>;
  auto kern = gemm_w8a16_kernel<XT, BN, KS>;
  static bool configured[64] = {false};
  static int clusters[64] = {0};
  int dev = 0;
  QL_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(QL_ERR_UNSUPPORTED, "linear_w8a16: device index %d", dev);
  if (!configured[dev]) {
    QL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic));
    if (KS > 1) {
      // how many clusters of this shape the device can hold at once (GPC sizes decide; it is not sms / KS)
      cudaLaunchConfig_t cfg = {};
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = KS, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
      cfg.gridDim = dim3(KS * sm_count()), cfg.blockDim = dim3(W8Warps<KS>::kThreads), cfg.dynamicSmemBytes = L::kDynamic;
      cfg.attrs = attr, cfg.numAttrs = 1;
      int n = 0;
      QL_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
      clusters[dev] = n;
    }
    configured[dev] = true;
  }
  if (max_clusters) *max_clusters = clusters[dev];
  return QL_OK;
}

template <typename XT, int BN, int KS>
int launch_w8_bn(const CUtensorMap &mx, const CUtensorMap &mw, W8Args args, cudaStream_t st) {
  using L = W8Smem<BN, KS>;
  auto kern = gemm_w8a16_kernel<XT, BN, KS>;
  int rc = configure_w8<XT, BN, KS>(nullptr);
  if (rc != QL_OK) return rc;
  const int tiles = args.tiles_m * args.tiles_n;
  if (KS > 1) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = KS, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(tiles * KS), cfg.blockDim = dim3(W8Warps<KS>::kThreads), cfg.dynamicSmemBytes = L::kDynamic, cfg.stream = st;
    cfg.attrs = attr, cfg.numAttrs = 1;
    QL_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, mx, mw, args));
  } else {
    const int grid = tiles < sm_count() ? tiles : sm_count();
    kern<<<grid, W8Warps<KS>::kThreads, L::kDynamic, st>>>(mx, mw, args);
  }
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

// QL_W8_KSPLIT: 1 = never split K over a cluster, 2 = wherever the shape allows; unset = choose
int read_w8_ksplit() {
  const char *e = getenv("QL_W8_KSPLIT");
  return e ? atoi(e) : 0;
}
int g_w8_ksplit = read_w8_ksplit();
int w8_ksplit_setting() { return g_w8_ksplit; }

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
  CUtensorMap mx, mw;
  int rc;
  if ((rc = make_map(&mx, KIND, X, M, K, BM)) != QL_OK) return rc;
  // One row tile: K split over a cluster of two, where every cluster of the grid can be resident at once, the grid
  // covers most of the device and each CTA still has a pipeline's worth of k-blocks.  (A four-way split over tiles of
  // 320 or 384 columns has fewer, fatter CTAs: the device holds 33 clusters of four at this size, and what bounds the
  // kernel, the shared-memory traffic of widening per SM, grows when the weights are spread over fewer SMs.)
  const int want = w8_ksplit_setting(); // 0 = choose, 1 = never, 2 = whenever the shape allows
  if (args.tiles_m == 1 && want != 1 && args.num_kb % 2 == 0 && args.num_kb / 2 >= (want == 0 ? 8 : 1)) {
    int room = 0;
    if ((rc = configure_w8<XT, 160, 2>(&room)) != QL_OK) return rc;
    args.tiles_n = (N + 159) / 160;
    args.group_m = 1;
    if (args.tiles_n <= room && (want == 2 || args.tiles_n * 2 > sm_count() / 2)) {
      if ((rc = make_map_bytes(&mw, W, N, K, BKE, 160)) != QL_OK) return rc;
      return launch_w8_bn<XT, 160, 2>(mx, mw, args, st);
    }
  }
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
  if ((rc = make_map_bytes(&mw, W, N, K, BKE, best_bn)) != QL_OK) return rc;
  switch (best_bn) {
  case 256: return launch_w8_bn<XT, 256, 1>(mx, mw, args, st);
  case 128: return launch_w8_bn<XT, 128, 1>(mx, mw, args, st);
  case 96: return launch_w8_bn<XT, 96, 1>(mx, mw, args, st);
  case 80: return launch_w8_bn<XT, 80, 1>(mx, mw, args, st);
  case 64: return launch_w8_bn<XT, 64, 1>(mx, mw, args, st);
  case 48: return launch_w8_bn<XT, 48, 1>(mx, mw, args, st);
  default: return launch_w8_bn<XT, 32, 1>(mx, mw, args, st);
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

void w8_reload_tuning() { g_w8_ksplit = read_w8_ksplit(); }

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
