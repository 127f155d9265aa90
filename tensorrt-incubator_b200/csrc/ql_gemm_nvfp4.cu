// Block-scaled NVFP4 GEMM on the 5th-generation tensor cores (sm_100a only):
//     Y[M,N] = (dq(A)[M,K] . dq(B)[N,K]^T),   dq(X)[r,k] = e2m1(X[r,k]) * e4m3(SX[r, k/16]) * gX
// A and B are what tensorrt.dynamic_quantize produces (TensorRTOps.td:3279-3358 of the reference: e2m1 data, two per
// byte with the first element in the low nibble, e4m3 scales for blocks of 16 along K, one f32 "double quantization"
// scale per tensor); the product of the two dequantized operands is what the reference's documented use --
// dynamic_quantize -> dequantize -> dequantize -> matrix_multiply -- computes, with the two dequantize steps done by
// the tensor core itself: `tcgen05.mma.kind::mxf4nvf4.block_scale` multiplies every 16-element partial dot product
// by the two block scales, which it reads from tensor memory.  The tensor scales gA * gB are applied in the epilogue.
//
// One persistent CTA per SM, 6 warps, 128 x 224 output tiles: the widest tile whose two accumulators (448 columns)
// still leave tensor memory room for one k step of scales (48), and wide tiles matter because per MMA the scales of
// 128 + N rows have to be copied into tensor memory, which is what bounds this kernel (128 x 128 tiles: 1.81 ms on
// 8192 x 28672 x 8192; these: 1.39 ms).
//   warp 0   one lane issues, per k step of 256 elements, the TMA loads of the [128 x 128 B] A and [224 x 128 B] B tiles
//            (128-byte swizzle) and two bulk copies of block scales (2 KiB for A, 4 KiB for B), all completing on the
//            stage's barrier
//   warp 1   allocates tensor memory; per stage one lane copies the scales from shared to tensor memory
//            (tcgen05.cp 32x128b.warpx4) and issues four MMAs (M=128, N=224, K=64)
//   warps 2-5 epilogue on a double-buffered accumulator
// The tensor core wants the scales of 128 rows x 4 blocks as one 512-byte chunk, laid out as 32 rows of 16 bytes:
// byte 16 * (r % 32) + 4 * (r / 32) + b holds the scale of row r, block b; in tensor memory that is 4 columns, row r in
// column r / 32, and an operand of more than 128 rows continues in the next 4 columns.  The operator's scale tensors are
// row-major [rows, K/16], so a small kernel rewrites both into that order, tile by tile (scratch of the call), before
// the GEMM.
// Every wait is bounded, as in the other tensor-core kernels.
#include <cuda.h>
#include <cstdlib>

#include "ql_common.cuh"
#include "ql_tc_common.cuh"

namespace ql {
namespace {

constexpr int FBN = 224;                      // tile width: two accumulators of 224 columns and the scales fill tensor memory
constexpr int FSTAGES = 4;
constexpr int kF4Threads = 192;
constexpr int F_TILE_BYTES = BM * BK_BYTES;   // 16 KiB: 128 rows x 256 e2m1 (the A tile)
constexpr int F_TILE_B_BYTES = FBN * BK_BYTES; // 28 KiB: the B tile
constexpr int F_SF_BYTES = 2048;              // scales of 128 rows x 16 blocks
constexpr int F_SFB_GROUPS = (FBN + 127) / 128; // groups of 128 rows of B, the last one padded
constexpr int F_STAGE_BYTES = F_TILE_BYTES + F_TILE_B_BYTES + (1 + F_SFB_GROUPS) * F_SF_BYTES;
static_assert(F_STAGE_BYTES % 1024 == 0 && FBN % 32 == 0 && 2 * FBN + 16 + 16 * F_SFB_GROUPS <= 512, "tile shape");

struct F4Smem {
  static constexpr int kTiles = FSTAGES * F_STAGE_BYTES;
  static constexpr int kBarriers = kTiles; // full[S], empty[S], tfull[2], tempty[2], drain
  static constexpr int kTmemPtr = kBarriers + (2 * FSTAGES + 5) * 8;
  static constexpr int kAbort = kTmemPtr + 4;
  static constexpr int kTotal = kAbort + 4;
  static constexpr int kDynamic = kTotal + 1024;
};

struct F4Args {
  void *Y;
  const uint8_t *sfa, *sfb; // scales in chunk order: [tile][k step][128-row group of the tile][2048 bytes]
  const float *ga, *gb;     // tensor scales (device scalars; null = 1)
  int y_dtype;
  int M, N;
  int num_ks;               // k steps of 256 elements
  int tiles_m, tiles_n;
  int *status;
};

// Row-major scales [rows, kb] (one byte per block of 16) -> chunk order, zero-padded to whole chunks.  A tile of
// `tile_rows` rows is cut into `groups` groups of 128 rows (the last one padded); per tile and k step the groups'
// 2048-byte chunks follow one another.
__global__ void __launch_bounds__(256) sf_reorder_kernel(const uint8_t *__restrict__ in, uint32_t *__restrict__ out, int rows, int kb, int num_ks,
                                                         int tile_rows, int groups, int64_t n_words) {
  const int64_t w = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (w >= n_words) return;
  const int64_t per_tile = (int64_t)num_ks * groups * 512;
  const int tile = (int)(w / per_tile);
  const int rem = (int)(w % per_tile);
  const int s = rem / (groups * 512), v2 = rem % (groups * 512);
  const int sub = v2 / 512, v = v2 % 512;
  const int j = v / 128, cw = v % 128;
  const int local = sub * 128 + (cw % 4) * 32 + cw / 4;
  const int row = tile * tile_rows + local;
  const int b0 = (s * 4 + j) * 4;
  uint32_t word = 0;
  if (local < tile_rows && row < rows) {
#pragma unroll
    for (int i = 0; i < 4; i++)
      if (b0 + i < kb) word |= (uint32_t)in[(int64_t)row * kb + b0 + i] << (8 * i);
  }
  out[w] = word;
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// 32 rows x 16 bytes, rows 16 bytes apart (8-row core matrices of 128 bytes, 128 bytes apart), no swizzle
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;          // leading byte offset: unused (one core matrix along K)
  d |= (uint64_t)(128 >> 4) << 32; // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;          // descriptor version
  return d;
}
__device__ __forceinline__ void tc_copy_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void tc_mma_f4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                          uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
               : "memory");
}
// Instruction descriptor of the block-scaled kinds: e2m1 operands (format 1), e4m3 scales (0), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24, scale-factor byte ids 0, dense K = 64.
__device__ __forceinline__ uint32_t make_f4_idesc() {
  uint32_t d = 0;
  d |= 1u << 7;
  d |= 1u << 10;
  d |= (uint32_t)(FBN >> 3) << 17;
  d |= (uint32_t)(BM >> 4) << 24;
  return d;
}

// 32 columns of one accumulator row, times the tensor scales, rounded to y's type and stored
__device__ __forceinline__ void f4_store_chunk(const F4Args &args, const uint32_t (&r)[32], int m, int n, float g) {
  const size_t o = (size_t)m * (size_t)args.N + n;
  const int cols = min(32, args.N - n);
  if (args.y_dtype == QL_F32) {
    float *y = static_cast<float *>(args.Y) + o;
    for (int j = 0; j < cols; j++) y[j] = __uint_as_float(r[j]) * g;
  } else if (args.y_dtype == QL_F16) {
    __half *y = static_cast<__half *>(args.Y) + o;
    if (cols == 32 && (args.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(args.Y) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        __stcs(reinterpret_cast<uint4 *>(y + j), make_uint4(pack2<__half>(__uint_as_float(r[j]) * g, __uint_as_float(r[j + 1]) * g),
                                                            pack2<__half>(__uint_as_float(r[j + 2]) * g, __uint_as_float(r[j + 3]) * g),
                                                            pack2<__half>(__uint_as_float(r[j + 4]) * g, __uint_as_float(r[j + 5]) * g),
                                                            pack2<__half>(__uint_as_float(r[j + 6]) * g, __uint_as_float(r[j + 7]) * g)));
    } else {
      for (int j = 0; j < cols; j++) y[j] = __float2half_rn(__uint_as_float(r[j]) * g);
    }
  } else {
    __nv_bfloat16 *y = static_cast<__nv_bfloat16 *>(args.Y) + o;
    if (cols == 32 && (args.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(args.Y) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        __stcs(reinterpret_cast<uint4 *>(y + j),
               make_uint4(pack2<__nv_bfloat16>(__uint_as_float(r[j]) * g, __uint_as_float(r[j + 1]) * g),
                          pack2<__nv_bfloat16>(__uint_as_float(r[j + 2]) * g, __uint_as_float(r[j + 3]) * g),
                          pack2<__nv_bfloat16>(__uint_as_float(r[j + 4]) * g, __uint_as_float(r[j + 5]) * g),
                          pack2<__nv_bfloat16>(__uint_as_float(r[j + 6]) * g, __uint_as_float(r[j + 7]) * g)));
    } else {
      for (int j = 0; j < cols; j++) y[j] = __float2bfloat16_rn(__uint_as_float(r[j]) * g);
    }
  }
}

__global__ void __launch_bounds__(kF4Threads, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const F4Args args) {
  using L = F4Smem;
  constexpr uint32_t kTmemCols = 512;           // 2 x 224 accumulator columns, then one k step's scales: 16 columns of A's, 32 of B's
  constexpr uint32_t kSfCol0 = 2 * FBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarriers;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (FSTAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * FSTAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * FSTAGES + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * FSTAGES + 4);
  volatile uint32_t *tmem_ptr_smem = reinterpret_cast<volatile uint32_t *>(smem + L::kTmemPtr);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = args.tiles_m * args.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < FSTAGES; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
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
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mt = tile % args.tiles_m, nt = tile / args.tiles_m; // row tiles of one column tile run side by side: B stays in L2
        const uint8_t *sfa = args.sfa + (size_t)mt * args.num_ks * F_SF_BYTES;
        const uint8_t *sfb = args.sfb + (size_t)nt * args.num_ks * (F_SFB_GROUPS * F_SF_BYTES);
        for (int ks = 0; ks < args.num_ks; ks++) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, args.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * F_STAGE_BYTES, b_dst = a_dst + F_TILE_BYTES, s_dst = b_dst + F_TILE_B_BYTES;
          mbar_expect_tx(full_bar(stage), F_STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, full_bar(stage), ks * BK_BYTES, mt * BM);   // coordinates in bytes of packed e2m1
          tma_load_2d(b_dst, &map_b, full_bar(stage), ks * BK_BYTES, nt * FBN);
          bulk_load(s_dst, sfa + (size_t)ks * F_SF_BYTES, F_SF_BYTES, full_bar(stage));
          bulk_load(s_dst + F_SF_BYTES, sfb + (size_t)ks * (F_SFB_GROUPS * F_SF_BYTES), F_SFB_GROUPS * F_SF_BYTES, full_bar(stage));
          issued++;
          if (++stage == FSTAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const long long pending = issued < FSTAGES ? issued : FSTAGES;
        for (long long i = 0; i < pending; i++) {
          stage = (stage == 0) ? FSTAGES - 1 : stage - 1;
          if (stage == FSTAGES - 1) phase ^= 1;
          const long long t0 = clock64();
          while (!mbar_try_wait(full_bar(stage), phase) && clock64() - t0 < kWaitLimitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ scale copies + MMA issue
    if (lane == 0) {
      const uint32_t idesc = make_f4_idesc();
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, it++) {
        const int buf = it & 1;
        if (!mbar_wait(tempty_bar(buf), ((it >> 1) & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * FBN);
        for (int ks = 0; ks < args.num_ks; ks++) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, args.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * F_STAGE_BYTES, s_addr = a_addr + F_TILE_BYTES + F_TILE_B_BYTES;
          // One slot of scale columns, rewritten every k step: the copies and the MMAs of one thread run in issue order,
          // so a copy cannot overtake the MMAs that still read the slot.  A's scales: 4 columns per MMA (rows r of the
          // tile in column r / 32); B's: 4 columns per group of 128 rows, the groups side by side.
          const uint32_t t_sfa = tmem_base + kSfCol0, t_sfb = t_sfa + 16;
#pragma unroll
          for (int j = 0; j < 4; j++) { // one 512-byte chunk = the scales of 128 rows for one MMA (4 blocks of 16)
            tc_copy_sf(t_sfa + 4 * j, make_sf_desc(s_addr + 512 * j));
#pragma unroll
            for (int gI = 0; gI < F_SFB_GROUPS; gI++)
              tc_copy_sf(t_sfb + 4 * (F_SFB_GROUPS * j + gI), make_sf_desc(s_addr + F_SF_BYTES * (1 + gI) + 512 * j));
          }
          const uint64_t adesc = make_smem_desc(a_addr), bdesc = make_smem_desc(a_addr + F_TILE_BYTES);
#pragma unroll
          for (int j = 0; j < 4; j++) // each MMA consumes 64 elements = 32 bytes of K; +2 in the address field
            tc_mma_f4(tmem_d, adesc + 2 * j, bdesc + 2 * j, idesc, t_sfa + 4 * j, t_sfb + 4 * F_SFB_GROUPS * j, (ks | j) != 0 ? 1u : 0u);
          tc_commit(empty_bar(stage));
          if (++stage == FSTAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(tfull_bar(buf));
      }
      tc_commit(drain_bar);
      const long long t0 = clock64();
      while (!mbar_try_wait(drain_bar, 0)) {
        if (clock64() - t0 > kWaitLimitCycles) { atomicCAS(args.status, 0, ST_TIMEOUT_DRAIN); break; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    const float g = (args.ga ? __ldg(args.ga) : 1.f) * (args.gb ? __ldg(args.gb) : 1.f);
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, it++) {
      const int buf = it & 1;
      const int mt = tile % args.tiles_m, nt = tile / args.tiles_m;
      if (!mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int m = mt * BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * FBN);
#pragma unroll 1
      for (int c = 0; c < FBN / 32; c++) {
        uint32_t r[32];
        tmem_load_32(taddr + c * 32, r);
        const int n = nt * FBN + c * 32;
        if (m < args.M && n < args.N) f4_store_chunk(args, r, m, n, g);
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

// ------------------------------------------------------------------------------------------------------------------
// The same product on CTA pairs: 256 x 224 tiles, `tcgen05.mma.cta_group::2` (M = 256) issued by the pair's leader.
// Each CTA loads its own 128 rows of A, its own half of the B tile (112 rows), the scales of its A rows and the scales of
// the whole B tile (each CTA's tensor core multiplies its rows by all 224 columns, so it needs them all), every copy a
// TMA tile load that completes on the leader's barrier.  Per MMA a CTA then reads 128 + 112 rows of operands from its
// shared memory instead of 128 + 224: 64 bytes per cycle at the fp4 rate, where the one-CTA tile needs 98.
// Same bits as the one-CTA kernel (tests), but not faster (1.44 against 1.38 ms on 8192 x 28672 x 8192), and it is not
// selected unless asked for: timing runs with the MMAs or the scale copies left out showed that both kernels are bound by
// the scale copies (the copies alone take as long as the whole kernel, the MMAs alone two thirds of it; 12 copies of
// 512 bytes per k step at about 120 cycles each, one 32-bit cell per cycle and lane quadrant), and a pair issues as many
// copies per k step as a single CTA does.
constexpr int PSTAGES = 5;
constexpr int P_B_ROWS = FBN / 2;                                   // rows of the B tile one CTA holds
constexpr int P_TILE_B_BYTES = P_B_ROWS * BK_BYTES;                 // 14 KiB
constexpr int P_STAGE_BYTES = F_TILE_BYTES + P_TILE_B_BYTES + (1 + F_SFB_GROUPS) * F_SF_BYTES; // 36 KiB
static_assert(P_STAGE_BYTES % 1024 == 0 && P_B_ROWS % 8 == 0, "pair stage layout");

struct P4Smem {
  static constexpr int kTiles = PSTAGES * P_STAGE_BYTES;
  static constexpr int kBarriers = kTiles; // full[S], empty[S], tfull[2], tempty[2], drain
  static constexpr int kTmemPtr = kBarriers + (2 * PSTAGES + 5) * 8;
  static constexpr int kAbort = kTmemPtr + 4;
  static constexpr int kTotal = kAbort + 4;
  static constexpr int kDynamic = kTotal + 1024;
};

__device__ __forceinline__ void f4_copy_sf_pair(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void f4_mma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                            uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
               : "memory");
}

// args.tiles_m counts 256-row tiles here.  map_sfa / map_sfb see the re-ordered scales as rows of 256 bytes.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kF4Threads, 1)
gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb, const F4Args args) {
  using L = P4Smem;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kSfCol0 = 2 * FBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarriers;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (PSTAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * PSTAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * PSTAGES + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * PSTAGES + 4);
  volatile uint32_t *tmem_ptr_smem = reinterpret_cast<volatile uint32_t *>(smem + L::kTmemPtr);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_tiles = args.tiles_m * args.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8); // four epilogue warps in each CTA of the pair
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_ptr_smem)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all(); // the partner's barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const int mt = tile % args.tiles_m, nt = tile / args.tiles_m;
        const int m0 = mt * 256 + (int)rank * BM, n0 = nt * FBN + (int)rank * P_B_ROWS;
        // rows of 256 bytes in the re-ordered scales: A's by 128-row tile, B's by 224-column tile
        const int sfa_row0 = (2 * mt + (int)rank) * args.num_ks * (F_SF_BYTES / 256);
        const int sfb_row0 = nt * args.num_ks * (F_SFB_GROUPS * F_SF_BYTES / 256);
        for (int ks = 0; ks < args.num_ks; ks++) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, args.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * P_STAGE_BYTES, b_dst = a_dst + F_TILE_BYTES, s_dst = b_dst + P_TILE_B_BYTES;
          const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * P_STAGE_BYTES); // both CTAs' bytes land on the leader's barrier
          tma_load_2d_pair(a_dst, &map_a, leader_full, ks * BK_BYTES, m0);
          tma_load_2d_pair(b_dst, &map_b, leader_full, ks * BK_BYTES, n0);
          tma_load_2d_pair(s_dst, &map_sfa, leader_full, 0, sfa_row0 + ks * (F_SF_BYTES / 256));
          tma_load_2d_pair(s_dst + F_SF_BYTES, &map_sfb, leader_full, 0, sfb_row0 + ks * (F_SFB_GROUPS * F_SF_BYTES / 256));
          issued++;
          if (++stage == PSTAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        signal_partner_abort(smem_u32((const void *)abort_flag), rank);
        if (rank == 0) { // both CTAs' loads complete on the leader's barriers: let the ones in flight land
          const long long pending = issued < PSTAGES ? issued : PSTAGES;
          for (long long i = 0; i < pending; i++) {
            stage = (stage == 0) ? PSTAGES - 1 : stage - 1;
            if (stage == PSTAGES - 1) phase ^= 1;
            const long long t0 = clock64();
            while (!mbar_try_wait(full_bar(stage), phase) && clock64() - t0 < kWaitLimitCycles) {}
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ scale copies + MMA issue (leader only)
    if (lane == 0 && rank == 0) {
      uint32_t idesc = make_f4_idesc();
      idesc &= ~(0x1Fu << 24);
      idesc |= (uint32_t)(256 >> 4) << 24; // M = 256 over the pair
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, it++) {
        const int buf = it & 1;
        if (!mbar_wait(tempty_bar(buf), ((it >> 1) & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * FBN);
        for (int ks = 0; ks < args.num_ks; ks++) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, args.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * P_STAGE_BYTES, s_addr = a_addr + F_TILE_BYTES + P_TILE_B_BYTES;
          const uint32_t t_sfa = tmem_base + kSfCol0, t_sfb = t_sfa + 16;
#pragma unroll
          for (int j = 0; j < 4; j++) { // in both CTAs: from the CTA's own shared memory into its own tensor memory
            f4_copy_sf_pair(t_sfa + 4 * j, make_sf_desc(s_addr + 512 * j));
#pragma unroll
            for (int gI = 0; gI < F_SFB_GROUPS; gI++)
              f4_copy_sf_pair(t_sfb + 4 * (F_SFB_GROUPS * j + gI), make_sf_desc(s_addr + F_SF_BYTES * (1 + gI) + 512 * j));
          }
          const uint64_t adesc = make_smem_desc(a_addr), bdesc = make_smem_desc(a_addr + F_TILE_BYTES);
#pragma unroll
          for (int j = 0; j < 4; j++)
            f4_mma_pair(tmem_d, adesc + 2 * j, bdesc + 2 * j, idesc, t_sfa + 4 * j, t_sfb + 4 * F_SFB_GROUPS * j, (ks | j) != 0 ? 1u : 0u);
          tc_commit_pair(map_to_cta(empty_bar(stage), 0));
          tc_commit_pair(map_to_cta(empty_bar(stage), 1));
          if (++stage == PSTAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          tc_commit_pair(map_to_cta(tfull_bar(buf), 0));
          tc_commit_pair(map_to_cta(tfull_bar(buf), 1));
        }
      }
      if (!ok) signal_partner_abort(smem_u32((const void *)abort_flag), rank);
      tc_commit_pair(map_to_cta(drain_bar, 0));
      const long long t0 = clock64();
      while (!mbar_try_wait(drain_bar, 0)) {
        if (clock64() - t0 > kWaitLimitCycles) { atomicCAS(args.status, 0, ST_TIMEOUT_DRAIN); break; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    const float g = (args.ga ? __ldg(args.ga) : 1.f) * (args.gb ? __ldg(args.gb) : 1.f);
    int it = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, it++) {
      const int buf = it & 1;
      const int mt = tile % args.tiles_m, nt = tile / args.tiles_m;
      if (!mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int m = mt * 256 + (int)rank * BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * FBN);
#pragma unroll 1
      for (int c = 0; c < FBN / 32; c++) {
        uint32_t r[32];
        tmem_load_32(taddr + c * 32, r);
        const int n = nt * FBN + c * 32;
        if (m < args.M && n < args.N) f4_store_chunk(args, r, m, n, g);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0)); // the leader owns the accumulator hand-over
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all(); // neither CTA may leave while the pair's MMAs or barriers can still touch it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

int check_f4_operand(const char *op, const char *name, const ql_tensor *d, const ql_tensor *s, const ql_tensor *g) {
  if (!d || !s) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: %s is null", op, name);
  if (d->dtype != QL_F4E2M1 || s->dtype != QL_F8E4M3) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: %s: data must be f4E2M1FN and scales f8E4M3FN", op, name);
  if (d->rank != 2 || s->rank != 2) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: %s: data and scales must be 2-D", op, name);
  if (d->shape[1] % 16 != 0 || s->shape[0] != d->shape[0] || s->shape[1] != d->shape[1] / 16)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: %s: scales must hold one entry per block of 16 along the last dimension", op, name);
  if (g && (g->dtype != QL_F32 || numel(g) != 1 || !g->data))
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: %s: the double-quantization scale must be one f32 value", op, name);
  if (numel(d) > 0 && (!d->data || !s->data)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: %s has no data pointer", op, name);
  return QL_OK;
}

// QL_NVFP4_KERNEL = pair: use the CTA-pair kernel wherever it can run (read once, again by ql_reload_tuning).  Unset, or
// anything else: the one-CTA kernel, which is the faster of the two (see the pair kernel's comment).
int read_f4_choice() {
  const char *e = getenv("QL_NVFP4_KERNEL");
  return !e ? 0 : (e[0] == 'o' ? 1 : (e[0] == 'p' ? 2 : 0));
}
int g_f4_choice = read_f4_choice();

// CTA pairs of the pair kernel the device holds at once (0 = cannot run it)
int f4_resident_pairs() {
  static int cached[64] = {0};
  static bool known[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!known[dev]) {
    int n = 0;
    if (cudaFuncSetAttribute(gemm_nvfp4_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P4Smem::kDynamic) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * sm_count(), 1, 1);
      cfg.blockDim = dim3(kF4Threads, 1, 1);
      cfg.dynamicSmemBytes = P4Smem::kDynamic;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_nvfp4_pair_kernel, &cfg) != cudaSuccess) n = 0;
    }
    cudaGetLastError();
    cached[dev] = n;
    known[dev] = true;
  }
  return cached[dev];
}

} // namespace

void f4_reload_tuning() { g_f4_choice = read_f4_choice(); }

} // namespace ql

using namespace ql;

extern "C" int ql_gemm_nvfp4(const ql_tensor *a, const ql_tensor *a_scales, const ql_tensor *a_global, const ql_tensor *b,
                             const ql_tensor *b_scales, const ql_tensor *b_global, ql_tensor *y, void *stream) {
  const char *op = "gemm_nvfp4";
  int rc;
  if ((rc = check_f4_operand(op, "a", a, a_scales, a_global)) != QL_OK) return rc;
  if ((rc = check_f4_operand(op, "b", b, b_scales, b_global)) != QL_OK) return rc;
  if (!y || y->rank != 2 || !is_float_dtype(y->dtype)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: y must be a 2-D f32, f16 or bf16 tensor", op);
  const int64_t M = a->shape[0], K = a->shape[1], N = b->shape[0];
  if (b->shape[1] != K) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: inner dimensions differ (%lld vs %lld)", op, (long long)K, (long long)b->shape[1]);
  if (y->shape[0] != M || y->shape[1] != N) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: y must be [M,N] = [%lld,%lld]", op, (long long)M, (long long)N);
  if (M == 0 || N == 0) return QL_OK;
  if (!y->data) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: y has no data pointer", op);
  if (K == 0 || K % 32 != 0 || !aligned16(a->data) || !aligned16(b->data))
    return set_error(QL_ERR_UNSUPPORTED, "%s: needs K (%lld) to be a non-zero multiple of 32 and 16-byte aligned operands", op, (long long)K);
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return set_error(QL_ERR_UNSUPPORTED, "%s: dimension too large", op);
  cudaStream_t st = (cudaStream_t)stream;

  F4Args args;
  args.Y = y->data;
  args.ga = a_global ? static_cast<const float *>(a_global->data) : nullptr;
  args.gb = b_global ? static_cast<const float *>(b_global->data) : nullptr;
  args.y_dtype = y->dtype;
  args.M = (int)M;
  args.N = (int)N;
  args.num_ks = (int)((K + 255) / 256);
  args.tiles_m = (int)((M + BM - 1) / BM);
  args.tiles_n = (int)((N + FBN - 1) / FBN);
  args.status = device_status_word();
  if (!args.status) return set_error(QL_ERR_CUDA, "%s: could not allocate the device status word", op);

  // both operands' block scales in the order the tensor core reads them, in scratch of this call
  const size_t sfa_bytes = (size_t)args.tiles_m * args.num_ks * F_SF_BYTES, sfb_bytes = (size_t)args.tiles_n * args.num_ks * F_SFB_GROUPS * F_SF_BYTES;
  uint8_t *scratch = nullptr;
  keep_scratch_pool_warm();
  QL_CUDA_TRY(cudaMallocAsync(&scratch, sfa_bytes + sfb_bytes, st));
  args.sfa = scratch;
  args.sfb = scratch + sfa_bytes;
  const int64_t wa = (int64_t)(sfa_bytes / 4), wb = (int64_t)(sfb_bytes / 4);
  sf_reorder_kernel<<<(unsigned)((wa + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t *>(a_scales->data), reinterpret_cast<uint32_t *>(scratch), (int)M,
                                                                  (int)(K / 16), args.num_ks, BM, 1, wa);
  sf_reorder_kernel<<<(unsigned)((wb + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t *>(b_scales->data),
                                                                  reinterpret_cast<uint32_t *>(scratch + sfa_bytes), (int)N, (int)(K / 16), args.num_ks, FBN, F_SFB_GROUPS, wb);
  count_launches(2);
  rc = QL_OK;
  CUtensorMap ma, mb;
  const int tiles_m256 = (int)((M + 255) / 256);
  const int pairs = g_f4_choice == 2 ? f4_resident_pairs() : 0;
  if (pairs > 0) {
    // CTA pairs on 256 x 224 tiles; the scales travel as TMA tiles too (rows of 256 bytes of the re-ordered scratch)
    CUtensorMap msa, msb;
    args.tiles_m = tiles_m256;
    if ((rc = make_map(&ma, KIND_F8, a->data, M, K / 2, BM)) == QL_OK && (rc = make_map(&mb, KIND_F8, b->data, N, K / 2, P_B_ROWS)) == QL_OK &&
        (rc = make_map_bytes(&msa, args.sfa, (int64_t)(sfa_bytes / 256), 256, 256, F_SF_BYTES / 256)) == QL_OK &&
        (rc = make_map_bytes(&msb, args.sfb, (int64_t)(sfb_bytes / 256), 256, 256, F_SFB_GROUPS * F_SF_BYTES / 256)) == QL_OK) {
      const int tiles = args.tiles_m * args.tiles_n;
      const int clusters = tiles < pairs ? tiles : pairs;
      gemm_nvfp4_pair_kernel<<<2 * clusters, kF4Threads, P4Smem::kDynamic, st>>>(ma, mb, msa, msb, args);
      count_launches(1);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) rc = cuda_error(e, "gemm_nvfp4_pair_kernel");
    }
  } else if ((rc = make_map(&ma, KIND_F8, a->data, M, K / 2, BM)) == QL_OK && (rc = make_map(&mb, KIND_F8, b->data, N, K / 2, FBN)) == QL_OK) {
    // packed e2m1: a row is K / 2 bytes; the maps see bytes, like the e4m3 maps
    static bool configured[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess && dev >= 0 && dev < 64 && !configured[dev]) {
      e = cudaFuncSetAttribute(gemm_nvfp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F4Smem::kDynamic);
      configured[dev] = e == cudaSuccess;
    }
    if (e != cudaSuccess) rc = cuda_error(e, "cudaFuncSetAttribute");
    else {
      const int tiles = args.tiles_m * args.tiles_n;
      const int grid = tiles < sm_count() ? tiles : sm_count();
      gemm_nvfp4_kernel<<<grid, kF4Threads, F4Smem::kDynamic, st>>>(ma, mb, args);
      count_launches(1);
      e = cudaGetLastError();
      if (e != cudaSuccess) rc = cuda_error(e, "gemm_nvfp4_kernel");
    }
  }
  cudaError_t fe = cudaFreeAsync(scratch, st);
  if (rc == QL_OK && fe != cudaSuccess) return cuda_error(fe, "cudaFreeAsync");
  return rc;
}
