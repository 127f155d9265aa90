// Dense quantized GEMMs on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a only:
//     Y[M,N] = (A[M,K] . B[N,K]^T) * sa[m] * sb[n]
// A and B are K-major ("row-major [rows, K]"), e4m3 / int8 / bf16 / f16; accumulation is f32
// (s32 for int8) in tensor memory; the dequantization scales are applied in the epilogue and the
// result is rounded once to bf16 / f16.  This is the fused form of the reference composition
// dequantize -> matmul (tripy/nvtripy/frontend/module/linear.py:127-151) for operands that are
// both quantized, and of tensorrt.matrix_multiply (TensorRTOps.td:1986-2080) for 16-bit operands.
//
// One persistent CTA per SM, 6 warps:
//   warp 0   one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//            into a 4-stage ring of [128 x 128 B] A tiles and [BN x 128 B] B tiles
//   warp 1   allocates tensor memory; one lane issues tcgen05.mma (M=128, N=BN, K=32 bytes) from
//            shared-memory descriptors and commits to the ring's "empty" barriers and to the
//            accumulator's "full" barrier
//   warps 2-5 epilogue: tcgen05.ld of the accumulator (two buffers, so the next tile's main loop
//            overlaps), scales, conversion, 16-byte global stores
// Every wait is bounded: when a limit runs out the kernel records a code in `status`, stops
// issuing work, drains what it issued and returns.
#include <cuda.h>

#include "ql_common.cuh"

namespace ql {
namespace {

enum { KIND_F8 = 0, KIND_I8 = 1, KIND_BF16 = 2, KIND_F16 = 3 };

constexpr int BM = 128;
constexpr int BK_BYTES = 128; // one 128-byte swizzle row of K per stage
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK_BYTES;
constexpr int kGemmThreads = 192;
constexpr long long kWaitLimitCycles = 1ll << 31; // about a second

// status codes written by the kernel
enum { ST_OK = 0, ST_TIMEOUT_EMPTY = 1, ST_TIMEOUT_FULL = 2, ST_TIMEOUT_TMEM_EMPTY = 3, ST_TIMEOUT_TMEM_FULL = 4, ST_TIMEOUT_DRAIN = 5 };

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.b32 %0, 1, 0, p;\n\t}"
               : "=r"(done)
               : "r"(bar), "r"(parity)
               : "memory");
  return done != 0;
}
// Bounded wait.  Gives up after kWaitLimitCycles or as soon as another role has given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag != 0) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = code;
      atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the 128-byte
// swizzle TMA applies: groups of 8 rows are 1024 bytes apart (stride byte offset), the leading
// byte offset is unused for swizzled K-major layouts, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <int KIND, int BN>
__device__ __forceinline__ uint32_t make_instr_desc() {
  uint32_t d = 0;
  if (KIND == KIND_I8) {
    d |= 2u << 4;              // accumulate in s32
    d |= 1u << 7 | 1u << 10;   // signed 8-bit A and B
  } else {
    d |= 1u << 4;              // accumulate in f32
    if (KIND == KIND_BF16) d |= 1u << 7 | 1u << 10;
    // e4m3 and f16 are format 0 of their kinds
  }
  // both operands K-major: bits 15 and 16 stay 0
  d |= (uint32_t)(BN >> 3) << 17;
  d |= (uint32_t)(BM >> 4) << 24;
  return d;
}

template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == KIND_F8) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else if constexpr (KIND == KIND_I8) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <typename OutT> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}

struct GemmArgs {
  void *Y;
  const float *sa; // null = 1, else one value (sa_n == 1) or one per row of A
  const float *sb; // null = 1, else one value (sb_n == 1) or one per row of B
  int sa_n, sb_n;
  int M, N;
  int num_kb;      // K blocks of 128 bytes (the last may be partial: TMA fills zeros)
  int k_elems_per_block;
  int tiles_m, tiles_n;
  int group_m;     // m-tiles per scheduling group (see tile_coords)
  int *status;
};

// Tile order.  Consecutive tile indices (which run concurrently on neighbouring SMs) walk a band
// of `group_m` row tiles across all column tiles before moving to the next band, so the A rows of
// the band stay in L2 while every B tile is streamed through once per band.
__device__ __forceinline__ void tile_coords(const GemmArgs &a, int tile, int *mt, int *nt) {
  const int per_group = a.group_m * a.tiles_n;
  const int grp = tile / per_group;
  const int first_m = grp * a.group_m;
  const int gsz = min(a.group_m, a.tiles_m - first_m);
  const int local = tile - grp * per_group;
  *mt = first_m + local % gsz;
  *nt = local / gsz;
}

template <int BN> struct SmemLayout {
  static constexpr int kBStage = BN * BK_BYTES;
  static constexpr int kStage = A_STAGE_BYTES + kBStage;
  static constexpr int kTiles = STAGES * kStage;
  static constexpr int kBarriers = kTiles;            // full[S], empty[S], tmem_full[2], tmem_empty[2], drain
  static constexpr int kTmemPtr = kBarriers + (2 * STAGES + 5) * 8;
  static constexpr int kAbort = kTmemPtr + 4;
  static constexpr int kTotal = kAbort + 4;
  static constexpr int kDynamic = kTotal + 1024;      // slack to align the ring to 1024 bytes
};

template <int KIND, int BN, typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs args) {
  using L = SmemLayout<BN>;
  constexpr uint32_t kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarriers;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 4);
  volatile uint32_t *tmem_ptr_smem = reinterpret_cast<volatile uint32_t *>(smem + L::kTmemPtr);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = args.tiles_m * args.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4); // one arrival per epilogue warp
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mt, nt;
        tile_coords(args, tile, &mt, &nt);
        const int m0 = mt * BM, n0 = nt * BN;
        for (int kb = 0; kb < args.num_kb; kb++) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, args.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * L::kStage, b_dst = a_dst + A_STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), L::kStage);
          tma_load_2d(a_dst, &map_a, full_bar(stage), kb * args.k_elems_per_block, m0);
          tma_load_2d(b_dst, &map_b, full_bar(stage), kb * args.k_elems_per_block, n0);
          issued++;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // let the loads that are still in flight land before the CTA's shared memory goes away
        const long long pending = issued < STAGES ? issued : STAGES;
        for (long long i = 0; i < pending; i++) {
          stage = (stage == 0) ? STAGES - 1 : stage - 1;
          if (stage == STAGES - 1) phase ^= 1;
          const long long t0 = clock64();
          while (!mbar_try_wait(full_bar(stage), phase) && clock64() - t0 < kWaitLimitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc<KIND, BN>();
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, it++) {
        const int buf = it & 1;
        if (!mbar_wait(tempty_bar(buf), ((it >> 1) & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < args.num_kb; kb++) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, args.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * L::kStage;
          const uint64_t adesc = make_smem_desc(a_addr), bdesc = make_smem_desc(a_addr + A_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK_BYTES / 32; k++) // each MMA consumes 32 bytes of K; +2 in the address field
            tc_mma<KIND>(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(tfull_bar(buf));
      }
      // every MMA issued above must have finished before tensor memory is released
      tc_commit(drain_bar);
      const long long t0 = clock64();
      while (!mbar_try_wait(drain_bar, 0)) {
        if (clock64() - t0 > kWaitLimitCycles) { atomicCAS(args.status, 0, ST_TIMEOUT_DRAIN); break; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3; // tensor-memory lanes [32*quad, 32*quad+32) belong to this warp
    OutT *Y = static_cast<OutT *>(args.Y);
    const bool vec_ok = (args.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, it++) {
      const int buf = it & 1;
      int mt, nt;
      tile_coords(args, tile, &mt, &nt);
      const int m0 = mt * BM, n0 = nt * BN;
      if (!mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int m = m0 + quad * 32 + lane;
      float sa = 1.f;
      if (args.sa) sa = (args.sa_n == 1) ? __ldg(args.sa) : (m < args.M ? __ldg(args.sa + m) : 0.f);
      const float sb_scalar = (args.sb && args.sb_n == 1) ? __ldg(args.sb) : 1.f;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        tmem_load_32(taddr + c * 32, r);
        const int n = n0 + c * 32;
        if (m < args.M && n < args.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; j++) {
            float acc = (KIND == KIND_I8) ? (float)(int)r[j] : __uint_as_float(r[j]);
            float s = sa * sb_scalar;
            if (args.sb && args.sb_n != 1) s = sa * ((n + j < args.N) ? __ldg(args.sb + n + j) : 0.f);
            v[j] = acc * s;
          }
          OutT *row = Y + (size_t)m * args.N + n;
          if (vec_ok && n + 32 <= args.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o = make_uint4(pack2<OutT>(v[j], v[j + 1]), pack2<OutT>(v[j + 2], v[j + 3]),
                                   pack2<OutT>(v[j + 4], v[j + 5]), pack2<OutT>(v[j + 6], v[j + 7]));
              __stcs(reinterpret_cast<uint4 *>(row + j), o); // written once, never re-read here: keep it out of L2's way
            }
          } else {
            for (int j = 0; j < 32 && n + j < args.N; j++) row[j] = FloatIO<OutT>::from_f32(v[j]);
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

// ----------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn *out) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    QL_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || !p) return set_error(QL_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  *out = fn;
  return QL_OK;
}

// [rows, K] row-major matrix of `esize`-byte elements, box = [box_rows, 128 bytes], 128-byte swizzle
int make_map(CUtensorMap *map, int kind, const void *ptr, int64_t rows, int64_t K, int box_rows) {
  EncodeTiledFn enc;
  int rc = get_encode_fn(&enc);
  if (rc != QL_OK) return rc;
  const int esize = (kind == KIND_F8 || kind == KIND_I8) ? 1 : 2;
  CUtensorMapDataType dt = (kind == KIND_F8 || kind == KIND_I8) ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : (kind == KIND_BF16)                ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * esize};
  cuuint32_t box[2] = {(cuuint32_t)(BK_BYTES / esize), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(QL_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return QL_OK;
}

template <int KIND, int BN, typename OutT>
int launch_gemm_bn(const CUtensorMap &ma, const CUtensorMap &mb, GemmArgs args, cudaStream_t st) {
  using L = SmemLayout<BN>;
  auto kern = gemm_tc_kernel<KIND, BN, OutT>;
  static bool configured[64] = {false};
  int dev = 0;
  QL_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    QL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic));
    configured[dev] = true;
  }
  args.tiles_n = (args.N + BN - 1) / BN;
  const int tiles = args.tiles_m * args.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kGemmThreads, L::kDynamic, st>>>(ma, mb, args);
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

template <int KIND, typename OutT>
int launch_gemm_kind(const void *A, const void *B, GemmArgs args, int64_t K, cudaStream_t st) {
  const int sms = sm_count();
  int bn = 32;
  for (int cand : {256, 128, 64}) {
    if ((int64_t)args.tiles_m * ((args.N + cand - 1) / cand) >= sms) { bn = cand; break; }
  }
  if (args.N <= 32) bn = 32;
  CUtensorMap ma, mb;
  int rc;
  if ((rc = make_map(&ma, KIND, A, args.M, K, BM)) != QL_OK) return rc;
  if ((rc = make_map(&mb, KIND, B, args.N, K, bn)) != QL_OK) return rc;
  switch (bn) {
  case 256: return launch_gemm_bn<KIND, 256, OutT>(ma, mb, args, st);
  case 128: return launch_gemm_bn<KIND, 128, OutT>(ma, mb, args, st);
  case 64: return launch_gemm_bn<KIND, 64, OutT>(ma, mb, args, st);
  default: return launch_gemm_bn<KIND, 32, OutT>(ma, mb, args, st);
  }
}

int check_gemm(const char *op, const ql_tensor *a, const ql_tensor *b, const ql_tensor *sa, const ql_tensor *sb,
               const ql_tensor *y, int want_dtype_a, int want_dtype_b) {
  if (!a || !b || !y) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  if (a->rank != 2 || b->rank != 2 || y->rank != 2)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: operands must be 2-D ([M,K], [N,K], [M,N])", op);
  if (a->dtype != want_dtype_a || b->dtype != want_dtype_b)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: unexpected operand types %d, %d", op, a->dtype, b->dtype);
  if (!(y->dtype == QL_BF16 || y->dtype == QL_F16)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: y must be bf16 or f16", op);
  if (a->shape[1] != b->shape[1])
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: inner dimensions differ (%lld vs %lld)", op, (long long)a->shape[1], (long long)b->shape[1]);
  if (y->shape[0] != a->shape[0] || y->shape[1] != b->shape[0])
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: y must be [M,N] = [%lld,%lld]", op, (long long)a->shape[0], (long long)b->shape[0]);
  const ql_tensor *sc[2] = {sa, sb};
  const int64_t want[2] = {a->shape[0], b->shape[0]};
  for (int i = 0; i < 2; i++) {
    if (!sc[i]) continue;
    if (sc[i]->dtype != QL_F32) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: scales must be f32", op);
    int64_t n = numel(sc[i]);
    if (!(n == 1 || (sc[i]->rank == 1 && n == want[i])))
      return set_error(QL_ERR_INVALID_ARGUMENT, "%s: a scale must be a scalar or one value per row of its operand", op);
    if (!sc[i]->data) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: scale has no data pointer", op);
  }
  if (!aligned16(a->data) || !aligned16(b->data))
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: operands must be 16-byte aligned", op);
  if (a->shape[0] > INT32_MAX || b->shape[0] > INT32_MAX || a->shape[1] > INT32_MAX)
    return set_error(QL_ERR_UNSUPPORTED, "%s: dimension too large", op);
  return QL_OK;
}

template <int KIND>
int run_gemm(const char *op, const ql_tensor *a, const ql_tensor *b, const ql_tensor *sa, const ql_tensor *sb, ql_tensor *y,
             void *stream) {
  const int64_t M = a->shape[0], K = a->shape[1], N = b->shape[0];
  if (M == 0 || N == 0) return QL_OK;
  const int esize = (KIND == KIND_F8 || KIND == KIND_I8) ? 1 : 2;
  if (K == 0 || (K * esize) % 16 != 0)
    return set_error(QL_ERR_UNSUPPORTED, "%s: K * element size must be a non-zero multiple of 16 bytes (K=%lld)", op, (long long)K);
  GemmArgs args;
  args.Y = y->data;
  args.sa = sa ? static_cast<const float *>(sa->data) : nullptr;
  args.sb = sb ? static_cast<const float *>(sb->data) : nullptr;
  args.sa_n = sa ? (int)numel(sa) : 1;
  args.sb_n = sb ? (int)numel(sb) : 1;
  args.M = (int)M;
  args.N = (int)N;
  args.k_elems_per_block = BK_BYTES / esize;
  args.num_kb = (int)((K * esize + BK_BYTES - 1) / BK_BYTES);
  args.tiles_m = (int)((M + BM - 1) / BM);
  args.tiles_n = 0;
  {
    // a band of A of about 16 MiB stays L2-resident while B streams through
    const int64_t band = (16ll << 20) / ((int64_t)BM * K * esize);
    args.group_m = (int)(band < 4 ? 4 : band);
    if (args.group_m > args.tiles_m) args.group_m = args.tiles_m;
  }
  args.status = device_status_word();
  if (!args.status) return set_error(QL_ERR_CUDA, "%s: could not allocate the device status word", op);
  cudaStream_t st = (cudaStream_t)stream;
  if (y->dtype == QL_BF16) return launch_gemm_kind<KIND, __nv_bfloat16>(a->data, b->data, args, K, st);
  return launch_gemm_kind<KIND, __half>(a->data, b->data, args, K, st);
}

} // namespace

// Y[M,N] = (X[M,K] . W[N,K]^T) * sb[n]; X, W and Y of the same 16-bit type (QL_BF16 / QL_F16).
int gemm16_device(int dtype, const void *X, const void *W, const float *sb, int sb_n, void *Y, int M, int N, int K,
                  cudaStream_t st) {
  ql_tensor x{const_cast<void *>(X), dtype, 2, {M, K}}, w{const_cast<void *>(W), dtype, 2, {N, K}}, y{Y, dtype, 2, {M, N}};
  ql_tensor s{const_cast<float *>(sb), QL_F32, 1, {sb_n}};
  if (dtype == QL_BF16) return run_gemm<KIND_BF16>("gemm_16", &x, &w, nullptr, sb ? &s : nullptr, &y, st);
  return run_gemm<KIND_F16>("gemm_16", &x, &w, nullptr, sb ? &s : nullptr, &y, st);
}

} // namespace ql

using namespace ql;

extern "C" {

int ql_gemm_fp8(const ql_tensor *xq, const ql_tensor *wq, const ql_tensor *sx, const ql_tensor *sw, ql_tensor *y, void *stream) {
  int rc = check_gemm("gemm_fp8", xq, wq, sx, sw, y, QL_F8E4M3, QL_F8E4M3);
  if (rc != QL_OK) return rc;
  return run_gemm<KIND_F8>("gemm_fp8", xq, wq, sx, sw, y, stream);
}

int ql_gemm_i8(const ql_tensor *xq, const ql_tensor *wq, const ql_tensor *sx, const ql_tensor *sw, ql_tensor *y, void *stream) {
  int rc = check_gemm("gemm_i8", xq, wq, sx, sw, y, QL_I8, QL_I8);
  if (rc != QL_OK) return rc;
  return run_gemm<KIND_I8>("gemm_i8", xq, wq, sx, sw, y, stream);
}

int ql_gemm_16(const ql_tensor *x, const ql_tensor *w, const ql_tensor *sw, ql_tensor *y, void *stream) {
  if (!x || !w) return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_16: null tensor");
  int rc = check_gemm("gemm_16", x, w, nullptr, sw, y, x->dtype, x->dtype);
  if (rc != QL_OK) return rc;
  if (x->dtype == QL_BF16) return run_gemm<KIND_BF16>("gemm_16", x, w, nullptr, sw, y, stream);
  if (x->dtype == QL_F16) return run_gemm<KIND_F16>("gemm_16", x, w, nullptr, sw, y, stream);
  return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_16: operands must be bf16 or f16");
}

// Last status code a GEMM kernel recorded on the current device (0 = none); synchronises the device.
int ql_gemm_status(int32_t *code) {
  int *w = device_status_word();
  if (!w) return set_error(QL_ERR_CUDA, "gemm_status: no status word");
  int v = 0;
  QL_CUDA_TRY(cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost));
  if (code) *code = v;
  if (v != 0) {
    cudaMemset(w, 0, sizeof(int));
    return set_error(QL_ERR_DEVICE_TIMEOUT, "a GEMM kernel gave up waiting (code %d)", v);
  }
  return QL_OK;
}
}
