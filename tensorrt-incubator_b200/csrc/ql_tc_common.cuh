// PTX wrappers and host helpers shared by the tcgen05 kernels (sm_100a): mbarrier, TMA tile loads,
// tcgen05 fences / commit / MMA issue / tensor-memory loads, shared-memory matrix descriptors and
// tensor-map construction.
#pragma once

#include <cuda.h>

#include "ql_common.cuh"

namespace ql {
namespace {

enum { KIND_F8 = 0, KIND_I8 = 1, KIND_BF16 = 2, KIND_F16 = 3 };

constexpr int BM = 128;       // rows of A per CTA tile = M of one tcgen05.mma
constexpr int BK_BYTES = 128; // one 128-byte swizzle row of K per stage
constexpr long long kWaitLimitCycles = 1ll << 31; // about a second

// status codes the kernels record when a bounded wait runs out
enum { ST_OK = 0, ST_TIMEOUT_EMPTY = 1, ST_TIMEOUT_FULL = 2, ST_TIMEOUT_TMEM_EMPTY = 3, ST_TIMEOUT_TMEM_FULL = 4, ST_TIMEOUT_DRAIN = 5, ST_TIMEOUT_READY = 6 };

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
// try_wait with a suspend-time hint: the thread may sleep in hardware for up to `ns` nanoseconds and is
// woken as soon as the phase completes, instead of re-issuing the probe in a tight loop.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
               "selp.b32 %0, 1, 0, p;\n\t}"
               : "=r"(done)
               : "r"(bar), "r"(parity), "r"(ns)
               : "memory");
  return done != 0;
}
// Bounded wait.  Gives up after kWaitLimitCycles or as soon as another role has given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait_hint(bar, parity, 20000u)) {
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

// Bulk tensor store of a [32 rows x 128 bytes] box from shared memory; completion is tracked per issuing thread in
// bulk async-groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until at most N of this thread's bulk groups still have to read their shared-memory source
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

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

__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Writes by ordinary stores that the tensor core (async proxy) will read need this fence first.
// ---- thread-block clusters and CTA pairs
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of one CTA of a pair, completing on the pair leader's barrier
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t leader_bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(x), "r"(y)
               : "memory");
}
// A role that gave up tells the pair's other CTA, whose roles would otherwise each run into their own limit.
__device__ __forceinline__ void signal_partner_abort(uint32_t abort_addr, uint32_t rank) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_cta(abort_addr, rank ^ 1u)), "r"(1u) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ----------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline int get_encode_fn(EncodeTiledFn *out) {
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

// [rows, K] row-major matrix of `esize`-byte elements, box = [box_rows, 128 bytes], 128-byte swizzle.
// A tensor map is a pure function of (address, shape, box, type), so the last few are kept per thread: a decode
// loop that calls the same layers again and again does not pay the driver's encoder on every launch, and an
// entry whose buffer was freed and reallocated at the same address with the same shape is still correct.
inline int make_map(CUtensorMap *map, int kind, const void *ptr, int64_t rows, int64_t K, int box_rows) {
  struct Entry {
    const void *ptr;
    int64_t rows, K;
    int box_rows, kind;
    CUtensorMap map;
  };
  constexpr int kEntries = 32;
  static thread_local Entry cache[kEntries] = {};
  const uintptr_t h = reinterpret_cast<uintptr_t>(ptr) >> 8;
  Entry &e = cache[(h ^ (h >> 7) ^ (uintptr_t)box_rows ^ ((uintptr_t)rows << 1)) % kEntries];
  if (e.ptr == ptr && ptr != nullptr && e.rows == rows && e.K == K && e.box_rows == box_rows && e.kind == kind) {
    *map = e.map;
    return QL_OK;
  }
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
  e.ptr = ptr;
  e.rows = rows;
  e.K = K;
  e.box_rows = box_rows;
  e.kind = kind;
  e.map = *map;
  return QL_OK;
}


// Result matrix [rows, cols] of `esize`-byte elements with `ld` elements between rows, box = [32 rows, 128 bytes],
// 128-byte swizzle: the epilogue parks 32 rows x 128 bytes in shared memory and one bulk store writes them out as
// whole 128-byte lines (rows and columns beyond the matrix are clipped by the copy engine).
inline int make_map_out(CUtensorMap *map, int dtype, const void *ptr, int64_t rows, int64_t cols, int64_t ld) {
  struct Entry {
    const void *ptr;
    int64_t rows, cols, ld;
    int dtype;
    CUtensorMap map;
  };
  constexpr int kEntries = 16;
  static thread_local Entry cache[kEntries] = {};
  const uintptr_t h = reinterpret_cast<uintptr_t>(ptr) >> 8;
  Entry &e = cache[(h ^ (h >> 7) ^ (uintptr_t)rows) % kEntries];
  if (e.ptr == ptr && ptr != nullptr && e.rows == rows && e.cols == cols && e.ld == ld && e.dtype == dtype) {
    *map = e.map;
    return QL_OK;
  }
  EncodeTiledFn enc;
  int rc = get_encode_fn(&enc);
  if (rc != QL_OK) return rc;
  const int esize = dtype == QL_F32 ? 4 : 2;
  CUtensorMapDataType dt = dtype == QL_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == QL_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * esize};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esize), 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(QL_ERR_CUDA, "cuTensorMapEncodeTiled (result) failed with code %d", (int)r);
  e.ptr = ptr;
  e.rows = rows;
  e.cols = cols;
  e.ld = ld;
  e.dtype = dtype;
  e.map = *map;
  return QL_OK;
}

// [rows, K] row-major bytes, box = [box_rows, box_bytes], no swizzle (tiles read back by ordinary loads)
inline int make_map_bytes(CUtensorMap *map, const void *ptr, int64_t rows, int64_t row_bytes, int box_bytes, int box_rows) {
  EncodeTiledFn enc;
  int rc = get_encode_fn(&enc);
  if (rc != QL_OK) return rc;
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(QL_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return QL_OK;
}

} // namespace
} // namespace ql
