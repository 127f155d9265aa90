// Dense quantized GEMMs on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a only:
//     Y[M,N] = (A[M,K] . B[N,K]^T) * sa[m] * sb[n]
// A and B are K-major ("row-major [rows, K]"), e4m3 / int8 / bf16 / f16; accumulation is f32
// (s32 for int8) in tensor memory; the dequantization scales are applied in the epilogue and the
// result is rounded once to bf16 / f16.  This is the fused form of the reference composition
// dequantize -> matmul (tripy/nvtripy/frontend/module/linear.py:127-151) for operands that are
// both quantized, and of tensorrt.matrix_multiply (TensorRTOps.td:1986-2080) for 16-bit operands.
//
// One persistent CTA per SM, 6 warps:
//   warp 0   one lane issues TMA tile loads (128-byte swizzle; every CTA fetches its own tiles)
//            into a 4-stage ring of [128 x 128 B] A tiles and [BN x 128 B] B tiles
//   warp 1   allocates tensor memory; one lane issues tcgen05.mma (M=128, N=BN, K=32 bytes) from
//            shared-memory descriptors and commits to the ring's "empty" barriers and to the
//            accumulator's "full" barrier
//   warps 2-5 epilogue: tcgen05.ld of the accumulator (two buffers, so the next tile's main loop
//            overlaps), scales, conversion, 16-byte global stores
// Every wait is bounded: when a limit runs out the kernel records a code in `status`, stops
// issuing work, drains what it issued and returns.
#include <cuda.h>
#include <cstdlib>
#include <cstring>

#include "ql_common.cuh"
#include "ql_tc_common.cuh"

namespace ql {
void wo_reload_tuning(); // ql_wo_linear.cu
void w8_reload_tuning(); // ql_gemm_w8a16.cu
void f4_reload_tuning(); // ql_gemm_nvfp4.cu
// ql_gemm_simt.cu
int launch_gemm_simt(int dtype, const void *A, const void *B, const float *sa, int sa_n, const float *sb, int sb_n, const void *bias,
                     int bias_dtype, void *Y, int y_dtype, int batch, int M, int N, int K, int64_t a_m, int64_t a_k, int64_t b_k,
                     int64_t b_n, int64_t ldy, int64_t a_batch, int64_t b_batch, int64_t y_batch, cudaStream_t st);
namespace {

constexpr int STAGES = 4;

// Tuning switches from the environment, read once per process (not on every launch).
struct Tuning {
  bool one_cta, two_kernels, not_cooperative, direct_stores;
  int group_m;
};
Tuning read_tuning() {
  Tuning v;
  v.one_cta = getenv("QL_GEMM_ONE_CTA") != nullptr;
  v.two_kernels = getenv("QL_W8_TWO_KERNELS") != nullptr;
  v.not_cooperative = getenv("QL_W8_NOT_COOPERATIVE") != nullptr;
  v.direct_stores = getenv("QL_GEMM_DIRECT_STORES") != nullptr; // results by per-lane stores instead of bulk stores
  const char *e = getenv("QL_GEMM_GROUP_M");
  v.group_m = e ? atoi(e) : 0;
  return v;
}
Tuning &tuning() {
  static Tuning t = read_tuning();
  return t;
}
constexpr int A_STAGE_BYTES = BM * BK_BYTES;
constexpr int kGemmThreads = 192;


struct GemmArgs {
  void *Y;
  const float *sa; // null = 1, else one value (sa_n == 1) or one per row of A
  const void *sb;  // null = 1, else one value (sb_n == 1) or one per row of B, of type sb_dtype
  int sb_dtype;
  const void *bias; // null, or one value per column of Y (type bias_dtype), added after the scales
  int bias_dtype;
  int sa_n, sb_n;
  int M, N;
  int num_kb;      // K blocks of 128 bytes (the last may be partial: TMA fills zeros)
  int k_elems_per_block;
  int tiles_m, tiles_n;
  int group_m;     // m-tiles per scheduling group (see tile_coords)
  int *status;
  float *row_amax; // non-null: SwiGLU epilogue (see swiglu_chunk); max|result| of every row is merged in here
  int tma_store;   // the CTA-pair kernel writes Y with bulk tensor stores through shared memory (see StoreStage)
  int64_t ldy;     // elements between rows of Y (N, or the full width when Y is a column slice)
  int peer_mode;   // QL_PEER_*: how the epilogue writes Y
  int rows_per_rank;               // QL_PEER_ADD_OWNER: rows [r * rows_per_rank, ...) belong to rank r
  void *owner_y[QL_MAX_PEERS];     // QL_PEER_ADD_OWNER: Y as it lies in each rank's replica
};

// 16 bytes of finished output.  Locally: a streaming store (written once, never re-read here, so it
// stays out of L2's way).  For the peer modes `p` is an address of an NVSwitch replication group that
// maps the same buffer on every GPU of the group: one `multimem.st` lands the tile in all of them
// (an all-gather done by the epilogue), one `multimem.red` adds it into all of them (an all-reduce
// done by the epilogue, summing in the output type as the collective library does), and a plain `red`
// through a peer mapping adds it into the one replica that owns the row (a reduce-scatter done by the
// epilogue).  All are posted writes: the kernel waits on no peer, and they are complete when the kernel is.
template <typename OutT>
__device__ __forceinline__ void store_out16(OutT *p, const uint4 &o, int peer_mode) {
  if (peer_mode == QL_PEER_NONE) {
    __stcs(reinterpret_cast<uint4 *>(p), o);
  } else if (peer_mode == QL_PEER_STORE_ALL) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(__uint_as_float(o.x)),
                 "f"(__uint_as_float(o.y)), "f"(__uint_as_float(o.z)), "f"(__uint_as_float(o.w))
                 : "memory");
  } else if (peer_mode == QL_PEER_ADD_ALL) {
    if constexpr (FloatIO<OutT>::kDtype == QL_F16)
      asm volatile("multimem.red.relaxed.sys.global.add.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w)
                   : "memory");
    else
      asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w)
                   : "memory");
  } else { // QL_PEER_ADD_OWNER: p already points into the owner's replica
    if constexpr (FloatIO<OutT>::kDtype == QL_F16)
      asm volatile("red.relaxed.sys.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w)
                   : "memory");
    else
      asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w)
                   : "memory");
  }
}

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

// Peer modes write through shared memory: in tensor memory a lane owns a row, so a direct store would send
// 32 separate 16-byte pieces per instruction over NVLink (measured: 69 GB/s).  Each epilogue warp instead parks
// 32 rows x 64 columns in its own staging rows and sends them out again with 8 lanes per row, 128 contiguous
// bytes per row and instruction.  Row pitch 144 bytes keeps both directions free of bank conflicts.
constexpr int kPeerRowBytes = 144;
constexpr int kPeerStageWarp = 32 * kPeerRowBytes;
constexpr int kPeerStageBytes = 4 * kPeerStageWarp;

template <typename OutT>
__device__ __forceinline__ void peer_flush(const uint8_t *stage, int lane, OutT *Y, const GemmArgs &args, int m_base, int n_base, int ncols) {
  // the 32 rows of a warp lie inside one 128-row tile, and owners change at multiples of 128 rows
  if (args.peer_mode == QL_PEER_ADD_OWNER) Y = static_cast<OutT *>(args.owner_y[min(m_base / args.rows_per_rank, QL_MAX_PEERS - 1)]);
  __syncwarp();
  const int lanes_per_row = ncols / 8, rows_per_instr = 32 / lanes_per_row;
  const int rsub = lane / lanes_per_row, cw = lane % lanes_per_row;
  for (int r0 = 0; r0 < 32; r0 += rows_per_instr) {
    const int r = r0 + rsub, m = m_base + r, n = n_base + cw * 8;
    const uint4 o = *reinterpret_cast<const uint4 *>(stage + r * kPeerRowBytes + cw * 16);
    if (m < args.M && n + 8 <= args.N) store_out16<OutT>(Y + (size_t)m * (size_t)args.ldy + n, o, args.peer_mode);
  }
  __syncwarp();
}

// sa * (scale of columns n .. n+31) for one chunk.  Issued before the accumulators are fetched from tensor memory,
// so that the two latencies overlap; the per-column loads are 16-byte loads every lane shares.
__device__ __forceinline__ void load_chunk_scales(const GemmArgs &args, int n, float sa, float sb_scalar, float (&s)[32]) {
  if (!args.sb || args.sb_n == 1) {
    const float v = sa * sb_scalar;
#pragma unroll
    for (int j = 0; j < 32; j++) s[j] = v;
  } else if (n + 32 <= args.N && (reinterpret_cast<uintptr_t>(args.sb) & 15) == 0 && args.sb_dtype == QL_F32) {
    const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(args.sb) + n);
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float4 q = __ldg(p + j);
      s[4 * j] = sa * q.x;
      s[4 * j + 1] = sa * q.y;
      s[4 * j + 2] = sa * q.z;
      s[4 * j + 3] = sa * q.w;
    }
  } else if (n + 32 <= args.N && (reinterpret_cast<uintptr_t>(args.sb) & 15) == 0) { // 16-bit scales: 32 values in 64 bytes
    const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(args.sb) + n);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint4 q = __ldg(p + j);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; i++) {
        float lo, hi;
        if (args.sb_dtype == QL_F16) {
          const __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
          lo = __low2float(h);
          hi = __high2float(h);
        } else {
          lo = __uint_as_float(w[i] << 16);
          hi = __uint_as_float(w[i] & 0xFFFF0000u);
        }
        s[8 * j + 2 * i] = sa * lo;
        s[8 * j + 2 * i + 1] = sa * hi;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; j++) s[j] = sa * ((n + j < args.N) ? load_scale(args.sb, args.sb_dtype, n + j) : 0.f);
  }
}

// One epilogue warp's 32 rows x 32 columns of accumulators (lane = row m, columns n .. n+31) -> scaled output.
// `stage` = this warp's staging rows (peer modes only), `c` = index of the chunk within the tile, `last` = no
// chunk follows in this tile.
template <int KIND, typename OutT>
__device__ __forceinline__ void emit_chunk(const GemmArgs &args, OutT *Y, bool vec_ok, const uint32_t (&r)[32], int m, int n,
                                           const float (&s)[32], uint8_t *stage, int lane, int c, bool last) {
  const bool peer = args.peer_mode != QL_PEER_NONE; // the same for every thread of the grid
  if (!peer && !(m < args.M && n < args.N)) return;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; j++) {
    float acc = (KIND == KIND_I8) ? (float)(int)r[j] : __uint_as_float(r[j]);
    v[j] = acc * s[j];
  }
  if (args.bias) { // the same address in every lane: one broadcast load per column
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] += (n + j < args.N) ? load_scale(args.bias, args.bias_dtype, n + j) : 0.f;
  }
  if constexpr (sizeof(OutT) == 4) {
    // f32 result (never a peer mode): 128 bytes per lane and chunk
    float *row = reinterpret_cast<float *>(Y) + (size_t)m * (size_t)args.ldy + n;
    if (vec_ok && n + 32 <= args.N) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) __stcs(reinterpret_cast<float4 *>(row + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
    } else {
      for (int j = 0; j < 32 && n + j < args.N; j++) row[j] = v[j];
    }
  } else {
    if (peer) {
      uint8_t *p = stage + lane * kPeerRowBytes + (c & 1) * 64;
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4 *>(p + j * 2) = make_uint4(pack2<OutT>(v[j], v[j + 1]), pack2<OutT>(v[j + 2], v[j + 3]),
                                                           pack2<OutT>(v[j + 4], v[j + 5]), pack2<OutT>(v[j + 6], v[j + 7]));
      if ((c & 1) || last) peer_flush<OutT>(stage, lane, Y, args, m - lane, n - (c & 1) * 32, (c & 1) ? 64 : 32);
      return;
    }
    OutT *row = Y + (size_t)m * (size_t)args.ldy + n;
    if (vec_ok && n + 32 <= args.N) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 o = make_uint4(pack2<OutT>(v[j], v[j + 1]), pack2<OutT>(v[j + 2], v[j + 3]), pack2<OutT>(v[j + 4], v[j + 5]),
                             pack2<OutT>(v[j + 6], v[j + 7]));
        __stcs(reinterpret_cast<uint4 *>(row + j), o); // written once, never re-read here: keep it out of L2's way
      }
    } else {
      for (int j = 0; j < 32 && n + j < args.N; j++) row[j] = FloatIO<OutT>::from_f32(v[j]);
    }
  }
}

// SwiGLU epilogue of a gate/up projection whose weight rows are interleaved in groups of 32 (rows [64b, 64b + 32) =
// gate channels [32b, 32b + 32), rows [64b + 32, 64b + 64) = the up channels of the same indices): the two
// accumulator chunks of a thread hold gate and up of the same 32 channels, so a = silu(gate) * up is formed in
// registers and written once, in the output type, to Y[m, 32b ..] (Y has N / 2 columns).  The row maximum of the
// rounded values is kept in `rmax` for the per-token scale of the quantize step that follows.
template <typename OutT>
__device__ __forceinline__ void swiglu_chunk(const GemmArgs &args, OutT *Y, bool vec_ok, uint32_t taddr, int m, int n, float sa,
                                             float sb_scalar, float &rmax) {
  uint32_t r[32];
  float s[32], g[32];
  load_chunk_scales(args, n, sa, sb_scalar, s);
  tmem_load_32(taddr, r);
#pragma unroll
  for (int j = 0; j < 32; j++) g[j] = __uint_as_float(r[j]) * s[j];
  load_chunk_scales(args, n + 32, sa, sb_scalar, s);
  tmem_load_32(taddr + 32, r);
  if (!(m < args.M && n < args.N)) return;
  uint32_t w[16];
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    const float a0 = silu_mul(g[j], __uint_as_float(r[j]) * s[j]), a1 = silu_mul(g[j + 1], __uint_as_float(r[j + 1]) * s[j + 1]);
    w[j >> 1] = pack2<OutT>(a0, a1);
    const OutT *h = reinterpret_cast<const OutT *>(&w[j >> 1]);
    rmax = fmaxf(rmax, fmaxf(fabsf(FloatIO<OutT>::to_f32(h[0])), fabsf(FloatIO<OutT>::to_f32(h[1]))));
  }
  OutT *row = Y + (size_t)m * (size_t)args.ldy + (n >> 1);
  if (vec_ok) {
#pragma unroll
    for (int j = 0; j < 16; j += 4) __stcs(reinterpret_cast<uint4 *>(row) + (j >> 2), make_uint4(w[j], w[j + 1], w[j + 2], w[j + 3]));
  } else {
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const OutT *h = reinterpret_cast<const OutT *>(&w[j]);
      row[2 * j] = h[0];
      row[2 * j + 1] = h[1];
    }
  }
}

// Results leave the CTA-pair kernel through shared memory.  In tensor memory a lane owns a row, so a direct store
// sends 32 separate 16-byte pieces per instruction, half a sector each: the epilogue then takes longer than the
// MMAs of a tile with K below about 4096 bytes and the kernel is bound by it.  Instead each epilogue warp parks
// 32 rows x 128 bytes in its own staging buffer (laid out with the copy engine's 128-byte swizzle, which also keeps
// the quarter-warp's 16-byte writes on distinct banks) and one lane issues a bulk tensor store that writes whole
// 128-byte lines and clips rows and columns beyond the matrix.  Two buffers per warp, used in turn: a buffer is
// rewritten once the store issued from it two steps earlier has read it.
struct StoreStage {
  uint8_t *base; // 2 x 4096 bytes, 1024-byte aligned
  int buf;
  __device__ __forceinline__ void begin(int lane) { // before the first write into the current buffer
    if (lane == 0) bulk_wait_read<1>();
    __syncwarp();
  }
  __device__ __forceinline__ void put(int lane, int piece, const uint4 &v) { // 16-byte piece `piece` (0..7) of row `lane`
    *reinterpret_cast<uint4 *>(base + buf * 4096 + lane * 128 + ((piece ^ (lane & 7)) << 4)) = v;
  }
  __device__ __forceinline__ void send(const CUtensorMap *map, int lane, int x, int y) { // the buffer is complete
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map, smem_u32(base + buf * 4096), x, y);
      bulk_commit();
    }
    buf ^= 1;
  }
  __device__ __forceinline__ void finish(int lane) { // before the CTA's shared memory goes away
    if (lane == 0) bulk_wait_all<0>();
    __syncwarp();
  }
};

// emit_chunk through the staging buffers: chunk `c` of the tile is columns n .. n+31 of rows m_base .. m_base+31.
template <int KIND, typename OutT>
__device__ __forceinline__ void emit_chunk_tma(const GemmArgs &args, const CUtensorMap *map_y, const uint32_t (&r)[32], int m_base, int n,
                                               const float (&s)[32], StoreStage &st, int lane, int c) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; j++) {
    float acc = (KIND == KIND_I8) ? (float)(int)r[j] : __uint_as_float(r[j]);
    v[j] = acc * s[j];
  }
  if (args.bias) {
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] += (n + j < args.N) ? load_scale(args.bias, args.bias_dtype, n + j) : 0.f;
  }
  if constexpr (sizeof(OutT) == 4) { // 32 columns fill the 128-byte row
    st.begin(lane);
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      st.put(lane, j >> 2, make_uint4(__float_as_uint(v[j]), __float_as_uint(v[j + 1]), __float_as_uint(v[j + 2]), __float_as_uint(v[j + 3])));
    st.send(map_y, lane, n, m_base);
  } else { // two chunks fill the row
    const int half = c & 1;
    if (half == 0) st.begin(lane);
#pragma unroll
    for (int j = 0; j < 32; j += 8)
      st.put(lane, half * 4 + (j >> 3), make_uint4(pack2<OutT>(v[j], v[j + 1]), pack2<OutT>(v[j + 2], v[j + 3]), pack2<OutT>(v[j + 4], v[j + 5]),
                                                   pack2<OutT>(v[j + 6], v[j + 7])));
    if (half == 1) st.send(map_y, lane, n - 32, m_base);
  }
}

// swiglu_chunk through the staging buffers: pair `c` of the tile gives result columns (n >> 1) .. (n >> 1) + 31.
template <typename OutT>
__device__ __forceinline__ void swiglu_chunk_tma(const GemmArgs &args, const CUtensorMap *map_y, uint32_t taddr, int m_base, int n, float sa,
                                                 float sb_scalar, float &rmax, StoreStage &st, int lane, int c) {
  uint32_t r[32];
  float s[32], g[32];
  load_chunk_scales(args, n, sa, sb_scalar, s);
  tmem_load_32(taddr, r);
#pragma unroll
  for (int j = 0; j < 32; j++) g[j] = __uint_as_float(r[j]) * s[j];
  load_chunk_scales(args, n + 32, sa, sb_scalar, s);
  tmem_load_32(taddr + 32, r);
  const int half = c & 1;
  const bool live = m_base + lane < args.M && n < args.N;
  if (half == 0) st.begin(lane);
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int k = j + 2 * i;
      const float a0 = silu_mul(g[k], __uint_as_float(r[k]) * s[k]), a1 = silu_mul(g[k + 1], __uint_as_float(r[k + 1]) * s[k + 1]);
      w[i] = pack2<OutT>(a0, a1);
      const OutT *h = reinterpret_cast<const OutT *>(&w[i]);
      if (live) rmax = fmaxf(rmax, fmaxf(fabsf(FloatIO<OutT>::to_f32(h[0])), fabsf(FloatIO<OutT>::to_f32(h[1]))));
    }
    st.put(lane, half * 4 + (j >> 3), make_uint4(w[0], w[1], w[2], w[3]));
  }
  if (half == 1) st.send(map_y, lane, (n >> 1) - 32, m_base);
}

// The whole accumulator of one tile (BN columns from tensor-memory address taddr) through swiglu_chunk.
template <int BN, typename OutT>
__device__ __forceinline__ void swiglu_tile(const GemmArgs &args, OutT *Y, bool vec_ok, uint32_t taddr, int m, int n0, float sa, float sb_scalar) {
  float rmax = 0.f;
#pragma unroll 1
  for (int c = 0; c < BN / 64; c++) swiglu_chunk<OutT>(args, Y, vec_ok, taddr + c * 64, m, n0 + c * 64, sa, sb_scalar, rmax);
  // non-negative floats order like their bit patterns
  if (m < args.M && rmax > 0.f) atomicMax(reinterpret_cast<int *>(args.row_amax) + m, __float_as_int(rmax));
}

template <int BN> struct SmemLayout {
  static constexpr int kBStage = BN * BK_BYTES;
  static constexpr int kStage = A_STAGE_BYTES + kBStage;
  static constexpr int kTiles = STAGES * kStage;
  static constexpr int kBarriers = kTiles;            // full[S], empty[S], tmem_full[2], tmem_empty[2], drain
  static constexpr int kTmemPtr = kBarriers + (2 * STAGES + 5) * 8;
  static constexpr int kAbort = kTmemPtr + 4;
  static constexpr int kPeerStage = (kAbort + 4 + 15) & ~15; // staging rows of the peer-mode epilogue
  static constexpr int kTotal = kPeerStage + kPeerStageBytes;
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
    uint8_t *stage = smem + L::kPeerStage + quad * kPeerStageWarp;
    const bool vec_ok = (args.ldy % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
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
      const float sb_scalar = (args.sb && args.sb_n == 1) ? load_scale(args.sb, args.sb_dtype, 0) : 1.f;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
      bool fused = false;
      if constexpr (KIND == KIND_F8 && sizeof(OutT) == 2 && BN >= 64) {
        if (args.row_amax) {
          swiglu_tile<BN, OutT>(args, Y, vec_ok, taddr, m, n0, sa, sb_scalar);
          fused = true;
        }
      }
#pragma unroll 1
      for (int c = 0; c < (fused ? 0 : BN / 32); c++) {
        uint32_t r[32];
        float sc[32];
        const int n = n0 + c * 32;
        load_chunk_scales(args, n, sa, sb_scalar, sc);
        tmem_load_32(taddr + c * 32, r);
        emit_chunk<KIND, OutT>(args, Y, vec_ok, r, m, n, sc, stage, lane, c, c == BN / 32 - 1);
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
// ----------------------------------------------------------------------------------------------
// Two-CTA variant (cta_group::2): a pair of CTAs on neighbouring SMs forms a cluster and computes a
// 256 x 256 tile with one M=256 MMA stream issued by the pair's leader.  Each CTA loads its own 128
// rows of A and its own half (128 rows) of the B tile, so a stage is 32 KiB instead of 48 KiB: seven
// stages fit, and L2 -> shared-memory traffic per flop drops by a third.  Every
// CTA fetches what it needs itself and signals the leader's "full" barrier (the .cta_group::2 form of
// the tile load allows the barrier to live in the pair's other CTA).
// ----------------------------------------------------------------------------------------------
constexpr int BN2 = 256;
constexpr int B2_STAGE_BYTES = (BN2 / 2) * BK_BYTES;
constexpr int STAGE2_BYTES = A_STAGE_BYTES + B2_STAGE_BYTES;

// Six pipeline stages of 32 KiB and 32 KiB of epilogue staging.  PEER = the instantiation whose epilogue may
// write to peers (its staging rows lie in the same area).
template <bool PEER> struct Smem2 {
  static constexpr int kStages = 6;
  static constexpr int kTiles = kStages * STAGE2_BYTES;
  static constexpr int kStage = kTiles;                      // epilogue staging: 4 warps x 2 x 4096 bytes of StoreStage,
  static constexpr int kStageBytes = 4 * 2 * 4096;           // or the peer-mode rows (kPeerStageBytes), which are smaller
  static constexpr int kPeerStage = kStage;
  static constexpr int kBarriers = kStage + kStageBytes;     // full[S], empty[S], tfull[2], tempty[2], drain
  static constexpr int kTmemPtr = kBarriers + (2 * kStages + 5) * 8;
  static constexpr int kAbort = kTmemPtr + 4;
  static constexpr int kTotal = kAbort + 4;
  static constexpr int kDynamic = kTotal + 1024;
};
static_assert(kPeerStageBytes <= Smem2<true>::kStageBytes, "the peer-mode staging rows share the store staging area");

template <int KIND>
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == KIND_F8) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else if constexpr (KIND == KIND_I8) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}

template <int KIND>
__device__ __forceinline__ uint32_t make_instr_desc_pair() {
  // same fields as the one-CTA descriptor with M = 256
  uint32_t d = make_instr_desc<KIND, BN2>();
  d &= ~(0x1Fu << 24);
  d |= (uint32_t)(256 >> 4) << 24;
  return d;
}

// W8A16 inside the pair kernel.  The B operand's tensor map points at a 16-bit scratch copy of the int8 weights
// that eight extra warps per CTA produce while the GEMM runs: the weights are cut into chunks of 8 rows, CTA i
// widens chunks i, i + grid, ... in order and bumps the counter of the chunk's tile; a TMA producer waits until the 32 chunks
// of a 256-row tile are there before its first load of that tile.  Tiles are walked in rising column order, so
// only the first wave waits noticeably (one chunk per CTA), and the rest of the conversion's HBM traffic hides
// under the MMAs.  The launch is cooperative (all CTAs resident), so a waiting producer cannot starve the CTA
// that owes it a chunk; waits are bounded all the same.  The last CTA to finish clears the counters.
// (Widening per tile in shared memory inside this kernel, with converter warps feeding the MMA's B operand, was
// built and measured: 362 us at M = 2048 with sixteen warps converting every k-block together, 202-215 us with the
// warps split into four groups taking k-blocks in turn, against 147 us here; deeper rings changed nothing.  ncu
// showed the converter warps stalled in the proxy fence and on the barriers; the limiter was not identified.)
constexpr int kWidenThreads = 256;
constexpr int kWidenChunkRows = 8;
struct WidenArgs {
  const uint8_t *raw; // int8 [N, K]
  void *wide;         // XT [N, K] scratch
  int *ready;         // one counter per 256-row tile of W, then the exit counter
  int N, K;
};

template <typename XT, int I>
__device__ __forceinline__ uint32_t widen_i8_pair(uint32_t w) {
  if constexpr (FloatIO<XT>::kDtype == QL_F16) {
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

__device__ __forceinline__ bool wait_counter(const int *ctr, int need, volatile int *abort_flag, int *status, int code) {
  const long long t0 = clock64();
  for (;;) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= need) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
    __nanosleep(200);
  }
}

// args.tiles_m counts 256-row tiles here; args.tiles_n counts 256-column tiles.
template <int KIND, typename OutT, bool PEER, bool WIDEN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(WIDEN ? kGemmThreads + kWidenThreads : kGemmThreads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_y, const GemmArgs args, const WidenArgs wargs) {
  using L = Smem2<PEER>;
  constexpr int STAGES2 = L::kStages;
  constexpr uint32_t kTmemCols = 512; // two 256-column accumulators
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarriers;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES2 + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES2 + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES2 + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * STAGES2 + 4);
  volatile uint32_t *tmem_ptr_smem = reinterpret_cast<volatile uint32_t *>(smem + L::kTmemPtr);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_tiles = args.tiles_m * args.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; s++) {
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
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int mt, nt;
        tile_coords(args, tile, &mt, &nt);
        const int m0 = mt * 256 + (int)rank * BM, n0 = nt * BN2 + (int)rank * (BN2 / 2);
        if constexpr (WIDEN) {
          const int chunks = (wargs.N + kWidenChunkRows - 1) / kWidenChunkRows, per_tile = BN2 / kWidenChunkRows;
          const int need = min(per_tile, chunks - nt * per_tile);
          if (!wait_counter(wargs.ready + nt, need, abort_flag, args.status, ST_TIMEOUT_READY)) { ok = false; break; }
          asm volatile("fence.proxy.async;" ::: "memory"); // the chunks were written with ordinary stores
        }
        for (int kb = 0; kb < args.num_kb; kb++) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, args.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + stage * STAGE2_BYTES, b_dst = a_dst + A_STAGE_BYTES;
          const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE2_BYTES); // both CTAs' bytes land on the leader's barrier
          tma_load_2d_pair(a_dst, &map_a, leader_full, kb * args.k_elems_per_block, m0);
          tma_load_2d_pair(b_dst, &map_b, leader_full, kb * args.k_elems_per_block, n0);
          issued++;
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        signal_partner_abort(smem_u32((const void *)abort_flag), rank);
        if (rank == 0) {
          // Both CTAs' loads complete on the leader's barriers: let the ones still in flight land before either
          // CTA's shared memory goes away (the partner cannot leave before the cluster barrier at the end).
          const long long pending = issued < STAGES2 ? issued : STAGES2;
          for (long long i = 0; i < pending; i++) {
            stage = (stage == 0) ? STAGES2 - 1 : stage - 1;
            if (stage == STAGES2 - 1) phase ^= 1;
            const long long t0 = clock64();
            while (!mbar_try_wait(full_bar(stage), phase) && clock64() - t0 < kWaitLimitCycles) {}
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_instr_desc_pair<KIND>();
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, it++) {
        const int buf = it & 1;
        if (!mbar_wait(tempty_bar(buf), ((it >> 1) & 1) ^ 1, abort_flag, args.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN2);
        for (int kb = 0; kb < args.num_kb; kb++) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, args.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * STAGE2_BYTES;
          const uint64_t adesc = make_smem_desc(a_addr), bdesc = make_smem_desc(a_addr + A_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK_BYTES / 32; k++)
            tc_mma_pair<KIND>(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          // the stage is free in both CTAs once these MMAs have read it
          tc_commit_pair(map_to_cta(empty_bar(stage), 0));
          tc_commit_pair(map_to_cta(empty_bar(stage), 1));
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
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
  } else if (WIDEN && warp >= 6) {
    // ------------------------------------------------------------------ weight wideners (warps 6 and up, both CTAs)
    const int ct = threadIdx.x - kGemmThreads;
    const int chunks = (wargs.N + kWidenChunkRows - 1) / kWidenChunkRows;
    for (int c = blockIdx.x; c < chunks; c += gridDim.x) {
      const int r0 = c * kWidenChunkRows, rows = min(kWidenChunkRows, wargs.N - r0);
      const uint4 *src = reinterpret_cast<const uint4 *>(wargs.raw + (size_t)r0 * wargs.K);
      uint4 *dst = reinterpret_cast<uint4 *>(static_cast<OutT *>(wargs.wide) + (size_t)r0 * wargs.K);
      const int n16 = rows * (wargs.K / 16);
#pragma unroll 8
      for (int i = ct; i < n16; i += kWidenThreads) {
        const uint4 w = __ldcs(src + i);
        dst[2 * i] = make_uint4(widen_i8_pair<OutT, 0>(w.x), widen_i8_pair<OutT, 2>(w.x), widen_i8_pair<OutT, 0>(w.y), widen_i8_pair<OutT, 2>(w.y));
        dst[2 * i + 1] = make_uint4(widen_i8_pair<OutT, 0>(w.z), widen_i8_pair<OutT, 2>(w.z), widen_i8_pair<OutT, 0>(w.w), widen_i8_pair<OutT, 2>(w.w));
      }
      __threadfence();
      asm volatile("fence.proxy.async;" ::: "memory");            // TMA (async proxy) will read what was just stored
      asm volatile("bar.sync 1, %0;" ::"n"(kWidenThreads) : "memory"); // the whole chunk is out before it is announced
      if (ct == 0) asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(wargs.ready + c / (BN2 / kWidenChunkRows)) : "memory");
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    OutT *Y = static_cast<OutT *>(args.Y);
    uint8_t *stage = PEER ? smem + L::kPeerStage + quad * kPeerStageWarp : nullptr;
    StoreStage sst{smem + L::kStage + quad * 8192, 0};
    const bool tma_out = !PEER && args.tma_store; // the same for every thread of the grid
    const bool vec_ok = (args.ldy % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
    int it = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, it++) {
      const int buf = it & 1;
      int mt, nt;
      tile_coords(args, tile, &mt, &nt);
      const int m0 = mt * 256 + (int)rank * BM, n0 = nt * BN2;
      if (!mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag, args.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int m_base = m0 + quad * 32, m = m_base + lane;
      float sa = 1.f;
      if (args.sa) sa = (args.sa_n == 1) ? __ldg(args.sa) : (m < args.M ? __ldg(args.sa + m) : 0.f);
      const float sb_scalar = (args.sb && args.sb_n == 1) ? load_scale(args.sb, args.sb_dtype, 0) : 1.f;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN2);
      bool fused = false;
      if constexpr (KIND == KIND_F8 && sizeof(OutT) == 2 && !PEER && !WIDEN) {
        if (args.row_amax) {
          if (tma_out) {
            float rmax = 0.f;
#pragma unroll 1
            for (int c = 0; c < BN2 / 64; c++)
              swiglu_chunk_tma<OutT>(args, &map_y, taddr + c * 64, m_base, n0 + c * 64, sa, sb_scalar, rmax, sst, lane, c);
            if (m < args.M && rmax > 0.f) atomicMax(reinterpret_cast<int *>(args.row_amax) + m, __float_as_int(rmax));
          } else {
            swiglu_tile<BN2, OutT>(args, Y, vec_ok, taddr, m, n0, sa, sb_scalar);
          }
          fused = true;
        }
      }
#pragma unroll 1
      for (int c = 0; c < (fused ? 0 : BN2 / 32); c++) {
        uint32_t r[32];
        float sc[32];
        const int n = n0 + c * 32;
        load_chunk_scales(args, n, sa, sb_scalar, sc);
        tmem_load_32(taddr + c * 32, r);
        if (tma_out) emit_chunk_tma<KIND, OutT>(args, &map_y, r, m_base, n, sc, sst, lane, c);
        else emit_chunk<KIND, OutT>(args, Y, vec_ok, r, m, n, sc, stage, lane, c, c == BN2 / 32 - 1);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0)); // the leader owns the accumulator hand-over
    }
    if (tma_out) sst.finish(lane);
    if (!ok && lane == 0) signal_partner_abort(smem_u32((const void *)abort_flag), rank);
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all(); // neither CTA may leave while the pair's MMAs or barriers can still touch it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
  if constexpr (WIDEN) {
    // the last CTA out leaves the counters at zero for the next launch
    if (threadIdx.x == 0) {
      const int tiles_w = (wargs.N + BN2 - 1) / BN2;
      __threadfence();
      if (atomicAdd(wargs.ready + tiles_w, 1) == (int)gridDim.x - 1) {
        for (int i = 0; i <= tiles_w; i++) wargs.ready[i] = 0;
        __threadfence();
      }
    }
  }
}

// The CTA-pair kernel's variants: plain, with the peer-mode epilogue, with the int8 weights widened inside.
enum { PAIR_PLAIN = 0, PAIR_PEER = 2, PAIR_WIDEN = 3 };
template <int KIND, typename OutT, int V>
auto pair_kernel() {
  return gemm_tc2_kernel<KIND, OutT, V == PAIR_PEER, V == PAIR_WIDEN>;
}
template <int V> constexpr int pair_smem() { return V == PAIR_PEER ? Smem2<true>::kDynamic : Smem2<false>::kDynamic; }
template <int V> constexpr int pair_threads() { return V == PAIR_WIDEN ? kGemmThreads + kWidenThreads : kGemmThreads; }

// Largest number of CTA pairs that can be resident at once on this device (0 = pairs unavailable).
template <int KIND, typename OutT, int V>
int max_resident_pairs() {
  static int cached[64] = {0};
  static bool known[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!known[dev]) {
    auto kern = pair_kernel<KIND, OutT, V>();
    const int smem_bytes = pair_smem<V>();
    int n = 0;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * sm_count(), 1, 1);
      cfg.blockDim = dim3(pair_threads<V>(), 1, 1);
      cfg.dynamicSmemBytes = smem_bytes;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) n = 0;
      cudaGetLastError();
    }
    cached[dev] = n;
    known[dev] = true;
  }
  return cached[dev];
}

template <int KIND, typename OutT, int V>
int launch_gemm_pair(const void *A, const void *B, GemmArgs args, int64_t K, int pairs, cudaStream_t st, WidenArgs wargs = WidenArgs{}) {
  CUtensorMap ma, mb, my;
  int rc;
  if ((rc = make_map(&ma, KIND, A, args.M, K, BM)) != QL_OK) return rc;
  if ((rc = make_map(&mb, KIND, B, args.N, K, BN2 / 2)) != QL_OK) return rc;
  // results through shared memory and bulk stores wherever the copy engine can address them
  args.tma_store = 0;
  memset(&my, 0, sizeof(my));
  if (V != PAIR_PEER && aligned16(args.Y) && (args.ldy * (int64_t)sizeof(OutT)) % 16 == 0 && !tuning().direct_stores) {
    const int64_t cols = args.row_amax ? args.N / 2 : args.N;
    if ((rc = make_map_out(&my, FloatIO<OutT>::kDtype, args.Y, args.M, cols, args.ldy)) != QL_OK) return rc;
    args.tma_store = 1;
  }
  constexpr int kTileN = BN2;
  args.tiles_m = (args.M + 255) / 256;
  args.tiles_n = (args.N + kTileN - 1) / kTileN;
  args.group_m = (args.group_m + 1) / 2; // bands were sized in 128-row tiles
  if (args.group_m < 1) args.group_m = 1;
  if (args.group_m > args.tiles_m) args.group_m = args.tiles_m;
  const int tiles = args.tiles_m * args.tiles_n;
  const int clusters = tiles < pairs ? tiles : pairs;
  if constexpr (V == PAIR_WIDEN) {
    // column-major walk over the whole M: the weight tiles are needed in the order they are widened
    args.group_m = args.tiles_m;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * clusters, 1, 1);
    cfg.blockDim = dim3(pair_threads<V>(), 1, 1);
    cfg.dynamicSmemBytes = pair_smem<V>();
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeCooperative; // every CTA resident: producers wait on chunks other CTAs widen
    attr.val.cooperative = tuning().not_cooperative ? 0 : 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, pair_kernel<KIND, OutT, V>(), ma, mb, my, args, wargs);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return QL_ERR_UNSUPPORTED; // the caller falls back to the two-kernel route
    }
  } else {
    pair_kernel<KIND, OutT, V>()<<<2 * clusters, pair_threads<V>(), pair_smem<V>(), st>>>(ma, mb, my, args, wargs);
  }
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
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
  if (args.M > 256 && args.N >= 512 && !tuning().one_cta) {
    // (256 x 512 tiles per pair were built and measured: a quarter less L2 traffic per flop, but with a single
    // accumulator the hand-over between tiles is exposed; 1.51 ms against 1.44 ms for 8192 x 28672 x 8192 fp8.)
    const long long tiles2 = (long long)((args.M + 255) / 256) * ((args.N + BN2 - 1) / BN2);
    if constexpr (KIND == KIND_F8 && sizeof(OutT) == 2) {
      if (args.peer_mode != QL_PEER_NONE) {
        const int pairs = max_resident_pairs<KIND, OutT, PAIR_PEER>();
        if (pairs > 0 && tiles2 >= pairs) return launch_gemm_pair<KIND, OutT, PAIR_PEER>(A, B, args, K, pairs, st);
      }
    }
    if (args.peer_mode == QL_PEER_NONE) {
      const int pairs = max_resident_pairs<KIND, OutT, PAIR_PLAIN>();
      if (pairs > 0 && tiles2 >= pairs) return launch_gemm_pair<KIND, OutT, PAIR_PLAIN>(A, B, args, K, pairs, st);
    }
  }
  int bn = 32;
  for (int cand : {256, 128, 64}) {
    if ((int64_t)args.tiles_m * ((args.N + cand - 1) / cand) >= sms) { bn = cand; break; }
  }
  if (args.N <= 32) bn = 32;
  if (args.row_amax && bn < 64) bn = 64; // the SwiGLU epilogue pairs two 32-column chunks
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

// Shapes, types and scales of Y = (A . B^T) * sa * sb + bias.  Says nothing about which kernel can run it.
int check_gemm(const char *op, const ql_tensor *a, const ql_tensor *b, const ql_tensor *sa, const ql_tensor *sb, const ql_tensor *bias,
               const ql_tensor *y, int want_dtype_a, int want_dtype_b) {
  if (!a || !b || !y) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  if (a->rank != 2 || b->rank != 2 || y->rank != 2)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: operands must be 2-D ([M,K], [N,K], [M,N])", op);
  if (a->dtype != want_dtype_a || b->dtype != want_dtype_b)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: unexpected operand types %d, %d", op, a->dtype, b->dtype);
  if (!is_float_dtype(y->dtype)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: y must be f32, bf16 or f16", op);
  if (a->shape[1] != b->shape[1])
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: inner dimensions differ (%lld vs %lld)", op, (long long)a->shape[1], (long long)b->shape[1]);
  if (y->shape[0] != a->shape[0] || y->shape[1] != b->shape[0])
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: y must be [M,N] = [%lld,%lld]", op, (long long)a->shape[0], (long long)b->shape[0]);
  const ql_tensor *sc[2] = {sa, sb};
  const int64_t want[2] = {a->shape[0], b->shape[0]};
  for (int i = 0; i < 2; i++) {
    if (!sc[i]) continue;
    if (sc[i]->dtype != QL_F32) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: scales must be f32", op);
    if (sc[i]->rank < 0 || sc[i]->rank > QL_MAX_RANK) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: bad scale rank", op);
    int64_t n = numel(sc[i]);
    if (!(n == 1 || (sc[i]->rank == 1 && n == want[i])))
      return set_error(QL_ERR_INVALID_ARGUMENT, "%s: a scale must be a scalar or one value per row of its operand", op);
    if (!sc[i]->data) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: scale has no data pointer", op);
  }
  if (bias) {
    if (!is_float_dtype(bias->dtype) || bias->rank != 1 || bias->shape[0] != b->shape[0])
      return set_error(QL_ERR_INVALID_ARGUMENT, "%s: bias must be a float vector with one value per output column", op);
    if (!bias->data && bias->shape[0] > 0) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: bias has no data pointer", op);
  }
  if (numel(a) > 0 && !a->data) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: x has no data pointer", op);
  if (numel(b) > 0 && !b->data) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: w has no data pointer", op);
  if (numel(y) > 0 && !y->data) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: y has no data pointer", op);
  if (a->shape[0] > INT32_MAX || b->shape[0] > INT32_MAX || a->shape[1] > INT32_MAX)
    return set_error(QL_ERR_UNSUPPORTED, "%s: dimension too large", op);
  return QL_OK;
}

// The tensor-core kernels take K-major operands whose rows are whole 16-byte units from a 16-byte aligned base
// (the TMA rules) and write 16-bit results, or f32 results of the quantized kinds.  Everything else -- f32
// operands, K = 4, odd strides, unaligned views -- runs on the general kernel (ql_gemm_simt.cu).
template <int KIND>
bool tensor_core_ok(const ql_tensor *a, const ql_tensor *b, const ql_tensor *y) {
  const int esize = (KIND == KIND_F8 || KIND == KIND_I8) ? 1 : 2;
  const int64_t K = a->shape[1];
  if (K == 0 || (K * esize) % 16 != 0) return false;
  if (!aligned16(a->data) || !aligned16(b->data)) return false;
  if (y->dtype == QL_F32) return KIND == KIND_F8 || KIND == KIND_I8;
  return true;
}

int run_simt(const ql_tensor *a, const ql_tensor *b, const ql_tensor *sa, const ql_tensor *sb, const ql_tensor *bias, ql_tensor *y,
             void *stream) {
  const int64_t M = a->shape[0], K = a->shape[1], N = b->shape[0];
  return launch_gemm_simt(a->dtype, a->data, b->data, sa ? static_cast<const float *>(sa->data) : nullptr, sa ? (int)numel(sa) : 1,
                          sb ? static_cast<const float *>(sb->data) : nullptr, sb ? (int)numel(sb) : 1, bias ? bias->data : nullptr,
                          bias ? bias->dtype : QL_F32, y->data, y->dtype, 1, (int)M, (int)N, (int)K, K, 1, 1, K, N, 0, 0, 0,
                          (cudaStream_t)stream);
}

template <int KIND>
int run_gemm(const char *op, const ql_tensor *a, const ql_tensor *b, const ql_tensor *sa, const ql_tensor *sb, const ql_tensor *bias,
             ql_tensor *y, void *stream, int64_t ldy = 0, int peer_mode = QL_PEER_NONE, const ql_peer_buffer *dest = nullptr,
             int64_t offset = 0, float *row_amax = nullptr) {
  const int64_t M = a->shape[0], K = a->shape[1], N = b->shape[0];
  if (M == 0 || N == 0) return QL_OK;
  const int esize = (KIND == KIND_F8 || KIND == KIND_I8) ? 1 : 2;
  if (!tensor_core_ok<KIND>(a, b, y)) {
    if (row_amax) return QL_ERR_UNSUPPORTED; // the caller says so in its own words
    if (peer_mode != QL_PEER_NONE)
      return set_error(QL_ERR_UNSUPPORTED, "%s: peer modes need K * element size to be a non-zero multiple of 16 bytes (K=%lld) and aligned operands",
                       op, (long long)K);
    return run_simt(a, b, sa, sb, bias, y, stream);
  }
  GemmArgs args;
  args.Y = y->data;
  args.sa = sa ? static_cast<const float *>(sa->data) : nullptr;
  args.sb = sb ? sb->data : nullptr;
  args.sb_dtype = sb ? sb->dtype : QL_F32;
  args.bias = bias ? bias->data : nullptr;
  args.bias_dtype = bias ? bias->dtype : QL_F32;
  args.sa_n = sa ? (int)numel(sa) : 1;
  args.sb_n = sb ? (int)numel(sb) : 1;
  args.M = (int)M;
  args.N = (int)N;
  args.k_elems_per_block = BK_BYTES / esize;
  args.num_kb = (int)((K * esize + BK_BYTES - 1) / BK_BYTES);
  args.tiles_m = (int)((M + BM - 1) / BM);
  args.tiles_n = 0;
  {
    // A band of row tiles of A stays L2-resident while B streams through once per band.  Measured on B200: about
    // 16 MiB of A, but never fewer than 16 row tiles (2048 rows) while those stay under 64 MiB: with long rows
    // (K = 28672) 4 tiles per band re-streamed B eight times and cost 7 % against 16 tiles per band.
    const int64_t tile_bytes = (int64_t)BM * K * esize;
    int64_t band = (16ll << 20) / tile_bytes;
    const int64_t wide = (64ll << 20) / tile_bytes;
    if (band < 16) band = wide < 16 ? wide : 16;
    args.group_m = (int)(band < 4 ? 4 : band);
    if (tuning().group_m > 0) args.group_m = tuning().group_m; // tuning aid
    if (args.group_m > args.tiles_m) args.group_m = args.tiles_m;
  }
  args.ldy = ldy > 0 ? ldy : N;
  args.peer_mode = peer_mode;
  args.rows_per_rank = 1;
  for (int r = 0; r < QL_MAX_PEERS; r++) args.owner_y[r] = nullptr;
  if (peer_mode == QL_PEER_ADD_OWNER) {
    args.rows_per_rank = (int)(M / dest->world);
    for (int r = 0; r < dest->world; r++) args.owner_y[r] = static_cast<char *>(dest->replica[r]) + offset * 2;
  }
  args.status = device_status_word();
  if (!args.status) return set_error(QL_ERR_CUDA, "%s: could not allocate the device status word", op);
  args.row_amax = row_amax;
  args.tma_store = 0;
  if (row_amax) args.ldy = N / 2;
  cudaStream_t st = (cudaStream_t)stream;
  if (y->dtype == QL_BF16) return launch_gemm_kind<KIND, __nv_bfloat16>(a->data, b->data, args, K, st);
  if (y->dtype == QL_F16) return launch_gemm_kind<KIND, __half>(a->data, b->data, args, K, st);
  if constexpr (KIND == KIND_F8 || KIND == KIND_I8) return launch_gemm_kind<KIND, float>(a->data, b->data, args, K, st);
  return set_error(QL_ERR_UNSUPPORTED, "%s: unreachable output type", op);
}

} // namespace

// Y[M,N] = (X[M,K] . W[N,K]^T) * sb[n]; X, W and Y of the same 16-bit type (QL_BF16 / QL_F16).
int gemm16_device(int dtype, const void *X, const void *W, const float *sb, int sb_n, void *Y, int M, int N, int K,
                  cudaStream_t st) {
  ql_tensor x{const_cast<void *>(X), dtype, 2, {M, K}}, w{const_cast<void *>(W), dtype, 2, {N, K}}, y{Y, dtype, 2, {M, N}};
  ql_tensor s{const_cast<float *>(sb), QL_F32, 1, {sb_n}};
  if (dtype == QL_BF16) return run_gemm<KIND_BF16>("gemm_16", &x, &w, nullptr, sb ? &s : nullptr, nullptr, &y, st);
  return run_gemm<KIND_F16>("gemm_16", &x, &w, nullptr, sb ? &s : nullptr, nullptr, &y, st);
}

// Y[M,N] = (X[M,K] . widen(Wq[N,K])^T) * scale[n] in one launch: the pair kernel with the int8 -> 16-bit conversion
// running ahead of the tiles (see WidenArgs).  `wide` = [N,K] scratch of X's type, `counters` = ceil(N/256) + 1
// zeroed ints.  Returns QL_ERR_UNSUPPORTED (without touching the error text) when the shape or the device does not
// suit it; the caller then widens in a kernel of its own.
template <int KIND, typename XT>
int gemm16_widen_t(const void *X, const void *Wraw, void *wide, int *counters, const void *scale, int sdt, void *Y, int M, int N, int K,
                   cudaStream_t st) {
  const int pairs = max_resident_pairs<KIND, XT, PAIR_WIDEN>();
  const long long tiles2 = (long long)((M + 255) / 256) * ((N + BN2 - 1) / BN2);
  // Worth it from about four waves of tiles on: the wideners are slower than a kernel of their own (they share the
  // SMs with the GEMM), and with few waves the first one waits for most of the weights.
  if (pairs <= 0 || tiles2 < 4ll * pairs) return QL_ERR_UNSUPPORTED;
  GemmArgs args;
  args.Y = Y;
  args.sa = nullptr;
  args.sb = scale;
  args.sb_dtype = sdt;
  args.bias = nullptr;
  args.bias_dtype = QL_F32;
  args.sa_n = 1;
  args.sb_n = N;
  args.M = M;
  args.N = N;
  args.k_elems_per_block = BK_BYTES / 2;
  args.num_kb = (int)(((int64_t)K * 2 + BK_BYTES - 1) / BK_BYTES);
  args.tiles_m = (M + BM - 1) / BM;
  args.tiles_n = 0;
  args.group_m = args.tiles_m;
  args.ldy = N;
  args.peer_mode = QL_PEER_NONE;
  args.rows_per_rank = 1;
  for (int r = 0; r < QL_MAX_PEERS; r++) args.owner_y[r] = nullptr;
  args.status = device_status_word();
  args.row_amax = nullptr;
  args.tma_store = 0;
  if (!args.status) return set_error(QL_ERR_CUDA, "linear_w8a16: could not allocate the device status word");
  WidenArgs w;
  w.raw = static_cast<const uint8_t *>(Wraw);
  w.wide = wide;
  w.ready = counters;
  w.N = N;
  w.K = K;
  return launch_gemm_pair<KIND, XT, PAIR_WIDEN>(X, wide, args, K, pairs, st, w);
}

int gemm16_widen_device(int dtype, const void *X, const void *Wraw, void *wide, int *counters, const void *scale, int sdt, void *Y,
                        int M, int N, int K, cudaStream_t st) {
  if (M <= 256 || N < 512 || K % 16 != 0 || !aligned16(Wraw) || !aligned16(wide) || !aligned16(X) || tuning().two_kernels)
    return QL_ERR_UNSUPPORTED;
  if (dtype == QL_BF16) return gemm16_widen_t<KIND_BF16, __nv_bfloat16>(X, Wraw, wide, counters, scale, sdt, Y, M, N, K, st);
  return gemm16_widen_t<KIND_F16, __half>(X, Wraw, wide, counters, scale, sdt, Y, M, N, K, st);
}

} // namespace ql

using namespace ql;

extern "C" {

int ql_gemm_fp8(const ql_tensor *xq, const ql_tensor *wq, const ql_tensor *sx, const ql_tensor *sw, ql_tensor *y, void *stream) {
  int rc = check_gemm("gemm_fp8", xq, wq, sx, sw, nullptr, y, QL_F8E4M3, QL_F8E4M3);
  if (rc != QL_OK) return rc;
  return run_gemm<KIND_F8>("gemm_fp8", xq, wq, sx, sw, nullptr, y, stream);
}

int ql_gemm_fp8_peer(const ql_tensor *xq, const ql_tensor *wq, const ql_tensor *sx, const ql_tensor *sw,
                     const ql_peer_buffer *dest, int32_t y_dtype, int64_t ldy, int64_t offset, int peer_mode, void *stream) {
  if (!dest || !xq || !wq) return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_fp8_peer: null argument");
  if (dest->world < 1 || dest->world > QL_MAX_PEERS || dest->rank < 0 || dest->rank >= dest->world)
    return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_fp8_peer: bad world / rank (%d / %d)", dest->world, dest->rank);
  if (peer_mode < QL_PEER_NONE || peer_mode > QL_PEER_ADD_OWNER)
    return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_fp8_peer: unknown peer mode %d", peer_mode);
  if (xq->rank != 2 || wq->rank != 2) return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_fp8_peer: operands must be 2-D");
  if (!(y_dtype == QL_BF16 || y_dtype == QL_F16)) return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_fp8_peer: y must be bf16 or f16");
  const int64_t M = xq->shape[0], N = wq->shape[0];
  char *base = static_cast<char *>((peer_mode == QL_PEER_STORE_ALL || peer_mode == QL_PEER_ADD_ALL) ? dest->all : dest->replica[dest->rank]);
  if (!base) return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_fp8_peer: the buffer has no address for this mode");
  if (offset < 0 || ldy < N) return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_fp8_peer: ldy (%lld) is smaller than N (%lld)", (long long)ldy, (long long)N);
  ql_tensor y{base + offset * 2, y_dtype, 2, {M, N}};
  int rc = check_gemm("gemm_fp8_peer", xq, wq, sx, sw, nullptr, &y, QL_F8E4M3, QL_F8E4M3);
  if (rc != QL_OK) return rc;
  if (peer_mode != QL_PEER_NONE) {
    // the peer writes exist as 16-byte vectors only
    if (N % 32 != 0 || ldy % 8 != 0 || offset % 8 != 0 || !aligned16(base))
      return set_error(QL_ERR_UNSUPPORTED, "gemm_fp8_peer: peer modes need N %% 32 == 0, ldy %% 8 == 0, offset %% 8 == 0 and a 16-byte aligned buffer");
  }
  if (peer_mode == QL_PEER_ADD_OWNER) {
    if (M % ((int64_t)dest->world * 128) != 0)
      return set_error(QL_ERR_UNSUPPORTED, "gemm_fp8_peer: add-to-owner needs M (%lld) to be a multiple of 128 x world", (long long)M);
    for (int r = 0; r < dest->world; r++)
      if (!dest->replica[r]) return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_fp8_peer: replica %d has no address", r);
  }
  return run_gemm<KIND_F8>("gemm_fp8_peer", xq, wq, sx, sw, nullptr, &y, stream, ldy, peer_mode, dest, offset);
}

// Gate/up projection of a gated MLP with SwiGLU done by the epilogue; see include/qlinear_b200.h.
int ql_gemm_fp8_swiglu(const ql_tensor *xq, const ql_tensor *wq, const ql_tensor *sx, const ql_tensor *sw, ql_tensor *act,
                       ql_tensor *row_amax, void *stream) {
  const char *op = "gemm_fp8_swiglu";
  if (!xq || !wq || !act || !row_amax) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  if (act->rank != 2 || wq->rank != 2 || act->shape[1] * 2 != wq->shape[0])
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: act must be [M, N/2] for interleaved gate/up weights [N, K]", op);
  if (!(act->dtype == QL_BF16 || act->dtype == QL_F16)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: act must be bf16 or f16", op);
  if (wq->shape[0] % 64 != 0) return set_error(QL_ERR_UNSUPPORTED, "%s: N (%lld) must be a multiple of 64 (gate and up interleaved in groups of 32)", op, (long long)wq->shape[0]);
  ql_tensor y{act->data, act->dtype, 2, {act->shape[0], wq->shape[0]}}; // the GEMM's logical result, never materialised
  int rc = check_gemm(op, xq, wq, sx, sw, nullptr, &y, QL_F8E4M3, QL_F8E4M3);
  if (rc != QL_OK) return rc;
  if (row_amax->dtype != QL_F32 || row_amax->rank != 1 || row_amax->shape[0] != act->shape[0] || (!row_amax->data && act->shape[0] > 0))
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: row_amax must be f32 [M]", op);
  if (act->shape[0] == 0 || act->shape[1] == 0) return QL_OK;
  QL_CUDA_TRY(cudaMemsetAsync(row_amax->data, 0, sizeof(float) * (size_t)act->shape[0], (cudaStream_t)stream));
  rc = run_gemm<KIND_F8>(op, xq, wq, sx, sw, nullptr, &y, stream, 0, QL_PEER_NONE, nullptr, 0, static_cast<float *>(row_amax->data));
  if (rc == QL_ERR_UNSUPPORTED)
    return set_error(QL_ERR_UNSUPPORTED, "%s: needs K (%lld) to be a non-zero multiple of 16 and 16-byte aligned operands", op, (long long)xq->shape[1]);
  return rc;
}

int ql_gemm_i8(const ql_tensor *xq, const ql_tensor *wq, const ql_tensor *sx, const ql_tensor *sw, ql_tensor *y, void *stream) {
  int rc = check_gemm("gemm_i8", xq, wq, sx, sw, nullptr, y, QL_I8, QL_I8);
  if (rc != QL_OK) return rc;
  return run_gemm<KIND_I8>("gemm_i8", xq, wq, sx, sw, nullptr, y, stream);
}

int ql_gemm_16(const ql_tensor *x, const ql_tensor *w, const ql_tensor *sw, ql_tensor *y, void *stream) {
  if (!x || !w) return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_16: null tensor");
  if (!(x->dtype == QL_BF16 || x->dtype == QL_F16)) return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_16: operands must be bf16 or f16");
  int rc = check_gemm("gemm_16", x, w, nullptr, sw, nullptr, y, x->dtype, x->dtype);
  if (rc != QL_OK) return rc;
  if (y->dtype != x->dtype) return set_error(QL_ERR_INVALID_ARGUMENT, "gemm_16: y must have the operands' type");
  if (x->dtype == QL_BF16) return run_gemm<KIND_BF16>("gemm_16", x, w, nullptr, sw, nullptr, y, stream);
  return run_gemm<KIND_F16>("gemm_16", x, w, nullptr, sw, nullptr, y, stream);
}

// Y = (X . W^T) * sx * sw + bias: the forward of tp.Linear (tripy/nvtripy/frontend/module/linear.py:127-151) after
// its quantize / dequantize pairs have been folded into scales.  X [M,K] and W [N,K] share one type
// (f32, f16, bf16, e4m3 or int8); Y is f32, f16 or bf16.
int ql_linear(const ql_tensor *x, const ql_tensor *w, const ql_tensor *sx, const ql_tensor *sw, const ql_tensor *bias, ql_tensor *y,
              void *stream) {
  if (!x || !w) return set_error(QL_ERR_INVALID_ARGUMENT, "linear: null tensor");
  const int d = x->dtype;
  if (!(is_float_dtype(d) || d == QL_F8E4M3 || d == QL_I8))
    return set_error(QL_ERR_INVALID_ARGUMENT, "linear: operands must be f32, f16, bf16, e4m3 or int8");
  int rc = check_gemm("linear", x, w, sx, sw, bias, y, d, d);
  if (rc != QL_OK) return rc;
  if (is_float_dtype(d) && y->dtype != d)
    return set_error(QL_ERR_INVALID_ARGUMENT, "linear: floating-point operands give a result of their own type"); // matmul.py:31-34
  switch (d) {
  case QL_F8E4M3: return run_gemm<KIND_F8>("linear", x, w, sx, sw, bias, y, stream);
  case QL_I8: return run_gemm<KIND_I8>("linear", x, w, sx, sw, bias, y, stream);
  case QL_BF16: return run_gemm<KIND_BF16>("linear", x, w, sx, sw, bias, y, stream);
  case QL_F16: return run_gemm<KIND_F16>("linear", x, w, sx, sw, bias, y, stream);
  default: return y->shape[0] == 0 || y->shape[1] == 0 ? QL_OK : run_simt(x, w, sx, sw, bias, y, stream);
  }
}

// C = A @ B (tensorrt.matrix_multiply with both operands kNONE, TensorRTOps.td:1986-2080; tp.matmul,
// tripy/nvtripy/frontend/ops/matmul.py:29-108): A [..., M, K], B [..., K, N], C [..., M, N], equal ranks >= 2, one
// float type.  Leading dimensions of an operand are either all equal to C's or all 1 (broadcast).
int ql_matmul(const ql_tensor *a, const ql_tensor *b, ql_tensor *c, void *stream) {
  const char *op = "matmul";
  if (!a || !b || !c) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null tensor", op);
  if (!is_float_dtype(a->dtype) || b->dtype != a->dtype || c->dtype != a->dtype)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: operands and result must share one of f32, f16, bf16", op);
  const int R = a->rank;
  if (R < 2 || R > QL_MAX_RANK || b->rank != R || c->rank != R)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: operands and result must have equal ranks >= 2", op);
  const int64_t M = a->shape[R - 2], K = a->shape[R - 1], N = b->shape[R - 1];
  if (b->shape[R - 2] != K || c->shape[R - 2] != M || c->shape[R - 1] != N)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: [..., %lld, %lld] @ [..., %lld, %lld] does not give [..., %lld, %lld]", op, (long long)M,
                     (long long)K, (long long)b->shape[R - 2], (long long)N, (long long)c->shape[R - 2], (long long)c->shape[R - 1]);
  int64_t batch = 1, a_lead = 1, b_lead = 1;
  for (int i = 0; i < R - 2; i++) {
    batch *= c->shape[i];
    a_lead *= a->shape[i];
    b_lead *= b->shape[i];
    if (!((a->shape[i] == c->shape[i] || a->shape[i] == 1) && (b->shape[i] == c->shape[i] || b->shape[i] == 1)))
      return set_error(QL_ERR_INVALID_ARGUMENT, "%s: leading dimension %d does not broadcast", op, i);
  }
  if (!((a_lead == batch || a_lead == 1) && (b_lead == batch || b_lead == 1)))
    return set_error(QL_ERR_UNSUPPORTED, "%s: leading dimensions of an operand must be all equal to the result's or all 1", op);
  if (batch == 0 || M == 0 || N == 0) return QL_OK;
  if (!a->data || !b->data || !c->data) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: tensor without a data pointer", op);
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || batch > INT32_MAX) return set_error(QL_ERR_UNSUPPORTED, "%s: dimension too large", op);
  return launch_gemm_simt(a->dtype, a->data, b->data, nullptr, 1, nullptr, 1, nullptr, QL_F32, c->data, c->dtype, (int)batch, (int)M, (int)N,
                          (int)K, K, 1, N, 1, N, a_lead == 1 ? 0 : M * K, b_lead == 1 ? 0 : K * N, M * N, (cudaStream_t)stream);
}

// Re-reads the QL_* tuning variables (they are otherwise read once, at the first GEMM of the process).
int ql_reload_tuning(void) {
  tuning() = read_tuning();
  wo_reload_tuning();
  w8_reload_tuning();
  f4_reload_tuning();
  return QL_OK;
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
