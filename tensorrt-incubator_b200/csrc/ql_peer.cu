// Cross-GPU helpers of the fused GEMM + collective path: a barrier between the ranks of one box and a
// broadcast of a rank's rows to every replica.  One process per GPU; each rank launches these on its own
// GPU, so the barrier's ranks never share a device.  The reference has no multi-GPU execution of this path.
#include <atomic>

#include "ql_common.cuh"

namespace ql {
namespace {

constexpr long long kPeerWaitLimitCycles = 1ll << 34; // about ten seconds: ranks are separate processes
constexpr int ST_TIMEOUT_PEER = 7;
std::atomic<long long> g_peer_wait_limit{kPeerWaitLimitCycles};

struct FlagPtrs {
  uint32_t *flags[QL_MAX_PEERS];
};

// flags (per rank, uint32): [0, world) = the barrier number each peer has reached, written by that peer;
// [world] = how many barriers this rank has entered (touched by this kernel only).
__global__ void peer_barrier_kernel(FlagPtrs p, int world, int rank, int *status, long long limit_cycles) {
  __shared__ uint32_t epoch_s;
  const int t = threadIdx.x;
  if (t == 0) {
    epoch_s = p.flags[rank][world] + 1;
    p.flags[rank][world] = epoch_s;
  }
  __syncthreads();
  const uint32_t epoch = epoch_s;
  if (t < world) {
    // everything this GPU did before the barrier (earlier kernels of the stream) is ordered before the flag
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[t] + rank), "r"(epoch) : "memory");
    const uint32_t *mine = p.flags[rank] + t;
    const long long t0 = clock64();
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if (clock64() - t0 > limit_cycles) { // a peer never arrived: record it and let the stream go on
        atomicCAS(status, 0, ST_TIMEOUT_PEER);
        break;
      }
      __nanosleep(64);
    }
    __threadfence_system();
  }
  __syncthreads();
}

__global__ void peer_broadcast_kernel(const uint4 *__restrict__ src, uint4 *dst_all, int64_t n16) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint4 v = __ldcs(src + i);
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst_all + i), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
  }
}

// In-switch all-reduce of one rank's share of a buffer: `multimem.ld_reduce` makes the NVSwitch fetch the same 16
// bytes from every replica and add them (f32 accumulation, one rounding), `multimem.st` writes the sum back into
// every replica.  Every rank runs this on a disjoint range, between two barriers.
template <bool kHalf>
__global__ void peer_reduce_kernel(uint4 *all, int64_t n16) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    uint32_t a, b, c, d;
    if (kHalf)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(all + i) : "memory");
    else
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(all + i) : "memory");
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(all + i), "f"(__uint_as_float(a)),
                 "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
                 : "memory");
  }
}

int check_peer(const char *op, const ql_peer_buffer *b) {
  if (!b) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: null buffer", op);
  if (b->world < 1 || b->world > QL_MAX_PEERS || b->rank < 0 || b->rank >= b->world)
    return set_error(QL_ERR_INVALID_ARGUMENT, "%s: bad world / rank (%d / %d)", op, b->world, b->rank);
  for (int r = 0; r < b->world; r++)
    if (!b->replica[r]) return set_error(QL_ERR_INVALID_ARGUMENT, "%s: replica %d has no address", op, r);
  return QL_OK;
}

} // namespace
} // namespace ql

using namespace ql;

extern "C" {

int ql_peer_barrier(const ql_peer_buffer *flags, void *stream) {
  int rc = check_peer("peer_barrier", flags);
  if (rc != QL_OK) return rc;
  int *status = device_status_word();
  if (!status) return set_error(QL_ERR_CUDA, "peer_barrier: could not allocate the device status word");
  FlagPtrs p;
  for (int r = 0; r < QL_MAX_PEERS; r++) p.flags[r] = r < flags->world ? static_cast<uint32_t *>(flags->replica[r]) : nullptr;
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(p, flags->world, flags->rank, status, g_peer_wait_limit.load(std::memory_order_relaxed));
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

int ql_set_peer_wait_limit(int64_t cycles) {
  g_peer_wait_limit.store(cycles > 0 ? (long long)cycles : kPeerWaitLimitCycles, std::memory_order_relaxed);
  return QL_OK;
}

int ql_peer_reduce(const ql_peer_buffer *buf, int32_t dtype, int64_t offset, int64_t bytes, void *stream) {
  int rc = check_peer("peer_reduce", buf);
  if (rc != QL_OK) return rc;
  if (!buf->all) return set_error(QL_ERR_INVALID_ARGUMENT, "peer_reduce: the buffer has no replication address");
  if (dtype != QL_BF16 && dtype != QL_F16) return set_error(QL_ERR_INVALID_ARGUMENT, "peer_reduce: elements must be bf16 or f16");
  if (offset < 0 || bytes < 0 || offset % 16 != 0 || bytes % 16 != 0)
    return set_error(QL_ERR_INVALID_ARGUMENT, "peer_reduce: offset and size must be multiples of 16 bytes");
  if (bytes == 0) return QL_OK;
  const int64_t n16 = bytes / 16;
  uint4 *all = reinterpret_cast<uint4 *>(static_cast<char *>(buf->all) + offset);
  int64_t blocks = (n16 + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (dtype == QL_F16) peer_reduce_kernel<true><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(all, n16);
  else peer_reduce_kernel<false><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(all, n16);
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}

int ql_peer_broadcast(const ql_peer_buffer *buf, int64_t offset, int64_t bytes, void *stream) {
  int rc = check_peer("peer_broadcast", buf);
  if (rc != QL_OK) return rc;
  if (!buf->all) return set_error(QL_ERR_INVALID_ARGUMENT, "peer_broadcast: the buffer has no replication address");
  if (offset < 0 || bytes < 0 || offset % 16 != 0 || bytes % 16 != 0)
    return set_error(QL_ERR_INVALID_ARGUMENT, "peer_broadcast: offset and size must be multiples of 16 bytes");
  if (bytes == 0) return QL_OK;
  const int64_t n16 = bytes / 16;
  const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const char *>(buf->replica[buf->rank]) + offset);
  uint4 *dst = reinterpret_cast<uint4 *>(static_cast<char *>(buf->all) + offset);
  int64_t blocks = (n16 + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  peer_broadcast_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(src, dst, n16);
  count_launches(1);
  QL_CUDA_TRY(cudaGetLastError());
  return QL_OK;
}
}
