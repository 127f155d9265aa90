// NCCL communicators and collectives behind the C ABI: what the executor runtime's NCCL module offers its programs
// (executor/lib/Runtime/Backend/Lua/Modules/NCCL/NCCLModule.cpp:233-345 of the reference: __nccl_comm_init_rank,
// __nccl_comm_split, __nccl_all_reduce_<op>_<type>, __nccl_reduce_scatter_<op>_<type>, __nccl_all_gather,
// __nccl_all_to_all, __nccl_permute), with the reference's conventions: communicators are created non-blocking,
// and every call ends by polling ncclCommGetAsyncError until the communicator has left ncclInProgress or a time
// limit (5 s unless changed) has passed (NCCLModule.cpp:88-106), so a peer that never joins surfaces as an error
// status and not as a stuck host thread.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy the process already holds if there is one), so the
// library loads and everything else in it works on a machine without NCCL; these entry points then return
// QL_ERR_UNSUPPORTED.  The fused GEMM + collective kernels of this library do not use NCCL at all; this module is
// the plain collective a compiled program calls by name.
#include <chrono>
#include <cstring>
#include <dlfcn.h>
#include <mutex>

#include "ql_common.cuh"

#if __has_include(<nccl.h>)
#include <nccl.h>
#define QL_HAVE_NCCL_HEADER 1
#else
#define QL_HAVE_NCCL_HEADER 0
#endif

struct ql_nccl_comm {
  uint32_t magic;
  void *comm; // ncclComm_t
  int rank, num_ranks, device;
  int64_t timeout_ms;
};

namespace ql {
namespace {

constexpr uint32_t kCommMagic = 0x4e43434cu; // "NCCL"

#if QL_HAVE_NCCL_HEADER
struct NcclApi {
  void *handle = nullptr;
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRankConfig) CommInitRankConfig = nullptr;
  decltype(&ncclCommSplit) CommSplit = nullptr;
  decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  decltype(&ncclCommAbort) CommAbort = nullptr;
  decltype(&ncclCommUserRank) CommUserRank = nullptr;
  decltype(&ncclCommCount) CommCount = nullptr;
  decltype(&ncclAllReduce) AllReduce = nullptr;
  decltype(&ncclReduceScatter) ReduceScatter = nullptr;
  decltype(&ncclAllGather) AllGather = nullptr;
  decltype(&ncclSend) Send = nullptr;
  decltype(&ncclRecv) Recv = nullptr;
  decltype(&ncclGroupStart) GroupStart = nullptr;
  decltype(&ncclGroupEnd) GroupEnd = nullptr;
  decltype(&ncclGetErrorString) GetErrorString = nullptr;
  decltype(&ncclGetVersion) GetVersion = nullptr;
  bool ok = false;
};

NcclApi &api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    // the copy already mapped into the process (a framework's bundled NCCL) first, so that one process holds one NCCL
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!a.handle) a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!a.handle) a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!a.handle) return;
    bool all = true;
#define QL_BIND(member, symbol)                                                                \
  a.member = reinterpret_cast<decltype(a.member)>(dlsym(a.handle, symbol));                    \
  all = all && a.member != nullptr;
    QL_BIND(GetUniqueId, "ncclGetUniqueId")
    QL_BIND(CommInitRankConfig, "ncclCommInitRankConfig")
    QL_BIND(CommSplit, "ncclCommSplit")
    QL_BIND(CommGetAsyncError, "ncclCommGetAsyncError")
    QL_BIND(CommDestroy, "ncclCommDestroy")
    QL_BIND(CommAbort, "ncclCommAbort")
    QL_BIND(CommUserRank, "ncclCommUserRank")
    QL_BIND(CommCount, "ncclCommCount")
    QL_BIND(AllReduce, "ncclAllReduce")
    QL_BIND(ReduceScatter, "ncclReduceScatter")
    QL_BIND(AllGather, "ncclAllGather")
    QL_BIND(Send, "ncclSend")
    QL_BIND(Recv, "ncclRecv")
    QL_BIND(GroupStart, "ncclGroupStart")
    QL_BIND(GroupEnd, "ncclGroupEnd")
    QL_BIND(GetErrorString, "ncclGetErrorString")
    QL_BIND(GetVersion, "ncclGetVersion")
#undef QL_BIND
    a.ok = all;
  });
  return a;
}

int no_nccl() {
  return set_error(QL_ERR_UNSUPPORTED, "nccl: %s", api().handle ? "libnccl.so.2 lacks an entry point this module binds" : "libnccl.so.2 could not be loaded");
}

int nccl_error(ncclResult_t r, const char *what) {
  return set_error(QL_ERR_CUDA, "nccl: %s failed: %s", what, api().GetErrorString ? api().GetErrorString(r) : "?");
}

// Poll until the communicator has left ncclInProgress, or the limit has passed.
int wait_ready(void *comm, int64_t timeout_ms, const char *what) {
  const auto start = std::chrono::steady_clock::now();
  ncclResult_t state = ncclSuccess;
  for (;;) {
    ncclResult_t r = api().CommGetAsyncError(static_cast<ncclComm_t>(comm), &state);
    if (r != ncclSuccess) return nccl_error(r, "ncclCommGetAsyncError");
    if (state != ncclInProgress) break;
    const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - start).count();
    if (ms > timeout_ms)
      return set_error(QL_ERR_DEVICE_TIMEOUT, "nccl: %s: timed out after %lld ms waiting for the communicator", what, (long long)timeout_ms);
  }
  if (state != ncclSuccess) return set_error(QL_ERR_CUDA, "nccl: %s: asynchronous error: %s", what, api().GetErrorString(state));
  return QL_OK;
}

bool to_nccl_type(int dtype, ncclDataType_t *t) {
  switch (dtype) {
  case QL_F32: *t = ncclFloat32; return true;
  case QL_F16: *t = ncclFloat16; return true;
  case QL_BF16: *t = ncclBfloat16; return true;
  case QL_I8: *t = ncclInt8; return true;
  case QL_F8E4M3: *t = ncclUint8; return true; // moved as bytes (gather / all-to-all); never reduced
  default: return false;
  }
}

bool to_nccl_op(int op, ncclRedOp_t *o) {
  switch (op) {
  case QL_NCCL_SUM: *o = ncclSum; return true;
  case QL_NCCL_PROD: *o = ncclProd; return true;
  case QL_NCCL_MIN: *o = ncclMin; return true;
  case QL_NCCL_MAX: *o = ncclMax; return true;
  case QL_NCCL_AVG: *o = ncclAvg; return true;
  default: return false;
  }
}

int check_comm(const ql_nccl_comm *c, const char *what) {
  if (!c || c->magic != kCommMagic || !c->comm) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: %s: not a communicator", what);
  return QL_OK;
}

int finish_create(ncclComm_t comm, int device, int64_t timeout_ms, ql_nccl_comm **out, const char *what) {
  int rc = wait_ready(comm, timeout_ms, what);
  if (rc != QL_OK) {
    api().CommAbort(comm);
    return rc;
  }
  int rank = 0, n = 0;
  ncclResult_t r = api().CommUserRank(comm, &rank);
  if (r == ncclSuccess) r = api().CommCount(comm, &n);
  if (r != ncclSuccess) {
    api().CommAbort(comm);
    return nccl_error(r, what);
  }
  ql_nccl_comm *c = new ql_nccl_comm{kCommMagic, comm, rank, n, device, timeout_ms};
  *out = c;
  return QL_OK;
}
#endif // QL_HAVE_NCCL_HEADER

} // namespace
} // namespace ql

using namespace ql;

extern "C" {

#if QL_HAVE_NCCL_HEADER

int ql_nccl_version(int32_t *version) {
  if (!version) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: null argument");
  if (!api().ok) return no_nccl();
  int v = 0;
  ncclResult_t r = api().GetVersion(&v);
  if (r != ncclSuccess) return nccl_error(r, "ncclGetVersion");
  *version = v;
  return QL_OK;
}

int ql_nccl_unique_id(void *id) {
  if (!id) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: null argument");
  if (!api().ok) return no_nccl();
  static_assert(sizeof(ncclUniqueId) == QL_NCCL_UNIQUE_ID_BYTES, "unique id size");
  ncclUniqueId u;
  ncclResult_t r = api().GetUniqueId(&u);
  if (r != ncclSuccess) return nccl_error(r, "ncclGetUniqueId");
  memcpy(id, &u, sizeof(u));
  return QL_OK;
}

int ql_nccl_comm_init_rank(int32_t rank, int32_t num_ranks, int32_t device, const void *id, int64_t timeout_ms, ql_nccl_comm **out) {
  if (!id || !out) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: null argument");
  if (num_ranks < 1 || rank < 0 || rank >= num_ranks) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: rank %d of %d", rank, num_ranks);
  if (!api().ok) return no_nccl();
  if (timeout_ms <= 0) timeout_ms = 5000;
  QL_CUDA_TRY(cudaSetDevice(device));
  ncclUniqueId u;
  memcpy(&u, id, sizeof(u));
  ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
  config.blocking = 0;
  ncclComm_t comm = nullptr;
  ncclResult_t r = api().CommInitRankConfig(&comm, num_ranks, u, rank, &config);
  if (r != ncclSuccess && r != ncclInProgress) return nccl_error(r, "ncclCommInitRankConfig");
  return finish_create(comm, device, timeout_ms, out, "comm_init_rank");
}

int ql_nccl_comm_split(ql_nccl_comm *parent, int32_t color, int32_t key, ql_nccl_comm **out) {
  int rc = check_comm(parent, "comm_split");
  if (rc != QL_OK) return rc;
  if (!out) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: null argument");
  // the source communicator has to be ready before it is split (NCCLModule.cpp:183-197)
  if ((rc = wait_ready(parent->comm, parent->timeout_ms, "comm_split")) != QL_OK) return rc;
  ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
  config.blocking = 0;
  config.splitShare = 1;
  ncclComm_t child = nullptr;
  ncclResult_t r = api().CommSplit(static_cast<ncclComm_t>(parent->comm), color, key, &child, &config);
  if (r != ncclSuccess && r != ncclInProgress) return nccl_error(r, "ncclCommSplit");
  if ((rc = wait_ready(parent->comm, parent->timeout_ms, "comm_split")) != QL_OK) return rc;
  if (!child) { // color was NCCL_SPLIT_NOCOLOR: this rank is in no new communicator
    *out = nullptr;
    return QL_OK;
  }
  return finish_create(child, parent->device, parent->timeout_ms, out, "comm_split");
}

int ql_nccl_comm_rank(const ql_nccl_comm *c, int32_t *rank, int32_t *num_ranks) {
  int rc = check_comm(c, "comm_rank");
  if (rc != QL_OK) return rc;
  if (rank) *rank = c->rank;
  if (num_ranks) *num_ranks = c->num_ranks;
  return QL_OK;
}

int ql_nccl_comm_destroy(ql_nccl_comm *c) {
  if (!c) return QL_OK;
  int rc = check_comm(c, "comm_destroy");
  if (rc != QL_OK) return rc;
  // a communicator that is not healthy is aborted, not finalized
  rc = wait_ready(c->comm, c->timeout_ms, "comm_destroy");
  ncclResult_t r = rc == QL_OK ? api().CommDestroy(static_cast<ncclComm_t>(c->comm)) : api().CommAbort(static_cast<ncclComm_t>(c->comm));
  c->magic = 0;
  c->comm = nullptr;
  delete c;
  if (rc != QL_OK) return rc;
  if (r != ncclSuccess && r != ncclInProgress) return nccl_error(r, "ncclCommDestroy");
  return QL_OK;
}

int ql_nccl_all_reduce(ql_nccl_comm *c, const void *send, void *recv, uint64_t count, int32_t dtype, int32_t op, void *stream) {
  int rc = check_comm(c, "all_reduce");
  if (rc != QL_OK) return rc;
  ncclDataType_t t;
  ncclRedOp_t o;
  if (!to_nccl_type(dtype, &t) || dtype == QL_F8E4M3) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: all_reduce: unsupported element type %d", dtype);
  if (!to_nccl_op(op, &o)) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: all_reduce: unknown reduction %d", op);
  if (count && (!send || !recv)) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: all_reduce: null buffer");
  ncclResult_t r = api().AllReduce(send, recv, count, t, o, static_cast<ncclComm_t>(c->comm), static_cast<cudaStream_t>(stream));
  if (r != ncclSuccess && r != ncclInProgress) return nccl_error(r, "ncclAllReduce");
  count_launches(1);
  return wait_ready(c->comm, c->timeout_ms, "all_reduce");
}

int ql_nccl_reduce_scatter(ql_nccl_comm *c, const void *send, void *recv, uint64_t recv_count, int32_t dtype, int32_t op, void *stream) {
  int rc = check_comm(c, "reduce_scatter");
  if (rc != QL_OK) return rc;
  ncclDataType_t t;
  ncclRedOp_t o;
  if (!to_nccl_type(dtype, &t) || dtype == QL_F8E4M3) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: reduce_scatter: unsupported element type %d", dtype);
  if (!to_nccl_op(op, &o)) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: reduce_scatter: unknown reduction %d", op);
  if (recv_count && (!send || !recv)) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: reduce_scatter: null buffer");
  ncclResult_t r = api().ReduceScatter(send, recv, recv_count, t, o, static_cast<ncclComm_t>(c->comm), static_cast<cudaStream_t>(stream));
  if (r != ncclSuccess && r != ncclInProgress) return nccl_error(r, "ncclReduceScatter");
  count_launches(1);
  return wait_ready(c->comm, c->timeout_ms, "reduce_scatter");
}

int ql_nccl_all_gather(ql_nccl_comm *c, const void *send, void *recv, uint64_t send_bytes, void *stream) {
  int rc = check_comm(c, "all_gather");
  if (rc != QL_OK) return rc;
  if (send_bytes && (!send || !recv)) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: all_gather: null buffer");
  ncclResult_t r = api().AllGather(send, recv, send_bytes, ncclInt8, static_cast<ncclComm_t>(c->comm), static_cast<cudaStream_t>(stream));
  if (r != ncclSuccess && r != ncclInProgress) return nccl_error(r, "ncclAllGather");
  count_launches(1);
  return wait_ready(c->comm, c->timeout_ms, "all_gather");
}

int ql_nccl_all_to_all(ql_nccl_comm *c, const void *send, void *recv, uint64_t total_bytes, void *stream) {
  int rc = check_comm(c, "all_to_all");
  if (rc != QL_OK) return rc;
  if (total_bytes % (uint64_t)c->num_ranks != 0)
    return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: all_to_all: %llu bytes do not divide over %d ranks", (unsigned long long)total_bytes, c->num_ranks);
  if (total_bytes && (!send || !recv)) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: all_to_all: null buffer");
  const uint64_t each = total_bytes / (uint64_t)c->num_ranks;
  ncclComm_t comm = static_cast<ncclComm_t>(c->comm);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ncclResult_t r = api().GroupStart();
  for (int p = 0; p < c->num_ranks && (r == ncclSuccess || r == ncclInProgress); p++) {
    r = api().Send(static_cast<const char *>(send) + p * each, each, ncclInt8, p, comm, st);
    if (r == ncclSuccess || r == ncclInProgress) r = api().Recv(static_cast<char *>(recv) + p * each, each, ncclInt8, p, comm, st);
  }
  ncclResult_t e = api().GroupEnd();
  if (r != ncclSuccess && r != ncclInProgress) return nccl_error(r, "ncclSend / ncclRecv");
  if (e != ncclSuccess && e != ncclInProgress) return nccl_error(e, "ncclGroupEnd");
  count_launches(1);
  return wait_ready(c->comm, c->timeout_ms, "all_to_all");
}

int ql_nccl_permute(ql_nccl_comm *c, const void *send, void *recv, int32_t send_to, int32_t recv_from, uint64_t bytes, void *stream) {
  int rc = check_comm(c, "permute");
  if (rc != QL_OK) return rc;
  if (send_to >= c->num_ranks || recv_from >= c->num_ranks) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: permute: peer out of range");
  ncclComm_t comm = static_cast<ncclComm_t>(c->comm);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // a negative peer means this rank does not send (or does not receive), as in a collective permute with gaps; a
  // rank that receives nothing gets zeros (NCCLModule.cpp:360-366)
  if (recv_from < 0 && bytes) {
    if (!recv) return set_error(QL_ERR_INVALID_ARGUMENT, "nccl: permute: null buffer");
    QL_CUDA_TRY(cudaMemsetAsync(recv, 0, bytes, st));
  }
  ncclResult_t r = api().GroupStart();
  if (send_to >= 0 && (r == ncclSuccess || r == ncclInProgress)) r = api().Send(send, bytes, ncclInt8, send_to, comm, st);
  if (recv_from >= 0 && (r == ncclSuccess || r == ncclInProgress)) r = api().Recv(recv, bytes, ncclInt8, recv_from, comm, st);
  ncclResult_t e = api().GroupEnd();
  if (r != ncclSuccess && r != ncclInProgress) return nccl_error(r, "ncclSend / ncclRecv");
  if (e != ncclSuccess && e != ncclInProgress) return nccl_error(e, "ncclGroupEnd");
  count_launches(1);
  return wait_ready(c->comm, c->timeout_ms, "permute");
}

#else // no nccl.h when the library was built

static int built_without() { return set_error(QL_ERR_UNSUPPORTED, "nccl: the library was built without nccl.h"); }
int ql_nccl_version(int32_t *) { return built_without(); }
int ql_nccl_unique_id(void *) { return built_without(); }
int ql_nccl_comm_init_rank(int32_t, int32_t, int32_t, const void *, int64_t, ql_nccl_comm **) { return built_without(); }
int ql_nccl_comm_split(ql_nccl_comm *, int32_t, int32_t, ql_nccl_comm **) { return built_without(); }
int ql_nccl_comm_rank(const ql_nccl_comm *, int32_t *, int32_t *) { return built_without(); }
int ql_nccl_comm_destroy(ql_nccl_comm *) { return built_without(); }
int ql_nccl_all_reduce(ql_nccl_comm *, const void *, void *, uint64_t, int32_t, int32_t, void *) { return built_without(); }
int ql_nccl_reduce_scatter(ql_nccl_comm *, const void *, void *, uint64_t, int32_t, int32_t, void *) { return built_without(); }
int ql_nccl_all_gather(ql_nccl_comm *, const void *, void *, uint64_t, void *) { return built_without(); }
int ql_nccl_all_to_all(ql_nccl_comm *, const void *, void *, uint64_t, void *) { return built_without(); }
int ql_nccl_permute(ql_nccl_comm *, const void *, void *, int32_t, int32_t, uint64_t, void *) { return built_without(); }

#endif

} // extern "C"
