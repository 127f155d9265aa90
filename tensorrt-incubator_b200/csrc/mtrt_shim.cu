// The executor runtime's CUDA module behind the reference's own symbols (mtrt_cuda_*), so that
// host code generated for the reference runs unchanged while the hot kernels come from this
// library.  Reference implementation this stands in for:
// mlir-tensorrt/executor/lib/Runtime/Backend/C/CUDAModule.cpp (module load / get function /
// launch / streams / events / allocation).
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "mtrt_cuda_module.h"
#include "ql_common.cuh"

namespace {

thread_local char g_mtrt_error[512] = "";

void fail(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_mtrt_error, sizeof(g_mtrt_error), fmt, ap);
  va_end(ap);
  fprintf(stderr, "mtrt_cuda: %s\n", g_mtrt_error);
}

#define RT_TRY(expr, ret)                                                                          \
  do {                                                                                             \
    cudaError_t _e = (expr);                                                                       \
    if (_e != cudaSuccess) {                                                                       \
      fail("%s: %s", #expr, cudaGetErrorString(_e));                                               \
      return ret;                                                                                  \
    }                                                                                              \
  } while (0)

// ---- driver entry points, resolved at run time so that the library loads without a driver ----
struct Driver {
  CUresult (*moduleLoadDataEx)(CUmodule *, const void *, unsigned, CUjit_option *, void **) = nullptr;
  CUresult (*moduleUnload)(CUmodule) = nullptr;
  CUresult (*moduleGetFunction)(CUfunction *, CUmodule, const char *) = nullptr;
  CUresult (*launchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                           void **, void **) = nullptr;
  CUresult (*getErrorString)(CUresult, const char **) = nullptr;
  bool ok = false;
};

Driver &driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [](const char *name, void **fn) {
      cudaDriverEntryPointQueryResult q;
      return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess && *fn;
    };
    d.ok = get("cuModuleLoadDataEx", (void **)&d.moduleLoadDataEx) && get("cuModuleUnload", (void **)&d.moduleUnload) &&
           get("cuModuleGetFunction", (void **)&d.moduleGetFunction) && get("cuLaunchKernel", (void **)&d.launchKernel) &&
           get("cuGetErrorString", (void **)&d.getErrorString);
  });
  return d;
}

const char *drv_msg(CUresult r) {
  const char *m = "unknown driver error";
  if (driver().getErrorString) driver().getErrorString(r, &m);
  return m ? m : "unknown driver error";
}

// ---- handles ----------------------------------------------------------------------------------
constexpr uint32_t kModuleMagic = 0x514C4D4Fu, kFunctionMagic = 0x514C464Eu;

struct OpSpec {
  std::string op;
  std::map<std::string, std::string> kv;
};

struct ShimFunction {
  uint32_t magic = kFunctionMagic;
  bool library = false;
  OpSpec spec;         // library kernels
  CUfunction fn = nullptr; // JIT-compiled kernels
};

struct ShimModule {
  uint32_t magic = kModuleMagic;
  std::string ptx;
  CUmodule jit = nullptr;
  std::vector<ShimFunction *> functions;
};

std::mutex g_alias_mutex;
std::map<std::string, std::string> g_aliases;
bool g_manifest_read = false;

void read_manifest_once() {
  if (g_manifest_read) return;
  g_manifest_read = true;
  const char *path = getenv("QL_MTRT_MANIFEST");
  if (!path) return;
  std::ifstream f(path);
  std::string line;
  while (std::getline(f, line)) {
    size_t eq = line.find('=');
    if (eq == std::string::npos || line[0] == '#') continue;
    auto trim = [](std::string s) {
      size_t a = s.find_first_not_of(" \t\r"), b = s.find_last_not_of(" \t\r");
      return a == std::string::npos ? std::string() : s.substr(a, b - a + 1);
    };
    // split at the first '=' that follows the kernel name (specs contain '=' themselves)
    g_aliases[trim(line.substr(0, eq))] = trim(line.substr(eq + 1));
  }
}

bool parse_spec(const std::string &text, OpSpec *out) {
  if (text.rfind("ql:", 0) != 0) return false;
  std::stringstream ss(text.substr(3));
  std::string item;
  bool first = true;
  while (std::getline(ss, item, ';')) {
    if (first) { out->op = item; first = false; continue; }
    size_t eq = item.find('=');
    if (eq == std::string::npos) return false;
    out->kv[item.substr(0, eq)] = item.substr(eq + 1);
  }
  return !out->op.empty();
}

int dtype_of(const std::string &s) {
  if (s == "f32") return QL_F32;
  if (s == "f16") return QL_F16;
  if (s == "bf16") return QL_BF16;
  if (s == "i8") return QL_I8;
  if (s == "i4") return QL_I4;
  if (s == "f8" || s == "f8E4M3FN") return QL_F8E4M3;
  if (s == "f4" || s == "f4E2M1FN") return QL_F4E2M1;
  return -1;
}

std::string get(const OpSpec &s, const char *k, const char *dflt = "") {
  auto it = s.kv.find(k);
  return it == s.kv.end() ? std::string(dflt) : it->second;
}

// args[i] points at the i-th kernel parameter.  A memref parameter arrives unpacked, as the compiler's launch
// convention lays it out (compiler/lib/Passes/1_Core/KernelToCUDA/KernelToCUDA.cpp:94-108): the aligned base
// pointer, then -- only where they are not compile-time constants -- the offset, every dynamic size and every
// dynamic stride, each an `index` (i64).  In a kernel spec a dynamic dimension is written `?` (shape=?x4096,
// M=?); for the dense row-major memrefs these kernels take, the offset is the constant 0 and stride i is dynamic
// exactly when a dimension to its right is, so the cursor below knows how many values follow each pointer.
struct ArgCursor {
  void **args;
  int next;
  bool ok;
  void *pointer() { return *reinterpret_cast<void **>(args[next++]); }
  int64_t index() { return *reinterpret_cast<int64_t *>(args[next++]); }
  // Fills t->data and resolves the `?` dimensions of t (marked by -1) from the arguments.
  void memref(ql_tensor *t) {
    t->data = pointer();
    bool dynamic_right[QL_MAX_RANK + 1] = {false};
    for (int i = t->rank - 1; i >= 0; i--) dynamic_right[i] = dynamic_right[i + 1] || t->shape[i] < 0;
    for (int i = 0; i < t->rank; i++)
      if (t->shape[i] < 0) {
        t->shape[i] = index();
        if (t->shape[i] < 0) ok = false;
      }
    // the dynamic strides follow the sizes, outermost first; each must be the dense one
    int64_t expect[QL_MAX_RANK];
    int64_t run = 1;
    for (int i = t->rank - 1; i >= 0; i--) {
      expect[i] = run;
      run *= t->shape[i];
    }
    for (int i = 0; i < t->rank; i++)
      if (dynamic_right[i + 1] && index() != expect[i]) ok = false;
  }
};

bool shape_spec(const std::string &s, ql_tensor *t) { // "4096x4096", "?x4096" (`?` = -1, resolved from the arguments), "" = scalar
  t->rank = 0;
  if (s.empty() || s == "scalar") return true;
  std::stringstream ss(s);
  std::string d;
  while (std::getline(ss, d, 'x')) {
    if (t->rank >= QL_MAX_RANK) return false;
    t->shape[t->rank++] = (d == "?") ? -1 : atoll(d.c_str());
  }
  return true;
}

int64_t dim_spec(const std::string &v) { return v == "?" ? -1 : atoll(v.c_str()); }

void launch_library_kernel(const OpSpec &s, CUstream stream, void **args) {
  int rc = QL_OK;
  ArgCursor cur{args, 0, true};
  const char *strided = "a memref argument is not dense row-major (dynamic stride differs from the dense one) or has a negative size";
  if (s.op == "quantize" || s.op == "dequantize") {
    ql_tensor in{}, sc{}, out{};
    in.dtype = dtype_of(get(s, "in"));
    out.dtype = dtype_of(get(s, "out"));
    sc.dtype = dtype_of(get(s, "scale", "f32"));
    if (!shape_spec(get(s, "shape"), &in)) return fail("bad shape in kernel spec");
    out.rank = in.rank;
    memcpy(out.shape, in.shape, sizeof(in.shape));
    ql_qdq_attrs at{};
    std::string axis = get(s, "axis");
    if (!axis.empty()) {
      at.has_axis = 1;
      at.axis = atoi(axis.c_str());
      sc.rank = 1;
      sc.shape[0] = (at.axis >= 0 && at.axis < in.rank) ? in.shape[at.axis] : 0;
    } else if (!shape_spec(get(s, "scale_shape"), &sc)) {
      return fail("bad scale_shape in kernel spec");
    }
    std::string mode = get(s, "fp8_mode", "direct");
    at.fp8_mode = mode == "via_f16" ? QL_FP8_VIA_F16 : mode == "stablehlo" ? QL_FP8_STABLEHLO : QL_FP8_DIRECT;
    cur.memref(&in);
    cur.memref(&sc);
    cur.memref(&out);
    if (!cur.ok) return fail("%s", strided);
    rc = (s.op == "quantize") ? ql_quantize(&in, &sc, &out, &at, stream) : ql_dequantize(&in, &sc, &out, &at, stream);
  } else if (s.op == "linear_w8a16" || s.op == "linear_w4a16") {
    const int64_t M = dim_spec(get(s, "M")), N = atoll(get(s, "N").c_str()), K = atoll(get(s, "K").c_str());
    const int xd = dtype_of(get(s, "x", "bf16"));
    ql_tensor x{nullptr, xd, 2, {M, K}}, y{nullptr, xd, 2, {M, N}}, w{nullptr, s.op == "linear_w8a16" ? QL_I8 : QL_I4, 2, {N, K}}, sc{};
    sc.dtype = dtype_of(get(s, "scale", "f16"));
    if (s.op == "linear_w8a16") {
      sc.rank = 1;
      sc.shape[0] = N;
    } else {
      const int64_t B = atoll(get(s, "block", "128").c_str());
      sc.rank = 2;
      sc.shape[0] = N;
      sc.shape[1] = B > 0 ? K / B : 0;
    }
    cur.memref(&x);
    cur.memref(&w);
    cur.memref(&sc);
    cur.memref(&y);
    if (!cur.ok) return fail("%s", strided);
    rc = s.op == "linear_w8a16" ? ql_linear_w8a16(&x, &w, &sc, &y, stream) : ql_linear_w4a16(&x, &w, &sc, &y, stream);
  } else if (s.op == "gemm_fp8" || s.op == "gemm_i8") {
    const int64_t M = dim_spec(get(s, "M")), N = atoll(get(s, "N").c_str()), K = atoll(get(s, "K").c_str());
    const int qd = s.op == "gemm_fp8" ? QL_F8E4M3 : QL_I8;
    const int64_t nsx = dim_spec(get(s, "sx", "1")), nsw = atoll(get(s, "sw", "1").c_str());
    ql_tensor x{nullptr, qd, 2, {M, K}}, w{nullptr, qd, 2, {N, K}};
    ql_tensor sx{nullptr, QL_F32, nsx == 1 ? 0 : 1, {nsx}}, sw{nullptr, QL_F32, nsw == 1 ? 0 : 1, {nsw}};
    ql_tensor y{nullptr, dtype_of(get(s, "out", "bf16")), 2, {M, N}};
    cur.memref(&x);
    cur.memref(&w);
    cur.memref(&sx);
    cur.memref(&sw);
    cur.memref(&y);
    if (!cur.ok) return fail("%s", strided);
    rc = s.op == "gemm_fp8" ? ql_gemm_fp8(&x, &w, &sx, &sw, &y, stream) : ql_gemm_i8(&x, &w, &sx, &sw, &y, stream);
  } else if (s.op == "dynamic_quantize") {
    // args: input, double_quant_scale (rank 0), result (f4), scales (f8)
    ql_tensor in{}, gs{}, out{}, sc{};
    in.dtype = dtype_of(get(s, "in", "f32"));
    gs.dtype = dtype_of(get(s, "scale", "f32"));
    out.dtype = QL_F4E2M1;
    sc.dtype = QL_F8E4M3;
    if (!shape_spec(get(s, "shape"), &in) || in.rank < 1) return fail("bad shape in kernel spec");
    const int axis = atoi(get(s, "axis", "-1").c_str());
    const int ax = axis < 0 ? in.rank + axis : axis;
    out.rank = sc.rank = in.rank;
    memcpy(out.shape, in.shape, sizeof(in.shape));
    memcpy(sc.shape, in.shape, sizeof(in.shape));
    if (ax >= 0 && ax < in.rank && in.shape[ax] >= 0) sc.shape[ax] = in.shape[ax] / 16;
    cur.memref(&in);
    cur.memref(&gs);
    cur.memref(&out);
    cur.memref(&sc);
    if (!cur.ok) return fail("%s", strided);
    rc = ql_dynamic_quantize(&in, &gs, ax, atoi(get(s, "block_size", "16").c_str()), &out, &sc, stream);
  } else {
    return fail("unknown library kernel '%s'", s.op.c_str());
  }
  if (rc != QL_OK) fail("%s", ql_last_error());
}

ShimModule *as_module(CUmodule m) {
  ShimModule *sm = reinterpret_cast<ShimModule *>(m);
  return (sm && sm->magic == kModuleMagic) ? sm : nullptr;
}

} // namespace

extern "C" {

const char *mtrt_cuda_last_error() { return g_mtrt_error; }

int32_t ql_mtrt_bind_kernel(const char *kernel_name, const char *op_spec) {
  OpSpec s;
  if (!kernel_name || !op_spec || !parse_spec(op_spec, &s)) {
    fail("bind_kernel: the spec must look like \"ql:<op>;key=value;...\"");
    return 1;
  }
  std::lock_guard<std::mutex> lock(g_alias_mutex);
  g_aliases[kernel_name] = op_spec;
  return 0;
}

int32_t mtrt_cuda_get_active_device() {
  int32_t d = 0;
  RT_TRY(cudaGetDevice(&d), 0);
  return d;
}
int32_t mtrt_cuda_set_active_device(int32_t device) {
  RT_TRY(cudaSetDevice(device), 0);
  return device;
}
int32_t mtrt_cuda_get_device(int32_t device) {
  int n = 0;
  RT_TRY(cudaGetDeviceCount(&n), 0);
  if (device < 0 || device >= n) {
    fail("device %d out of range (%d devices)", device, n);
    return 0;
  }
  return device;
}
int32_t mtrt_cuda_get_current_device() { return mtrt_cuda_get_active_device(); }
int32_t mtrt_cuda_get_program_device(int32_t logicalId) {
  if (logicalId != 0) fail("only single-device programs are supported (logical device %d)", logicalId);
  return mtrt_cuda_get_active_device();
}

CUstream mtrt_cuda_stream_create() {
  cudaStream_t s = nullptr;
  RT_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), nullptr);
  return reinterpret_cast<CUstream>(s);
}
void mtrt_cuda_stream_destroy(CUstream stream) { RT_TRY(cudaStreamDestroy(reinterpret_cast<cudaStream_t>(stream)), ); }
void mtrt_cuda_stream_sync(CUstream stream) { RT_TRY(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)), ); }

cudaEvent_t mtrt_cuda_event_create(int32_t device) {
  int prev = 0;
  RT_TRY(cudaGetDevice(&prev), nullptr);
  if (device != prev) RT_TRY(cudaSetDevice(device), nullptr);
  cudaEvent_t e = nullptr;
  cudaError_t err = cudaEventCreate(&e);
  if (device != prev) cudaSetDevice(prev);
  RT_TRY(err, nullptr);
  return e;
}
void mtrt_cuda_event_release(cudaEvent_t event) { RT_TRY(cudaEventDestroy(event), ); }
void mtrt_cuda_stream_record_event(CUstream stream, cudaEvent_t event) {
  RT_TRY(cudaEventRecord(event, reinterpret_cast<cudaStream_t>(stream)), );
}
void mtrt_cuda_stream_wait_event(CUstream stream, cudaEvent_t event) {
  RT_TRY(cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(stream), event, 0), );
}
void mtrt_cuda_event_sync(cudaEvent_t event) { RT_TRY(cudaEventSynchronize(event), ); }
float mtrt_cuda_event_elapsed_msec(cudaEvent_t start, cudaEvent_t end) {
  float ms = 0.f;
  RT_TRY(cudaEventElapsedTime(&ms, start, end), 0.f);
  return ms;
}

void *mtrt_cuda_alloc_async(CUstream stream, int64_t size, int32_t alignment, int8_t isHostPinned, int8_t isManaged) {
  (void)alignment; // every CUDA allocation is aligned to at least 256 bytes
  void *p = nullptr;
  if (isHostPinned) {
    RT_TRY(cudaHostAlloc(&p, (size_t)size, cudaHostAllocDefault), nullptr);
  } else if (isManaged) {
    RT_TRY(cudaMallocManaged(&p, (size_t)size), nullptr);
  } else {
    ql::keep_scratch_pool_warm();
    RT_TRY(cudaMallocAsync(&p, (size_t)size, reinterpret_cast<cudaStream_t>(stream)), nullptr);
  }
  return p;
}
void mtrt_cuda_memcpy_async(CUstream stream, void *src, void *dest, int64_t size) {
  RT_TRY(cudaMemcpyAsync(dest, src, (size_t)size, cudaMemcpyDefault, reinterpret_cast<cudaStream_t>(stream)), );
}
void mtrt_cuda_free(CUstream stream, void *ptr, int8_t isHostPinned, int8_t isManaged) {
  if (isHostPinned) RT_TRY(cudaFreeHost(ptr), );
  else if (isManaged) RT_TRY(cudaFree(ptr), );
  else RT_TRY(cudaFreeAsync(ptr, reinterpret_cast<cudaStream_t>(stream)), );
}

CUmodule mtrt_cuda_module_load_from_ptx(const char *ptxData, size_t ptxLen) {
  if (!ptxData && ptxLen) {
    fail("module_load_from_ptx: null data");
    return nullptr;
  }
  ShimModule *m = new ShimModule();
  m->ptx.assign(ptxData ? ptxData : "", ptxLen);
  return reinterpret_cast<CUmodule>(m);
}

CUmodule mtrt_cuda_module_load_from_ptx_file(const char *filename, size_t filenameLength) {
  std::string path(filename ? filename : "", filenameLength);
  // "program.rtexe#segment": the module bytes are a data segment of a compiled executable
  const size_t hash = path.rfind('#');
  if (hash != std::string::npos && hash >= 6 && path.compare(hash - 6, 6, ".rtexe") == 0) {
    ql_rtexe *exe = nullptr;
    if (ql_rtexe_open(path.substr(0, hash).c_str(), &exe) != QL_OK) {
      fail("could not open artifact '%s': %s", path.c_str(), ql_last_error());
      return nullptr;
    }
    const int idx = ql_rtexe_find_segment(exe, path.substr(hash + 1).c_str());
    ql_rtexe_segment_info info;
    CUmodule mod = nullptr;
    if (idx < 0 || ql_rtexe_segment(exe, idx, &info) != QL_OK) fail("executable '%s' has no data segment '%s'", path.substr(0, hash).c_str(), path.substr(hash + 1).c_str());
    else mod = mtrt_cuda_module_load_from_ptx(static_cast<const char *>(info.data), (size_t)info.size);
    ql_rtexe_close(exe);
    return mod;
  }
  std::ifstream f(path, std::ios::binary);
  if (!f) {
    fail("could not open artifact '%s'", path.c_str());
    return nullptr;
  }
  std::stringstream ss;
  ss << f.rdbuf();
  std::string data = ss.str();
  return mtrt_cuda_module_load_from_ptx(data.data(), data.size());
}

void mtrt_cuda_module_unload(CUmodule module) {
  ShimModule *m = as_module(module);
  if (!m) return fail("module_unload: not a module handle of this library");
  if (m->jit && driver().ok) driver().moduleUnload(m->jit);
  for (ShimFunction *f : m->functions) delete f;
  m->magic = 0;
  delete m;
}

CUfunction mtrt_cuda_module_get_function(CUmodule cumodule, const char *name, int64_t length) {
  ShimModule *m = as_module(cumodule);
  if (!m) {
    fail("module_get_function: not a module handle of this library");
    return nullptr;
  }
  std::string nm(name ? name : "", (size_t)(length > 0 ? length : 0));
  std::string spec_text = nm;
  {
    std::lock_guard<std::mutex> lock(g_alias_mutex);
    read_manifest_once();
    auto it = g_aliases.find(nm);
    if (it != g_aliases.end()) spec_text = it->second;
  }
  ShimFunction *f = new ShimFunction();
  if (parse_spec(spec_text, &f->spec)) {
    f->library = true;
  } else {
    Driver &d = driver();
    if (!d.ok) {
      delete f;
      fail("the CUDA driver is not available: cannot JIT kernel '%s'", nm.c_str());
      return nullptr;
    }
    if (!m->jit) {
      std::string z = m->ptx; // the driver wants NUL-terminated PTX
      CUresult r = d.moduleLoadDataEx(&m->jit, z.c_str(), 0, nullptr, nullptr);
      if (r != CUDA_SUCCESS) {
        delete f;
        fail("cuModuleLoadDataEx: %s", drv_msg(r));
        return nullptr;
      }
    }
    CUresult r = d.moduleGetFunction(&f->fn, m->jit, nm.c_str());
    if (r != CUDA_SUCCESS) {
      delete f;
      fail("cuModuleGetFunction('%s'): %s", nm.c_str(), drv_msg(r));
      return nullptr;
    }
  }
  m->functions.push_back(f);
  return reinterpret_cast<CUfunction>(f);
}

void mtrt_cuda_launch_kernel(CUfunction cudaFuncPtr, int32_t gridX, int32_t gridY, int32_t gridZ, int32_t blockX,
                             int32_t blockY, int32_t blockZ, int32_t dynamicSharedMemory, CUstream stream, void **args) {
  ShimFunction *f = reinterpret_cast<ShimFunction *>(cudaFuncPtr);
  if (!f || f->magic != kFunctionMagic) return fail("launch_kernel: not a function handle of this library");
  g_mtrt_error[0] = 0;
  if (f->library) {
    // the hand-written kernel picks its own launch shape; the caller's grid describes generated code
    launch_library_kernel(f->spec, stream, args);
    return;
  }
  CUresult r = driver().launchKernel(f->fn, gridX, gridY, gridZ, blockX, blockY, blockZ, dynamicSharedMemory, stream, args, nullptr);
  if (r != CUDA_SUCCESS) fail("cuLaunchKernel: %s", drv_msg(r));
}

} // extern "C"
