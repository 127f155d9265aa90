/*
 * The executor runtime's CUDA module C ABI, as generated host code and the Lua/EmitC backends call
 * it.  Same symbols, argument order and meaning as the reference's
 *   mlir-tensorrt/executor/lib/Runtime/Backend/C/CUDAModule.h:57-120
 * (Lua builtins __cuda_load_module / __cuda_get_function / __cuda_launch,
 *  executor/lib/Runtime/Backend/Lua/Modules/CUDA/CUDAModule.cpp:287-342, forward to these).
 *
 * What differs behind the symbols: a kernel whose name resolves to one of the hand-written
 * sm_100a kernels of this library (see "Kernel names" below) is launched from the library's own
 * image with the library's own grid; any other name is looked up in the PTX the caller supplied,
 * JIT-compiled by the driver, exactly as the reference does.  Failures do not abort the process:
 * the call returns null / does nothing and mtrt_cuda_last_error() carries the message.
 *
 * Kernel names.  A name of the form "ql:<op>;<key>=<value>;..." selects a library kernel; any other
 * name is first looked up among the aliases registered with ql_mtrt_bind_kernel (or listed in the
 * file named by the environment variable QL_MTRT_MANIFEST, one "name = ql:..." per line).
 *   ql:quantize;in=f32;out=i8;scale=f32;shape=4096x4096                 args: in, scale, out
 *   ql:quantize;in=f16;out=i8;scale=f16;shape=11008x4096;axis=0
 *   ql:quantize;in=f16;out=i4;scale=f16;shape=4096x4096;scale_shape=4096x32
 *   ql:dequantize;in=i8;out=f32;scale=f32;shape=4096x4096               args: in, scale, out
 *   ql:linear_w8a16;x=bf16;scale=f16;M=16;N=11008;K=4096                args: x, w, scale, y
 *   ql:linear_w4a16;x=f16;scale=f16;M=8;N=4096;K=4096;block=128         args: x, w, scale, y
 *   ql:gemm_fp8;out=bf16;M=8192;N=28672;K=8192;sx=1;sw=1                args: xq, wq, sx, sw, y
 * Arguments follow the reference's launch convention (compiler/lib/Passes/1_Core/KernelToCUDA/KernelToCUDA.cpp:94-108,
 * 163-175): args[i] points to the i-th kernel parameter; a memref contributes its aligned base pointer and then,
 * only where they are not compile-time constants, its offset, dynamic sizes and dynamic strides as i64 values.  A
 * dynamic dimension is written `?` in a spec (shape=?x4096, M=?): the kernel then reads that size (and the strides
 * that depend on it, which must be the dense row-major ones) from the arguments after the memref's pointer:
 *   ql:quantize;in=f32;out=i8;scale=f32;shape=?x4096        args: in, in.size0, scale, out, out.size0
 *   ql:linear_w8a16;x=bf16;scale=f16;M=?;N=11008;K=4096     args: x, x.size0, w, scale, y, y.size0
 */
#ifndef MTRT_CUDA_MODULE_H
#define MTRT_CUDA_MODULE_H

#include <stddef.h>
#include <stdint.h>

#include "cuda.h"
#include "cuda_runtime_api.h"

#ifdef __cplusplus
extern "C" {
#endif

#define MTRT_CAPI_EXPORTED __attribute__((visibility("default")))

MTRT_CAPI_EXPORTED int32_t mtrt_cuda_get_active_device();
MTRT_CAPI_EXPORTED int32_t mtrt_cuda_set_active_device(int32_t device);
MTRT_CAPI_EXPORTED int32_t mtrt_cuda_get_device(int32_t device);
MTRT_CAPI_EXPORTED CUstream mtrt_cuda_stream_create();
MTRT_CAPI_EXPORTED void mtrt_cuda_stream_destroy(CUstream stream);
MTRT_CAPI_EXPORTED void mtrt_cuda_stream_sync(CUstream stream);

MTRT_CAPI_EXPORTED cudaEvent_t mtrt_cuda_event_create(int32_t device);
MTRT_CAPI_EXPORTED void mtrt_cuda_event_release(cudaEvent_t event);
MTRT_CAPI_EXPORTED void mtrt_cuda_stream_record_event(CUstream stream, cudaEvent_t event);
MTRT_CAPI_EXPORTED void mtrt_cuda_stream_wait_event(CUstream stream, cudaEvent_t event);
MTRT_CAPI_EXPORTED void mtrt_cuda_event_sync(cudaEvent_t event);
MTRT_CAPI_EXPORTED float mtrt_cuda_event_elapsed_msec(cudaEvent_t start, cudaEvent_t end);

MTRT_CAPI_EXPORTED void *mtrt_cuda_alloc_async(CUstream stream, int64_t size, int32_t alignment, int8_t isHostPinned,
                                               int8_t isManaged);
MTRT_CAPI_EXPORTED void mtrt_cuda_memcpy_async(CUstream stream, void *src, void *dest, int64_t size);
MTRT_CAPI_EXPORTED void mtrt_cuda_free(CUstream stream, void *ptr, int8_t isHostPinned, int8_t isManaged);

MTRT_CAPI_EXPORTED CUmodule mtrt_cuda_module_load_from_ptx(const char *ptxData, size_t ptxLen);
MTRT_CAPI_EXPORTED CUmodule mtrt_cuda_module_load_from_ptx_file(const char *filename, size_t filenameLength);
MTRT_CAPI_EXPORTED void mtrt_cuda_module_unload(CUmodule module);
/* `name` is not NUL-terminated; `length` gives its size (C/CUDAModule.cpp:217-224). */
MTRT_CAPI_EXPORTED CUfunction mtrt_cuda_module_get_function(CUmodule cumodule, const char *name, int64_t length);
MTRT_CAPI_EXPORTED void mtrt_cuda_launch_kernel(CUfunction cudaFuncPtr, int32_t gridX, int32_t gridY, int32_t gridZ,
                                                int32_t blockX, int32_t blockY, int32_t blockZ,
                                                int32_t dynamicSharedMemory, CUstream stream, void **args);
MTRT_CAPI_EXPORTED int32_t mtrt_cuda_get_current_device();
MTRT_CAPI_EXPORTED int32_t mtrt_cuda_get_program_device(int32_t logicalId);

/* Additions of this library (no counterpart in the reference): the message of the calling thread's
 * last failed mtrt_cuda_* call ("" if none), and the alias table described above. */
MTRT_CAPI_EXPORTED const char *mtrt_cuda_last_error();
MTRT_CAPI_EXPORTED int32_t ql_mtrt_bind_kernel(const char *kernel_name, const char *op_spec);

/* Type-erased forms of the calls above, for host code generated through EmitC: that code passes every handle and
 * buffer as `void *`, so each entry point has an inline `<name>_cwrapper` that casts and forwards (same names and
 * parameter lists as mlir-tensorrt/executor/lib/Runtime/Backend/C/CUDAModule.h:130-205). */
#define MTRT_CW static inline
MTRT_CW void *mtrt_cuda_stream_create_cwrapper() { return (void *)mtrt_cuda_stream_create(); }
MTRT_CW void mtrt_cuda_stream_destroy_cwrapper(void *stream) { mtrt_cuda_stream_destroy((CUstream)stream); }
MTRT_CW void mtrt_cuda_stream_sync_cwrapper(void *stream) { mtrt_cuda_stream_sync((CUstream)stream); }
MTRT_CW void *mtrt_cuda_event_create_cwrapper(int32_t device) { return (void *)mtrt_cuda_event_create(device); }
MTRT_CW void mtrt_cuda_event_release_cwrapper(void *event) { mtrt_cuda_event_release((cudaEvent_t)event); }
MTRT_CW void mtrt_cuda_stream_record_event_cwrapper(void *stream, void *event) {
  mtrt_cuda_stream_record_event((CUstream)stream, (cudaEvent_t)event);
}
MTRT_CW void mtrt_cuda_stream_wait_event_cwrapper(void *stream, void *event) {
  mtrt_cuda_stream_wait_event((CUstream)stream, (cudaEvent_t)event);
}
MTRT_CW void mtrt_cuda_event_sync_cwrapper(void *event) { mtrt_cuda_event_sync((cudaEvent_t)event); }
MTRT_CW float mtrt_cuda_event_elapsed_msec_cwrapper(void *start, void *end) {
  return mtrt_cuda_event_elapsed_msec((cudaEvent_t)start, (cudaEvent_t)end);
}
MTRT_CW void *mtrt_cuda_alloc_async_cwrapper(void *stream, int64_t size, int32_t alignment, int8_t isHostPinned, int8_t isManaged) {
  return mtrt_cuda_alloc_async((CUstream)stream, size, alignment, isHostPinned, isManaged);
}
MTRT_CW void mtrt_cuda_memcpy_async_cwrapper(void *stream, void *src, void *dest, int64_t size) {
  mtrt_cuda_memcpy_async((CUstream)stream, src, dest, size);
}
MTRT_CW void mtrt_cuda_free_cwrapper(void *stream, void *ptr, int8_t isHostPinned, int8_t isManaged) {
  mtrt_cuda_free((CUstream)stream, ptr, isHostPinned, isManaged);
}
MTRT_CW void *mtrt_cuda_module_load_from_ptx_cwrapper(void *ptxData, size_t ptxLen) {
  return (void *)mtrt_cuda_module_load_from_ptx((const char *)ptxData, ptxLen);
}
MTRT_CW void *mtrt_cuda_module_load_from_ptx_file_cwrapper(void *filename, size_t filenameLength) {
  return (void *)mtrt_cuda_module_load_from_ptx_file((const char *)filename, filenameLength);
}
MTRT_CW void mtrt_cuda_module_unload_cwrapper(void *module) { mtrt_cuda_module_unload((CUmodule)module); }
MTRT_CW void *mtrt_cuda_module_get_function_cwrapper(void *cumodule, void *name, int64_t length) {
  return (void *)mtrt_cuda_module_get_function((CUmodule)cumodule, (const char *)name, length);
}
MTRT_CW void mtrt_cuda_launch_kernel_cwrapper(void *cudaFuncPtr, int32_t gridX, int32_t gridY, int32_t gridZ, int32_t blockX,
                                              int32_t blockY, int32_t blockZ, int32_t dynamicSharedMemory, void *stream, void *args) {
  mtrt_cuda_launch_kernel((CUfunction)cudaFuncPtr, gridX, gridY, gridZ, blockX, blockY, blockZ, dynamicSharedMemory, (CUstream)stream,
                          (void **)args);
}
MTRT_CW int32_t mtrt_cuda_get_current_device_cwrapper() { return mtrt_cuda_get_current_device(); }
#undef MTRT_CW

#ifdef __cplusplus
}
#endif
#endif /* MTRT_CUDA_MODULE_H */
