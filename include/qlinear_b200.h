/*
 * qlinear_b200 -- C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * Every entry point takes plain pointers and sizes, is stream-ordered on the caller's stream
 * (a cudaStream_t / CUstream passed as void*), never synchronises the device and returns a
 * ql_status; ql_last_error() gives the message of the calling thread's last failure.  All
 * tensors are dense, row-major and live in device memory unless stated otherwise.
 *
 * Reference interfaces each group replaces (paths inside NVIDIA/TensorRT-Incubator):
 *   tensorrt.quantize      mlir-tensorrt/tensorrt/include/mlir-tensorrt-dialect/TensorRT/IR/TensorRTOps.td:3091-3273
 *   tensorrt.dequantize    .../TensorRTOps.td:3364-3506
 *   argument rules         mlir-tensorrt/tensorrt/lib/TensorRT/IR/Verification.cpp:1182-1380
 *   tp.quantize/dequantize tripy/nvtripy/frontend/ops/quantize.py:39-119, dequantize.py:39-114
 *   tp.Linear / matmul     tripy/nvtripy/frontend/module/linear.py:112-151, frontend/ops/matmul.py:29-108
 */
#ifndef QLINEAR_B200_H
#define QLINEAR_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QL_API __attribute__((visibility("default")))
#define QL_MAX_RANK 8

typedef enum {
  QL_F32 = 0,
  QL_F16 = 1,
  QL_BF16 = 2,
  QL_I8 = 3,
  QL_I4 = 4,     /* two values per byte, first element in the low nibble */
  QL_F8E4M3 = 5, /* e4m3fn: no infinities, 0x7F/0xFF are NaN, largest finite 448 */
  QL_F4E2M1 = 6  /* e2m1fn (0, 0.5, 1, 1.5, 2, 3, 4, 6 and negatives): two per byte, first element in the low nibble */
} ql_dtype;

typedef enum {
  QL_OK = 0,
  QL_ERR_INVALID_ARGUMENT = 1, /* violates the operator's argument rules; message says which */
  QL_ERR_UNSUPPORTED = 2,      /* legal for the reference operator but not built here */
  QL_ERR_CUDA = 3,             /* a CUDA call failed; message carries cudaGetErrorString */
  QL_ERR_NO_DEVICE = 4,        /* no usable sm_100 device / driver */
  QL_ERR_DEVICE_TIMEOUT = 5    /* a bounded on-device wait ran out (kernel returned early) */
} ql_status;

/* fp8 quantize semantics found in the reference tree; QL_FP8_DIRECT is the operator's
 * specification (one rounding from the f32 quotient, saturate to +-448). */
typedef enum {
  QL_FP8_DIRECT = 0,
  QL_FP8_VIA_F16 = 1,   /* f32 -> f16 -> e4m3, as kernel/lib/Kernel/Transforms/NormalizeQuantizedConversions.cpp:43-80 lowers it */
  QL_FP8_STABLEHLO = 2  /* divide, round to integer, clamp, convert in the input type
                           (compiler/lib/Dialect/StablehloExt/Transforms/StablehloRaiseQDQ.cpp:233-265).  The one
                           mode that also changes int8 and int4 results: for f16 / bf16 input the quotient is rounded
                           to that type before the round to integer, where the operator itself divides in f32. */
} ql_fp8_mode;

typedef struct {
  void *data;                 /* device pointer (scales may also be device pointers only) */
  int32_t dtype;              /* ql_dtype */
  int32_t rank;               /* 0 = scalar */
  int64_t shape[QL_MAX_RANK]; /* logical element counts; QL_I4 tensors hold ceil(numel/2) bytes */
} ql_tensor;

/* Attributes of tensorrt.quantize / tensorrt.dequantize.  The mode follows the scale's rank as in
 * the reference verifier: rank 0 = per-tensor (axis must be absent), rank 1 = per-channel (axis
 * required, scale length == input.shape[axis]), rank == input rank = block quantization (axis
 * absent; exactly one differing dimension, the last or second last; block size =
 * input.shape[d] / scale.shape[d]). */
typedef struct {
  int32_t has_axis;
  int32_t axis;
  int32_t fp8_mode; /* ql_fp8_mode; ignored unless the quantized type is QL_F8E4M3 */
} ql_qdq_attrs;

QL_API int ql_version(void);
QL_API const char *ql_last_error(void);
/* Number of kernels this library has launched in this process since it was loaded. */
QL_API uint64_t ql_launch_count(void);
/* Device properties the host side needs: SM count, compute capability (major*10+minor). */
QL_API int ql_device_info(int32_t *sm_count, int32_t *compute_capability);

/* output = clamp(round_half_even(input / (f32)scale), qmin, qmax) as i8 / i4, or the saturating
 * e4m3 conversion of the quotient.  input: f32 | f16 | bf16.  scale: f32 | f16 | bf16. */
QL_API int ql_quantize(const ql_tensor *input, const ql_tensor *scale, ql_tensor *output,
                       const ql_qdq_attrs *attrs, void *stream);

/* output = (out type)((f32)input * (f32)scale).  input: i8 | i4 | e4m3.  output: f32 | f16 | bf16. */
QL_API int ql_dequantize(const ql_tensor *input, const ql_tensor *scale, ql_tensor *output,
                         const ql_qdq_attrs *attrs, void *stream);

/* One pass that writes both quantize(input) and dequantize(quantize(input)); `dequantized` has the
 * input's type.  Bit-identical to ql_quantize followed by ql_dequantize. */
QL_API int ql_quantize_dequantize(const ql_tensor *input, const ql_tensor *scale,
                                  ql_tensor *quantized, ql_tensor *dequantized,
                                  const ql_qdq_attrs *attrs, void *stream);

/* Dynamic scales (the reference only accepts constant scales; its user guide defines
 * scale = amax / maxbound, tripy/docs/pre0_user_guides/02-quantization.md:104-112):
 * scale[j] = max|input| over group j, divided by `maxbound` in f32, rounded to scale->dtype.
 * Groups follow scale->rank exactly as in ql_qdq_attrs. */
QL_API int ql_amax_scale(const ql_tensor *input, ql_tensor *scale, const ql_qdq_attrs *attrs,
                         float maxbound, void *stream);

/* No counterpart in the reference.  Same result as ql_amax_scale, for callers that are not allowed
 * to allocate device memory while they run -- a runtime that planned and accounted for every buffer
 * before execution started, or a latency-bound serving loop where an allocation might block or fail.
 * ql_amax_scale parks its f32 max|x| accumulators in stream-ordered scratch memory when the scales
 * are 16-bit; this variant parks them in a fixed array inside the library instead and calls no
 * allocator of any kind.
 *   - At most QL_NOALLOC_MAX_SCALES scales (groups) per call; more is rejected with
 *     QL_ERR_UNSUPPORTED and a message naming the limit.  The array costs that many floats
 *     (256 KiB) on every GPU that loads the library, until the process exits.
 *   - The first call on each device looks up the array's device address; make that first call
 *     before starting any stream capture on that device.
 *   - All calls on a device share the one array (it is re-zeroed at the start of each call), so two
 *     calls whose GPU work may overlap -- different streams without an ordering between them --
 *     race on it.  Order them, or use ql_amax_scale for one of them. */
#define QL_NOALLOC_MAX_SCALES 65536
QL_API int ql_amax_scale_noalloc(const ql_tensor *input, ql_tensor *scale, const ql_qdq_attrs *attrs,
                                 float maxbound, void *stream);

/* NVFP4.  ql_dynamic_quantize is tensorrt.dynamic_quantize (TensorRTOps.td:3279-3358; checks and wording of
 * Verification.cpp:1270-1290): blocks of 16 along `axis` (the last axis; the second last is legal for the operator
 * but not built), scales [..., K/16] = e4m3((max|block| / 6) / double_quant_scale), result = e2m1(x / (scale *
 * double_quant_scale)).  ql_dequantize_nvfp4 is the operator's documented inverse, the two tensorrt.dequantize
 * steps in one pass: output = e2m1 value * (e4m3 scale * double_quant_scale).  double_quant_scale is a rank-0
 * device tensor.  Data tensors of type QL_F4E2M1 carry their logical shape; the buffer holds numel / 2 bytes. */
QL_API int ql_dynamic_quantize(const ql_tensor *input, const ql_tensor *double_quant_scale, int32_t axis,
                               int32_t block_size, ql_tensor *result, ql_tensor *scales, void *stream);
QL_API int ql_dequantize_nvfp4(const ql_tensor *data, const ql_tensor *scales, const ql_tensor *double_quant_scale,
                               ql_tensor *output, void *stream);

/* Block-scaled NVFP4 GEMM: Y[M,N] = dq(a)[M,K] . dq(b)[N,K]^T with dq(x)[r,k] = e2m1 * e4m3 scale[r, k/16] * global, i.e.
 * tensorrt.matrix_multiply of two operands that went through tensorrt.dynamic_quantize and its two dequantize steps
 * (TensorRTOps.td:3279-3358, 1986-2080), with the dequantization done by the tensor core
 * (tcgen05.mma kind::mxf4nvf4, block scales read from tensor memory; f32 accumulation).  a, b: QL_F4E2M1 [M,K], [N,K];
 * *_scales: QL_F8E4M3 [rows, K/16] as ql_dynamic_quantize writes them; *_global: f32 scalar or null (= 1);
 * y: f32 | f16 | bf16.  Needs K % 32 == 0 and 16-byte aligned data (QL_ERR_UNSUPPORTED otherwise: dequantize and
 * use ql_linear).  Takes scratch for the re-ordered scales from the stream-ordered allocator. */
QL_API int ql_gemm_nvfp4(const ql_tensor *a, const ql_tensor *a_scales, const ql_tensor *a_global, const ql_tensor *b,
                         const ql_tensor *b_scales, const ql_tensor *b_global, ql_tensor *y, void *stream);

/* Weight-only linear layers, Y[M,N] = X[M,K] . dequantize(W)[N,K]^T with f32 accumulation
 * (linear.py:140-151 with quant_dtype set and no input scale).
 *   w8: W int8 [N,K], scale [N] per output channel (weight_quant_dim = 0)
 *   w4: W int4 packed [N,K/2], scale [N, K/block] (block quantization along K)
 * X and Y are f16 or bf16 (same type); scales f32, f16 or bf16. */
QL_API int ql_linear_w8a16(const ql_tensor *x, const ql_tensor *w, const ql_tensor *scale,
                           ql_tensor *y, void *stream);
QL_API int ql_linear_w4a16(const ql_tensor *x, const ql_tensor *w, const ql_tensor *scale,
                           ql_tensor *y, void *stream);
/* Either of the two, chosen by w->dtype, with flags.  QL_WEIGHTS_CONSTANT: w and scale were written before the
 * kernel that precedes this call on the stream was launched -- true of the weights of a compiled program, which
 * are constants (the reference requires constant scales, TensorRTOps.td:3113-3114, and Linear's weights are
 * parameters).  With at most 64 rows of x the kernel is then launched so that it may start while its predecessor
 * is still finishing (programmatic dependent launch): it fetches its first weights, waits for the predecessor to
 * complete, and only then reads x and writes y.  Without the flag the launch is ordered like any other. */
#define QL_WEIGHTS_CONSTANT 1u
QL_API int ql_linear_weight_only(const ql_tensor *x, const ql_tensor *w, const ql_tensor *scale, ql_tensor *y,
                                 uint32_t flags, void *stream);

/* Quantized GEMMs on the tensor cores, Y[M,N] = (Xq[M,K] . Wq[N,K]^T) * sx * sw, f32 (fp8) or
 * s32 (int8) accumulation, scales applied in the epilogue, Y bf16, f16 or f32.
 * sx: f32 scalar or [M] (per token); sw: f32 scalar or [N] (per output channel).
 * Shapes the tensor-core kernels cannot take (K not a multiple of 16 bytes, operands not 16-byte aligned) run on
 * a general CUDA-core kernel with the same arithmetic. */
QL_API int ql_gemm_fp8(const ql_tensor *xq, const ql_tensor *wq, const ql_tensor *sx,
                       const ql_tensor *sw, ql_tensor *y, void *stream);
QL_API int ql_gemm_i8(const ql_tensor *xq, const ql_tensor *wq, const ql_tensor *sx,
                      const ql_tensor *sw, ql_tensor *y, void *stream);
/* ---- Tensor-parallel layers over the GPUs of one box: the fp8 GEMM with its collective done by the epilogue.
 * No reference counterpart: the reference has no multi-GPU execution of this path.
 *
 * A ql_peer_buffer describes one buffer that exists on every rank ("replica"), one process per GPU:
 *   replica[r]  the address, in this process, of rank r's copy (peer-mapped device memory; replica[rank] is local);
 *   all         an address in an NVSwitch replication group (CUDA multicast object) covering all replicas: a
 *               `multimem` write to it lands in every replica.
 * The caller allocates and maps the buffer (any symmetric-memory allocator; the Python layer uses torch's).
 *
 * ql_gemm_fp8_peer computes this rank's [M, N] result and writes it at element offset `offset` of a row-major
 * buffer with `ldy` elements per row, in one of three ways:
 *   QL_PEER_STORE_ALL  stores it in every replica: column-parallel GEMM + all-gather in one kernel;
 *   QL_PEER_ADD_ALL    adds it into every replica (sum in the output type): row-parallel GEMM + all-reduce in
 *                      one kernel; every replica receives world x the data, so this suits two ranks;
 *   QL_PEER_ADD_OWNER  adds each row into the replica of the rank that owns it (rank r owns rows
 *                      [r * M / world, (r + 1) * M / world), M / world a multiple of 128): row-parallel GEMM +
 *                      reduce-scatter in one kernel; ql_peer_broadcast of the owned rows completes the all-reduce.
 * Adds need zeros (or a bias) in the target rows before any rank starts.  The kernels wait on no peer; all their
 * remote writes are posted.  ql_peer_barrier orders ranks: work queued before it on every rank's stream is
 * complete and visible before work queued after it starts on any rank.  `flags` is a peer buffer of
 * (world + 1) uint32, zero-initialised, used by nothing else.  Its wait is bounded (about ten seconds); a rank
 * that gives up records it for ql_gemm_status.  Peer modes need N % 32 == 0, ldy % 8 == 0, offset % 8 == 0. */
#define QL_MAX_PEERS 8
typedef enum { QL_PEER_NONE = 0, QL_PEER_STORE_ALL = 1, QL_PEER_ADD_ALL = 2, QL_PEER_ADD_OWNER = 3 } ql_peer_mode;
typedef struct {
  void *replica[QL_MAX_PEERS];
  void *all;
  int32_t world;
  int32_t rank;
} ql_peer_buffer;
QL_API int ql_gemm_fp8_peer(const ql_tensor *xq, const ql_tensor *wq, const ql_tensor *sx, const ql_tensor *sw,
                            const ql_peer_buffer *dest, int32_t y_dtype, int64_t ldy, int64_t offset, int peer_mode,
                            void *stream);
QL_API int ql_peer_barrier(const ql_peer_buffer *flags, void *stream);
/* Diagnostics: how many SM clock cycles ql_peer_barrier waits for a peer before it gives up (0 restores the
 * default of 2^34, about ten seconds).  Process-wide; applies to barriers launched after the call. */
QL_API int ql_set_peer_wait_limit(int64_t cycles);
/* In-switch all-reduce of bytes [offset, offset + bytes) (bf16 or f16 elements, 16-byte units): the NVSwitch adds
 * that range of all replicas in f32 and the sum replaces it in every replica.  Ranks call it on disjoint ranges
 * between two ql_peer_barrier calls; with a GEMM that wrote its partial result into the local replica this is a
 * row-parallel all-reduce in which every sum is rounded once. */
QL_API int ql_peer_reduce(const ql_peer_buffer *buf, int32_t dtype, int64_t offset, int64_t bytes, void *stream);
/* copies bytes [offset, offset + bytes) of this rank's replica to the same range of every replica (16-byte units) */
QL_API int ql_peer_broadcast(const ql_peer_buffer *buf, int64_t offset, int64_t bytes, void *stream);
/* 16-bit GEMM Y = (X . W^T) * sw, X and W both bf16 or both f16 ([M,K], [N,K]); sw may be null. */
QL_API int ql_gemm_16(const ql_tensor *x, const ql_tensor *w, const ql_tensor *sw, ql_tensor *y,
                      void *stream);

/* The forward of tp.Linear (tripy/nvtripy/frontend/module/linear.py:127-151) once its quantize / dequantize pairs are
 * folded into scales: Y[M,N] = (X[M,K] . W[N,K]^T) * sx * sw + bias[n].  X and W share one type: f32, f16, bf16
 * (then Y has that type, as tp.matmul requires: frontend/ops/matmul.py:31-34), e4m3 or int8 (Y f32, f16 or bf16).
 * sx, sw: null, f32 scalar, or one value per row of X / of W.  bias: null or [N] of any float type, added in f32
 * before the single rounding to Y's type.  16-bit and 8-bit operands with 16-byte aligned rows run on the
 * tensor cores; everything else (f32 operands, K = 4, unaligned views) on a general CUDA-core kernel. */
QL_API int ql_linear(const ql_tensor *x, const ql_tensor *w, const ql_tensor *sx, const ql_tensor *sw,
                     const ql_tensor *bias, ql_tensor *y, void *stream);
/* C = A @ B: tensorrt.matrix_multiply with both operands kNONE (TensorRTOps.td:1986-2080), what tp.matmul emits
 * (tripy/nvtripy/frontend/ops/matmul.py:29-108).  A [..., M, K], B [..., K, N], C [..., M, N]: equal ranks >= 2, one
 * float type, f32 accumulation.  The leading dimensions of an operand are all equal to C's or all 1 (broadcast);
 * 1-D operands and mixed broadcasts are reshaped by the caller (the Python layer does). */
QL_API int ql_matmul(const ql_tensor *a, const ql_tensor *b, ql_tensor *c, void *stream);

/* Row kernels of the quantized MLP block (RMSNorm / SwiGLU are not reference operators; the quantize
 * step inside them is tensorrt.quantize with one scale per row, scale = max|row| / 448):
 *   rmsnorm_quant_fp8: r = x * rsqrt(mean(x^2) + eps) (weight 1); q = e4m3(r / s[t]); x [T,H] bf16|f16
 *   swiglu_quant_fp8:  a = silu(gate) * up with gate_up = [gate | up] [T, 2I]; q = e4m3(a / s[t]), q [T,I]
 * q is e4m3, scale f32 [T]; row lengths must be multiples of 16. */
QL_API int ql_rmsnorm_quant_fp8(const ql_tensor *x, float eps, ql_tensor *q, ql_tensor *scale, void *stream);
QL_API int ql_swiglu_quant_fp8(const ql_tensor *gate_up, ql_tensor *q, ql_tensor *scale, void *stream);
/* The same two steps with SwiGLU moved into the gate/up projection's epilogue, so that the [T, 2I] projection is
 * never written to memory:
 *   gemm_fp8_swiglu:   wq [2I, K] holds the gate and up weights interleaved in groups of 32 rows (rows [64b, 64b+32)
 *                      = gate channels [32b, 32b+32), rows [64b+32, 64b+64) = up channels [32b, 32b+32)), sw (scalar
 *                      or [2I]) in the same order.  act[t, i] = silu(g) * u with g, u the scaled f32 sums of channel
 *                      i, rounded once to act's type (bf16 | f16); row_amax[t] = max_i |act[t, i]| (f32 [T],
 *                      overwritten).  Needs K % 16 == 0 and 16-byte aligned operands (QL_ERR_UNSUPPORTED otherwise).
 *   quantize_rows_fp8: tensorrt.quantize per row with the scale formed from row maxima: scale[t] = row_amax[t] / 448
 *                      (1 for an all-zero row), q = e4m3(a / scale[t]).  a [T, I] bf16 | f16, I % 16 == 0. */
QL_API int ql_gemm_fp8_swiglu(const ql_tensor *xq, const ql_tensor *wq, const ql_tensor *sx, const ql_tensor *sw,
                              ql_tensor *act, ql_tensor *row_amax, void *stream);
QL_API int ql_quantize_rows_fp8(const ql_tensor *a, const ql_tensor *row_amax, ql_tensor *q, ql_tensor *scale, void *stream);

/* The tensor-core kernels bound every on-device wait (mbarrier, tensor-memory hand-over) by a
 * cycle limit; a kernel that runs out records a code and returns early instead of hanging.  This
 * call synchronises the device, returns QL_ERR_DEVICE_TIMEOUT if a code was recorded since the
 * last call (and clears it), and stores the code in *code when code is not null. */
QL_API int ql_gemm_status(int32_t *code);
/* Diagnostics: the library reads its QL_* tuning variables from the environment once, at the first GEMM of the
 * process; this makes it read them again (not thread-safe against GEMM calls in flight on other host threads). */
QL_API int ql_reload_tuning(void);

/* ---- Compiled executables (`.rtexe`).  The reference's translation step writes a FlatBuffers file
 * (executor/include/mlir-executor/Runtime/API/Executable.fbs) whose data segments carry, among the program's
 * constants, the PTX or cubin of each cuda.compiled_module; its runtime hands those bytes to __cuda_load_module
 * (executor/lib/Runtime/Backend/Lua/Modules/CUDA/CUDAModule.cpp:287-300), i.e. to mtrt_cuda_module_load_from_ptx.
 * These calls read the same segments without that runtime (host side only, no GPU needed); in addition
 * mtrt_cuda_module_load_from_ptx_file accepts "path/program.rtexe#segment_name". */
typedef struct ql_rtexe ql_rtexe;
typedef enum { QL_RTEXE_DATA = 0, QL_RTEXE_PTX = 1, QL_RTEXE_CUBIN = 2, QL_RTEXE_FATBIN = 3 } ql_rtexe_kind;
typedef struct {
  const char *name;            /* the global's symbol name; valid until ql_rtexe_close */
  const void *data;            /* the segment's bytes inside the opened file (null when it has none) */
  uint64_t size;
  uint64_t uninitialized_size; /* size of a segment that is only reserved, not filled */
  uint32_t alignment;
  int32_t constant;
  int32_t address_space;       /* PointerType of the schema: 0 host, 1 pinned_host, 2 device, 3 unified, 4 unknown */
  int32_t kind;                /* ql_rtexe_kind, guessed from the bytes */
} ql_rtexe_segment_info;
QL_API int ql_rtexe_open(const char *path, ql_rtexe **out);
QL_API int ql_rtexe_open_memory(const void *bytes, uint64_t size, ql_rtexe **out); /* the bytes are copied */
QL_API void ql_rtexe_close(ql_rtexe *exe);
QL_API const char *ql_rtexe_name(const ql_rtexe *exe);
QL_API int32_t ql_rtexe_num_segments(const ql_rtexe *exe);
QL_API int ql_rtexe_segment(const ql_rtexe *exe, int32_t index, ql_rtexe_segment_info *info);
QL_API int ql_rtexe_find_segment(const ql_rtexe *exe, const char *name); /* index, or -1 */

/* ---- NCCL communicators and collectives, as the executor runtime's NCCL module offers them to compiled programs
 * (executor/lib/Runtime/Backend/Lua/Modules/NCCL/NCCLModule.cpp:233-385: __nccl_comm_init_rank, __nccl_comm_split,
 * __nccl_comm_rank / _num_ranks, __nccl_all_reduce_<op>_<type>, __nccl_reduce_scatter_<op>_<type>,
 * __nccl_all_gather, __nccl_all_to_all, __nccl_permute).  Same conventions: communicators are non-blocking, and
 * every call ends by polling ncclCommGetAsyncError until the communicator has left ncclInProgress or `timeout_ms`
 * (5000 when <= 0, the reference's value; NCCLModule.cpp:88-106) has passed, returning QL_ERR_DEVICE_TIMEOUT then.
 * (The first all_to_all / permute of a communicator connects every pair of ranks; on eight GPUs that alone took longer
 * than five seconds, so a communicator meant for those should be created with a larger limit.)
 * NCCL itself is bound at run time (libnccl.so.2); without it these return QL_ERR_UNSUPPORTED and the rest of the
 * library is unaffected.  Buffers are device pointers; `stream` is a cudaStream_t.  The fused GEMM + collective
 * entry points above do not go through NCCL. */
#define QL_NCCL_UNIQUE_ID_BYTES 128
typedef struct ql_nccl_comm ql_nccl_comm;
typedef enum { QL_NCCL_SUM = 0, QL_NCCL_PROD = 1, QL_NCCL_MIN = 2, QL_NCCL_MAX = 3, QL_NCCL_AVG = 4 } ql_nccl_op;
QL_API int ql_nccl_version(int32_t *version);
/* 128 bytes that rank 0 makes and every rank of the new communicator must be given (the runtime's _get_nccl_unique_id) */
QL_API int ql_nccl_unique_id(void *id);
/* makes `device` current, as __nccl_comm_init_rank does */
QL_API int ql_nccl_comm_init_rank(int32_t rank, int32_t num_ranks, int32_t device, const void *id, int64_t timeout_ms,
                                  ql_nccl_comm **out);
/* *out is null for a rank that passes color -1 (no new communicator) */
QL_API int ql_nccl_comm_split(ql_nccl_comm *parent, int32_t color, int32_t key, ql_nccl_comm **out);
QL_API int ql_nccl_comm_rank(const ql_nccl_comm *comm, int32_t *rank, int32_t *num_ranks);
/* finalizes a healthy communicator, aborts one that is in error or still busy after its time limit */
QL_API int ql_nccl_comm_destroy(ql_nccl_comm *comm);
/* dtype: QL_F32, QL_F16, QL_BF16 or QL_I8; op: ql_nccl_op */
QL_API int ql_nccl_all_reduce(ql_nccl_comm *comm, const void *send, void *recv, uint64_t count, int32_t dtype, int32_t op,
                              void *stream);
QL_API int ql_nccl_reduce_scatter(ql_nccl_comm *comm, const void *send, void *recv, uint64_t recv_count, int32_t dtype,
                                  int32_t op, void *stream);
/* bytes: recv holds num_ranks * send_bytes */
QL_API int ql_nccl_all_gather(ql_nccl_comm *comm, const void *send, void *recv, uint64_t send_bytes, void *stream);
/* total_bytes / num_ranks bytes go to, and come from, every rank */
QL_API int ql_nccl_all_to_all(ql_nccl_comm *comm, const void *send, void *recv, uint64_t total_bytes, void *stream);
/* send to `send_to` and receive from `recv_from`; -1 = no send / no receive (the receive buffer is then zeroed) */
QL_API int ql_nccl_permute(ql_nccl_comm *comm, const void *send, void *recv, int32_t send_to, int32_t recv_from,
                           uint64_t bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* QLINEAR_B200_H */
