/* C ABI of the B200 execution backend for Accelerate (hot path: execution of the
 * fused delayed AST on one GPU).
 *
 * A Haskell module `Data.Array.Accelerate.B200` binds these entry points with
 * `foreign import ccall safe` and exposes run/runN with the types of the
 * reference backends (Interpreter.hs:93-126).  Citations name the reference
 * interface each entry point stands in for (paths relative to the reference
 * project, src/Data/Array/Accelerate/...).
 *
 * Conventions: every function returns 0 on success or a B200_ERR_* code;
 * b200_last_error() gives the message of the calling thread's last failure.
 * All entry points are thread-safe (one mutex per context); none aborts the
 * process.  Host buffers stay owned by the caller (GHC pinned memory,
 * Array/Data.hs:331-334) and are only read or written during the call.
 */
#ifndef ACCELERATE_B200_H
#define ACCELERATE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_ctx b200_ctx;
typedef struct b200_program b200_program;

enum {
  B200_OK = 0,
  B200_ERR_PARSE = 1,       /* malformed program text */
  B200_ERR_TYPE = 2,        /* ill-typed program */
  B200_ERR_COMPILE = 3,     /* NVRTC rejected a generated kernel (internal error) */
  B200_ERR_CUDA = 4,        /* a CUDA call failed, or the CUDA driver is missing */
  B200_ERR_BOUNDS = 5,      /* the reference's boundsCheck failures: "empty array", "empty segment",
                               "shape mismatch", "index out of bounds" (Error.hs:52-63) */
  B200_ERR_UNSUPPORTED = 6,
  B200_ERR_ARG = 7,
  B200_ERR_TIMEOUT = 8,     /* a bounded device-side wait gave up */
  B200_ERR_ARITH = 9        /* integer division by zero (GHC's ArithException DivideByZero, raised by
                               quot/rem/div/mod in Interpreter.hs:1328-1344) */
};

/* Message of the last failure on this thread (valid until the next call). */
const char* b200_last_error(void);

/* Open a context on CUDA device `device` (a backend handle; the analogue of the
 * implicit global state behind Interpreter.run, Interpreter.hs:93-103).
 * Fails with B200_ERR_CUDA when no GPU or driver is present: there is no CPU
 * fallback. */
int b200_ctx_create(int device, uint32_t flags, b200_ctx** out);
void b200_ctx_destroy(b200_ctx* ctx);

/* Device arrays in struct-of-arrays layout, one buffer per scalar leaf of the
 * element type, row-major, innermost dimension last (Representation/Array.hs:43-46,
 * Array/Data.hs:95-98; device side of Array/Remote/Class.hs:47-73 mallocRemote).
 * `elt_type` is the element type as text: i8..i64, u8..u64, f32, f64 or
 * "(tup t1 t2 ...)". */
int b200_array_new(b200_ctx* ctx, const char* elt_type, int rank, const int64_t* shape, uint64_t* id);
/* Adopt device memory owned by the caller (one pointer per leaf); never freed. */
int b200_array_wrap(b200_ctx* ctx, const char* elt_type, int rank, const int64_t* shape, void* const* leaf_ptrs,
                    uint64_t* id);
/* pokeRemote / peekRemote (Array/Remote/Class.hs:58-66): copy one leaf. */
int b200_array_upload(b200_ctx* ctx, uint64_t id, int leaf, const void* host, size_t bytes);
int b200_array_download(b200_ctx* ctx, uint64_t id, int leaf, void* host, size_t bytes);
/* peekRemote without waiting: the copy runs on a second stream, after everything submitted so far, and
 * beside later uploads and kernels (PCIe carries both directions at once).  `host` should be pinned
 * memory and must not be read before b200_sync has returned; the array may be freed right away (its
 * memory is only reused once the copy has completed; memory adopted with b200_array_wrap stays the
 * caller's to keep until then).  peekRemote (Array/Remote/Class.hs:61-62) of a backend that
 * works asynchronously; the reference tracks such work as a `Task` polled for completion
 * (Array/Remote/LRU.hs:101-110), here b200_sync is the completion point. */
int b200_array_download_async(b200_ctx* ctx, uint64_t id, int leaf, void* host, size_t bytes);
/* Lazy pokeRemote: remember the host payload of one leaf; it is copied to the device the first time
 * the array is used (as a program input, by b200_array_devptr or by b200_array_download), as the
 * reference's memory table uploads an array on its first withRemote (Array/Remote/LRU.hs:140-199).
 * The payload must stay valid and unchanged until the call that uses the array has returned (the
 * Haskell side keeps it alive with touchArrayData, Array/Data.hs:250-255).  An explicit
 * b200_array_upload of the same leaf replaces it. */
int b200_array_adopt_host(b200_ctx* ctx, uint64_t id, int leaf, const void* host, size_t bytes);
/* Release (callable from any thread, e.g. a GHC finalizer; Array/Remote/Table.hs:271-284). */
int b200_array_free(b200_ctx* ctx, uint64_t id);
int b200_array_rank(b200_ctx* ctx, uint64_t id, int* rank);
int b200_array_shape(b200_ctx* ctx, uint64_t id, int64_t* shape);
int b200_array_num_leaves(b200_ctx* ctx, uint64_t id, int* n);
/* Scalar type name of a leaf ("f32", ...); pointer valid for the process lifetime. */
int b200_array_leaf_type(b200_ctx* ctx, uint64_t id, int leaf, const char** name);
int b200_array_devptr(b200_ctx* ctx, uint64_t id, int leaf, void** ptr);

/* Load a program: the text serialisation of a DelayedAfun (Trafo/Delayed.hs:41-60),
 * i.e. what Interpreter.runN obtains from convertAfun (Interpreter.hs:110-118).
 * Parses, type-checks and generates the kernels' scalar code; kernels are
 * compiled by NVRTC on first use and cached by content hash (in memory and in
 * $ACCELERATE_B200_CACHE_DIR). */
int b200_program_load(b200_ctx* ctx, const char* text, size_t len, b200_program** out);
void b200_program_free(b200_program* prog);
int b200_program_num_inputs(b200_program* prog, int* n);
int b200_program_num_outputs(b200_program* prog, int* n);
/* Execute (evalOpenAcc, Interpreter.hs:175-259): inputs bound in declaration
 * order; outputs are fresh arrays owned by the context (free with
 * b200_array_free).  Asynchronous: results are complete after b200_sync or a
 * download. */
int b200_program_run(b200_program* prog, const uint64_t* in_ids, int n_in, uint64_t* out_ids, int n_out);

/* Wait for all work of the context (asynchronous downloads included) and report device-side failures. */
int b200_sync(b200_ctx* ctx);

/* Counters (monitoring.c:26-32 in the reference's cbits): [0] kernels launched,
 * [1] bytes host->device, [2] bytes device->host, [3] kernels compiled,
 * [4] kernel-cache hits (memory), [5] kernel-cache hits (disk),
 * [6] device bytes currently allocated, [7] programs run. */
int b200_stats(b200_ctx* ctx, int64_t out[8]);

/* The CUDA stream the context launches on (a cudaStream_t), for callers that
 * time kernels with their own events. */
int b200_ctx_stream(b200_ctx* ctx, void** stream);

/* Generate and NVRTC-compile every kernel of a program for sm_100a without
 * touching a GPU (build-time check).  `log` receives diagnostics. */
int b200_compile_check(const char* text, size_t len, char* log, size_t log_len);
/* Generated CUDA source of node `node` (default variant), for inspection. */
int b200_kernel_source(const char* text, size_t len, int node, char* out, size_t out_len);

/* Diagnostic (no counterpart in the reference; used by the host-side tests): 1 when a scan along
 * rows of `n` elements of `elt_bytes` bytes each (`rows` rows, right-to-left if `right`) meets the
 * 16-byte alignment rule of the bulk copies in the shared-memory ring kernel, 0 when it has to take
 * the register kernel. */
int b200_scan_ring_aligned(int elt_bytes, int64_t n, int64_t rows, int right);

/* Inclusive prefix sum (scanl1 (+)) of `n` Int32 values, device to device,
 * WITHOUT allocating anything.  It has no counterpart in the reference: it
 * exists for callers that may not allocate device memory themselves nor let
 * this library do it — a host runtime whose collector owns all device memory
 * and lends out only the input and output buffers, or a caller on a path where
 * cudaMalloc's implicit device synchronisation is unacceptable.
 *
 * `in` and `out` are device pointers on the current device, 4-byte aligned
 * (16-byte alignment of both enables the vector path).  They may not overlap,
 * and in == out is not allowed either: tiles are read through the read-only
 * data path while other tiles are being written.  `stream` is a cudaStream_t
 * (NULL = default stream).  The call is synchronous: it blocks the calling host
 * thread until the result is complete (it copies a status word back and
 * synchronises `stream`).  The look-back descriptors of the scan
 * live in a fixed __device__ array of about 1 MB that every GPU using this
 * library holds until the process exits, hence:
 *   - n may not exceed B200_NOALLOC_SCAN_MAX_ELEMS; more is refused (B200_ERR_ARG);
 *   - calls on the same GPU share that array and must not overlap in time
 *     (concurrent calls race on it); the array keeps the last call's contents
 *     and each call clears what it needs before use;
 *   - the first call on each device resolves the array's device address; make
 *     that first call before beginning any stream capture.
 * On failure the message is available from b200_last_error(). */
#define B200_NOALLOC_SCAN_MAX_ELEMS (1LL << 28)
int b200_scanl1_add_i32_noalloc(const int32_t* in, int32_t* out, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif
