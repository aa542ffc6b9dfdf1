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
typedef struct b200_group b200_group;

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
 * `elt_type` is the element type as text: i8..i64, u8..u64, f32, f64, f16 (Half, Type.hs:127: two bytes
 * per element) or "(tup t1 t2 ...)". */
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
/* The memory table (Array/Remote/Table.hs:89-100, LRU.hs:140-199): the device copy of a host array,
 * keyed by the array's unique id (Array/Unique.hs:48-51), so that an array passed to several runs is
 * uploaded once.  The first call for a key creates the device array and adopts the host payload
 * (one pointer per scalar leaf; copied at first use, as with b200_array_adopt_host, so the payload
 * must stay valid and unchanged until then); later calls with the same key return a new id for the
 * SAME device array without touching the host pointers.  Ids are released with b200_array_free as
 * usual; the table's own reference lives until b200_array_forget (the host array's finalizer,
 * Array/Remote/Table.hs:271-284) or b200_ctx_destroy.  A key seen again with another type or shape
 * is an error (B200_ERR_ARG). */
int b200_array_intern(b200_ctx* ctx, uint64_t key, const char* elt_type, int rank, const int64_t* shape,
                      const void* const* host_leaves, uint64_t* id);
int b200_array_forget(b200_ctx* ctx, uint64_t key);
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

/* For a program that is exactly one rank-2 stencil or stencil2 node: compute only rows
 * [row_lo, row_hi) of its result, into the existing array `out_id` (same shape and element type as
 * the result; the other rows are left alone).  This is how a caller splits one stencil application
 * into the rows that need freshly exchanged halo rows and the rows that do not (stencilOp,
 * Interpreter.hs:637-649, restricted to a range of its index space). */
int b200_program_run_rows(b200_program* prog, const uint64_t* in_ids, int n_in, uint64_t out_id, int64_t row_lo,
                          int64_t row_hi);
/* The same for two ranges of rows in one launch, [row_lo, row_hi) and, above it, [row_lo2, row_hi2): the rows at
 * either edge of a slab once the neighbours' halo rows have arrived. */
int b200_program_run_rows2(b200_program* prog, const uint64_t* in_ids, int n_in, uint64_t out_id, int64_t row_lo,
                           int64_t row_hi, int64_t row_lo2, int64_t row_hi2);

/* Wait for all work of the context (asynchronous downloads included) and report device-side failures. */
int b200_sync(b200_ctx* ctx);

/* Counters (monitoring.c:26-32 in the reference's cbits): [0] kernels launched,
 * [1] bytes host->device, [2] bytes device->host, [3] kernels compiled,
 * [4] kernel-cache hits (memory), [5] kernel-cache hits (disk),
 * [6] device bytes currently allocated, [7] programs run. */
int b200_stats(b200_ctx* ctx, int64_t out[8]);

/* The context's device memory: [0] bytes in live arrays, [1] bytes of freed buffers kept for reuse (the
 * reference's nursery, Array/Remote/Nursery.hs:55-117: a freed buffer is handed to the next allocation of the
 * same size, sizes being rounded up to a chunk as in Array/Remote/Table.hs:176-205), [2] buffers kept,
 * [3] allocations served from them so far, [4] permutations that updated their defaults array in place
 * because it was a temporary used only there (Language.hs:764-765). */
int b200_memory_stats(b200_ctx* ctx, int64_t out[5]);

/* Hand every kept buffer back to the driver (Table.hs:342-344, `purge`).  Done by itself when an allocation
 * fails for lack of memory. */
int b200_ctx_purge(b200_ctx* ctx);

/* The CUDA stream the context launches on (a cudaStream_t), for callers that
 * time kernels with their own events. */
int b200_ctx_stream(b200_ctx* ctx, void** stream);

/* ---- several GPUs -----------------------------------------------------------------------------
 * The reference has no multi-device backend; these entry points carry the exchange steps of the
 * data-parallel skeletons split over several GPUs (one context per GPU; contexts may live in one
 * process or in several).  Arrays are split along their outermost dimension and stay resident.
 * A group owns an NCCL communicator (NCCL is loaded at run time; B200_ERR_UNSUPPORTED if it is
 * missing).  All exchanges are enqueued on the context's streams and do not synchronise the host.
 * Every call is collective: all ranks of the group make it, in the same order.  A rank that does not
 * arrive within `deadline_s` seconds (60 if <= 0) makes the call fail with B200_ERR_TIMEOUT on the
 * others and aborts the group. */
#define B200_GROUP_ID_BYTES 128
/* A fresh rendezvous id: one rank creates it and hands the bytes to the others by any host channel. */
int b200_group_unique_id(uint8_t out[B200_GROUP_ID_BYTES]);
int b200_group_create(b200_ctx* ctx, const uint8_t id[B200_GROUP_ID_BYTES], int rank, int world, double deadline_s,
                      b200_group** out);
void b200_group_destroy(b200_group* group);
int b200_group_rank(b200_group* group, int* rank, int* world);
/* Folds and scan carries: every rank's array `src` (n elements, any rank, same n everywhere) becomes
 * elements [r*n, (r+1)*n) of a new vector of world*n elements, in rank order, on every rank. */
int b200_group_all_gather(b200_group* group, uint64_t src, uint64_t* dst);
/* Permute: element-wise reduction of `arr` over the ranks, in place.  op: 0 (+), 1 min, 2 max, 3 (*). */
int b200_group_all_reduce(b200_group* group, uint64_t arr, int op);
/* Stencils: `arr` is a (top + rows + bot) x cols row slab with `top`/`bot` spare rows for the
 * neighbours' rows.  Sends this rank's first and last `radius` rows to ranks `up` / `down` (-1 = no such
 * neighbour) and receives theirs into the spare rows.  With `overlap` the exchange runs on a second
 * stream, after everything submitted so far and beside whatever is submitted next;
 * b200_group_halo_wait makes the context's stream wait for it (call it before launching work that
 * reads the spare rows). */
int b200_group_halo_exchange(b200_group* group, uint64_t arr, int64_t top, int64_t rows, int64_t bot, int64_t radius,
                             int up, int down, int overlap);
int b200_group_halo_wait(b200_group* group);

/* Generate and NVRTC-compile every kernel of a program for sm_100a without
 * touching a GPU (build-time check).  `log` receives diagnostics. */
int b200_compile_check(const char* text, size_t len, char* log, size_t log_len);
/* Generated CUDA source of node `node` (default variant), for inspection. */
int b200_kernel_source(const char* text, size_t len, int node, char* out, size_t out_len);
/* The program as the library runs it: arrays of SIMD vectors (`(vec n t)`, Type.hs:140-152) that enter or
 * leave the program are declared as arrays of t with one more, innermost, dimension of extent n, which is
 * the reference's layout for them byte for byte (Array/Data.hs:108-119), and regrouped by a `generate`
 * each.  Text without such arrays comes back unchanged.  For inspection and for the tests. */
int b200_program_lowered(const char* text, size_t len, char* out, size_t out_len);

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
