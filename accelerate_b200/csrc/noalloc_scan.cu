// b200_scanl1_add_i32_noalloc: inclusive prefix sum of 32-bit integers for
// callers that are not allowed to allocate device memory.
//
// Who cannot allocate: code that runs inside somebody else's memory budget or
// on a latency path where a cudaMalloc (which may synchronise the whole device,
// or fail once the memory has been handed out) is unacceptable — for example a
// host runtime whose garbage collector owns every device byte and hands this
// library nothing but the input and output buffers, or a plugin called while a
// memory pool is frozen.  The regular entry points (b200_program_run) allocate
// their results and their look-back descriptors from the stream-ordered pool;
// this one allocates nothing at all: the caller passes input and output, and
// the descriptors of the single-pass scan live in a file-scope __device__ array.
//
// Limits and sharing rules (also stated in include/accelerate_b200.h):
//  * at most B200_NOALLOC_SCAN_MAX_ELEMS (2^28) elements per call; larger
//    inputs are refused with B200_ERR_ARG;
//  * every GPU that loads this library carries the array (about 1 MB) until
//    the process exits;
//  * all calls on one GPU share the array.  It keeps whatever the previous
//    call left, so each call first clears the words that must start at zero
//    (tile status words, ticket counter, error word).  Two calls that overlap
//    on the same GPU (different streams or threads) race on it: serialise them;
//  * the first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, once per device, with that device current).  Make
//    that first call before starting any stream capture.
//
// The kernel is the library's own single-pass scan skeleton (skeletons/scan.cuh)
// instantiated ahead of time for `scanl1 (+)` on Int32.
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <string>

#include "../../include/accelerate_b200.h"

namespace {
#include "prelude.cuh"

// ---- what the code generator would emit for scanl1 (+) over a manifest Vector Int32 ----
#define ACC_SEEDED 0
#define ACC_RIGHT 0
#define ACC_SCAN2 0
#define ACC_COMMUTATIVE 1
#define SCAN_PACKED 1
#define SCAN_T i32
#define SCAN_T_BYTES 4
#define SCAN_MIN_BLOCKS 4
struct E_i32 { i32 l0; };
typedef E_i32 elt_t;
__device__ __forceinline__ E_i32 acc_shfl_down(const E_i32& v, int d) { E_i32 r; r.l0 = acc_shfl1_down(v.l0, d); return r; }
__device__ __forceinline__ E_i32 acc_shfl_up(const E_i32& v, int d) { E_i32 r; r.l0 = acc_shfl1_up(v.l0, d); return r; }
__device__ __forceinline__ E_i32 acc_shfl_idx(const E_i32& v, int d) { E_i32 r; r.l0 = acc_shfl1_idx(v.l0, d); return r; }
struct Params {
  const i32* __restrict__ in_l0;
  i32* __restrict__ out0_l0;
  i64 n, rows, tiles_per_row, in_vec, out_vec, status, agg, incl, counter, epoch, err, spin_limit;
};
__device__ __forceinline__ E_i32 D0_get(const Params& p, i64 row, i64 j) {
  (void)row;
  E_i32 r;
  r.l0 = __ldg(p.in_l0 + j);
  return r;
}
__device__ __forceinline__ void D0_get4(const Params& p, i64 row, i64 j, E_i32 (&o)[4]) {
  (void)row;
  i32 v[4];
  acc_ld4(p.in_l0 + j, v);
#pragma unroll
  for (int k = 0; k < 4; ++k) o[k].l0 = v[k];
}
__device__ __forceinline__ E_i32 F_combine(const Params&, const E_i32& a, const E_i32& b) {
  E_i32 r;
  r.l0 = (i32)((u32)a.l0 + (u32)b.l0);  // Int32 addition wraps
  return r;
}
__device__ __forceinline__ void OUT0_store(const Params& p, i64 lin, const E_i32& v) { p.out0_l0[lin] = v.l0; }
__device__ __forceinline__ void OUT0_store4(const Params& p, i64 lin, const E_i32 (&v)[4]) {
  i32 w[4] = {v[0].l0, v[1].l0, v[2].l0, v[3].l0};
  acc_st4(p.out0_l0 + lin, w);
}
#define acc_scan acc_scan_i32_noalloc
#include "scan.cuh"
#undef acc_scan

// ---- the scratch: never allocated, never freed -------------------------------------------
constexpr long long kMaxElems = 1LL << 28;                      // B200_NOALLOC_SCAN_MAX_ELEMS
constexpr long long kMaxTiles = kMaxElems / SCAN_TILE;
constexpr size_t kHeadBytes = 256;                              // [0] ticket counter, [1] error word
constexpr size_t kStatusBytes = (size_t)kMaxTiles * 8;     // one packed {status, value} word per tile
constexpr size_t kValueBytes = (size_t)kMaxTiles * sizeof(E_i32);
constexpr size_t kScratchBytes = kHeadBytes + kStatusBytes + 2 * kValueBytes;
static __device__ __align__(256) unsigned char g_scan_scratch[kScratchBytes];

// In host code `g_scan_scratch` is only a stand-in for the symbol, not a device
// address: the address is looked up once per device and remembered here.
constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};

}  // namespace

namespace accb200 { void set_last_error(const std::string& msg); }

namespace {
int fail(int code, const std::string& msg) {
  accb200::set_last_error(msg);
  return code;
}
}  // namespace

extern "C" int b200_scanl1_add_i32_noalloc(const int32_t* in, int32_t* out, int64_t n, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n < 0) return fail(B200_ERR_ARG, "b200_scanl1_add_i32_noalloc: negative length");
  if (n > kMaxElems)
    return fail(B200_ERR_ARG, "b200_scanl1_add_i32_noalloc: " + std::to_string(n) +
                                  " elements exceed B200_NOALLOC_SCAN_MAX_ELEMS (" + std::to_string(kMaxElems) +
                                  "); the fixed scratch array cannot describe more tiles");
  if (n == 0) return B200_OK;
  if (!in || !out) return fail(B200_ERR_ARG, "b200_scanl1_add_i32_noalloc: null device pointer");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(B200_ERR_ARG, "b200_scanl1_add_i32_noalloc: device index out of range");
  unsigned char* base = nullptr;
  {
    // set-up, once per device, with that device current
    std::lock_guard<std::mutex> g(g_mu);
    if (!g_scratch_addr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_scan_scratch);
      if (e != cudaSuccess) return fail(B200_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
      g_scratch_addr[dev] = (unsigned char*)p;
    }
    base = g_scratch_addr[dev];
  }
  const long long tiles = (n + SCAN_TILE - 1) / SCAN_TILE;
  // the array keeps the previous call's contents: clear the counter, the error word and
  // the status words this call will read
  e = cudaMemsetAsync(base, 0, kHeadBytes + (size_t)tiles * 8, stream);
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
  Params p;
  p.in_l0 = in;
  p.out0_l0 = out;
  p.n = n;
  p.rows = 1;
  p.tiles_per_row = tiles;
  const bool aligned = (((uintptr_t)in | (uintptr_t)out) & 15) == 0;
  p.in_vec = aligned ? 1 : 0;
  p.out_vec = aligned ? 1 : 0;
  p.status = (i64)(uintptr_t)(base + kHeadBytes);
  p.agg = (i64)(uintptr_t)(base + kHeadBytes + kStatusBytes);
  p.incl = (i64)(uintptr_t)(base + kHeadBytes + kStatusBytes + kValueBytes);
  p.counter = (i64)(uintptr_t)(base);
  p.err = (i64)(uintptr_t)(base + 4);
  p.epoch = 1;                      // status words were just cleared, so any non-zero epoch works
  p.spin_limit = 1 << 22;
  acc_scan_i32_noalloc<<<(unsigned)tiles, SCAN_THREADS, 0, stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, std::string("kernel launch: ") + cudaGetErrorString(e));
  // synchronous by contract: the status word is read back and the stream synchronised before returning
  int err_word = 0;
  e = cudaMemcpyAsync(&err_word, base + 4, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(B200_ERR_CUDA, std::string("b200_scanl1_add_i32_noalloc: ") + cudaGetErrorString(e));
  if (err_word != 0) return fail(B200_ERR_TIMEOUT, "b200_scanl1_add_i32_noalloc: a look-back wait exceeded its limit; the output is incomplete");
  return B200_OK;
}
