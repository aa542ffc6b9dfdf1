// Runtime of the B200 backend: device arrays, kernel compilation (NVRTC) with a
// content-hashed cache, host-side evaluation of extents, and one launcher per
// array node.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "codegen.hpp"
#include "ir.hpp"

namespace accb200 {

// ---- driver entry points, resolved through the runtime (no link-time libcuda) ----
struct Driver {
  CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*ModuleGetGlobal)(CUdeviceptr*, size_t*, CUmodule, const char*) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**,
                           void**) = nullptr;
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*OccupancyMaxActiveBlocksPerMultiprocessor)(int*, CUfunction, int, size_t) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  void load();
};

// ---- compiled kernels --------------------------------------------------------------
struct CompiledKernel {
  CUmodule module = nullptr;
  CUfunction fn = nullptr;
  int max_blocks_per_sm = 0;  // for the launch configuration it was queried with
};

// Compile `source` for sm_100a; returns the cubin.  Throws Error(B200_ERR_COMPILE)
// with the NVRTC log.  Results are cached on disk by content hash.
struct CompileStats { std::atomic<long long> compiled{0}, disk_hits{0}; };
// `force` skips the disk cache lookup (and replaces the cached file).
std::string compile_to_cubin(const std::string& source, const std::string& name, CompileStats* stats, bool force = false);
std::string content_hash(const std::string& s);

// ---- device arrays -------------------------------------------------------------------
struct Ctx;
struct Buffer {
  Ctx* ctx = nullptr;
  void* ptr = nullptr;
  size_t bytes = 0;
  size_t capacity = 0;          // what was asked of the allocator (bytes rounded up to the nursery's chunk)
  bool owned = true;
  // No work that touches this block is queued on the context's main stream: it was created for the caller
  // from a nursery block whose previous owner's work had finished, and has not been handed to a program, a
  // download or an exchange since.  An upload into such a buffer need not wait for the kernels in flight.
  bool fresh = false;
  cudaEvent_t busy = nullptr;   // last asynchronous download of this buffer (on the copy-out stream)
  cudaEvent_t reuse = nullptr;  // the event that came with the block from the nursery: goes back there with it
  ~Buffer();
};
struct DevArray {
  Type elt;
  std::vector<Ty> leaf_ty;
  std::vector<int64_t> shape;
  std::vector<std::shared_ptr<Buffer>> leaf;
  // host payloads adopted but not copied yet (one per leaf, nullptr = nothing pending)
  std::vector<const void*> pending;
  int64_t size() const;
  bool aligned16() const;
};
typedef std::shared_ptr<DevArray> DevArrayP;

struct Ctx {
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  cudaStream_t d2h_stream = nullptr;   // asynchronous downloads run here, beside kernels and uploads
  cudaStream_t h2d_stream = nullptr;   // uploads run here: they wait for the copy, not for the kernels in flight
  cudaEvent_t h2d_fence = nullptr;
  // A small kernel that may run beside a large one of the same node (the frame of a staged stencil) goes
  // to this higher-priority stream, forked from and joined to `stream` with the two events.
  cudaStream_t aux_stream = nullptr;
  cudaEvent_t aux_fork = nullptr, aux_join = nullptr;
  // buffers released while a download was still reading them: freed once that copy has completed,
  // without making the main stream wait for it
  struct Deferred { void* ptr; size_t bytes, capacity; cudaEvent_t done, reuse; };
  std::vector<Deferred> deferred;
  void reap(bool wait);
  // Freed buffers wait here, by size, for the next allocation of the same size (the reference's
  // nursery, Array/Remote/Nursery.hs:55-108, searched by exact size after rounding requests up to a
  // chunk, Array/Remote/Table.hs:176-205).  A block handed back to the driver's pool may be split,
  // and getting a large block out of the pool again after a synchronisation has been seen to stall
  // the host for milliseconds; a block kept here is reused as it is.  Everything that uses a block
  // runs on `stream` (downloads on the other stream are waited for before a block gets here), so
  // reuse needs no further ordering.
  struct Nursery {
    std::mutex mu;
    struct Block { void* ptr; cudaEvent_t released; };   // `released`: recorded on the main stream when the block came here
    std::multimap<size_t, Block> blocks;
    size_t bytes = 0, limit = 0;
    long long hits = 0;
  } nursery;
  static constexpr size_t kChunk = 512;
  // into the nursery, or back to the driver when it is full; `ev` is an event to record the release with
  // (one is created when none is given)
  void release(void* ptr, size_t capacity, cudaEvent_t ev = nullptr);
  void purge();                               // everything in the nursery back to the driver
  Driver drv;
  std::mutex mu;
  std::map<uint64_t, DevArrayP> arrays;
  uint64_t next_id = 1;
  std::map<uint64_t, DevArrayP> table;   // device copies of host arrays by the host array's unique id
  // device words: [0] error status, [1] fold ticket counter, [2] scan ticket counter, [3] scan exit counter, [4..6] permute kernel choice (verdict, count, ticket)
  int* d_words = nullptr;
  // scan descriptors (persistent, epoch-tagged)
  // One region per descriptor layout (width, spacing, region offsets: the layout string), at most
  // kScanRegions of them, the least recently used one making room.  Epoch tags tell one launch from the
  // next only while status words stay where they are; under another layout the words a launch polls
  // could hold an earlier launch's VALUE bits, so layouts never share memory (clearing a shared buffer
  // at every change of layout cost a memset of up to 17 MB in front of every scan of a mixed program).
  struct ScanRegion { void* ptr = nullptr; size_t bytes = 0; uint32_t epoch = 0; uint64_t last_use = 0; };
  std::map<std::string, ScanRegion> scan_regions;
  static constexpr size_t kScanRegions = 8;
  uint64_t scan_clock = 0;
  uint32_t scan_epoch = 0;      // epoch of the launch that scan_descriptors was last called for
  std::map<std::string, CompiledKernel> kernels;  // by content hash of the source
  CompileStats cstats;
  std::atomic<long long> launches{0}, h2d{0}, d2h{0}, mem_hits{0}, allocated{0}, runs{0}, inplace_permutes{0};
  long long spin_limit = 1 << 22;

  DevArrayP new_array(const Type& elt, const std::vector<int64_t>& shape, bool for_caller = false);
  // Host -> device copy of one leaf on the upload stream; returns when the host buffer may be reused.
  void upload(Buffer& b, const void* host, size_t bytes);
  // `for_caller`: the buffer is created through the C ABI for host data (it may turn out `fresh`)
  std::shared_ptr<Buffer> alloc(size_t bytes, bool for_caller = false);
  void check(cudaError_t e, const char* what);
  void check(CUresult e, const char* what);
  CompiledKernel& kernel(const std::string& source, const std::string& entry, int threads, size_t dyn_smem);
  void* scan_descriptors(size_t bytes, const std::string& layout);
};

// ---- programs ------------------------------------------------------------------------
struct NodeState {
  Glue glue;
  bool has_glue = false;
  std::map<std::string, CompiledKernel*> kernel_memo;   // by skeleton, entry point and variant (entries of Ctx::kernels, which only grows)
};
struct Program {
  Ctx* ctx = nullptr;
  std::unique_ptr<ProgramIR> ir;
  std::vector<NodeState> nodes;                      // by Node::id, the bodies of control nodes included
  std::vector<std::vector<std::string>> dead_after;  // by Node::id: arrays whose last use is that node
  std::map<std::string, DevArrayP> constants;        // arrays embedded with (use ...), uploaded at load time
  void analyse_liveness();
  void upload_constants();                           // needs ctx; called once by b200_program_load
  void run(const std::vector<DevArrayP>& inputs, std::vector<DevArrayP>& outputs);
  // A program that is one rank-2 stencil (or stencil2) node: produce rows [row_lo, row_hi) of its
  // result in the existing array `out` (same shape and element type as the result).
  // (`row_lo2 < row_hi2`: a second range of rows, above the first, computed by the same launch)
  void run_rows(const std::vector<DevArrayP>& inputs, const DevArrayP& out, int64_t row_lo, int64_t row_hi, int64_t row_lo2 = 0, int64_t row_hi2 = 0);

 private:
  struct Window { DevArrayP out; int64_t lo, hi, lo2, hi2; };
  const Window* window = nullptr;
  typedef std::map<std::string, DevArrayP> Env;
  void liveness_of(const std::vector<Node>& nodes, const std::vector<std::string>& keep);
  void exec(const std::vector<Node>& nodes, Env& env);
  void exec_kernel_node(const Node& n, Env& env);
  std::vector<DevArrayP> call(const Body& b, const std::vector<DevArrayP>& args, Env& env);
};

// Source text of one kernel variant: prelude, defines, generated code, skeleton.
std::string assemble_source(const Glue& g, const std::string& skeleton, const std::map<std::string, std::string>& variant);
// Whether the bulk copies of the ring scan kernel would be 16-byte aligned for rows of m elements.
bool scan_ring_aligned(int elt_bytes, int64_t m, int64_t rows, bool right);
// Default variants of a node (used by the build-time compile check).
std::vector<std::pair<std::string, std::map<std::string, std::string>>> default_variants(const Node& n, const Glue& g);

}  // namespace accb200

// the handles of the C ABI
struct b200_ctx { accb200::Ctx c; };
struct b200_program { accb200::Program p; };
