// extern "C" surface of the backend (declared in include/accelerate_b200.h).
#include <cstring>
#include <string>

#include "../../include/accelerate_b200.h"
#include "runtime.hpp"

using namespace accb200;

namespace {
thread_local std::string g_error;

int fail(const Error& e) {
  g_error = e.what();
  return e.code;
}
int fail_std(const std::exception& e) {
  g_error = e.what();
  return B200_ERR_ARG;
}
#define B200_TRY try {
#define B200_END                     \
  return B200_OK;                    \
  }                                  \
  catch (const Error& e) { return fail(e); } \
  catch (const std::exception& e) { return fail_std(e); }

DevArrayP lookup(Ctx& c, uint64_t id) {
  auto it = c.arrays.find(id);
  if (it == c.arrays.end()) throw Error(B200_ERR_ARG, "unknown array id " + std::to_string(id));
  return it->second;
}
// the same for an array that is about to be used on the main stream (or handed out as a raw pointer)
DevArrayP lookup_used(Ctx& c, uint64_t id) {
  DevArrayP a = lookup(c, id);
  for (auto& b : a->leaf) b->fresh = false;
  return a;
}
bool mentions_vector(const Type& t) {
  if (t.vec) return true;
  for (auto& c : t.e)
    if (mentions_vector(c)) return true;
  return false;
}
// element type of an array the caller creates.  SIMD vectors have no array type of their own here: an
// `Array sh (Vec n t)` is created as an array of t of shape sh :. n, the same bytes (Array/Data.hs:108-119).
Type parse_type_text(const char* s) {
  Sx x = parse_sexp(s, strlen(s));
  Type t = parse_type(x);
  if (mentions_vector(t)) throw Error(B200_ERR_TYPE, "an array of (vec n t) is created as an array of t with one more, innermost, dimension of extent n");
  return t;
}
// every node that launches kernels, the bodies of control nodes included, in program order
void kernel_nodes(const std::vector<Node>& ns, std::vector<const Node*>& out) {
  for (auto& n : ns) {
    if (n.kind == N_USE || n.kind == N_ACOND || n.kind == N_AWHILE || n.kind == N_APPLY || n.kind == N_ATRACE) {
      for (auto& b : n.body) kernel_nodes(b.nodes, out);
    } else if (n.kind != N_RESHAPE) {
      out.push_back(&n);
    }
  }
}
void build_nodes(Program& p) {
  p.nodes.resize(p.ir->n_nodes);
  std::vector<const Node*> ks;
  kernel_nodes(p.ir->nodes, ks);
  for (const Node* n : ks) {
    p.nodes[n->id].glue = build_glue(*n, p.ir->arrays);
    p.nodes[n->id].has_glue = true;
  }
}
}  // namespace

namespace accb200 {
// lets other translation units of the library (the ahead-of-time kernels) report through b200_last_error
void set_last_error(const std::string& msg) { g_error = msg; }
}  // namespace accb200

extern "C" {

const char* b200_last_error(void) { return g_error.c_str(); }

int b200_ctx_create(int device, uint32_t flags, b200_ctx** out) {
  (void)flags;
  B200_TRY
  if (!out) throw Error(B200_ERR_ARG, "null output pointer");
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess || ndev == 0)
    throw Error(B200_ERR_CUDA, std::string("no CUDA device available (") + cudaGetErrorString(e) + "); this backend has no CPU fallback");
  if (device < 0 || device >= ndev) throw Error(B200_ERR_ARG, "device index out of range");
  auto h = std::make_unique<b200_ctx>();
  Ctx& c = h->c;
  c.device = device;
  c.check(cudaSetDevice(device), "cudaSetDevice");
  c.check(cudaFree(nullptr), "context creation");
  c.drv.load();
  cudaDeviceProp prop;
  c.check(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
  if (prop.major != 10) throw Error(B200_ERR_CUDA, "this backend is built for sm_100a (B200) only; found compute capability " +
                                                    std::to_string(prop.major) + "." + std::to_string(prop.minor));
  c.sm_count = prop.multiProcessorCount;
  c.check(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking), "cudaStreamCreate");
  c.check(cudaStreamCreateWithFlags(&c.d2h_stream, cudaStreamNonBlocking), "cudaStreamCreate");
  c.check(cudaStreamCreateWithFlags(&c.h2d_stream, cudaStreamNonBlocking), "cudaStreamCreate");
  c.check(cudaEventCreateWithFlags(&c.h2d_fence, cudaEventDisableTiming), "cudaEventCreate");
  {
    int lo = 0, hi = 0;
    c.check(cudaDeviceGetStreamPriorityRange(&lo, &hi), "cudaDeviceGetStreamPriorityRange");
    c.check(cudaStreamCreateWithPriority(&c.aux_stream, cudaStreamNonBlocking, hi), "cudaStreamCreateWithPriority");
    c.check(cudaEventCreateWithFlags(&c.aux_fork, cudaEventDisableTiming), "cudaEventCreate");
    c.check(cudaEventCreateWithFlags(&c.aux_join, cudaEventDisableTiming), "cudaEventCreate");
  }
  // keep freed blocks in the stream-ordered pool instead of returning them to the driver
  cudaMemPool_t pool;
  c.check(cudaDeviceGetDefaultMemPool(&pool, device), "cudaDeviceGetDefaultMemPool");
  uint64_t threshold = ~0ull;
  c.check(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold), "cudaMemPoolSetAttribute");
  {
    size_t free_b = 0, total_b = 0;
    c.check(cudaMemGetInfo(&free_b, &total_b), "cudaMemGetInfo");
    c.nursery.limit = total_b / 2;
  }
  c.check(cudaMalloc((void**)&c.d_words, 64), "cudaMalloc");
  c.check(cudaMemset(c.d_words, 0, 64), "cudaMemset");
  if (const char* s = getenv("ACCELERATE_B200_SPIN_LIMIT")) c.spin_limit = atoll(s);
  *out = h.release();
  B200_END
}

void b200_ctx_destroy(b200_ctx* ctx) {
  if (!ctx) return;
  Ctx& c = ctx->c;
  cudaSetDevice(c.device);
  cudaStreamSynchronize(c.stream);
  cudaStreamSynchronize(c.d2h_stream);
  if (c.aux_stream) cudaStreamSynchronize(c.aux_stream);
  {
    std::lock_guard<std::mutex> g(c.mu);
    c.arrays.clear();
    c.table.clear();
    c.reap(true);
    c.purge();
    for (auto& k : c.kernels)
      if (k.second.module) c.drv.ModuleUnload(k.second.module);
    c.kernels.clear();
    for (auto& r : c.scan_regions)
      if (r.second.ptr) cudaFreeAsync(r.second.ptr, c.stream);
    c.scan_regions.clear();
  }
  cudaStreamSynchronize(c.stream);
  cudaFree(c.d_words);
  cudaStreamDestroy(c.d2h_stream);
  if (c.h2d_fence) cudaEventDestroy(c.h2d_fence);
  if (c.h2d_stream) cudaStreamDestroy(c.h2d_stream);
  if (c.aux_fork) cudaEventDestroy(c.aux_fork);
  if (c.aux_join) cudaEventDestroy(c.aux_join);
  if (c.aux_stream) cudaStreamDestroy(c.aux_stream);
  cudaStreamDestroy(c.stream);
  delete ctx;
}

int b200_array_new(b200_ctx* ctx, const char* elt_type, int rank, const int64_t* shape, uint64_t* id) {
  B200_TRY
  if (!ctx || !elt_type || !id || rank < 0 || (rank > 0 && !shape)) throw Error(B200_ERR_ARG, "bad argument");
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  DevArrayP a = c.new_array(parse_type_text(elt_type), std::vector<int64_t>(shape, shape + rank), true);
  *id = c.next_id++;
  c.arrays[*id] = a;
  B200_END
}

int b200_array_wrap(b200_ctx* ctx, const char* elt_type, int rank, const int64_t* shape, void* const* leaf_ptrs, uint64_t* id) {
  B200_TRY
  if (!ctx || !elt_type || !id || rank < 0 || (rank > 0 && !shape) || !leaf_ptrs) throw Error(B200_ERR_ARG, "bad argument");
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.mu);
  auto a = std::make_shared<DevArray>();
  a->elt = parse_type_text(elt_type);
  a->leaf_ty = a->elt.leaves();
  a->shape.assign(shape, shape + rank);
  const int64_t n = a->size();
  for (size_t l = 0; l < a->leaf_ty.size(); ++l) {
    auto b = std::make_shared<Buffer>();
    b->ctx = &c;
    b->ptr = leaf_ptrs[l];
    b->bytes = (size_t)n * ty_bytes[a->leaf_ty[l]];
    b->owned = false;
    a->leaf.push_back(b);
  }
  *id = c.next_id++;
  c.arrays[*id] = a;
  B200_END
}

int b200_array_upload(b200_ctx* ctx, uint64_t id, int leaf, const void* host, size_t bytes) {
  B200_TRY
  if (!ctx) throw Error(B200_ERR_ARG, "null context");
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  DevArrayP a = lookup(c, id);
  if (leaf < 0 || (size_t)leaf >= a->leaf.size()) throw Error(B200_ERR_ARG, "leaf index out of range");
  if (bytes != a->leaf[leaf]->bytes) throw Error(B200_ERR_ARG, "upload size does not match the array");
  if ((size_t)leaf < a->pending.size()) a->pending[leaf] = nullptr;      // an explicit upload replaces an adopted payload
  if (bytes) {
    if (!host) throw Error(B200_ERR_ARG, "null host pointer");
    c.upload(*a->leaf[leaf], host, bytes);
  }
  B200_END
}

// Copy adopted host payloads now: the array is about to be used on the device (caller holds c.mu).
static void materialise(Ctx& c, DevArray& a) {
  for (size_t k = 0; k < a.pending.size(); ++k) {
    if (!a.pending[k]) continue;
    // (the owner of the host buffers may let go of them as soon as the call that triggered the copy returns:
    // Ctx::upload waits for the copy)
    c.upload(*a.leaf[k], a.pending[k], a.leaf[k]->bytes);
    a.pending[k] = nullptr;
  }
}

int b200_array_adopt_host(b200_ctx* ctx, uint64_t id, int leaf, const void* host, size_t bytes) {
  B200_TRY
  if (!ctx) throw Error(B200_ERR_ARG, "null context");
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.mu);
  DevArrayP a = lookup(c, id);
  if (leaf < 0 || (size_t)leaf >= a->leaf.size()) throw Error(B200_ERR_ARG, "leaf index out of range");
  if (bytes != a->leaf[leaf]->bytes) throw Error(B200_ERR_ARG, "payload size does not match the array");
  if (bytes && !host) throw Error(B200_ERR_ARG, "null host pointer");
  if (a->pending.size() != a->leaf.size()) a->pending.assign(a->leaf.size(), nullptr);
  a->pending[leaf] = bytes ? host : nullptr;
  B200_END
}

static int check_device_status(Ctx& c) {
  int words[4] = {0, 0, 0, 0};
  c.check(cudaMemcpyAsync(words, c.d_words, 4, cudaMemcpyDeviceToHost, c.stream), "cudaMemcpyAsync");
  c.check(cudaStreamSynchronize(c.stream), "cudaStreamSynchronize");
  if (words[0] != 0) {
    c.check(cudaMemsetAsync(c.d_words, 0, 16, c.stream), "cudaMemsetAsync");  // also re-arms the ticket counters
    if (words[0] == 1001) throw Error(B200_ERR_BOUNDS, "empty segment");
    if (words[0] == 1002) throw Error(B200_ERR_ARITH, "divide by zero");
    if (words[0] == 1003) throw Error(B200_ERR_BOUNDS, "index out of bounds");
    throw Error(B200_ERR_TIMEOUT, "a device-side wait exceeded its limit (status " + std::to_string(words[0]) + "); results are incomplete");
  }
  return 0;
}

int b200_array_download(b200_ctx* ctx, uint64_t id, int leaf, void* host, size_t bytes) {
  B200_TRY
  if (!ctx) throw Error(B200_ERR_ARG, "null context");
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  DevArrayP a = lookup_used(c, id);
  if (leaf < 0 || (size_t)leaf >= a->leaf.size()) throw Error(B200_ERR_ARG, "leaf index out of range");
  if (bytes != a->leaf[leaf]->bytes) throw Error(B200_ERR_ARG, "download size does not match the array");
  materialise(c, *a);
  if (bytes) {
    if (!host) throw Error(B200_ERR_ARG, "null host pointer");
    c.check(cudaMemcpyAsync(host, a->leaf[leaf]->ptr, bytes, cudaMemcpyDeviceToHost, c.stream), "cudaMemcpyAsync(D2H)");
    c.d2h += (long long)bytes;
  }
  check_device_status(c);
  B200_END
}

int b200_array_download_async(b200_ctx* ctx, uint64_t id, int leaf, void* host, size_t bytes) {
  B200_TRY
  if (!ctx) throw Error(B200_ERR_ARG, "null context");
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  DevArrayP a = lookup_used(c, id);
  if (leaf < 0 || (size_t)leaf >= a->leaf.size()) throw Error(B200_ERR_ARG, "leaf index out of range");
  if (bytes != a->leaf[leaf]->bytes) throw Error(B200_ERR_ARG, "download size does not match the array");
  materialise(c, *a);
  if (bytes) {
    if (!host) throw Error(B200_ERR_ARG, "null host pointer");
    Buffer& b = *a->leaf[leaf];
    // the copy waits for everything enqueued on the main stream so far (the array's producer among it)
    cudaEvent_t produced;
    c.check(cudaEventCreateWithFlags(&produced, cudaEventDisableTiming), "cudaEventCreate");
    c.check(cudaEventRecord(produced, c.stream), "cudaEventRecord");
    c.check(cudaStreamWaitEvent(c.d2h_stream, produced, 0), "cudaStreamWaitEvent");
    c.check(cudaEventDestroy(produced), "cudaEventDestroy");      // released once it has completed
    c.check(cudaMemcpyAsync(host, b.ptr, bytes, cudaMemcpyDeviceToHost, c.d2h_stream), "cudaMemcpyAsync(D2H)");
    if (!b.busy) c.check(cudaEventCreateWithFlags(&b.busy, cudaEventDisableTiming), "cudaEventCreate");
    c.check(cudaEventRecord(b.busy, c.d2h_stream), "cudaEventRecord");
    c.d2h += (long long)bytes;
  }
  B200_END
}

int b200_array_intern(b200_ctx* ctx, uint64_t key, const char* elt_type, int rank, const int64_t* shape,
                      const void* const* host_leaves, uint64_t* id) {
  B200_TRY
  if (!ctx || !elt_type || !id || rank < 0 || (rank > 0 && !shape)) throw Error(B200_ERR_ARG, "bad argument");
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.mu);
  const Type elt = parse_type_text(elt_type);
  const std::vector<int64_t> sh(shape, shape + rank);
  auto it = c.table.find(key);
  DevArrayP a;
  if (it != c.table.end()) {
    a = it->second;
    if (a->elt != elt || a->shape != sh) throw Error(B200_ERR_ARG, "array key " + std::to_string(key) + " was registered with another type or shape");
  } else {
    c.check(cudaSetDevice(c.device), "cudaSetDevice");
    a = c.new_array(elt, sh, true);
    if (a->size() > 0) {
      if (!host_leaves) throw Error(B200_ERR_ARG, "null host pointer");
      a->pending.assign(a->leaf.size(), nullptr);
      for (size_t l = 0; l < a->leaf.size(); ++l) {
        if (!host_leaves[l]) throw Error(B200_ERR_ARG, "null host pointer");
        a->pending[l] = host_leaves[l];
      }
    }
    c.table[key] = a;
  }
  *id = c.next_id++;
  c.arrays[*id] = a;
  B200_END
}

int b200_array_forget(b200_ctx* ctx, uint64_t key) {
  B200_TRY
  if (!ctx) throw Error(B200_ERR_ARG, "null context");
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.mu);
  c.table.erase(key);
  B200_END
}

int b200_array_free(b200_ctx* ctx, uint64_t id) {
  B200_TRY
  if (!ctx) throw Error(B200_ERR_ARG, "null context");
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.mu);
  if (!c.arrays.erase(id)) throw Error(B200_ERR_ARG, "unknown array id " + std::to_string(id));
  B200_END
}

int b200_array_rank(b200_ctx* ctx, uint64_t id, int* rank) {
  B200_TRY
  std::lock_guard<std::mutex> g(ctx->c.mu);
  *rank = (int)lookup(ctx->c, id)->shape.size();
  B200_END
}
int b200_array_shape(b200_ctx* ctx, uint64_t id, int64_t* shape) {
  B200_TRY
  std::lock_guard<std::mutex> g(ctx->c.mu);
  DevArrayP a = lookup(ctx->c, id);
  for (size_t d = 0; d < a->shape.size(); ++d) shape[d] = a->shape[d];
  B200_END
}
int b200_array_num_leaves(b200_ctx* ctx, uint64_t id, int* n) {
  B200_TRY
  std::lock_guard<std::mutex> g(ctx->c.mu);
  *n = (int)lookup(ctx->c, id)->leaf.size();
  B200_END
}
int b200_array_leaf_type(b200_ctx* ctx, uint64_t id, int leaf, const char** name) {
  B200_TRY
  std::lock_guard<std::mutex> g(ctx->c.mu);
  DevArrayP a = lookup(ctx->c, id);
  if (leaf < 0 || (size_t)leaf >= a->leaf_ty.size()) throw Error(B200_ERR_ARG, "leaf index out of range");
  *name = ty_name[a->leaf_ty[leaf]];
  B200_END
}
int b200_array_devptr(b200_ctx* ctx, uint64_t id, int leaf, void** ptr) {
  B200_TRY
  std::lock_guard<std::mutex> g(ctx->c.mu);
  DevArrayP a = lookup_used(ctx->c, id);
  if (leaf < 0 || (size_t)leaf >= a->leaf.size()) throw Error(B200_ERR_ARG, "leaf index out of range");
  ctx->c.check(cudaSetDevice(ctx->c.device), "cudaSetDevice");
  materialise(ctx->c, *a);
  *ptr = a->leaf[leaf]->ptr;
  B200_END
}

int b200_program_load(b200_ctx* ctx, const char* text, size_t len, b200_program** out) {
  B200_TRY
  if (!ctx || !text || !out) throw Error(B200_ERR_ARG, "bad argument");
  auto h = std::make_unique<b200_program>();
  h->p.ctx = &ctx->c;
  h->p.ir = parse_program(text, len);
  build_nodes(h->p);
  {
    // arrays embedded with (use ...) go to the device once, here
    Ctx& c = ctx->c;
    std::lock_guard<std::mutex> g(c.mu);
    c.check(cudaSetDevice(c.device), "cudaSetDevice");
    h->p.upload_constants();
  }
  *out = h.release();
  B200_END
}
void b200_program_free(b200_program* prog) { delete prog; }
int b200_program_num_inputs(b200_program* prog, int* n) {
  B200_TRY
  *n = (int)prog->p.ir->inputs.size();
  B200_END
}
int b200_program_num_outputs(b200_program* prog, int* n) {
  B200_TRY
  *n = (int)prog->p.ir->outputs.size();
  B200_END
}

int b200_program_run(b200_program* prog, const uint64_t* in_ids, int n_in, uint64_t* out_ids, int n_out) {
  B200_TRY
  if (!prog) throw Error(B200_ERR_ARG, "null program");
  Ctx& c = *prog->p.ctx;
  std::lock_guard<std::mutex> g(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  std::vector<DevArrayP> ins, outs;
  for (int k = 0; k < n_in; ++k) ins.push_back(lookup_used(c, in_ids[k]));
  for (auto& a : ins) materialise(c, *a);
  prog->p.run(ins, outs);
  if ((int)outs.size() != n_out) throw Error(B200_ERR_ARG, "program yields " + std::to_string(outs.size()) + " arrays");
  for (int k = 0; k < n_out; ++k) {
    out_ids[k] = c.next_id++;
    c.arrays[out_ids[k]] = outs[k];
  }
  B200_END
}

int b200_program_run_rows(b200_program* prog, const uint64_t* in_ids, int n_in, uint64_t out_id, int64_t row_lo, int64_t row_hi) {
  B200_TRY
  if (!prog) throw Error(B200_ERR_ARG, "null program");
  Ctx& c = *prog->p.ctx;
  std::lock_guard<std::mutex> g(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  std::vector<DevArrayP> ins;
  for (int k = 0; k < n_in; ++k) ins.push_back(lookup_used(c, in_ids[k]));
  for (auto& a : ins) materialise(c, *a);
  prog->p.run_rows(ins, lookup_used(c, out_id), row_lo, row_hi);
  B200_END
}

int b200_program_run_rows2(b200_program* prog, const uint64_t* in_ids, int n_in, uint64_t out_id, int64_t row_lo, int64_t row_hi,
                           int64_t row_lo2, int64_t row_hi2) {
  B200_TRY
  if (!prog) throw Error(B200_ERR_ARG, "null program");
  Ctx& c = *prog->p.ctx;
  std::lock_guard<std::mutex> g(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  std::vector<DevArrayP> ins;
  for (int k = 0; k < n_in; ++k) ins.push_back(lookup_used(c, in_ids[k]));
  for (auto& a : ins) materialise(c, *a);
  prog->p.run_rows(ins, lookup_used(c, out_id), row_lo, row_hi, row_lo2, row_hi2);
  B200_END
}

int b200_sync(b200_ctx* ctx) {
  B200_TRY
  if (!ctx) throw Error(B200_ERR_ARG, "null context");
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  c.check(cudaStreamSynchronize(c.d2h_stream), "cudaStreamSynchronize");
  c.reap(true);
  check_device_status(c);
  B200_END
}

int b200_stats(b200_ctx* ctx, int64_t out[8]) {
  B200_TRY
  Ctx& c = ctx->c;
  out[0] = c.launches;
  out[1] = c.h2d;
  out[2] = c.d2h;
  out[3] = c.cstats.compiled;
  out[4] = c.mem_hits;
  out[5] = c.cstats.disk_hits;
  out[6] = c.allocated;
  out[7] = c.runs;
  B200_END
}

int b200_memory_stats(b200_ctx* ctx, int64_t out[5]) {
  B200_TRY
  Ctx& c = ctx->c;
  std::lock_guard<std::mutex> g(c.nursery.mu);
  out[0] = c.allocated;
  out[1] = (int64_t)c.nursery.bytes;
  out[2] = (int64_t)c.nursery.blocks.size();
  out[3] = c.nursery.hits;
  out[4] = c.inplace_permutes;
  B200_END
}

int b200_ctx_purge(b200_ctx* ctx) {
  B200_TRY
  Ctx& c = ctx->c;
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  c.purge();
  B200_END
}

int b200_ctx_stream(b200_ctx* ctx, void** stream) {
  B200_TRY
  *stream = (void*)ctx->c.stream;
  B200_END
}

int b200_compile_check(const char* text, size_t len, char* log, size_t log_len) {
  std::string msg;
  int rc = B200_OK;
  try {
    Program p;
    p.ir = parse_program(text, len);
    build_nodes(p);
    std::vector<const Node*> ks;
    kernel_nodes(p.ir->nodes, ks);
    for (const Node* kn : ks) {
      for (auto& v : default_variants(*kn, p.nodes[kn->id].glue)) {
        std::string src = assemble_source(p.nodes[kn->id].glue, v.first, v.second);
        CompileStats cs;
        compile_to_cubin(src, v.first, &cs);
        msg += "ok " + v.first + " (" + std::to_string(src.size()) + " bytes of source, " + (cs.compiled ? "compiled" : "from the disk cache") + ")\n";
      }
    }
  } catch (const Error& e) {
    msg += e.what();
    rc = fail(e);
  } catch (const std::exception& e) {
    msg += e.what();
    rc = fail_std(e);
  }
  if (log && log_len) {
    size_t n = std::min(log_len - 1, msg.size());
    memcpy(log, msg.data() + (msg.size() - n), n);
    log[n] = 0;
  }
  return rc;
}

int b200_scan_ring_aligned(int elt_bytes, int64_t n, int64_t rows, int right) {
  return scan_ring_aligned(elt_bytes, n, rows, right != 0) ? 1 : 0;
}

int b200_kernel_source(const char* text, size_t len, int node, char* out, size_t out_len) {
  B200_TRY
  Program p;
  p.ir = parse_program(text, len);
  build_nodes(p);
  // `node` counts top-level nodes
  if (node < 0 || (size_t)node >= p.ir->nodes.size() || !p.nodes[p.ir->nodes[node].id].has_glue) throw Error(B200_ERR_ARG, "no such kernel node");
  const Node& kn = p.ir->nodes[node];
  auto vs = default_variants(kn, p.nodes[kn.id].glue);
  size_t which = 0;
  if (const char* e = getenv("ACCELERATE_B200_SOURCE_VARIANT")) which = (size_t)atoi(e);
  if (which >= vs.size()) throw Error(B200_ERR_ARG, "no such kernel variant");
  std::string src = assemble_source(p.nodes[kn.id].glue, vs[which].first, vs[which].second);
  if (out && out_len) {
    size_t n = std::min(out_len - 1, src.size());
    memcpy(out, src.data(), n);
    out[n] = 0;
  }
  B200_END
}

int b200_program_lowered(const char* text, size_t len, char* out, size_t out_len) {
  B200_TRY
  if (!text || !out || !out_len) throw Error(B200_ERR_ARG, "bad argument");
  const std::string src = program_text_lowered(text, len);
  if (src.size() + 1 > out_len) throw Error(B200_ERR_ARG, "buffer too small for the program text");
  memcpy(out, src.data(), src.size() + 1);
  B200_END
}

}  // extern "C"
