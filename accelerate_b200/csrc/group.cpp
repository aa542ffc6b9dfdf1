// Multi-GPU exchange steps behind the C ABI: one context (one GPU, one process or thread) per rank,
// joined into a group that owns an NCCL communicator.  The sharded skeletons need three exchanges:
// all-gather of per-rank partial results (folds, scan carries), all-reduce of privately accumulated
// permute targets, and the halo rows of row slabs between neighbouring ranks (stencils).  All of
// them are enqueued on CUDA streams of the context; none synchronises the host.
//
// NCCL is loaded at run time (dlopen), so the library has no link-time dependency on it and
// single-GPU users never touch it.  The communicator is created in non-blocking mode and every
// NCCL call is followed by a bounded wait for its completion status, so a rank that never joins
// ends in B200_ERR_TIMEOUT instead of a hang.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstring>
#include <string>
#include <thread>

#include "../../include/accelerate_b200.h"
#include "runtime.hpp"

using namespace accb200;

namespace accb200 { void set_last_error(const std::string& msg); }

namespace {

struct Nccl {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  std::string error;

  bool load() {
    if (handle) return true;
    std::vector<std::string> names;
    if (const char* e = getenv("ACCELERATE_B200_NCCL_LIB")) names.push_back(e);
    names.push_back("libnccl.so.2");
    names.push_back("libnccl.so");
    for (auto& n : names) {
      // a copy that the process already holds (e.g. the one a Python framework brought) is reused
      handle = dlopen(n.c_str(), RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
      if (!handle) handle = dlopen(n.c_str(), RTLD_NOW | RTLD_GLOBAL);
      if (handle) break;
    }
    if (!handle) { error = "NCCL (libnccl.so.2) could not be loaded; set ACCELERATE_B200_NCCL_LIB"; return false; }
    auto sym = [&](const char* s) -> void* {
      void* f = dlsym(handle, s);
      if (!f) error = std::string("NCCL symbol ") + s + " is missing";
      return f;
    };
#define B200_NCCL_SYM(field, name) field = (decltype(field))sym(name); if (!field) { handle = nullptr; return false; }
    B200_NCCL_SYM(GetUniqueId, "ncclGetUniqueId")
    B200_NCCL_SYM(CommInitRankConfig, "ncclCommInitRankConfig")
    B200_NCCL_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
    B200_NCCL_SYM(CommDestroy, "ncclCommDestroy")
    B200_NCCL_SYM(CommAbort, "ncclCommAbort")
    B200_NCCL_SYM(AllGather, "ncclAllGather")
    B200_NCCL_SYM(AllReduce, "ncclAllReduce")
    B200_NCCL_SYM(Send, "ncclSend")
    B200_NCCL_SYM(Recv, "ncclRecv")
    B200_NCCL_SYM(GroupStart, "ncclGroupStart")
    B200_NCCL_SYM(GroupEnd, "ncclGroupEnd")
    B200_NCCL_SYM(GetErrorString, "ncclGetErrorString")
#undef B200_NCCL_SYM
    return true;
  }
};

Nccl g_nccl;
std::mutex g_nccl_mu;

int fail(int code, const std::string& msg) {
  set_last_error(msg);
  return code;
}

}  // namespace

struct b200_group {
  Ctx* ctx = nullptr;
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  double deadline_s = 60.0;
  cudaStream_t comm_stream = nullptr;   // halo exchanges that overlap kernels run here
  cudaEvent_t ready = nullptr;          // compute stream -> comm stream: the rows to send exist
  cudaEvent_t halo_done = nullptr;      // comm stream -> compute stream: the halo rows have arrived
  bool halo_pending = false;
};

namespace {

// Completion of the last NCCL call(s) on a non-blocking communicator, with a host deadline.
int settle(b200_group* g, ncclResult_t r, const char* what) {
  const auto t0 = std::chrono::steady_clock::now();
  while (r == ncclInProgress) {
    ncclResult_t st = ncclSuccess;
    ncclResult_t q = g_nccl.CommGetAsyncError(g->comm, &st);
    if (q != ncclSuccess) { r = q; break; }
    r = st;
    if (r != ncclInProgress) break;
    if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > g->deadline_s) {
      g_nccl.CommAbort(g->comm);
      g->comm = nullptr;
      return fail(B200_ERR_TIMEOUT, std::string(what) + ": the other ranks did not answer within " + std::to_string((int)g->deadline_s) + " s; the group was aborted");
    }
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  if (r != ncclSuccess) return fail(B200_ERR_CUDA, std::string(what) + ": " + g_nccl.GetErrorString(r));
  return B200_OK;
}

bool nccl_type(Ty t, ncclDataType_t* out) {
  switch (t) {
    case I8: *out = ncclInt8; return true;
    case U8: *out = ncclUint8; return true;
    case I32: *out = ncclInt32; return true;
    case U32: *out = ncclUint32; return true;
    case I64: *out = ncclInt64; return true;
    case U64: *out = ncclUint64; return true;
    case F32: *out = ncclFloat32; return true;
    case F64: *out = ncclFloat64; return true;
    default: return false;      // 16-bit integers travel as bytes; they have no reduction in NCCL
  }
}

DevArrayP lookup(Ctx& c, uint64_t id) {
  auto it = c.arrays.find(id);
  if (it == c.arrays.end()) throw Error(B200_ERR_ARG, "unknown array id " + std::to_string(id));
  for (auto& b : it->second->leaf) b->fresh = false;      // about to be used on the context's streams
  return it->second;
}

}  // namespace

#define B200_GROUP_TRY try {
#define B200_GROUP_END                                                        \
  return B200_OK;                                                             \
  }                                                                           \
  catch (const Error& e) { return fail(e.code, e.what()); }                   \
  catch (const std::exception& e) { return fail(B200_ERR_ARG, e.what()); }

extern "C" {

int b200_group_unique_id(uint8_t out[B200_GROUP_ID_BYTES]) {
  std::lock_guard<std::mutex> g(g_nccl_mu);
  if (!g_nccl.load()) return fail(B200_ERR_UNSUPPORTED, g_nccl.error);
  static_assert(sizeof(ncclUniqueId) == B200_GROUP_ID_BYTES, "unique id size");
  ncclUniqueId id;
  ncclResult_t r = g_nccl.GetUniqueId(&id);
  if (r != ncclSuccess) return fail(B200_ERR_CUDA, std::string("ncclGetUniqueId: ") + g_nccl.GetErrorString(r));
  memcpy(out, &id, sizeof id);
  return B200_OK;
}

int b200_group_create(b200_ctx* ctx_, const uint8_t id_[B200_GROUP_ID_BYTES], int rank, int world, double deadline_s, b200_group** out) {
  B200_GROUP_TRY
  if (!ctx_ || !id_ || !out || world < 1 || rank < 0 || rank >= world) throw Error(B200_ERR_ARG, "bad argument");
  {
    std::lock_guard<std::mutex> g(g_nccl_mu);
    if (!g_nccl.load()) throw Error(B200_ERR_UNSUPPORTED, g_nccl.error);
  }
  Ctx& c = ctx_->c;
  auto g = std::make_unique<b200_group>();
  g->ctx = &c;
  g->rank = rank;
  g->world = world;
  if (deadline_s > 0) g->deadline_s = deadline_s;
  std::lock_guard<std::mutex> lk(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  ncclUniqueId id;
  memcpy(&id, id_, sizeof id);
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;
  ncclResult_t r = g_nccl.CommInitRankConfig(&g->comm, world, id, rank, &cfg);
  if (r != ncclSuccess && r != ncclInProgress) throw Error(B200_ERR_CUDA, std::string("ncclCommInitRankConfig: ") + g_nccl.GetErrorString(r));
  if (int rc = settle(g.get(), ncclInProgress, "b200_group_create")) return rc;
  c.check(cudaStreamCreateWithFlags(&g->comm_stream, cudaStreamNonBlocking), "cudaStreamCreate");
  c.check(cudaEventCreateWithFlags(&g->ready, cudaEventDisableTiming), "cudaEventCreate");
  c.check(cudaEventCreateWithFlags(&g->halo_done, cudaEventDisableTiming), "cudaEventCreate");
  *out = g.release();
  B200_GROUP_END
}

void b200_group_destroy(b200_group* g) {
  if (!g) return;
  if (g->ctx) {
    cudaSetDevice(g->ctx->device);
    cudaStreamSynchronize(g->ctx->stream);
    if (g->comm_stream) cudaStreamSynchronize(g->comm_stream);
  }
  if (g->comm) g_nccl.CommDestroy(g->comm);
  if (g->ready) cudaEventDestroy(g->ready);
  if (g->halo_done) cudaEventDestroy(g->halo_done);
  if (g->comm_stream) cudaStreamDestroy(g->comm_stream);
  delete g;
}

int b200_group_rank(b200_group* g, int* rank, int* world) {
  if (!g) return fail(B200_ERR_ARG, "null group");
  if (rank) *rank = g->rank;
  if (world) *world = g->world;
  return B200_OK;
}

int b200_group_all_gather(b200_group* g, uint64_t src, uint64_t* dst) {
  B200_GROUP_TRY
  if (!g || !g->comm || !dst) throw Error(B200_ERR_ARG, "bad argument (or the group was aborted)");
  Ctx& c = *g->ctx;
  std::lock_guard<std::mutex> lk(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  DevArrayP a = lookup(c, src);
  // rank r's array becomes elements [r*n, (r+1)*n) of a vector of world*n elements
  const int64_t n = a->size();
  DevArrayP out = c.new_array(a->elt, {n * g->world});
  ncclResult_t r = g_nccl.GroupStart();
  for (size_t l = 0; l < a->leaf.size() && r == ncclSuccess; ++l)
    r = g_nccl.AllGather(a->leaf[l]->ptr, out->leaf[l]->ptr, (size_t)n * ty_bytes[a->leaf_ty[l]], ncclInt8, g->comm, c.stream);
  if (r == ncclSuccess || r == ncclInProgress) r = g_nccl.GroupEnd();
  if (int rc = settle(g, r == ncclSuccess ? ncclSuccess : r, "b200_group_all_gather")) return rc;
  *dst = c.next_id++;
  c.arrays[*dst] = out;
  B200_GROUP_END
}

int b200_group_all_reduce(b200_group* g, uint64_t arr, int op) {
  B200_GROUP_TRY
  if (!g || !g->comm) throw Error(B200_ERR_ARG, "bad argument (or the group was aborted)");
  static const ncclRedOp_t ops[4] = {ncclSum, ncclMin, ncclMax, ncclProd};
  if (op < 0 || op > 3) throw Error(B200_ERR_ARG, "unknown reduction");
  Ctx& c = *g->ctx;
  std::lock_guard<std::mutex> lk(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  DevArrayP a = lookup(c, arr);
  const int64_t n = a->size();
  ncclResult_t r = g_nccl.GroupStart();
  for (size_t l = 0; l < a->leaf.size() && r == ncclSuccess; ++l) {
    ncclDataType_t t;
    if (!nccl_type(a->leaf_ty[l], &t)) {
      g_nccl.GroupEnd();
      throw Error(B200_ERR_UNSUPPORTED, "all-reduce of 16-bit integers");
    }
    r = g_nccl.AllReduce(a->leaf[l]->ptr, a->leaf[l]->ptr, (size_t)n, t, ops[op], g->comm, c.stream);
  }
  if (r == ncclSuccess || r == ncclInProgress) r = g_nccl.GroupEnd();
  if (int rc = settle(g, r, "b200_group_all_reduce")) return rc;
  B200_GROUP_END
}

int b200_group_halo_exchange(b200_group* g, uint64_t arr, int64_t top, int64_t rows, int64_t bot, int64_t radius, int up, int down,
                             int overlap) {
  B200_GROUP_TRY
  if (!g || !g->comm) throw Error(B200_ERR_ARG, "bad argument (or the group was aborted)");
  Ctx& c = *g->ctx;
  std::lock_guard<std::mutex> lk(c.mu);
  c.check(cudaSetDevice(c.device), "cudaSetDevice");
  DevArrayP a = lookup(c, arr);
  if (a->shape.size() != 2 || a->shape[0] != top + rows + bot || radius < 0 || rows < radius ||
      (up >= 0 && top != radius) || (down >= 0 && bot != radius) || up >= g->world || down >= g->world)
    throw Error(B200_ERR_ARG, "halo exchange: the array is not a (top + rows + bot) x cols slab with halo rows for the given neighbours");
  const int64_t cols = a->shape[1];
  cudaStream_t s = c.stream;
  if (overlap) {
    // the exchange runs beside the kernels submitted next; b200_group_halo_wait joins it
    c.check(cudaEventRecord(g->ready, c.stream), "cudaEventRecord");
    c.check(cudaStreamWaitEvent(g->comm_stream, g->ready, 0), "cudaStreamWaitEvent");
    s = g->comm_stream;
  }
  ncclResult_t r = g_nccl.GroupStart();
  for (size_t l = 0; l < a->leaf.size(); ++l) {
    const size_t rowb = (size_t)cols * ty_bytes[a->leaf_ty[l]];
    char* base = (char*)a->leaf[l]->ptr;
    // sends first (up, down), then receives (from down, from up): with two ranks and a wrap
    // boundary both neighbours are the same peer, and messages between one pair match in order
    if (up >= 0 && (r == ncclSuccess || r == ncclInProgress)) r = g_nccl.Send(base + (size_t)top * rowb, (size_t)radius * rowb, ncclInt8, up, g->comm, s);
    if (down >= 0 && (r == ncclSuccess || r == ncclInProgress)) r = g_nccl.Send(base + (size_t)(top + rows - radius) * rowb, (size_t)radius * rowb, ncclInt8, down, g->comm, s);
    if (down >= 0 && (r == ncclSuccess || r == ncclInProgress)) r = g_nccl.Recv(base + (size_t)(top + rows) * rowb, (size_t)radius * rowb, ncclInt8, down, g->comm, s);
    if (up >= 0 && (r == ncclSuccess || r == ncclInProgress)) r = g_nccl.Recv(base, (size_t)radius * rowb, ncclInt8, up, g->comm, s);
  }
  if (r == ncclSuccess || r == ncclInProgress) r = g_nccl.GroupEnd();
  if (int rc = settle(g, r, "b200_group_halo_exchange")) return rc;
  if (overlap) {
    c.check(cudaEventRecord(g->halo_done, g->comm_stream), "cudaEventRecord");
    g->halo_pending = true;
  }
  B200_GROUP_END
}

int b200_group_halo_wait(b200_group* g) {
  B200_GROUP_TRY
  if (!g) throw Error(B200_ERR_ARG, "null group");
  Ctx& c = *g->ctx;
  std::lock_guard<std::mutex> lk(c.mu);
  if (g->halo_pending) {
    c.check(cudaSetDevice(c.device), "cudaSetDevice");
    c.check(cudaStreamWaitEvent(c.stream, g->halo_done, 0), "cudaStreamWaitEvent");
    g->halo_pending = false;
  }
  B200_GROUP_END
}

}  // extern "C"
