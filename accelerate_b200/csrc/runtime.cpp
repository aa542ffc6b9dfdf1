// Device arrays, kernel lookup, host-side extent evaluation and node launchers.
#include "runtime.hpp"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>

namespace accb200 {

// ---- driver -----------------------------------------------------------------------------
void Driver::load() {
  auto get = [](const char* name) -> void* {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qr;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &qr);
    if (e != cudaSuccess || !fn) throw Error(B200_ERR_CUDA, std::string("CUDA driver entry point '") + name + "' is unavailable");
    return fn;
  };
  ModuleLoadData = (decltype(ModuleLoadData))get("cuModuleLoadData");
  ModuleUnload = (decltype(ModuleUnload))get("cuModuleUnload");
  ModuleGetFunction = (decltype(ModuleGetFunction))get("cuModuleGetFunction");
  ModuleGetGlobal = (decltype(ModuleGetGlobal))get("cuModuleGetGlobal");
  LaunchKernel = (decltype(LaunchKernel))get("cuLaunchKernel");
  FuncSetAttribute = (decltype(FuncSetAttribute))get("cuFuncSetAttribute");
  OccupancyMaxActiveBlocksPerMultiprocessor =
      (decltype(OccupancyMaxActiveBlocksPerMultiprocessor))get("cuOccupancyMaxActiveBlocksPerMultiprocessor");
  GetErrorString = (decltype(GetErrorString))get("cuGetErrorString");
}

// ---- context ------------------------------------------------------------------------------
void Ctx::check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw Error(B200_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
void Ctx::check(CUresult e, const char* what) {
  if (e != CUDA_SUCCESS) {
    const char* s = nullptr;
    if (drv.GetErrorString) drv.GetErrorString(e, &s);
    throw Error(B200_ERR_CUDA, std::string(what) + ": " + (s ? s : "unknown driver error"));
  }
}

Buffer::~Buffer() {
  if (!ctx) return;
  if (busy) {
    cudaSetDevice(ctx->device);
    if (owned && ptr && cudaEventQuery(busy) != cudaSuccess) {
      ctx->deferred.push_back({ptr, bytes, capacity, busy, reuse});     // a download is still reading the buffer
      return;
    }
    cudaEventDestroy(busy);
  }
  if (owned && ptr) {
    cudaSetDevice(ctx->device);
    ctx->release(ptr, capacity, reuse);
    ctx->allocated -= (long long)bytes;
  } else if (reuse) {
    cudaEventDestroy(reuse);
  }
}

void Ctx::release(void* ptr, size_t capacity, cudaEvent_t ev) {
  {
    std::lock_guard<std::mutex> g(nursery.mu);
    if (capacity && nursery.bytes + capacity <= nursery.limit) {
      if (!ev && cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) ev = nullptr;
      if (ev) cudaEventRecord(ev, stream);
      nursery.blocks.emplace(capacity, Nursery::Block{ptr, ev});
      nursery.bytes += capacity;
      return;
    }
  }
  if (ev) cudaEventDestroy(ev);
  cudaFreeAsync(ptr, stream);
}

void Ctx::purge() {
  std::lock_guard<std::mutex> g(nursery.mu);
  for (auto& b : nursery.blocks) {
    if (b.second.released) cudaEventDestroy(b.second.released);
    cudaFreeAsync(b.second.ptr, stream);
  }
  nursery.blocks.clear();
  nursery.bytes = 0;
}

void Ctx::upload(Buffer& b, const void* host, size_t bytes) {
  if (!bytes) return;
  if (b.busy && cudaEventQuery(b.busy) != cudaSuccess) check(cudaStreamWaitEvent(h2d_stream, b.busy, 0), "cudaStreamWaitEvent");
  if (!b.fresh) {
    // the block may still be read or written by work queued on the main stream: the copy goes behind it
    check(cudaEventRecord(h2d_fence, stream), "cudaEventRecord");
    check(cudaStreamWaitEvent(h2d_stream, h2d_fence, 0), "cudaStreamWaitEvent");
  }
  check(cudaMemcpyAsync(b.ptr, host, bytes, cudaMemcpyHostToDevice, h2d_stream), "cudaMemcpyAsync(H2D)");
  // the caller's buffer may be reused or collected as soon as we return; and whatever is launched on the
  // main stream from now on finds the data in place
  check(cudaStreamSynchronize(h2d_stream), "cudaStreamSynchronize");
  h2d += (long long)bytes;
}

void Ctx::reap(bool wait) {
  size_t kept = 0;
  for (auto& d : deferred) {
    if (wait) cudaEventSynchronize(d.done);
    if (cudaEventQuery(d.done) == cudaSuccess) {
      cudaEventDestroy(d.done);
      release(d.ptr, d.capacity, d.reuse);
      allocated -= (long long)d.bytes;
    } else {
      deferred[kept++] = d;
    }
  }
  deferred.resize(kept);
}

std::shared_ptr<Buffer> Ctx::alloc(size_t bytes, bool for_caller) {
  auto b = std::make_shared<Buffer>();
  b->ctx = this;
  b->bytes = bytes;
  if (bytes) {
    if (!deferred.empty()) reap(false);
    const size_t cap = (bytes + kChunk - 1) / kChunk * kChunk;
    b->capacity = cap;
    {
      std::lock_guard<std::mutex> g(nursery.mu);
      auto it = nursery.blocks.find(cap);
      if (it != nursery.blocks.end()) {
        b->ptr = it->second.ptr;
        if (it->second.released) {
          b->fresh = for_caller && cudaEventQuery(it->second.released) == cudaSuccess;
          b->reuse = it->second.released;          // travels with the block
        }
        nursery.blocks.erase(it);
        nursery.bytes -= cap;
        nursery.hits++;
      }
    }
    if (!b->ptr) {
      cudaError_t e = cudaMallocAsync(&b->ptr, cap, stream);
      if (e == cudaErrorMemoryAllocation) {
        // out of memory: give the nursery back and try once more (Table.hs:199-204)
        cudaGetLastError();
        purge();
        check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        e = cudaMallocAsync(&b->ptr, cap, stream);
      }
      check(e, "cudaMallocAsync");
    }
    allocated += (long long)bytes;
  }
  return b;
}

int64_t DevArray::size() const {
  int64_t n = 1;
  for (int64_t d : shape) {
    if (d <= 0) return 0;
    n *= d;
  }
  return n;
}
bool DevArray::aligned16() const {
  for (auto& b : leaf)
    if (((uintptr_t)b->ptr & 15) != 0) return false;
  return true;
}

DevArrayP Ctx::new_array(const Type& elt, const std::vector<int64_t>& shape, bool for_caller) {
  auto a = std::make_shared<DevArray>();
  a->elt = elt;
  a->leaf_ty = elt.leaves();
  a->shape = shape;
  const int64_t n = a->size();
  for (Ty t : a->leaf_ty) a->leaf.push_back(alloc((size_t)n * ty_bytes[t], for_caller));
  return a;
}

CompiledKernel& Ctx::kernel(const std::string& source, const std::string& entry, int threads, size_t dyn_smem) {
  const std::string key = content_hash(source) + ":" + entry;
  auto it = kernels.find(key);
  if (it != kernels.end()) {
    mem_hits++;
    return it->second;
  }
  const long long hits_before = cstats.disk_hits;
  std::string cubin = compile_to_cubin(source, entry, &cstats);
  CompiledKernel k;
  CUresult lr = drv.ModuleLoadData(&k.module, cubin.data());
  if (lr != CUDA_SUCCESS && cstats.disk_hits != hits_before) {
    // the image came from the disk cache and the driver rejects it: compile afresh and replace the file
    cubin = compile_to_cubin(source, entry, &cstats, true);
    lr = drv.ModuleLoadData(&k.module, cubin.data());
  }
  check(lr, "cuModuleLoadData");
  check(drv.ModuleGetFunction(&k.fn, k.module, entry.c_str()), "cuModuleGetFunction");
  {
    // scalar helpers that can fail (integer division) report through this context's status word
    CUdeviceptr slot = 0;
    size_t slot_bytes = 0;
    if (drv.ModuleGetGlobal(&slot, &slot_bytes, k.module, "acc_status_word") == CUDA_SUCCESS && slot_bytes == sizeof(void*)) {
      void* word = d_words;
      check(cudaMemcpyAsync((void*)slot, &word, sizeof word, cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync");
      check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    }
  }
  if (dyn_smem > 32 * 1024)   // static + dynamic shared memory beyond 48 KB needs the opt-in
    check(drv.FuncSetAttribute(k.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)dyn_smem), "cuFuncSetAttribute");
  int nb = 0;
  check(drv.OccupancyMaxActiveBlocksPerMultiprocessor(&nb, k.fn, threads, dyn_smem), "cuOccupancyMaxActiveBlocksPerMultiprocessor");
  k.max_blocks_per_sm = std::max(1, nb);
  return kernels.emplace(key, k).first->second;
}

void* Ctx::scan_descriptors(size_t bytes, const std::string& layout) {
  ScanRegion& r = scan_regions[layout];
  // status words of a fresh (zeroed) region never match an epoch >= 1
  if (bytes > r.bytes || r.epoch >= (1u << 29)) {
    if (r.ptr) check(cudaFreeAsync(r.ptr, stream), "cudaFreeAsync");
    r.ptr = nullptr;
    r.bytes = 0;
    if (scan_regions.size() > kScanRegions) {
      auto victim = scan_regions.end();
      for (auto it = scan_regions.begin(); it != scan_regions.end(); ++it)
        if (&it->second != &r && (victim == scan_regions.end() || it->second.last_use < victim->second.last_use)) victim = it;
      if (victim != scan_regions.end()) {
        if (victim->second.ptr) check(cudaFreeAsync(victim->second.ptr, stream), "cudaFreeAsync");
        scan_regions.erase(victim);
      }
    }
    const size_t want = std::max(bytes, (size_t)1 << 16);
    check(cudaMallocAsync(&r.ptr, want, stream), "cudaMallocAsync");
    check(cudaMemsetAsync(r.ptr, 0, want, stream), "cudaMemsetAsync");
    r.bytes = want;
    r.epoch = 0;
  }
  r.last_use = ++scan_clock;
  scan_epoch = ++r.epoch;
  return r.ptr;
}

// The ring scan kernel fetches whole tiles with cp.async.bulk, which needs 16-byte aligned global
// addresses.  A tile of row `row` starts at element row*m + q0 (left scans) or row*m + m - q0 - tile
// (right scans) with q0 a multiple of the tile; tiles are multiples of 16 bytes, so the condition is
// on the row pitch alone, and only where it enters the address.
bool scan_ring_aligned(int elt_bytes, int64_t m, int64_t rows, bool right) {
  if (elt_bytes <= 0) return false;
  if (rows <= 1 && !right) return true;
  return (m * elt_bytes) % 16 == 0;
}

// ---- source assembly -------------------------------------------------------------------------
std::string assemble_source(const Glue& g, const std::string& skeleton, const std::map<std::string, std::string>& variant) {
  std::ostringstream o;
  // (the defines come first: they are only text, and the prelude tests some of them)
  for (auto& d : g.defines) o << "#define " << d.first << " " << d.second << "\n";
  for (auto& d : variant) o << "#define " << d.first << " " << d.second << "\n";
  o << prelude_source() << "\n";
  if (skeleton == "stencil") o << skeleton_source("stencil_pre") << "\n";
  if (skeleton == "stencil2d") o << skeleton_source("stencil2d_pre") << "\n";
  o << g.code << "\n" << skeleton_source(skeleton) << "\n";
  return o.str();
}

namespace {

struct StencilTile { int t0, t1, t2, threads; };
StencilTile stencil_tile(int rank) {
  if (rank == 1) return {1, 1, 2048, 256};
  if (rank == 2) return {1, 32, 128, 256};
  return {4, 8, 64, 256};
}
// resident CTAs per SM the scan kernel is compiled for (register budget)
constexpr int SCAN_DESC_STRIDE_DEFAULT = 16;
constexpr int SCAN_BACKOFF_DEFAULT = 0;
// elements per thread (4 per round): large tiles keep the look-back chain off the critical path
int scan_rounds(const Type& elt) {
  size_t bytes = 0;
  for (Ty t : elt.leaves()) bytes += ty_bytes[t];
  return bytes <= 8 ? 8 : 4;
}
// Short rows: the kernel's time is the latency of one tile plus the look-back chain, so many small
// tiles that all start at once beat few large ones.
constexpr int64_t SCAN_SMALL_ELEMS = 1 << 21;
constexpr int SCAN_SMALL_ROUNDS = 2;
bool scan_is_small(int64_t total_elems) {
  // ACCELERATE_B200_SCAN_NO_SMALL lets tests reach the long-row kernels with inputs a CPU check finishes quickly
  return total_elems <= SCAN_SMALL_ELEMS && !getenv("ACCELERATE_B200_SCAN_NO_SMALL");
}
std::map<std::string, std::string> scan_variant(const Type& elt, bool small = false) {
  size_t bytes = 0;
  for (Ty t : elt.leaves()) bytes += ty_bytes[t];
  const int rounds = small ? std::min(scan_rounds(elt), SCAN_SMALL_ROUNDS) : scan_rounds(elt);
  const std::string minb = bytes * rounds <= 16 ? "4" : (bytes * rounds <= 64 ? "2" : "1");
  return {{"SCAN_MIN_BLOCKS", minb}, {"SCAN_ROUNDS", std::to_string(rounds)}};
}
// Spacing of look-back descriptors (in descriptors) and pause after an unsuccessful poll.
// Spread descriptors cost total_tiles * 16 * stride bytes of scratch, so long lists of tiles stay dense.
int scan_desc_stride(int64_t total_tiles) {
  // at most 64 MiB of descriptors
  return total_tiles <= 262144 ? SCAN_DESC_STRIDE_DEFAULT : (total_tiles <= 1048576 ? 4 : 1);
}
void scan_poll_variant(std::map<std::string, std::string>& v, int64_t total_tiles) {
  v["SCAN_DESC_STRIDE"] = std::to_string(scan_desc_stride(total_tiles));
  v["SCAN_BACKOFF_NS"] = std::to_string(SCAN_BACKOFF_DEFAULT);
}
// Shape of the shared-memory ring scan kernel: tiles of 1024*rounds elements, `slots` tiles in flight per
// CTA, `minb` CTAs per SM, one look-back and one reducer warp, `look` descriptors polled per lane step,
// finishers take a slot once it is scanned (grab 1), one look-back descriptor per `batch` tiles.
struct RingShape { int rounds, slots, minb, lbw, redw, look, grab, batch; };
RingShape scan_ring_shape(int bytes) { return {bytes <= 4 ? 8 : 4, 3, 2, 1, 1, 4, 1, 2}; }
std::map<std::string, std::string> scan_ring_variant(const RingShape& r, int64_t total_tiles) {
  std::map<std::string, std::string> v = {{"SCAN_RING", "1"}, {"SCAN_ROUNDS", std::to_string(r.rounds)}, {"SCAN_SLOTS", std::to_string(r.slots)},
                                          {"SCAN_MIN_BLOCKS", std::to_string(r.minb)}, {"SCAN_LB_WARPS", std::to_string(r.lbw)},
                                          {"RING_RED_WARPS", std::to_string(r.redw)}, {"SCAN_LOOK", std::to_string(r.look)},
                                          {"RING_GRAB_STATE", std::to_string(r.grab)}, {"RING_BATCH", std::to_string(r.batch)}};
  scan_poll_variant(v, total_tiles);
  return v;
}
// launch shape of the register-window rank-2 stencil kernel: warps per CTA, rows per warp task,
// CTAs per SM asked of the compiler, rows loaded ahead
struct Stencil2dShape { int warps, rows, minb, depth; };
Stencil2dShape stencil2d_shape() { return {4, 32, 1, 4}; }
// acc_stencil2d_bulk: warps per CTA, CTAs per SM asked of the compiler, row slots per warp, rows per warp
// task, and the bytes per point (all inputs) from which it replaces the register kernel
struct Stencil2dBulkShape { int warps, minb, slots, rows, min_point_bytes; };
Stencil2dBulkShape stencil2d_bulk_shape() { return {4, 4, 8, 64, 8}; }
std::map<std::string, std::string> stencil2d_bulk_variant(const Stencil2dBulkShape& bs) {
  return {{"ST2_BULK", "1"}, {"ACC_OPT_PARAMS", "1"}, {"ST2_DEPTH", "0"}, {"SCAN_TILE", "128"}, {"ST2_WARPS", std::to_string(bs.warps)},
          {"ST2_MIN_BLOCKS", std::to_string(bs.minb)}, {"ST2B_SLOTS", std::to_string(bs.slots)}, {"ST2B_ROWS", std::to_string(bs.rows)}};
}
std::map<std::string, std::string> stencil2d_variant();
std::map<std::string, std::string> stencil2d_frame_variant() {
  std::map<std::string, std::string> v = stencil2d_variant();
  v["ST2_FRAME"] = "1";
  v["ACC_OPT_PARAMS"] = "1";
  v["ST2_ROWS"] = "8";
  return v;
}
std::map<std::string, std::string> stencil2d_variant() {
  Stencil2dShape s = stencil2d_shape();
  return {{"ST2_WARPS", std::to_string(s.warps)}, {"ST2_ROWS", std::to_string(s.rows)}, {"ST2_MIN_BLOCKS", std::to_string(s.minb)},
          {"ST2_DEPTH", std::to_string(s.depth)}};
}
std::map<std::string, std::string> stencil_variant(int rank) {
  StencilTile t = stencil_tile(rank);
  return {{"ST_T0", std::to_string(t.t0)}, {"ST_T1", std::to_string(t.t1)}, {"ST_T2", std::to_string(t.t2)},
          {"ST_THREADS", std::to_string(t.threads)}};
}

}  // namespace

std::vector<std::pair<std::string, std::map<std::string, std::string>>> default_variants(const Node& n, const Glue& g) {
  std::vector<std::pair<std::string, std::map<std::string, std::string>>> v;
  switch (n.kind) {
    case N_GENERATE: v.push_back({"elementwise", {}}); break;
    case N_FOLD:
      v.push_back({"fold", {{"FOLD_G", "32"}, {"ACC_STREAM_LOADS", "1"}}});
      v.push_back({"fold", {{"FOLD_G", "4"}, {"ACC_STREAM_LOADS", "1"}}});
      break;
    case N_FOLDSEG: v.push_back({"foldseg", {{"FOLDSEG_G", "32"}, {"ACC_STREAM_LOADS", "1"}}}); break;
    case N_SCAN: case N_SCAN2: {
      for (bool small : {false, true}) {
        auto sv = scan_variant(n.elt, small);
        scan_poll_variant(sv, 1);
        v.push_back({"scan", sv});
      }
      if (g.defines.count("D0_STREAM_NLEAVES") && g.defines.at("D0_STREAM_NLEAVES") == "1" && g.defines.at("SCAN_PACKED") == "1" &&
          g.defines.at("D0_STREAM_BYTES") == g.defines.at("SCAN_T_BYTES"))
        v.push_back({"scan", scan_ring_variant(scan_ring_shape(atoi(g.defines.at("SCAN_T_BYTES").c_str())), 1)});
      break;
    }
    case N_PERMUTE: {
      v.push_back({"permute", {}});
      const std::string& m = g.defines.at("PERMUTE_MODE");
      if (m.find("ATOMIC") != std::string::npos) {
        v.push_back({"permute", {{"PERMUTE_SMEM", "1"}, {"PERMUTE_THREADS", "1024"}}});
        if (m == "PERMUTE_ATOMIC_ADD" && g.defines.at("PERMUTE_BYTES") == "4" && g.defines.at("PERMUTE_FLOAT") == "0")
        {
          v.push_back({"permute", {{"PERMUTE_SMEM16", "1"}, {"PERMUTE_THREADS", "1024"}, {"PERMUTE_CHOICE_ID", "1"}}});
          v.push_back({"permute", {{"PERMUTE_SAMPLE", "1"}}});
        }
      }
      break;
    }
    case N_STENCIL: case N_STENCIL2:
      v.push_back({"stencil", stencil_variant(n.d[0].rank)});
      if (n.d[0].rank == 2) {
        v.push_back({"stencil2d", stencil2d_variant()});
        if (g.defines.count("ST2_BULK_OK") && g.defines.at("ST2_BULK_OK") == "1") {
          v.push_back({"stencil2d", stencil2d_bulk_variant(stencil2d_bulk_shape())});
          v.push_back({"stencil2d", stencil2d_frame_variant()});
        }
        {
          auto tv = stencil2d_variant();
          tv["ST2_TWOWIN"] = "1";
          tv["ACC_OPT_PARAMS"] = "1";
          v.push_back({"stencil2d", tv});
        }
      }
      break;
    default: break;   // reshape and the host-evaluated nodes launch nothing
  }
  return v;
}

// ---- host-side evaluation of closed scalar expressions (extents, sizes) ----------------------
namespace {

struct HVal {
  Type ty;
  std::vector<int64_t> i;   // integer leaves (also Bool)
  std::vector<double> f;    // floating leaves (parallel vector; the unused one is 0)
};

struct HostEval {
  Ctx* ctx;
  const std::map<std::string, DevArrayP>* env;
  std::vector<std::pair<std::string, HVal>> vars;

  const DevArray& array(const std::string& n) {
    auto it = env->find(n);
    if (it == env->end() || !it->second) throw Error(B200_ERR_ARG, "array '" + n + "' is not bound");
    return *it->second;
  }
  static int64_t wrap(Ty t, uint64_t v) {
    switch (t) {
      case I8: return (int8_t)v; case I16: return (int16_t)v; case I32: return (int32_t)v;
      case U8: return (uint8_t)v; case U16: return (uint16_t)v; case U32: return (uint32_t)v;
      default: return (int64_t)v;
    }
  }
  HVal scalar_i(Ty t, int64_t v) { HVal r; r.ty = Type::scalar(t); r.i = {v}; r.f = {0}; return r; }
  HVal scalar_f(Ty t, double v) {
    if (t == F32) v = (double)(float)v;
    if (t == F16) v = (double)half_to_float(half_from_float((float)v));  // through Float, as Numeric.Half does
    HVal r; r.ty = Type::scalar(t); r.i = {0}; r.f = {v}; return r;
  }
  HVal read(const DevArray& a, int64_t lin) {
    if (lin < 0 || lin >= a.size()) throw Error(B200_ERR_BOUNDS, "index out of bounds");
    HVal r;
    r.ty = a.elt;
    for (size_t l = 0; l < a.leaf_ty.size(); ++l) {
      Ty t = a.leaf_ty[l];
      unsigned char buf[8] = {0};
      ctx->check(cudaMemcpyAsync(buf, (char*)a.leaf[l]->ptr + lin * ty_bytes[t], ty_bytes[t], cudaMemcpyDeviceToHost, ctx->stream), "cudaMemcpyAsync");
      ctx->check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
      ctx->d2h += ty_bytes[t];
      if (t == F32) { float v; memcpy(&v, buf, 4); r.i.push_back(0); r.f.push_back(v); }
      else if (t == F64) { double v; memcpy(&v, buf, 8); r.i.push_back(0); r.f.push_back(v); }
      else if (t == F16) { uint16_t v; memcpy(&v, buf, 2); r.i.push_back(0); r.f.push_back((double)half_to_float(v)); }
      else { uint64_t v = 0; memcpy(&v, buf, ty_bytes[t]); r.i.push_back(wrap(t, v)); r.f.push_back(0); }
    }
    return r;
  }
  HVal eval(const Expr& e) {
    switch (e.kind) {
      case X_CONST: {
        Ty t = e.ty.s;
        if (ty_is_float(t)) return scalar_f(t, e.lit == "inf" ? 1e308 * 10 : (e.lit == "-inf" ? -1e308 * 10 : strtod(e.lit.c_str(), nullptr)));
        if (ty_is_signed(t)) return scalar_i(t, wrap(t, (uint64_t)strtoll(e.lit.c_str(), nullptr, 10)));
        return scalar_i(t, wrap(t, strtoull(e.lit.c_str(), nullptr, 10)));
      }
      case X_VAR:
        for (size_t k = vars.size(); k-- > 0;)
          if (vars[k].first == e.name) return vars[k].second;
        throw Error(B200_ERR_TYPE, "unbound variable in host expression");
      case X_LET: {
        vars.emplace_back(e.name, eval(*e.a[0]));
        HVal r = eval(*e.a[1]);
        vars.pop_back();
        return r;
      }
      case X_TUP: {
        HVal r;
        r.ty = e.ty;
        for (auto& c : e.a) {
          HVal v = eval(*c);
          r.i.insert(r.i.end(), v.i.begin(), v.i.end());
          r.f.insert(r.f.end(), v.f.begin(), v.f.end());
        }
        return r;
      }
      case X_SNOC: {
        HVal r;
        r.ty = e.ty;
        for (auto& c : e.a) {
          HVal v = eval(*c);
          r.i.insert(r.i.end(), v.i.begin(), v.i.end());
          r.f.insert(r.f.end(), v.f.begin(), v.f.end());
        }
        return r;
      }
      case X_INIT: {
        HVal v = eval(*e.a[0]);
        size_t drop = v.ty.e.back().nleaves();
        HVal r;
        r.ty = e.ty;
        r.i.assign(v.i.begin(), v.i.end() - drop);
        r.f.assign(v.f.begin(), v.f.end() - drop);
        return r;
      }
      case X_PRJ: {
        HVal v = eval(*e.a[0]);
        size_t off = 0;
        for (int k = 0; k < e.n; ++k) off += v.ty.e[k].nleaves();
        size_t cnt = v.ty.e[e.n].nleaves();
        HVal r;
        r.ty = e.ty;
        r.i.assign(v.i.begin() + off, v.i.begin() + off + cnt);
        r.f.assign(v.f.begin() + off, v.f.begin() + off + cnt);
        return r;
      }
      case X_COND: return eval(*e.a[0]).i[0] != 0 ? eval(*e.a[1]) : eval(*e.a[2]);
      case X_SHAPE: {
        const DevArray& a = array(e.name);
        HVal r;
        r.ty = e.ty;
        r.i = a.shape;
        r.f.assign(a.shape.size(), 0);
        return r;
      }
      case X_SHAPESIZE: {
        HVal s = eval(*e.a[0]);
        int64_t n = 1;
        for (int64_t d : s.i) n = d <= 0 ? 0 : n * d;
        for (int64_t d : s.i) if (d <= 0) n = 0;
        return scalar_i(I64, n);
      }
      case X_TOINDEX: {
        HVal sh = eval(*e.a[0]), ix = eval(*e.a[1]);
        int64_t r = 0;
        for (size_t d = 0; d < sh.i.size(); ++d) r = r * sh.i[d] + ix.i[d];
        return scalar_i(I64, r);
      }
      case X_FROMINDEX: {
        HVal sh = eval(*e.a[0]);
        int64_t i = eval(*e.a[1]).i[0];
        HVal r;
        r.ty = e.ty;
        r.i.assign(sh.i.size(), 0);
        r.f.assign(sh.i.size(), 0);
        for (size_t d = sh.i.size(); d-- > 0;) {
          if (d == 0) { r.i[0] = i; break; }
          if (sh.i[d] == 0) throw Error(B200_ERR_ARITH, "divide by zero");
          r.i[d] = i % sh.i[d];
          i /= sh.i[d];
        }
        return r;
      }
      case X_INDEX: {
        const DevArray& a = array(e.name);
        HVal ix = eval(*e.a[0]);
        int64_t lin = 0;
        for (size_t d = 0; d < a.shape.size(); ++d) {
          if (ix.i[d] < 0 || ix.i[d] >= a.shape[d]) throw Error(B200_ERR_BOUNDS, "index out of bounds");
          lin = lin * a.shape[d] + ix.i[d];
        }
        return read(a, lin);
      }
      case X_LINDEX: return read(array(e.name), eval(*e.a[0]).i[0]);
      case X_APP: {
        std::vector<HVal> args;
        for (auto& c : e.a) args.push_back(eval(*c));
        size_t mark = vars.size();
        for (size_t k = 0; k < args.size(); ++k) vars.emplace_back(e.f[0]->params[k], args[k]);
        HVal r = eval(*e.f[0]->body);
        vars.resize(mark);
        return r;
      }
      case X_PRIM: {
        std::vector<HVal> x;
        for (auto& c : e.a) x.push_back(eval(*c));
        if (x.size() == 1 && x[0].ty.tuple) {
          HVal a = x[0];
          x.clear();
          x.push_back(scalar_i(e.t1, a.i[0]));
          x.back().f[0] = a.f[0];
          x.push_back(scalar_i(e.t1, a.i[1]));
          x.back().f[0] = a.f[1];
        }
        const Ty t = e.t1;
        if (ty_is_float(t)) {
          double a = x[0].f[0], b = x.size() > 1 ? x[1].f[0] : 0;
          switch (e.op) {
            case P_ADD: return scalar_f(t, a + b);
            case P_SUB: return scalar_f(t, a - b);
            case P_MUL: return scalar_f(t, a * b);
            case P_FDIV: return scalar_f(t, a / b);
            case P_LT: return scalar_i(U8, a < b);
            case P_GT: return scalar_i(U8, a > b);
            case P_LE: return scalar_i(U8, a <= b);
            case P_GE: return scalar_i(U8, a >= b);
            case P_EQ: return scalar_i(U8, a == b);
            case P_NE: return scalar_i(U8, a != b);
            case P_TRUNCATE: return scalar_i(e.t2, wrap(e.t2, (uint64_t)(int64_t)a));
            default: break;
          }
          throw Error(B200_ERR_UNSUPPORTED, std::string("host evaluation of floating primitive '") + prim_name[e.op] + "'");
        }
        int64_t a = x[0].i[0], b = x.size() > 1 ? x[1].i[0] : 0;
        const bool sg = ty_is_signed(t);
        auto W = [&](uint64_t v) { return scalar_i(t, wrap(t, v)); };
        switch (e.op) {
          case P_ADD: return W((uint64_t)a + (uint64_t)b);
          case P_SUB: return W((uint64_t)a - (uint64_t)b);
          case P_MUL: return W((uint64_t)a * (uint64_t)b);
          case P_NEG: return W((uint64_t)0 - (uint64_t)a);
          case P_ABS: return W(sg && a < 0 ? (uint64_t)0 - (uint64_t)a : (uint64_t)a);
          case P_MIN: return W((sg ? a <= b : (uint64_t)a <= (uint64_t)b) ? a : b);
          case P_MAX: return W((sg ? a <= b : (uint64_t)a <= (uint64_t)b) ? b : a);
          case P_QUOT: case P_REM: case P_IDIV: case P_MOD: {
            if (b == 0) throw Error(B200_ERR_ARITH, "divide by zero");
            int64_t q, r;
            if (sg) {
              if (b == -1) { q = (int64_t)((uint64_t)0 - (uint64_t)a); r = 0; }
              else { q = a / b; r = a % b; }
              if ((e.op == P_IDIV || e.op == P_MOD) && r != 0 && ((r < 0) != (b < 0))) { q -= 1; r += b; }
            } else {
              q = (int64_t)((uint64_t)a / (uint64_t)b);
              r = (int64_t)((uint64_t)a % (uint64_t)b);
            }
            return W((uint64_t)((e.op == P_QUOT || e.op == P_IDIV) ? q : r));
          }
          case P_LT: return scalar_i(U8, sg ? a < b : (uint64_t)a < (uint64_t)b);
          case P_GT: return scalar_i(U8, sg ? a > b : (uint64_t)a > (uint64_t)b);
          case P_LE: return scalar_i(U8, sg ? a <= b : (uint64_t)a <= (uint64_t)b);
          case P_GE: return scalar_i(U8, sg ? a >= b : (uint64_t)a >= (uint64_t)b);
          case P_EQ: return scalar_i(U8, a == b);
          case P_NE: return scalar_i(U8, a != b);
          case P_LAND: return scalar_i(U8, a != 0 && b != 0);
          case P_LOR: return scalar_i(U8, a != 0 || b != 0);
          case P_LNOT: return scalar_i(U8, a == 0);
          case P_FROMINTEGRAL:
            if (ty_is_float(e.t2)) return scalar_f(e.t2, sg ? (double)a : (double)(uint64_t)a);
            return scalar_i(e.t2, wrap(e.t2, (uint64_t)a));
          default: break;
        }
        throw Error(B200_ERR_UNSUPPORTED, std::string("host evaluation of primitive '") + prim_name[e.op] + "'");
      }
      default: break;
    }
    throw Error(B200_ERR_UNSUPPORTED, "expression form not supported in an extent");
  }
};

// ---- launching ----------------------------------------------------------------------------------
struct Launcher {
  Ctx* ctx;
  const std::map<std::string, DevArrayP>* env;
  const Glue* glue;
  std::map<std::string, int64_t> named;
  std::vector<DevArrayP> outs;

  DevArrayP arr(const std::string& n) const {
    auto it = env->find(n);
    if (it == env->end() || !it->second) throw Error(B200_ERR_ARG, "array '" + n + "' is not bound");
    return it->second;
  }
  std::vector<uint64_t> block() const {
    std::vector<uint64_t> pb;
    for (auto& s : glue->slots) {
      switch (s.kind) {
        case Slot::ARR_LEAF: pb.push_back((uint64_t)(uintptr_t)arr(s.name)->leaf[s.idx]->ptr); break;
        case Slot::ARR_DIM: pb.push_back((uint64_t)arr(s.name)->shape[s.idx]); break;
        case Slot::OUT_LEAF: pb.push_back((uint64_t)(uintptr_t)outs.at(s.idx / 64)->leaf[s.idx % 64]->ptr); break;
        case Slot::NAMED: {
          auto it = named.find(s.name);
          pb.push_back(it == named.end() ? 0 : (uint64_t)it->second);
          break;
        }
      }
    }
    if (pb.empty()) pb.push_back(0);
    if (pb.size() * 8 > 4000) throw Error(B200_ERR_UNSUPPORTED, "kernel parameter block exceeds 4 KB");
    return pb;
  }
  void launch(CompiledKernel& k, int64_t grid, int threads, size_t smem, cudaStream_t on = nullptr) {
    if (grid <= 0) return;
    if (grid > 2147483647LL) throw Error(B200_ERR_UNSUPPORTED, "grid too large");
    std::vector<uint64_t> pb = block();
    void* args[1] = {pb.data()};
    ctx->check(ctx->drv.LaunchKernel(k.fn, (unsigned)grid, 1, 1, (unsigned)threads, 1, 1, (unsigned)smem, (CUstream)(on ? on : ctx->stream), args, nullptr),
               "cuLaunchKernel");
    ctx->launches++;
  }
  // extent of a delayed operand + whether its streams all have exactly that shape
  void bind_delayed(const std::string& D, const std::vector<int64_t>& ext, size_t k) {
    bool fast = true;
    for (auto& a : glue->streams.at(k)) {
      DevArrayP x = arr(a);
      if (x->shape != ext || !x->aligned16()) fast = false;
    }
    for (size_t d = 0; d < ext.size(); ++d) named[D + "_e" + std::to_string(d)] = ext[d];
    named[D + "_fast"] = fast ? 1 : 0;
  }
  bool fast(const std::string& D) const { return named.at(D + "_fast") != 0; }
};

int64_t prod_outer(const std::vector<int64_t>& sh) {
  int64_t r = 1;
  for (size_t d = 0; d + 1 < sh.size(); ++d) r = sh[d] <= 0 ? 0 : r * sh[d];
  for (size_t d = 0; d + 1 < sh.size(); ++d) if (sh[d] <= 0) r = 0;
  return r;
}
int64_t size_of(const std::vector<int64_t>& sh) {
  int64_t r = 1;
  for (int64_t d : sh) if (d <= 0) return 0; else r *= d;
  return r;
}
int pow2_at_least(int64_t v) {
  int g = 1;
  while (g < v && g < 32) g <<= 1;
  return g;
}
size_t struct_bytes(const Type& elt) {
  // size of the generated element struct (natural alignment, C layout)
  size_t off = 0, maxa = 1;
  for (Ty t : elt.leaves()) {
    size_t a = ty_bytes[t];
    off = (off + a - 1) / a * a + a;
    maxa = std::max(maxa, a);
  }
  off = (off + maxa - 1) / maxa * maxa;
  return std::max(off, (size_t)1);
}

}  // namespace

// Arrays are released right after their last use, so a chain of nodes (e.g. one
// hundred stencil iterations) holds two or three arrays at a time, not all of them.
// Inside the body of a control node only the arrays the body defines are released there; a control
// node counts as a use of every array its bodies mention.
void Program::liveness_of(const std::vector<Node>& ns, const std::vector<std::string>& keep) {
  std::map<std::string, int> last;        // array defined in this list -> id of the node that uses it last
  std::map<std::string, bool> local;
  for (auto& n : ns)
    for (auto& o : n.outs) local[o] = true;
  for (auto& n : ns) {
    std::vector<std::string> used;
    node_arrays(n, used);
    for (auto& u : used)
      if (local.count(u)) last[u] = n.id;
    for (auto& o : n.outs)
      if (!last.count(o)) last[o] = n.id;  // never read: dies where it is born
    for (auto& b : n.body) {
      std::vector<std::string> k = b.outs;
      liveness_of(b.nodes, k);
    }
  }
  for (auto& kv : last) {
    bool kept = false;
    for (auto& o : keep) kept = kept || o == kv.first;
    if (!kept) dead_after[kv.second].push_back(kv.first);
  }
}

void Program::analyse_liveness() {
  dead_after.assign(ir->n_nodes, {});
  liveness_of(ir->nodes, ir->outputs);
}

void Program::upload_constants() {
  std::vector<const Node*> todo;
  std::vector<const std::vector<Node>*> stack = {&ir->nodes};
  while (!stack.empty()) {
    const std::vector<Node>* ns = stack.back();
    stack.pop_back();
    for (auto& n : *ns) {
      if (n.kind == N_USE) todo.push_back(&n);
      for (auto& b : n.body) stack.push_back(&b.nodes);
    }
  }
  for (const Node* n : todo) {
    DevArrayP a = ctx->new_array(n->elt, n->use_shape);
    for (size_t l = 0; l < a->leaf.size(); ++l)
      if (a->leaf[l]->bytes) {
        ctx->check(cudaMemcpyAsync(a->leaf[l]->ptr, n->use_data[l].data(), a->leaf[l]->bytes, cudaMemcpyHostToDevice, ctx->stream), "cudaMemcpyAsync(H2D)");
        ctx->h2d += (long long)a->leaf[l]->bytes;
      }
    constants[n->outs[0]] = a;
  }
  if (!todo.empty()) ctx->check(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
}

void Program::run(const std::vector<DevArrayP>& inputs, std::vector<DevArrayP>& outputs) {
  Ctx& c = *ctx;
  if ((int)dead_after.size() != ir->n_nodes) analyse_liveness();
  if (inputs.size() != ir->inputs.size()) throw Error(B200_ERR_ARG, "wrong number of input arrays");
  Env env;
  for (size_t k = 0; k < inputs.size(); ++k) {
    const ArrayInfo& ai = ir->arrays.at(ir->inputs[k]);
    if (!inputs[k] || inputs[k]->elt != ai.elt || (int)inputs[k]->shape.size() != ai.rank)
      throw Error(B200_ERR_ARG, "input '" + ir->inputs[k] + "' has the wrong element type or rank");
    env[ir->inputs[k]] = inputs[k];
  }
  c.runs++;
  exec(ir->nodes, env);
  outputs.clear();
  for (auto& o : ir->outputs) outputs.push_back(env.at(o));
}

void Program::run_rows(const std::vector<DevArrayP>& inputs, const DevArrayP& out, int64_t row_lo, int64_t row_hi, int64_t row_lo2, int64_t row_hi2) {
  if (ir->nodes.size() != 1 || (ir->nodes[0].kind != N_STENCIL && ir->nodes[0].kind != N_STENCIL2) || ir->outputs.size() != 1 ||
      ir->outputs[0] != ir->nodes[0].outs[0])
    throw Error(B200_ERR_ARG, "a row window needs a program that is exactly one stencil node");
  if (!out) throw Error(B200_ERR_ARG, "null output array");
  if (row_lo2 < row_hi2 && (row_lo2 < row_hi || row_lo >= row_hi)) throw Error(B200_ERR_ARG, "row windows: the second range must lie above a non-empty first one");
  Window w{out, row_lo, row_hi, row_lo2, std::max(row_lo2, row_hi2)};
  struct Guard { const Window*& slot; ~Guard() { slot = nullptr; } } guard{window};
  window = &w;
  std::vector<DevArrayP> outs;
  run(inputs, outs);
}

// Evaluate an array-level function: bind the parameters, run the nodes, collect the results and
// drop everything the body defined.
std::vector<DevArrayP> Program::call(const Body& b, const std::vector<DevArrayP>& args, Env& env) {
  if (args.size() != b.params.size()) throw Error(B200_ERR_ARG, "array function applied to the wrong number of arguments");
  for (size_t k = 0; k < args.size(); ++k) env[b.params[k]] = args[k];
  exec(b.nodes, env);
  std::vector<DevArrayP> r;
  for (auto& o : b.outs) r.push_back(env.at(o));
  for (auto& pn : b.params) env.erase(pn);
  for (auto& n : b.nodes)
    for (auto& o : n.outs) env.erase(o);
  return r;
}

// "Vector (Z :. 3) [1,2,3]": constructor by rank, shape, elements in row-major order (tuples in parentheses).
static std::string trace_render(Ctx& c, const DevArray& a) {
  const int64_t n = a.size();
  std::vector<std::string> host(a.leaf.size());
  for (size_t l = 0; l < a.leaf.size(); ++l) {
    host[l].resize((size_t)n * ty_bytes[a.leaf_ty[l]]);
    if (n) c.check(cudaMemcpyAsync(&host[l][0], a.leaf[l]->ptr, host[l].size(), cudaMemcpyDeviceToHost, c.stream), "cudaMemcpyAsync");
  }
  c.check(cudaStreamSynchronize(c.stream), "cudaStreamSynchronize");
  const size_t rank = a.shape.size();
  std::string out = rank == 0 ? "Scalar" : rank == 1 ? "Vector" : rank == 2 ? "Matrix" : "Array";
  out += rank ? " (Z" : " Z";
  for (int64_t d : a.shape) out += " :. " + std::to_string(d);
  out += rank ? ") [" : " [";
  char buf[64];
  for (int64_t i = 0; i < n; ++i) {
    if (i) out += ",";
    if (a.leaf.size() > 1) out += "(";
    for (size_t l = 0; l < a.leaf.size(); ++l) {
      if (l) out += ",";
      const char* q = host[l].data() + (size_t)i * ty_bytes[a.leaf_ty[l]];
      switch (a.leaf_ty[l]) {
        case I8: snprintf(buf, sizeof buf, "%d", (int)*(const int8_t*)q); break;
        case I16: { int16_t v; memcpy(&v, q, 2); snprintf(buf, sizeof buf, "%d", (int)v); break; }
        case I32: { int32_t v; memcpy(&v, q, 4); snprintf(buf, sizeof buf, "%d", v); break; }
        case I64: { int64_t v; memcpy(&v, q, 8); snprintf(buf, sizeof buf, "%lld", (long long)v); break; }
        case U8: snprintf(buf, sizeof buf, "%u", (unsigned)*(const uint8_t*)q); break;
        case U16: { uint16_t v; memcpy(&v, q, 2); snprintf(buf, sizeof buf, "%u", (unsigned)v); break; }
        case U32: { uint32_t v; memcpy(&v, q, 4); snprintf(buf, sizeof buf, "%u", v); break; }
        case U64: { uint64_t v; memcpy(&v, q, 8); snprintf(buf, sizeof buf, "%llu", (unsigned long long)v); break; }
        case F32: { float v; memcpy(&v, q, 4); snprintf(buf, sizeof buf, "%.9g", (double)v); break; }
        case F16: { uint16_t v; memcpy(&v, q, 2); snprintf(buf, sizeof buf, "%.5g", (double)half_to_float(v)); break; }
        default: { double v; memcpy(&v, q, 8); snprintf(buf, sizeof buf, "%.17g", v); break; }
      }
      out += buf;
    }
    if (a.leaf.size() > 1) out += ")";
  }
  return out + "]";
}

void Program::exec(const std::vector<Node>& ns, Env& env) {
  Ctx& c = *ctx;
  for (const Node& n : ns) {
    struct Reaper {
      Env& env;
      const std::vector<std::string>& dead;
      ~Reaper() { for (auto& d : dead) env.erase(d); }
    } reaper{env, dead_after[n.id]};
    switch (n.kind) {
      case N_USE: {
        auto it = constants.find(n.outs[0]);
        if (it == constants.end()) throw Error(B200_ERR_ARG, "embedded array '" + n.outs[0] + "' was not uploaded");
        env[n.outs[0]] = it->second;
        break;
      }
      case N_ACOND: {
        // Interpreter.hs:217-219: the predicate is a scalar expression (it may read arrays)
        HostEval he{&c, &env, {}};
        const bool yes = he.eval(*n.pred).i[0] != 0;
        std::vector<DevArrayP> r = call(n.body[yes ? 0 : 1], {}, env);
        for (size_t k = 0; k < n.outs.size(); ++k) env[n.outs[k]] = r[k];
        break;
      }
      case N_AWHILE: {
        // Interpreter.hs:221-229: iterate while the condition's result, read at linear index 0, is True
        std::vector<DevArrayP> state;
        for (auto& a : n.args) state.push_back(env.at(a));
        for (;;) {
          std::vector<DevArrayP> cnd = call(n.body[0], state, env);
          HostEval he{&c, &env, {}};
          if (he.read(*cnd[0], 0).i[0] == 0) break;
          state = call(n.body[1], state, env);
        }
        for (size_t k = 0; k < n.outs.size(); ++k) env[n.outs[k]] = state[k];
        break;
      }
      case N_APPLY: {
        std::vector<DevArrayP> args;
        for (auto& a : n.args) args.push_back(env.at(a));
        std::vector<DevArrayP> r = call(n.body[0], args, env);
        for (size_t k = 0; k < n.outs.size(); ++k) env[n.outs[k]] = r[k];
        break;
      }
      case N_ATRACE: {
        // Interpreter.hs:215, atraceOp (:873-880): the message, then ": " and the arrays if there are any, on
        // standard error.  The arrays are rendered by this library (trace_render), not by the `show` of the
        // host program's Message, which cannot cross the boundary.
        std::string line = n.message;
        for (size_t k = 0; k < n.shown.size(); ++k) line += (k ? ", " : ": ") + trace_render(c, *env.at(n.shown[k]));
        fprintf(stderr, "%s\n", line.c_str());
        fflush(stderr);
        for (size_t k = 0; k < n.outs.size(); ++k) env[n.outs[k]] = env.at(n.args[k]);
        break;
      }
      default: exec_kernel_node(n, env);
    }
  }
}

// The kernel of one node for one variant.  Assembling the source text and hashing it (what Ctx::kernel
// keys on) costs tens of microseconds, too much for every launch of a program that runs many small
// kernels, so a node remembers the kernels it has asked for by skeleton, entry point and variant.
static CompiledKernel& node_kernel(Ctx& c, NodeState& st, const char* skeleton, const std::map<std::string, std::string>& variant, const char* entry,
                                   int threads, size_t smem) {
  std::string key = skeleton;
  key += '|';
  key += entry;
  for (auto& kv : variant) {
    key += '|';
    key += kv.first;
    key += '=';
    key += kv.second;
  }
  auto it = st.kernel_memo.find(key);
  if (it != st.kernel_memo.end()) {
    c.mem_hits++;
    return *it->second;
  }
  CompiledKernel& k = c.kernel(assemble_source(st.glue, skeleton, variant), entry, threads, smem);
  st.kernel_memo[key] = &k;
  return k;
}

void Program::exec_kernel_node(const Node& n, Env& env_ref) {
  Ctx& c = *ctx;
  Env& env = env_ref;
  {
    HostEval he{&c, &env, {}};
    if (n.kind == N_RESHAPE) {
      // reshapeOp (Interpreter.hs:293-303): same data, new shape; sizes must agree
      std::vector<int64_t> sh = he.eval(*n.extent).i;
      DevArrayP src = env.at(n.arr);
      if (size_of(sh) != src->size()) throw Error(B200_ERR_BOUNDS, "shape mismatch");
      auto a = std::make_shared<DevArray>(*src);
      a->shape = sh;
      env[n.outs[0]] = a;
      return;
    }
    NodeState& st = nodes[n.id];
    Launcher L{&c, &env, &st.glue, {}, {}};
    L.named["err"] = (int64_t)(uintptr_t)(c.d_words + 0);
    L.named["spin_limit"] = c.spin_limit;
    switch (n.kind) {
      case N_GENERATE: {
        std::vector<int64_t> sh = he.eval(*n.extent).i;
        const int64_t total = size_of(sh);
        DevArrayP out = c.new_array(n.elt, sh);
        L.outs = {out};
        env[n.outs[0]] = out;
        if (total == 0) break;
        L.bind_delayed("D0", sh, 0);
        const int64_t inner = sh.empty() ? 1 : sh.back();
        L.named["n"] = total;
        L.named["vec"] = (L.fast("D0") && (sh.size() <= 1 || inner % 4 == 0)) ? 1 : 0;
        CompiledKernel& k = node_kernel(c, st, "elementwise", {}, "acc_generate", 256, 0);
        int64_t work = L.named["vec"] ? (total + 3) / 4 : total;
        int64_t grid = std::min<int64_t>((work + 255) / 256, (int64_t)c.sm_count * k.max_blocks_per_sm * 4);
        L.launch(k, std::max<int64_t>(grid, 1), 256, 0);
        break;
      }
      case N_FOLD: {
        std::vector<int64_t> ext = he.eval(*n.d[0].extent).i;
        const int64_t m = std::max<int64_t>(ext.back(), 0);
        const int64_t rows = prod_outer(ext);
        std::vector<int64_t> osh(ext.begin(), ext.end() - 1);
        if (!n.seed && m == 0) throw Error(B200_ERR_BOUNDS, "empty array");  // Interpreter.hs:386
        DevArrayP out = c.new_array(n.elt, osh);
        L.outs = {out};
        env[n.outs[0]] = out;
        if (rows == 0) break;
        L.bind_delayed("D0", ext, 0);
        L.named["n"] = m;
        L.named["rows"] = rows;
        L.named["vec"] = (L.fast("D0") && (rows == 1 || m % 4 == 0)) ? 1 : 0;
        if (rows <= 8 && (rows == 1 || m >= (1 << 16))) {
          std::map<std::string, std::string> var = {{"FOLD_G", "32"}, {"ACC_STREAM_LOADS", "1"}};
          CompiledKernel& k = node_kernel(c, st, "fold", var, "acc_fold_all", 256, 0);
          const int64_t ntiles = (m + 1023) / 1024;
          int64_t grid = std::max<int64_t>(1, std::min<int64_t>(ntiles, (int64_t)c.sm_count * k.max_blocks_per_sm));
          const size_t sb = struct_bytes(n.elt);
          // per-CTA partial results, then the per-CTA flags, in one buffer
          const size_t part_bytes = ((size_t)grid * sb + 16 + 255) / 256 * 256;
          auto scratch = c.alloc(part_bytes + (size_t)grid * 4);
          L.named["scratch"] = (int64_t)(uintptr_t)scratch->ptr;
          L.named["flags"] = (int64_t)(uintptr_t)((char*)scratch->ptr + part_bytes);
          L.named["counter"] = (int64_t)(uintptr_t)(c.d_words + 1);
          for (int64_t r = 0; r < rows; ++r) {
            L.named["row"] = r;
            L.launch(k, grid, 256, 0);
          }
        } else {
          const int g = pow2_at_least((m + 7) / 8);
          std::map<std::string, std::string> var = {{"FOLD_G", std::to_string(g)}, {"ACC_STREAM_LOADS", "1"}};
          CompiledKernel& k = node_kernel(c, st, "fold", var, "acc_fold_rows", 256, 0);
          const int64_t warps = (rows + (32 / g) - 1) / (32 / g);
          int64_t grid = std::min<int64_t>((warps + 7) / 8, (int64_t)c.sm_count * k.max_blocks_per_sm);
          L.launch(k, std::max<int64_t>(grid, 1), 256, 0);
        }
        break;
      }
      case N_FOLDSEG: {
        std::vector<int64_t> ext = he.eval(*n.d[0].extent).i;
        std::vector<int64_t> sext = he.eval(*n.d[1].extent).i;
        if (sext[0] <= 0) throw Error(B200_ERR_BOUNDS, "empty segment descriptor");  // Interpreter.hs:398
        const int64_t segs = sext[0] - 1;
        const int64_t m = std::max<int64_t>(ext.back(), 0);
        const int64_t rows = prod_outer(ext);
        std::vector<int64_t> osh(ext.begin(), ext.end() - 1);
        osh.push_back(segs);
        DevArrayP out = c.new_array(n.elt, osh);
        L.outs = {out};
        env[n.outs[0]] = out;
        if (rows * segs == 0) break;
        L.bind_delayed("D0", ext, 0);
        L.bind_delayed("D1", sext, 1);
        L.named["segs"] = segs;
        L.named["rows"] = rows;
        L.named["vec"] = (L.fast("D0") && (rows == 1 || m % 4 == 0)) ? 1 : 0;
        const int g = pow2_at_least((m / std::max<int64_t>(segs, 1) + 7) / 8);
        std::map<std::string, std::string> var = {{"FOLDSEG_G", std::to_string(g)}, {"ACC_STREAM_LOADS", "1"}};
        CompiledKernel& k = node_kernel(c, st, "foldseg", var, "acc_foldseg", 256, 0);
        const int64_t warps = (rows * segs + (32 / g) - 1) / (32 / g);
        int64_t grid = std::min<int64_t>((warps + 7) / 8, (int64_t)c.sm_count * k.max_blocks_per_sm);
        L.launch(k, std::max<int64_t>(grid, 1), 256, 0);
        break;
      }
      case N_SCAN: case N_SCAN2: {
        std::vector<int64_t> ext = he.eval(*n.d[0].extent).i;
        const int64_t m = std::max<int64_t>(ext.back(), 0);
        const int64_t rows = prod_outer(ext);
        const int mode = n.kind == N_SCAN2 ? 2 : (n.seed ? 1 : 0);
        std::vector<int64_t> osh(ext.begin(), ext.end());
        osh.back() = mode == 1 ? m + 1 : m;
        DevArrayP out = c.new_array(n.elt, osh);
        L.outs = {out};
        env[n.outs[0]] = out;
        if (mode == 2) {
          DevArrayP sums = c.new_array(n.elt, std::vector<int64_t>(ext.begin(), ext.end() - 1));
          L.outs.push_back(sums);
          env[n.outs[1]] = sums;
        }
        if (rows == 0 || (mode == 0 && m == 0)) break;
        L.bind_delayed("D0", ext, 0);
        const bool small = scan_is_small(rows * m);
        const int64_t tile = 8 * (int64_t)(small ? std::min(scan_rounds(n.elt), SCAN_SMALL_ROUNDS) : scan_rounds(n.elt)) * 128;
        const int64_t tiles_per_row = std::max<int64_t>(1, (m + tile - 1) / tile);
        const int64_t total_tiles = rows * tiles_per_row;
        const bool right = n.right;
        bool in_vec = L.fast("D0") && (right ? (m % 4 == 0) : (rows == 1 || m % 4 == 0));
        bool out_vec;
        if (mode == 1) out_vec = right ? ((m + 1) % 4 == 0) : (rows == 1 || (m + 1) % 4 == 0);
        else out_vec = right ? (m % 4 == 0) : (rows == 1 || m % 4 == 0);
        L.named["n"] = m;
        L.named["rows"] = rows;
        L.named["in_vec"] = in_vec;
        L.named["out_vec"] = out_vec;
        L.named["counter"] = (int64_t)(uintptr_t)(c.d_words + 2);
        // shared-memory ring kernel: one scalar leaf in, one scalar leaf of the same size out
        {
          const auto& df = st.glue.defines;
          const bool packed = df.count("SCAN_PACKED") && df.at("SCAN_PACKED") == "1";
          const bool one_stream = df.count("D0_STREAM_NLEAVES") && df.at("D0_STREAM_NLEAVES") == "1" && packed &&
                                  df.at("D0_STREAM_BYTES") == df.at("SCAN_T_BYTES");
          const int bytes = packed ? atoi(df.at("SCAN_T_BYTES").c_str()) : 0;
          const bool want = bytes <= 8 && !small;
          if (one_stream && want && L.fast("D0") && in_vec && out_vec && scan_ring_aligned(bytes, m, rows, right)) {
            const RingShape rs = scan_ring_shape(bytes);
            const int rounds = rs.rounds, slots = rs.slots, look = rs.look;
            const int64_t rtile = 8 * (int64_t)rounds * 128;
            const int64_t r_tiles_per_row = std::max<int64_t>(1, (m + rtile - 1) / rtile);
            const int64_t r_total = rows * r_tiles_per_row;
            // (8-byte elements: one more kilobyte per finisher warp, through which results are transposed for the stores)
            const size_t smem = (size_t)slots * rtile * bytes + (bytes == 8 ? 8 * 1024 : 0);
            // look-back descriptors describe batches of rs.batch consecutive tiles of a row
            const int64_t batches_per_row = (r_tiles_per_row + rs.batch - 1) / rs.batch;
            const int64_t total_batches = rows * batches_per_row;
            std::map<std::string, std::string> var = scan_ring_variant(rs, total_batches);
            const int dstride = scan_desc_stride(total_batches);
            const size_t r_status = ((size_t)total_batches * 16 * dstride + 255) / 256 * 256;
            const int64_t groups_per_row = (batches_per_row + 32 * look - 1) / (32 * look);
            const size_t g_status = ((size_t)(rows * groups_per_row) * 16 * dstride + 255) / 256 * 256;
            char* rbase = (char*)c.scan_descriptors(r_status + g_status, "ring/" + std::to_string(bytes) + "/" + std::to_string(dstride) + "/" + std::to_string(r_status));
            L.named["gstatus"] = (int64_t)(uintptr_t)(rbase + r_status);
            L.named["groups_per_row"] = groups_per_row;
            L.named["tiles_per_row"] = r_tiles_per_row;
            L.named["total_tiles"] = r_total;
            L.named["batches_per_row"] = batches_per_row;
            L.named["total_batches"] = total_batches;
            L.named["status"] = (int64_t)(uintptr_t)rbase;
            L.named["epoch"] = c.scan_epoch;
            const int threads = 256 + 32 * rs.redw + 32 * rs.lbw;     // 8 finisher warps, the reducer warps, the look-back warps
            CompiledKernel& k = node_kernel(c, st, "scan", var, "acc_scan_ring", threads, smem);
            const int64_t grid = std::min<int64_t>(total_batches, (int64_t)c.sm_count * k.max_blocks_per_sm);
            L.launch(k, grid, threads, smem);
            break;
          }
        }
        {
          const auto& df = st.glue.defines;
          const bool packed = df.count("SCAN_PACKED") && df.at("SCAN_PACKED") == "1";
          const int dstride = scan_desc_stride(total_tiles);
          const size_t sb = struct_bytes(n.elt);
          const size_t status_bytes = ((size_t)total_tiles * 16 * dstride + 255) / 256 * 256;  // packed descriptors take up to 16 bytes
          const size_t val_bytes = ((size_t)total_tiles * sb + 255) / 256 * 256;
          const std::string layout = (packed ? "packed/" + df.at("SCAN_T_BYTES") : "tuple/" + std::to_string(sb)) + "/" + std::to_string(dstride) + "/" +
                                     std::to_string(status_bytes) + "/" + std::to_string(val_bytes);
          char* base = (char*)c.scan_descriptors(status_bytes + 2 * val_bytes, layout);
          L.named["tiles_per_row"] = tiles_per_row;
          L.named["status"] = (int64_t)(uintptr_t)base;
          L.named["agg"] = (int64_t)(uintptr_t)(base + status_bytes);
          L.named["incl"] = (int64_t)(uintptr_t)(base + status_bytes + val_bytes);
          L.named["epoch"] = c.scan_epoch;
        }
        auto svar = scan_variant(n.elt, small);
        scan_poll_variant(svar, total_tiles);
        CompiledKernel& k = node_kernel(c, st, "scan", svar, "acc_scan", 256, 0);
        L.launch(k, total_tiles, 256, 0);
        break;
      }
      case N_PERMUTE: {
        DevArrayP def = env.at(n.arr);
        std::vector<int64_t> ext = he.eval(*n.d[0].extent).i;
        const int64_t total = size_of(ext);
        // "If the array of default values is only used once, it will be updated in-place" (Language.hs:764-765):
        // the defaults are a temporary of this run that nobody else holds (no caller's handle, no embedded
        // constant, no reshaped view, no second name), this node is its last use, and the node's scalar code
        // does not read it.  Otherwise the permutation works on a copy.
        bool in_place = def.use_count() == 2;      // the environment's reference and this one
        {
          const std::vector<std::string>& dead = dead_after[n.id];
          in_place = in_place && std::find(dead.begin(), dead.end(), n.arr) != dead.end();
          for (auto& b : def->leaf) in_place = in_place && b->owned && b.use_count() == 1;
          for (auto& sl : st.glue.slots)
            if ((sl.kind == Slot::ARR_LEAF || sl.kind == Slot::ARR_DIM) && sl.name == n.arr) in_place = false;
          for (auto& pend : def->pending) in_place = in_place && pend == nullptr;
        }
        DevArrayP out = in_place ? def : c.new_array(n.elt, def->shape);
        if (!in_place)
          for (size_t l = 0; l < out->leaf.size(); ++l)
            if (out->leaf[l]->bytes)
              c.check(cudaMemcpyAsync(out->leaf[l]->ptr, def->leaf[l]->ptr, out->leaf[l]->bytes, cudaMemcpyDeviceToDevice, c.stream), "cudaMemcpyAsync");
        if (in_place) c.inplace_permutes++;
        L.outs = {out};
        env[n.outs[0]] = out;
        if (total == 0) break;
        L.bind_delayed("P", ext, 0);
        const int64_t inner = ext.empty() ? 1 : ext.back();
        const int64_t out_n = out->size();
        L.named["n"] = total;
        L.named["vec"] = (L.fast("P") && (ext.size() <= 1 || inner % 4 == 0)) ? 1 : 0;
        L.named["out_n"] = out_n;
        for (size_t d = 0; d < def->shape.size(); ++d) L.named["out_d" + std::to_string(d)] = def->shape[d];
        const std::string& mode = st.glue.defines.at("PERMUTE_MODE");
        std::shared_ptr<Buffer> locks;
        if (mode == "PERMUTE_LOCK") {
          locks = c.alloc((size_t)std::max<int64_t>(out_n, 1) * 4);
          c.check(cudaMemsetAsync(locks->ptr, 0, locks->bytes, c.stream), "cudaMemsetAsync");
          L.named["locks"] = (int64_t)(uintptr_t)locks->ptr;
        }
        const bool atomic = mode.find("ATOMIC") != std::string::npos;
        const int bytes = atomic ? atoi(st.glue.defines.at("PERMUTE_BYTES").c_str()) : 0;
        const int64_t cap = 200 * 1024;
        const bool int_add32 = mode == "PERMUTE_ATOMIC_ADD" && bytes == 4 && st.glue.defines.at("PERMUTE_FLOAT") == "0";
        const bool fields16 = int_add32 && out_n > cap / 4 && (out_n + 1) / 2 <= 56 * 1024 && total >= 8 * out_n;
        L.named["choice"] = 0;
        if (fields16) {
          // (+) on 32-bit integers, target too large for a CTA-private 32-bit copy but not for 16-bit
          // fields.  A sample of the input decides on the device between that kernel and the faster
          // partial 32-bit copy below (see acc_permute_sample); both are launched.
          int* choice = c.d_words + 4;
          L.named["choice"] = (int64_t)(uintptr_t)choice;
          L.named["priv"] = std::min<int64_t>(out_n, cap / bytes);
          L.named["priv16"] = 0;
          CompiledKernel& ks = node_kernel(c, st, "permute", {{"PERMUTE_SAMPLE", "1"}}, "acc_permute_sample", 1024, 0);
          L.launch(ks, (std::min<int64_t>(total, 65536) + 1023) / 1024, 1024, 0);
          const int64_t words16 = (out_n + 1) / 2;
          const size_t smem = (size_t)words16 * 4;
          std::map<std::string, std::string> var = {{"PERMUTE_SMEM16", "1"}, {"PERMUTE_THREADS", "1024"}, {"PERMUTE_CHOICE_ID", "1"}};
          CompiledKernel& k = node_kernel(c, st, "permute", var, "acc_permute", 1024, smem);
          if (smem > 48 * 1024) c.check(c.drv.FuncSetAttribute(k.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)smem), "cuFuncSetAttribute");
          L.named["priv16"] = words16;
          const int64_t work = (total + 3) / 4;
          int64_t grid = std::min<int64_t>((work + 1023) / 1024, (int64_t)c.sm_count);
          L.launch(k, std::max<int64_t>(grid, 1), 1024, smem);
          // (falls through to the partial 32-bit copy, which runs only if the sample chose it)
        }
        if (atomic && out_n > 0 && total >= 8 * out_n && total >= (1 << 16)) {
          // CTA-private copy of the first `priv` target elements in shared memory
          const int64_t priv = std::min<int64_t>(out_n, cap / bytes);
          const size_t smem = (size_t)priv * bytes;
          std::map<std::string, std::string> var = {{"PERMUTE_SMEM", "1"}, {"PERMUTE_THREADS", "1024"}};
          CompiledKernel& k = node_kernel(c, st, "permute", var, "acc_permute", 1024, smem);
          if (smem > 48 * 1024) c.check(c.drv.FuncSetAttribute(k.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)smem), "cuFuncSetAttribute");
          int nb = 1;
          c.check(c.drv.OccupancyMaxActiveBlocksPerMultiprocessor(&nb, k.fn, 1024, smem), "occupancy");
          L.named["priv"] = priv;
          const int64_t work = (total + 3) / 4;
          int64_t grid = std::min<int64_t>((work + 1023) / 1024, (int64_t)c.sm_count * std::max(nb, 1));
          L.launch(k, std::max<int64_t>(grid, 1), 1024, smem);
        } else {
          L.named["priv"] = 0;
          CompiledKernel& k = node_kernel(c, st, "permute", {}, "acc_permute", 512, 0);
          const int64_t work = L.named["vec"] ? (total + 3) / 4 : total;
          int64_t grid = std::min<int64_t>((work + 511) / 512, (int64_t)c.sm_count * k.max_blocks_per_sm * 2);
          L.launch(k, std::max<int64_t>(grid, 1), 512, 0);
        }
        break;
      }
      case N_STENCIL: case N_STENCIL2: {
        const int rank = n.d[0].rank;
        std::vector<std::vector<int64_t>> ext;
        for (auto& d : n.d) ext.push_back(he.eval(*d.extent).i);
        std::vector<int64_t> osh = ext[0];
        for (size_t a = 1; a < ext.size(); ++a)
          for (int d = 0; d < rank; ++d) osh[d] = std::min(osh[d], ext[a][d]);  // Shape.hs:81-91
        if (window && (rank != 2 || window->out->shape != osh || window->out->elt != n.elt || window->lo < 0 || window->hi > osh[0] || window->lo > window->hi ||
                       window->hi2 > osh[0]))
          throw Error(B200_ERR_ARG, "row window: the output array does not have the shape and type of the stencil's result, or the rows lie outside it");
        DevArrayP out = window ? window->out : c.new_array(n.elt, osh);
        L.outs = {out};
        env[n.outs[0]] = out;
        if (size_of(osh) == 0 || (window && window->lo == window->hi)) break;
        for (size_t a = 0; a < ext.size(); ++a) L.bind_delayed("D" + std::to_string(a), ext[a], a);
        int64_t o[3] = {1, 1, 1};
        for (int d = 0; d < rank; ++d) o[d + 3 - rank] = osh[d];
        StencilTile t = stencil_tile(rank);
        const int64_t tiles0 = (o[0] + t.t0 - 1) / t.t0, tiles1 = (o[1] + t.t1 - 1) / t.t1, tiles2 = (o[2] + t.t2 - 1) / t.t2;
        L.named["o0"] = o[0];
        L.named["o1"] = o[1];
        L.named["o2"] = o[2];
        L.named["tiles1"] = tiles1;
        L.named["tiles2"] = tiles2;
        L.named["vec"] = (o[2] % 4 == 0 && out->aligned16()) ? 1 : 0;
        const int64_t row0 = window ? window->lo : 0, row1 = window ? window->hi : o[1];
        L.named["row0"] = row0;
        L.named["row1"] = row1;
        if (rank == 2 && o[1] < 2000000000 && o[2] < 2000000000) {
          // register-window kernel: warp tasks of 128 columns x ST2_ROWS (32) rows
          const Stencil2dShape shp = stencil2d_shape();
          const int warps = shp.warps, rows = shp.rows;
          const int64_t strips = (o[2] + 119) / 120, rowblocks = (row1 - row0 + rows - 1) / rows;  // 120 output columns per warp
          L.named["tiles1"] = rowblocks;
          L.named["tiles2"] = strips;
          const std::map<std::string, std::string> var = stencil2d_variant();
          // Rows staged through shared memory (acc_stencil2d_bulk) for the middle of the arrays, when the
          // register windows of acc_stencil2d are wide (8 bytes or more per point over all inputs: they
          // then leave too few registers for rows requested ahead); acc_stencil2d computes the frame.
          const auto& df = st.glue.defines;
          const Stencil2dBulkShape bs = stencil2d_bulk_shape();
          int64_t point_bytes = 0, min_e1 = o[2];
          bool staged = !window && df.count("ST2_BULK_OK") && df.at("ST2_BULK_OK") == "1" && L.named["vec"] == 1;
          for (size_t a = 0; a < ext.size() && staged; ++a) {
            const std::string D = "D" + std::to_string(a);
            staged = L.fast(D) && ext[a][1] % 4 == 0 && df.count(D + "_STREAM_BYTES");
            if (staged) point_bytes += atoi(df.at(D + "_STREAM_BYTES").c_str());
            min_e1 = std::min(min_e1, ext[a][1]);
          }
          const int64_t ry = atoi(df.at("ST_RYMAX").c_str());
          const int64_t mid_strips = staged ? std::min<int64_t>(std::max<int64_t>((min_e1 - 124) / 120, 0), strips - 1) : 0;
          const int64_t mid_r0 = ry, mid_r1 = o[1] - ry;
          if (staged && point_bytes >= bs.min_point_bytes && mid_strips > 0 && mid_r1 - mid_r0 >= bs.rows) {
            const std::map<std::string, std::string> bvar = stencil2d_bulk_variant(bs);
            const size_t smem = (size_t)bs.warps * bs.slots * 128 * point_bytes;
            CompiledKernel& kb = node_kernel(c, st, "stencil2d", bvar, "acc_stencil2d_bulk", bs.warps * 32, smem);
            // The frame first, on the auxiliary stream: strip 0 and the strips after the middle ones over all rows,
            // the rows above and below the middle of the middle strips.  Its few warps march down their tasks at
            // the pace of dependent loads, so it runs beside the staged kernel instead of after it, in tasks of
            // 8 rows.
            const int frows = 8;
            const int64_t ra = (o[1] + frows - 1) / frows, rc = (mid_r0 + frows - 1) / frows, rd = (o[1] - mid_r1 + frows - 1) / frows;
            const int64_t frame_tasks = (strips - mid_strips) * ra + mid_strips * (rc + rd);
            L.named["row0"] = 0;
            L.named["row1"] = o[1];
            L.named["tiles1"] = ra;
            L.named["tiles2"] = strips;
            L.named["fr_strips"] = mid_strips;
            L.named["fr_r0"] = mid_r0;
            L.named["fr_r1"] = mid_r1;
            std::map<std::string, std::string> fvar = stencil2d_frame_variant();
            CompiledKernel& kf = node_kernel(c, st, "stencil2d", fvar, "acc_stencil2d", warps * 32, 0);
            c.check(cudaEventRecord(c.aux_fork, c.stream), "cudaEventRecord");
            c.check(cudaStreamWaitEvent(c.aux_stream, c.aux_fork, 0), "cudaStreamWaitEvent");
            L.launch(kf, (frame_tasks + warps - 1) / warps, warps * 32, 0, c.aux_stream);
            c.check(cudaEventRecord(c.aux_join, c.aux_stream), "cudaEventRecord");
            const int64_t mid_blocks = (mid_r1 - mid_r0 + bs.rows - 1) / bs.rows;
            L.named["row0"] = mid_r0;
            L.named["row1"] = mid_r1;
            L.named["strip0"] = 1;
            L.named["tiles1"] = mid_blocks;
            L.named["tiles2"] = mid_strips;
            L.launch(kb, (mid_strips * mid_blocks + bs.warps - 1) / bs.warps, bs.warps * 32, smem);
            c.check(cudaStreamWaitEvent(c.stream, c.aux_join, 0), "cudaStreamWaitEvent");
            break;
          }
          CompiledKernel& k2 = node_kernel(c, st, "stencil2d", var, "acc_stencil2d", warps * 32, 0);
          if (window && window->hi2 > window->lo2) {
            // two row ranges in one launch (the rows at either edge of a slab)
            std::map<std::string, std::string> tvar = var;
            tvar["ST2_TWOWIN"] = "1";
            tvar["ACC_OPT_PARAMS"] = "1";
            const int64_t both = rowblocks + (window->hi2 - window->lo2 + rows - 1) / rows;
            L.named["tiles1"] = both;
            L.named["row2"] = window->lo2;
            L.named["row3"] = window->hi2;
            CompiledKernel& kt = node_kernel(c, st, "stencil2d", tvar, "acc_stencil2d", warps * 32, 0);
            L.launch(kt, (strips * both + warps - 1) / warps, warps * 32, 0);
            break;
          }
          const int64_t ctas = (strips * rowblocks + warps - 1) / warps;
          L.launch(k2, ctas, warps * 32, 0);  // one warp per task; the hardware scheduler balances the tail
          break;
        }
        CompiledKernel& k = node_kernel(c, st, "stencil", stencil_variant(rank), "acc_stencil", t.threads, 0);
        L.launch(k, tiles0 * tiles1 * tiles2, t.threads, 0);
        break;
      }
      default: break;
    }
  }
}

}  // namespace accb200
