// NVRTC compilation of generated kernel sources for sm_100a, with a
// content-hashed on-disk cache of the resulting cubins.  The reference keys its
// kernel cache on a SHA3 digest of the AST (Analysis/Hash.hs:107); here the
// generated CUDA source itself (which is a function of the AST and of nothing
// else) is hashed together with the compiler options and the NVRTC version.
#include <nvrtc.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

#include "runtime.hpp"

namespace accb200 {

namespace {

// 128-bit content hash: two independent 64-bit FNV-1a streams.
void fnv2(const std::string& s, uint64_t& a, uint64_t& b) {
  a = 0xcbf29ce484222325ull;
  b = 0x84222325cbf29ce4ull;
  for (unsigned char c : s) {
    a = (a ^ c) * 0x100000001b3ull;
    b = (b ^ (c + 0x9e)) * 0x1000000000001b3ull + 0x632be59bd9b4e019ull;
  }
}

const char* const kOptions[] = {"--gpu-architecture=sm_100a", "--std=c++17", "--fmad=false", "--diag-suppress=177,550"};
const int kNumOptions = 4;

std::string cache_dir() {
  const char* e = getenv("ACCELERATE_B200_CACHE_DIR");
  if (e && *e) return e;
  const char* h = getenv("HOME");
  return std::string(h && *h ? h : "/tmp") + "/.cache/accelerate-b200";
}

void mkdirs(const std::string& path) {
  std::string cur;
  for (size_t i = 0; i < path.size(); ++i) {
    cur += path[i];
    if (path[i] == '/' || i + 1 == path.size()) mkdir(cur.c_str(), 0755);
  }
}

// A cached file is trusted only if it is a complete ELF image: magic, 64-bit class, and a section
// header table that lies inside the file (a file cut short by a full disk or a killed writer fails
// this; so does a file that is not a cubin at all).
bool plausible_cubin(const std::string& b) {
  if (b.size() < 64 || memcmp(b.data(), "\x7f" "ELF", 4) != 0 || b[4] != 2) return false;
  uint64_t shoff;
  uint16_t shentsize, shnum;
  memcpy(&shoff, b.data() + 0x28, 8);
  memcpy(&shentsize, b.data() + 0x3A, 2);
  memcpy(&shnum, b.data() + 0x3C, 2);
  return shoff >= 64 && shoff + (uint64_t)shentsize * shnum <= b.size();
}

std::atomic<unsigned long long> g_tmp_counter{0};

}  // namespace

std::string content_hash(const std::string& s) {
  uint64_t a, b;
  fnv2(s, a, b);
  char buf[40];
  snprintf(buf, sizeof buf, "%016llx%016llx", (unsigned long long)a, (unsigned long long)b);
  return buf;
}

std::string compile_to_cubin(const std::string& source, const std::string& name, CompileStats* stats, bool force) {
  int major = 0, minor = 0;
  nvrtcVersion(&major, &minor);
  std::string keytext = source;
  for (int i = 0; i < kNumOptions; ++i) keytext += std::string("\n//opt ") + kOptions[i];
  keytext += "\n//nvrtc " + std::to_string(major) + "." + std::to_string(minor);
  const std::string key = content_hash(keytext);
  const bool use_disk = !(getenv("ACCELERATE_B200_NO_DISK_CACHE"));
  const std::string dir = cache_dir();
  const std::string path = dir + "/" + key + ".cubin";
  if (use_disk && !force && !getenv("ACCELERATE_B200_FORCE_RECOMP")) {
    std::ifstream f(path, std::ios::binary);
    if (f) {
      std::stringstream ss;
      ss << f.rdbuf();
      std::string cubin = ss.str();
      if (plausible_cubin(cubin)) {
        if (stats) stats->disk_hits++;
        return cubin;
      }
      // damaged cache file: fall through, compile, and replace it
    }
  }
  nvrtcProgram prog;
  nvrtcResult r = nvrtcCreateProgram(&prog, source.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr);
  if (r != NVRTC_SUCCESS) throw Error(B200_ERR_COMPILE, std::string("nvrtcCreateProgram: ") + nvrtcGetErrorString(r));
  r = nvrtcCompileProgram(prog, kNumOptions, kOptions);
  if (r != NVRTC_SUCCESS) {
    size_t n = 0;
    nvrtcGetProgramLogSize(prog, &n);
    std::string log(n, '\0');
    if (n) nvrtcGetProgramLog(prog, &log[0]);
    nvrtcDestroyProgram(&prog);
    if (getenv("ACCELERATE_B200_DUMP_CC")) fprintf(stderr, "%s\n", source.c_str());
    throw Error(B200_ERR_COMPILE, "NVRTC failed for kernel '" + name + "':\n" + log);
  }
  size_t n = 0;
  nvrtcGetCUBINSize(prog, &n);
  std::string cubin(n, '\0');
  nvrtcGetCUBIN(prog, &cubin[0]);
  nvrtcDestroyProgram(&prog);
  if (stats) stats->compiled++;
  if (use_disk) {
    mkdirs(dir);
    // unique per writer: two contexts or threads of one process may compile the same kernel at once
    const std::string tmp = path + ".tmp" + std::to_string((long long)getpid()) + "." + std::to_string(g_tmp_counter.fetch_add(1));
    std::ofstream f(tmp, std::ios::binary);
    if (f) {
      f.write(cubin.data(), (std::streamsize)cubin.size());
      f.close();
      rename(tmp.c_str(), path.c_str());  // atomic publish; concurrent writers produce identical bytes
    }
  }
  return cubin;
}

}  // namespace accb200
