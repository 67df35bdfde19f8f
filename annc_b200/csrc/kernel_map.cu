// KERNEL_MAP_FILE: the size -> runtime-symbol table of the kernel selector, for a dispatcher
// that runs without XLA.  Grammar, acceptance rules and lookup order follow
// annc/service/cpu/xla/kernel_selector_ops_rewriter.cc:108-263 and the IntervalMap at :50-104:
//   [kernel](e1,e2,...) -> symbol      kernel in {gemv, gemm, batch3d, batch4d, argmax}
//   element = N | * | A:B | A:*        ranks 2, 3, 4, 5, 3; `(*)` alone means any size
// All white space is dropped first.  A line that does not parse or has the wrong rank is
// skipped; an unknown kernel name ends the load (entries read so far stay).  Lookup walks the
// entries in key order (kernel type, then the ranges compared lexicographically) and returns
// the first whose ranges contain the sizes.  Host-only code.
#include <dlfcn.h>

#include <climits>
#include <cstdlib>
#include <fstream>
#include <map>
#include <mutex>
#include <regex>
#include <sstream>
#include <string>
#include <vector>

#include "common.h"

namespace annc {
namespace {

enum KernelType { kGEMV, kGEMM, kBATCH3D, kBATCH4D, kARGMAX };
using Range = std::pair<int, int>;
using RangeSet = std::vector<Range>;
const Range kAny = {0, INT_MAX};

std::mutex g_mu;
std::map<std::pair<KernelType, RangeSet>, std::string> g_map;

bool kernel_type(const std::string& name, KernelType* ty, int* rank) {
  static const struct { const char* n; KernelType t; int r; } k[] = {
      {"gemv", kGEMV, 2}, {"gemm", kGEMM, 3}, {"batch3d", kBATCH3D, 4}, {"batch4d", kBATCH4D, 5},
      {"argmax", kARGMAX, 3}};
  for (const auto& e : k)
    if (name == e.n) {
      *ty = e.t;
      *rank = e.r;
      return true;
    }
  return false;
}

// "*" -> INT_MAX, digits -> value; -1 when the number does not fit an int.
int parse_int(const std::string& s) {
  if (s == "*") return INT_MAX;
  errno = 0;
  char* end = nullptr;
  const long v = strtol(s.c_str(), &end, 10);
  if (errno != 0 || *end != 0 || v < 0 || v > INT_MAX) return -1;
  return (int)v;
}

Range parse_range(const std::string& s) {
  if (s == "*") return kAny;
  const size_t c = s.find(':');
  if (c == std::string::npos) {
    const int v = parse_int(s);
    return {v, v};
  }
  return {parse_int(s.substr(0, c)), parse_int(s.substr(c + 1))};
}

struct Parsed {
  std::string kernel, symbol;
  RangeSet sizes;
  bool valid = false;
};

Parsed parse_line(std::string line) {
  std::string t;
  for (char ch : line)
    if (!isspace((unsigned char)ch)) t.push_back(ch);
  static const std::regex pat(
      R"(^\[(.+)\]\(((?:(?:\d+|\*|\d+:(?:\d+|\*)),)*(?:\d+|\*|\d+:(?:\d+|\*)))\)->(.+))");
  Parsed p;
  std::smatch m;
  if (!std::regex_match(t, m, pat)) return p;
  p.kernel = m[1];
  std::stringstream ss(m[2]);
  std::string tok;
  while (std::getline(ss, tok, ',')) {
    const Range r = parse_range(tok);
    if (r.first == -1 || r.second == -1) return p;
    p.sizes.push_back(r);
  }
  p.symbol = m[3];
  p.valid = true;
  return p;
}

// Returns the number of entries in the map after the load, or -1 - (line number) style
// negatives are not used: problems are reported through `bad_lines`.
int load_stream(std::istream& in, int* bad_lines) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_map.clear();
  std::string line;
  int bad = 0;
  while (std::getline(in, line)) {
    if (!line.empty() && line.back() == '\r') line.pop_back();
    Parsed p = parse_line(line);
    if (!p.valid) {
      ++bad;
      continue;
    }
    KernelType ty;
    int rank;
    if (!kernel_type(p.kernel, &ty, &rank)) {
      ++bad;
      break;  // the reference stops reading at an unknown kernel type
    }
    if (p.sizes.size() == 1 && p.sizes[0] == kAny) p.sizes.assign(rank, kAny);
    if ((int)p.sizes.size() != rank) {
      ++bad;
      continue;
    }
    g_map[{ty, p.sizes}] = p.symbol;
  }
  if (bad_lines) *bad_lines = bad;
  return (int)g_map.size();
}

thread_local std::string t_symbol;

}  // namespace
}  // namespace annc

using namespace annc;

extern "C" {

int annc_kernel_map_load(const char* path, int* bad_lines) {
  if (!path) path = getenv("KERNEL_MAP_FILE");
  if (bad_lines) *bad_lines = 0;
  if (!path) return fail(ANNC_ERR_INVALID_ARGUMENT, "KERNEL_MAP_FILE is not set");
  std::ifstream f(path);
  if (!f.is_open()) return fail(ANNC_ERR_INVALID_ARGUMENT, "cannot open kernel map file %s", path);
  load_stream(f, bad_lines);
  return ANNC_OK;
}

int annc_kernel_map_load_text(const char* text, int* bad_lines) {
  ANNC_REQUIRE(text, ANNC_ERR_INVALID_ARGUMENT, "null text");
  std::istringstream ss(text);
  load_stream(ss, bad_lines);
  return ANNC_OK;
}

int annc_kernel_map_size(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  return (int)g_map.size();
}

void annc_kernel_map_clear(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_map.clear();
}

const char* annc_kernel_map_lookup(const char* kernel, const int* sizes, int num_sizes) {
  if (!kernel || !sizes) return nullptr;
  KernelType ty;
  int rank;
  if (!kernel_type(kernel, &ty, &rank)) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  for (const auto& e : g_map) {
    if (e.first.first != ty) continue;
    const RangeSet& r = e.first.second;
    if ((int)r.size() != num_sizes) continue;
    bool match = true;
    for (int i = 0; i < num_sizes && match; ++i) match = sizes[i] >= r[i].first && sizes[i] <= r[i].second;
    if (match) {
      t_symbol = e.second;
      return t_symbol.c_str();
    }
  }
  return nullptr;
}

void* annc_kernel_map_resolve(const char* kernel, const int* sizes, int num_sizes) {
  const char* sym = annc_kernel_map_lookup(kernel, sizes, num_sizes);
  if (!sym) return nullptr;
  Dl_info info;
  if (!dladdr(reinterpret_cast<void*>(&annc_kernel_map_resolve), &info) || !info.dli_fname) return nullptr;
  void* h = dlopen(info.dli_fname, RTLD_NOW | RTLD_NOLOAD);
  if (!h) return nullptr;
  void* p = dlsym(h, sym);
  dlclose(h);
  return p;
}

}  // extern "C"
