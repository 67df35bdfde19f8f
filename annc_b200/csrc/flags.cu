// ANNC_FLAGS gating and the custom-call registry.
//
// Grammar, defaults and group expansion of annc/service/cpu/annc_flags.cc:10-131:
// tokens "--name", "--name=value" separated by blanks; value true / 1 / empty
// means on, anything else off; "--graph-opt" switches on every GRAPH_OPT flag,
// "--gemm-opt" every GEMM_OPT flag; an unknown name is reported on stderr and
// still stored; parsing stops at a token that does not start with "--".
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>

#include "common.h"

namespace annc {
namespace {

enum Group { GRAPH_OPT, GEMM_OPT, TF_OPT, NONE };
struct FlagDef {
  const char* name;
  bool dflt;
  Group group;
};
const FlagDef kFlags[] = {
    {"matmul", false, GEMM_OPT},         {"layout-matmul", false, GEMM_OPT},
    {"batch-matmul", false, NONE},       {"matmul-add", false, NONE},
    {"matmul-add-relu", false, NONE},    {"sps-emd-2", false, GRAPH_OPT},
    {"pooling", false, NONE},            {"disable-tf-matmul-fusion", false, GEMM_OPT},
    {"annc-pass", true, TF_OPT},
};

using FlagMap = std::map<std::string, bool>;

FlagMap parse(const char* env, bool verbose) {
  FlagMap v;
  for (const auto& f : kFlags) v[f.name] = f.dflt;
  if (!env || !env[0]) return v;
  const std::string s(env);
  size_t pos = 0;
  const size_t n = s.size();
  auto skip = [&](size_t p) {
    while (p < n && s[p] == ' ') ++p;
    return p;
  };
  while (pos < n) {
    pos = skip(pos);
    if (pos >= n) break;
    if (s.compare(pos, 2, "--") != 0) {
      if (verbose)
        fprintf(stderr, "[ANNC ERROR] Invalid flag syntax: expected '--' at position%zu in: %s\n",
                pos, s.c_str());
      break;
    }
    pos += 2;
    const size_t key_start = pos;
    while (pos < n && s[pos] != '=' && s[pos] != ' ') ++pos;
    const bool has_eq = pos < n && s[pos] == '=';
    const std::string key = s.substr(key_start, pos - key_start);
    std::string value = "true";
    if (has_eq) {
      size_t vs = pos + 1, ve = vs;
      while (ve < n && s[ve] != ' ') ++ve;
      value = s.substr(vs, ve - vs);
      pos = ve;
    } else {
      pos = skip(pos);
    }
    if (key == "graph-opt" || key == "gemm-opt") {
      const Group g = key == "graph-opt" ? GRAPH_OPT : GEMM_OPT;
      for (const auto& f : kFlags)
        if (f.group == g) v[f.name] = true;
      continue;
    }
    if (v.find(key) == v.end() && verbose) {
      fprintf(stderr, "[ANNC ERROR] Unknown flag: '%s'. Valid flags are:", key.c_str());
      for (const auto& f : kFlags) fprintf(stderr, "%s\n", f.name);
    }
    const bool on = value == "true" || value == "1" || value.empty();
    v[key] = on;
    if (on && verbose) printf("enabled flag : --%s\n", key.c_str());
  }
  return v;
}

const FlagMap& env_flags() {
  static const FlagMap flags = parse(getenv("ANNC_FLAGS"), true);
  return flags;
}

bool lookup(const FlagMap& m, const char* name) {
  auto it = m.find(name);
  return it != m.end() && it->second;
}

}  // namespace
}  // namespace annc

extern "C" {

int annc_flags_is_enabled(const char* name) {
  return name && annc::lookup(annc::env_flags(), name) ? 1 : 0;
}

int annc_flags_is_enabled_in(const char* flags, const char* name) {
  if (!name) return 0;
  const annc::FlagMap m = annc::parse(flags, false);
  return annc::lookup(m, name) ? 1 : 0;
}

void* annc_lookup_custom_call(const char* target) {
  if (!target || !annc_flags_is_enabled("annc-pass")) return nullptr;
  struct Entry {
    const char* name;
    void* fn;
  };
  static const Entry table[] = {
      {"__matmul", (void*)&__matmul},
      {"__batch_matmul", (void*)&__batch_matmul},
      {"__matmul_add", (void*)&__matmul_add},
      {"__matmul_add_relu", (void*)&__matmul_add_relu},
      {"__reduce_mean", (void*)&__reduce_mean},
      {"__pooling", (void*)&__pooling},
      {"__layout_matmul", (void*)&__layout_matmul},
  };
  for (const auto& e : table)
    if (strcmp(e.name, target) == 0) return e.fn;
  return nullptr;
}

// Benefit order of register_gemm_rewriters (gemm_rewriter.cc:116-134):
// matmul_add_relu 3, matmul_add 2, the rest 1; a longer pattern only applies when
// the dot is followed by the ops it names.
const char* annc_select_gemm_target(int pattern, int rhs_is_parameter) {
  if (!annc_flags_is_enabled("annc-pass")) return nullptr;
  if (pattern == 3) return annc_flags_is_enabled("batch-matmul") ? "__batch_matmul" : nullptr;
  if (pattern >= 2 && annc_flags_is_enabled("matmul-add-relu")) return "__matmul_add_relu";
  if (pattern >= 1 && annc_flags_is_enabled("matmul-add")) return "__matmul_add";
  if (rhs_is_parameter && annc_flags_is_enabled("layout-matmul")) return "__layout_matmul";
  if (annc_flags_is_enabled("matmul")) return "__matmul";
  return nullptr;
}

}  // extern "C"
