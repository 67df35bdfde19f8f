// TEST INFRASTRUCTURE ONLY.  extern "C" door into the reference's own
// ANNC_FLAGS parser, compiled from the reference sources where they lie
// (annc/service/cpu/annc_flags.cc) by oracle/Makefile into oracle/_ref/.
// Each call builds a fresh annc::ANNCFlags, whose constructor re-reads the
// ANNC_FLAGS environment variable (annc_flags.cc:36-51), so a test can try
// many flag strings in one process.
#include <cstdlib>
#include <string>

#include "annc_flags.h"

extern "C" int annc_ref_flag_enabled(const char* flags_env, const char* name) {
  if (flags_env) {
    setenv("ANNC_FLAGS", flags_env, 1);
  } else {
    unsetenv("ANNC_FLAGS");
  }
  annc::ANNCFlags f;
  return f.is_enabled(name) ? 1 : 0;
}
