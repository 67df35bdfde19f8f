#include "common.h"
#include "gemm.h"
namespace annc { namespace gemm {
bool tc_supported(const annc_gemm_desc&, int) { return false; }
int run_tc(const annc_gemm_desc&, int, cudaStream_t) { return fail(ANNC_ERR_UNSUPPORTED, "tc gemm not built"); }
}}
