#include "ptx.cuh"
namespace bsa {
bool sm100_fwd_supported(const bsa_fwd_params*, const char** why) { *why = "not built yet"; return false; }
int sm100_fwd(const bsa_fwd_params*, cudaStream_t) { return BSA_E_UNSUPPORTED; }
bool sm100_bwd_supported(const bsa_bwd_params*, const char** why) { *why = "not built yet"; return false; }
int sm100_bwd(const bsa_bwd_params*, cudaStream_t) { return BSA_E_UNSUPPORTED; }
}
