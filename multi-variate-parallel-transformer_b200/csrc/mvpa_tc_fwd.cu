// placeholder until the tcgen05 forward lands
#include "mvpa_common.cuh"
namespace mvpa {
bool tc_fwd_supported(const Args&) { return false; }
size_t tc_fwd_workspace_bytes(const mvpa_problem*) { return 0; }
int tc_fwd(const Args&, void*, size_t, cudaStream_t) { set_error("tcgen05 forward not built"); return MVPA_ERR_UNSUPPORTED; }
}
