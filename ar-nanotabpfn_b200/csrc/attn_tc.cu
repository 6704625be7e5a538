// placeholder until the tcgen05 kernel lands
#include "attn.cuh"
namespace artab {
bool ctx_attn_tc_supported(int, int) { return false; }
int launch_ctx_attn_tc(const CtxAttnArgs&, cudaStream_t) { set_error("tcgen05 context attention not built"); return ARTAB_EINVAL; }
}
