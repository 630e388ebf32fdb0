// tcgen05 / TMEM attention kernels (placeholder until the tensor-core path lands).
#include "common.cuh"

namespace wm {

bool tc_fwd_supported(const wm_attn_args&) { return false; }
int tc_attn_fwd(const wm_attn_args&, cudaStream_t) { return fail(WM_EUNSUPPORTED, "tcgen05 forward is not built"); }
bool tc_bwd_supported(const wm_attn_args&) { return false; }
int tc_attn_bwd(const wm_attn_args&, cudaStream_t) { return fail(WM_EUNSUPPORTED, "tcgen05 backward is not built"); }
size_t tc_attn_bwd_workspace(const wm_attn_args&) { return 0; }

}  // namespace wm
