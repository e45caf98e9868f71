#include "attn_sm100.cuh"
namespace ads { namespace sm100 {
bool supported(const ads_attn_shape*) { return false; }
size_t workspace_bytes(const ads_attn_shape*) { return 256; }
int solve(const simt::Params&, int, void*, cudaStream_t) { set_error("tcgen05 path not built"); return ADS_ERR_UNSUPPORTED; }
int fwd(const simt::Params&, int, void*, cudaStream_t) { set_error("tcgen05 path not built"); return ADS_ERR_UNSUPPORTED; }
int bwd(const simt::Params&, int, void*, cudaStream_t) { set_error("tcgen05 path not built"); return ADS_ERR_UNSUPPORTED; }
}}
