// Tensor-core (tcgen05 + TMEM + TMA) kernels of the AdaSplash-2 attention path.
#pragma once
#include "attn_simt.cuh"

namespace ads {
namespace sm100 {

// fp16 / bf16 inputs with a head dim the kernels were built for.
bool supported(const ads_attn_shape* s);
// Recommended workspace (status word + the solver's overflow area) and the minimum every entry
// point accepts (the status word alone).
size_t workspace_bytes(const ads_attn_shape* s);
size_t min_workspace_bytes();
int solve(const simt::Params& p, int dtype, void* ws, size_t ws_bytes, cudaStream_t st);
int fwd(const simt::Params& p, int dtype, void* ws, cudaStream_t st);
int bwd(const simt::Params& p, int dtype, void* ws, cudaStream_t st);
int debug_waits(long long max_wait_cycles, int withhold_loads);

}  // namespace sm100
}  // namespace ads
