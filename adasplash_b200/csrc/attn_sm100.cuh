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

// The first-generation semantics on the tensor cores (attn_sm100_v1.cu): alpha = 1.5 or 2,
// causal or full attention, taken from Params::alpha / Params::causal.
namespace v1 {
bool supported(const ads_attn_shape* s);
int solve(const simt::Params& p, int dtype, void* ws, size_t ws_bytes, cudaStream_t st);
int fwd(const simt::Params& p, int dtype, void* ws, cudaStream_t st);
int bwd(const simt::Params& p, int dtype, void* ws, cudaStream_t st);
int set_wait_constants_v1(long long max_wait_cycles, int withhold_loads);
}  // namespace v1

}  // namespace sm100
}  // namespace ads
