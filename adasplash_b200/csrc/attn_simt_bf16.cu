// CUDA-core attention kernels instantiated for __nv_bfloat16 inputs.
#include "attn_simt_launch.cuh"
namespace ads { namespace simt {
template int launch_solve<__nv_bfloat16>(const Params&, cudaStream_t);
template int launch_fwd<__nv_bfloat16>(const Params&, cudaStream_t);
template int launch_bwd<__nv_bfloat16>(const Params&, cudaStream_t);
}}
