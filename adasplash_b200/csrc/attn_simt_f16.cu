// CUDA-core attention kernels instantiated for __half inputs.
#include "attn_simt_launch.cuh"
namespace ads { namespace simt {
template int launch_solve<__half>(const Params&, cudaStream_t);
template int launch_fwd<__half>(const Params&, cudaStream_t);
template int launch_bwd<__half>(const Params&, cudaStream_t);
}}
