// CUDA-core attention kernels instantiated for float inputs.
#include "attn_simt_launch.cuh"
namespace ads { namespace simt {
template int launch_solve<float>(const Params&, cudaStream_t);
template int launch_fwd<float>(const Params&, cudaStream_t);
template int launch_bwd<float>(const Params&, cudaStream_t);
}}
