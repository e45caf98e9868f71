// Gather kernels over the row supports exported by the tensor-core solver (support.cuh,
// sparse_rows.cu).
#pragma once
#include "attn_simt.cuh"

namespace ads {
namespace sparse {

// Shapes for which the solver exports supports: what its candidate lists can express.
bool supported(const ads_attn_shape* s);
size_t support_bytes(const ads_attn_shape* s);
// Scratch the backward needs beside the status word when it is given a support buffer.
size_t bwd_scratch_bytes(const ads_attn_shape* s);
// Cursor and per-head counters -> 0 (before the solver runs).
int clear_header(const simt::Params& p, cudaStream_t st);
// Largest squared key-row norm per kv head into the buffer (after clear_header; needed by the
// solver's export above alpha = 1.5).
int key_norms(const simt::Params& p, int dtype, cudaStream_t st);
// out / out2 of every head whose supports were exported; other heads are left alone.
int fwd(const simt::Params& p, int dtype, cudaStream_t st);
// dq, dk, dv of the same heads (dk / dv of a kv head: all its query heads).
int bwd(const simt::Params& p, int dtype, cudaStream_t st);

}  // namespace sparse
}  // namespace ads
