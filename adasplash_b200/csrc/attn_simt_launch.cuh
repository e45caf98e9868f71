// Host launchers of the CUDA-core attention kernels; included once per dtype.
#pragma once
#include "attn_simt.cuh"

namespace ads {
namespace simt {

template <typename K>
inline int set_smem(K kernel, size_t bytes, const char* what) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute(%zu): %s", what, bytes, cudaGetErrorString(e));
    return ADS_ERR_CUDA;
  }
  return ADS_OK;
}

#define ADS_DISPATCH_D(D_, ...)                                             \
  switch (D_) {                                                             \
    case 16: { constexpr int DD = 16; __VA_ARGS__ } break;                         \
    case 32: { constexpr int DD = 32; __VA_ARGS__ } break;                         \
    case 64: { constexpr int DD = 64; __VA_ARGS__ } break;                         \
    case 128: { constexpr int DD = 128; __VA_ARGS__ } break;                       \
    case 256: { constexpr int DD = 256; __VA_ARGS__ } break;                       \
    default: set_error("unsupported head dim %d", D_); return ADS_ERR_UNSUPPORTED; \
  }

template <typename T> int launch_solve(const Params& p, cudaStream_t st) {
  dim3 grid(p.nb, p.Hq, p.B);
  ADS_DISPATCH_D(p.D, {
    size_t sm = 2 * Cfg<DD>::tile_floats * sizeof(float);
    if (int rc = set_smem(solve_kernel<T, DD>, sm, "solve")) return rc;
    solve_kernel<T, DD><<<grid, kThreads, sm, st>>>(p);
  })
  return check_launch("simt::solve");
}

template <typename T> int launch_fwd(const Params& p, cudaStream_t st) {
  dim3 grid(p.nb, p.Hq, p.B);
  ADS_DISPATCH_D(p.D, {
    size_t sm = (2 * Cfg<DD>::tile_floats + 2 * 64 * kPPitch) * sizeof(float);
    if (int rc = set_smem(fwd_kernel<T, DD>, sm, "fwd")) return rc;
    fwd_kernel<T, DD><<<grid, kThreads, sm, st>>>(p);
  })
  return check_launch("simt::fwd");
}

template <typename T> int launch_bwd(const Params& p, cudaStream_t st) {
  const int stages = p.bwd_stages ? p.bwd_stages : 0xF;
  if (stages & ADS_BWD_DELTA) {
    long long rows = (long long)p.B * p.Hq * p.N;
    const long long per_block = (long long)(kDeltaThreads / 32) * delta_rows_per_warp<T>(p.D);
    unsigned grid = (unsigned)((rows + per_block - 1) / per_block);
    bwd_delta_kernel<T><<<grid, kDeltaThreads, 0, st>>>((const T*)p.out2_in, (const T*)p.dout, p.delta,
                                              p.varlen, p.varlen_is_i64, p.B, p.Hq, p.N, p.D);
    if (int rc = check_launch("simt::bwd_delta")) return rc;
  }
  if (stages & ADS_BWD_TRANSPOSE) {
    long long words = (long long)p.B * p.Hq * p.rows_padded * p.n_words;
    unsigned grid = (unsigned)((words + 255) / 256);
    transpose_bitmap_kernel<<<grid, 256, 0, st>>>(p.bmask, p.bmask_t, p.B * p.Hq, p.rows_padded, p.n_words);
    if (int rc = check_launch("simt::transpose_bitmap")) return rc;
  }
  ADS_DISPATCH_D(p.D, {
    size_t sm = (3 * Cfg<DD>::tile_floats + 64 * kPPitch) * sizeof(float);
    if (stages & ADS_BWD_DQ) {
      if (int rc = set_smem(bwd_dq_kernel<T, DD>, sm, "bwd_dq")) return rc;
      bwd_dq_kernel<T, DD><<<dim3(p.nb, p.Hq, p.B), kThreads, sm, st>>>(p);
      if (int rc = check_launch("simt::bwd_dq")) return rc;
    }
    if (stages & ADS_BWD_DKV) {
      if (int rc = set_smem(bwd_dkv_kernel<T, DD>, sm, "bwd_dkv")) return rc;
      bwd_dkv_kernel<T, DD><<<dim3(p.nb, p.Hkv, p.B), kThreads, sm, st>>>(p);
      if (int rc = check_launch("simt::bwd_dkv")) return rc;
    }
  })
  return ADS_OK;
}

}  // namespace simt
}  // namespace ads
