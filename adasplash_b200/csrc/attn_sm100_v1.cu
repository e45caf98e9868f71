// Tensor-core kernels for the first-generation semantics (adasplash/adasplash_block_mask.py:
// `sparse_attn(q, k, v, alpha, is_causal, varlen, niter)`): any alpha in (1, 2], causal or full
// attention.  The same kernel templates as the AdaSplash-2 path, instantiated with the other row
// math (alpha = 2: p = u, Jacobian weight 1 on the support) and without the causal tile ranges;
// a translation unit of its own so that the two sets of kernels compile side by side.
#include "sm100_launch.cuh"

namespace ads {
namespace sm100 {
namespace v1 {

namespace {

template <typename T, int D>
int solve_td(const simt::Params& p, void* ws, size_t ws_bytes, cudaStream_t st) {
  return solve_t<T, D, true>(p, ws, ws_bytes, st);   // alpha and the mask are run-time parameters of the solver
}

// row math of the kernels: 0 = alpha 1.5, 1 = alpha 2, 2 = any other alpha (lg2 / ex2 powers)
inline int alpha_mode(float alpha) { return alpha == 1.5f ? 0 : (alpha == 2.0f ? 1 : 2); }

template <typename T, int D>
int fwd_td(const simt::Params& p, void* ws, cudaStream_t st) {
  switch (alpha_mode(p.alpha) * 2 + (p.causal ? 1 : 0)) {
    case 0: return fwd_t<T, D, 0, false>(p, ws, st);
    case 1: return fwd_t<T, D, 0, true>(p, ws, st);
    case 2: return fwd_t<T, D, 1, false>(p, ws, st);
    case 3: return fwd_t<T, D, 1, true>(p, ws, st);
    case 4: return fwd_t<T, D, 2, false>(p, ws, st);
    default: return fwd_t<T, D, 2, true>(p, ws, st);
  }
}

template <typename T, int D>
int bwd_td(const simt::Params& p, void* ws, cudaStream_t st) {
  switch (alpha_mode(p.alpha) * 2 + (p.causal ? 1 : 0)) {
    case 0: return bwd_t<T, D, 0, false>(p, ws, st);
    case 1: return bwd_t<T, D, 0, true>(p, ws, st);
    case 2: return bwd_t<T, D, 1, false>(p, ws, st);
    case 3: return bwd_t<T, D, 1, true>(p, ws, st);
    case 4: return bwd_t<T, D, 2, false>(p, ws, st);
    default: return bwd_t<T, D, 2, true>(p, ws, st);
  }
}

template <typename F64, typename F128>
int by_head_dim(int D, F64 f64, F128 f128) {
  switch (D) {
    case 16: case 32:  // zero-padded to 64 columns by the TMA loads
    case 64: return f64();
    case 128: return f128();
  }
  set_error("sm100: head dim %d not built", D);
  return ADS_ERR_UNSUPPORTED;
}

}  // namespace

int solve(const simt::Params& p, int dtype, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (dtype == ADS_F16)
    return by_head_dim(p.D, [&] { return solve_td<__half, 64>(p, ws, ws_bytes, st); },
                       [&] { return solve_td<__half, 128>(p, ws, ws_bytes, st); });
  return by_head_dim(p.D, [&] { return solve_td<__nv_bfloat16, 64>(p, ws, ws_bytes, st); },
                     [&] { return solve_td<__nv_bfloat16, 128>(p, ws, ws_bytes, st); });
}

int fwd(const simt::Params& p, int dtype, void* ws, cudaStream_t st) {
  if (dtype == ADS_F16)
    return by_head_dim(p.D, [&] { return fwd_td<__half, 64>(p, ws, st); }, [&] { return fwd_td<__half, 128>(p, ws, st); });
  return by_head_dim(p.D, [&] { return fwd_td<__nv_bfloat16, 64>(p, ws, st); },
                     [&] { return fwd_td<__nv_bfloat16, 128>(p, ws, st); });
}

int bwd(const simt::Params& p, int dtype, void* ws, cudaStream_t st) {
  if (dtype == ADS_F16)
    return by_head_dim(p.D, [&] { return bwd_td<__half, 64>(p, ws, st); }, [&] { return bwd_td<__half, 128>(p, ws, st); });
  return by_head_dim(p.D, [&] { return bwd_td<__nv_bfloat16, 64>(p, ws, st); },
                     [&] { return bwd_td<__nv_bfloat16, 128>(p, ws, st); });
}

int set_wait_constants_v1(long long max_wait_cycles, int withhold_loads) {
  return set_wait_constants(max_wait_cycles, withhold_loads);
}

}  // namespace v1
}  // namespace sm100
}  // namespace ads
