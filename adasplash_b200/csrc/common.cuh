// Shared helpers for the sm_100a entmax attention kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdio>

#include "../../include/adasplash_b200.h"

namespace ads {

constexpr float kMaskedScore = -10000.0f;  // fill value of causal / padded keys
constexpr int kTile = 64;                  // block-mask granularity (rows and keys)

void set_error(const char* fmt, ...);
extern std::atomic<long long> g_launches;

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return ADS_ERR_CUDA;
  }
  return ADS_OK;
}

template <typename T> struct DT;
template <> struct DT<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct DT<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct DT<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// Round an fp32 value to T and back (what a Triton `.to(dtype)` does to an operand).
template <typename T> __device__ __forceinline__ float round_to(float v) {
  return DT<T>::to_f(DT<T>::from_f(v));
}

__device__ __forceinline__ int load_len(const void* varlen, int is_i64, int b, int n) {
  if (varlen == nullptr) return n;
  long long v = is_i64 ? reinterpret_cast<const long long*>(varlen)[b]
                       : (long long)reinterpret_cast<const int*>(varlen)[b];
  if (v < 0) v = 0;
  if (v > n) v = n;
  return (int)v;
}

// Histogram bin count of the attention solver: the largest of {8,4,2} whose
// packed 64/BINS-bit counter would hold ceil(N/64) (adasplash_v2.py:273-289).
// The counters here are plain 32-bit integers; BINS is kept because it fixes
// the start bracket and therefore the trajectory of tau.
inline int select_bins(int n_ctx) {
  long long max_count = (n_ctx + 63) / 64;
  if (max_count <= 255) return 8;
  if (max_count <= 65535) return 4;
  return 2;
}

struct HalleyState {
  float t, lo, hi;
};

// One Halley step with bisection fallback for f(t) = sum [z-t]_+^2 - 1
// (adasplash_v2.py:68-90).  a0 = sum u^2, a1 = sum u, a2 = #support.
__device__ __forceinline__ void halley_bisect_update(HalleyState& s, float a0, float a1, float a2) {
  const float eps = 1e-5f;
  float ff = a0 - 1.0f;
  float df = -2.0f * a1;
  float ddf = 2.0f * a2;
  if (ff > 0.f) s.lo = s.t;
  if (ff < 0.f) s.hi = s.t;
  float nt = s.t - (ff * df) / (df * df - 0.5f * ff * ddf);
  bool good = (nt > s.lo - eps) && (nt < s.hi + eps);
  s.t = good ? nt : 0.5f * (s.lo + s.hi);
}

// The same step for f(t) = sum [z-t]_+^c0 - 1 with any alpha: a0 = sum u^c0,
// a1 = sum u^(c0-1), a2 = sum u^(c0-2) (adasplash_block_mask.py:40-296; for
// alpha = 2 the second derivative vanishes and the step is Newton's).
__device__ __forceinline__ void halley_bisect_update_generic(HalleyState& s, float a0, float a1,
                                                            float a2, float c0, float c1) {
  const float eps = 1e-5f;
  float ff = a0 - 1.0f;
  float df = -c0 * a1;
  float ddf = c0 * c1 * a2;
  if (ff > 0.f) s.lo = s.t;
  if (ff < 0.f) s.hi = s.t;
  float nt = s.t - (2.0f * ff * df) / (2.0f * df * df - ff * ddf);
  bool good = (nt > s.lo - eps) && (nt < s.hi + eps);
  s.t = good ? nt : 0.5f * (s.lo + s.hi);
}

// Closed-form lower bound of tau from a BINS-bin histogram of z - tau0 on [0,1]
// (adasplash_v2.py:434-461).  cnt[b] = raw count of bin b (top bin still
// includes the row maximum itself).
template <int MAXB>
__device__ __forceinline__ float hist_tau_alpha15(const int* cnt, int bins, float tau0) {
  float sz = 1.f, sn = 1.f, szz = 1.f;
  for (int sj = bins - 1; sj >= 0; --sj) {
    float c = (float)(cnt[sj] - (sj == bins - 1 ? 1 : 0));
    float e = (float)sj / (float)bins;
    float nzz = szz + c * (e * e);
    float nz = sz + c * e;
    float nn = sn + c;
    bool good = (nn * e * e - 2.f * nz * e + nzz) < 1.0f;
    if (good) { szz = nzz; sz = nz; sn = nn; }
  }
  return tau0 + (sz - sqrtf(sz * sz - sn * (szz - 1.0f))) / sn;
}

}  // namespace ads
