// Row-wise entmax forward / backward for sm_100a (HBM-bound).
//
// One group of TPR threads owns one row and keeps it in registers, so the row
// is read from HBM exactly once and the result written once: 8 bytes per fp32
// element forward, 12 backward.  Reductions are warp shuffles, plus one shared
// memory hop when a row spans several warps.  Rows too long for registers use a
// streaming variant that re-reads the row from L2/HBM.
//
// Only the elements within 1 of the row maximum can be in the support (the largest
// probability [z_max - tau]_+^(1/(alpha-1)) is at most 1, so tau >= z_max - 1).  After the
// maximum is known, every thread notes which of its own elements those are -- a handful per
// row for peaked inputs -- in a few private shared-memory slots, in the order it holds them;
// the histogram and every refinement step then run over the slots.  A thread with more
// candidates than slots (nearly flat rows) sweeps all of its elements instead; both ways add
// the same terms in the same order, so the result does not depend on which one ran.
//
// The threshold search follows adasplash/triton_entmax_v2.py:361-536 (4-bin
// histogram lower bound, quadratic start on the bin-centre model, Halley /
// Newton / secant / bisection refinement); the backward follows :539-617.
#include "common.cuh"

namespace ads {
namespace {

constexpr int kBins = 4;  // triton_entmax_v2.py:386

struct Sum3 { float a, b, c; };

// Barrier among the TPR threads of one row group (a CTA may hold two groups of 64 threads that
// take different routes through the solver, so CTA-wide barriers would not match up).
template <int TPR>
__device__ __forceinline__ void group_sync() {
  if constexpr (TPR > 32) {
    if constexpr (TPR >= 128) __syncthreads();   // one group per CTA
    else asm volatile("bar.sync %0, %1;" ::"r"(1 + (int)(threadIdx.x / TPR)), "r"(TPR) : "memory");
  } else {
    __syncwarp();
  }
}

template <int TPR>
struct GroupReduce {
  // smem: [2][CTA_WARPS][4] floats, double buffered by `phase`
  float* smem;
  int phase;
  int group_warp0;  // first warp index of this group inside the CTA
  __device__ GroupReduce(float* s) : smem(s), phase(0) {
    group_warp0 = (threadIdx.x / TPR) * (TPR / 32);
  }
  template <typename Op>
  __device__ __forceinline__ void reduce4(float v[4], Op op) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = op(v[i], __shfl_xor_sync(0xffffffffu, v[i], o));
    }
    if constexpr (TPR > 32) {
      const int warps_cta = blockDim.x / 32;
      float* buf = smem + phase * warps_cta * 4;
      int w = threadIdx.x / 32;
      if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) buf[w * 4 + i] = v[i];
      }
      group_sync<TPR>();
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = buf[group_warp0 * 4 + i];
      for (int g = 1; g < TPR / 32; ++g) {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = op(v[i], buf[(group_warp0 + g) * 4 + i]);
      }
      phase ^= 1;
    }
  }
};

struct OpAdd { __device__ __forceinline__ float operator()(float a, float b) const { return a + b; } };
struct OpMax { __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); } };

__device__ __forceinline__ float masked_pow(float x, bool m, float c, int fast_math) {
  // triton_entmax_v2.py:22-39: fast_powf(x, c), or exp2(log2(max(x, 1e-6)) * c) -- both are
  // the approximate ex2 / lg2 units in the reference's build.  Evaluated on the support only.
  if (!m) return 0.f;
  const float base = fast_math ? x : fmaxf(x, 1e-6f);
  return exp2f(__log2f(base) * c);
}

// base^c0, base^(c0-1), base^(c0-2) for one support element: one lg2, one ex2 and two
// fast divisions instead of three lg2/ex2 pairs.
__device__ __forceinline__ void pow3(float u, float c0, int fast_math, float& p0, float& p1, float& p2) {
  const float base = fast_math ? u : fmaxf(u, 1e-6f);
  p0 = exp2f(__log2f(base) * c0);
  p1 = __fdividef(p0, base);
  p2 = __fdividef(p1, base);
}

__device__ __forceinline__ float f_hist(float tau, float t_shift, const float* raw) {
  // bin-centre model sum_b c_b [centre_b - tau]_+^2 - 1 (triton_entmax_v2.py:164-204)
  float acc = 0.f;
#pragma unroll
  for (int b = 0; b < kBins; ++b) {
    float d = (t_shift + (b + 0.5f) / kBins) - tau;
    float dp = d > 0.f ? d : 0.f;
    acc += raw[b] * dp * dp;
  }
  return acc - 1.0f;
}

__device__ __forceinline__ float muller_init(float a, float c, float t_shift, const float* raw) {
  // triton_entmax_v2.py:207-322
  const float eps = 1e-10f;
  float b = 0.5f * (a + c);
  float fa = f_hist(a, t_shift, raw), fb = f_hist(b, t_shift, raw), fc = f_hist(c, t_shift, raw);
  float denom = (a - b) * (a - c) * (b - c);
  float mid = 0.5f * (a + c);
  float A = (fa * (b - c) + fb * (c - a) + fc * (a - b)) / denom;
  float B = (fa * (c * c - b * b) + fb * (a * a - c * c) + fc * (b * b - a * a)) / denom;
  float C = (fa * b * c * (b - c) + fb * a * c * (c - a) + fc * a * b * (a - b)) / denom;
  float x_lin = fabsf(B) > eps ? -C / B : mid;
  float disc = B * B - 4.f * A * C;
  float sq = sqrtf(fmaxf(disc, 0.f));
  float r1 = (-B + sq) / (2.f * A), r2 = (-B - sq) / (2.f * A);
  bool v1 = (r1 >= a) && (r1 <= c), v2 = (r2 >= a) && (r2 <= c);
  float d1 = fabsf(c - r1), d2 = fabsf(c - r2);
  float xq = (v1 && v2) ? (d1 <= d2 ? r1 : r2) : (v1 ? r1 : (v2 ? r2 : mid));
  float sden = fc - fa;
  float xs = fabsf(sden) > eps ? c - fc * (c - a) / sden : mid;
  if (!(disc >= 0.f)) xq = xs;
  float x = (fabsf(A) < eps) ? x_lin : xq;
  if (fabsf(denom) < eps) x = mid;
  return fminf(fmaxf(x, a), c);
}

struct Hybrid {
  float t, lo, hi, t_prev, f_prev;
};

__device__ __forceinline__ void hybrid_update(Hybrid& s, float a0, float a1, float a2, float c0,
                                              float c1, float alpha, bool allow_secant) {
  // triton_entmax_v2.py:42-110
  const float eps = 1e-6f, eps_den = 1e-12f;
  float t = s.t;
  float ff = a0 - 1.0f, df = -c0 * a1, ddf = c0 * c1 * a2;
  if (ff > 0.f) s.lo = t;
  if (ff < 0.f) s.hi = t;
  bool has = false;
  float cand = 0.f;
  {
    float den = 2.f * df * df - ff * ddf;
    float th = t - (2.f * ff * df) / den;
    bool ok = (th > s.lo - eps) && (th < s.hi + eps) && !isinf(th) && (fabsf(den) > eps_den) &&
              (alpha <= 1.5f);
    if (ok) { cand = th; has = true; }
  }
  if (!has) {
    float tn = t - ff / df;
    bool ok = (tn > s.lo - eps) && (tn < s.hi + eps) && !isinf(tn) && (fabsf(df) > eps_den) &&
              (alpha <= 2.0f);
    if (ok) { cand = tn; has = true; }
  }
  if (!has && allow_secant) {
    float den = ff - s.f_prev;
    float ts = t - ff * (t - s.t_prev) / den;
    bool ok = (ts > s.lo - eps) && (ts < s.hi + eps) && !isinf(ts) && (fabsf(den) > eps_den);
    if (ok) { cand = ts; has = true; }
  }
  s.t_prev = t;
  s.f_prev = ff;
  s.t = has ? cand : 0.5f * (s.lo + s.hi);
}

// ---------------------------------------------------------------------------
// Row sources: where the (alpha-1)-scaled row elements come from.
// ---------------------------------------------------------------------------
template <typename T, int TPR, int NV, bool VEC>
struct RegRow {
  float v[NV * 4];
  int cols, tl;
  __device__ __forceinline__ int col_of(int c, int e) const {
    return VEC ? (c * TPR + tl) * 4 + e : (c * 4 + e) * TPR + tl;
  }
  __device__ __forceinline__ void load(const T* row, int cols_, float sc) {
    cols = cols_;
    tl = threadIdx.x % TPR;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      if constexpr (VEC) {
        int c0 = (c * TPR + tl) * 4;
        if (c0 < cols) {  // cols % 4 == 0 on this path
          if constexpr (sizeof(T) == 4) {
            float4 q = *reinterpret_cast<const float4*>(row + c0);
            v[c * 4 + 0] = q.x * sc; v[c * 4 + 1] = q.y * sc;
            v[c * 4 + 2] = q.z * sc; v[c * 4 + 3] = q.w * sc;
          } else {
            uint2 q = *reinterpret_cast<const uint2*>(row + c0);
            const T* h = reinterpret_cast<const T*>(&q);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[c * 4 + e] = DT<T>::to_f(h[e]) * sc;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) v[c * 4 + e] = -INFINITY;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int col = col_of(c, e);
          v[c * 4 + e] = col < cols ? DT<T>::to_f(row[col]) * sc : -INFINITY;
        }
      }
    }
  }
  // Chunk c of this thread was copied to sbuf[(c * nthreads + tid) * 4 elements] (VEC layout).
  __device__ __forceinline__ void load_staged(const T* sbuf, int nthreads, int cols_, float sc) {
    cols = cols_;
    tl = threadIdx.x % TPR;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const int c0 = (c * TPR + tl) * 4;
      const T* src = sbuf + (size_t)(c * nthreads + threadIdx.x) * 4;
      if (c0 < cols) {
        if constexpr (sizeof(T) == 4) {
          const float4 q = *reinterpret_cast<const float4*>(src);
          v[c * 4 + 0] = q.x * sc; v[c * 4 + 1] = q.y * sc;
          v[c * 4 + 2] = q.z * sc; v[c * 4 + 3] = q.w * sc;
        } else {
          const uint2 q = *reinterpret_cast<const uint2*>(src);
          const T* h = reinterpret_cast<const T*>(&q);
#pragma unroll
          for (int e = 0; e < 4; ++e) v[c * 4 + e] = DT<T>::to_f(h[e]) * sc;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[c * 4 + e] = -INFINITY;
      }
    }
  }
  template <typename F> __device__ __forceinline__ void for_each(F f) const {
#pragma unroll
    for (int i = 0; i < NV * 4; ++i) f(v[i]);
  }
  // maximum of this thread's elements (independent chains instead of one dependent one)
  __device__ __forceinline__ float max() const {
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV * 4; i += 4) {
      m0 = fmaxf(m0, fmaxf(v[i], v[i + 1]));
      m1 = fmaxf(m1, fmaxf(v[i + 2], v[i + 3]));
    }
    return fmaxf(m0, m1);
  }
  // f(x) for every element >= thr, in element order; groups of four are skipped with one test
  template <typename F> __device__ __forceinline__ void for_each_at_least(float thr, F f) const {
#pragma unroll
    for (int i = 0; i < NV * 4; i += 4) {
      const float m4 = fmaxf(fmaxf(v[i], v[i + 1]), fmaxf(v[i + 2], v[i + 3]));
      if (m4 >= thr) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (v[i + e] >= thr) f(v[i + e]);
      }
    }
  }
  template <typename F> __device__ __forceinline__ void store(T* row, F f) const {
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      if constexpr (VEC) {
        int c0 = (c * TPR + tl) * 4;
        if (c0 < cols) {
          if constexpr (sizeof(T) == 4) {
            float4 q = make_float4(f(v[c * 4]), f(v[c * 4 + 1]), f(v[c * 4 + 2]), f(v[c * 4 + 3]));
            *reinterpret_cast<float4*>(row + c0) = q;
          } else {
            uint2 q;
            T* h = reinterpret_cast<T*>(&q);
#pragma unroll
            for (int e = 0; e < 4; ++e) h[e] = DT<T>::from_f(f(v[c * 4 + e]));
            *reinterpret_cast<uint2*>(row + c0) = q;
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int col = col_of(c, e);
          if (col < cols) row[col] = DT<T>::from_f(f(v[c * 4 + e]));
        }
      }
    }
  }
};

template <typename T, int TPR>
struct StreamRow {  // re-reads the row from global memory on every pass
  const T* row;
  int cols, tl;
  float sc;
  __device__ __forceinline__ void load(const T* r, int cols_, float sc_) {
    row = r; cols = cols_; sc = sc_; tl = threadIdx.x % TPR;
  }
  template <typename F> __device__ __forceinline__ void for_each(F f) const {
    for (int c = tl; c < cols; c += TPR) f(DT<T>::to_f(row[c]) * sc);
  }
  __device__ __forceinline__ float max() const {
    float m = -INFINITY;
    for (int c = tl; c < cols; c += TPR) m = fmaxf(m, DT<T>::to_f(row[c]) * sc);
    return m;
  }
  template <typename F> __device__ __forceinline__ void for_each_at_least(float thr, F f) const {
    for (int c = tl; c < cols; c += TPR) {
      const float x = DT<T>::to_f(row[c]) * sc;
      if (x >= thr) f(x);
    }
  }
  template <typename F> __device__ __forceinline__ void store(T* out, F f) const {
    for (int c = tl; c < cols; c += TPR) out[c] = DT<T>::from_f(f(DT<T>::to_f(row[c]) * sc));
  }
};

constexpr int kCandSlots = 8;  // candidates a thread keeps in shared memory (slot j of thread t: [j * blockDim.x + t])

// Maximum over the TPR threads of a row group.  Inside a warp it is one integer reduction on an
// order-preserving image of the float (redux.sync has no float form before this image).
__device__ __forceinline__ int ordered_int(float x) {
  const int i = __float_as_int(x);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ordered_float(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

template <int TPR>
__device__ __forceinline__ float group_max(float x, float* smem_max) {
  float m = ordered_float(__reduce_max_sync(0xffffffffu, ordered_int(x)));
  if constexpr (TPR > 32) {
    const int w = threadIdx.x / 32, g0 = (threadIdx.x / TPR) * (TPR / 32);
    if ((threadIdx.x & 31) == 0) smem_max[w] = m;
    group_sync<TPR>();
    m = smem_max[g0];
    for (int g = 1; g < TPR / 32; ++g) m = fmaxf(m, smem_max[g0 + g]);
    // smem_max is not written again by this kernel: no second barrier needed
  }
  return m;
}

template <typename T, int TPR, typename Row>
__device__ __forceinline__ void entmax_fwd_row(Row& r, T* yrow, float* tau_out, long long row_idx,
                                               bool row_ok, float alpha, int n_iter, int use_hist,
                                               int fast_math, float* smem, float* smem_max,
                                               float* s_cand) {
  GroupReduce<TPR> red(smem);
  const int mode = (alpha == 1.5f) ? 0 : (alpha == 2.0f ? 1 : 2);
  const float c0 = 1.0f / (alpha - 1.0f), c1 = c0 - 1.0f, c2 = c1 - 1.0f;
  (void)c2;
  float red4[4];
  // stage 1: maximum of the scaled row
  const float mx = group_max<TPR>(r.max(), smem_max);
  // Candidates: tau never falls below max - 1 (minus the 1e-6 slack of the bracket test), so
  // nothing below that can enter a sum.  Each thread keeps its own in its own slots.
  int n_cand = 0;
  {
    float* mine = s_cand + threadIdx.x;
    const int stride = blockDim.x;
    r.for_each_at_least(mx - 1.0f - 1e-5f, [&](float x) {
      if (n_cand < kCandSlots) mine[n_cand * stride] = x;
      ++n_cand;
    });
  }
  // The threshold search: `each(f)` calls f on every candidate this thread is responsible for and
  // `reduce_sums` adds the partial sums over the threads that take part.
  Hybrid s;
  auto solve = [&](auto each, auto reduce_sums) {
    if (use_hist && alpha <= 2.0f) {
      // stage 2: 4-bin histogram of x - (max-1) on [0,1]; cumulative counts
      // N_b = #{proj*4 >= b} give the same bins as floor(proj*4) clamped to 3.
      float t_init = mx - 1.0f;
      float n0 = 0.f, n1 = 0.f, n2 = 0.f, n3 = 0.f;
      each([&](float x) {
        const float d = x - t_init;
        if (d >= 0.f) {  // only the few elements within 1 of the row maximum land in a bin
          const float p4 = d * (float)kBins;
          n0 += 1.f;
          n1 += (p4 >= 1.f) ? 1.f : 0.f;
          n2 += (p4 >= 2.f) ? 1.f : 0.f;
          n3 += (p4 >= 3.f) ? 1.f : 0.f;
        }
      });
      red4[0] = n0; red4[1] = n1; red4[2] = n2; red4[3] = n3;
      reduce_sums(red4);
      float raw[kBins] = {red4[0] - red4[1], red4[1] - red4[2], red4[2] - red4[3], red4[3]};
      float t0;
      if (mode == 0) {
        int cnt[kBins] = {(int)raw[0], (int)raw[1], (int)raw[2], (int)raw[3]};
        t0 = hist_tau_alpha15<kBins>(cnt, kBins, t_init);
      } else {  // alpha == 2 (triton_entmax_v2.py:113-131)
        float sz = 1.f, sk = 1.f;
        for (int sj = kBins - 1; sj >= 0; --sj) {
          float c = raw[sj] - (sj == kBins - 1 ? 1.f : 0.f);
          float e = (float)sj / kBins;
          float nz = sz + c * e, nk = sk + c;
          if ((nz - nk * e) < 1.0f) { sz = nz; sk = nk; }
        }
        t0 = t_init + (sz - 1.0f) / sk;
      }
      s.lo = t0;
      s.hi = t0 + 1.0f / kBins;
      s.t = muller_init(s.lo, s.hi, t_init, raw);
    } else {
      s.hi = mx;
      s.lo = mx - 1.0f;
      s.t = 0.5f * (s.lo + s.hi);
    }
    s.t_prev = s.t;
    s.f_prev = 0.f;
    // stage 3: refinement
    for (int it = 0; it < n_iter; ++it) {
      float a0 = 0.f, a1 = 0.f, a2 = 0.f;
      const float t = s.t;
      if (mode == 1) {
        each([&](float x) { if (x > t) { a0 += x - t; a1 += 1.f; } });
      } else if (mode == 0) {
        each([&](float x) {
          if (x > t) {  // the support is a small part of the row
            const float u = x - t;
            a0 = fmaf(u, u, a0); a1 += u; a2 += 1.f;
          }
        });
      } else {
        each([&](float x) {
          if (x > t) {  // the support is a small part of the row: skip the transcendental work elsewhere
            float p0, p1, p2;
            pow3(x - t, c0, fast_math, p0, p1, p2);
            a0 += p0; a1 += p1; a2 += p2;
          }
        });
      }
      red4[0] = a0; red4[1] = a1; red4[2] = a2; red4[3] = 0.f;
      reduce_sums(red4);
      hybrid_update(s, red4[0], red4[1], red4[2], c0, c1, alpha, it > 0);
    }
  };
  // Every thread works through its own slots, or through all of its elements if they did not fit
  // (same elements above any threshold >= max - 1 - 1e-5, same order), and the sums are reduced
  // over the group.  Two alternatives were measured slower on 16384 x 4096 (0.117 vs 0.096 ms for
  // alpha = 1.5, 0.21 / 0.30 vs 0.20 ms for alpha = 1.333): gathering the row's candidates in one
  // list that every warp works through by itself without barriers, and letting the first warp of
  // the group do the whole search alone.  The search is a dependent chain per row; what pays is
  // more rows in flight, not fewer instructions.
  solve([&](auto f) {
          if (n_cand <= kCandSlots) {
            const float* mine = s_cand + threadIdx.x;
            for (int j = 0; j < n_cand; ++j) f(mine[j * blockDim.x]);
          } else {
            r.for_each(f);
          }
        },
        [&](float v[4]) { red.reduce4(v, OpAdd()); });
  // stage 4: output
  const float t = s.t;
  if (row_ok) {
    if (mode == 1) {
      r.store(yrow, [&](float x) { return x > t ? x - t : 0.f; });
    } else if (mode == 0) {
      r.store(yrow, [&](float x) { float u = x > t ? x - t : 0.f; return u * u; });
    } else {
      r.store(yrow, [&](float x) { return masked_pow(fmaxf(x - t, 0.f), x > t, c0, fast_math); });
    }
    if (tau_out != nullptr && (threadIdx.x % TPR) == 0) tau_out[row_idx] = t;
  }
}

// (Rows in flight per SM bound this kernel: a row's life is a DRAM round trip plus a chain of
// reductions, so the register cap -- 8 CTAs of 128 threads instead of 6 -- is worth 10 %.)
template <typename T, int TPR, int NV, bool VEC>
__global__ void __launch_bounds__((TPR > 128 ? TPR : 128), (TPR <= 128 ? 8 : 1))
entmax_fwd_reg_kernel(const T* __restrict__ x, T* __restrict__ y, float* __restrict__ tau_out,
                      long long rows, int cols, float alpha, int n_iter, int use_hist,
                      int fast_math) {
  constexpr int THREADS = TPR > 128 ? TPR : 128;
  __shared__ float smem[2 * 32 * 4];
  __shared__ float smem_max[32];
  __shared__ float s_cand[kCandSlots * THREADS];
  const int rows_per_cta = blockDim.x / TPR;
  const int grp = threadIdx.x / TPR;
  long long row = (long long)blockIdx.x * rows_per_cta + grp;
  bool ok = row < rows;
  long long rr = ok ? row : rows - 1;
  RegRow<T, TPR, NV, VEC> r;
  r.load(x + rr * cols, cols, alpha - 1.0f);
  entmax_fwd_row<T, TPR>(r, y + rr * cols, tau_out, rr, ok, alpha, n_iter, use_hist, fast_math, smem,
                         smem_max, s_cand);
}

// The same, for matrices with many rows: a row group walks kPipeRows consecutive rows and, while
// it works on one, its threads' chunks of the next are already on their way into shared memory
// (cp.async, 4 elements per chunk; a thread reads back only what it copied itself, so the copy
// needs no barrier).  That doubles the rows in flight per SM at the same register budget.
constexpr int kPipeRows = 4;

template <int BYTES>
__device__ __forceinline__ void cp_async(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  if constexpr (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(gmem_src) : "memory");
}

template <typename T, int TPR, int NV>
__global__ void __launch_bounds__((TPR > 128 ? TPR : 128), (TPR <= 128 ? 8 : 1))
entmax_fwd_pipe_kernel(const T* __restrict__ x, T* __restrict__ y, float* __restrict__ tau_out,
                       long long rows, int cols, float alpha, int n_iter, int use_hist,
                       int fast_math) {
  constexpr int THREADS = TPR > 128 ? TPR : 128;
  __shared__ float smem[2 * 32 * 4];
  __shared__ float smem_max[32];
  __shared__ float s_cand[kCandSlots * THREADS];
  __shared__ __align__(16) T s_row[THREADS * NV * 4];
  const int groups = THREADS / TPR;
  const int grp = threadIdx.x / TPR, tl = threadIdx.x % TPR;
  const long long first = ((long long)blockIdx.x * groups + grp) * kPipeRows;
  auto prefetch = [&](long long row) {
    if (row < rows) {
      const T* src = x + row * cols;
#pragma unroll
      for (int c = 0; c < NV; ++c) {
        const int c0 = (c * TPR + tl) * 4;
        if (c0 < cols) cp_async<4 * sizeof(T)>(s_row + (size_t)(c * THREADS + threadIdx.x) * 4, src + c0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  prefetch(first);
  for (int i = 0; i < kPipeRows; ++i) {
    const long long row = first + i;
    const bool ok = row < rows;   // a group beyond the matrix still runs the barriers of its CTA
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    RegRow<T, TPR, NV, true> r;
    r.load_staged(s_row, THREADS, cols, alpha - 1.0f);
    if (!ok) {
#pragma unroll
      for (int e = 0; e < NV * 4; ++e) r.v[e] = 0.f;
    }
    if (i + 1 < kPipeRows) prefetch(row + 1);
    const long long rr = ok ? row : rows - 1;
    entmax_fwd_row<T, TPR>(r, y + rr * cols, tau_out, rr, ok, alpha, n_iter, use_hist, fast_math, smem,
                           smem_max, s_cand);
    group_sync<TPR>();  // the reduction buffers are reused by the next row
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
entmax_fwd_stream_kernel(const T* __restrict__ x, T* __restrict__ y, float* __restrict__ tau_out,
                         long long rows, int cols, float alpha, int n_iter, int use_hist,
                         int fast_math) {
  __shared__ float smem[2 * 32 * 4];
  __shared__ float smem_max[32];
  __shared__ float s_cand[kCandSlots * 1024];
  long long row = blockIdx.x;
  StreamRow<T, 1024> r;
  r.load(x + row * cols, cols, alpha - 1.0f);
  entmax_fwd_row<T, 1024>(r, y + row * cols, tau_out, row, true, alpha, n_iter, use_hist, fast_math, smem,
                          smem_max, s_cand);
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
__device__ __forceinline__ float bwd_u(float y, float alpha, int mode, int fast_math) {
  bool m = y > 0.f;
  if (mode == 1) return m ? 1.f : 0.f;
  if (mode == 0) return m ? sqrtf(y) : 0.f;
  return masked_pow(y, m, 2.0f - alpha, fast_math);
}

template <typename T, int TPR, int NV, bool VEC>
__global__ void __launch_bounds__((TPR > 128 ? TPR : 128))
entmax_bwd_reg_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                      long long rows, int cols, float alpha, int fast_math) {
  __shared__ float smem[2 * 32 * 4];
  const int rows_per_cta = blockDim.x / TPR;
  long long row = (long long)blockIdx.x * rows_per_cta + threadIdx.x / TPR;
  bool ok = row < rows;
  long long rr = ok ? row : rows - 1;
  const int mode = (alpha == 1.5f) ? 0 : (alpha == 2.0f ? 1 : 2);
  RegRow<T, TPR, NV, VEC> ry, rdy;
  ry.load(y + rr * cols, cols, 1.0f);
  rdy.load(dy + rr * cols, cols, 1.0f);
  float su = 0.f, sud = 0.f;
#pragma unroll
  for (int i = 0; i < NV * 4; ++i) {
    // out-of-range slots hold -inf in both rows: y > 0 is false there, u = 0
    float u = bwd_u(ry.v[i], alpha, mode, fast_math);
    ry.v[i] = u;
    float d = (u != 0.f) ? rdy.v[i] : 0.f;
    rdy.v[i] = d;
    su += u;
    sud = fmaf(u, d, sud);
  }
  GroupReduce<TPR> red(smem);
  float red4[4] = {su, sud, 0.f, 0.f};
  red.reduce4(red4, OpAdd());
  float scalar = red4[1] / red4[0];
  if (ok) {
    // grad = u*dy - scalar*u (triton_entmax_v2.py:616)
#pragma unroll
    for (int i = 0; i < NV * 4; ++i) rdy.v[i] = ry.v[i] * rdy.v[i] - scalar * ry.v[i];
    rdy.store(dx + rr * cols, [](float g) { return g; });
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
entmax_bwd_stream_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                         long long rows, int cols, float alpha, int fast_math) {
  __shared__ float smem[2 * 32 * 4];
  long long row = blockIdx.x;
  const int mode = (alpha == 1.5f) ? 0 : (alpha == 2.0f ? 1 : 2);
  const T* yr = y + row * cols;
  const T* dr = dy + row * cols;
  float su = 0.f, sud = 0.f;
  for (int c = threadIdx.x; c < cols; c += 1024) {
    float u = bwd_u(DT<T>::to_f(yr[c]), alpha, mode, fast_math);
    su += u;
    sud = fmaf(u, DT<T>::to_f(dr[c]), sud);
  }
  GroupReduce<1024> red(smem);
  float red4[4] = {su, sud, 0.f, 0.f};
  red.reduce4(red4, OpAdd());
  float scalar = red4[1] / red4[0];
  T* xr = dx + row * cols;
  for (int c = threadIdx.x; c < cols; c += 1024) {
    float u = bwd_u(DT<T>::to_f(yr[c]), alpha, mode, fast_math);
    xr[c] = DT<T>::from_f(u * DT<T>::to_f(dr[c]) - scalar * u);
  }
}

template <typename T, int TPR, int NV>
int launch_fwd_cfg(const T* x, T* y, float* tau, long long rows, int cols, float alpha, int n_iter,
                   int use_hist, int fast_math, bool vec, cudaStream_t st) {
  const int threads = TPR > 128 ? TPR : 128;
  const int rpc = threads / TPR;
  unsigned grid = (unsigned)((rows + rpc - 1) / rpc);
  if constexpr (TPR <= 128) {
    if (vec && rows >= 8192) {
      const long long per_cta = (long long)rpc * kPipeRows;
      entmax_fwd_pipe_kernel<T, TPR, NV><<<(unsigned)((rows + per_cta - 1) / per_cta), threads, 0, st>>>(
          x, y, tau, rows, cols, alpha, n_iter, use_hist, fast_math);
      return check_launch("entmax_fwd");
    }
  }
  if (vec)
    entmax_fwd_reg_kernel<T, TPR, NV, true><<<grid, threads, 0, st>>>(x, y, tau, rows, cols, alpha, n_iter, use_hist, fast_math);
  else
    entmax_fwd_reg_kernel<T, TPR, NV, false><<<grid, threads, 0, st>>>(x, y, tau, rows, cols, alpha, n_iter, use_hist, fast_math);
  return check_launch("entmax_fwd");
}

template <typename T>
int launch_fwd(const void* xv, void* yv, float* tau, long long rows, long long cols, float alpha,
               int n_iter, int use_hist, int fast_math, cudaStream_t st) {
  const T* x = (const T*)xv;
  T* y = (T*)yv;
  const size_t vec_bytes = 4 * sizeof(T);
  bool vec = (cols % 4 == 0) && ((uintptr_t)x % vec_bytes == 0) && ((uintptr_t)y % vec_bytes == 0);
  int c = (int)cols;
#define ADS_FWD(TPR, NV) return launch_fwd_cfg<T, TPR, NV>(x, y, tau, rows, c, alpha, n_iter, use_hist, fast_math, vec, st)
  if (cols <= 128) ADS_FWD(32, 1);
  if (cols <= 512) ADS_FWD(32, 4);
  if (cols <= 1024) ADS_FWD(32, 8);
  if (cols <= 2048) ADS_FWD(64, 8);
  if (cols <= 4096) ADS_FWD(128, 8);  // measured best of (32,32), (64,16), (128,8), (256,4) on 16384 x 4096
  if (cols <= 8192) ADS_FWD(256, 8);
  if (cols <= 16384) ADS_FWD(512, 8);
  if (cols <= 32768) ADS_FWD(1024, 8);
#undef ADS_FWD
  entmax_fwd_stream_kernel<T><<<(unsigned)rows, 1024, 0, st>>>(x, y, tau, rows, c, alpha, n_iter, use_hist, fast_math);
  return check_launch("entmax_fwd_stream");
}

template <typename T, int TPR, int NV>
int launch_bwd_cfg(const T* y, const T* dy, T* dx, long long rows, int cols, float alpha,
                   int fast_math, bool vec, cudaStream_t st) {
  const int threads = TPR > 128 ? TPR : 128;
  const int rpc = threads / TPR;
  unsigned grid = (unsigned)((rows + rpc - 1) / rpc);
  if (vec)
    entmax_bwd_reg_kernel<T, TPR, NV, true><<<grid, threads, 0, st>>>(y, dy, dx, rows, cols, alpha, fast_math);
  else
    entmax_bwd_reg_kernel<T, TPR, NV, false><<<grid, threads, 0, st>>>(y, dy, dx, rows, cols, alpha, fast_math);
  return check_launch("entmax_bwd");
}

template <typename T>
int launch_bwd(const void* yv, const void* dyv, void* dxv, long long rows, long long cols,
               float alpha, int fast_math, cudaStream_t st) {
  const T* y = (const T*)yv;
  const T* dy = (const T*)dyv;
  T* dx = (T*)dxv;
  const size_t vb = 4 * sizeof(T);
  bool vec = (cols % 4 == 0) && ((uintptr_t)y % vb == 0) && ((uintptr_t)dy % vb == 0) && ((uintptr_t)dx % vb == 0);
  int c = (int)cols;
#define ADS_BWD(TPR, NV) return launch_bwd_cfg<T, TPR, NV>(y, dy, dx, rows, c, alpha, fast_math, vec, st)
  if (cols <= 128) ADS_BWD(32, 1);
  if (cols <= 512) ADS_BWD(32, 4);
  if (cols <= 1024) ADS_BWD(64, 4);
  if (cols <= 2048) ADS_BWD(128, 4);
  if (cols <= 4096) ADS_BWD(256, 4);
  if (cols <= 8192) ADS_BWD(512, 4);
  if (cols <= 16384) ADS_BWD(1024, 4);
#undef ADS_BWD
  entmax_bwd_stream_kernel<T><<<(unsigned)rows, 1024, 0, st>>>(y, dy, dx, rows, c, alpha, fast_math);
  return check_launch("entmax_bwd_stream");
}

}  // namespace
}  // namespace ads

extern "C" int adasplash_entmax_fwd(const void* x, void* y, float* tau_out, int64_t rows,
                                    int64_t cols, float alpha, int32_t n_iter,
                                    int32_t use_histogram, int32_t fast_math, int32_t dtype,
                                    void* stream) {
  using namespace ads;
  if (rows < 0 || cols < 0 || !(alpha > 1.0f) || n_iter < 0) {
    set_error("entmax_fwd: bad argument (rows=%lld cols=%lld alpha=%f n_iter=%d)", (long long)rows,
              (long long)cols, alpha, n_iter);
    return ADS_ERR_BAD_ARG;
  }
  if (rows == 0 || cols == 0) return ADS_OK;
  if (x == nullptr || y == nullptr) { set_error("entmax_fwd: null pointer"); return ADS_ERR_BAD_ARG; }
  if (cols > 0x7fffffffLL || rows > 0x7fffffffLL) { set_error("entmax_fwd: size too large"); return ADS_ERR_UNSUPPORTED; }
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case ADS_F32: return launch_fwd<float>(x, y, tau_out, rows, cols, alpha, n_iter, use_histogram, fast_math, st);
    case ADS_F16: return launch_fwd<__half>(x, y, tau_out, rows, cols, alpha, n_iter, use_histogram, fast_math, st);
    case ADS_BF16: return launch_fwd<__nv_bfloat16>(x, y, tau_out, rows, cols, alpha, n_iter, use_histogram, fast_math, st);
  }
  set_error("entmax_fwd: unknown dtype %d", dtype);
  return ADS_ERR_BAD_ARG;
}

extern "C" int adasplash_entmax_bwd(const void* y, const void* dy, void* dx, int64_t rows,
                                    int64_t cols, float alpha, int32_t fast_math, int32_t dtype,
                                    void* stream) {
  using namespace ads;
  if (rows < 0 || cols < 0 || !(alpha > 1.0f)) { set_error("entmax_bwd: bad argument"); return ADS_ERR_BAD_ARG; }
  if (rows == 0 || cols == 0) return ADS_OK;
  if (y == nullptr || dy == nullptr || dx == nullptr) { set_error("entmax_bwd: null pointer"); return ADS_ERR_BAD_ARG; }
  if (cols > 0x7fffffffLL || rows > 0x7fffffffLL) { set_error("entmax_bwd: size too large"); return ADS_ERR_UNSUPPORTED; }
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case ADS_F32: return launch_bwd<float>(y, dy, dx, rows, cols, alpha, fast_math, st);
    case ADS_F16: return launch_bwd<__half>(y, dy, dx, rows, cols, alpha, fast_math, st);
    case ADS_BF16: return launch_bwd<__nv_bfloat16>(y, dy, dx, rows, cols, alpha, fast_math, st);
  }
  set_error("entmax_bwd: unknown dtype %d", dtype);
  return ADS_ERR_BAD_ARG;
}
