// CUDA-core (fp32 FMA) kernels of the AdaSplash-2 attention path: any input
// dtype, any head dim in {16..256}, fp32 accumulation.  They serve fp32 inputs
// (tcgen05 has no fp32 MMA), head dims the tensor-core kernels do not cover,
// and as an on-device cross-check of the tensor-core kernels.
//
// Tiling: one CTA of 256 threads owns a 64x64 score tile; thread (ty,tx) of a
// 16x16 grid holds rows ty+16i and columns tx+16j (i,j < 4).  Operand tiles
// live in shared memory as fp32 with a row pitch of D+4 floats so that the
// float4 reads of the inner product are conflict-free.
#pragma once
#include "common.cuh"

namespace ads {
namespace simt {

constexpr int kThreads = 256;
constexpr int kPPitch = 65;  // pitch of the 64x64 P / dS staging tiles

template <int D> struct Cfg {
  static constexpr int pitch = D + 4;
  static constexpr int tile_floats = 64 * pitch;
  static constexpr int dcols = D / 16;  // output columns per thread
};

struct Idx {
  int ty, tx;
  __device__ Idx() : ty(threadIdx.x >> 4), tx(threadIdx.x & 15) {}
};

// Load rows [row0, row0+64) of a (N, D) matrix into an fp32 tile, multiplying
// by `scale` and optionally rounding to T (the reference's scaled operand).
// Rows >= limit are zero (masked loads, adasplash_v2.py:220-222).
template <typename T, int D, bool ROUND>
__device__ __forceinline__ void load_tile(float* s, const T* g, int row0, int limit, float scale) {
  constexpr int P = Cfg<D>::pitch;
  constexpr int VPR = D / 4;  // 4-element groups per row
  for (int idx = threadIdx.x; idx < 64 * VPR; idx += kThreads) {
    int r = idx / VPR, c4 = (idx % VPR) * 4;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + r < limit) {
      const T* p = g + (size_t)(row0 + r) * D + c4;
      float f[4];
      if constexpr (sizeof(T) == 4) {
        float4 q = *reinterpret_cast<const float4*>(p);
        f[0] = q.x; f[1] = q.y; f[2] = q.z; f[3] = q.w;
      } else {
        uint2 q = *reinterpret_cast<const uint2*>(p);
        const T* h = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) f[e] = DT<T>::to_f(h[e]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        f[e] *= scale;
        if constexpr (ROUND) f[e] = round_to<T>(f[e]);
      }
      o = make_float4(f[0], f[1], f[2], f[3]);
    }
    *reinterpret_cast<float4*>(s + r * P + c4) = o;
  }
}

// acc[i][j] = <A[ty+16i, :], B[tx+16j, :]>
template <int D>
__device__ __forceinline__ void tile_dot(const float* sA, const float* sB, const Idx& id,
                                         float acc[4][4]) {
  constexpr int P = Cfg<D>::pitch;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 4
  for (int d = 0; d < D; d += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(sA + (id.ty + 16 * i) * P + d);
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = *reinterpret_cast<const float4*>(sB + (id.tx + 16 * j) * P + d);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
        acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
        acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
        acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
      }
  }
}

// The masked score tile of adasplash_v2.py:93-119: keep z where col <= row and
// col < len, else -10000.
__device__ __forceinline__ void mask_scores(float acc[4][4], const Idx& id, int m0, int n0, int len,
                                            bool causal = true) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int row = m0 + id.ty + 16 * i;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int col = n0 + id.tx + 16 * j;
      bool ok = (!causal || col <= row) && (col < len);
      acc[i][j] = ok ? acc[i][j] : kMaskedScore;
    }
  }
}

__device__ __forceinline__ float row16_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float row16_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ int row16_sumi(int v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// out[i][c] += sum_j sP[(ty+16i)][j] * sV[j][tx+16c]   (P row-major 64x64, pitch 65)
template <int D>
__device__ __forceinline__ void tile_pv(const float* sP, const float* sV, const Idx& id,
                                        float (*out)[Cfg<D>::dcols]) {
  constexpr int P = Cfg<D>::pitch;
  constexpr int DC = Cfg<D>::dcols;
#pragma unroll 2
  for (int j = 0; j < 64; ++j) {
    float p[4], v[DC];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = sP[(id.ty + 16 * i) * kPPitch + j];
#pragma unroll
    for (int c = 0; c < DC; ++c) v[c] = sV[j * P + id.tx + 16 * c];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < DC; ++c) out[i][c] = fmaf(p[i], v[c], out[i][c]);
  }
}

// out[i][c] += sum_q sP[q][(ty+16i)] * sX[q][tx+16c]   (transposed use of the staging tile)
template <int D>
__device__ __forceinline__ void tile_ptx(const float* sP, const float* sX, const Idx& id,
                                         float (*out)[Cfg<D>::dcols]) {
  constexpr int P = Cfg<D>::pitch;
  constexpr int DC = Cfg<D>::dcols;
#pragma unroll 2
  for (int q = 0; q < 64; ++q) {
    float p[4], v[DC];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = sP[q * kPPitch + id.ty + 16 * i];
#pragma unroll
    for (int c = 0; c < DC; ++c) v[c] = sX[q * P + id.tx + 16 * c];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < DC; ++c) out[i][c] = fmaf(p[i], v[c], out[i][c]);
  }
}

// Powers of the clipped score u = [z - tau]_+ for a given alpha:
//   p  = u^(1/(alpha-1))            attention weight
//   g  = u^(1/(alpha-1) - 1)        = p^(2-alpha), the weight of the entmax Jacobian
// alpha = 1.5 (u*u, u) and alpha = 2 (u, 1[u>0]) are exact multiplications; other
// alphas go through the approximate lg2 / ex2 units on the support only.
struct Powers {
  float c0, c1;
  int mode;  // 0: alpha = 1.5, 1: alpha = 2, 2: generic
  __device__ __forceinline__ explicit Powers(float alpha) {
    mode = (alpha == 1.5f) ? 0 : (alpha == 2.0f ? 1 : 2);
    c0 = 1.0f / (alpha - 1.0f);
    c1 = c0 - 1.0f;
  }
  __device__ __forceinline__ float p(float u) const {
    if (mode == 0) return u * u;
    if (mode == 1) return u;
    return u > 0.f ? exp2f(c0 * __log2f(u)) : 0.f;
  }
  __device__ __forceinline__ float g(float u) const {
    if (mode == 0) return u;
    if (mode == 1) return u > 0.f ? 1.f : 0.f;
    return u > 0.f ? exp2f(c1 * __log2f(u)) : 0.f;
  }
};

struct Params {
  const void* q; const void* k; const void* v;
  const void* varlen; int varlen_is_i64;
  float* taus; int32_t* bmask;
  void* out; void* out2;
  const void* dout; const void* out2_in; float* delta; int32_t* bmask_t;
  void* dq; void* dk; void* dv;
  int B, Hq, Hkv, N, D, niter, bins;
  int nb, n_words, rows_padded;
  float sm_scale;   // fp32(1/sqrt(D))
  int tau_given;    // solve kernel: 1 = only build the bitmap from taus
  int bwd_stages;   // 0 = all kernels of the backward, else a mask of ADS_BWD_*
  float alpha;      // entmax alpha in (1, 2]
  int causal;       // 1 = causal mask
  float zscale;     // fp32((alpha-1) * sm_scale): scores are z = zscale * q.k
  void* support;    // row-support buffer of the tensor-core path (support.cuh), or null
  void* bwd_scratch;  // with it, in the backward: room for the entries sorted by key (workspace + 256)
};

// ---------------------------------------------------------------------------
// Solver: row max -> histogram lower bound -> Halley refinements -> bitmap.
// One launch performs all sweeps; the scaled Q tile stays in shared memory and
// the K tiles are re-streamed (they are L2 resident per head).
// ---------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) solve_kernel(Params p) {
  extern __shared__ __align__(16) float smem[];
  float* sQ = smem;
  float* sK = smem + Cfg<D>::tile_floats;
  const Idx id;
  const int m = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const int m0 = m * kTile;
  if (m0 >= len) return;
  const int kvh = h / (p.Hq / p.Hkv);
  const T* qg = (const T*)p.q + ((size_t)b * p.Hq + h) * (size_t)p.N * D;
  const T* kg = (const T*)p.k + ((size_t)b * p.Hkv + kvh) * (size_t)p.N * D;
  float* tg = p.taus + ((size_t)b * p.Hq + h) * (size_t)p.N;
  int32_t* bm = p.bmask + (((size_t)b * p.Hq + h) * p.rows_padded + m) * (size_t)p.n_words;
  const float sc = p.zscale;
  load_tile<T, D, true>(sQ, qg, m0, len, sc);
  const bool causal = p.causal != 0;
  const bool v2_path = causal && p.alpha == 1.5f;  // the reference's AdaSplash-2 trajectory
  const int up_to = causal ? min(m0 + kTile, len) : len;
  const int ntiles = (up_to + kTile - 1) / kTile;
  float acc[4][4];
  HalleyState st[4];

  auto sweep = [&](auto&& per_tile) {
    for (int n = 0; n < ntiles; ++n) {
      __syncthreads();
      load_tile<T, D, false>(sK, kg, n * kTile, len, 1.0f);
      __syncthreads();
      tile_dot<D>(sQ, sK, id, acc);
      mask_scores(acc, id, m0, n * kTile, len, causal);
      per_tile(n);
    }
  };

  if (!p.tau_given) {
    // sweep 1: row maximum (adasplash_v2.py:236-266)
    float mx[4] = {-1.0e3f, -1.0e3f, -1.0e3f, -1.0e3f};
    sweep([&](int) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mx[i] = fmaxf(mx[i], acc[i][j]);
    });
    float tau0[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) tau0[i] = row16_max(mx[i]) - 1.0f;
    if (!v2_path) {
      // generic alpha / non-causal (adasplash_block_mask.py:170-176): bracket
      // [max - 1, max - n^(1-alpha)], start at its midpoint
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = m0 + id.ty + 16 * i;
        const float n = 1.0f + (float)(causal ? row : len);
        st[i].lo = tau0[i];
        st[i].hi = tau0[i] + 1.0f - exp2f((1.0f - p.alpha) * log2f(n));
        st[i].t = 0.5f * (st[i].lo + st[i].hi);
      }
    } else {
    // sweep 2: histogram of z - tau0 on [0,1] (adasplash_v2.py:387-431), as
    // cumulative counts N_b = #{(z - tau0) * BINS >= b}
    int cnt[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 8; ++c) cnt[i][c] = 0;
    const float fb = (float)p.bins;
    sweep([&](int) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float pr = (acc[i][j] - tau0[i]) * fb;
#pragma unroll
          for (int c = 0; c < 8; ++c) cnt[i][c] += (pr >= (float)c) ? 1 : 0;
        }
    });
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int bins_cnt[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) cnt[i][c] = row16_sumi(cnt[i][c]);
      for (int c = 0; c < p.bins; ++c) bins_cnt[c] = cnt[i][c] - (c + 1 < p.bins ? cnt[i][c + 1] : 0);
      float t1 = hist_tau_alpha15<8>(bins_cnt, p.bins, tau0[i]);
      st[i].lo = t1;
      st[i].hi = t1 + 1.0f / fb;
      st[i].t = 0.5f * (st[i].lo + st[i].hi);
    }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int row = m0 + id.ty + 16 * i;
      st[i].t = row < len ? tg[row] : 0.f;
      st[i].lo = st[i].hi = st[i].t;
    }
  }
  // refinement sweeps; the last one also records the bitmap for the tau that
  // enters it (adasplash_v2.py:567-675)
  // Generic path: niter updates, then a bitmap-only sweep at the lower end of the
  // bracket (tau_lo <= tau*, so no tile of the support can be missed).
  const Powers pw(p.alpha);
  const int total = p.tau_given ? 1 : p.niter + 1;
  for (int it = 0; it < total; ++it) {
    const bool last = (it == total - 1);
    const bool bitmap_only = last && !v2_path && !p.tau_given;
    float a0[4] = {0, 0, 0, 0}, a1[4] = {0, 0, 0, 0}, a2[4] = {0, 0, 0, 0};
    uint32_t cur = 0u;  // bitmap word under construction (thread 0 only)
    sweep([&](int n) {
      int hit = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // rows at or beyond len carry q = 0 and never count as hits
        bool row_ok = (m0 + id.ty + 16 * i) < len;
#pragma unroll
        const float thr = bitmap_only ? st[i].lo : st[i].t;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          bool mk = acc[i][j] > thr;
          float u = mk ? (acc[i][j] - thr) : 0.f;
          if (pw.mode == 0) {
            a0[i] = fmaf(u, u, a0[i]);
            a1[i] += u;
            a2[i] += mk ? 1.f : 0.f;
          } else if (mk) {
            const float g = pw.g(u);
            a0[i] += pw.p(u);
            a1[i] += g;
            a2[i] += (pw.mode == 2) ? g / u : 0.f;
          }
          hit |= (mk && row_ok) ? 1 : 0;
        }
      }
      if (last) {
        int any = __syncthreads_or(hit);
        if (threadIdx.x == 0) {
          if (any) cur |= (1u << (n & 31));
          if ((n & 31) == 31 || n == ntiles - 1) {
            bm[n >> 5] = (int32_t)cur;
            cur = 0u;
          }
        }
      }
    });
    if (!p.tau_given && !bitmap_only) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float s0 = row16_sum(a0[i]), s1 = row16_sum(a1[i]), s2 = row16_sum(a2[i]);
        if (v2_path) halley_bisect_update(st[i], s0, s1, s2);
        else halley_bisect_update_generic(st[i], s0, s1, s2, pw.c0, pw.c1);
      }
    }
  }
  if (!p.tau_given && id.tx == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int row = m0 + id.ty + 16 * i;
      if (row < len) tg[row] = st[i].t;
    }
  }
}

// ---------------------------------------------------------------------------
// Sparse forward (adasplash_v2.py:696-835)
// ---------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) fwd_kernel(Params p) {
  extern __shared__ __align__(16) float smem[];
  constexpr int DC = Cfg<D>::dcols;
  float* sQ = smem;
  float* sKV = sQ + Cfg<D>::tile_floats;
  float* sP = sKV + Cfg<D>::tile_floats;
  float* sU = sP + 64 * kPPitch;
  const Idx id;
  const int m = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const int m0 = m * kTile;
  const size_t qoff = ((size_t)b * p.Hq + h) * (size_t)p.N * D;
  T* og = (T*)p.out + qoff;
  T* o2g = (T*)p.out2 + qoff;
  float o[4][DC], o2[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < DC; ++c) { o[i][c] = 0.f; o2[i][c] = 0.f; }
  float supp[4] = {0, 0, 0, 0};
  const Powers pw(p.alpha);
  if (m0 < len) {
    const int kvh = h / (p.Hq / p.Hkv);
    const T* qg = (const T*)p.q + qoff;
    const size_t kvoff = ((size_t)b * p.Hkv + kvh) * (size_t)p.N * D;
    const T* kg = (const T*)p.k + kvoff;
    const T* vg = (const T*)p.v + kvoff;
    const float* tg = p.taus + ((size_t)b * p.Hq + h) * (size_t)p.N;
    const int32_t* bm = p.bmask + (((size_t)b * p.Hq + h) * p.rows_padded + m) * (size_t)p.n_words;
    load_tile<T, D, true>(sQ, qg, m0, len, p.zscale);
    float t[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int row = m0 + id.ty + 16 * i;
      t[i] = row < len ? tg[row] : 0.f;
    }
    float acc[4][4];
    for (int w = 0; w < p.n_words; ++w) {
      uint32_t word = (uint32_t)bm[w];
      while (word) {
        int n = (w << 5) + __ffs(word) - 1;
        word &= word - 1;
        __syncthreads();
        load_tile<T, D, false>(sKV, kg, n * kTile, len, 1.0f);
        __syncthreads();
        tile_dot<D>(sQ, sKV, id, acc);
        mask_scores(acc, id, m0, n * kTile, len, p.causal != 0);
        __syncthreads();
        load_tile<T, D, false>(sKV, vg, n * kTile, len, 1.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float u = fmaxf(acc[i][j] - t[i], 0.f);
            const float gw = pw.g(u);
            supp[i] += gw;
            sP[(id.ty + 16 * i) * kPPitch + id.tx + 16 * j] = round_to<T>(pw.p(u));
            sU[(id.ty + 16 * i) * kPPitch + id.tx + 16 * j] = round_to<T>(gw);
          }
        __syncthreads();
        tile_pv<D>(sP, sKV, id, o);
        tile_pv<D>(sU, sKV, id, o2);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int row = m0 + id.ty + 16 * i;
    if (row >= p.N) continue;
    bool valid = row < len;
    float s = row16_sum(supp[i]);
    float inv = valid ? 1.0f / s : 0.f;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      int d = id.tx + 16 * c;
      og[(size_t)row * D + d] = DT<T>::from_f(valid ? o[i][c] : 0.f);
      o2g[(size_t)row * D + d] = DT<T>::from_f(valid ? o2[i][c] * inv : 0.f);
    }
  }
}

// ---------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------
// delta[row] = sum_d out2[row,d] * dO[row,d] in fp32 (adasplash_v2.py:838-898)
// HBM-bound: every lane moves 16 bytes per load, D*sizeof(T)/16 lanes share a row (D is a
// power of two >= 16, so that count is a power of two), and a warp keeps kDeltaUnroll groups
// of rows in flight.
constexpr int kDeltaUnroll = 4;
constexpr int kDeltaThreads = 256;

template <typename T>
__host__ __device__ constexpr int delta_rows_per_warp(int D) {
  const int vec = 16 / (int)sizeof(T);
  const int lpr = D / vec < 32 ? D / vec : 32;   // lanes per row
  return (32 / lpr) * kDeltaUnroll;
}

template <typename T>
__global__ void __launch_bounds__(kDeltaThreads)
bwd_delta_kernel(const T* __restrict__ o2, const T* __restrict__ dout, float* __restrict__ delta,
                 const void* varlen, int is_i64, int B, int H, int N, int D,
                 const int32_t* __restrict__ skip = nullptr, int Hkv = 1) {
  constexpr int VEC = 16 / (int)sizeof(T);
  const int chunks = D / VEC;                     // 16-byte chunks per row
  const int lpr = chunks < 32 ? chunks : 32;      // lanes per row
  const int rows_pass = 32 / lpr;                 // rows a warp covers per pass
  const int lane = threadIdx.x & 31;
  const int sub = lane / lpr, li = lane % lpr;
  const long long total = (long long)B * H * N;
  const long long warp_id = (long long)blockIdx.x * (kDeltaThreads / 32) + threadIdx.x / 32;
  const long long row0 = warp_id * (rows_pass * kDeltaUnroll);
  if (skip != nullptr && row0 < total) {
    // the warp's rows lie in one head or two neighbours: leave if the gather kernels own both
    const long long last = min(total, row0 + rows_pass * kDeltaUnroll) - 1;
    const long long h0 = row0 / N, h1 = last / N;
    const int G = H / Hkv;
    if (h1 - h0 <= 1 && skip[(h0 / H) * Hkv + (h0 % H) / G] == 0 && skip[(h1 / H) * Hkv + (h1 % H) / G] == 0) return;
  }
  float acc[kDeltaUnroll];
#pragma unroll
  for (int u = 0; u < kDeltaUnroll; ++u) {
    acc[u] = 0.f;
    const long long row = row0 + u * rows_pass + sub;
    if (row < total) {
      const int b = (int)(row / ((long long)H * N));
      const int r = (int)(row % N);
      // heads of a kv head whose counter is zero belong to the gather kernels (support.cuh)
      const bool mine = skip == nullptr || skip[b * Hkv + (int)((row / N) % H) / (H / Hkv)] != 0;
      if (mine && r < load_len(varlen, is_i64, b, N)) {
        const uint4* a = reinterpret_cast<const uint4*>(o2 + row * D);
        const uint4* g = reinterpret_cast<const uint4*>(dout + row * D);
        for (int c = li; c < chunks; c += lpr) {
          const uint4 va = a[c], vg = g[c];
          const T* ea = reinterpret_cast<const T*>(&va);
          const T* eg = reinterpret_cast<const T*>(&vg);
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc[u] = fmaf(DT<T>::to_f(ea[e]), DT<T>::to_f(eg[e]), acc[u]);
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kDeltaUnroll; ++u) {
    float s = acc[u];
    for (int o = lpr >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const long long row = row0 + u * rows_pass + sub;
    if (li == 0 && row < total) delta[row] = s;
  }
}

// out[n][w] bit j = in[32w+j][n/32] bit (n%32)   (adasplash_v2.py:901-940)
static __global__ void transpose_bitmap_kernel(const int32_t* __restrict__ in, int32_t* __restrict__ out,
                                        int heads, int rows_padded, int n_words,
                                        const int32_t* __restrict__ skip = nullptr, int Hq = 1, int Hkv = 1) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long per_head = (long long)rows_padded * n_words;
  if (idx >= per_head * heads) return;
  long long hd = idx / per_head;
  // heads of a kv head whose counter is zero belong to the gather kernels (support.cuh)
  if (skip != nullptr && skip[(hd / Hq) * Hkv + (hd % Hq) / (Hq / Hkv)] == 0) return;
  int rem = (int)(idx % per_head);
  int n = rem / n_words, w = rem % n_words;
  const uint32_t* src = (const uint32_t*)in + hd * per_head;
  uint32_t acc = 0;
  if (n < n_words * 32) {
    for (int j = 0; j < 32; ++j) {
      int r = 32 * w + j;
      if (r < rows_padded) acc |= ((src[(size_t)r * n_words + (n >> 5)] >> (n & 31)) & 1u) << j;
    }
  }
  out[idx] = (int32_t)acc;
}

// dQ (adasplash_v2.py:943-1079)
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) bwd_dq_kernel(Params p) {
  extern __shared__ __align__(16) float smem[];
  constexpr int DC = Cfg<D>::dcols;
  float* sQ = smem;
  float* sDO = sQ + Cfg<D>::tile_floats;
  float* sKV = sDO + Cfg<D>::tile_floats;
  float* sDS = sKV + Cfg<D>::tile_floats;
  const Idx id;
  const int m = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const int m0 = m * kTile;
  const size_t qoff = ((size_t)b * p.Hq + h) * (size_t)p.N * D;
  T* dqg = (T*)p.dq + qoff;
  float dq[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < DC; ++c) dq[i][c] = 0.f;
  const Powers pw(p.alpha);
  if (m0 < len) {
    const int kvh = h / (p.Hq / p.Hkv);
    const size_t kvoff = ((size_t)b * p.Hkv + kvh) * (size_t)p.N * D;
    const T* kg = (const T*)p.k + kvoff;
    const T* vg = (const T*)p.v + kvoff;
    const size_t toff = ((size_t)b * p.Hq + h) * (size_t)p.N;
    const int32_t* bm = p.bmask + (((size_t)b * p.Hq + h) * p.rows_padded + m) * (size_t)p.n_words;
    load_tile<T, D, true>(sQ, (const T*)p.q + qoff, m0, len, p.zscale);
    load_tile<T, D, false>(sDO, (const T*)p.dout + qoff, m0, len, 1.0f);
    float t[4], dl[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int row = m0 + id.ty + 16 * i;
      t[i] = row < len ? p.taus[toff + row] : 0.f;
      dl[i] = row < len ? p.delta[toff + row] : 0.f;
    }
    float dp[4][4], acc[4][4];
    for (int w = 0; w < p.n_words; ++w) {
      uint32_t word = (uint32_t)bm[w];
      while (word) {
        int n = (w << 5) + __ffs(word) - 1;
        word &= word - 1;
        __syncthreads();
        load_tile<T, D, false>(sKV, vg, n * kTile, len, 1.0f);
        __syncthreads();
        tile_dot<D>(sDO, sKV, id, dp);
        __syncthreads();
        load_tile<T, D, false>(sKV, kg, n * kTile, len, 1.0f);
        __syncthreads();
        tile_dot<D>(sQ, sKV, id, acc);
        mask_scores(acc, id, m0, n * kTile, len, p.causal != 0);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float gw = pw.g(fmaxf(acc[i][j] - t[i], 0.f));
            sDS[(id.ty + 16 * i) * kPPitch + id.tx + 16 * j] = round_to<T>(gw * (dp[i][j] - dl[i]));
          }
        __syncthreads();
        tile_pv<D>(sDS, sKV, id, dq);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int row = m0 + id.ty + 16 * i;
    if (row >= p.N) continue;
    bool valid = row < len;
#pragma unroll
    for (int c = 0; c < DC; ++c)
      dqg[(size_t)row * D + id.tx + 16 * c] = DT<T>::from_f(valid ? dq[i][c] * p.sm_scale : 0.f);
  }
}

// dK, dV (adasplash_v2.py:1082-1234): one CTA per (kv tile, kv head, batch);
// loops the q heads of the group and the q tiles whose bit is set in the
// transposed bitmap.  K is the scaled+rounded operand here, Q is raw.
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) bwd_dkv_kernel(Params p) {
  extern __shared__ __align__(16) float smem[];
  constexpr int DC = Cfg<D>::dcols;
  float* sK = smem;
  float* sV = sK + Cfg<D>::tile_floats;
  float* sX = sV + Cfg<D>::tile_floats;  // Q, then dO, then Q again
  float* sP = sX + Cfg<D>::tile_floats;
  const Idx id;
  const int n = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const int n0 = n * kTile;
  const int G = p.Hq / p.Hkv;
  const size_t kvoff = ((size_t)b * p.Hkv + kvh) * (size_t)p.N * D;
  float dk[4][DC], dv[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < DC; ++c) { dk[i][c] = 0.f; dv[i][c] = 0.f; }
  const Powers pw(p.alpha);
  if (n0 < len) {
    load_tile<T, D, true>(sK, (const T*)p.k + kvoff, n0, len, p.zscale);
    load_tile<T, D, false>(sV, (const T*)p.v + kvoff, n0, len, 1.0f);
    for (int g = 0; g < G; ++g) {
      const int h = kvh * G + g;
      const size_t qoff = ((size_t)b * p.Hq + h) * (size_t)p.N * D;
      const size_t toff = ((size_t)b * p.Hq + h) * (size_t)p.N;
      const T* qg = (const T*)p.q + qoff;
      const T* dog = (const T*)p.dout + qoff;
      const int32_t* bt = p.bmask_t + (((size_t)b * p.Hq + h) * p.rows_padded + n) * (size_t)p.n_words;
      for (int w = 0; w < p.n_words; ++w) {
        uint32_t word = (uint32_t)bt[w];
        while (word) {
          int m = (w << 5) + __ffs(word) - 1;
          word &= word - 1;
          const int m0 = m * kTile;
          float t[4], dl[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            int row = m0 + id.ty + 16 * i;
            t[i] = row < len ? p.taus[toff + row] : 0.f;
            dl[i] = row < len ? p.delta[toff + row] : 0.f;
          }
          float s[4][4], dp[4][4];
          __syncthreads();
          load_tile<T, D, false>(sX, qg, m0, len, 1.0f);
          __syncthreads();
          tile_dot<D>(sX, sK, id, s);   // s[i][j]: q row ty+16i, key tx+16j
          mask_scores(s, id, m0, n0, len, p.causal != 0);
          __syncthreads();
          load_tile<T, D, false>(sX, dog, m0, len, 1.0f);
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float u = fmaxf(s[i][j] - t[i], 0.f);
              s[i][j] = pw.g(u);
              sP[(id.ty + 16 * i) * kPPitch + id.tx + 16 * j] = round_to<T>(pw.p(u));
            }
          __syncthreads();
          tile_dot<D>(sX, sV, id, dp);  // dP = dO V^T
          tile_ptx<D>(sP, sX, id, dv);  // dV += P^T dO
          __syncthreads();
          load_tile<T, D, false>(sX, qg, m0, len, 1.0f);
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              sP[(id.ty + 16 * i) * kPPitch + id.tx + 16 * j] = round_to<T>(s[i][j] * (dp[i][j] - dl[i]));
          __syncthreads();
          tile_ptx<D>(sP, sX, id, dk);  // dK += dS^T Q
        }
      }
    }
  }
  T* dkg = (T*)p.dk + kvoff;
  T* dvg = (T*)p.dv + kvoff;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int row = n0 + id.ty + 16 * i;
    if (row >= p.N) continue;
    bool valid = row < len;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      dkg[(size_t)row * D + id.tx + 16 * c] = DT<T>::from_f(valid ? dk[i][c] * p.sm_scale : 0.f);
      dvg[(size_t)row * D + id.tx + 16 * c] = DT<T>::from_f(valid ? dv[i][c] : 0.f);
    }
  }
}

// host-side launchers, one translation unit per dtype
template <typename T> int launch_solve(const Params& p, cudaStream_t st);
template <typename T> int launch_fwd(const Params& p, cudaStream_t st);
template <typename T> int launch_bwd(const Params& p, cudaStream_t st);

}  // namespace simt
}  // namespace ads
