// Gather kernels over the row supports exported by the tensor-core solver (support.cuh).
//
// A query row's output is sum_j p_ij V_j over the few keys j of its support, so one warp per row
// reads the row's (key, u) pairs and the V rows they name -- a few hundred bytes per pair, all
// from L2 -- instead of re-computing dense score tiles.  The arithmetic is the tile kernels':
// p = rn(u^2) and w = rn(u) in the input dtype, fp32 accumulation, out2 = (sum w V) / (sum u)
// (adasplash_v2.py:696-835).
#include "sparse_rows.cuh"

#include <mutex>
#include <type_traits>

#include "support.cuh"

namespace ads {
namespace sparse {
namespace {

constexpr int kRowThreads = 256;     // forward gather: eight warps of 32 rows
constexpr int kBwdRowThreads = 256;  // backward by rows: the eight warps of one 256-row block

struct RowsParams {
  const void* v; void* out; void* out2;
  const void* varlen; int varlen_is_i64;
  int B, Hq, Hkv, N, Dg;
  float alpha;   // 1.5 (AdaSplash-2 and first-generation calls), 2 or any value in (1, 2)
  sup::View sv;
};

// Two 16-bit elements <-> two fp32 values.  The accumulations below run on pairs: Blackwell's
// packed fp32 multiply-add (`__ffma2_rn`) does two lanes of fp32 per instruction, which halves
// the instruction count of these issue-bound kernels.
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t x);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t x) {
  return make_float2(__uint_as_float(x << 16), __uint_as_float(x & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t x) {
  return __half22float2(*reinterpret_cast<const __half2*>(&x));
}
template <typename T> __device__ __forceinline__ uint32_t pack2f(float2 v);
template <> __device__ __forceinline__ uint32_t pack2f<__nv_bfloat16>(float2 v) {
  const __nv_bfloat162 r = __float22bfloat162_rn(v);
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pack2f<__half>(float2 v) {
  const __half2 r = __float22half2_rn(v);
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float2 (&f)[4]) {
  f[0] = unpack2<T>(raw.x); f[1] = unpack2<T>(raw.y); f[2] = unpack2<T>(raw.z); f[3] = unpack2<T>(raw.w);
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float2* f) {
  return make_uint4(pack2f<T>(f[0]), pack2f<T>(f[1]), pack2f<T>(f[2]), pack2f<T>(f[3]));
}
__device__ __forceinline__ float2 splat(float x) { return make_float2(x, x); }

// The four row groups of a warp work in lockstep on one row each, as long as the longest of the
// four supports; so each group takes its eight rows in the order of their entry counts, and rows
// of similar length meet.  Returns this lane's row's rank inside its group (0 = most entries).
__device__ __forceinline__ int rank_in_group(uint32_t cnt, int lane) {
  int rank = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t cj = __shfl_sync(0xffffffffu, cnt, (lane & ~7) + j);
    rank += (cj > cnt || (cj == cnt && j < (lane & 7))) ? 1 : 0;
  }
  return rank;
}
// The row (0..31) of group `grp` whose rank is `i`.
__device__ __forceinline__ int row_of_rank(int my_rank, int i, int grp) {
  const uint32_t sel = __ballot_sync(0xffffffffu, my_rank == i);
  return grp * 8 + __ffs((sel >> (grp * 8)) & 0xffu) - 1;
}

// One warp per 32 consecutive query rows of a head, eight lanes per row: lane gl of a group owns
// the 16-byte chunks gl and (CH = 2, head dim 128) 8 + gl of the head dimension, so a V row is
// one or two coalesced 128-byte requests per group and every instruction of the accumulation
// serves four (row, key) pairs.  Group g takes rows 8g .. 8g+7 one after the other; the eight
// lanes fetch up to eight of the row's entries with one load and pass them round with shuffles.
constexpr int kRowsPerWarp = 32;

template <typename T, int CH>
__global__ void __launch_bounds__(kRowThreads) fwd_rows_kernel(RowsParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, gl = lane & 7;
  const int chunks = (p.N + kRowsPerWarp - 1) / kRowsPerWarp;  // per head
  const long long wg = (long long)blockIdx.x * (kRowThreads / 32) + warp;
  if (wg >= (long long)p.B * p.Hq * chunks) return;
  const int bh = (int)(wg / chunks), r0 = (int)(wg % chunks) * kRowsPerWarp;
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  if (p.sv.dense[b * p.Hkv + kvh] != 0) return;  // the tile kernels own this head
  const bool lane_on = gl * 8 < p.Dg;
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const size_t row_base = (size_t)bh * p.N;
  // rows at or beyond the sequence length have no entries (the solver wrote nothing for them)
  const uint2 rw = (r0 + lane < len) ? p.sv.rows[row_base + r0 + lane] : make_uint2(0u, 0u);
  const T* vb = (const T*)p.v + (size_t)(b * p.Hkv + kvh) * p.N * p.Dg + gl * 8;
  const simt::Powers powers(p.alpha);
  const int my_rank = rank_in_group(rw.y, lane);
#pragma unroll 1
  for (int i = 0; i < 8; ++i) {
    const int rr = row_of_rank(my_rank, i, grp);  // this group's row inside the chunk
    const uint32_t first = __shfl_sync(0xffffffffu, rw.x, rr), cnt = __shfl_sync(0xffffffffu, rw.y, rr);
    const uint32_t cnt_max = __reduce_max_sync(0xffffffffu, cnt);
    float2 ao[CH * 4], ao2[CH * 4];
#pragma unroll
    for (int e = 0; e < CH * 4; ++e) { ao[e] = splat(0.f); ao2[e] = splat(0.f); }
    float supp = 0.f;
    for (uint32_t k0 = 0; k0 < cnt_max; k0 += 8) {
      const uint2 ent = (k0 + gl < cnt) ? p.sv.entries[first + k0 + gl] : make_uint2(0u, 0u);
#pragma unroll
      for (int hb = 0; hb < 8; hb += 4) {
        if (k0 + hb >= cnt_max) break;
        uint4 raw[4][CH];
        float u[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // four entries of each group in flight
          const uint32_t key = __shfl_sync(0xffffffffu, ent.x, hb + j, 8);
          u[j] = __uint_as_float(__shfl_sync(0xffffffffu, ent.y, hb + j, 8));  // 0 beyond the row's entries
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            raw[j][c] = make_uint4(0u, 0u, 0u, 0u);
            if (k0 + hb + j < cnt && lane_on) raw[j][c] = *reinterpret_cast<const uint4*>(vb + (size_t)key * p.Dg + c * 64);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // p = u^(1/(alpha-1)) and the Jacobian weight g = u^(1/(alpha-1)-1): u^2 and u for alpha = 1.5
          const float uj = fmaxf(u[j], 0.f);  // alpha > 1.5: entries a rounding below tau are listed too
          const float gj = powers.g(uj);
          const float2 pw = splat(round_to<T>(powers.p(uj))), uw = splat(round_to<T>(gj));
          supp += gj;
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            float2 vf[4];
            unpack8<T>(raw[j][c], vf);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              ao[c * 4 + e] = __ffma2_rn(pw, vf[e], ao[c * 4 + e]);
              ao2[c * 4 + e] = __ffma2_rn(uw, vf[e], ao2[c * 4 + e]);
            }
          }
        }
      }
    }
    const float2 inv = splat(supp > 0.f ? 1.0f / supp : 0.f);
#pragma unroll
    for (int e = 0; e < CH * 4; ++e) ao2[e] = __fmul2_rn(ao2[e], inv);
    if (lane_on && r0 + rr < p.N) {
      T* o = (T*)p.out + (row_base + r0 + rr) * p.Dg + gl * 8;
      T* o2 = (T*)p.out2 + (row_base + r0 + rr) * p.Dg + gl * 8;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        *reinterpret_cast<uint4*>(o + c * 64) = pack8<T>(ao + c * 4);
        *reinterpret_cast<uint4*>(o2 + c * 64) = pack8<T>(ao2 + c * 4);
      }
    }
  }
}

// Largest squared norm of a key row per kv head (the solver's export needs it above alpha = 1.5
// to bound the difference between the two roundings of a score).  One warp per key row.
template <typename T>
__global__ void __launch_bounds__(256) key_norm_max_kernel(const T* __restrict__ k, float* __restrict__ kmax2,
                                                           const void* varlen, int is_i64, int B, int Hkv, int N, int D) {
  const long long row_g = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row_g >= (long long)B * Hkv * N) return;
  const int lane = threadIdx.x & 31;
  const int bkv = (int)(row_g / N), r = (int)(row_g % N);
  if (r >= load_len(varlen, is_i64, bkv / Hkv, N)) return;
  float s = 0.f;
  for (int d = lane; d < D; d += 32) { const float x = DT<T>::to_f(k[row_g * D + d]); s = fmaf(x, x, s); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) atomicMax(reinterpret_cast<int*>(kmax2) + bkv, __float_as_int(s));  // non-negative floats order as ints
}

template <typename T>
int key_norms_t(const simt::Params& p, cudaStream_t st) {
  const sup::View sv = sup::view(p.support, nullptr, p.B, p.Hq, p.Hkv, p.N);
  const long long rows = (long long)p.B * p.Hkv * p.N;
  key_norm_max_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const T*)p.k, sv.kmax2, p.varlen, p.varlen_is_i64,
                                                                   p.B, p.Hkv, p.N, p.D);
  return check_launch("sparse::key_norm_max");
}

template <typename T>
int fwd_t(const simt::Params& p, cudaStream_t st) {
  RowsParams rp;
  rp.v = p.v; rp.out = p.out; rp.out2 = p.out2;
  rp.varlen = p.varlen; rp.varlen_is_i64 = p.varlen_is_i64;
  rp.B = p.B; rp.Hq = p.Hq; rp.Hkv = p.Hkv; rp.N = p.N; rp.Dg = p.D;
  rp.alpha = p.alpha;
  rp.sv = sup::view(p.support, nullptr, p.B, p.Hq, p.Hkv, p.N);
  const long long warps = (long long)p.B * p.Hq * ((p.N + kRowsPerWarp - 1) / kRowsPerWarp);
  const unsigned grid = (unsigned)((warps + kRowThreads / 32 - 1) / (kRowThreads / 32));
  if (p.D > 64) fwd_rows_kernel<T, 2><<<grid, kRowThreads, 0, st>>>(rp);
  else fwd_rows_kernel<T, 1><<<grid, kRowThreads, 0, st>>>(rp);
  return check_launch("sparse::fwd_rows");
}

// ---------------------------------------------------------------------------
// Backward, by rows: dQ, and the entries re-ordered by key for the key kernel.
// ---------------------------------------------------------------------------
struct BwdParams {
  const void* q; const void* k; const void* v; const void* dout; const void* out2;
  const float* taus;
  void* dq; void* dk; void* dv;
  const void* varlen; int varlen_is_i64;
  int B, Hq, Hkv, N, Dg;
  float sm_scale;   // fp32(1/sqrt(D))
  float zscale;     // fp32((alpha-1) * sm_scale): z = zscale * q.k
  float alpha;
  int causal;       // 0 = full attention (first-generation semantics only)
  sup::View sv;
};

__device__ __forceinline__ float group_sum8(float x) {  // over the eight lanes of a row group
  x += __shfl_xor_sync(0xffffffffu, x, 4, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 2, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 1, 8);
  return x;
}

// The arithmetic of the tile kernels (adasplash_v2.py:943-1234), pair by pair:
//   dP = dO_i . V_j;  delta_i = out2_i . dO_i;
//   query side:  dS = rn(g(u) (dP - delta)) with the solver's u;  dQ_i = sm_scale * sum_j dS K_j;
//   key side, which the reference computes from K~ = rn(k * (alpha-1)/sqrt(D)) and the raw q:
//     u' = K~_j . q_i - tau_i;  P^T = rn(p(u')), dS^T = rn(g(u') (dP - delta)) where u' > 0;
//   p(u) = u^(1/(alpha-1)), g(u) = u^(1/(alpha-1) - 1): u^2 and u for alpha = 1.5.
// Same warp layout as the forward gather: 32 rows per warp, eight lanes per row; the eight warps
// of a CTA take the 256 rows of one solver CTA, whose entries form one contiguous run.  The
// key-side values go to shared memory at the entry's slot, are sorted there by (key, row) once
// the 256 rows are done, and leave as the block's run of `by_key`.
template <typename T, int CH>
__global__ void __launch_bounds__(kBwdRowThreads) bwd_rows_kernel(BwdParams p) {
  extern __shared__ uint2 sort_buf[];  // [kBlockCap]
  __shared__ uint32_t s_tot[kBwdRowThreads / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, gl = lane & 7;
  const int blocks = (p.N + sup::kBlockRows - 1) / sup::kBlockRows;  // per head
  const int bh = (int)(blockIdx.x / blocks), blk = (int)(blockIdx.x % blocks);
  const int r0 = blk * sup::kBlockRows + warp * kRowsPerWarp;  // this warp's first row
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  if (p.sv.dense[b * p.Hkv + kvh] != 0) return;  // the tile kernels own this head (the whole CTA leaves)
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const size_t row_base = (size_t)bh * p.N;
  const uint2 rw = (r0 + lane < len) ? p.sv.rows[row_base + r0 + lane] : make_uint2(0u, 0u);
  // the block's run starts at its first row's first entry
  const uint32_t run0 = (blk * sup::kBlockRows < len) ? p.sv.rows[row_base + blk * sup::kBlockRows].x : 0u;
  uint32_t wtot = rw.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wtot += __shfl_xor_sync(0xffffffffu, wtot, o);
  if (lane == 0) s_tot[warp] = wtot;
  uint2* sb = sort_buf;
  const size_t kv_base = (size_t)(b * p.Hkv + kvh) * p.N * p.Dg + gl * 8;
  const T* kb_ = (const T*)p.k + kv_base;
  const T* vb = (const T*)p.v + kv_base;
  const simt::Powers powers(p.alpha);
  // (taking the rows in the order of their entry counts, as the forward gather does, made this
  // kernel slower: 1.39 against 1.28 ms on the headline workload)
#pragma unroll 1
  for (int i = 0; i < 8; ++i) {
    const int rr = grp * 8 + i, row = r0 + rr;
    const uint32_t first = __shfl_sync(0xffffffffu, rw.x, rr), cnt = __shfl_sync(0xffffffffu, rw.y, rr);
    const uint32_t cnt_max = __reduce_max_sync(0xffffffffu, cnt);
    const bool row_ok = row < len;
    float2 qf[CH * 4], gf[CH * 4], dq[CH * 4];
    float2 dl2 = splat(0.f);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      uint4 rq = make_uint4(0u, 0u, 0u, 0u), rg = rq, ro = rq;
      if (row_ok) {
        const size_t off = (row_base + row) * p.Dg + gl * 8 + c * 64;
        rq = *reinterpret_cast<const uint4*>((const T*)p.q + off);
        rg = *reinterpret_cast<const uint4*>((const T*)p.dout + off);
        ro = *reinterpret_cast<const uint4*>((const T*)p.out2 + off);
      }
      float2 o8[4];
      unpack8<T>(rq, *reinterpret_cast<float2(*)[4]>(qf + c * 4));
      unpack8<T>(rg, *reinterpret_cast<float2(*)[4]>(gf + c * 4));
      unpack8<T>(ro, o8);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        dq[c * 4 + e] = splat(0.f);
        dl2 = __ffma2_rn(o8[e], gf[c * 4 + e], dl2);
      }
    }
    const float delta = group_sum8(dl2.x + dl2.y);
    const float tau = row_ok ? p.taus[row_base + row] : 0.f;
    const float2 zs2 = splat(p.zscale);
    for (uint32_t k0 = 0; k0 < cnt_max; k0 += 8) {
      const uint2 ent = (k0 + gl < cnt) ? p.sv.entries[first + k0 + gl] : make_uint2(0u, 0u);
#pragma unroll
      for (int hb = 0; hb < 8; hb += 2) {
        if (k0 + hb >= cnt_max) break;
        uint4 rk[2][CH], rv[2][CH];
        uint32_t key[2];
        float u[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          key[j] = __shfl_sync(0xffffffffu, ent.x, hb + j, 8);
          u[j] = __uint_as_float(__shfl_sync(0xffffffffu, ent.y, hb + j, 8));  // 0 beyond the row's entries
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            rk[j][c] = make_uint4(0u, 0u, 0u, 0u);
            rv[j][c] = make_uint4(0u, 0u, 0u, 0u);
            if (k0 + hb + j < cnt) {
              rk[j][c] = *reinterpret_cast<const uint4*>(kb_ + (size_t)key[j] * p.Dg + c * 64);
              rv[j][c] = *reinterpret_cast<const uint4*>(vb + (size_t)key[j] * p.Dg + c * 64);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float2 kf[CH * 4];
          float2 dp2 = splat(0.f), zk2 = splat(0.f);
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            float2 v8[4];
            unpack8<T>(rv[j][c], v8);
            unpack8<T>(rk[j][c], *reinterpret_cast<float2(*)[4]>(kf + c * 4));
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              dp2 = __ffma2_rn(gf[c * 4 + e], v8[e], dp2);
              // K~ = rn(k * fp32(0.5/sqrt(D))), two elements per conversion
              const float2 kt = unpack2<T>(pack2f<T>(__fmul2_rn(kf[c * 4 + e], zs2)));
              zk2 = __ffma2_rn(qf[c * 4 + e], kt, zk2);
            }
          }
          const float dp = group_sum8(dp2.x + dp2.y);
          const float zk = group_sum8(zk2.x + zk2.y);
          const float dd = dp - delta;
          const float2 dsq = splat(round_to<T>(powers.g(fmaxf(u[j], 0.f)) * dd));
#pragma unroll
          for (int e = 0; e < CH * 4; ++e) dq[e] = __ffma2_rn(dsq, kf[e], dq[e]);
          const float uk = zk - tau;
          if (gl == 0 && k0 + hb + j < cnt) {
            const uint32_t slot = first - run0 + k0 + hb + j;
            const uint32_t vals = uk > 0.f ? pack2f<T>(make_float2(powers.p(uk), powers.g(uk) * dd)) : 0u;
            if (slot < (uint32_t)sup::kBlockCap) sb[slot] = make_uint2((key[j] << 8) | (uint32_t)(warp * kRowsPerWarp + rr), vals);
          }
        }
      }
    }
    if (row < p.N) {
      T* o = (T*)p.dq + (row_base + row) * p.Dg + gl * 8;
      const float2 sc2 = splat(p.sm_scale);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        float2 s8[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) s8[e] = __fmul2_rn(dq[c * 4 + e], sc2);
        *reinterpret_cast<uint4*>(o + c * 64) = pack8<T>(s8);
      }
    }
  }
  // sort the block's entries by (key, row): bitonic network over the next power of two
  __syncthreads();
  uint32_t total = 0;
#pragma unroll
  for (int w = 0; w < kBwdRowThreads / 32; ++w) total += s_tot[w];
  total = min(total, (uint32_t)sup::kBlockCap);  // the solver exports no denser block
  uint32_t n2 = 64;
  while (n2 < total) n2 <<= 1;
  for (uint32_t t = total + threadIdx.x; t < n2; t += kBwdRowThreads) sb[t] = make_uint2(0xffffffffu, 0u);
  __syncthreads();
  for (uint32_t k = 2; k <= n2; k <<= 1) {
    for (uint32_t j = k >> 1; j > 0; j >>= 1) {
      for (uint32_t pi = threadIdx.x; pi < n2 / 2; pi += kBwdRowThreads) {  // the pi-th pair (t, t | j) of this stage
        const uint32_t t = ((pi & ~(j - 1)) << 1) | (pi & (j - 1)), x = t | j;
        const uint2 a = sb[t], c = sb[x];
        const bool up = (t & k) == 0;
        if (up ? a.x > c.x : a.x < c.x) { sb[t] = c; sb[x] = a; }
      }
      // With distances up to 32 a warp's pairs lie in 64-element windows that no other warp
      // touches, so stages at those distances only need the warp in step.
      const uint32_t jn = j > 1 ? (j >> 1) : k;  // the distance of the stage that follows
      if (j > 32 || jn > 32) __syncthreads(); else __syncwarp();
    }
  }
  __syncthreads();
  for (uint32_t t = threadIdx.x; t < total; t += kBwdRowThreads) p.sv.by_key[run0 + t] = sb[t];
  if (threadIdx.x == 0) p.sv.blocks[(size_t)bh * blocks + blk] = make_uint2(run0, total);
  // where each 32-key block starts in the sorted run: the key kernel reads its bounds from this
  // table instead of searching the run in global memory
  const int nkb1 = (p.N + sup::kTableKeys - 1) / sup::kTableKeys + 1;
  uint16_t* tab = p.sv.kb_off + ((size_t)bh * blocks + blk) * nkb1;
  for (int kbi = threadIdx.x; kbi < nkb1; kbi += kBwdRowThreads) {
    const uint32_t key = (uint32_t)(kbi * sup::kTableKeys) << 8;
    uint32_t a = 0, z = total;
    while (a < z) { const uint32_t m = (a + z) >> 1; if (sb[m].x < key) a = m + 1; else z = m; }
    tab[kbi] = (uint16_t)a;
  }
}

// ---------------------------------------------------------------------------
// Backward, by keys: dK, dV of 64 keys per CTA.
// ---------------------------------------------------------------------------
// Eight warps; warp w owns keys 4w .. 4w+3 of the CTA's 32, eight lanes per key, each lane D/8
// elements of that key's dK and dV in registers.  For each query head of the group and each
// 256-row block from the diagonal on, a thread reads where the block's entries of these 32 keys
// lie in the block's sorted run (the row kernel left a table); the warps copy those segments to
// shared memory at the offsets a
// block-wide scan gives them -- the order (head, row block, key, row) is fixed -- and the staged
// entries are regrouped by key with a stable counting sort.  The eight lanes of a key then run
// through the key's range four entries at a time (the Q / dO rows of all four requested before
// the first is used) and add P^T dO_i and dS^T Q_i.  No atomics: every sum has a fixed order.
constexpr int kKeyThreads = 256;
constexpr int kKeyWarps = kKeyThreads / 32;
constexpr int kKeysPerCta = sup::kTableKeys;  // 32: two CTAs fit an SM, and one's serial phases overlap the other's walk
constexpr int kStage = 1024;  // entries staged per round

template <typename T, int D>
__global__ void __launch_bounds__(kKeyThreads, 2) bwd_keys_kernel(BwdParams p) {
  constexpr int CH = D / 64;  // 16-byte loads per lane and row
  __shared__ uint2 s_ent[kStage];       // ((absolute row << 6) | key inside the block, P^T | dS^T << 16)
  __shared__ uint2 s_srt[kStage];       // the same, regrouped by key
  __shared__ uint32_t s_wsum[kKeyWarps];
  __shared__ uint32_t s_src[kKeyThreads], s_cnt[kKeyThreads], s_off[kKeyThreads];  // one segment per row block
  __shared__ uint32_t s_kcnt[kKeysPerCta], s_kpos[kKeysPerCta + 1];
  __shared__ uint16_t s_ccnt[(kStage / 32) * kKeysPerCta];  // [chunk of 32 staged entries][key]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, gl = lane & 7;
  const int nkb = (p.N + kKeysPerCta - 1) / kKeysPerCta;
  const int bkv = blockIdx.x / nkb, kb = blockIdx.x % nkb;
  if (p.sv.dense[bkv] != 0) return;  // the tile kernels own this head
  const int b = bkv / p.Hkv, kvh = bkv % p.Hkv;
  const int G = p.Hq / p.Hkv;
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const int blocks = (p.N + sup::kBlockRows - 1) / sup::kBlockRows;
  const int blocks_used = (len + sup::kBlockRows - 1) / sup::kBlockRows;  // row blocks with a valid row
  const int nkb1 = nkb + 1;
  float2 ak[CH * 4], av[CH * 4];
#pragma unroll
  for (int e = 0; e < CH * 4; ++e) { ak[e] = splat(0.f); av[e] = splat(0.f); }
  const uint32_t my_local = (uint32_t)(warp * 4 + grp);  // this lane's key inside the block
  const uint32_t key0 = (uint32_t)(kb * kKeysPerCta);
  auto to_f = [](uint32_t bits16v) -> float {
    if (std::is_same<T, __nv_bfloat16>::value) return __uint_as_float(bits16v << 16);
    const uint16_t hv = (uint16_t)bits16v;
    return __half2float(*reinterpret_cast<const __half*>(&hv));
  };
  for (int g = 0; g < G; ++g) {
    const int bh = b * p.Hq + kvh * G + g;
    // the eight lanes of a key read 128 contiguous bytes of a row per load
    const T* qh = (const T*)p.q + (size_t)bh * p.N * D + gl * 8;
    const T* gh = (const T*)p.dout + (size_t)bh * p.N * D + gl * 8;
    // causal: rows >= key, so the first row block that can hold these keys is the one of key0
    for (int c0 = p.causal ? (int)key0 / sup::kBlockRows : 0; c0 < blocks_used; c0 += kKeyThreads) {
      const int c = c0 + (int)threadIdx.x;
      uint32_t lo = 0, hi = 0, src0 = 0;
      if (c < blocks_used) {
        const size_t bi = (size_t)bh * blocks + c;
        const uint16_t* tab = p.sv.kb_off + bi * nkb1 + kb;
        lo = tab[0]; hi = tab[1];
        src0 = p.sv.blocks[bi].x + lo;
      }
      // block-wide exclusive scan of the counts: where each thread's entries go
      const uint32_t n_mine = hi - lo;
      uint32_t incl = n_mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      __syncthreads();  // the previous batch has been walked
      if (lane == 31) s_wsum[warp] = incl;
      s_src[threadIdx.x] = src0;
      s_cnt[threadIdx.x] = n_mine;
      __syncthreads();
      uint32_t off = incl - n_mine, total = 0;
#pragma unroll
      for (int w = 0; w < kKeyWarps; ++w) {
        const uint32_t t = s_wsum[w];
        off += (w < warp) ? t : 0u;
        total += t;
      }
      s_off[threadIdx.x] = off;
      const int n_here = min(kKeyThreads, blocks_used - c0);
      for (uint32_t r0 = 0; r0 < total; r0 += kStage) {
        __syncthreads();  // the segment table is written / the previous round has been walked
        // a warp copies a segment, 32 entries per trip (segments of the first row blocks are long:
        // their rows see few keys)
        for (int t = warp; t < n_here; t += kKeyWarps) {
          const uint32_t n = s_cnt[t], o = s_off[t];
          const uint2* src = p.sv.by_key + s_src[t];
          for (uint32_t e = lane; e < n; e += 32) {
            const uint32_t pos = o + e - r0;  // wraps for entries of earlier rounds
            if (pos < (uint32_t)kStage) {
              const uint2 ent = src[e];
              const uint32_t row = (uint32_t)(c0 + t) * sup::kBlockRows + (ent.x & 255u);
              s_ent[pos] = make_uint2((row << 6) | ((ent.x >> 8) - key0), ent.y);
            }
          }
        }
        __syncthreads();
        const uint32_t m = min((uint32_t)kStage, total - r0);
        // Regroup the staged entries by key, keeping their order inside a key (a stable counting
        // sort over the 64 keys; entries with zero weights drop out): each key's entries then
        // lie in one range of s_srt.  Per 32-entry chunk the lanes with the same key rank
        // themselves with a match; a thread per key turns the chunks' counts into offsets.
        const uint32_t n_chunks = (m + 31) >> 5;
        uint2 held[kStage / 32 / kKeyWarps];
        uint32_t ranks[kStage / 32 / kKeyWarps];
#pragma unroll
        for (int i = 0; i < kStage / 32 / kKeyWarps; ++i) {
          const uint32_t c = (uint32_t)(warp + i * kKeyWarps);
          held[i] = make_uint2(0u, 0u);
          ranks[i] = 0u;
          if (c < n_chunks) {
            const uint32_t e = c * 32 + lane;
            if (e < m) held[i] = s_ent[e];
            const bool live = held[i].y != 0u;
            const uint32_t ek = live ? (held[i].x & 63u) : (64u + (uint32_t)lane);  // dead lanes match nobody (keys are < 32)
            const uint32_t same = __match_any_sync(0xffffffffu, ek);
            ranks[i] = __popc(same & ((1u << lane) - 1u));
            s_ccnt[c * kKeysPerCta + lane] = 0;
            __syncwarp();
            if (live && ranks[i] == 0u) s_ccnt[c * kKeysPerCta + ek] = (uint16_t)__popc(same);
          }
        }
        __syncthreads();
        if (threadIdx.x < kKeysPerCta) {
          uint32_t running = 0;
          for (uint32_t c = 0; c < n_chunks; ++c) {
            const uint32_t t = s_ccnt[c * kKeysPerCta + threadIdx.x];
            s_ccnt[c * kKeysPerCta + threadIdx.x] = (uint16_t)running;
            running += t;
          }
          s_kcnt[threadIdx.x] = running;
        }
        __syncthreads();
        if (warp == 0) {
          static_assert(kKeysPerCta == 32, "one key counter per lane");
          const uint32_t cmine = s_kcnt[lane];
          uint32_t incl2 = cmine;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, incl2, o);
            if (lane >= o) incl2 += up;
          }
          s_kpos[lane] = incl2 - cmine;
          if (lane == 31) s_kpos[kKeysPerCta] = incl2;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kStage / 32 / kKeyWarps; ++i) {
          const uint32_t c = (uint32_t)(warp + i * kKeyWarps);
          if (c < n_chunks && held[i].y != 0u) {
            const uint32_t ek = held[i].x & 63u;
            s_srt[s_kpos[ek] + s_ccnt[c * kKeysPerCta + ek] + ranks[i]] = held[i];
          }
        }
        __syncthreads();
        uint32_t e = s_kpos[my_local];
        const uint32_t e_end = s_kpos[my_local + 1];
        while (__any_sync(0xffffffffu, e < e_end)) {
          uint4 rq[4][CH], rg[4][CH];
          uint32_t ys[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // the rows of four entries of each key in flight
            ys[j] = 0u;
            if (e + j < e_end) {
              const uint2 ent = s_srt[e + j];
              ys[j] = ent.y;
              const size_t roff = (size_t)(ent.x >> 6) * D;
#pragma unroll
              for (int c = 0; c < CH; ++c) {
                rq[j][c] = *reinterpret_cast<const uint4*>(qh + roff + c * 64);
                rg[j][c] = *reinterpret_cast<const uint4*>(gh + roff + c * 64);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (ys[j] != 0u) {   // staged entries all have non-zero weights
              const float2 pT = splat(to_f(ys[j] & 0xffffu)), dsT = splat(to_f(ys[j] >> 16));
#pragma unroll
              for (int c = 0; c < CH; ++c) {
                float2 q8[4], g8[4];
                unpack8<T>(rq[j][c], q8);
                unpack8<T>(rg[j][c], g8);
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                  ak[c * 4 + x] = __ffma2_rn(dsT, q8[x], ak[c * 4 + x]);
                  av[c * 4 + x] = __ffma2_rn(pT, g8[x], av[c * 4 + x]);
                }
              }
            }
          }
          e += 4;
        }
      }
    }
  }
  const int key = (int)key0 + (int)my_local;
  if (key < p.N) {
    T* dk = (T*)p.dk + ((size_t)bkv * p.N + key) * D + gl * 8;
    T* dv = (T*)p.dv + ((size_t)bkv * p.N + key) * D + gl * 8;
    const float2 sc2 = splat(p.sm_scale);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      float2 s8[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) s8[x] = __fmul2_rn(ak[c * 4 + x], sc2);
      *reinterpret_cast<uint4*>(dk + c * 64) = pack8<T>(s8);
      *reinterpret_cast<uint4*>(dv + c * 64) = pack8<T>(av + c * 4);
    }
  }
}

template <typename T>
int bwd_t(const simt::Params& p, cudaStream_t st) {
  BwdParams bp;
  bp.q = p.q; bp.k = p.k; bp.v = p.v; bp.dout = p.dout; bp.out2 = p.out2_in;
  bp.taus = p.taus; bp.dq = p.dq; bp.dk = p.dk; bp.dv = p.dv;
  bp.varlen = p.varlen; bp.varlen_is_i64 = p.varlen_is_i64;
  bp.B = p.B; bp.Hq = p.Hq; bp.Hkv = p.Hkv; bp.N = p.N; bp.Dg = p.D;
  bp.sm_scale = p.sm_scale; bp.zscale = p.zscale;
  bp.alpha = p.alpha; bp.causal = p.causal;
  bp.sv = sup::view(p.support, p.bwd_scratch, p.B, p.Hq, p.Hkv, p.N);
  static_assert(sup::kBlockRows == (kBwdRowThreads / 32) * kRowsPerWarp, "one CTA per row block");
  const unsigned grid = (unsigned)((long long)p.B * p.Hq * ((p.N + sup::kBlockRows - 1) / sup::kBlockRows));
  const size_t sm = (size_t)sup::kBlockCap * sizeof(uint2);
  auto rows_kernel = p.D > 64 ? bwd_rows_kernel<T, 2> : bwd_rows_kernel<T, 1>;
  {
    static std::mutex mu;
    static bool done[2][128] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 128 || !done[p.D > 64][dev]) {
      cudaError_t e = cudaFuncSetAttribute(rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
      if (e != cudaSuccess) { set_error("sparse::bwd_rows: cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return ADS_ERR_CUDA; }
      if (dev >= 0 && dev < 128) done[p.D > 64][dev] = true;
    }
  }
  rows_kernel<<<grid, kBwdRowThreads, sm, st>>>(bp);
  if (int rc = check_launch("sparse::bwd_rows")) return rc;
  const unsigned kgrid = (unsigned)((long long)p.B * p.Hkv * ((p.N + kKeysPerCta - 1) / kKeysPerCta));
  if (p.D > 64) bwd_keys_kernel<T, 128><<<kgrid, kKeyThreads, 0, st>>>(bp);
  else bwd_keys_kernel<T, 64><<<kgrid, kKeyThreads, 0, st>>>(bp);
  return check_launch("sparse::bwd_keys");
}

}  // namespace

bool supported(const ads_attn_shape* s) {
  // 16-bit inputs on the tensor-core solver, any alpha, causal or full attention, head dim 64 or
  // 128, key indices that fit 16 bits
  if (s->dtype != ADS_F16 && s->dtype != ADS_BF16) return false;
  if (s->D != 64 && s->D != 128) return false;
  if (s->N > 65536) return false;
  return true;
}

size_t support_bytes(const ads_attn_shape* s) { return sup::bytes(s->B, s->Hq, s->Hkv, s->N); }
size_t bwd_scratch_bytes(const ads_attn_shape* s) { return sup::scratch_bytes(s->B, s->Hq, s->Hkv, s->N); }

int clear_header(const simt::Params& p, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(p.support, 0, sup::header_bytes(p.B, p.Hkv), st);
  if (e != cudaSuccess) { set_error("support header memset: %s", cudaGetErrorString(e)); return ADS_ERR_CUDA; }
  return ADS_OK;
}

int key_norms(const simt::Params& p, int dtype, cudaStream_t st) {
  if (dtype == ADS_F16) return key_norms_t<__half>(p, st);
  return key_norms_t<__nv_bfloat16>(p, st);
}

int fwd(const simt::Params& p, int dtype, cudaStream_t st) {
  if (dtype == ADS_F16) return fwd_t<__half>(p, st);
  return fwd_t<__nv_bfloat16>(p, st);
}

int bwd(const simt::Params& p, int dtype, cudaStream_t st) {
  if (dtype == ADS_F16) return bwd_t<__half>(p, st);
  return bwd_t<__nv_bfloat16>(p, st);
}

}  // namespace sparse
}  // namespace ads
