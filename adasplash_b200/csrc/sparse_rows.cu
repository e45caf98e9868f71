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

constexpr int kRowThreads = 256;

struct RowsParams {
  const void* v; void* out; void* out2;
  const void* varlen; int varlen_is_i64;
  int B, Hq, Hkv, N, Dg;
  sup::View sv;
};

// eight 16-bit elements <-> fp32
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = DT<T>::to_f(e[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = DT<T>::from_f(f[i]);
  return raw;
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
#pragma unroll 1
  for (int i = 0; i < 8; ++i) {
    const int rr = grp * 8 + i;  // this group's row inside the chunk
    const uint32_t first = __shfl_sync(0xffffffffu, rw.x, rr), cnt = __shfl_sync(0xffffffffu, rw.y, rr);
    const uint32_t cnt_max = __reduce_max_sync(0xffffffffu, cnt);
    float ao[CH * 8], ao2[CH * 8];
#pragma unroll
    for (int e = 0; e < CH * 8; ++e) { ao[e] = 0.f; ao2[e] = 0.f; }
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
          const float pw = round_to<T>(u[j] * u[j]), uw = round_to<T>(u[j]);
          supp += u[j];
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            float vf[8];
            unpack8<T>(raw[j][c], vf);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              ao[c * 8 + e] = fmaf(pw, vf[e], ao[c * 8 + e]);
              ao2[c * 8 + e] = fmaf(uw, vf[e], ao2[c * 8 + e]);
            }
          }
        }
      }
    }
    const float inv = supp > 0.f ? 1.0f / supp : 0.f;
#pragma unroll
    for (int e = 0; e < CH * 8; ++e) ao2[e] *= inv;
    if (lane_on && r0 + rr < p.N) {
      T* o = (T*)p.out + (row_base + r0 + rr) * p.Dg + gl * 8;
      T* o2 = (T*)p.out2 + (row_base + r0 + rr) * p.Dg + gl * 8;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        *reinterpret_cast<uint4*>(o + c * 64) = pack8<T>(ao + c * 8);
        *reinterpret_cast<uint4*>(o2 + c * 64) = pack8<T>(ao2 + c * 8);
      }
    }
  }
}

template <typename T>
int fwd_t(const simt::Params& p, cudaStream_t st) {
  RowsParams rp;
  rp.v = p.v; rp.out = p.out; rp.out2 = p.out2;
  rp.varlen = p.varlen; rp.varlen_is_i64 = p.varlen_is_i64;
  rp.B = p.B; rp.Hq = p.Hq; rp.Hkv = p.Hkv; rp.N = p.N; rp.Dg = p.D;
  rp.sv = sup::view(p.support, p.B, p.Hq, p.Hkv, p.N);
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
  float zscale;     // fp32(0.5 * sm_scale): z = zscale * q.k
  sup::View sv;
};

__device__ __forceinline__ float group_sum8(float x) {  // over the eight lanes of a row group
  x += __shfl_xor_sync(0xffffffffu, x, 4, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 2, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 1, 8);
  return x;
}

template <typename T>
__device__ __forceinline__ uint32_t bits16(float x) {
  const T t = DT<T>::from_f(x);
  return (uint32_t)*reinterpret_cast<const uint16_t*>(&t);
}

// The arithmetic of the tile kernels (adasplash_v2.py:943-1234), pair by pair:
//   dP = dO_i . V_j;  delta_i = out2_i . dO_i;
//   query side:  dS = rn(u (dP - delta)) with the solver's u;  dQ_i = sm_scale * sum_j dS K_j;
//   key side, which the reference computes from K~ = rn(k * 0.5/sqrt(D)) and the raw q:
//     u' = K~_j . q_i - tau_i;  P^T = rn(u'^2), dS^T = rn(u' (dP - delta)) where u' > 0.
// Same warp layout as the forward gather: 32 rows per warp, eight lanes per row.  The key-side
// values go to shared memory at the entry's slot, are sorted there by (key, row) once the 32
// rows are done, and leave as the chunk's run of `by_key`.
template <typename T, int CH>
__global__ void __launch_bounds__(kRowThreads) bwd_rows_kernel(BwdParams p) {
  extern __shared__ uint2 sort_buf[];  // [warps][kChunkCap]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, gl = lane & 7;
  const int chunks = (p.N + kRowsPerWarp - 1) / kRowsPerWarp;  // per head
  const long long wg = (long long)blockIdx.x * (kRowThreads / 32) + warp;
  if (wg >= (long long)p.B * p.Hq * chunks) return;
  const int bh = (int)(wg / chunks), chunk = (int)(wg % chunks), r0 = chunk * kRowsPerWarp;
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  if (p.sv.dense[b * p.Hkv + kvh] != 0) return;  // the tile kernels own this head
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const size_t row_base = (size_t)bh * p.N;
  const uint2 rw = (r0 + lane < len) ? p.sv.rows[row_base + r0 + lane] : make_uint2(0u, 0u);
  const uint32_t run0 = __shfl_sync(0xffffffffu, rw.x, 0);
  uint32_t total = rw.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  total = min(total, (uint32_t)sup::kChunkCap);  // the solver exports no denser chunk
  uint2* sb = sort_buf + warp * sup::kChunkCap;
  const size_t kv_base = (size_t)(b * p.Hkv + kvh) * p.N * p.Dg + gl * 8;
  const T* kb_ = (const T*)p.k + kv_base;
  const T* vb = (const T*)p.v + kv_base;
#pragma unroll 1
  for (int i = 0; i < 8; ++i) {
    const int rr = grp * 8 + i, row = r0 + rr;
    const uint32_t first = __shfl_sync(0xffffffffu, rw.x, rr), cnt = __shfl_sync(0xffffffffu, rw.y, rr);
    const uint32_t cnt_max = __reduce_max_sync(0xffffffffu, cnt);
    const bool row_ok = row < len;
    float qf[CH * 8], gf[CH * 8], dq[CH * 8];
    float delta = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      uint4 rq = make_uint4(0u, 0u, 0u, 0u), rg = rq, ro = rq;
      if (row_ok) {
        const size_t off = (row_base + row) * p.Dg + gl * 8 + c * 64;
        rq = *reinterpret_cast<const uint4*>((const T*)p.q + off);
        rg = *reinterpret_cast<const uint4*>((const T*)p.dout + off);
        ro = *reinterpret_cast<const uint4*>((const T*)p.out2 + off);
      }
      float q8[8], g8[8], o8[8];
      unpack8<T>(rq, q8); unpack8<T>(rg, g8); unpack8<T>(ro, o8);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        qf[c * 8 + e] = q8[e]; gf[c * 8 + e] = g8[e]; dq[c * 8 + e] = 0.f;
        delta = fmaf(o8[e], g8[e], delta);
      }
    }
    delta = group_sum8(delta);
    const float tau = row_ok ? p.taus[row_base + row] : 0.f;
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
          float kf[CH * 8];
          float dp = 0.f, zk = 0.f;
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            float v8[8], k8[8];
            unpack8<T>(rv[j][c], v8);
            unpack8<T>(rk[j][c], k8);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              kf[c * 8 + e] = k8[e];
              dp = fmaf(gf[c * 8 + e], v8[e], dp);
              zk = fmaf(qf[c * 8 + e], round_to<T>(k8[e] * p.zscale), zk);
            }
          }
          dp = group_sum8(dp);
          zk = group_sum8(zk);
          const float dd = dp - delta;
          const float dsq = round_to<T>(u[j] * dd);
#pragma unroll
          for (int e = 0; e < CH * 8; ++e) dq[e] = fmaf(dsq, kf[e], dq[e]);
          const float uk = zk - tau;
          if (gl == 0 && k0 + hb + j < cnt) {
            const uint32_t slot = first - run0 + k0 + hb + j;
            const uint32_t vals = uk > 0.f ? (bits16<T>(uk * uk) | (bits16<T>(uk * dd) << 16)) : 0u;
            if (slot < (uint32_t)sup::kChunkCap) sb[slot] = make_uint2((key[j] << 8) | (uint32_t)rr, vals);
          }
        }
      }
    }
    if (row < p.N) {
      T* o = (T*)p.dq + (row_base + row) * p.Dg + gl * 8;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        float s8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) s8[e] = dq[c * 8 + e] * p.sm_scale;
        *reinterpret_cast<uint4*>(o + c * 64) = pack8<T>(s8);
      }
    }
  }
  // sort the chunk's entries by (key, row): bitonic network over the next power of two
  uint32_t n2 = 32;
  while (n2 < total) n2 <<= 1;
  for (uint32_t t = total + lane; t < n2; t += 32) sb[t] = make_uint2(0xffffffffu, 0u);
  __syncwarp();
  for (uint32_t k = 2; k <= n2; k <<= 1) {
    for (uint32_t j = k >> 1; j > 0; j >>= 1) {
      for (uint32_t t = lane; t < n2; t += 32) {
        const uint32_t x = t ^ j;
        if (x > t) {
          const uint2 a = sb[t], c = sb[x];
          const bool up = (t & k) == 0;
          if (up ? a.x > c.x : a.x < c.x) { sb[t] = c; sb[x] = a; }
        }
      }
      __syncwarp();
    }
  }
  for (uint32_t t = lane; t < total; t += 32) p.sv.by_key[run0 + t] = sb[t];
  if (lane == 0) p.sv.chunks[(size_t)bh * chunks + chunk] = make_uint2(run0, total);
}

// ---------------------------------------------------------------------------
// Backward, by keys: dK, dV of 64 keys per CTA.
// ---------------------------------------------------------------------------
// Warp w owns keys 8w .. 8w+7 of the block; a lane holds D/32 elements of dK and of dV of each of
// the eight keys in registers.  For each query head of the group and each 32-row chunk from the
// diagonal on, a thread finds the chunk's entries of these 64 keys by binary search in the
// chunk's sorted run and copies them to shared memory at the offset a block-wide scan gives it --
// the order (head, chunk, key, row) is fixed; every warp then walks the staged entries, picks
// those of its keys and adds P^T dO_i and dS^T Q_i, the Q / dO rows of four entries in flight.
// No atomics: every sum has a fixed order.
constexpr int kKeyThreads = 256;
constexpr int kKeysPerCta = 64;
constexpr int kStage = 2048;  // entries staged per round

template <typename T, int EL> struct LaneVec;
template <typename T> struct LaneVec<T, 4> { using type = uint2; };
template <typename T> struct LaneVec<T, 2> { using type = uint32_t; };

template <typename T, int D>
__global__ void __launch_bounds__(kKeyThreads) bwd_keys_kernel(BwdParams p) {
  constexpr int EL = D / 32;  // elements per lane
  using LV = typename LaneVec<T, EL>::type;
  __shared__ uint2 s_ent[kStage];       // ((absolute row << 6) | key inside the block, P^T | dS^T << 16)
  __shared__ uint32_t s_wsum[kKeyThreads / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (p.N + kKeysPerCta - 1) / kKeysPerCta;
  const int bkv = blockIdx.x / nkb, kb = blockIdx.x % nkb;
  if (p.sv.dense[bkv] != 0) return;  // the tile kernels own this head
  const int b = bkv / p.Hkv, kvh = bkv % p.Hkv;
  const int G = p.Hq / p.Hkv;
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const int chunks = (p.N + sup::kChunkRows - 1) / sup::kChunkRows;
  const int chunks_used = (len + sup::kChunkRows - 1) / sup::kChunkRows;  // chunks with a valid row
  float ak[8][EL], av[8][EL];
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
#pragma unroll
    for (int e = 0; e < EL; ++e) { ak[kk][e] = 0.f; av[kk][e] = 0.f; }
  const uint32_t key0 = (uint32_t)(kb * kKeysPerCta);
  const uint32_t key_lo = key0 << 8, key_hi = (key0 + kKeysPerCta) << 8;
  auto to_f = [](uint32_t bits16v) -> float {
    if (std::is_same<T, __nv_bfloat16>::value) return __uint_as_float(bits16v << 16);
    const uint16_t hv = (uint16_t)bits16v;
    return __half2float(*reinterpret_cast<const __half*>(&hv));
  };
  for (int g = 0; g < G; ++g) {
    const int bh = b * p.Hq + kvh * G + g;
    const T* qh = (const T*)p.q + (size_t)bh * p.N * D + lane * EL;
    const T* gh = (const T*)p.dout + (size_t)bh * p.N * D + lane * EL;
    // causal: rows >= key, so the first chunk that can hold these keys is the one of key0
    for (int c0 = (int)key0 / sup::kChunkRows; c0 < chunks_used; c0 += kKeyThreads) {
      const int c = c0 + (int)threadIdx.x;
      uint32_t lo = 0, hi = 0;
      const uint2* run = p.sv.by_key;
      if (c < chunks_used) {
        const uint2 tab = p.sv.chunks[(size_t)bh * chunks + c];
        run += tab.x;
        // lower bounds of key_lo and key_hi in the sorted run
        uint32_t a = 0, z = tab.y;
        while (a < z) { const uint32_t m = (a + z) >> 1; if (run[m].x < key_lo) a = m + 1; else z = m; }
        lo = a; z = tab.y;
        while (a < z) { const uint32_t m = (a + z) >> 1; if (run[m].x < key_hi) a = m + 1; else z = m; }
        hi = a;
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
      __syncthreads();
      uint32_t off = incl - n_mine, total = 0;
#pragma unroll
      for (int w = 0; w < kKeyThreads / 32; ++w) {
        const uint32_t t = s_wsum[w];
        off += (w < warp) ? t : 0u;
        total += t;
      }
      for (uint32_t r0 = 0; r0 < total; r0 += kStage) {
        if (r0 > 0) __syncthreads();  // the previous round has been walked
        for (uint32_t e = 0; e < n_mine; ++e) {
          const uint32_t pos = off + e - r0;  // wraps for entries of earlier rounds
          if (pos < (uint32_t)kStage) {
            const uint2 ent = run[lo + e];
            const uint32_t row = (uint32_t)c * sup::kChunkRows + (ent.x & 31u);
            s_ent[pos] = make_uint2((row << 6) | ((ent.x >> 8) - key0), ent.y);
          }
        }
        __syncthreads();
        const uint32_t m = min((uint32_t)kStage, total - r0);
        for (uint32_t e0 = 0; e0 < m; e0 += 32) {
          const uint2 ent = (e0 + lane < m) ? s_ent[e0 + lane] : make_uint2(0u, 0u);
          // entries of this warp's eight keys with a non-zero weight
          uint32_t pick = __ballot_sync(0xffffffffu, ent.y != 0u && ((ent.x >> 3) & 7u) == (uint32_t)warp);
          while (pick) {
            LV rq[4], rg[4];
            uint32_t xs[4], ys[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // the rows of four entries in flight
              const int src = pick ? __ffs(pick) - 1 : 0;
              xs[j] = __shfl_sync(0xffffffffu, ent.x, src);
              ys[j] = pick ? __shfl_sync(0xffffffffu, ent.y, src) : 0u;
              if (!pick) ys[j] = 0u;
              pick &= pick - 1;
              const size_t roff = (size_t)(xs[j] >> 6) * D;
              rq[j] = LV(); rg[j] = LV();
              if (ys[j] != 0u) {
                rq[j] = *reinterpret_cast<const LV*>(qh + roff);
                rg[j] = *reinterpret_cast<const LV*>(gh + roff);
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (ys[j] == 0u) continue;  // the same for every lane
              const float pT = to_f(ys[j] & 0xffffu), dsT = to_f(ys[j] >> 16);
              float qv[EL], gv[EL];
              const T* eq = reinterpret_cast<const T*>(&rq[j]);
              const T* eg = reinterpret_cast<const T*>(&rg[j]);
#pragma unroll
              for (int x = 0; x < EL; ++x) { qv[x] = DT<T>::to_f(eq[x]); gv[x] = DT<T>::to_f(eg[x]); }
              const uint32_t kk = xs[j] & 7u;
#pragma unroll
              for (int t = 0; t < 8; ++t) {
                if (kk == (uint32_t)t) {
#pragma unroll
                  for (int x = 0; x < EL; ++x) { ak[t][x] = fmaf(dsT, qv[x], ak[t][x]); av[t][x] = fmaf(pT, gv[x], av[t][x]); }
                }
              }
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const int key = (int)key0 + warp * 8 + kk;
    if (key < p.N) {
      __align__(8) T outk[EL];
      __align__(8) T outv[EL];
#pragma unroll
      for (int x = 0; x < EL; ++x) { outk[x] = DT<T>::from_f(ak[kk][x] * p.sm_scale); outv[x] = DT<T>::from_f(av[kk][x]); }
      *reinterpret_cast<LV*>((T*)p.dk + ((size_t)bkv * p.N + key) * D + lane * EL) = *reinterpret_cast<const LV*>(outk);
      *reinterpret_cast<LV*>((T*)p.dv + ((size_t)bkv * p.N + key) * D + lane * EL) = *reinterpret_cast<const LV*>(outv);
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
  bp.sm_scale = p.sm_scale; bp.zscale = 0.5f * p.sm_scale;
  bp.sv = sup::view(p.support, p.B, p.Hq, p.Hkv, p.N);
  const long long warps = (long long)p.B * p.Hq * ((p.N + kRowsPerWarp - 1) / kRowsPerWarp);
  const unsigned grid = (unsigned)((warps + kRowThreads / 32 - 1) / (kRowThreads / 32));
  const size_t sm = (size_t)(kRowThreads / 32) * sup::kChunkCap * sizeof(uint2);
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
  rows_kernel<<<grid, kRowThreads, sm, st>>>(bp);
  if (int rc = check_launch("sparse::bwd_rows")) return rc;
  const unsigned kgrid = (unsigned)((long long)p.B * p.Hkv * ((p.N + kKeysPerCta - 1) / kKeysPerCta));
  if (p.D > 64) bwd_keys_kernel<T, 128><<<kgrid, kKeyThreads, 0, st>>>(bp);
  else bwd_keys_kernel<T, 64><<<kgrid, kKeyThreads, 0, st>>>(bp);
  return check_launch("sparse::bwd_keys");
}

}  // namespace

bool supported(const ads_attn_shape* s) {
  // 16-bit inputs on the tensor-core solver, causal alpha = 1.5, key indices that fit 16 bits
  if (s->dtype != ADS_F16 && s->dtype != ADS_BF16) return false;
  if (s->D != 64 && s->D != 128) return false;
  if (s->N > 65536) return false;
  if (!((s->alpha == 0.f || s->alpha == 1.5f) && s->non_causal == 0)) return false;
  return true;
}

size_t support_bytes(const ads_attn_shape* s) { return sup::bytes(s->B, s->Hq, s->Hkv, s->N); }

int clear_header(const simt::Params& p, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(p.support, 0, sup::header_bytes(p.B, p.Hkv), st);
  if (e != cudaSuccess) { set_error("support header memset: %s", cudaGetErrorString(e)); return ADS_ERR_CUDA; }
  return ADS_OK;
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
