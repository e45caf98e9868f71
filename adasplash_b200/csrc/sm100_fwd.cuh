// Sparse forward on the tensor cores (adasplash_v2.py:696-835).
//
// One CTA owns a 128-row query tile of one head and walks the 128-key tiles in
// which the block mask has at least one of its four 64x64 bits set.  Per tile:
//   S  = Q~ K^T            tcgen05.mma, operands in shared memory (TMA), fp32 in TMEM
//   u  = max(S - tau, 0)   one thread per row reads its TMEM lane
//   P  = rn(u*u), U = rn(u) written back over S in TMEM as 16-bit pairs
//   O += P V, O2 += U V    tcgen05.mma with the A operand in TMEM, V in shared memory
// S is double buffered so that the S product of tile j+1 overlaps the row work
// of tile j.  The row work of a tile is a chain of TMEM round trips, so sixteen
// row warps share it: two groups alternate on the tiles (group g owns S buffer g),
// and inside a group the warps w and w+4 own the same 32 TMEM lanes (rows) and
// split the 128 keys in halves.  That puts four warps on every scheduler to hide
// the TMEM and ALU latency.
// Sub-tiles whose bit is clear contribute exactly zero, as in the reference,
// which never visits them.
#pragma once
#include <type_traits>

#include "sm100_common.cuh"

namespace ads {
namespace sm100 {

constexpr int kFwdThreads = 640;  // 16 row warps (four per TMEM lane quarter) + TMA warp + three MMA warps
constexpr int kFwdRowThreads = 512;
constexpr int kFwdGroupThreads = 256;  // row threads that work on one tile
constexpr int kFwdKStages = 2;
constexpr int kFwdVStages = 3;
constexpr int kFwdTmemCols = 512;

template <int D>
struct FwdSmem {
  static constexpr int tile_bytes = (D / 64) * kPanelBytes;
  static constexpr int q_off = 0;
  static constexpr int k_off = tile_bytes;
  static constexpr int v_off = k_off + kFwdKStages * tile_bytes;
  static constexpr int bar_off = v_off + kFwdVStages * tile_bytes;
  static constexpr int n_bars = 2 + 2 * kFwdKStages + 2 * kFwdVStages + 6 + 1;
  static constexpr int misc_off = bar_off + n_bars * 8;
  static constexpr int supp_off = misc_off + 64;  // [4][128] floats: partial sums of u per (group, half)
  static constexpr size_t bytes = 1024 + supp_off + 4 * 128 * 4;
};

// Pack two fp32 values as 16-bit pairs (first value in the low half).
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Zero the rows [first_row, 128) of a swizzled 128-row tile (whole 128-byte rows,
// so the swizzle does not matter).  Called by one full warp.
__device__ __forceinline__ void zero_tile_rows(uint8_t* tile, int panels, int first_row, int lane) {
  if (first_row < 0) first_row = 0;
  const int nrows = 128 - first_row;
  for (int pn = 0; pn < panels; ++pn) {
    uint4* base = reinterpret_cast<uint4*>(tile + pn * kPanelBytes + first_row * 128);
    for (int v = lane; v < nrows * 8; v += 32) base[v] = make_uint4(0, 0, 0, 0);
  }
  ptx::fence_proxy_async_smem();
  __syncwarp();
}

// AM selects the row math: 0 = alpha 1.5 (p = u^2, weight u), 1 = alpha 2 (p = u, weight 1[u>0]),
// 2 = any alpha in (1, 2) through the lg2 / ex2 units (p = u^(1/(alpha-1)), weight p / u);
// CAUSAL = false is full attention (every key tile up to the sequence length, no diagonal mask).
// <0, true> is the AdaSplash-2 path; the others serve the first-generation semantics.
template <typename T, int D, int AM = 0, bool CAUSAL = true>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmV, TcParams p) {
  using L = FwdSmem<D>;
  constexpr int PANELS = D / 64;
  constexpr int KSTEPS = D / 16;
  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t O_COL = 256, O2_COL = 256 + D;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem + L::q_off;
  uint8_t* sK = smem + L::k_off;
  uint8_t* sV = smem + L::v_off;
  uint64_t* bars = (uint64_t*)(smem + L::bar_off);
  uint64_t* q_full = bars + 0;
  uint64_t* q_ready = bars + 1;
  uint64_t* k_full = bars + 2;
  uint64_t* k_empty = k_full + kFwdKStages;
  uint64_t* v_full = k_empty + kFwdKStages;
  uint64_t* v_empty = v_full + kFwdVStages;
  uint64_t* s_full = v_empty + kFwdVStages;
  uint64_t* p_full = s_full + 2;
  uint64_t* s_free = p_full + 2;
  uint64_t* o_full = s_free + 2;
  uint32_t* tmem_holder = (uint32_t*)(smem + L::misc_off);
  volatile int* cta_abort = (volatile int*)(smem + L::misc_off + 4);
  int* start_status = (int*)(smem + L::misc_off + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // head-major order: the CTAs in flight share a few heads, whose K / V stay in L2;
  // inside a head the longest (latest) query tiles start first
  const int qt = p.nq - 1 - (int)(blockIdx.x % p.nq);
  const int bh = blockIdx.x / p.nq;
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  // rows whose supports the solver exported are done by the gather kernels (support.cuh)
  if (p.sup_on && p.sup.dense[b * p.Hkv + kvh] == 0) return;
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const int m0 = qt * kBlockM;
  // Dg = head dim of the tensors in global memory (p.d_true).  It equals D except for head dims
  // 16 and 32, which run the D = 64 instantiation: TMA fills the missing columns of every tile
  // with zeros (they add nothing to any product) and only the first Dg columns are stored.
  const int Dg = p.d_true;
  T* og = (T*)p.out + (size_t)bh * p.N * Dg;
  T* o2g = (T*)p.out2 + (size_t)bh * p.N * Dg;
  if (m0 >= len) {
    // fully padded query tile: its output rows are zero
    for (int v = threadIdx.x; v < kBlockM * (Dg / 8); v += kFwdThreads) {
      const int rr = m0 + v / (Dg / 8);
      if (rr < p.N) {
        reinterpret_cast<uint4*>(og + (size_t)rr * Dg)[v % (Dg / 8)] = make_uint4(0, 0, 0, 0);
        reinterpret_cast<uint4*>(o2g + (size_t)rr * Dg)[v % (Dg / 8)] = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }
  const int T_tiles = CAUSAL ? qt + 1 : (len + kBlockN - 1) / kBlockN;

  if (threadIdx.x == 0) {
    *start_status = *(volatile int*)p.status;
    *cta_abort = 0;
  }
  const int32_t* bm_head = p.bmask + (size_t)bh * p.rows_padded * p.n_words;
  if (warp == 17) {
    if (lane == 0) {
      ptx::mbar_init(q_full, 1);
      ptx::mbar_init(q_ready, kFwdRowThreads / 32);
      for (int s = 0; s < kFwdKStages; ++s) { ptx::mbar_init(k_full + s, 1); ptx::mbar_init(k_empty + s, 1); }
      for (int s = 0; s < kFwdVStages; ++s) { ptx::mbar_init(v_full + s, 1); ptx::mbar_init(v_empty + s, 2); }
      for (int s = 0; s < 2; ++s) {
        ptx::mbar_init(s_full + s, 1);
        ptx::mbar_init(p_full + s, kFwdGroupThreads / 32);
        ptx::mbar_init(s_free + s, 2);
      }
      ptx::mbar_init(o_full, 2);
      ptx::fence_mbar_init();
    }
    __syncwarp();
    ptx::tmem_alloc(tmem_holder, kFwdTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (*start_status != 0) {
    if (warp == 17) ptx::tmem_dealloc(*tmem_holder, kFwdTmemCols);
    return;
  }
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 16) {
    // ---------------- TMA producer ----------------
    if (ptx::elect_one()) {
      ptx::prefetch_tmap(&tmQ);
      ptx::prefetch_tmap(&tmK);
      ptx::prefetch_tmap(&tmV);
      ptx::mbar_arrive_expect_tx(q_full, L::tile_bytes);
      for (int pn = 0; pn < PANELS; ++pn) ptx::tma_load_3d(sQ + pn * kPanelBytes, &tmQ, q_full, pn * 64, m0, bh);
      const int kv_head = b * p.Hkv + kvh;
      TileScan scan(bm_head, qt, T_tiles, p.rows_padded, p.n_words);
      int kt;
      uint32_t flags;
      for (int j = 0; !ptx::c_withhold_loads && scan.next(kt, flags); ++j) {
        const int ks = j % kFwdKStages, vs = j % kFwdVStages;
        if (*cta_abort) break;
        if (!ptx::mbar_wait(k_empty + ks, ((j / kFwdKStages) & 1) ^ 1)) { raise_abort(cta_abort, p.status, kStTimeoutProducer); break; }
        ptx::mbar_arrive_expect_tx(k_full + ks, L::tile_bytes);
        for (int pn = 0; pn < PANELS; ++pn)
          ptx::tma_load_3d(sK + ks * L::tile_bytes + pn * kPanelBytes, &tmK, k_full + ks, pn * 64, kt * kBlockN, kv_head);
        if (!ptx::mbar_wait(v_empty + vs, ((j / kFwdVStages) & 1) ^ 1)) { raise_abort(cta_abort, p.status, kStTimeoutProducer); break; }
        ptx::mbar_arrive_expect_tx(v_full + vs, L::tile_bytes);
        for (int pn = 0; pn < PANELS; ++pn)
          ptx::tma_load_3d(sV + vs * L::tile_bytes + pn * kPanelBytes, &tmV, v_full + vs, pn * 64, kt * kBlockN, kv_head);
      }
    }
  } else if (warp == 17) {
    // ---------------- S issuer (whole warp stays converged; lane 0 issues) ----------------
    // The tensor pipe only runs what has been issued, and an issuing thread that waits on a
    // barrier or commits leaves it idle.  The S products and the P.V products therefore come
    // from two warps: while one is between tiles the other keeps the pipe busy.
    constexpr uint32_t idesc_s = ptx::make_idesc(FMT, kBlockM, kBlockN, 0, 0);
    bool ok = true;
    if (lane == 0) ok = ptx::mbar_wait(q_ready, 0);
    ok = __all_sync(0xffffffffu, ok);
    TileScan scan(bm_head, qt, T_tiles, p.rows_padded, p.n_words);
    int kt;
    uint32_t flags;
    for (int j = 0; ok && scan.next(kt, flags); ++j) {
      const int ks = j % kFwdKStages, buf = j & 1;
      if (*cta_abort) { ok = false; break; }
      if (ptx::elect_one()) {
        ok = ptx::mbar_wait(k_full + ks, (j / kFwdKStages) & 1) && ptx::mbar_wait(s_free + buf, ((j >> 1) & 1) ^ 1);
        if (ok) {
          ptx::tc_fence_after_sync();
          const uint32_t a0 = ptx::smem_u32(sQ), b0 = ptx::smem_u32(sK + ks * L::tile_bytes);
          const uint32_t d = tmem_base + buf * kBlockN;
#pragma unroll
          for (int kk = 0; kk < KSTEPS; ++kk) {
            const uint32_t off = (kk >> 2) * kPanelBytes + (kk & 3) * 32;
            ptx::mma_ss(d, ptx::make_smem_desc(a0 + off, 16, 1024), ptx::make_smem_desc(b0 + off, 16, 1024),
                        idesc_s, kk > 0);
          }
          ptx::mma_commit(k_empty + ks);
          ptx::mma_commit(s_full + buf);
        }
      }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok && lane == 0 && !*cta_abort) raise_abort(cta_abort, p.status, kStTimeoutMma);
  } else if (warp == 18 || warp == 19) {
    // ---------------- P.V issuer (warp 18: O += P V) and U.V issuer (warp 19: O2 += U V) ----------------
    constexpr uint32_t idesc_pv = ptx::make_idesc(FMT, kBlockM, D, 0, 1);
    const uint32_t acc = tmem_base + (warp == 18 ? O_COL : O2_COL);
    const uint32_t a_shift = warp == 18 ? 0u : 16u;  // U sits 16 columns after P in every 32-column chunk
    bool ok = true;
    TileScan scan(bm_head, qt, T_tiles, p.rows_padded, p.n_words);
    int kt, kt_next = 0;
    uint32_t flags;
    bool have = scan.next(kt, flags);
    for (int j = 0; ok && have; ++j) {
      const int vs = j % kFwdVStages, buf = j & 1;
      const bool have_next = scan.next(kt_next, flags);
      if (*cta_abort) { ok = false; break; }
      if (lane == 0) ok = ptx::mbar_wait(v_full + vs, (j / kFwdVStages) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      uint8_t* vt = sV + vs * L::tile_bytes;
      // padded keys: V = 0 (both issuers write the same zeros before their own products)
      if ((kt + 1) * kBlockN > len) zero_tile_rows(vt, PANELS, len - kt * kBlockN, lane);
      if (ptx::elect_one()) {
        ok = ptx::mbar_wait(p_full + buf, (j >> 1) & 1);
        if (ok) {
          ptx::tc_fence_after_sync();
          const uint32_t v0 = ptx::smem_u32(vt);
          const uint32_t pbase = tmem_base + buf * kBlockN + a_shift;
#pragma unroll
          for (int kk = 0; kk < kBlockN / 16; ++kk) {
            const uint64_t bd = ptx::make_smem_desc(v0 + kk * 2048, kPanelBytes, 1024);
            ptx::mma_ts(acc, pbase + (kk >> 1) * 32 + (kk & 1) * 8, bd, idesc_pv, (j > 0 || kk > 0));
          }
          ptx::mma_commit(v_empty + vs);
          ptx::mma_commit(s_free + buf);
          if (!have_next) ptx::mma_commit(o_full);
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      kt = kt_next;
      have = have_next;
    }
    if (!ok && lane == 0 && !*cta_abort) raise_abort(cta_abort, p.status, kStTimeoutMma);
  } else {
    // ---------------- row warps: thread = (score row, key half) ----------------
    const int wq = warp & 3;            // TMEM lanes 32*wq .. 32*wq+31
    const int half = (warp >> 2) & 1;   // keys 64*half .. 64*half+63 of a tile
    const int group = warp >> 3;        // tiles j with (j & 1) == group, S buffer `group`
    const int r = wq * 32 + lane;
    const int row = m0 + r;
    const bool row_ok = row < len;
    const int rb = wq >> 1;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(wq * 32) << 16);
    float* s_supp = (float*)(smem + L::supp_off);
    bool dead = false;
    if (!ptx::mbar_wait_warp(q_full, 0)) { raise_abort(cta_abort, p.status, kStTimeoutEpilogue); dead = true; }
    if (!dead) {
      const float sc = (AM == 0 && CAUSAL) ? 0.5f * p.sm_scale : p.zscale;
      for (int v = threadIdx.x; v < L::tile_bytes / 16; v += kFwdRowThreads) {
        uint4* ptr = reinterpret_cast<uint4*>(sQ) + v;
        const int vrow = ((v * 16) % kPanelBytes) / 128;
        uint4 val = *ptr;
        T* e = reinterpret_cast<T*>(&val);
        const bool keep = (m0 + vrow) < len;
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] = DT<T>::from_f(keep ? DT<T>::to_f(e[j]) * sc : 0.f);
        *ptr = val;
      }
      ptx::fence_proxy_async_smem();
    }
    ptx::mbar_arrive_warp(q_ready);
    const float tau = row_ok ? p.taus[(size_t)bh * p.N + row] : 0.f;
    const simt::Powers powers(p.alpha);   // used by the generic-alpha instantiation only
    float supp = 0.f;
    TileScan scan(bm_head, qt, T_tiles, p.rows_padded, p.n_words);
    int kt, n_active = 0;
    uint32_t flags;
    for (int j = 0; !dead && scan.next(kt, flags); ++j) {
      const int buf = j & 1;
      n_active = j + 1;
      if (buf != group) continue;
      const bool sub_on = (flags >> (2 * rb + half)) & 1u;  // this thread's 64x64 sub-tile
      if (*cta_abort) { dead = true; break; }
      if (!ptx::mbar_wait_warp(s_full + buf, (j >> 1) & 1)) { raise_abort(cta_abort, p.status, kStTimeoutEpilogue); dead = true; break; }
      ptx::tc_fence_after_sync();
      const int n0 = kt * kBlockN;
      const bool need_mask = (CAUSAL && kt == qt) || (n0 + kBlockN > len);
      // score -> (rn(p), rn(weight)) of two neighbours, and the row's sum of weights
      auto emit = [&](float u0, float u1, uint32_t& pw, uint32_t& uw) {
        if constexpr (AM == 0) {
          supp += u0 + u1;
          pw = pack2<T>(u0 * u0, u1 * u1);
          uw = pack2<T>(u0, u1);
        } else if constexpr (AM == 1) {
          const float g0 = u0 > 0.f ? 1.f : 0.f, g1 = u1 > 0.f ? 1.f : 0.f;
          supp += g0 + g1;
          pw = pack2<T>(u0, u1);
          uw = pack2<T>(g0, g1);
        } else {
          const float g0 = powers.g(u0), g1 = powers.g(u1);
          supp += g0 + g1;
          pw = pack2<T>(powers.p(u0), powers.p(u1));
          uw = pack2<T>(g0, g1);
        }
      };
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int ch = 2 * half + cc;
        const uint32_t caddr = lane_addr + buf * kBlockN + ch * 32;
        uint32_t pk[16], uk[16];
        if (!sub_on) {
#pragma unroll
          for (int c = 0; c < 16; ++c) { pk[c] = 0u; uk[c] = 0u; }
        } else {
          uint32_t raw[32];
          ptx::tmem_ld32(caddr, raw);
          ptx::tmem_ld_wait();
          const float* v = reinterpret_cast<const float*>(raw);
          if (need_mask) {
            const int col0 = n0 + ch * 32;
            const int lim = (CAUSAL ? min(row, len - 1) : len - 1) - col0;  // columns c <= lim survive
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              float u0 = fmaxf(v[c] - tau, 0.f), u1 = fmaxf(v[c + 1] - tau, 0.f);
              if (c > lim) u0 = 0.f;
              if (c + 1 > lim) u1 = 0.f;
              emit(u0, u1, pk[c >> 1], uk[c >> 1]);
            }
          } else {
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              const float u0 = fmaxf(v[c] - tau, 0.f), u1 = fmaxf(v[c + 1] - tau, 0.f);
              emit(u0, u1, pk[c >> 1], uk[c >> 1]);
            }
          }
        }
        ptx::tmem_st16(caddr, pk);
        ptx::tmem_st16(caddr + 16, uk);
      }
      ptx::tmem_st_wait();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive_warp(p_full + buf);
    }
    // the four threads of a row add up their partial sums of u
    s_supp[(group * 2 + half) * 128 + r] = supp;
    ptx::bar_sync(1, kFwdRowThreads);
    supp = (s_supp[r] + s_supp[128 + r]) + (s_supp[256 + r] + s_supp[384 + r]);
    // epilogue: O, O2 -> global; the four threads of a row share the D/32 column chunks
    if (!dead && n_active > 0) {
      if (!ptx::mbar_wait_warp(o_full, 0)) { raise_abort(cta_abort, p.status, kStTimeoutEpilogue); dead = true; }
    }
    if (!dead) {  // TMEM loads are warp-collective: only the global stores are per-row
      ptx::tc_fence_after_sync();
      const float inv = (row_ok && supp > 0.f) ? 1.0f / supp : 0.f;
      const int ch = group * 2 + half;
      if (ch < D / 32) {
        uint32_t ro[32], ro2[32];
        if (n_active > 0) {
          ptx::tmem_ld32(lane_addr + O_COL + ch * 32, ro);
          ptx::tmem_ld32(lane_addr + O2_COL + ch * 32, ro2);
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) { ro[c] = 0u; ro2[c] = 0u; }
        }
        const float* fo = reinterpret_cast<const float*>(ro);
        const float* fo2 = reinterpret_cast<const float*>(ro2);
        uint32_t po[16], po2[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          po[c >> 1] = row_ok ? pack2<T>(fo[c], fo[c + 1]) : 0u;
          po2[c >> 1] = row_ok ? pack2<T>(fo2[c] * inv, fo2[c + 1] * inv) : 0u;
        }
        uint4* dst = reinterpret_cast<uint4*>(og + (size_t)row * Dg + ch * 32);
        uint4* dst2 = reinterpret_cast<uint4*>(o2g + (size_t)row * Dg + ch * 32);
        if (row < p.N) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            if (ch * 32 + q4 * 8 < Dg) {
              dst[q4] = make_uint4(po[q4 * 4], po[q4 * 4 + 1], po[q4 * 4 + 2], po[q4 * 4 + 3]);
              dst2[q4] = make_uint4(po2[q4 * 4], po2[q4 * 4 + 1], po2[q4 * 4 + 2], po2[q4 * 4 + 3]);
            }
          }
        }
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*cta_abort && threadIdx.x == 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 17) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kFwdTmemCols);
  }
}

}  // namespace sm100
}  // namespace ads
