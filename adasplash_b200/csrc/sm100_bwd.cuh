// Backward on the tensor cores (adasplash_v2.py:943-1234).
//
// dQ kernel: one CTA per 128-row query tile, walking the active 128-key tiles.
//   S = Q~ K^T, dP = dO V^T (operands in shared memory), u = max(S - tau, 0),
//   dS = rn(u (dP - delta)) written over S in TMEM, dQ += dS K (A operand in TMEM,
//   K read MN-major from the same shared-memory tile).  S is double buffered; dP has one
//   buffer, which the row warps copy to registers and hand back before their row work.
//   Eight row warps (TMEM lane = score row, two threads per row), one TMA warp and
//   three MMA-issuing warps, one per product.
//
// dK/dV kernel: one CTA per 128-key tile of one kv head, walking the q heads of
//   the group and, per head, the 64-row query blocks whose bit is set in the
//   transposed block mask.  S^T = K~ Q^T, dP^T = V dO^T (128 keys x 64 queries),
//   P^T = rn(u^2) and dS^T = rn(u (dP - delta)) written over S^T in TMEM (the dP^T
//   buffer is handed back as soon as the row warps hold it in registers),
//   dV += P^T dO, dK += dS^T Q.  K is the scaled + rounded operand here and Q is
//   raw, as in the reference.  S^T / dP^T are double buffered.  Sixteen row warps
//   (TMEM lane = key row, four threads per row), one producer warp (TMA for the
//   blocks, plain loads for tau / delta) and four MMA-issuing warps, one per product.
//
// Why several issuing warps: the tensor pipe only runs what has been issued, and a
// thread that waits on a barrier or commits leaves it idle for the length of that
// round trip (~250-400 cycles per hop measured).  With one warp per product the gaps
// of one are filled by the products of the others.
#pragma once
#include <type_traits>

#include "sm100_fwd.cuh"

namespace ads {
namespace sm100 {

// ---------------------------------------------------------------------------
// dQ
// ---------------------------------------------------------------------------
constexpr int kDqThreads = 384;   // 8 row warps + TMA warp + three MMA warps
constexpr int kDqRowThreads = 256;
constexpr int kDqKStages = 3;
constexpr int kDqVStages = 2;
constexpr int kDqTmemCols = 512;

template <int D>
struct DqSmem {
  static constexpr int tile_bytes = (D / 64) * kPanelBytes;
  static constexpr int q_off = 0;
  static constexpr int do_off = tile_bytes;
  static constexpr int k_off = 2 * tile_bytes;
  static constexpr int v_off = k_off + kDqKStages * tile_bytes;
  static constexpr int bar_off = v_off + kDqVStages * tile_bytes;
  static constexpr int n_bars = 2 + 2 * kDqKStages + 2 * kDqVStages + 2 + 1 + 2 + 2 + 1 + 1;
  static constexpr int misc_off = bar_off + n_bars * 8;
  static constexpr size_t bytes = 1024 + misc_off + 64;
};

// AM / CAUSAL as in the forward kernel (sm100_fwd.cuh).
template <typename T, int D, int AM = 0, bool CAUSAL = true>
__global__ void __launch_bounds__(kDqThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
              const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
              TcParams p) {
  using L = DqSmem<D>;
  constexpr int PANELS = D / 64;
  constexpr int KSTEPS = D / 16;
  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t DP_COL = 256, DQ_COL = 384;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem + L::q_off;
  uint8_t* sDO = smem + L::do_off;
  uint8_t* sK = smem + L::k_off;
  uint8_t* sV = smem + L::v_off;
  uint64_t* bars = (uint64_t*)(smem + L::bar_off);
  uint64_t* q_full = bars + 0;
  uint64_t* q_ready = bars + 1;
  uint64_t* k_full = bars + 2;
  uint64_t* k_empty = k_full + kDqKStages;
  uint64_t* v_full = k_empty + kDqKStages;
  uint64_t* v_empty = v_full + kDqVStages;
  uint64_t* s_full = v_empty + kDqVStages;   // [2]
  uint64_t* dp_full = s_full + 2;            // [1]
  uint64_t* p_full = dp_full + 1;            // [2] dS written, dP consumed
  uint64_t* s_free = p_full + 2;             // [2]
  uint64_t* dq_full = s_free + 2;
  uint64_t* dp_free = dq_full + 1;           // the row warps hold dP in registers: the buffer may be rewritten
  uint32_t* tmem_holder = (uint32_t*)(smem + L::misc_off);
  volatile int* cta_abort = (volatile int*)(smem + L::misc_off + 4);
  int* start_status = (int*)(smem + L::misc_off + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // head-major order: the CTAs in flight share a few heads, whose K / V stay in L2
  const int qt = p.nq - 1 - (int)(blockIdx.x % p.nq);
  const int bh = blockIdx.x / p.nq;
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  if (p.sup_on && p.sup.dense[b * p.Hkv + kvh] == 0) return;  // the gather kernels own this head
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const int m0 = qt * kBlockM;
  const int Dg = p.d_true;  // head dim in global memory (16 / 32 run the D = 64 instantiation)
  T* dqg = (T*)p.dq + (size_t)bh * p.N * Dg;
  if (m0 >= len) {
    for (int v = threadIdx.x; v < kBlockM * (Dg / 8); v += kDqThreads) {
      const int rr = m0 + v / (Dg / 8);
      if (rr < p.N) reinterpret_cast<uint4*>(dqg + (size_t)rr * Dg)[v % (Dg / 8)] = make_uint4(0, 0, 0, 0);
    }
    return;
  }
  const int T_tiles = CAUSAL ? qt + 1 : (len + kBlockN - 1) / kBlockN;
  const int32_t* bm_head = p.bmask + (size_t)bh * p.rows_padded * p.n_words;

  if (threadIdx.x == 0) {
    *start_status = *(volatile int*)p.status;
    *cta_abort = 0;
  }
  if (warp == 9) {
    if (lane == 0) {
      ptx::mbar_init(q_full, 1);
      ptx::mbar_init(q_ready, kDqRowThreads / 32);
      for (int s = 0; s < kDqKStages; ++s) { ptx::mbar_init(k_full + s, 1); ptx::mbar_init(k_empty + s, 1); }
      for (int s = 0; s < kDqVStages; ++s) { ptx::mbar_init(v_full + s, 1); ptx::mbar_init(v_empty + s, 1); }
      for (int s = 0; s < 2; ++s) {
        ptx::mbar_init(s_full + s, 1);
        ptx::mbar_init(p_full + s, kDqRowThreads / 32);
        ptx::mbar_init(s_free + s, 1);
      }
      ptx::mbar_init(dp_full, 1);
      ptx::mbar_init(dq_full, 1);
      ptx::mbar_init(dp_free, kDqRowThreads / 32);
      ptx::fence_mbar_init();
    }
    __syncwarp();
    ptx::tmem_alloc(tmem_holder, kDqTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (*start_status != 0) {
    if (warp == 9) ptx::tmem_dealloc(*tmem_holder, kDqTmemCols);
    return;
  }
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 8) {
    if (lane == 0) {
      ptx::prefetch_tmap(&tmQ); ptx::prefetch_tmap(&tmDO); ptx::prefetch_tmap(&tmK); ptx::prefetch_tmap(&tmV);
      ptx::mbar_arrive_expect_tx(q_full, 2 * L::tile_bytes);
      for (int pn = 0; pn < PANELS; ++pn) {
        ptx::tma_load_3d(sQ + pn * kPanelBytes, &tmQ, q_full, pn * 64, m0, bh);
        ptx::tma_load_3d(sDO + pn * kPanelBytes, &tmDO, q_full, pn * 64, m0, bh);
      }
      const int kv_head = b * p.Hkv + kvh;
      TileScan scan(bm_head, qt, T_tiles, p.rows_padded, p.n_words);
      int kt;
      uint32_t flags;
      for (int j = 0; !ptx::c_withhold_loads && scan.next(kt, flags); ++j) {
        const int ks = j % kDqKStages, vs = j % kDqVStages;
        if (*cta_abort) break;
        if (!ptx::mbar_wait(k_empty + ks, ((j / kDqKStages) & 1) ^ 1)) { raise_abort(cta_abort, p.status, kStTimeoutProducer); break; }
        ptx::mbar_arrive_expect_tx(k_full + ks, L::tile_bytes);
        for (int pn = 0; pn < PANELS; ++pn)
          ptx::tma_load_3d(sK + ks * L::tile_bytes + pn * kPanelBytes, &tmK, k_full + ks, pn * 64, kt * kBlockN, kv_head);
        if (!ptx::mbar_wait(v_empty + vs, ((j / kDqVStages) & 1) ^ 1)) { raise_abort(cta_abort, p.status, kStTimeoutProducer); break; }
        ptx::mbar_arrive_expect_tx(v_full + vs, L::tile_bytes);
        for (int pn = 0; pn < PANELS; ++pn)
          ptx::tma_load_3d(sV + vs * L::tile_bytes + pn * kPanelBytes, &tmV, v_full + vs, pn * 64, kt * kBlockN, kv_head);
      }
    }
  } else if (warp == 9) {
    // ---------------- S issuer: S_j = Q~ K_j^T into S buffer j&1 ----------------
    // Three warps issue the three products of a tile, so that the waits and commits of one
    // overlap the MMAs of the others (an issuing thread that waits leaves the tensor pipe idle).
    constexpr uint32_t idesc_s = ptx::make_idesc(FMT, kBlockM, kBlockN, 0, 0);
    bool ok = true;
    if (lane == 0) ok = ptx::mbar_wait(q_ready, 0);
    ok = __all_sync(0xffffffffu, ok);
    TileScan scan(bm_head, qt, T_tiles, p.rows_padded, p.n_words);
    int kt;
    uint32_t flags;
    for (int j = 0; ok && scan.next(kt, flags); ++j) {
      const int ks = j % kDqKStages, buf = j & 1;
      if (*cta_abort) { ok = false; break; }
      if (lane == 0) {
        ok = ptx::mbar_wait(k_full + ks, (j / kDqKStages) & 1) && ptx::mbar_wait(s_free + buf, ((j >> 1) & 1) ^ 1);
        if (ok) {
          ptx::tc_fence_after_sync();
          const uint32_t a0 = ptx::smem_u32(sQ), b0 = ptx::smem_u32(sK + ks * L::tile_bytes);
#pragma unroll
          for (int kk = 0; kk < KSTEPS; ++kk) {
            const uint32_t off = (kk >> 2) * kPanelBytes + (kk & 3) * 32;
            ptx::mma_ss(tmem_base + buf * kBlockN, ptx::make_smem_desc(a0 + off, 16, 1024),
                        ptx::make_smem_desc(b0 + off, 16, 1024), idesc_s, kk > 0);
          }
          ptx::mma_commit(s_full + buf);
        }
      }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok && lane == 0 && !*cta_abort) raise_abort(cta_abort, p.status, kStTimeoutMma);
  } else if (warp == 10) {
    // ---------------- dP issuer: dP_j = dO V_j^T into the single dP buffer ----------------
    constexpr uint32_t idesc_s = ptx::make_idesc(FMT, kBlockM, kBlockN, 0, 0);
    bool ok = true;
    if (lane == 0) ok = ptx::mbar_wait(q_ready, 0);
    ok = __all_sync(0xffffffffu, ok);
    TileScan scan(bm_head, qt, T_tiles, p.rows_padded, p.n_words);
    int kt;
    uint32_t flags;
    for (int j = 0; ok && scan.next(kt, flags); ++j) {
      const int vs = j % kDqVStages;
      if (*cta_abort) { ok = false; break; }
      if (lane == 0) {
        ok = ptx::mbar_wait(v_full + vs, (j / kDqVStages) & 1);
        // the row warps have dP_{j-1} in registers (they say so before their row work)
        if (ok && j > 0) ok = ptx::mbar_wait(dp_free, (j - 1) & 1);
        if (ok) {
          ptx::tc_fence_after_sync();
          const uint32_t a0 = ptx::smem_u32(sDO), b0 = ptx::smem_u32(sV + vs * L::tile_bytes);
#pragma unroll
          for (int kk = 0; kk < KSTEPS; ++kk) {
            const uint32_t off = (kk >> 2) * kPanelBytes + (kk & 3) * 32;
            ptx::mma_ss(tmem_base + DP_COL, ptx::make_smem_desc(a0 + off, 16, 1024),
                        ptx::make_smem_desc(b0 + off, 16, 1024), idesc_s, kk > 0);
          }
          ptx::mma_commit(v_empty + vs);
          ptx::mma_commit(dp_full);
        }
      }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok && lane == 0 && !*cta_abort) raise_abort(cta_abort, p.status, kStTimeoutMma);
  } else if (warp == 11) {
    // ---------------- dQ issuer: dQ += dS_j K_j ----------------
    constexpr uint32_t idesc_dq = ptx::make_idesc(FMT, kBlockM, D, 0, 1);
    bool ok = true;
    TileScan scan(bm_head, qt, T_tiles, p.rows_padded, p.n_words);
    int kt, kt_next = 0;
    uint32_t flags;
    bool have = scan.next(kt, flags);
    for (int j = 0; ok && have; ++j) {
      const int ks = j % kDqKStages, buf = j & 1;
      const bool have_next = scan.next(kt_next, flags);
      if (*cta_abort) { ok = false; break; }
      uint8_t* ktile = sK + ks * L::tile_bytes;
      // padded keys: K rows = 0 for the dS K product (S_j, the other reader of this
      // tile, has completed: its commit precedes p_full in program order of the row warps)
      const bool fix_k = (kt + 1) * kBlockN > len;
      if (lane == 0) ok = ptx::mbar_wait(p_full + buf, (j >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (fix_k) zero_tile_rows(ktile, PANELS, len - kt * kBlockN, lane);
      if (lane == 0) {
        ptx::tc_fence_after_sync();
        const uint32_t k0 = ptx::smem_u32(ktile);
        const uint32_t pbase = tmem_base + buf * kBlockN;
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk) {
          const uint64_t bd = ptx::make_smem_desc(k0 + kk * 2048, kPanelBytes, 1024);
          ptx::mma_ts(tmem_base + DQ_COL, pbase + (kk >> 1) * 32 + (kk & 1) * 8, bd, idesc_dq, (j > 0 || kk > 0));
        }
        ptx::mma_commit(k_empty + ks);
        ptx::mma_commit(s_free + buf);
        if (!have_next) ptx::mma_commit(dq_full);
      }
      kt = kt_next;
      have = have_next;
    }
    if (!ok && lane == 0 && !*cta_abort) raise_abort(cta_abort, p.status, kStTimeoutMma);
  } else {
    const int wq = warp & 3;     // TMEM lanes 32*wq .. 32*wq+31
    const int half = warp >> 2;  // keys 64*half .. 64*half+63 of each tile
    const int r = wq * 32 + lane;
    const int row = m0 + r;
    const bool row_ok = row < len;
    const int rb = wq >> 1;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(wq * 32) << 16);
    bool dead = false;
    if (!ptx::mbar_wait_warp(q_full, 0)) { raise_abort(cta_abort, p.status, kStTimeoutEpilogue); dead = true; }
    if (!dead) {
      const float sc = (AM == 0 && CAUSAL) ? 0.5f * p.sm_scale : p.zscale;
      for (int v = threadIdx.x; v < L::tile_bytes / 16; v += kDqRowThreads) {
        uint4* ptr = reinterpret_cast<uint4*>(sQ) + v;
        const int vrow = ((v * 16) % kPanelBytes) / 128;
        uint4 val = *ptr;
        T* e = reinterpret_cast<T*>(&val);
        const bool keep = (m0 + vrow) < len;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) e[jj] = DT<T>::from_f(keep ? DT<T>::to_f(e[jj]) * sc : 0.f);
        *ptr = val;
      }
      ptx::fence_proxy_async_smem();
    }
    ptx::mbar_arrive_warp(q_ready);
    const float tau = row_ok ? p.taus[(size_t)bh * p.N + row] : 0.f;
    const float dl = row_ok ? p.delta[(size_t)bh * p.N + row] : 0.f;
    const simt::Powers powers(p.alpha);   // used by the generic-alpha instantiation only
    const bool rows_full = m0 + kBlockM <= len;
    TileScan scan(bm_head, qt, T_tiles, p.rows_padded, p.n_words);
    int kt, n_active = 0;
    uint32_t flags;
    for (int j = 0; !dead && scan.next(kt, flags); ++j) {
      const int buf = j & 1;
      n_active = j + 1;
      const bool sub_on = (flags >> (2 * rb + half)) & 1u;
      if (*cta_abort) { dead = true; break; }
      if (!ptx::mbar_wait_warp(s_full + buf, (j >> 1) & 1) || !ptx::mbar_wait_warp(dp_full, j & 1)) {
        raise_abort(cta_abort, p.status, kStTimeoutEpilogue);
        dead = true;
        break;
      }
      ptx::tc_fence_after_sync();
      const int n0 = kt * kBlockN;
      const bool need_mask = (CAUSAL && kt == qt) || (n0 + kBlockN > len);
      // This thread's 64 values of dP go to registers first and the single dP buffer is handed
      // back at once: dO V^T of the next tile runs during the row work of this one.
      uint32_t rp[64];
      if (sub_on) {
        ptx::tmem_ld32(lane_addr + DP_COL + half * 64, rp);
        ptx::tmem_ld32(lane_addr + DP_COL + half * 64 + 32, rp + 32);
        ptx::tmem_ld_wait();
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive_warp(dp_free);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int ch = 2 * half + cc;
        const uint32_t caddr = lane_addr + buf * kBlockN + ch * 32;
        uint32_t dk[16];
        if (!sub_on) {
#pragma unroll
          for (int c = 0; c < 16; ++c) dk[c] = 0u;
        } else {
          uint32_t rs[32];
          ptx::tmem_ld32(caddr, rs);
          ptx::tmem_ld_wait();
          const float* s = reinterpret_cast<const float*>(rs);
          const float* dp = reinterpret_cast<const float*>(rp + cc * 32);
          if (!need_mask && rows_full) {
            // every (row, key) pair of the tile is causal and inside the sequence
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              if constexpr (AM == 0) {
                const float u0 = fmaxf(s[c] - tau, 0.f), u1 = fmaxf(s[c + 1] - tau, 0.f);
                dk[c >> 1] = pack2<T>(u0 * (dp[c] - dl), u1 * (dp[c + 1] - dl));
              } else if constexpr (AM == 1) {  // alpha = 2: the Jacobian weight is 1 on the support
                dk[c >> 1] = pack2<T>(s[c] > tau ? dp[c] - dl : 0.f, s[c + 1] > tau ? dp[c + 1] - dl : 0.f);
              } else {  // any alpha: weight u^(1/(alpha-1) - 1)
                dk[c >> 1] = pack2<T>(powers.g(fmaxf(s[c] - tau, 0.f)) * (dp[c] - dl),
                                      powers.g(fmaxf(s[c + 1] - tau, 0.f)) * (dp[c + 1] - dl));
              }
            }
          } else {
            const int lim = need_mask ? ((CAUSAL ? min(row, len - 1) : len - 1) - (n0 + ch * 32)) : 64;  // columns c <= lim survive
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              const float u0 = s[c] - tau, u1 = s[c + 1] - tau;
              // select, not multiply: dP of a padded key or row may be anything
              const float w0 = AM == 0 ? u0 : (AM == 1 ? 1.f : powers.g(fmaxf(u0, 0.f)));
              const float w1 = AM == 0 ? u1 : (AM == 1 ? 1.f : powers.g(fmaxf(u1, 0.f)));
              const float d0 = (u0 > 0.f && c <= lim) ? w0 * (dp[c] - dl) : 0.f;
              const float d1 = (u1 > 0.f && c + 1 <= lim) ? w1 * (dp[c + 1] - dl) : 0.f;
              dk[c >> 1] = pack2<T>(d0, d1);
            }
          }
        }
        ptx::tmem_st16(caddr, dk);
      }
      ptx::tmem_st_wait();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive_warp(p_full + buf);
    }
    if (!dead && n_active > 0) {
      if (!ptx::mbar_wait_warp(dq_full, 0)) { raise_abort(cta_abort, p.status, kStTimeoutEpilogue); dead = true; }
    }
    if (!dead) {  // TMEM loads are warp-collective: only the global stores are per-row
      ptx::tc_fence_after_sync();
#pragma unroll 1
      for (int cc = 0; cc < D / 64; ++cc) {
        const int ch = half * (D / 64) + cc;
        uint32_t ro[32];
        if (n_active > 0) {
          ptx::tmem_ld32(lane_addr + DQ_COL + ch * 32, ro);
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) ro[c] = 0u;
        }
        const float* fo = reinterpret_cast<const float*>(ro);
        uint32_t po[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2)
          po[c >> 1] = row_ok ? pack2<T>(fo[c] * p.sm_scale, fo[c + 1] * p.sm_scale) : 0u;
        uint4* dst = reinterpret_cast<uint4*>(dqg + (size_t)row * Dg + ch * 32);
        if (row < p.N) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            if (ch * 32 + q4 * 8 < Dg) dst[q4] = make_uint4(po[q4 * 4], po[q4 * 4 + 1], po[q4 * 4 + 2], po[q4 * 4 + 3]);
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
  if (warp == 9) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kDqTmemCols);
  }
}

// ---------------------------------------------------------------------------
// dK, dV
// ---------------------------------------------------------------------------
constexpr int kDkvThreads = 672;    // 16 row warps (4 lane quarters x 4 column slices) + TMA warp + four MMA warps
constexpr int kDkvRowThreads = 512;
constexpr int kDkvStages = 3;       // (Q block, dO block) pairs in flight
constexpr int kDkvTmemCols = 512;
constexpr int kQBlock = 64;         // query rows per step (one block-mask row block)
constexpr int kQPanelBytes = kQBlock * 128;

template <int D>
struct DkvSmem {
  static constexpr int tile_bytes = (D / 64) * kPanelBytes;     // 128-key K / V tile
  static constexpr int qblk_bytes = (D / 64) * kQPanelBytes;    // 64-row Q / dO block
  static constexpr int k_off = 0;
  static constexpr int v_off = tile_bytes;
  static constexpr int q_off = 2 * tile_bytes;
  static constexpr int do_off = q_off + kDkvStages * qblk_bytes;
  static constexpr int bar_off = do_off + kDkvStages * qblk_bytes;
  static constexpr int n_bars = 2 + 2 * kDkvStages + 2 + 2 + 2 + 1 + 2;
  static constexpr int misc_off = bar_off + n_bars * 8;
  static constexpr int td_off = (misc_off + 64 + 15) & ~15;     // [stages][tau 64 | delta 64] floats, 16-byte aligned (read as float4)
  static constexpr size_t bytes = 1024 + td_off + kDkvStages * 128 * 4;
};

// Walks (q head of the group, 64-row query block) pairs whose bit is set in rows
// 2nt / 2nt+1 of the transposed block mask.  flags: bit0 = keys 0..63 of the
// tile, bit1 = keys 64..127.
template <bool CAUSAL = true>
struct QBlockScan {
  const int32_t* bmt;
  int G, h0, rows_padded, n_words, nt, n_qblocks;
  int g, m;
  const uint32_t* r0;
  const uint32_t* r1;
  uint32_t w0, w1;
  __device__ QBlockScan(const int32_t* bmask_t, int b, int Hq, int G_, int kvh, int nt_, int n_qblocks_,
                        int rows_padded_, int n_words_)
      : bmt(bmask_t), G(G_), rows_padded(rows_padded_), n_words(n_words_), nt(nt_), n_qblocks(n_qblocks_),
        g(-1), m(0), r0(nullptr), r1(nullptr), w0(0), w1(0) {
    h0 = b * Hq + kvh * G_;
    m = n_qblocks;  // forces a head switch on the first call
  }
  __device__ __forceinline__ bool next(int& g_out, int& m_out, uint32_t& flags) {
    for (;;) {
      if (m >= n_qblocks) {
        if (++g >= G) return false;
        r0 = reinterpret_cast<const uint32_t*>(bmt) + ((size_t)(h0 + g) * rows_padded + 2 * nt) * n_words;
        r1 = (2 * nt + 1) < rows_padded ? r0 + n_words : nullptr;
        m = CAUSAL ? 2 * nt : 0;  // causal: query blocks before the key tile never see it
        w0 = r0[m >> 5];
        w1 = r1 ? r1[m >> 5] : 0u;
      }
      while (m < n_qblocks) {
        if ((m & 31) == 0) { w0 = r0[m >> 5]; w1 = r1 ? r1[m >> 5] : 0u; }
        const uint32_t f = ((w0 >> (m & 31)) & 1u) | (((w1 >> (m & 31)) & 1u) << 1);
        const int cur = m++;
        if (f) { g_out = g; m_out = cur; flags = f; return true; }
      }
    }
  }
};

template <typename T, int D, int AM = 0, bool CAUSAL = true>
__global__ void __launch_bounds__(kDkvThreads, 1)
bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               const __grid_constant__ CUtensorMap tmQ64, const __grid_constant__ CUtensorMap tmDO64,
               TcParams p) {
  using L = DkvSmem<D>;
  constexpr int PANELS = D / 64;
  constexpr int KSTEPS = D / 16;
  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t DP_COL0 = 128, DK_COL = 256, DV_COL = 256 + D;  // S^T[2] at 0/64, dP^T[2] at 128/192
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem + L::k_off;
  uint8_t* sV = smem + L::v_off;
  uint8_t* sQ = smem + L::q_off;
  uint8_t* sDO = smem + L::do_off;
  uint64_t* bars = (uint64_t*)(smem + L::bar_off);
  uint64_t* kv_full = bars + 0;
  uint64_t* k_ready = bars + 1;
  uint64_t* x_full = bars + 2;               // [stages] Q block + dO block landed
  uint64_t* x_empty = x_full + kDkvStages;
  uint64_t* s_full = x_empty + kDkvStages;   // [2] S^T and dP^T of a step computed
  uint64_t* p_full = s_full + 2;             // [2] P^T and dS^T written
  uint64_t* s_free = p_full + 2;             // [2]
  uint64_t* acc_full = s_free + 2;
  uint64_t* dp_free = acc_full + 1;          // [2] the row warps hold dP^T in registers: the buffer may be rewritten
  uint32_t* tmem_holder = (uint32_t*)(smem + L::misc_off);
  volatile int* cta_abort = (volatile int*)(smem + L::misc_off + 4);
  int* start_status = (int*)(smem + L::misc_off + 8);
  float* s_td = (float*)(smem + L::td_off);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // head-major order; inside a head the low key tiles (most query blocks) start first
  const int nt = (int)(blockIdx.x % p.nq);
  const int bkv = blockIdx.x / p.nq;
  const int b = bkv / p.Hkv, kvh = bkv % p.Hkv;
  if (p.sup_on && p.sup.dense[bkv] == 0) return;  // the gather kernels own this head
  const int G = p.Hq / p.Hkv;
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const int n0 = nt * kBlockN;
  const int Dg = p.d_true;  // head dim in global memory (16 / 32 run the D = 64 instantiation)
  T* dkg = (T*)p.dk + (size_t)bkv * p.N * Dg;
  T* dvg = (T*)p.dv + (size_t)bkv * p.N * Dg;
  if (n0 >= len) {
    for (int v = threadIdx.x; v < kBlockN * (Dg / 8); v += kDkvThreads) {
      const int rr = n0 + v / (Dg / 8);
      if (rr < p.N) {
        reinterpret_cast<uint4*>(dkg + (size_t)rr * Dg)[v % (Dg / 8)] = make_uint4(0, 0, 0, 0);
        reinterpret_cast<uint4*>(dvg + (size_t)rr * Dg)[v % (Dg / 8)] = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }
  const int n_qblocks = (len + kQBlock - 1) / kQBlock;  // query blocks with at least one valid row

  if (threadIdx.x == 0) {
    *start_status = *(volatile int*)p.status;
    *cta_abort = 0;
  }
  if (warp == 17) {
    if (lane == 0) {
      ptx::mbar_init(kv_full, 1);
      ptx::mbar_init(k_ready, kDkvRowThreads / 32);
      for (int s = 0; s < kDkvStages; ++s) { ptx::mbar_init(x_full + s, 1); ptx::mbar_init(x_empty + s, 2); }
      for (int s = 0; s < 2; ++s) {
        ptx::mbar_init(s_full + s, 2);
        ptx::mbar_init(p_full + s, kDkvRowThreads / 32);
        ptx::mbar_init(s_free + s, 2);
        ptx::mbar_init(dp_free + s, kDkvRowThreads / 32);
      }
      ptx::mbar_init(acc_full, 2);
      ptx::fence_mbar_init();
    }
    __syncwarp();
    ptx::tmem_alloc(tmem_holder, kDkvTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (*start_status != 0) {
    if (warp == 17) ptx::tmem_dealloc(*tmem_holder, kDkvTmemCols);
    return;
  }
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 16) {
    // ---------------- producer: K / V tile, then per step the Q and dO blocks (TMA, lane 0) and
    // the tau / delta of the block's 64 query rows (plain loads by the 32 lanes, fetched one
    // step ahead into registers so that their latency is off the path) ----------------
    if (ptx::elect_one()) {
      ptx::prefetch_tmap(&tmK); ptx::prefetch_tmap(&tmV); ptx::prefetch_tmap(&tmQ64); ptx::prefetch_tmap(&tmDO64);
      ptx::mbar_arrive_expect_tx(kv_full, 2 * L::tile_bytes);
      for (int pn = 0; pn < PANELS; ++pn) {
        ptx::tma_load_3d(sK + pn * kPanelBytes, &tmK, kv_full, pn * 64, n0, bkv);
        ptx::tma_load_3d(sV + pn * kPanelBytes, &tmV, kv_full, pn * 64, n0, bkv);
      }
    }
    // lane l carries tau / delta of query rows 2l and 2l+1 of a block (0 beyond the sequence)
    auto fetch_td = [&](int g_, int m_, float (&r)[4]) {
      const size_t base = (size_t)(b * p.Hq + kvh * G + g_) * p.N;
      const int q0 = m_ * kQBlock + 2 * lane;
      r[0] = (q0 < len) ? p.taus[base + q0] : 0.f;
      r[1] = (q0 + 1 < len) ? p.taus[base + q0 + 1] : 0.f;
      r[2] = (q0 < len) ? p.delta[base + q0] : 0.f;
      r[3] = (q0 + 1 < len) ? p.delta[base + q0 + 1] : 0.f;
    };
    QBlockScan<CAUSAL> scan(p.bmask_t, b, p.Hq, G, kvh, nt, n_qblocks, p.rows_padded, p.n_words);
    int g, m, g_next = 0, m_next = 0;
    uint32_t flags;
    bool have = scan.next(g, m, flags);
    float td[4] = {0.f, 0.f, 0.f, 0.f};
    if (have) fetch_td(g, m, td);
    bool ok = !ptx::c_withhold_loads;
    for (int j = 0; ok && have; ++j) {
      const int st = j % kDkvStages;
      const int qh = b * p.Hq + kvh * G + g;
      const bool have_next = scan.next(g_next, m_next, flags);
      if (*cta_abort) break;
      if (lane == 0) ok = ptx::mbar_wait(x_empty + st, ((j / kDkvStages) & 1) ^ 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) raise_abort(cta_abort, p.status, kStTimeoutProducer); break; }
      float* dst = s_td + st * 128;
      *reinterpret_cast<float2*>(dst + 2 * lane) = make_float2(td[0], td[1]);
      *reinterpret_cast<float2*>(dst + 64 + 2 * lane) = make_float2(td[2], td[3]);
      __syncwarp();
      if (ptx::elect_one()) {
        ptx::mbar_arrive_expect_tx(x_full + st, 2 * L::qblk_bytes);  // releases the stores above to the waiters
        for (int pn = 0; pn < PANELS; ++pn) {
          ptx::tma_load_3d(sQ + st * L::qblk_bytes + pn * kQPanelBytes, &tmQ64, x_full + st, pn * 64, m * kQBlock, qh);
          ptx::tma_load_3d(sDO + st * L::qblk_bytes + pn * kQPanelBytes, &tmDO64, x_full + st, pn * 64, m * kQBlock, qh);
        }
      }
      if (have_next) fetch_td(g_next, m_next, td);
      g = g_next; m = m_next;
      have = have_next;
    }
  } else if (warp == 17 || warp == 18) {
    // ---------------- S^T issuer (warp 17: K~ Q_j^T) and dP^T issuer (warp 18: V dO_j^T) ----------------
    // Four warps issue the four products of a step, so that the waits and commits of one
    // overlap the MMAs of the others (an issuing thread that waits leaves the tensor pipe idle).
    constexpr uint32_t idesc_s = ptx::make_idesc(FMT, kBlockN, kQBlock, 0, 0);   // 128 keys x 64 queries
    const bool is_s = warp == 17;
    bool ok = true;
    if (lane == 0) ok = ptx::mbar_wait(k_ready, 0);
    ok = __all_sync(0xffffffffu, ok);
    QBlockScan<CAUSAL> scan(p.bmask_t, b, p.Hq, G, kvh, nt, n_qblocks, p.rows_padded, p.n_words);
    int g, m;
    uint32_t flags;
    for (int j = 0; ok && scan.next(g, m, flags); ++j) {
      const int st = j % kDkvStages, buf = j & 1;
      if (*cta_abort) { ok = false; break; }
      if (ptx::elect_one()) {
        // the S^T buffer holds P^T and dS^T until the dV / dK products are done; the dP^T buffer
        // is free as soon as the row warps have copied it to registers
        ok = ptx::mbar_wait(x_full + st, (j / kDkvStages) & 1) &&
             ptx::mbar_wait((is_s ? s_free : dp_free) + buf, ((j >> 1) & 1) ^ 1);
        if (ok) {
          ptx::tc_fence_after_sync();
          const uint32_t a0 = ptx::smem_u32(is_s ? sK : sV);
          const uint32_t b0 = ptx::smem_u32((is_s ? sQ : sDO) + st * L::qblk_bytes);
          const uint32_t d = tmem_base + (is_s ? 0u : DP_COL0) + buf * kQBlock;
#pragma unroll
          for (int kk = 0; kk < KSTEPS; ++kk) {
            const uint32_t offa = (kk >> 2) * kPanelBytes + (kk & 3) * 32;
            const uint32_t offb = (kk >> 2) * kQPanelBytes + (kk & 3) * 32;
            ptx::mma_ss(d, ptx::make_smem_desc(a0 + offa, 16, 1024), ptx::make_smem_desc(b0 + offb, 16, 1024),
                        idesc_s, kk > 0);
          }
          ptx::mma_commit(s_full + buf);
        }
      }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok && lane == 0 && !*cta_abort) raise_abort(cta_abort, p.status, kStTimeoutMma);
  } else if (warp == 19 || warp == 20) {
    // ---------------- dV issuer (warp 19: dV += P^T dO_j) and dK issuer (warp 20: dK += dS^T Q_j) ----------------
    constexpr uint32_t idesc_acc = ptx::make_idesc(FMT, kBlockN, D, 0, 1);        // 128 keys x D
    const bool is_dv = warp == 19;
    bool ok = true;
    QBlockScan<CAUSAL> scan(p.bmask_t, b, p.Hq, G, kvh, nt, n_qblocks, p.rows_padded, p.n_words);
    int g, m, g_next = 0, m_next = 0;
    uint32_t flags;
    bool have = scan.next(g, m, flags);
    for (int j = 0; ok && have; ++j) {
      const int st = j % kDkvStages, buf = j & 1;
      const bool have_next = scan.next(g_next, m_next, flags);
      if (*cta_abort) { ok = false; break; }
      if (lane == 0) ok = ptx::mbar_wait(p_full + buf, (j >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      uint8_t* bt = (is_dv ? sDO : sQ) + st * L::qblk_bytes;  // B operand: dO for dV, Q for dK
      if ((m + 1) * kQBlock > len) {
        // padded query rows: rows = 0 for the transposed product (the S^T / dP^T products that
        // read this block have completed before p_full)
        const int first = len - m * kQBlock;
        for (int pn = 0; pn < PANELS; ++pn) {
          uint4* bq = reinterpret_cast<uint4*>(bt + pn * kQPanelBytes + first * 128);
          for (int v = lane; v < (kQBlock - first) * 8; v += 32) bq[v] = make_uint4(0, 0, 0, 0);
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
      }
      if (ptx::elect_one()) {
        ptx::tc_fence_after_sync();
        const uint32_t b0 = ptx::smem_u32(bt);
        // P^T / dS^T: 16 queries = 8 packed columns per k-step, at the start of each 16-column group
        const uint32_t a = tmem_base + buf * kQBlock + (is_dv ? 0u : 8u);  // dS^T sits 8 columns after P^T
        const uint32_t acc = tmem_base + (is_dv ? DV_COL : DK_COL);
#pragma unroll
        for (int kk = 0; kk < kQBlock / 16; ++kk) {
          ptx::mma_ts(acc, a + kk * 16, ptx::make_smem_desc(b0 + kk * 2048, kQPanelBytes, 1024), idesc_acc,
                      (j > 0 || kk > 0));
        }
        ptx::mma_commit(x_empty + st);
        ptx::mma_commit(s_free + buf);
        if (!have_next) ptx::mma_commit(acc_full);
      }
      g = g_next; m = m_next;
      have = have_next;
    }
    if (!ok && lane == 0 && !*cta_abort) raise_abort(cta_abort, p.status, kStTimeoutMma);
  } else {
    // All sixteen row warps work on every step: warp w owns TMEM lanes 32*(w & 3) .. +31 (key
    // rows) and the sixteen query columns 16*(w >> 2) .. +15 of the block.  A short row phase
    // matters more than two steps in flight: S^T_j -> row work -> dV/dK_j -> S^T_{j+2} is a
    // dependent chain per buffer, and two groups of warps on different steps only slow each other.
    const int wq = warp & 3;
    const int slice = warp >> 2;
    const int r = wq * 32 + lane;        // key row inside the tile
    const int key = n0 + r;
    const bool key_ok = key < len;
    const int kh = wq >> 1;              // which 64-key half
    const simt::Powers powers(p.alpha);  // used by the generic-alpha instantiation only
    const uint32_t lane_addr = tmem_base + ((uint32_t)(wq * 32) << 16);
    bool dead = false;
    if (!ptx::mbar_wait_warp(kv_full, 0)) { raise_abort(cta_abort, p.status, kStTimeoutEpilogue); dead = true; }
    if (!dead) {
      // K~ = rn(k * fp32(0.5/sqrt(D))) in place; rows >= len -> 0 in K and V
      const float sc = (AM == 0 && CAUSAL) ? 0.5f * p.sm_scale : p.zscale;
      for (int v = threadIdx.x; v < L::tile_bytes / 16; v += kDkvRowThreads) {
        const int vrow = ((v * 16) % kPanelBytes) / 128;
        const bool keep = (n0 + vrow) < len;
        uint4* pk = reinterpret_cast<uint4*>(sK) + v;
        uint4 val = *pk;
        T* e = reinterpret_cast<T*>(&val);
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) e[jj] = DT<T>::from_f(keep ? DT<T>::to_f(e[jj]) * sc : 0.f);
        *pk = val;
        if (!keep) reinterpret_cast<uint4*>(sV)[v] = make_uint4(0, 0, 0, 0);
      }
      ptx::fence_proxy_async_smem();
    }
    ptx::mbar_arrive_warp(k_ready);
    // tau / delta of a step's 64 query rows arrive in shared memory with the step's Q / dO blocks
    QBlockScan<CAUSAL> scan(p.bmask_t, b, p.Hq, G, kvh, nt, n_qblocks, p.rows_padded, p.n_words);
    int g = 0, m = 0, n_active = 0;
    uint32_t flags = 0;
    for (int j = 0; scan.next(g, m, flags); ++j) {
      n_active = j + 1;
      const int buf = j & 1, it = j >> 1, st = j % kDkvStages;
      const float* td = s_td + st * 128;
      if (!(dead || *cta_abort)) {
        // x_full completed before the products behind s_full were issued; waiting on it here
        // as well makes the producer's tau / delta stores visible to this thread
        if (!ptx::mbar_wait_warp(s_full + buf, it & 1) || !ptx::mbar_wait_warp(x_full + st, (j / kDkvStages) & 1)) {
          raise_abort(cta_abort, p.status, kStTimeoutEpilogue);
          dead = true;
        }
      } else {
        dead = true;
      }
      if (!dead) {
        ptx::tc_fence_after_sync();
        const bool sub_on = (flags >> kh) & 1u;  // warp-uniform: the TMEM loads below are warp-collective
        const bool full = CAUSAL ? (n0 + kBlockN - 1 <= m * kQBlock) && ((m + 1) * kQBlock <= len)
                                 : (n0 + kBlockN <= len) && ((m + 1) * kQBlock <= len);
        {
          const int c0 = slice * 16;                // first query column of this thread
          const int q0 = m * kQBlock + c0;
          const uint32_t saddr = lane_addr + buf * kQBlock + c0;
          const uint32_t daddr = lane_addr + DP_COL0 + buf * kQBlock + c0;
          uint32_t pk[8], dk[8];
          if (!sub_on) {
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive_warp(dp_free + buf);
#pragma unroll
            for (int c = 0; c < 8; ++c) { pk[c] = 0u; dk[c] = 0u; }
          } else {
            uint32_t rs[16], rp[16];
            ptx::tmem_ld16(saddr, rs);
            ptx::tmem_ld16(daddr, rp);
            ptx::tmem_ld_wait();
            // dP^T is in registers: its buffer may take the next product already (dS^T goes
            // into the free half of this thread's S^T columns, not back there)
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive_warp(dp_free + buf);
            const float* s = reinterpret_cast<const float*>(rs);
            const float* dp = reinterpret_cast<const float*>(rp);
            const float* tq = td + c0;
            const float* dq_ = td + 64 + c0;
            if (full) {
              // every (key, query) pair of the step is causal and inside the sequence
#pragma unroll
              for (int c = 0; c < 16; c += 4) {
                const float4 t4 = *reinterpret_cast<const float4*>(tq + c);
                const float4 l4 = *reinterpret_cast<const float4*>(dq_ + c);
                const float u0 = fmaxf(s[c] - t4.x, 0.f), u1 = fmaxf(s[c + 1] - t4.y, 0.f);
                const float u2 = fmaxf(s[c + 2] - t4.z, 0.f), u3 = fmaxf(s[c + 3] - t4.w, 0.f);
                if constexpr (AM == 0) {
                  pk[c >> 1] = pack2<T>(u0 * u0, u1 * u1);
                  pk[(c >> 1) + 1] = pack2<T>(u2 * u2, u3 * u3);
                  dk[c >> 1] = pack2<T>(u0 * (dp[c] - l4.x), u1 * (dp[c + 1] - l4.y));
                  dk[(c >> 1) + 1] = pack2<T>(u2 * (dp[c + 2] - l4.z), u3 * (dp[c + 3] - l4.w));
                } else if constexpr (AM == 1) {  // alpha = 2: p = u, Jacobian weight 1 on the support
                  pk[c >> 1] = pack2<T>(u0, u1);
                  pk[(c >> 1) + 1] = pack2<T>(u2, u3);
                  dk[c >> 1] = pack2<T>(u0 > 0.f ? dp[c] - l4.x : 0.f, u1 > 0.f ? dp[c + 1] - l4.y : 0.f);
                  dk[(c >> 1) + 1] = pack2<T>(u2 > 0.f ? dp[c + 2] - l4.z : 0.f, u3 > 0.f ? dp[c + 3] - l4.w : 0.f);
                } else {  // any alpha
                  pk[c >> 1] = pack2<T>(powers.p(u0), powers.p(u1));
                  pk[(c >> 1) + 1] = pack2<T>(powers.p(u2), powers.p(u3));
                  dk[c >> 1] = pack2<T>(powers.g(u0) * (dp[c] - l4.x), powers.g(u1) * (dp[c + 1] - l4.y));
                  dk[(c >> 1) + 1] = pack2<T>(powers.g(u2) * (dp[c + 2] - l4.z), powers.g(u3) * (dp[c + 3] - l4.w));
                }
              }
            } else {
            // query column c is valid iff key <= q0 + c < len  <=>  lo <= c < hi
            const int lo = CAUSAL ? key - q0 : -(1 << 30), hi = key_ok ? len - q0 : 0;
#pragma unroll
            for (int c = 0; c < 16; c += 2) {
              const float2 t2 = *reinterpret_cast<const float2*>(tq + c);
              const float2 l2 = *reinterpret_cast<const float2*>(dq_ + c);
              const float u0 = s[c] - t2.x, u1 = s[c + 1] - t2.y;
              const bool ok0 = (u0 > 0.f) && (c >= lo) && (c < hi);
              const bool ok1 = (u1 > 0.f) && (c + 1 >= lo) && (c + 1 < hi);
              // select, not multiply: S / dP entries of padded rows may be anything
              if constexpr (AM == 0) {
                pk[c >> 1] = pack2<T>(ok0 ? u0 * u0 : 0.f, ok1 ? u1 * u1 : 0.f);
                dk[c >> 1] = pack2<T>(ok0 ? u0 * (dp[c] - l2.x) : 0.f, ok1 ? u1 * (dp[c + 1] - l2.y) : 0.f);
              } else if constexpr (AM == 1) {
                pk[c >> 1] = pack2<T>(ok0 ? u0 : 0.f, ok1 ? u1 : 0.f);
                dk[c >> 1] = pack2<T>(ok0 ? dp[c] - l2.x : 0.f, ok1 ? dp[c + 1] - l2.y : 0.f);
              } else {
                const float v0 = ok0 ? u0 : 0.f, v1 = ok1 ? u1 : 0.f;
                pk[c >> 1] = pack2<T>(powers.p(v0), powers.p(v1));
                dk[c >> 1] = pack2<T>(ok0 ? powers.g(v0) * (dp[c] - l2.x) : 0.f, ok1 ? powers.g(v1) * (dp[c + 1] - l2.y) : 0.f);
              }
            }
            }
          }
          // 16 queries = 8 packed columns each: P^T at the start of this thread's own 16
          // columns of S^T, dS^T in the other 8 (nobody else reads or writes those)
          ptx::tmem_st8(saddr, pk);
          ptx::tmem_st8(saddr + 8, dk);
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive_warp(p_full + buf);
      }
    }
    if (!dead && n_active > 0) {
      if (!ptx::mbar_wait_warp(acc_full, 0)) { raise_abort(cta_abort, p.status, kStTimeoutEpilogue); dead = true; }
    }
    if (!dead) {  // TMEM loads are warp-collective: only the global stores are per-row
      ptx::tc_fence_after_sync();
      const int ch = slice;  // the four threads of a key row share the D/32 column chunks
      if (ch < D / 32) {
        uint32_t rk[32], rv[32];
        if (n_active > 0) {
          ptx::tmem_ld32(lane_addr + DK_COL + ch * 32, rk);
          ptx::tmem_ld32(lane_addr + DV_COL + ch * 32, rv);
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) { rk[c] = 0u; rv[c] = 0u; }
        }
        const float* fk = reinterpret_cast<const float*>(rk);
        const float* fv = reinterpret_cast<const float*>(rv);
        uint32_t ok_[16], ov_[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          ok_[c >> 1] = key_ok ? pack2<T>(fk[c] * p.sm_scale, fk[c + 1] * p.sm_scale) : 0u;
          ov_[c >> 1] = key_ok ? pack2<T>(fv[c], fv[c + 1]) : 0u;
        }
        uint4* dst = reinterpret_cast<uint4*>(dkg + (size_t)key * Dg + ch * 32);
        uint4* dst2 = reinterpret_cast<uint4*>(dvg + (size_t)key * Dg + ch * 32);
        if (key < p.N) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            if (ch * 32 + q4 * 8 < Dg) {
              dst[q4] = make_uint4(ok_[q4 * 4], ok_[q4 * 4 + 1], ok_[q4 * 4 + 2], ok_[q4 * 4 + 3]);
              dst2[q4] = make_uint4(ov_[q4 * 4], ov_[q4 * 4 + 1], ov_[q4 * 4 + 2], ov_[q4 * 4 + 3]);
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
    ptx::tmem_dealloc(tmem_base, kDkvTmemCols);
  }
}

}  // namespace sm100
}  // namespace ads
