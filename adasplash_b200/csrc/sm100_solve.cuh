// Threshold solver + block-mask builder on the tensor cores.
//
// One CTA owns 256 query rows of one head -- two 128-row MMA tiles A and B --
// and runs the whole solve for them without leaving the SM.
// Both row tiles use every K tile that TMA brings in, which halves the L2 -> SM
// traffic per FLOP (a solver sweep has no other operand to amortise it: one
// 32 KB K tile per 128x128x128 product made it L2-bandwidth-bound).
//
//   * the two Q tiles are scaled by fp32(0.5/sqrt(D)), rounded to the input dtype
//     and parked in TMEM as A operands (columns 384..511), so the MMA reads only K
//     from shared memory: with both operands there, a 128x128x16 product needs all
//     of the 128 B/clk of shared-memory bandwidth and the TMA writes of K compete
//     with it;
//   * S_A = Q~_A K^T and S_B = Q~_B K^T rotate through three 128-column fp32 TMEM
//     buffers (product n goes to buffer n % 3): one is read by row group A, one by
//     row group B, one is being written, so the product of a group's next tile
//     overlaps its row work.  Each row tile has its own issuing warp (issuing an MMA
//     costs the thread as long as the product costs the pipe) with its own "buffer
//     free" barriers, and each row group its own "product done" barriers per buffer,
//     so that every waiter sees every phase of the barriers it waits on;
//   * inside a group, TMEM lane = score row, and the two warps that own the same
//     32 lanes split the 128 keys of a tile in halves (the row work of a tile is
//     a chain of TMEM round trips; two threads per row halve it).  The two
//     partial statistics of a row are combined once per sweep through shared
//     memory.
//
// Sweeps (adasplash_v2.py:151-681): row max -> tau0; BINS-bin histogram -> tau1;
// niter Halley/bisection steps; a last sweep that records, per 64x64 sub-tile,
// whether any score exceeds the tau entering the sweep, then one more step.
//
// Everything after the row maximum only looks at scores >= tau0 = max - 1: the
// histogram covers [tau0, tau0 + 1], and tau never falls below tau0 (the largest
// probability (z_max - tau)^2 is at most 1).  Those scores are a tiny part of a
// row, so the kernel computes S twice, not (3 + niter) times: sweep 1 finds the
// row maxima; sweep 2 appends every score >= tau0 (value and key index)
// to a per-thread list in a shared-memory pool; the histogram, the Halley steps
// and the final bitmap + step run on the lists.  The counts and bitmap bits are
// the same integers either way; the Halley sums add the same terms in list order.
// If the pool fills up (rows whose scores are nearly flat), sweep 2 goes on as a
// plain histogram sweep for the scores that find no room, and the CTA sweeps S
// for the remaining steps as well -- what the solve cost without lists.  When the
// caller wants the rows' supports (support.cuh), such a CTA first tries a third
// sweep that lists the scores above the histogram's lower bound -- far fewer --
// and runs its steps on those lists; the tail of the kernel exports the supports
// from whichever lists it ended up with.
// (One sweep with a running maximum does not work: the maximum of a row grows so
// slowly that three times as many scores pass "within 1 of the maximum so far"
// as are within 1 of the final one.)
#pragma once
#include <type_traits>

#include "sm100_fwd.cuh"

namespace ads {
namespace sm100 {

constexpr int kSolveStages = 3;  // K tiles in flight (two measured 5 % slower once the issuing warps stopped being the limit)
constexpr int kSolveThreads = 608;   // 2 row groups x 8 warps + TMA warp + one MMA warp per row tile
constexpr int kSolveRowThreads = 512;
constexpr int kSolveGroupThreads = 256;
constexpr int kSolveTmemCols = 512;  // three S buffers at columns 0 / 128 / 256, Q~_A, Q~_B from column 384
constexpr uint32_t kSolveQCol = 384;
constexpr int kSolveBufs = 3;
constexpr int kSolveRows = 2 * kBlockM;  // query rows per CTA

enum SweepMode : int { kModeMax = 0, kModeHist = 1, kModeHalley = 2, kModeFinal = 3, kModeCollect = 4, kModeRecollect = 5 };

// One entry of the candidate pool: a score >= tau0 of some row, its key index (sequences of more
// than 65536 keys: only the 64-key block it sits in), and the previous entry of the same
// thread's list (written with one 8-byte store).
struct __align__(8) Cand { float z; uint16_t key; uint16_t next; };
constexpr uint16_t kCandNil = 0xffff;

// Shared memory: K stages, barriers, exchange buffers, bitmap staging, then the two Q tiles and
// whatever is left of the budget.  The Q tiles are dead once Q~ sits in TMEM (before the first
// append), so the candidate pool is their space plus that remainder (D = 128: ~110 KB, 14000
// entries, 27 per thread on average).  Each row warp appends to its own sixteenth and hands
// out its slots by a warp vote.
constexpr int kSolveSmemBudget = 225 * 1024;

template <int D>
struct SolveSmem {
  static constexpr int tile_bytes = (D / 64) * kPanelBytes;
  static constexpr int k_off = 0;
  static constexpr int bar_off = k_off + kSolveStages * tile_bytes;
  static constexpr int n_bars = 2 + 2 * kSolveStages + 4 * kSolveBufs + 1;
  static constexpr int misc_off = bar_off + n_bars * 8;            // tmem base, abort flag, status, pool counters
  static constexpr int xchg_off = misc_off + 128;                  // [2 groups][2 halves][8][128] floats
  static constexpr int bits_off = xchg_off + 2 * 2 * 8 * 128 * 4;  // [4][n_words] words
  static __host__ __device__ int q_off(int n_words) { return (bits_off + 4 * n_words * 4 + 1023) & ~1023; }  // two Q tiles
  static __host__ __device__ int pool_entries(int n_words) { return (kSolveSmemBudget - 1024 - q_off(n_words)) / 8; }
  static size_t bytes(int) { return kSolveSmemBudget; }
};

// V1 = false is the AdaSplash-2 solver described above.  V1 = true serves the first-generation
// semantics on the same machinery (any alpha in (1, 2], causal or full attention;
// adasplash_block_mask.py:40-296): the same two sweeps (row maxima, candidates within 1 of the
// maximum), then no histogram: the bracket is [max - 1, max - n^(1-alpha)] with n the row's number
// of valid keys, niter Halley / bisection steps run on the candidates, and the block mask is
// taken at the lower end of the final bracket (tau_lo <= tau*: no tile of the support is missed).
template <typename T, int D, bool V1 = false>
__global__ void __launch_bounds__(kSolveThreads, 1)
solve_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
             TcParams p) {
  using L = SolveSmem<D>;
  constexpr int PANELS = D / 64;
  constexpr int KSTEPS = D / 16;
  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem + L::q_off(p.n_words);
  uint8_t* sK = smem + L::k_off;
  uint64_t* bars = (uint64_t*)(smem + L::bar_off);
  uint64_t* q_full = bars + 0;
  uint64_t* q_ready = bars + 1;
  uint64_t* k_full = bars + 2;
  uint64_t* k_empty = k_full + kSolveStages;
  uint64_t* s_full = k_empty + kSolveStages;  // [2 row tiles][3 S buffers]: each row group sees only its own products
  uint64_t* s_free = s_full + 2 * kSolveBufs;  // [row tile of the buffer's next product][3 S buffers]
  uint64_t* decide = s_free + 2 * kSolveBufs;              // the row warps have settled lists vs. full sweeps
  uint32_t* tmem_holder = (uint32_t*)(smem + L::misc_off);
  volatile int* cta_abort = (volatile int*)(smem + L::misc_off + 4);
  int* start_status = (int*)(smem + L::misc_off + 8);
  int* pool_used = (int*)(smem + L::misc_off + 32);   // [16]: entries used in each row warp's region
  volatile int* pool_ovf = (volatile int*)(smem + L::misc_off + 16);
  volatile int* pool_ovf2 = (volatile int*)(smem + L::misc_off + 20);  // ... and so did the lists of the third sweep
  int* pool_common = (int*)(smem + L::misc_off + 24);  // third sweep: entries used (one counter for the CTA)
  float* xchg = (float*)(smem + L::xchg_off);
  uint32_t* s_bits = (uint32_t*)(smem + L::bits_off);
  Cand* pool = (Cand*)sQ;  // the Q tiles are dead once Q~ is in TMEM (before the first append)
  const int warp_pool = L::pool_entries(p.n_words) / 16;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = p.B * p.Hq;
  const int npair = (p.nq + 1) / 2;
  const int pr_idx = npair - 1 - (int)(blockIdx.x / heads);  // heaviest row pairs first, across all heads
  const int bh = blockIdx.x % heads;
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const int m0 = pr_idx * kSolveRows;  // first row of tile A; tile B starts at m0 + 128
  if (m0 >= len) return;
  const bool b_on = (m0 + kBlockM) < len;           // row tile B has at least one valid row
  const int qtA = 2 * pr_idx, qtB = qtA + 1;        // their 128-row tile indices
  const bool full_attn = V1 && p.causal == 0;
  const int T_all = (len + kBlockN - 1) / kBlockN;  // key tiles of a row without the causal mask
  const int T_a = full_attn ? T_all : qtA + 1;      // key tiles of A: 0 .. qtA
  const int T_k = full_attn ? T_all : (b_on ? qtB + 1 : T_a);  // key tiles streamed per sweep
  const int nsweeps = p.tau_given ? 1 : p.niter + 3;
  // tiles streamed before the row warps decide (max sweep, histogram + collect sweep), and in
  // all if the candidate pool overflows (then the Halley .. final steps sweep S as well)
  const int total_first = p.tau_given ? T_k : 2 * T_k;
  const int total_full = nsweeps * T_k;
  // AdaSplash-2 solver: a CTA whose pool overflowed in sweep 2 sweeps once more for the scores
  // above the histogram's lower bound (see the row warps) before it resorts to full sweeps
  // -- when the rows' supports are wanted (the lists are what they are exported from) or when
  // it saves at least two sweeps.  (With niter = 1 and no export it is no gain: its appends cost
  // what the one sweep it saves would have.)
  const bool third_sweep = !V1 && !p.tau_given && (p.sup_on || p.niter >= 2);
  // Products are numbered in K-tile order (per K tile: A if it has one, then B); product n uses
  // S buffer n % 3 for the (n / 3)-th time.
  const int prods_per_sweep = b_on ? T_a + T_k : T_a;   // causal: T_k = T_a + 1
  auto product_in_sweep = [&](int kt, int g) -> int {
    return b_on ? (kt < T_a ? 2 * kt + g : T_a + kt) : kt;
  };

  if (threadIdx.x == 0) {
    *start_status = *(volatile int*)p.status;
    *cta_abort = 0;
    for (int w = 0; w < 16; ++w) pool_used[w] = 0;
    *pool_ovf = 0;
    *pool_ovf2 = 0;
  }
  if (warp == 17) {
    if (lane == 0) {
      ptx::mbar_init(q_full, 1);
      ptx::mbar_init(q_ready, kSolveRowThreads / 32);
      ptx::mbar_init(decide, kSolveRowThreads / 32);
      // a K stage is empty again when the issuers of both row tiles are through with it
      for (int s = 0; s < kSolveStages; ++s) { ptx::mbar_init(k_full + s, 1); ptx::mbar_init(k_empty + s, b_on ? 2 : 1); }
      for (int s = 0; s < 2 * kSolveBufs; ++s) ptx::mbar_init(s_full + s, 1);
      for (int s = 0; s < 2 * kSolveBufs; ++s) ptx::mbar_init(s_free + s, kSolveGroupThreads / 32);
      ptx::fence_mbar_init();
    }
    __syncwarp();
    ptx::tmem_alloc(tmem_holder, kSolveTmemCols);
    ptx::tmem_relinquish();
  }
  for (int w = threadIdx.x; w < 4 * p.n_words; w += kSolveThreads) s_bits[w] = 0u;
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (*start_status != 0) {  // an earlier CTA of this launch already failed: do nothing
    if (warp == 17) ptx::tmem_dealloc(*tmem_holder, kSolveTmemCols);
    return;
  }
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 16) {
    // ---------------- TMA producer ----------------
    if (ptx::elect_one()) {
      ptx::prefetch_tmap(&tmQ);
      ptx::prefetch_tmap(&tmK);
      ptx::mbar_arrive_expect_tx(q_full, 2 * L::tile_bytes);
      for (int t = 0; t < 2; ++t)
        for (int pn = 0; pn < PANELS; ++pn)
          ptx::tma_load_3d(sQ + t * L::tile_bytes + pn * kPanelBytes, &tmQ, q_full, pn * 64, m0 + t * kBlockM, bh);
      const int kv_head = b * p.Hkv + kvh;
      int total = total_first;
      // stage, its use parity and the key tile are carried along (no divisions in the loop)
      int st = 0, kt = 0;
      uint32_t use_par = 0;
      for (int i = 0; !ptx::c_withhold_loads; ++i) {
        if (i == total) {
          // the first sweeps are through: stream S again only if the row warps ask for it
          if (total == total_full + (third_sweep ? T_k : 0)) break;
          const bool second = total > total_first;  // the decision after the third sweep
          if (!ptx::mbar_wait(decide, second ? 1 : 0)) { raise_abort(cta_abort, p.status, kStTimeoutProducer); break; }
          if (!(second ? *pool_ovf2 : *pool_ovf)) break;
          total = (third_sweep && !second) ? total_first + T_k : total_full + (third_sweep ? T_k : 0);
        }
        if (*cta_abort) break;
        if (!ptx::mbar_wait(k_empty + st, use_par ^ 1)) {
          raise_abort(cta_abort, p.status, kStTimeoutProducer);
          break;
        }
        ptx::mbar_arrive_expect_tx(k_full + st, L::tile_bytes);
        for (int pn = 0; pn < PANELS; ++pn)
          ptx::tma_load_3d(sK + st * L::tile_bytes + pn * kPanelBytes, &tmK, k_full + st, pn * 64,
                           kt * kBlockN, kv_head);
        if (++st == kSolveStages) { st = 0; use_par ^= 1; }
        if (++kt == T_k) kt = 0;
      }
    }
  } else if (warp == 17 || warp == 18) {
    // ---------------- MMA issuers: warp 17 for row tile A, warp 18 for row tile B ----------------
    // Issuing one tcgen05.mma keeps the issuing thread busy for about as long as the 128x128x16
    // product keeps the tensor pipe (70 - 80 clocks measured, whatever the product's size), so a
    // single thread issuing for both row tiles fed the pipe at half its rate.  Products keep
    // their numbering in K-tile order (per K tile: A if it has one, then B) and product n its
    // buffer n % 3.  A buffer's "free" barrier is chosen by the row tile of the product that takes
    // the buffer next (the row warps know it when they let go of the buffer): each issuer is then
    // the only waiter of its three barriers and sees each of their phases in turn (a thread that
    // skips a phase of an mbarrier cannot tell the phase after it from the one before).
    const int g = warp - 17;
    if ((g == 0 || b_on) && ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::make_idesc(FMT, kBlockM, kBlockN, 0, 0);
      bool ok = ptx::mbar_wait(q_ready, 0);
      if (!ok) raise_abort(cta_abort, p.status, kStTimeoutMma);
      int total = total_first;
      // stage / key tile / number of the K tile's first product (and its buffer) are carried along
      int st = 0, kt = 0, n0p = 0, bf0 = 0;
      uint32_t k_par = 0, free_par = 0;  // bit b of free_par: parity of this issuer's next wait for buffer b
      const uint32_t a_tmem = tmem_base + kSolveQCol + g * (D / 2);
      for (int i = 0; ok; ++i) {
        if (i == total) {
          if (total == total_full + (third_sweep ? T_k : 0)) break;
          const bool second = total > total_first;
          if (!ptx::mbar_wait(decide, second ? 1 : 0)) { raise_abort(cta_abort, p.status, kStTimeoutMma); break; }
          if (!(second ? *pool_ovf2 : *pool_ovf)) break;
          total = (third_sweep && !second) ? total_first + T_k : total_full + (third_sweep ? T_k : 0);
        }
        if (*cta_abort) break;
        if (!ptx::mbar_wait(k_full + st, k_par)) { raise_abort(cta_abort, p.status, kStTimeoutMma); break; }
        const int has_a = kt < T_a ? 1 : 0;  // the diagonal key tile of B has nothing for A
        if (g == 1 || has_a) {
          const int skip = g == 1 ? has_a : 0;  // B's product follows A's
          int bf = bf0 + skip;
          if (bf >= kSolveBufs) bf -= kSolveBufs;
          if (n0p + skip >= kSolveBufs) {  // the buffer held a product before: the row warps must be through with it
            if (!ptx::mbar_wait(s_free + g * kSolveBufs + bf, (free_par >> bf) & 1u)) {
              raise_abort(cta_abort, p.status, kStTimeoutMma);
              break;
            }
            free_par ^= 1u << bf;
          }
          ptx::tc_fence_after_sync();
          const uint32_t b0 = ptx::smem_u32(sK + st * L::tile_bytes);
          const uint32_t d = tmem_base + bf * kBlockN;
#pragma unroll
          for (int kk = 0; kk < KSTEPS; ++kk) {
            const uint32_t off = (kk >> 2) * kPanelBytes + (kk & 3) * 32;
            ptx::mma_ts(d, a_tmem + kk * 8, ptx::make_smem_desc(b0 + off, 16, 1024), idesc, kk > 0);
          }
          ptx::mma_commit(s_full + g * kSolveBufs + bf);
          ptx::mma_commit(k_empty + st);
        } else {
          ptx::mbar_arrive(k_empty + st);
        }
        const int adv = has_a + (b_on ? 1 : 0);
        n0p += adv;
        bf0 += adv;
        if (bf0 >= kSolveBufs) bf0 -= kSolveBufs;
        if (++st == kSolveStages) { st = 0; k_par ^= 1; }
        if (++kt == T_k) kt = 0;
      }
    }
  } else {
    // ---------------- row groups: group t owns row tile t, one score row per thread ----------------
    const int grp = warp >> 3, half = (warp >> 2) & 1, wq = warp & 3;
    const int r = wq * 32 + lane;
    const int row = m0 + grp * kBlockM + r;
    const bool row_ok = row < len;
    const int rb = wq >> 1;
    const int qt = grp == 0 ? qtA : qtB;            // this group's 128-row tile index
    const bool grp_on = grp == 0 || b_on;
    const int T_g = full_attn ? T_all : qt + 1;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(wq * 32) << 16);
    bool dead = false;
    // Q~ = rn(q * fp32(0.5/sqrt(D))) (rows >= len -> 0), from the TMA tile in shared
    // memory into TMEM: the two threads of row r convert D/2 elements each (16-bit pairs, lane r)
    if (!ptx::mbar_wait_warp(q_full, 0)) { raise_abort(cta_abort, p.status, kStTimeoutEpilogue); dead = true; }
    if (!dead) {
      const float sc = row_ok ? (V1 ? p.zscale : 0.5f * p.sm_scale) : 0.f;
      const uint8_t* qtile = sQ + grp * L::tile_bytes;
#pragma unroll
      for (int hh = 0; hh < D / 64; ++hh) {  // 32 elements -> 16 packed columns per store; D/2 elements per thread
        const int h16 = half * (D / 64) + hh;
        uint32_t pk[16];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int e0 = (h16 * 4 + cc) * 8;               // first element of the 16-byte chunk
          const int pn = e0 >> 6, c = (e0 & 63) >> 3;      // panel, chunk inside the 128-byte row
          const uint4 val = *reinterpret_cast<const uint4*>(qtile + pn * kPanelBytes + r * 128 + ((c ^ (r & 7)) << 4));
          const T* e = reinterpret_cast<const T*>(&val);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            pk[cc * 4 + j] = pack2<T>(DT<T>::to_f(e[2 * j]) * sc, DT<T>::to_f(e[2 * j + 1]) * sc);
        }
        ptx::tmem_st16(lane_addr + kSolveQCol + grp * (D / 2) + h16 * 16, pk);
      }
      ptx::tmem_st_wait();
      ptx::tc_fence_before_sync();
    }
    ptx::mbar_arrive_warp(q_ready);

    // Above alpha = 1.5, when the rows' supports are wanted: the backward's key side decides
    // "score above tau" from its own product (K scaled and rounded, q raw), and the Jacobian
    // weight does not vanish at the threshold, so pairs within the two products' largest
    // possible difference below tau are listed and exported as well (with u <= 0: no weight on
    // the query side).  |Q~ k - q K~| <= 2^-8 zscale |q| |k| for 16-bit operands (unit roundoff
    // 2^-9 each); the largest key norm of the head comes from a small kernel run before this one.
    float margin = 0.f;
    if constexpr (V1) {
      if (p.sup_on && p.alpha > 1.5f && row_ok && !dead) {
        const T* qrow = (const T*)p.q_raw + ((size_t)bh * p.N + row) * p.d_true;
        float qn2 = 0.f;
        for (int d0 = 0; d0 < p.d_true; d0 += 8) {
          const uint4 raw8 = *reinterpret_cast<const uint4*>(qrow + d0);
          const T* e8 = reinterpret_cast<const T*>(&raw8);
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float x = DT<T>::to_f(e8[j]); qn2 = fmaf(x, x, qn2); }
        }
        margin = 0.00390625f * p.zscale * sqrtf(qn2 * p.sup.kmax2[b * p.Hkv + kvh]) + 1e-5f;
      }
    }

    float mx = -1.0e3f, tau0 = 0.f;
    int cnt[8];
    HalleyState hs;
    hs.t = hs.lo = hs.hi = 0.f;
    if (p.tau_given) hs.t = row_ok ? p.taus[((size_t)bh) * p.N + row] : 0.f;
    const float fbins = (float)p.bins;
    int sweep_no = 0;  // sweeps over S started so far (fixes the S buffer of every tile)
    uint32_t full_par = 0;  // bit b: parity of this group's next product in S buffer b
    float a0 = 0.f, a1 = 0.f, a2 = 0.f;
    const simt::Powers powers(V1 ? p.alpha : 1.5f);   // first-generation instantiation only
    uint16_t head = kCandNil;  // this thread's list of scores >= tau0
    int ncand = 0;             // its length (counted on the first walk)
    const bool wide = p.N > 65536;  // key indices do not fit the 16 bits of a list entry
    const int kb_shift = wide ? 0 : 6;
    bool compact = false;      // the list was copied to one contiguous run starting at run0
    int my_used = 0;           // entries of this warp's share of the pool handed out so far (the same in all lanes)
    int run0 = 0;

    // One pass over the S tiles of this group's causal range.  Instantiated once per sweep
    // kind, so that the per-group code carries no mode tests and each sweep runs a compact loop.
    // score j of group g (four consecutive scores) of a thread's 32: seven selects
    auto pick_group = [](const float* v, int g, int j) -> float {
      const bool b0 = (g & 1) != 0, b1 = (g & 2) != 0, b2 = (g & 4) != 0;
      const float t0 = b0 ? v[4 + j] : v[j], t1 = b0 ? v[12 + j] : v[8 + j];
      const float t2 = b0 ? v[20 + j] : v[16 + j], t3 = b0 ? v[28 + j] : v[24 + j];
      const float u0 = b1 ? t1 : t0, u1 = b1 ? t3 : t2;
      return b2 ? u1 : u0;
    };
    auto sweep_tiles = [&](auto mode_c) {
      constexpr int mode = decltype(mode_c)::value;
      const int sweep = sweep_no++;
      for (int kt = 0; kt < T_g; ++kt) {
        if (dead || *cta_abort) { dead = true; continue; }
        const int idx = product_in_sweep(kt, grp);
        const int n = sweep * prods_per_sweep + idx;
        const int bf = n % kSolveBufs;
        // the row tile of product n + 3, the next one in this buffer: its issuer waits for this release
        int idx3 = idx + kSolveBufs;
        while (idx3 >= prods_per_sweep) idx3 -= prods_per_sweep;
        const int g_next = b_on ? (idx3 < 2 * T_a ? (idx3 & 1) : 1) : 0;
        const uint32_t par = (full_par >> bf) & 1u;
        full_par ^= 1u << bf;
        if (!ptx::mbar_wait_warp(s_full + grp * kSolveBufs + bf, par)) {
          raise_abort(cta_abort, p.status, kStTimeoutEpilogue);
          dead = true;
          continue;
        }
        ptx::tc_fence_after_sync();
        const int n0 = kt * kBlockN;
        const bool need_mask = (!full_attn && kt == qt) || (n0 + kBlockN > len);
        const float a2_mark = a2;  // support count before this thread's 64 keys of the tile
        // rows beyond the sequence have all-zero scores (every key would be a candidate) and
        // need no tau; once any warp's share of the pool is full the lists are useless
        const bool collecting = mode == kModeCollect && row_ok && !*pool_ovf;
        unsigned long long packed = 0ull;  // eight 8-bit cumulative bin counters of this tile
        // Collecting takes scores from a hair below tau0: a Halley step may land up to 1e-5
        // below its bracket, and a sweep over S would then see those scores too.  The
        // histogram over the list tests each score against tau0 itself.
        const float thr = mode == kModeCollect ? tau0 - 2e-5f - margin : ((V1 && mode == kModeFinal) ? hs.lo : hs.t);
        // (Register budget: the kernel keeps nearly all of the SM's shared memory, which leaves
        // almost no L1 for local memory -- a spill in this loop costs an L2 round trip.)
#pragma unroll 1
        for (int q32 = 0; q32 < 2; ++q32) {  // this thread's 64 keys, 32 at a time
          uint32_t raw[32];
          const int c0 = half * 64 + q32 * 32;
          ptx::tmem_ld32(lane_addr + bf * kBlockN + c0, raw);
          ptx::tmem_ld_wait();
          if (q32 == 1) {  // the last of this buffer is in registers: hand it back before the row work
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive_warp(s_free + g_next * kSolveBufs + bf);
          }
          float* v = reinterpret_cast<float*>(raw);
          const int keybase = wide ? 2 * kt + half : n0 + c0;
          const int kmask = wide ? 0 : 0xffff;
          if (need_mask) {
            const int lim = (full_attn ? len - 1 : min(row, len - 1)) - (n0 + c0);  // columns c <= lim survive
#pragma unroll
            for (int c = 0; c < 32; ++c) v[c] = (c <= lim) ? v[c] : kMaskedScore;
          }
          if (mode == kModeMax) {
            // four independent chains: a single running max would serialise the dependent ops
            float m0_ = mx, m1_ = mx, m2_ = mx, m3_ = mx;
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              m0_ = ptx::fmax3(m0_, v[c], v[c + 1]);
              m1_ = ptx::fmax3(m1_, v[c + 2], v[c + 3]);
              m2_ = ptx::fmax3(m2_, v[c + 4], v[c + 5]);
              m3_ = ptx::fmax3(m3_, v[c + 6], v[c + 7]);
            }
            mx = fmaxf(fmaxf(m0_, m1_), fmaxf(m2_, m3_));
          } else if (mode == kModeCollect) {
            // The histogram sweep: every score within 1 of the row maximum goes to this
            // thread's list while the pool has room (and is binned from there after the
            // sweep), else straight into the histogram.  Those scores are a small part of a
            // row (a thread has one in every sixth tile on the headline workload), but some lane
            // of the warp has one in a third of all groups of four, and a warp that opens each
            // such group in turn spends its time in sparsely occupied branches.  So: mark the
            // groups without branching, then let the warp work through the marked groups in
            // rounds -- in a round every lane that has one moves it to the same four registers
            // and appends one score, all lanes in one pass through one copy of the code.
            uint32_t mg = 0u;
#pragma unroll
            for (int g4 = 0; g4 < 8; ++g4) {
              const float cm = fmaxf(ptx::fmax3(v[g4 * 4], v[g4 * 4 + 1], v[g4 * 4 + 2]), v[g4 * 4 + 3]);
              mg |= (cm >= thr) ? (1u << g4) : 0u;
            }
            float z0 = 0.f, z1 = 0.f, z2 = 0.f, z3 = 0.f;
            uint32_t pend = 0u;  // positions of the open group that are still to be taken
            int gbase = 0;
            while (__any_sync(0xffffffffu, (mg | pend) != 0u)) {
              if (pend == 0u && mg != 0u) {
                const int gsel = __ffs(mg) - 1;
                mg &= mg - 1u;
                // (a select tree, not a switch: the lanes' groups differ, and a switch would run
                // through up to eight cases one after the other)
                z0 = pick_group(v, gsel, 0); z1 = pick_group(v, gsel, 1);
                z2 = pick_group(v, gsel, 2); z3 = pick_group(v, gsel, 3);
                gbase = gsel * 4;
                pend = (z0 >= thr ? 1u : 0u) | (z1 >= thr ? 2u : 0u) | (z2 >= thr ? 4u : 0u) | (z3 >= thr ? 8u : 0u);
              }
              const bool has = pend != 0u;
              const int c = has ? __ffs(pend) - 1 : 0;
              pend &= pend - 1u;
              const float z = c == 0 ? z0 : (c == 1 ? z1 : (c == 2 ? z2 : z3));
              // to the list while there is room, else straight into the histogram; the warp's
              // share of the pool is its own, so the slots come from a vote, not from an atomic
              const bool want = has && collecting;
              const uint32_t votes = __ballot_sync(0xffffffffu, want);
              bool listed = false;
              if (want) {
                const int idx = my_used + __popc(votes & ((1u << lane) - 1u));
                if (idx < warp_pool) {
                  const int slot = warp * warp_pool + idx;
                  Cand e;
                  e.z = z; e.next = head;
                  e.key = (uint16_t)(keybase + ((gbase + c) & kmask));
                  pool[slot] = e;
                  head = (uint16_t)slot;
                  listed = true;
                } else {
                  *pool_ovf = 1;
                }
              }
              my_used += __popc(votes);
              if (has && !listed) {
                // bin = floor((z - tau0) * BINS) clamped to 7; one add of a byte pattern
                // bumps the cumulative counters N_0..N_bin (<= 64 hits per tile: no overflow)
                const float prj = (z - tau0) * fbins;
                if (prj >= 0.f) {
                  const int bsel = min(__float2int_rd(prj), 7);
                  packed += 0x0101010101010101ull >> ((7 - bsel) * 8);
                }
              }
            }
          } else if (mode == kModeRecollect) {
            // Third sweep of a CTA whose pool overflowed in the second: the histogram has given
            // every row the lower end of its bracket, which no later tau undercuts (by more than
            // the step's tolerance), and the scores above that are few -- the support and a
            // little more -- where the scores within 1 of the maximum were too many.  Same
            // rounds as above; one counter for the CTA, so that the whole pool is open to
            // whichever rows need it (per-warp shares with a common overflow area measured no
            // faster), bumped once per round and warp.
            const float thr_c = hs.lo - 2e-5f;
            uint32_t mg = 0u;
#pragma unroll
            for (int g4 = 0; g4 < 8; ++g4) {
              const float cm = fmaxf(ptx::fmax3(v[g4 * 4], v[g4 * 4 + 1], v[g4 * 4 + 2]), v[g4 * 4 + 3]);
              mg |= (cm >= thr_c) ? (1u << g4) : 0u;
            }
            float z0 = 0.f, z1 = 0.f, z2 = 0.f, z3 = 0.f;
            uint32_t pend = 0u;
            int gbase = 0;
            while (__any_sync(0xffffffffu, (mg | pend) != 0u)) {
              if (pend == 0u && mg != 0u) {
                const int gsel = __ffs(mg) - 1;
                mg &= mg - 1u;
                // (a select tree, not a switch: the lanes' groups differ, and a switch would run
                // through up to eight cases one after the other)
                z0 = pick_group(v, gsel, 0); z1 = pick_group(v, gsel, 1);
                z2 = pick_group(v, gsel, 2); z3 = pick_group(v, gsel, 3);
                gbase = gsel * 4;
                pend = (z0 >= thr_c ? 1u : 0u) | (z1 >= thr_c ? 2u : 0u) | (z2 >= thr_c ? 4u : 0u) | (z3 >= thr_c ? 8u : 0u);
              }
              const bool want = pend != 0u && row_ok;
              const int c = pend != 0u ? __ffs(pend) - 1 : 0;
              pend &= pend - 1u;
              const float z = c == 0 ? z0 : (c == 1 ? z1 : (c == 2 ? z2 : z3));
              const uint32_t votes = __ballot_sync(0xffffffffu, want);
              if (votes != 0u) {
                int base = 0;
                if (lane == 0) base = atomicAdd(pool_common, __popc(votes));
                base = __shfl_sync(0xffffffffu, base, 0);
                if (want) {
                  const int j = base + __popc(votes & ((1u << lane) - 1u));
                  if (j < 16 * warp_pool) {
                    Cand e;
                    e.z = z; e.next = head;
                    e.key = (uint16_t)(keybase + ((gbase + c) & kmask));
                    pool[j] = e;
                    head = (uint16_t)j;
                  } else {
                    *pool_ovf2 = 1;
                  }
                }
              }
            }
          } else {
            // the scores above the threshold are a tiny part of a row: look at
            // four at a time and only open a group that contains one
#pragma unroll
            for (int g4 = 0; g4 < 8; ++g4) {
              const float cm = fmaxf(ptx::fmax3(v[g4 * 4], v[g4 * 4 + 1], v[g4 * 4 + 2]), v[g4 * 4 + 3]);
              if (cm > thr) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  const float d = v[g4 * 4 + c] - thr;
                  if (V1 && mode == kModeHalley && p.alpha != 1.5f) {
                    // sum u^(1/(alpha-1)), sum of the Jacobian weights g, sum g / u
                    if (d > 0.f) {
                      const float gw = powers.g(d);
                      a0 += powers.p(d); a1 += gw; a2 += powers.mode == 2 ? gw / d : 0.f;
                    }
                  } else {
                    if (d > 0.f) { a0 = fmaf(d, d, a0); a1 += d; a2 += 1.f; }
                  }
                }
              }
            }
          }
        }
        if (packed != 0ull) {
#pragma unroll
          for (int bb = 0; bb < 8; ++bb) cnt[bb] += (int)((packed >> (8 * bb)) & 0xffull);
        }
        if (mode == kModeFinal) {
          // this warp covers 32 rows x 64 keys of the 64x64 sub-tile (row block rb, key block 2kt+half)
          const bool any = __any_sync(0xffffffffu, (a2 > a2_mark) && row_ok);
          if (lane == 0 && any) {
            const int kb = 2 * kt + half;
            atomicOr(&s_bits[(grp * 2 + rb) * p.n_words + (kb >> 5)], 1u << (kb & 31));
          }
        }
      }
    };

    // The two threads of a row exchange their partial statistics and both compute the same
    // new state.
    auto exchange = [&](int mode) {
      float* xb = xchg + grp * (2 * 8 * 128);
      float* mine = xb + half * (8 * 128);
      const float* other = xb + (half ^ 1) * (8 * 128);
      if (mode == kModeMax) {
        mine[r] = mx;
      } else if (mode == kModeHist) {
#pragma unroll
        for (int c = 0; c < 8; ++c) mine[c * 128 + r] = __int_as_float(cnt[c]);
      } else {
        mine[r] = a0; mine[128 + r] = a1; mine[256 + r] = a2;
      }
      ptx::bar_sync(1 + grp, kSolveGroupThreads);
      float o[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) o[c] = other[c * 128 + r];
      ptx::bar_sync(1 + grp, kSolveGroupThreads);  // everyone has read: the buffer may be rewritten
      if (mode == kModeMax) {
        mx = fmaxf(mx, o[0]);
        tau0 = mx - 1.0f;
      } else if (mode == kModeHist) {
        int bins_cnt[8], cum[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) cum[c] = cnt[c] + __float_as_int(o[c]);
        for (int c = 0; c < p.bins; ++c) bins_cnt[c] = cum[c] - (c + 1 < p.bins ? cum[c + 1] : 0);
        const float t1 = hist_tau_alpha15<8>(bins_cnt, p.bins, tau0);
        hs.lo = t1;
        hs.hi = t1 + 1.0f / fbins;
        hs.t = 0.5f * (hs.lo + hs.hi);
      } else if (!p.tau_given) {
        // fixed operand order so that both threads of a row get bit-identical sums
        const float s0 = half == 0 ? a0 + o[0] : o[0] + a0;
        const float s1 = half == 0 ? a1 + o[1] : o[1] + a1;
        const float s2 = half == 0 ? a2 + o[2] : o[2] + a2;
        if constexpr (V1) {
          if (mode == kModeHalley) halley_bisect_update_generic(hs, s0, s1, s2, 1.0f / (p.alpha - 1.0f), 1.0f / (p.alpha - 1.0f) - 1.0f);
        } else {
          halley_bisect_update(hs, s0, s1, s2);
        }
      }
    };
    auto reset_stats = [&]() {
      a0 = a1 = a2 = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) cnt[c] = 0;
    };

    bool full_sweeps = false;  // the candidate pool overflowed: every step sweeps S
    bool recollected = false;  // the lists are those of the third sweep: anywhere in the pool, not compacted
    if (p.tau_given) {
      // bitmap for a given tau: one sweep over S
      if (grp_on) {
        reset_stats();
        sweep_tiles(std::integral_constant<int, kModeFinal>{});
      }
    } else {
      if (grp_on) {
        reset_stats();
        sweep_tiles(std::integral_constant<int, kModeMax>{});
        exchange(kModeMax);
        sweep_tiles(std::integral_constant<int, kModeCollect>{});
        if (lane == 0) pool_used[warp] = my_used;
        __syncwarp();
        // the listed scores join the histogram
        // (a thread's list is no longer than its warp's share of the pool: the walks are bounded)
        for (int e = head, left = warp_pool; e != kCandNil && left > 0; --left) {
          const Cand c = pool[e];
          if constexpr (!V1) {
            const float prj = (c.z - tau0) * fbins;
            if (prj >= 0.f) {
              const int bsel = min(__float2int_rd(prj), 7);
#pragma unroll
              for (int bb = 0; bb < 8; ++bb) cnt[bb] += (bb <= bsel) ? 1 : 0;
            }
          }
          e = c.next;
          ++ncand;
        }
        if constexpr (V1) {
          // first-generation start (adasplash_block_mask.py:167-175): no histogram, the bracket
          // [max - 1, max - n^(1-alpha)], n = 1 + row index (causal) or 1 + sequence length
          const float nkeys = 1.0f + (float)(p.causal ? row : len);
          hs.lo = tau0;
          hs.hi = tau0 + 1.0f - exp2f((1.0f - p.alpha) * log2f(nkeys));
          hs.t = 0.5f * (hs.lo + hs.hi);
        } else {
          exchange(kModeHist);
        }
      }
      // lists or full sweeps: one decision for the CTA, which the producer and the MMA warps
      // are waiting for
      ptx::bar_sync(3, kSolveRowThreads);
      full_sweeps = *pool_ovf != 0;
      ptx::mbar_arrive_warp(decide);
      if (third_sweep && full_sweeps) {
        // ---- the lists of scores within 1 of the maximum did not fit: lists of the scores above
        // the histogram's lower bound, from one more sweep ----
        if (threadIdx.x == 0) *pool_common = 0;
        head = kCandNil;
        ncand = 0;
        ptx::bar_sync(3, kSolveRowThreads);
        if (grp_on) sweep_tiles(std::integral_constant<int, kModeRecollect>{});
        ptx::bar_sync(3, kSolveRowThreads);
        full_sweeps = *pool_ovf2 != 0;
        ptx::mbar_arrive_warp(decide);
        recollected = true;
      }
      if (grp_on && !full_sweeps) {
        // ---- Halley steps and the final step on this thread's list ----
        // If the warp's share of the pool has room behind the entries in use, every thread
        // first copies its list there as one contiguous run: the steps then read independent
        // addresses instead of chasing links.
        int incl = ncand;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += up;
        }
        const int used = min(pool_used[warp], warp_pool);
        compact = !recollected && used + __shfl_sync(0xffffffffu, incl, 31) <= warp_pool;
        run0 = warp * warp_pool + used + incl - ncand;
        if (compact) {
          int dst = run0;
          for (int e = head, left = ncand; e != kCandNil && left > 0; --left) {
            const Cand c = pool[e];
            pool[dst++] = c;
            e = c.next;
          }
        }
        __syncwarp();
        for (int it = 0; it <= p.niter; ++it) {
          const bool last = it == p.niter;
          reset_stats();
          auto visit = [&](const Cand c) {
            if constexpr (V1) {
              // niter steps on sum u^(1/(alpha-1)) - 1; the last round only records the 64x64
              // sub-tiles that hold a score above the lower end of the bracket
              if (last) {
                const int kb = c.key >> kb_shift;
                if (c.z > hs.lo && row_ok) atomicOr(&s_bits[(grp * 2 + rb) * p.n_words + (kb >> 5)], 1u << (kb & 31));
              } else {
                const float d = c.z - hs.t;
                if (d > 0.f) {
                  if (powers.mode == 0) { a0 = fmaf(d, d, a0); a1 += d; a2 += 1.f; }
                  else {
                    const float gw = powers.g(d);
                    a0 += powers.p(d); a1 += gw; a2 += powers.mode == 2 ? gw / d : 0.f;
                  }
                }
              }
            } else {
              const float d = c.z - hs.t;
              if (d > 0.f) {
                a0 = fmaf(d, d, a0); a1 += d; a2 += 1.f;
                // the final step also records the 64x64 sub-tiles that hold a score above the
                // tau entering it (row block rb of this group, key block c.kb)
                const int kb = c.key >> kb_shift;
                if (last && row_ok) atomicOr(&s_bits[(grp * 2 + rb) * p.n_words + (kb >> 5)], 1u << (kb & 31));
              }
            }
          };
          if (compact) {
            for (int k = 0; k < ncand; ++k) visit(pool[run0 + k]);
          } else {
            for (int e = head, left = recollected ? 16 * warp_pool : warp_pool; e != kCandNil && left > 0; --left) {
              const Cand c = pool[e];
              visit(c);
              e = c.next;
            }
          }
          exchange(last ? kModeFinal : kModeHalley);
        }
      } else if (grp_on) {
        // ---- the pool overflowed: every remaining step sweeps S ----
        for (int sw = 2; sw < nsweeps; ++sw) {
          reset_stats();
          if (sw == nsweeps - 1) {
            sweep_tiles(std::integral_constant<int, kModeFinal>{});
            exchange(kModeFinal);
          } else {
            sweep_tiles(std::integral_constant<int, kModeHalley>{});
            exchange(kModeHalley);
          }
        }
      }
    }
    ptx::bar_sync(3, kSolveRowThreads);  // every atomicOr on s_bits is done
    if (!*cta_abort) {
      for (int t = threadIdx.x; t < 4 * p.n_words; t += kSolveRowThreads) {
        const int rbi = t / p.n_words, w = t % p.n_words;
        const int mrow = 4 * pr_idx + rbi;  // 64-row block index
        if (mrow < p.rows_padded && (rbi < 2 || b_on))
          p.bmask[((size_t)bh * p.rows_padded + mrow) * p.n_words + w] = (int32_t)s_bits[t];
      }
      if (!p.tau_given && grp_on && half == 0 && row_ok) p.taus[(size_t)bh * p.N + row] = hs.t;
    }
    if (p.sup_on && !p.tau_given) {
      // ---- the rows' supports, for the gather kernels ----
      // Entry = (key, u = z - tau) for every listed score above the final tau whose 64x64
      // tile is in the block mask just built (what the tile kernels would visit); one run per
      // row: the keys of the row's first thread (low halves of the key tiles), then the second's.
      // Above alpha = 1.5 the backward's key side decides "score above tau" from its own product
      // (K scaled and rounded, q raw), and the Jacobian weight does not vanish at the threshold:
      // pairs within the two products' largest possible difference below tau are exported as well
      // (with u <= 0: no weight on the query side).  |Q~ k - q K~| <= 2^-8 zscale |q| |k| for 16-bit
      // operands (unit roundoff 2^-9 each).
      // the same for every thread of the CTA: its lists held (those of the second or of the third sweep)
      const bool can = !full_sweeps && !wide && !*cta_abort;
      int* cnts = reinterpret_cast<int*>(xchg) + grp * (2 * 8 * 128);
      int* extra = reinterpret_cast<int*>(xchg) + 128;        // [0..7] entries of each 32-row quarter, [8] base (beside the counts)
      const uint32_t* my_bits = s_bits + (grp * 2 + rb) * p.n_words;
      auto in_support = [&](const Cand c) -> bool {
        const int kb = c.key >> 6;
        return c.z > hs.t - margin && ((my_bits[kb >> 5] >> (kb & 31)) & 1u);
      };
      auto for_each = [&](auto&& f) {
        if (!(grp_on && row_ok)) return;
        if (compact) {
          for (int k = 0; k < ncand; ++k) f(pool[run0 + k]);
        } else {
          for (int e = head, left = recollected ? 16 * warp_pool : warp_pool; e != kCandNil && left > 0; --left) {
            const Cand c = pool[e];
            f(c);
            e = c.next;
          }
        }
      };
      int n_mine = 0;
      if (can) for_each([&](const Cand c) { n_mine += in_support(c) ? 1 : 0; });
      cnts[half * (8 * 128) + r] = n_mine;
      ptx::bar_sync(3, kSolveRowThreads);
      const int n_other = cnts[(half ^ 1) * (8 * 128) + r];
      const int tot = n_mine + n_other;   // both threads of a row hold the row's count
      int incl = tot;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (half == 0 && lane == 31) extra[grp * 4 + wq] = incl;
      ptx::bar_sync(3, kSolveRowThreads);
      int before = 0, total = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const int t = extra[w];
        before += (w < grp * 4 + wq) ? t : 0;
        total += t;
      }
      if (threadIdx.x == 0) {
        // one reservation per CTA; a CTA that cannot export (or whose rows are too dense for the
        // backward's sort) hands its kv head to the tile kernels
        uint32_t base = 0xffffffffu;
        int why = sup::kWhyPool;
        if (can && total <= sup::kBlockCap) {
          base = atomicAdd(p.sup.cursor, (uint32_t)total);
          if (base > p.sup.cap || (uint32_t)total > p.sup.cap - base) { base = 0xffffffffu; why = sup::kWhyFull; }
        } else if (can) {
          why = sup::kWhyBlock;
        }
        if (base == 0xffffffffu) {
          atomicAdd(p.sup.dense + b * p.Hkv + kvh, 1);
          atomicAdd(p.sup.cursor + 4 + why, 1u);  // diagnostics: CTAs that could not export, by reason
        }
        extra[8] = (int)base;
      }
      ptx::bar_sync(3, kSolveRowThreads);
      const uint32_t base = (uint32_t)extra[8];
      if (base != 0xffffffffu) {
        const uint32_t row_first = base + (uint32_t)(before + incl - tot);
        if (grp_on && row_ok && half == 0) p.sup.rows[(size_t)bh * p.N + row] = make_uint2(row_first, (uint32_t)tot);
        uint2* dst = p.sup.entries + row_first + (half ? n_other : 0);
        for_each([&](const Cand c) {
          if (in_support(c)) *dst++ = make_uint2((uint32_t)c.key, __float_as_uint(c.z - hs.t));
        });
      }
    }
  }

  // ---------------- teardown ----------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*cta_abort && threadIdx.x == 0) {
    // give copies that may still be in flight a bounded time to land before the
    // shared memory of this CTA is handed to the next one
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 17) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kSolveTmemCols);
  }
}

}  // namespace sm100
}  // namespace ads
