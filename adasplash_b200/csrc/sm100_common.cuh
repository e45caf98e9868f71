// Shared pieces of the tcgen05 attention kernels: tile geometry, TMA tensor map
// construction, the abort protocol of the bounded waits.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "attn_simt.cuh"
#include "sm100_ptx.cuh"
#include "support.cuh"

namespace ads {
namespace sm100 {

constexpr int kBlockM = 128;       // rows of one MMA tile (two 64-row mask tiles)
constexpr int kBlockN = 128;       // keys of one MMA tile (two 64-key mask tiles)
constexpr int kPanelBytes = 128 * 128;  // one 128-row x 64-element (128 B) swizzled panel

// Error codes written to the device status word by a bounded wait that gave up.
enum : int {
  kStTimeoutProducer = 101,
  kStTimeoutMma = 102,
  kStTimeoutEpilogue = 103,
};

struct TcParams {
  const void* varlen; int varlen_is_i64;
  float* taus; int32_t* bmask; const int32_t* bmask_t;
  void* out; void* out2;
  const float* delta;
  void* dq; void* dk; void* dv;
  int B, Hq, Hkv, N, niter, bins;
  int n_words, rows_padded;
  int d_true;        // head dim of the tensors in global memory (<= the kernel's template D)
  int nq;            // number of 128-row tiles = ceil(N / 128)
  float sm_scale;
  float zscale;      // fp32((alpha-1) * sm_scale): the Q (or K) operand is scaled by it, so S = z
  float alpha;       // 1.5 or 2.0 on these kernels
  int causal;        // 0 = full attention (first-generation semantics only)
  int tau_given;
  int* status;       // device status word (0 = ok)
  const void* q_raw; // q in global memory (the kernels read it through TMA; the solver's export reads rows)
  int sup_on;        // the caller gave a row-support buffer (support.cuh)
  sup::View sup;
};


// One wait failed: publish the code globally (first failure wins) and tell the CTA.
__device__ __forceinline__ void raise_abort(volatile int* cta_abort, int* status, int code) {
  *cta_abort = code;
  atomicCAS(status, 0, code);
}

// Walks the 128-key tiles of one 128-row query tile whose block mask has any of
// its four 64x64 bits set.  flags: bit0 = (rows 0..63, keys 0..63), bit1 = (rows
// 0..63, keys 64..127), bit2 / bit3 = the same for rows 64..127.  Every role of
// a CTA runs the same scan, so they agree on the tile sequence without a list.
struct TileScan {
  const uint32_t* r0;
  const uint32_t* r1;
  int n_tiles, kt;
  uint32_t w0, w1;
  __device__ TileScan(const int32_t* bm_head, int qt, int n_tiles_, int rows_padded, int n_words)
      : n_tiles(n_tiles_), kt(-1), w0(0), w1(0) {
    r0 = reinterpret_cast<const uint32_t*>(bm_head) + (size_t)(2 * qt) * n_words;
    r1 = (2 * qt + 1) < rows_padded ? r0 + n_words : nullptr;
  }
  __device__ __forceinline__ bool next(int& kt_out, uint32_t& flags) {
    while (++kt < n_tiles) {
      const int kb = 2 * kt;
      if ((kb & 31) == 0 || kt == 0) {
        w0 = r0[kb >> 5];
        w1 = r1 ? r1[kb >> 5] : 0u;
      }
      const uint32_t f = ((w0 >> (kb & 31)) & 3u) | (((w1 >> (kb & 31)) & 3u) << 2);
      if (f) { kt_out = kt; flags = f; return true; }
    }
    return false;
  }
};

// 3-D tensor map over a (heads, N, D) 16-bit tensor: box = 64 elements x 128 rows
// x 1 head, 128-byte swizzle, out-of-range rows read as zero.
int make_tmap(CUtensorMap* map, const void* base, int heads, int N, int D, int box_rows);

}  // namespace sm100
}  // namespace ads
