// Row supports: the element-sparse side of the attention path.
//
// An entmax-1.5 row has few non-zero probabilities (a handful to a few dozen out of thousands of
// keys), and the tensor-core solver ends its work holding every one of them in shared memory: its
// candidate lists are the scores within 1 of the row maximum, a superset of the support.  When a
// caller hands the solver a `support` buffer, each CTA writes, for its 256 query rows, the
// (key, score - tau) pairs of the support -- restricted to the 64x64 tiles of the block mask, so
// that the set is exactly what the tile kernels would visit -- as one contiguous run per row.
// The forward and the backward of those rows are then gathers over a few K / V / Q / dO rows per
// query instead of dense tiles (csrc/sparse_rows.cu).
//
// The choice between the two routes is made per (batch, kv head): a solver CTA that cannot
// export (its candidate pool overflowed twice and it fell back to sweeping S, or the entry array
// is full) bumps the head's `dense` counter; the tile kernels of a head return at once while the
// counter is zero, the gather kernels while it is not.
//
// The backward needs the same pairs by key as well (dK_j and dV_j sum over the rows that
// attend to key j).  Its row kernel leaves, for every 256-row block (the rows of one solver CTA),
// the block's entries sorted by (key, row) -- in the same slots of a second array -- and the key
// kernel finds the entries of its keys in each block through a table the row kernel leaves beside the run: no atomics, and a
// fixed summation order.
//
// The support buffer lives from the solve to the backward (it is saved with the forward's
// tensors), so it holds only what the solver writes; the backward's own arrays are scratch in
// that call's workspace.
//
// Layout of the support buffer (all offsets multiples of 256 bytes):
//   [0]      uint32 cursor: entries handed out so far (one atomicAdd per solver CTA);
//            words 4..7: solver CTAs that could not export, by reason (kWhy*)
//   [256]    int32 dense[B*Hkv]
//   kmax2    float [B*Hkv]: largest squared norm of a key row of the head (alpha > 1.5 only)
//   rows     uint2 [B*Hq*N]: (index of the row's first entry, number of entries)
//   entries  uint2 [cap]: (key index, fp32 bits of u = z - tau_final > 0)
// and of the backward's scratch (workspace + 256):
//   by_key   uint2 [cap]: (key << 8 | row inside its 256-row block, P^T | dS^T << 16 as 16-bit
//            values), each block's run sorted ascending; written by the backward
//   blocks   uint2 [B*Hq*ceil(N/256)]: (first entry of the block's run, its length)
//   kb_off   uint16 [B*Hq*ceil(N/256)][ceil(N/32)+1]: where the entries of each 32-key block
//            (the keys of one CTA of the key kernel) start inside a row block's sorted run (the
//            last one: the run's length)
#pragma once
#include <cstddef>
#include <cstdint>

#include <cuda_runtime.h>

namespace ads {
namespace sup {

constexpr int kEntriesPerRow = 32;  // capacity of the entry arrays, per query row of the problem
constexpr int kBlockRows = 256;     // rows whose entries the backward sorts together: one solver CTA
constexpr int kBlockCap = 8192;     // most entries such a block may hold (the solver checks)
constexpr int kTableKeys = 32;      // keys per entry of the key-block table = keys per CTA of the key kernel

// why a solver CTA did not export (counters in words 4..7 of the buffer)
enum : int {
  kWhyPool = 0,   // its candidate pool overflowed, in the third sweep as well (or a wait gave up)
  kWhyUnused = 1,
  kWhyBlock = 2,  // more than kBlockCap entries in its 256 rows
  kWhyFull = 3,   // the entry array is full
};

struct View {
  uint32_t* cursor;
  int32_t* dense;
  float* kmax2;
  uint2* rows;
  uint2* entries;
  uint2* by_key;
  uint2* blocks;
  uint16_t* kb_off;
  uint32_t cap;
};

__host__ __device__ inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

inline size_t bytes(int B, int Hq, int Hkv, int N) {
  const size_t rows = (size_t)B * Hq * N;
  return 256 + 2 * align256((size_t)B * Hkv * 4) + align256(rows * 8) + align256(rows * kEntriesPerRow * 8);
}

// Scratch of the backward on the gather route (by_key, blocks, kb_off).
inline size_t scratch_bytes(int B, int Hq, int Hkv, int N) {
  const size_t rows = (size_t)B * Hq * N;
  const size_t blocks = (size_t)B * Hq * ((N + kBlockRows - 1) / kBlockRows);
  const size_t nkb1 = (size_t)(N + kTableKeys - 1) / kTableKeys + 1;
  return align256(rows * kEntriesPerRow * 8) + align256(blocks * 8) + align256(blocks * nkb1 * 2);
}

// Bytes at the start of the buffer that the solver's launcher clears (cursor and counters).
inline size_t header_bytes(int B, int Hkv) { return 256 + 2 * align256((size_t)B * Hkv * 4); }

// `scratch` may be null outside the backward (the three arrays it holds are then unset).
inline View view(void* base, void* scratch, int B, int Hq, int Hkv, int N) {
  View v;
  uint8_t* p = (uint8_t*)base;
  const size_t rows = (size_t)B * Hq * N;
  v.cursor = (uint32_t*)p;
  v.dense = (int32_t*)(p + 256);
  v.kmax2 = (float*)(p + 256 + align256((size_t)B * Hkv * 4));
  v.rows = (uint2*)(p + 256 + 2 * align256((size_t)B * Hkv * 4));
  v.entries = (uint2*)((uint8_t*)v.rows + align256(rows * 8));
  v.by_key = nullptr; v.blocks = nullptr; v.kb_off = nullptr;
  if (scratch != nullptr) {
    const size_t blocks = (size_t)B * Hq * ((N + kBlockRows - 1) / kBlockRows);
    v.by_key = (uint2*)scratch;
    v.blocks = (uint2*)((uint8_t*)v.by_key + align256(rows * kEntriesPerRow * 8));
    v.kb_off = (uint16_t*)((uint8_t*)v.blocks + align256(blocks * 8));
  }
  const size_t cap = rows * kEntriesPerRow;
  v.cap = cap > 0xffffffffull ? 0xffffffffu : (uint32_t)cap;
  return v;
}

}  // namespace sup
}  // namespace ads
