/*
 * C ABI of the B200 (sm_100a) sparse entmax attention library.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream
 * (`void* stream` is a `cudaStream_t`), launches asynchronously on that stream,
 * never synchronises the host, and -- unless its comment says otherwise --
 * never allocates or frees memory: the caller owns every buffer, including
 * scratch.  Return value: 0 on success, otherwise an `ads_status` code; the
 * message of the last failure on the calling thread is returned by
 * `adasplash_last_error_string()`.
 *
 * The comments cite the interface of deep-spin/adasplash that each entry point
 * replaces (file:line inside that project).
 */
#ifndef ADASPLASH_B200_H_
#define ADASPLASH_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { ADS_F32 = 0, ADS_F16 = 1, ADS_BF16 = 2 } ads_dtype;

typedef enum {
  ADS_OK = 0,
  ADS_ERR_BAD_ARG = 1,      /* null pointer, negative size, bad enum            */
  ADS_ERR_UNSUPPORTED = 2,  /* head dim / dtype / size outside the built range  */
  ADS_ERR_WORKSPACE = 3,    /* scratch buffer missing or too small              */
  ADS_ERR_CUDA = 4,         /* a CUDA runtime / driver call failed              */
  ADS_ERR_TIMEOUT = 5       /* a bounded device-side wait gave up (status word) */
} ads_status;

/* Kernel family selection for the attention entry points. */
enum {
  ADS_PATH_AUTO = 0,   /* tcgen05/TMA kernels when dtype/head-dim allow, else SIMT */
  ADS_PATH_SIMT = 1,   /* fp32-accumulating CUDA-core kernels (any dtype, any D)   */
  ADS_PATH_TCGEN05 = 2 /* tensor-core kernels only; error if not applicable        */
};

/* alpha = 1.5 with the causal mask is the AdaSplash-2 path (adasplash/adasplash_v2.py).
 * Any other alpha in (1, 2] and / or full attention are the semantics of the reference's
 * first-generation kernels (adasplash/adasplash_block_mask.py:938-1232: `sparse_attn(q, k, v,
 * alpha, is_causal, varlen, niter)`, no grouped-query heads): a Halley / bisection solver on
 * [max-1, max-n^(1-alpha)], block mask at the lower end of the final bracket.  Both run on the
 * tensor-core kernels for 16-bit inputs with head dim <= 128, else on the CUDA-core kernels.
 *
 * Shape of one attention problem.  q is (B,Hq,N,D) contiguous, k and v are
 * (B,Hkv,N,D) contiguous, Hq % Hkv == 0, D in {16,32,64,128,256}, N >= 64
 * (adasplash/adasplash_v2.py:1245-1276).  `varlen` is NULL or B lengths
 * (int32, or int64 when varlen_is_i64 != 0) on the device. */
typedef struct {
  int32_t B, Hq, Hkv, N, D;
  int32_t dtype;          /* ads_dtype of q,k,v,out,dout,dq,dk,dv            */
  int32_t niter;          /* Halley refinements after the histogram start     */
  int32_t varlen_is_i64;
  int32_t path;           /* ADS_PATH_*                                       */
  int32_t bwd_stages;     /* 0 = whole backward; else a mask of ADS_BWD_* (timing aid) */
  float alpha;            /* entmax alpha in (1, 2]; 0 means 1.5                        */
  int32_t non_causal;     /* 0 = causal mask (key <= query), 1 = full attention         */
} ads_attn_shape;

/* Kernels of adasplash2_bwd, for `bwd_stages` (measurement only: a partial
 * backward leaves the skipped outputs untouched). */
enum { ADS_BWD_DELTA = 1, ADS_BWD_TRANSPOSE = 2, ADS_BWD_DQ = 4, ADS_BWD_DKV = 8 };

/* Row-wise entmax forward over the last dimension of a contiguous
 * (rows, cols) matrix.  Replaces `_entmax_triton.forward` / `_fwd_entmax`
 * (adasplash/triton_entmax_v2.py:361-536, :623-664).  alpha > 1; the caller
 * applies the wrapper rule of triton_entmax_v2.py:713-715 (alpha not in
 * {1.5, 2} => no histogram, n_iter >= 10).  `tau_out` may be NULL; if not, it
 * receives the final threshold of each row (fp32, rows entries). */
int adasplash_entmax_fwd(const void* x, void* y, float* tau_out, int64_t rows, int64_t cols,
                         float alpha, int32_t n_iter, int32_t use_histogram, int32_t fast_math,
                         int32_t dtype, void* stream);

/* Row-wise entmax backward: dx = u*(dy - sum(u dy)/sum(u)), u = y^(2-alpha) on
 * the support.  Replaces `_bwd_entmax` (adasplash/triton_entmax_v2.py:539-617). */
int adasplash_entmax_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t cols,
                         float alpha, int32_t fast_math, int32_t dtype, void* stream);

/* Bytes of scratch the attention entry points need for `shape` (256-byte aligned base
 * expected).  The first 256 bytes (the status word of the bounded device waits) are all that
 * adasplash2_solve, _mask_from_tau and _fwd use, and all that adasplash2_bwd uses without a
 * support buffer; with one, the backward keeps its key-sorted copy of the supports behind
 * them.  A workspace is only live during the call it is passed to. */
size_t adasplash2_workspace_bytes(const ads_attn_shape* shape);

/* Row supports (optional; no counterpart in the reference, whose kernels are block-sparse only).
 * An entmax row has few non-zero probabilities, and the tensor-core solver ends up holding all of
 * them on chip.  Given a `support` buffer of this many bytes (256-byte aligned), adasplash2_solve
 * also writes each query row's (key, score - tau) pairs -- exactly the entries the tile kernels
 * would visit under the block mask -- and adasplash2_fwd / adasplash2_bwd, handed the same
 * buffer, compute those rows as gathers over a few K / V / Q / dO rows instead of dense tiles.
 * The route is chosen per (batch, kv head) on the device: heads whose rows are too dense for the
 * solver's lists, or that find the buffer full, take the tile kernels as if no buffer had been
 * given.  Returns 0 for shapes without this route (CUDA-core path, head dims other than 64 / 128,
 * more than 65536 keys); NULL / 0 may always be passed instead of a buffer.  The buffer belongs
 * to one solve: pass it to the forward and backward of the same problem, unchanged. */
size_t adasplash2_support_bytes(const ads_attn_shape* shape);

/* Number of int32 words of one bitmap tensor (B,Hq,rows_padded,n_words) and its
 * two inner extents, in the layout of adasplash/adasplash_v2.py:1345-1350:
 * rows_padded = max(32, ceil32(ceil(N/64))), n_words = ceil(ceil(N/64)/32);
 * bit j of word w of row m <=> the 64x64 tile (q-tile m, k-tile 32w+j). */
int64_t adasplash2_bitmap_words(const ads_attn_shape* shape, int32_t* rows_padded,
                                int32_t* n_words);

/* Threshold solver + block-mask builder.  Replaces the launches of `_get_tau`,
 * `_get_tau_v2` and `_get_tau_v3` (adasplash/adasplash_v2.py:1287-1379).
 * Writes taus (B,Hq,N) fp32 and bmask (int32, zero-filled by this call).  The
 * bitmap is taken at the tau entering the last refinement sweep, as the
 * reference does (adasplash_v2.py:618-681). */
int adasplash2_solve(const void* q, const void* k, const void* varlen, float* taus,
                     int32_t* bmask, const ads_attn_shape* shape, void* workspace,
                     size_t workspace_bytes, void* support, size_t support_bytes, void* stream);

/* Block-mask builder alone: bit(m,n) = any(z > taus) on each valid 64x64 tile,
 * for thresholds supplied by the caller.  No reference entry point does only
 * this (it is the bitmap half of `_get_tau_v3`, adasplash_v2.py:618-674); it
 * exists so that bitmaps can be compared for identical fp32 taus. */
int adasplash2_mask_from_tau(const void* q, const void* k, const void* varlen,
                             const float* taus, int32_t* bmask, const ads_attn_shape* shape,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Sparse forward.  Replaces `_get_output` (adasplash/adasplash_v2.py:696-835,
 * launch at :1391-1419).  out and out2 have q's shape and dtype; rows at or
 * beyond varlen[b] are written as zero by this call. */
int adasplash2_fwd(const void* q, const void* k, const void* v, const void* varlen,
                   const float* taus, const int32_t* bmask, void* out, void* out2,
                   const ads_attn_shape* shape, void* workspace, size_t workspace_bytes,
                   void* support, size_t support_bytes, void* stream);

/* Backward.  Replaces `_bwd_preprocess`, `_bwd_q_kernel`, `transpose_bmask` and
 * `_bwd_kv_kernel` (adasplash/adasplash_v2.py:1441-1564).  `delta` (B,Hq,N fp32)
 * and `bmask_t` (same extent as bmask) are caller-owned scratch outputs.
 * dq (B,Hq,N,D), dk, dv (B,Hkv,N,D) in the input dtype; padded rows are zero.
 * dout and out2 must be 16-byte aligned. */
int adasplash2_bwd(const void* q, const void* k, const void* v, const void* dout,
                   const void* out2, const void* varlen, const float* taus,
                   const int32_t* bmask, int32_t* bmask_t, float* delta, void* dq, void* dk,
                   void* dv, const ads_attn_shape* shape, void* workspace,
                   size_t workspace_bytes, void* support, size_t support_bytes, void* stream);

/* Backward for callers that cannot allocate.  It has no counterpart in the
 * reference (whose host code allocates freely through torch).  It exists for
 * hosts that are handed their device pointers and may not call an allocator on
 * the way: framework plugins with a fixed tensor list, code that runs inside a
 * region where allocation is forbidden, processes with a pre-set memory budget.
 * Same result as adasplash2_bwd, but the three scratch buffers (status word,
 * delta, transposed block mask) are carved out of an array of
 * ADS_STATIC_SCRATCH_BYTES that is part of the library image on every GPU that
 * loads it.  The call makes no cudaMalloc / cudaFree and uses no allocating
 * library routine.  Limits and rules:
 *  - 256 + 4*B*Hq*N + 4*bitmap_words bytes (each rounded up to 256) must fit in
 *    ADS_STATIC_SCRATCH_BYTES, otherwise ADS_ERR_WORKSPACE is returned and
 *    nothing is launched;
 *  - the first call on each device looks up the array's device address (with
 *    that device current) and caches it; make that first call outside any
 *    stream capture;
 *  - all calls on one device share the array and it keeps the previous call's
 *    contents (the backward rewrites every word before reading it); two calls
 *    that overlap on the GPU -- different streams, or graphs replayed
 *    concurrently -- race on it.  Serialise them;
 *  - shape->bwd_stages must be 0 (ADS_ERR_BAD_ARG otherwise): a partial backward would read
 *    what an earlier call left in the array;
 *  - adasplash2_check_status(NULL, stream) reads the status word of this array;
 *  - the cached address lives as long as the device's primary context. */
#define ADS_STATIC_SCRATCH_BYTES (8u << 20)
int adasplash2_bwd_static(const void* q, const void* k, const void* v, const void* dout,
                          const void* out2, const void* varlen, const float* taus,
                          const int32_t* bmask, void* dq, void* dk, void* dv,
                          const ads_attn_shape* shape, void* stream);

/* Debug aid, the one entry point that synchronises: waits for `stream`, reads
 * the status word that the tensor-core kernels keep at the start of `workspace`
 * (NULL = the built-in scratch of adasplash2_bwd_static on the current device)
 * and returns ADS_ERR_TIMEOUT if a bounded device-side wait gave up (the code is
 * in the error string), ADS_OK otherwise.  No counterpart in the reference. */
int adasplash2_check_status(const void* workspace, void* stream);

/* Test hook for the give-up path of the bounded waits (no counterpart in the reference).
 * Sets, on the current device, the wait limit of the tensor-core kernels in SM clocks
 * (<= 0 restores the default 2^28) and whether their producer warps withhold the streamed
 * TMA loads, so that a wait runs into the limit: the kernel then records its code in the
 * status word, drains, frees its TMEM and returns; adasplash2_check_status reports
 * ADS_ERR_TIMEOUT.  Synchronous (two small copies to constant memory); call it with no
 * kernel of this library in flight, and restore (0, 0) afterwards. */
int adasplash2_debug_waits(int64_t max_wait_cycles, int32_t withhold_loads);

/* Which kernel family `ADS_PATH_AUTO` resolves to for `shape`
 * (ADS_PATH_SIMT or ADS_PATH_TCGEN05). */
int adasplash2_resolved_path(const ads_attn_shape* shape);

/* Number of kernels launched by this library since it was loaded (all threads). */
int64_t adasplash_launch_count(void);

const char* adasplash_last_error_string(void);

#ifdef __cplusplus
}
#endif
#endif /* ADASPLASH_B200_H_ */
