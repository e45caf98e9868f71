// Launchers of the tensor-core attention kernels, shared by the translation units that
// instantiate them (attn_sm100.cu: the AdaSplash-2 path; attn_sm100_v1.cu: alpha = 2 and full
// attention for the first-generation semantics).
#pragma once
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "attn_sm100.cuh"
#include "sm100_bwd.cuh"
#include "sm100_fwd.cuh"
#include "sm100_solve.cuh"

namespace ads {
namespace sm100 {
namespace {

constexpr int kMaxDevices = 128;

// The dynamic shared-memory limit of a kernel is a per-device attribute: set it the first
// time a kernel is launched on a device, not before every launch.  (Keyed by the kernel's
// address: kernels with the same signature share one instantiation of this template.)
template <typename K>
int set_smem(K kernel, size_t bytes, const char* what) {
  static std::mutex mu;
  static std::unordered_map<const void*, size_t> done[kMaxDevices];  // kernel -> bytes granted on device d
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = -1;
  if (dev >= 0) {
    std::lock_guard<std::mutex> lock(mu);
    auto it = done[dev].find((const void*)kernel);
    if (it != done[dev].end() && it->second >= bytes) return ADS_OK;
  }
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) {
    set_error("%s: cudaFuncSetAttribute(%zu): %s", what, bytes, cudaGetErrorString(e));
    return ADS_ERR_CUDA;
  }
  if (dev >= 0) {
    std::lock_guard<std::mutex> lock(mu);
    done[dev][(const void*)kernel] = bytes;
  }
  return ADS_OK;
}

TcParams to_tc(const simt::Params& p, void* ws) {
  TcParams t;
  memset(&t, 0, sizeof(t));
  t.varlen = p.varlen; t.varlen_is_i64 = p.varlen_is_i64;
  t.taus = p.taus; t.bmask = p.bmask; t.bmask_t = p.bmask_t;
  t.out = p.out; t.out2 = p.out2; t.delta = p.delta;
  t.dq = p.dq; t.dk = p.dk; t.dv = p.dv;
  t.B = p.B; t.Hq = p.Hq; t.Hkv = p.Hkv; t.N = p.N; t.niter = p.niter; t.bins = p.bins;
  t.n_words = p.n_words; t.rows_padded = p.rows_padded;
  t.d_true = p.D;
  t.nq = (p.N + kBlockM - 1) / kBlockM;
  t.sm_scale = p.sm_scale;
  t.zscale = p.zscale;
  t.alpha = p.alpha;
  t.causal = p.causal;
  t.tau_given = p.tau_given;
  t.status = (int*)ws;
  t.q_raw = p.q;
  t.sup_on = p.support != nullptr;
  if (t.sup_on) t.sup = sup::view(p.support, nullptr, p.B, p.Hq, p.Hkv, p.N);
  return t;
}

template <typename T, int D, bool V1 = false>
int solve_t(const simt::Params& p, void* ws, size_t ws_bytes, cudaStream_t st) {
  CUtensorMap tmQ, tmK;
  if (int rc = make_tmap(&tmQ, p.q, p.B * p.Hq, p.N, p.D, kBlockM)) return rc;
  if (int rc = make_tmap(&tmK, p.k, p.B * p.Hkv, p.N, p.D, kBlockN)) return rc;
  TcParams t = to_tc(p, ws);
  size_t sm = SolveSmem<D>::bytes(p.n_words);
  if (sm > 227 * 1024) { set_error("sm100::solve: sequence too long for the bitmap staging (%zu B smem)", sm); return ADS_ERR_UNSUPPORTED; }
  if (int rc = set_smem(solve_kernel<T, D, V1>, sm, "sm100::solve")) return rc;
  long long ctas = (long long)((t.nq + 1) / 2) * p.B * p.Hq;  // one CTA per 256 query rows
  solve_kernel<T, D, V1><<<(unsigned)ctas, kSolveThreads, sm, st>>>(tmQ, tmK, t);
  return check_launch("sm100::solve");
}

template <typename T, int D, int AM = 0, bool CAUSAL = true>
int fwd_t(const simt::Params& p, void* ws, cudaStream_t st) {
  CUtensorMap tmQ, tmK, tmV;
  if (int rc = make_tmap(&tmQ, p.q, p.B * p.Hq, p.N, p.D, kBlockM)) return rc;
  if (int rc = make_tmap(&tmK, p.k, p.B * p.Hkv, p.N, p.D, kBlockN)) return rc;
  if (int rc = make_tmap(&tmV, p.v, p.B * p.Hkv, p.N, p.D, kBlockN)) return rc;
  TcParams t = to_tc(p, ws);
  size_t sm = FwdSmem<D>::bytes;
  if (int rc = set_smem(fwd_kernel<T, D, AM, CAUSAL>, sm, "sm100::fwd")) return rc;
  long long ctas = (long long)t.nq * p.B * p.Hq;
  fwd_kernel<T, D, AM, CAUSAL><<<(unsigned)ctas, kFwdThreads, sm, st>>>(tmQ, tmK, tmV, t);
  return check_launch("sm100::fwd");
}

template <typename T, int D, int AM = 0, bool CAUSAL = true>
int bwd_t(const simt::Params& p, void* ws, cudaStream_t st) {
  const int stages = p.bwd_stages ? p.bwd_stages : 0xF;
  // with a row-support buffer, heads the gather kernels own are skipped by every kernel here
  const int32_t* skip = p.support != nullptr ? sup::view(p.support, nullptr, p.B, p.Hq, p.Hkv, p.N).dense : nullptr;
  if (stages & ADS_BWD_DELTA) {
    long long rows = (long long)p.B * p.Hq * p.N;
    const long long per_block = (long long)(simt::kDeltaThreads / 32) * simt::delta_rows_per_warp<T>(p.D);
    unsigned grid = (unsigned)((rows + per_block - 1) / per_block);
    simt::bwd_delta_kernel<T><<<grid, simt::kDeltaThreads, 0, st>>>((const T*)p.out2_in, (const T*)p.dout, p.delta,
                                                    p.varlen, p.varlen_is_i64, p.B, p.Hq, p.N, p.D, skip, p.Hkv);
    if (int rc = check_launch("sm100::bwd_delta")) return rc;
  }
  if (stages & ADS_BWD_TRANSPOSE) {
    long long words = (long long)p.B * p.Hq * p.rows_padded * p.n_words;
    unsigned grid = (unsigned)((words + 255) / 256);
    simt::transpose_bitmap_kernel<<<grid, 256, 0, st>>>(p.bmask, p.bmask_t, p.B * p.Hq, p.rows_padded, p.n_words, skip,
                                                        p.Hq, p.Hkv);
    if (int rc = check_launch("sm100::transpose_bitmap")) return rc;
  }
  CUtensorMap tmQ, tmDO, tmK, tmV, tmQ64, tmDO64;
  if (int rc = make_tmap(&tmQ, p.q, p.B * p.Hq, p.N, p.D, kBlockM)) return rc;
  if (int rc = make_tmap(&tmDO, p.dout, p.B * p.Hq, p.N, p.D, kBlockM)) return rc;
  if (int rc = make_tmap(&tmK, p.k, p.B * p.Hkv, p.N, p.D, kBlockN)) return rc;
  if (int rc = make_tmap(&tmV, p.v, p.B * p.Hkv, p.N, p.D, kBlockN)) return rc;
  if (int rc = make_tmap(&tmQ64, p.q, p.B * p.Hq, p.N, p.D, kQBlock)) return rc;
  if (int rc = make_tmap(&tmDO64, p.dout, p.B * p.Hq, p.N, p.D, kQBlock)) return rc;
  TcParams t = to_tc(p, ws);
  if (stages & ADS_BWD_DQ) {
    size_t sm = DqSmem<D>::bytes;
    if (int rc = set_smem(bwd_dq_kernel<T, D, AM, CAUSAL>, sm, "sm100::bwd_dq")) return rc;
    long long ctas = (long long)t.nq * p.B * p.Hq;
    bwd_dq_kernel<T, D, AM, CAUSAL><<<(unsigned)ctas, kDqThreads, sm, st>>>(tmQ, tmDO, tmK, tmV, t);
    if (int rc = check_launch("sm100::bwd_dq")) return rc;
  }
  if (stages & ADS_BWD_DKV) {
    size_t sm = DkvSmem<D>::bytes;
    if (int rc = set_smem(bwd_dkv_kernel<T, D, AM, CAUSAL>, sm, "sm100::bwd_dkv")) return rc;
    long long ctas = (long long)t.nq * p.B * p.Hkv;
    bwd_dkv_kernel<T, D, AM, CAUSAL><<<(unsigned)ctas, kDkvThreads, sm, st>>>(tmK, tmV, tmQ64, tmDO64, t);
    return check_launch("sm100::bwd_dkv");
  }
  return ADS_OK;
}


// The wait limit and the "issue no streamed loads" flag live in constant memory, one copy per
// translation unit: this sets the copy of the including unit on the current device.
inline int set_wait_constants(long long max_wait_cycles, int withhold_loads) {
  if (max_wait_cycles <= 0) max_wait_cycles = ptx::kMaxWaitCycles;
  cudaError_t e = cudaMemcpyToSymbol(ptx::c_wait_limit, &max_wait_cycles, sizeof(max_wait_cycles));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(ptx::c_withhold_loads, &withhold_loads, sizeof(withhold_loads));
  if (e != cudaSuccess) { set_error("debug_waits: %s", cudaGetErrorString(e)); return ADS_ERR_CUDA; }
  return ADS_OK;
}

}  // namespace
}  // namespace sm100
}  // namespace ads
