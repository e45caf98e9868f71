// Host side of the tensor-core attention kernels: TMA tensor maps, launches.
#include "attn_sm100.cuh"

#include <mutex>
#include <unordered_map>

#include "sm100_bwd.cuh"
#include "sm100_fwd.cuh"
#include "sm100_solve.cuh"

namespace ads {
namespace sm100 {

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  });
  return fn;
}

constexpr size_t kStatusBytes = 256;

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
  t.tau_given = p.tau_given;
  t.status = (int*)ws;
  return t;
}

template <typename T, int D>
int solve_t(const simt::Params& p, void* ws, size_t ws_bytes, cudaStream_t st) {
  CUtensorMap tmQ, tmK;
  if (int rc = make_tmap(&tmQ, p.q, p.B * p.Hq, p.N, p.D, kBlockM)) return rc;
  if (int rc = make_tmap(&tmK, p.k, p.B * p.Hkv, p.N, p.D, kBlockN)) return rc;
  TcParams t = to_tc(p, ws);
  size_t sm = SolveSmem<D>::bytes(p.n_words);
  if (sm > 227 * 1024) { set_error("sm100::solve: sequence too long for the bitmap staging (%zu B smem)", sm); return ADS_ERR_UNSUPPORTED; }
  if (int rc = set_smem(solve_kernel<T, D>, sm, "sm100::solve")) return rc;
  long long ctas = (long long)((t.nq + 1) / 2) * p.B * p.Hq;  // one CTA per 256 query rows
  solve_kernel<T, D><<<(unsigned)ctas, kSolveThreads, sm, st>>>(tmQ, tmK, t);
  return check_launch("sm100::solve");
}

template <typename T, int D>
int fwd_t(const simt::Params& p, void* ws, cudaStream_t st) {
  CUtensorMap tmQ, tmK, tmV;
  if (int rc = make_tmap(&tmQ, p.q, p.B * p.Hq, p.N, p.D, kBlockM)) return rc;
  if (int rc = make_tmap(&tmK, p.k, p.B * p.Hkv, p.N, p.D, kBlockN)) return rc;
  if (int rc = make_tmap(&tmV, p.v, p.B * p.Hkv, p.N, p.D, kBlockN)) return rc;
  TcParams t = to_tc(p, ws);
  size_t sm = FwdSmem<D>::bytes;
  if (int rc = set_smem(fwd_kernel<T, D>, sm, "sm100::fwd")) return rc;
  long long ctas = (long long)t.nq * p.B * p.Hq;
  fwd_kernel<T, D><<<(unsigned)ctas, kFwdThreads, sm, st>>>(tmQ, tmK, tmV, t);
  return check_launch("sm100::fwd");
}

template <typename T>
int fwd_d(const simt::Params& p, void* ws, cudaStream_t st) {
  switch (p.D) {
    case 16: case 32:  // zero-padded to 64 columns by the TMA loads
    case 64: return fwd_t<T, 64>(p, ws, st);
    case 128: return fwd_t<T, 128>(p, ws, st);
  }
  set_error("sm100: head dim %d not built", p.D);
  return ADS_ERR_UNSUPPORTED;
}

template <typename T, int D>
int bwd_t(const simt::Params& p, void* ws, cudaStream_t st) {
  const int stages = p.bwd_stages ? p.bwd_stages : 0xF;
  if (stages & ADS_BWD_DELTA) {
    long long rows = (long long)p.B * p.Hq * p.N;
    const long long per_block = (long long)(simt::kDeltaThreads / 32) * simt::delta_rows_per_warp<T>(p.D);
    unsigned grid = (unsigned)((rows + per_block - 1) / per_block);
    simt::bwd_delta_kernel<T><<<grid, simt::kDeltaThreads, 0, st>>>((const T*)p.out2_in, (const T*)p.dout, p.delta,
                                                    p.varlen, p.varlen_is_i64, p.B, p.Hq, p.N, p.D);
    if (int rc = check_launch("sm100::bwd_delta")) return rc;
  }
  if (stages & ADS_BWD_TRANSPOSE) {
    long long words = (long long)p.B * p.Hq * p.rows_padded * p.n_words;
    unsigned grid = (unsigned)((words + 255) / 256);
    simt::transpose_bitmap_kernel<<<grid, 256, 0, st>>>(p.bmask, p.bmask_t, p.B * p.Hq, p.rows_padded, p.n_words);
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
    if (int rc = set_smem(bwd_dq_kernel<T, D>, sm, "sm100::bwd_dq")) return rc;
    long long ctas = (long long)t.nq * p.B * p.Hq;
    bwd_dq_kernel<T, D><<<(unsigned)ctas, kDqThreads, sm, st>>>(tmQ, tmDO, tmK, tmV, t);
    if (int rc = check_launch("sm100::bwd_dq")) return rc;
  }
  if (stages & ADS_BWD_DKV) {
    size_t sm = DkvSmem<D>::bytes;
    if (int rc = set_smem(bwd_dkv_kernel<T, D>, sm, "sm100::bwd_dkv")) return rc;
    long long ctas = (long long)t.nq * p.B * p.Hkv;
    bwd_dkv_kernel<T, D><<<(unsigned)ctas, kDkvThreads, sm, st>>>(tmK, tmV, tmQ64, tmDO64, t);
    return check_launch("sm100::bwd_dkv");
  }
  return ADS_OK;
}

template <typename T>
int bwd_d(const simt::Params& p, void* ws, cudaStream_t st) {
  switch (p.D) {
    case 16: case 32:
    case 64: return bwd_t<T, 64>(p, ws, st);
    case 128: return bwd_t<T, 128>(p, ws, st);
  }
  set_error("sm100: head dim %d not built", p.D);
  return ADS_ERR_UNSUPPORTED;
}

template <typename T>
int solve_d(const simt::Params& p, void* ws, size_t ws_bytes, cudaStream_t st) {
  switch (p.D) {
    case 16: case 32:
    case 64: return solve_t<T, 64>(p, ws, ws_bytes, st);
    case 128: return solve_t<T, 128>(p, ws, ws_bytes, st);
  }
  set_error("sm100: head dim %d not built", p.D);
  return ADS_ERR_UNSUPPORTED;
}

}  // namespace

// Encoded tensor maps are a pure function of (base, heads, N, D, box rows): keep the last few
// hundred so that repeated calls on the same tensors (training steps, benchmarks, graph replays)
// skip the driver call.  A map holds no reference to the memory, so a stale entry is harmless: the
// same key always encodes the same map.
struct TmapKey {
  const void* base; int heads, N, D, box_rows;
  bool operator==(const TmapKey& o) const {
    return base == o.base && heads == o.heads && N == o.N && D == o.D && box_rows == o.box_rows;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = std::hash<const void*>()(k.base);
    for (int v : {k.heads, k.N, k.D, k.box_rows}) h = h * 1000003u ^ std::hash<int>()(v);
    return h;
  }
};

int make_tmap(CUtensorMap* map, const void* base, int heads, int N, int D, int box_rows) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  const TmapKey key{base, heads, N, D, box_rows};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *map = it->second; return ADS_OK; }
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) { set_error("cuTensorMapEncodeTiled not available from the driver"); return ADS_ERR_CUDA; }
  if (((uintptr_t)base & 15) != 0) { set_error("tensor base %p is not 16-byte aligned", base); return ADS_ERR_BAD_ARG; }
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)heads};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)N * D * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return ADS_ERR_CUDA; }
  {
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() >= 512) cache.clear();
    cache.emplace(key, *map);
  }
  return ADS_OK;
}

// Test hook behind adasplash2_debug_waits: wait limit (SM clocks) and "issue no streamed loads"
// flag of the tensor-core kernels on the current device.
int debug_waits(long long max_wait_cycles, int withhold_loads) {
  if (max_wait_cycles <= 0) max_wait_cycles = ptx::kMaxWaitCycles;
  cudaError_t e = cudaMemcpyToSymbol(ptx::c_wait_limit, &max_wait_cycles, sizeof(max_wait_cycles));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(ptx::c_withhold_loads, &withhold_loads, sizeof(withhold_loads));
  if (e != cudaSuccess) { set_error("debug_waits: %s", cudaGetErrorString(e)); return ADS_ERR_CUDA; }
  return ADS_OK;
}

bool supported(const ads_attn_shape* s) {
  if (s->dtype != ADS_F16 && s->dtype != ADS_BF16) return false;
  if (s->D != 16 && s->D != 32 && s->D != 64 && s->D != 128) return false;
  if (s->N > 262144) return false;
  return true;
}

size_t workspace_bytes(const ads_attn_shape*) { return kStatusBytes; }
size_t min_workspace_bytes() { return kStatusBytes; }

int solve(const simt::Params& p, int dtype, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (dtype == ADS_F16) return solve_d<__half>(p, ws, ws_bytes, st);
  return solve_d<__nv_bfloat16>(p, ws, ws_bytes, st);
}

int fwd(const simt::Params& p, int dtype, void* ws, cudaStream_t st) {
  if (dtype == ADS_F16) return fwd_d<__half>(p, ws, st);
  return fwd_d<__nv_bfloat16>(p, ws, st);
}

int bwd(const simt::Params& p, int dtype, void* ws, cudaStream_t st) {
  if (dtype == ADS_F16) return bwd_d<__half>(p, ws, st);
  return bwd_d<__nv_bfloat16>(p, ws, st);
}

}  // namespace sm100
}  // namespace ads
