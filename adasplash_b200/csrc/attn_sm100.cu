// Host side of the tensor-core attention kernels: TMA tensor maps, launches.
#include "sm100_launch.cuh"

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
// flag of the tensor-core kernels on the current device, in both translation units.
int debug_waits(long long max_wait_cycles, int withhold_loads) {
  if (int rc = set_wait_constants(max_wait_cycles, withhold_loads)) return rc;
  return v1::set_wait_constants_v1(max_wait_cycles, withhold_loads);
}

bool supported(const ads_attn_shape* s) {
  if (s->dtype != ADS_F16 && s->dtype != ADS_BF16) return false;
  if (s->D != 16 && s->D != 32 && s->D != 64 && s->D != 128) return false;
  if (s->N > 262144) return false;
  return true;
}

// Shapes the first-generation kernels cover: what `supported` covers, any alpha in (1, 2].
bool v1::supported(const ads_attn_shape* s) { return sm100::supported(s); }

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
