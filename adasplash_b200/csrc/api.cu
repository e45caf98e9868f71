// extern "C" entry points of the attention path: argument checks, kernel
// family selection, launches.  No allocation, no host synchronisation.
#include <cmath>
#include <cstdarg>
#include <cstring>

#include "attn_simt.cuh"
#include "attn_sm100.cuh"
#include "sparse_rows.cuh"

namespace ads {

static thread_local char g_err[512] = "";
std::atomic<long long> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

namespace {

struct Geometry {
  int nb, n_words, rows_padded;
};

Geometry geometry(int N) {
  Geometry g;
  g.nb = (N + kTile - 1) / kTile;
  g.n_words = (g.nb + 31) / 32;
  g.rows_padded = ((g.nb + 31) / 32) * 32;
  if (g.rows_padded < 32) g.rows_padded = 32;
  return g;
}

int check_shape(const ads_attn_shape* s, const char* who) {
  if (s == nullptr) { set_error("%s: null shape", who); return ADS_ERR_BAD_ARG; }
  // AdaSplash-2 requires N >= 64 (adasplash_v2.py:1265); the first-generation kernels take any N
  const bool v2_shape = (s->alpha == 0.f || s->alpha == 1.5f) && s->non_causal == 0;
  if (s->B < 1 || s->Hq < 1 || s->Hkv < 1 || s->N < (v2_shape ? kTile : 1) || s->niter < 0) {
    set_error("%s: bad shape B=%d Hq=%d Hkv=%d N=%d niter=%d (causal alpha = 1.5 needs N >= 64)", who, s->B,
              s->Hq, s->Hkv, s->N, s->niter);
    return ADS_ERR_BAD_ARG;
  }
  if (s->Hq % s->Hkv != 0) { set_error("%s: Hq=%d not a multiple of Hkv=%d", who, s->Hq, s->Hkv); return ADS_ERR_BAD_ARG; }
  if (s->D != 16 && s->D != 32 && s->D != 64 && s->D != 128 && s->D != 256) {
    set_error("%s: head dim %d not in {16,32,64,128,256}", who, s->D);
    return ADS_ERR_UNSUPPORTED;
  }
  if (s->dtype != ADS_F32 && s->dtype != ADS_F16 && s->dtype != ADS_BF16) {
    set_error("%s: unknown dtype %d", who, s->dtype);
    return ADS_ERR_BAD_ARG;
  }
  if (s->B > 65535 || s->Hq > 65535) { set_error("%s: B/Hq above 65535", who); return ADS_ERR_UNSUPPORTED; }
  if (s->alpha != 0.f && !(s->alpha > 1.0f && s->alpha <= 2.0f)) {
    set_error("%s: alpha=%f outside (1, 2]", who, s->alpha);
    return ADS_ERR_BAD_ARG;
  }
  if (s->path != ADS_PATH_AUTO && s->path != ADS_PATH_SIMT && s->path != ADS_PATH_TCGEN05) {
    set_error("%s: unknown path %d", who, s->path);
    return ADS_ERR_BAD_ARG;
  }
  return ADS_OK;
}

// causal alpha = 1.5: the AdaSplash-2 kernels; anything else: the first-generation semantics
bool is_v2(const ads_attn_shape* s) { return (s->alpha == 0.f || s->alpha == 1.5f) && s->non_causal == 0; }

int resolve_path(const ads_attn_shape* s, const char* who, int* path) {
  // tensor cores: 16-bit inputs, head dim up to 128 (any alpha, causal or full attention)
  bool tc_ok = is_v2(s) ? sm100::supported(s) : sm100::v1::supported(s);
  if (s->path == ADS_PATH_TCGEN05 && !tc_ok) {
    set_error("%s: tcgen05 path needs fp16/bf16 inputs and a head dim it was built for (got dtype=%d D=%d)",
              who, s->dtype, s->D);
    return ADS_ERR_UNSUPPORTED;
  }
  *path = (s->path == ADS_PATH_SIMT || !tc_ok) ? ADS_PATH_SIMT : ADS_PATH_TCGEN05;
  return ADS_OK;
}

simt::Params make_params(const ads_attn_shape* s) {
  simt::Params p;
  memset(&p, 0, sizeof(p));
  Geometry g = geometry(s->N);
  p.B = s->B; p.Hq = s->Hq; p.Hkv = s->Hkv; p.N = s->N; p.D = s->D;
  p.niter = s->niter;
  p.bins = select_bins(s->N);
  p.nb = g.nb; p.n_words = g.n_words; p.rows_padded = g.rows_padded;
  p.sm_scale = (float)(1.0 / std::sqrt((double)s->D));
  p.varlen_is_i64 = s->varlen_is_i64;
  p.bwd_stages = s->bwd_stages;
  p.alpha = s->alpha == 0.f ? 1.5f : s->alpha;
  p.causal = s->non_causal ? 0 : 1;
  p.zscale = (p.alpha - 1.0f) * p.sm_scale;
  return p;
}

// The first word of the workspace is the status word of the tensor-core kernels'
// bounded waits.  Every entry point clears it, whichever kernel family runs, so
// that adasplash2_check_status never reads an uninitialised value.
int clear_status(void* ws, size_t ws_bytes, cudaStream_t st, const char* who) {
  if (ws == nullptr || ws_bytes < sizeof(int)) return ADS_OK;
  cudaError_t e = cudaMemsetAsync(ws, 0, sizeof(int), st);
  if (e != cudaSuccess) { set_error("%s: memset status: %s", who, cudaGetErrorString(e)); return ADS_ERR_CUDA; }
  return ADS_OK;
}

// The row-support buffer takes part only on the tensor-core path of shapes the gather kernels
// cover; anywhere else it is ignored.  A buffer that is too small is an error.
int resolve_support(const ads_attn_shape* s, int path, void* support, size_t support_bytes, const char* who,
                    void** out) {
  *out = nullptr;
  if (support == nullptr || path != ADS_PATH_TCGEN05 || !sparse::supported(s)) return ADS_OK;
  const size_t need = sparse::support_bytes(s);
  if (support_bytes < need) {
    set_error("%s: support buffer too small (%zu < %zu)", who, support_bytes, need);
    return ADS_ERR_WORKSPACE;
  }
  if (((uintptr_t)support & 255) != 0) { set_error("%s: support buffer must be 256-byte aligned", who); return ADS_ERR_BAD_ARG; }
  *out = support;
  return ADS_OK;
}

template <typename F32, typename F16, typename BF16>
int by_dtype(int dtype, F32 f32, F16 f16, BF16 bf16) {
  switch (dtype) {
    case ADS_F32: return f32();
    case ADS_F16: return f16();
    default: return bf16();
  }
}

}  // namespace
}  // namespace ads

using namespace ads;

extern "C" const char* adasplash_last_error_string(void) { return g_err; }
extern "C" int64_t adasplash_launch_count(void) { return g_launches.load(); }

extern "C" int64_t adasplash2_bitmap_words(const ads_attn_shape* shape, int32_t* rows_padded,
                                           int32_t* n_words) {
  if (shape == nullptr || shape->N < 1) return -1;
  Geometry g = geometry(shape->N);
  if (rows_padded) *rows_padded = g.rows_padded;
  if (n_words) *n_words = g.n_words;
  return (int64_t)shape->B * shape->Hq * g.rows_padded * g.n_words;
}

extern "C" int adasplash2_resolved_path(const ads_attn_shape* shape) {
  if (check_shape(shape, "resolved_path")) return -1;
  int path;
  if (resolve_path(shape, "resolved_path", &path)) return -1;
  return path;
}

extern "C" size_t adasplash2_support_bytes(const ads_attn_shape* shape) {
  if (check_shape(shape, "support_bytes")) return 0;
  int path;
  if (resolve_path(shape, "support_bytes", &path)) return 0;
  if (path != ADS_PATH_TCGEN05 || !sparse::supported(shape)) return 0;
  return sparse::support_bytes(shape);
}

extern "C" size_t adasplash2_workspace_bytes(const ads_attn_shape* shape) {
  if (check_shape(shape, "workspace_bytes")) return 0;
  int path;
  if (resolve_path(shape, "workspace_bytes", &path)) return 0;
  if (path == ADS_PATH_TCGEN05) {
    // the status word, and for shapes with a gather route the backward's scratch behind it
    return sm100::workspace_bytes(shape) + (sparse::supported(shape) ? sparse::bwd_scratch_bytes(shape) : 0);
  }
  return 256;  // the CUDA-core kernels need no scratch; keep the pointer non-null
}

static int solve_common(const void* q, const void* k, const void* varlen, float* taus,
                        int32_t* bmask, const ads_attn_shape* s, void* ws, size_t ws_bytes,
                        void* support, size_t support_bytes, void* stream, int tau_given, const char* who) {
  if (int rc = check_shape(s, who)) return rc;
  if (!q || !k || !taus || !bmask) { set_error("%s: null pointer", who); return ADS_ERR_BAD_ARG; }
  int path;
  if (int rc = resolve_path(s, who, &path)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  simt::Params p = make_params(s);
  p.q = q; p.k = k; p.varlen = varlen; p.taus = taus; p.bmask = bmask; p.tau_given = tau_given;
  if (int rc = resolve_support(s, path, support, support_bytes, who, &p.support)) return rc;
  size_t bm_bytes = (size_t)s->B * s->Hq * p.rows_padded * p.n_words * sizeof(int32_t);
  cudaError_t e = cudaMemsetAsync(bmask, 0, bm_bytes, st);
  if (e != cudaSuccess) { set_error("%s: memset bitmap: %s", who, cudaGetErrorString(e)); return ADS_ERR_CUDA; }
  if (int rc = clear_status(ws, ws_bytes, st, who)) return rc;
  if (path == ADS_PATH_TCGEN05) {
    if (ws == nullptr || ws_bytes < sm100::min_workspace_bytes()) {
      set_error("%s: workspace too small (%zu < %zu)", who, ws_bytes, sm100::min_workspace_bytes());
      return ADS_ERR_WORKSPACE;
    }
    if (p.support != nullptr) {
      if (int rc = sparse::clear_header(p, st)) return rc;
      if (p.alpha > 1.5f) {
        if (int rc = sparse::key_norms(p, s->dtype, st)) return rc;
      }
    }
    return is_v2(s) ? sm100::solve(p, s->dtype, ws, ws_bytes, st) : sm100::v1::solve(p, s->dtype, ws, ws_bytes, st);
  }
  return by_dtype(
      s->dtype, [&] { return simt::launch_solve<float>(p, st); },
      [&] { return simt::launch_solve<__half>(p, st); },
      [&] { return simt::launch_solve<__nv_bfloat16>(p, st); });
}

extern "C" int adasplash2_solve(const void* q, const void* k, const void* varlen, float* taus,
                                int32_t* bmask, const ads_attn_shape* shape, void* workspace,
                                size_t workspace_bytes, void* support, size_t support_bytes,
                                void* stream) {
  return solve_common(q, k, varlen, taus, bmask, shape, workspace, workspace_bytes, support,
                      support_bytes, stream, 0, "adasplash2_solve");
}

extern "C" int adasplash2_mask_from_tau(const void* q, const void* k, const void* varlen,
                                        const float* taus, int32_t* bmask,
                                        const ads_attn_shape* shape, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  return solve_common(q, k, varlen, const_cast<float*>(taus), bmask, shape, workspace,
                      workspace_bytes, nullptr, 0, stream, 1, "adasplash2_mask_from_tau");
}

extern "C" int adasplash2_fwd(const void* q, const void* k, const void* v, const void* varlen,
                              const float* taus, const int32_t* bmask, void* out, void* out2,
                              const ads_attn_shape* s, void* ws, size_t ws_bytes, void* support,
                              size_t support_bytes, void* stream) {
  const char* who = "adasplash2_fwd";
  if (int rc = check_shape(s, who)) return rc;
  if (!q || !k || !v || !taus || !bmask || !out || !out2) { set_error("%s: null pointer", who); return ADS_ERR_BAD_ARG; }
  int path;
  if (int rc = resolve_path(s, who, &path)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  simt::Params p = make_params(s);
  p.q = q; p.k = k; p.v = v; p.varlen = varlen;
  p.taus = const_cast<float*>(taus); p.bmask = const_cast<int32_t*>(bmask);
  p.out = out; p.out2 = out2;
  if (int rc = resolve_support(s, path, support, support_bytes, who, &p.support)) return rc;
  if (int rc = clear_status(ws, ws_bytes, st, who)) return rc;
  if (path == ADS_PATH_TCGEN05) {
    if (ws == nullptr || ws_bytes < sm100::min_workspace_bytes()) {
      set_error("%s: workspace too small (%zu < %zu)", who, ws_bytes, sm100::min_workspace_bytes());
      return ADS_ERR_WORKSPACE;
    }
    if (p.support != nullptr) {  // heads whose supports were exported: a gather; the others: tiles
      if (int rc = sparse::fwd(p, s->dtype, st)) return rc;
    }
    return is_v2(s) ? sm100::fwd(p, s->dtype, ws, st) : sm100::v1::fwd(p, s->dtype, ws, st);
  }
  return by_dtype(
      s->dtype, [&] { return simt::launch_fwd<float>(p, st); },
      [&] { return simt::launch_fwd<__half>(p, st); },
      [&] { return simt::launch_fwd<__nv_bfloat16>(p, st); });
}

extern "C" int adasplash2_bwd(const void* q, const void* k, const void* v, const void* dout,
                              const void* out2, const void* varlen, const float* taus,
                              const int32_t* bmask, int32_t* bmask_t, float* delta, void* dq,
                              void* dk, void* dv, const ads_attn_shape* s, void* ws,
                              size_t ws_bytes, void* support, size_t support_bytes, void* stream) {
  const char* who = "adasplash2_bwd";
  if (int rc = check_shape(s, who)) return rc;
  if (!q || !k || !v || !dout || !out2 || !taus || !bmask || !bmask_t || !delta || !dq || !dk || !dv) {
    set_error("%s: null pointer", who);
    return ADS_ERR_BAD_ARG;
  }
  if ((((uintptr_t)dout) | ((uintptr_t)out2)) & 15) {  // the delta kernel reads 16 bytes per lane
    set_error("%s: dout and out2 must be 16-byte aligned", who);
    return ADS_ERR_BAD_ARG;
  }
  int path;
  if (int rc = resolve_path(s, who, &path)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  simt::Params p = make_params(s);
  p.q = q; p.k = k; p.v = v; p.varlen = varlen; p.dout = dout; p.out2_in = out2;
  p.taus = const_cast<float*>(taus); p.bmask = const_cast<int32_t*>(bmask);
  p.bmask_t = bmask_t; p.delta = delta; p.dq = dq; p.dk = dk; p.dv = dv;
  if (int rc = resolve_support(s, path, support, support_bytes, who, &p.support)) return rc;
  if (s->bwd_stages != 0) p.support = nullptr;  // single kernels of the tile route (timing aid)
  if (p.support != nullptr) {
    const size_t need = sm100::min_workspace_bytes() + sparse::bwd_scratch_bytes(s);
    if (ws == nullptr || ws_bytes < need) {
      set_error("%s: with a support buffer the backward needs %zu bytes of workspace (got %zu)", who, need, ws_bytes);
      return ADS_ERR_WORKSPACE;
    }
    p.bwd_scratch = (uint8_t*)ws + sm100::min_workspace_bytes();
  }
  if (int rc = clear_status(ws, ws_bytes, st, who)) return rc;
  if (path == ADS_PATH_TCGEN05) {
    if (ws == nullptr || ws_bytes < sm100::min_workspace_bytes()) {
      set_error("%s: workspace too small (%zu < %zu)", who, ws_bytes, sm100::min_workspace_bytes());
      return ADS_ERR_WORKSPACE;
    }
    if (p.support != nullptr) {
      if (int rc = sparse::bwd(p, s->dtype, st)) return rc;
    }
    return is_v2(s) ? sm100::bwd(p, s->dtype, ws, st) : sm100::v1::bwd(p, s->dtype, ws, st);
  }
  return by_dtype(
      s->dtype, [&] { return simt::launch_bwd<float>(p, st); },
      [&] { return simt::launch_bwd<__half>(p, st); },
      [&] { return simt::launch_bwd<__nv_bfloat16>(p, st); });
}

extern "C" int adasplash2_debug_waits(int64_t max_wait_cycles, int32_t withhold_loads) {
  return sm100::debug_waits((long long)max_wait_cycles, (int)withhold_loads);
}

namespace ads { int static_scratch_base(void** out); }

extern "C" int adasplash2_check_status(const void* workspace, void* stream) {
  if (workspace == nullptr) {
    // the caller of adasplash2_bwd_static owns no workspace: read the status word of the
    // library's built-in scratch on the current device
    void* base = nullptr;
    if (int rc = ads::static_scratch_base(&base)) return rc;
    workspace = base;
  }
  int host = 0;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(&host, workspace, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) { set_error("check_status: %s", cudaGetErrorString(e)); return ADS_ERR_CUDA; }
  if (host != 0) {
    set_error("a device-side wait timed out (code %d: 101 = TMA producer, 102 = MMA issuer, 103 = row warps)", host);
    return ADS_ERR_TIMEOUT;
  }
  return ADS_OK;
}
