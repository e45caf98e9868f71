// Backward entry point for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to get scratch memory at call time:
// a plugin that is handed device pointers by its framework and must not touch
// the allocator, code that runs between the capture calls of a larger program,
// or a process whose memory budget was fixed before it started.  For them the
// three scratch buffers of the backward (status word, delta, transposed block
// mask) live in one fixed array that is part of the loaded library image.
#include <mutex>

#include "common.cuh"

namespace {

// The built-in scratch: ADS_STATIC_SCRATCH_BYTES on every GPU that loads the
// library, held until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[ADS_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 128;
void* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mu;

inline size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

// `g_static_scratch` in host code is only a handle for the symbol, not a device
// address; the address on the current device comes from the runtime, once.  The cached
// address belongs to the device's primary context: it is valid as long as that context
// lives (a cudaDeviceReset in the host program invalidates it).
int static_scratch_address(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    ads::set_error("bwd_static: cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
    return ADS_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      ads::set_error("bwd_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return ADS_ERR_CUDA;
    }
    g_scratch_addr[dev] = p;
  }
  *out = static_cast<unsigned char*>(g_scratch_addr[dev]);
  return ADS_OK;
}

}  // namespace

// Address of the built-in scratch on the current device (the status word of the backward's
// bounded waits sits at its start); used by adasplash2_check_status(NULL, stream).
namespace ads {
int static_scratch_base(void** out) {
  unsigned char* base = nullptr;
  if (int rc = static_scratch_address(&base)) return rc;
  *out = base;
  return ADS_OK;
}
}  // namespace ads

extern "C" int adasplash2_bwd_static(const void* q, const void* k, const void* v, const void* dout,
                                     const void* out2, const void* varlen, const float* taus,
                                     const int32_t* bmask, void* dq, void* dk, void* dv,
                                     const ads_attn_shape* shape, void* stream) {
  if (shape == nullptr || shape->B < 1 || shape->Hq < 1 || shape->N < 1) {
    ads::set_error("adasplash2_bwd_static: bad shape");
    return ADS_ERR_BAD_ARG;
  }
  if (shape->bwd_stages != 0) {
    // a partial backward would read delta / the transposed mask that an earlier call, possibly
    // of another shape, left in the shared array
    ads::set_error("adasplash2_bwd_static: bwd_stages must be 0 (the whole backward)");
    return ADS_ERR_BAD_ARG;
  }
  int32_t rows_padded = 0, n_words = 0;
  const int64_t words = adasplash2_bitmap_words(shape, &rows_padded, &n_words);
  if (words < 0) { ads::set_error("adasplash2_bwd_static: bad shape"); return ADS_ERR_BAD_ARG; }
  const size_t status_bytes = 256;
  const size_t delta_bytes = round256((size_t)shape->B * shape->Hq * shape->N * sizeof(float));
  const size_t bitmap_bytes = round256((size_t)words * sizeof(int32_t));
  const size_t need = status_bytes + delta_bytes + bitmap_bytes;
  if (need > (size_t)ADS_STATIC_SCRATCH_BYTES) {
    ads::set_error("adasplash2_bwd_static: B*Hq*N = %lld rows need %zu bytes of scratch, the built-in buffer "
                   "holds %zu; use adasplash2_bwd with caller-owned scratch",
                   (long long)shape->B * shape->Hq * shape->N, need, (size_t)ADS_STATIC_SCRATCH_BYTES);
    return ADS_ERR_WORKSPACE;
  }
  unsigned char* base = nullptr;
  if (int rc = static_scratch_address(&base)) return rc;
  float* delta = reinterpret_cast<float*>(base + status_bytes);
  int32_t* bmask_t = reinterpret_cast<int32_t*>(base + status_bytes + delta_bytes);
  // Nothing has to be cleared by hand: the status word is reset by the backward
  // itself, delta and the transposed mask are fully rewritten by its first two
  // kernels before anything reads them.
  return adasplash2_bwd(q, k, v, dout, out2, varlen, taus, bmask, bmask_t, delta, dq, dk, dv, shape,
                        base, status_bytes, nullptr, 0, stream);
}
