// Gather kernels over the row supports exported by the tensor-core solver (support.cuh).
//
// A query row's output is sum_j p_ij V_j over the few keys j of its support, so one warp per row
// reads the row's (key, u) pairs and the V rows they name -- a few hundred bytes per pair, all
// from L2 -- instead of re-computing dense score tiles.  The arithmetic is the tile kernels':
// p = rn(u^2) and w = rn(u) in the input dtype, fp32 accumulation, out2 = (sum w V) / (sum u)
// (adasplash_v2.py:696-835).
#include "sparse_rows.cuh"

#include "support.cuh"

namespace ads {
namespace sparse {
namespace {

constexpr int kRowThreads = 256;

struct RowsParams {
  const void* v; void* out; void* out2;
  const void* varlen; int varlen_is_i64;
  int B, Hq, Hkv, N, Dg;
  sup::View sv;
};

// eight 16-bit elements <-> fp32
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = DT<T>::to_f(e[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = DT<T>::from_f(f[i]);
  return raw;
}

// One warp per 32 consecutive query rows of a head, eight lanes per row: lane gl of a group owns
// the 16-byte chunks gl and (CH = 2, head dim 128) 8 + gl of the head dimension, so a V row is
// one or two coalesced 128-byte requests per group and every instruction of the accumulation
// serves four (row, key) pairs.  Group g takes rows 8g .. 8g+7 one after the other; the eight
// lanes fetch up to eight of the row's entries with one load and pass them round with shuffles.
constexpr int kRowsPerWarp = 32;

template <typename T, int CH>
__global__ void __launch_bounds__(kRowThreads) fwd_rows_kernel(RowsParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, gl = lane & 7;
  const int chunks = (p.N + kRowsPerWarp - 1) / kRowsPerWarp;  // per head
  const long long wg = (long long)blockIdx.x * (kRowThreads / 32) + warp;
  if (wg >= (long long)p.B * p.Hq * chunks) return;
  const int bh = (int)(wg / chunks), r0 = (int)(wg % chunks) * kRowsPerWarp;
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  if (p.sv.dense[b * p.Hkv + kvh] != 0) return;  // the tile kernels own this head
  const bool lane_on = gl * 8 < p.Dg;
  const int len = load_len(p.varlen, p.varlen_is_i64, b, p.N);
  const size_t row_base = (size_t)bh * p.N;
  // rows at or beyond the sequence length have no entries (the solver wrote nothing for them)
  const uint2 rw = (r0 + lane < len) ? p.sv.rows[row_base + r0 + lane] : make_uint2(0u, 0u);
  const T* vb = (const T*)p.v + (size_t)(b * p.Hkv + kvh) * p.N * p.Dg + gl * 8;
#pragma unroll 1
  for (int i = 0; i < 8; ++i) {
    const int rr = grp * 8 + i;  // this group's row inside the chunk
    const uint32_t first = __shfl_sync(0xffffffffu, rw.x, rr), cnt = __shfl_sync(0xffffffffu, rw.y, rr);
    const uint32_t cnt_max = __reduce_max_sync(0xffffffffu, cnt);
    float ao[CH * 8], ao2[CH * 8];
#pragma unroll
    for (int e = 0; e < CH * 8; ++e) { ao[e] = 0.f; ao2[e] = 0.f; }
    float supp = 0.f;
    for (uint32_t k0 = 0; k0 < cnt_max; k0 += 8) {
      const uint2 ent = (k0 + gl < cnt) ? p.sv.entries[first + k0 + gl] : make_uint2(0u, 0u);
#pragma unroll
      for (int hb = 0; hb < 8; hb += 4) {
        if (k0 + hb >= cnt_max) break;
        uint4 raw[4][CH];
        float u[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // four entries of each group in flight
          const uint32_t key = __shfl_sync(0xffffffffu, ent.x, hb + j, 8);
          u[j] = __uint_as_float(__shfl_sync(0xffffffffu, ent.y, hb + j, 8));  // 0 beyond the row's entries
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            raw[j][c] = make_uint4(0u, 0u, 0u, 0u);
            if (k0 + hb + j < cnt && lane_on) raw[j][c] = *reinterpret_cast<const uint4*>(vb + (size_t)key * p.Dg + c * 64);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float pw = round_to<T>(u[j] * u[j]), uw = round_to<T>(u[j]);
          supp += u[j];
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            float vf[8];
            unpack8<T>(raw[j][c], vf);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              ao[c * 8 + e] = fmaf(pw, vf[e], ao[c * 8 + e]);
              ao2[c * 8 + e] = fmaf(uw, vf[e], ao2[c * 8 + e]);
            }
          }
        }
      }
    }
    const float inv = supp > 0.f ? 1.0f / supp : 0.f;
#pragma unroll
    for (int e = 0; e < CH * 8; ++e) ao2[e] *= inv;
    if (lane_on && r0 + rr < p.N) {
      T* o = (T*)p.out + (row_base + r0 + rr) * p.Dg + gl * 8;
      T* o2 = (T*)p.out2 + (row_base + r0 + rr) * p.Dg + gl * 8;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        *reinterpret_cast<uint4*>(o + c * 64) = pack8<T>(ao + c * 8);
        *reinterpret_cast<uint4*>(o2 + c * 64) = pack8<T>(ao2 + c * 8);
      }
    }
  }
}

template <typename T>
int fwd_t(const simt::Params& p, cudaStream_t st) {
  RowsParams rp;
  rp.v = p.v; rp.out = p.out; rp.out2 = p.out2;
  rp.varlen = p.varlen; rp.varlen_is_i64 = p.varlen_is_i64;
  rp.B = p.B; rp.Hq = p.Hq; rp.Hkv = p.Hkv; rp.N = p.N; rp.Dg = p.D;
  rp.sv = sup::view(p.support, p.B, p.Hq, p.Hkv, p.N);
  const long long warps = (long long)p.B * p.Hq * ((p.N + kRowsPerWarp - 1) / kRowsPerWarp);
  const unsigned grid = (unsigned)((warps + kRowThreads / 32 - 1) / (kRowThreads / 32));
  if (p.D > 64) fwd_rows_kernel<T, 2><<<grid, kRowThreads, 0, st>>>(rp);
  else fwd_rows_kernel<T, 1><<<grid, kRowThreads, 0, st>>>(rp);
  return check_launch("sparse::fwd_rows");
}

}  // namespace

bool supported(const ads_attn_shape* s) {
  // 16-bit inputs on the tensor-core solver, causal alpha = 1.5, key indices that fit 16 bits
  if (s->dtype != ADS_F16 && s->dtype != ADS_BF16) return false;
  if (s->D != 16 && s->D != 32 && s->D != 64 && s->D != 128) return false;
  if (s->N > 65536) return false;
  if (!((s->alpha == 0.f || s->alpha == 1.5f) && s->non_causal == 0)) return false;
  return true;
}

size_t support_bytes(const ads_attn_shape* s) { return sup::bytes(s->B, s->Hq, s->Hkv, s->N); }

int clear_header(const simt::Params& p, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(p.support, 0, sup::header_bytes(p.B, p.Hkv), st);
  if (e != cudaSuccess) { set_error("support header memset: %s", cudaGetErrorString(e)); return ADS_ERR_CUDA; }
  return ADS_OK;
}

int fwd(const simt::Params& p, int dtype, cudaStream_t st) {
  if (dtype == ADS_F16) return fwd_t<__half>(p, st);
  return fwd_t<__nv_bfloat16>(p, st);
}

}  // namespace sparse
}  // namespace ads
