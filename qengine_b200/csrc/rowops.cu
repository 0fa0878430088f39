// Row-wise kernels of a decode pass: embedding gather, zero-centred RMSNorm with fused residual,
// BF16 GEMV (off the W4 path), SwiGLU and the vocabulary argmax.
// Boundary: these replace launch_embed .. launch_argmax of the reference (csrc/ops.h:6-14).
// Every kernel treats rows independently and uses a row-count-independent operation order, so
// row r of an n-row call is bit-identical to a 1-row call (the verify == plain-decode property).
#include <algorithm>

#include "common.cuh"
#include "../../include/qengine_b200.h"

namespace qb {
namespace {

// ---------------------------------------------------------------------------------------------
// Embedding gather. Semantics of embed_kernel (reference csrc/basic.cu:16-26): out[r] =
// table[tok[r]], ids outside [0, V) give zeros. 16-byte copies when the rows allow it.
// ---------------------------------------------------------------------------------------------
__global__ void embed_rows_kernel(const bf16* table, const int* tok,
                                  bf16* out, int H, int V, long ldo, int vec) {
  dep_release();
  dep_wait();
  const int r = blockIdx.y;
  const int id = tok[r];
  const bool ok = id >= 0 && id < V;
  bf16* dst = out + (long)r * ldo;
  const bf16* src = table + (size_t)(ok ? id : 0) * H;
  if (vec) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;  // 8 elements per thread
    if (i * 8 < H)
      reinterpret_cast<uint4*>(dst)[i] = ok ? __ldg(reinterpret_cast<const uint4*>(src) + i)
                                            : make_uint4(0, 0, 0, 0);
  } else {
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8, e = min(i + 8, H); i < e; ++i)
      dst[i] = ok ? src[i] : tobf16(0.f);
  }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm1p (+ residual). Semantics of rmsnorm1p_kernel (reference csrc/basic.cu:29-54,
// python/qengine/reference.py:132-136): x = bf16(x + delta) written back when delta is given,
// out = bf16(x * rsqrt(mean x^2 + eps) * (1 + w)), fp32 math, one rounding.
// One CTA per row; a thread owns 8-element packets at stride blockDim, kept in registers
// (PKT packets, enough for H <= 8 * PKT * blockDim) so the row is read once.
// ---------------------------------------------------------------------------------------------
template <int PKT>
__global__ void __launch_bounds__(256)
rmsnorm1p_vec_kernel(bf16* x, const bf16* delta,
                     const bf16* w, bf16* out, int H, long ldx, long ldd,
                     long ldo, float eps) {
  dep_release();
  __shared__ float scratch[32];
  const int row = blockIdx.x, npk = H >> 3;
  // the weight is a constant: fetch it while the producer of x is still running
  uint4 wq[PKT];
#pragma unroll
  for (int p = 0; p < PKT; ++p) {
    const int i = threadIdx.x + p * blockDim.x;
    if (i < npk) wq[p] = __ldg(reinterpret_cast<const uint4*>(w) + i);
  }
  dep_wait();
  uint4* xr = reinterpret_cast<uint4*>(x + (long)row * ldx);
  const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + (long)row * ldd) : nullptr;
  float v[PKT][8];
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < PKT; ++p) {
    const int i = threadIdx.x + p * blockDim.x;
    if (i < npk) {
      widen8(xr[i], v[p]);
      if (dr) {
        float d[8];
        widen8(dr[i], d);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[p][e] = rnd(v[p][e] + d[e]);
        xr[i] = narrow8(v[p]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(v[p][e], v[p][e], ss);
    }
  }
  const float inv = rsqrtf(block_allsum(ss, scratch) / (float)H + eps);
  uint4* orow = reinterpret_cast<uint4*>(out + (long)row * ldo);
#pragma unroll
  for (int p = 0; p < PKT; ++p) {
    const int i = threadIdx.x + p * blockDim.x;
    if (i < npk) {
      float g[8], y[8];
      widen8(wq[p], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = v[p][e] * inv * (1.0f + g[e]);
      orow[i] = narrow8(y);
    }
  }
}

// Any H, any alignment: two passes over the row, same arithmetic per element.
__global__ void __launch_bounds__(256)
rmsnorm1p_any_kernel(bf16* x, const bf16* delta,
                     const bf16* w, bf16* out, int H, long ldx, long ldd,
                     long ldo, float eps) {
  dep_release();
  dep_wait();
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  bf16* xr = x + (long)row * ldx;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = tofloat(xr[c]);
    if (delta) {
      v = rnd(v + tofloat(delta[(long)row * ldd + c]));
      xr[c] = tobf16(v);  // re-read below by the same thread only
    }
    ss = fmaf(v, v, ss);
  }
  const float inv = rsqrtf(block_allsum(ss, scratch) / (float)H + eps);
  for (int c = threadIdx.x; c < H; c += blockDim.x)
    out[(long)row * ldo + c] = tobf16(tofloat(xr[c]) * inv * (1.0f + tofloat(w[c])));
}

// ---------------------------------------------------------------------------------------------
// BF16 GEMV, NR = 1..8 rows, one warp per weight row, weights read once for all rows.
// Semantics of gemv_bf16_kernel (reference csrc/basic.cu:99-155). A lane always walks k in the
// same order whatever NR is.
// ---------------------------------------------------------------------------------------------
constexpr int kGemvWarps = 8;

template <int NR>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_bf16_rows_kernel(const bf16* W, const bf16* x,
                      bf16* out, int N, int K, long ldx, long ldo) {
  dep_release();
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.x * kGemvWarps + (threadIdx.x >> 5);
  if (j >= N) { dep_wait(); return; }
  const int npk = K >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(W + (size_t)j * K);
  float acc[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) acc[r] = 0.f;
  bool waited = false;
  for (int p0 = lane; p0 < npk; p0 += 128) {
    uint4 wq[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (p0 + 32 * u < npk) wq[u] = __ldg(wr + p0 + 32 * u);
    if (!waited) { dep_wait(); waited = true; }  // weights are constants; x is produced upstream
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (p0 + 32 * u < npk) {
        float wf[8];
        widen8(wq[u], wf);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
          float xf[8];
          widen8(reinterpret_cast<const uint4*>(x + (long)r * ldx)[p0 + 32 * u], xf);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[r] = fmaf(wf[e], xf[e], acc[r]);
        }
      }
    }
  }
  if (!waited) dep_wait();
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const float s = warp_allsum(acc[r]);
    if (lane == 0) out[(long)r * ldo + j] = tobf16(s);
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU on unfused [gate | up] rows: bf16(bf16(silu(g)) * u) (reference csrc/basic.cu:157-170).
// ---------------------------------------------------------------------------------------------
__global__ void swiglu_rows_kernel(const bf16* gu, bf16* out, int I,
                                   long ldg, long ldo) {
  dep_release();
  dep_wait();
  const int r = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= I) return;
  const bf16* g = gu + (long)r * ldg;
  const float s = rnd(silu_acc(tofloat(g[i])));
  out[(long)r * ldo + i] = tobf16(s * tofloat(g[I + i]));
}

// ---------------------------------------------------------------------------------------------
// Argmax, torch semantics (reference csrc/basic.cu:173-239): NaN beats everything, then the
// larger value, then the lower index. A candidate is (value, index); index INT_MAX = "none".
// Stage 1: grid (nb, rows), CTA b scans a contiguous slab of the row with 16-byte loads when
// aligned. Stage 2: one CTA per row merges the nb candidates and maps through idmap.
// ---------------------------------------------------------------------------------------------
constexpr int kNone = 0x7fffffff;

__device__ __forceinline__ bool beats(float a, int ia, float b, int ib) {
  const bool an = a != a, bn = b != b;
  if (an != bn) return an;
  if (!an && a != b) return a > b;
  return ia < ib;
}
__device__ __forceinline__ void merge(float& v, int& i, float ov, int oi) {
  if (beats(ov, oi, v, i)) { v = ov; i = oi; }
}
__device__ __forceinline__ void block_best(float& v, int& i, float* sv, int* si) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    merge(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) { sv[w] = v; si[w] = i; }
  __syncthreads();
  if (w == 0) {
    v = lane < nw ? sv[lane] : -INFINITY;
    i = lane < nw ? si[lane] : kNone;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      merge(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
  }
}

__global__ void __launch_bounds__(256)
argmax_slab_kernel(const bf16* x, int n, long ldx, float* pv,
                   int* pi) {
  dep_release();
  dep_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row = blockIdx.y, nb = gridDim.x;
  const bf16* xr = x + (long)row * ldx;
  // slab of this CTA, in 8-element packets
  const int npk = (n + 7) >> 3;
  const int per = (npk + nb - 1) / nb;
  const int p0 = blockIdx.x * per, p1 = min(npk, p0 + per);
  const bool vec = ((reinterpret_cast<uintptr_t>(xr) & 15) == 0);
  float v = -INFINITY;
  int i = kNone;
  for (int p = p0 + threadIdx.x; p < p1; p += blockDim.x) {
    const int k0 = p * 8;
    if (vec && k0 + 8 <= n) {
      float f[8];
      widen8(reinterpret_cast<const uint4*>(xr)[p], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) merge(v, i, f[e], k0 + e);
    } else {
      for (int k = k0; k < min(k0 + 8, n); ++k) merge(v, i, tofloat(xr[k]), k);
    }
  }
  block_best(v, i, sv, si);
  if (threadIdx.x == 0) { pv[row * nb + blockIdx.x] = v; pi[row * nb + blockIdx.x] = i; }
}

__global__ void __launch_bounds__(256)
argmax_final_kernel(const float* pv, const int* pi, int nb,
                    int* out, const int* idmap, float* out_v, int base) {
  dep_release();
  dep_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row = blockIdx.x;
  float v = -INFINITY;
  int i = kNone;
  for (int k = threadIdx.x; k < nb; k += blockDim.x) merge(v, i, pv[row * nb + k], pi[row * nb + k]);
  block_best(v, i, sv, si);
  if (threadIdx.x == 0) {
    const int a = i == kNone ? 0 : i;  // a row of -inf only: index 0, like torch
    out[row] = (idmap ? idmap[a] : a) + base;
    if (out_v) out_v[row] = v;
  }
}

// Best of nparts (value, index) candidates per row; vals / idx are [nparts, rows]. Used to merge
// the per-rank winners of a vocabulary-split lm_head: same ordering rule as the local argmax, so
// the result equals the argmax over the whole vocabulary (ties go to the lowest global index).
__global__ void argmax_merge_kernel(const float* vals, const int* idx, int nparts, int rows, int* out) {
  dep_release();
  dep_wait();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float v = vals[row];
  int i = idx[row];
  for (int p = 1; p < nparts; ++p) merge(v, i, vals[p * rows + row], idx[p * rows + row]);
  out[row] = i;
}


inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool pdl_on() { return pdl_launch_enabled() && pdl_trigger_enabled(); }

}  // namespace
}  // namespace qb

using namespace qb;

extern "C" int qe_embed(const void* table, const int* tok, void* out, int n, int H, int V, long ldo,
                        void* stream) {
  if (n < 1 || H < 1) return QE_ERR_ARG;
  const int vec = (H % 8 == 0) && (ldo % 8 == 0) && aligned16(table) && aligned16(out);
  const int per_block = 256 * 8;
  return (int)launch(embed_rows_kernel, dim3((H + per_block - 1) / per_block, n), dim3(256), 0,
                     (cudaStream_t)stream, pdl_on(), (const bf16*)table, tok, (bf16*)out, H, V, ldo,
                     vec);
}

extern "C" int qe_rmsnorm1p(void* x, const void* delta, const void* w, void* out, int rows, int H,
                            long ldx, long ldd, long ldo, float eps, void* stream) {
  if (rows < 1 || H < 1) return QE_ERR_ARG;
  const bool vec = H % 8 == 0 && ldx % 8 == 0 && ldo % 8 == 0 && (!delta || ldd % 8 == 0) &&
                   aligned16(x) && aligned16(out) && aligned16(w) && (!delta || aligned16(delta));
  cudaStream_t s = (cudaStream_t)stream;
  bf16* X = (bf16*)x;
  const bf16 *D = (const bf16*)delta, *W = (const bf16*)w;
  bf16* O = (bf16*)out;
  if (vec && H <= 8 * 256 * 4) {
    const int npk = H / 8;
    if (npk <= 256) {
      const int threads = std::max(32, (npk + 31) / 32 * 32);
      return (int)launch(rmsnorm1p_vec_kernel<1>, dim3(rows), dim3(threads), 0, s, pdl_on(), X, D, W,
                         O, H, ldx, ldd, ldo, eps);
    }
    if (npk <= 512)
      return (int)launch(rmsnorm1p_vec_kernel<2>, dim3(rows), dim3(256), 0, s, pdl_on(), X, D, W, O,
                         H, ldx, ldd, ldo, eps);
    return (int)launch(rmsnorm1p_vec_kernel<4>, dim3(rows), dim3(256), 0, s, pdl_on(), X, D, W, O, H,
                       ldx, ldd, ldo, eps);
  }
  return (int)launch(rmsnorm1p_any_kernel, dim3(rows), dim3(256), 0, s, pdl_on(), X, D, W, O, H, ldx,
                     ldd, ldo, eps);
}

extern "C" int qe_gemv_bf16(const void* W, const void* x, void* out, int nr, int N, int K, long ldx,
                            long ldo, void* stream) {
  if (nr < 1 || nr > QE_MAX_ROWS || K % 8 || N < 1) return QE_ERR_ARG;
  if (!aligned16(W) || !aligned16(x) || ldx % 8) return QE_ERR_ARG;
  const dim3 grid((N + kGemvWarps - 1) / kGemvWarps), block(kGemvWarps * 32);
  cudaStream_t s = (cudaStream_t)stream;
  const bf16 *w = (const bf16*)W, *xx = (const bf16*)x;
  bf16* o = (bf16*)out;
  switch (nr) {
#define QB_ROWS(R) \
  case R: return (int)launch(gemv_bf16_rows_kernel<R>, grid, block, 0, s, pdl_on(), w, xx, o, N, K, ldx, ldo);
    QB_ROWS(1) QB_ROWS(2) QB_ROWS(3) QB_ROWS(4) QB_ROWS(5) QB_ROWS(6) QB_ROWS(7) QB_ROWS(8)
#undef QB_ROWS
  }
  return QE_ERR_ARG;
}

extern "C" int qe_swiglu(const void* gu, void* out, int n, int I, long ldg, long ldo, void* stream) {
  if (n < 1 || I < 1) return QE_ERR_ARG;
  return (int)launch(swiglu_rows_kernel, dim3((I + 255) / 256, n), dim3(256), 0,
                     (cudaStream_t)stream, pdl_on(), (const bf16*)gu, (bf16*)out, I, ldg, ldo);
}

extern "C" int qe_argmax_v(const void* x, int rows, int n, long ldx, float* pv, int* pi, int nb,
                           int* out, float* out_v, const int* idmap, int base, void* stream) {
  if (rows < 1 || n < 1 || nb < 1) return QE_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  int e = (int)launch(argmax_slab_kernel, dim3(nb, rows), dim3(256), 0, s, pdl_on(),
                      (const bf16*)x, n, ldx, pv, pi);
  if (e) return e;
  return (int)launch(argmax_final_kernel, dim3(rows), dim3(256), 0, s, pdl_on(), (const float*)pv,
                     (const int*)pi, nb, out, idmap, out_v, base);
}

extern "C" int qe_argmax(const void* x, int rows, int n, long ldx, float* pv, int* pi, int nb,
                         int* out, const int* idmap, void* stream) {
  return qe_argmax_v(x, rows, n, ldx, pv, pi, nb, out, nullptr, idmap, 0, stream);
}

extern "C" int qe_argmax_merge(const float* vals, const int* idx, int nparts, int rows, int* out,
                               void* stream) {
  if (nparts < 1 || rows < 1) return QE_ERR_ARG;
  return (int)launch(argmax_merge_kernel, dim3((rows + 31) / 32), dim3(32), 0, (cudaStream_t)stream,
                     pdl_on(), vals, idx, nparts, rows, out);
}

