// Gated GQA attention for decode / verify: n = 1..8 query rows at positions pos + t, causal over
// the KV cache. Boundary: replaces launch_attn_prep and launch_attn_decode of the reference
// (csrc/ops.h:25-30, kernels csrc/attn.cu:17-149); the math follows attention_qkv_from_proj and
// attention_core of the reference torch model (python/qengine/reference.py:252-272).
//
//   prep    per head: xn = bf16(x * rsqrt(mean x^2 + eps) * (1 + w)); rotate-half RoPE on the
//           first rd dims with bf16 rounding after every elementwise op (cos/sin rounded to
//           bf16 first); q -> q_out, k and raw v -> cache row pos + t (skipped past max_len).
//   decode  split-KV flash decoding: CTA (head, split, row) reduces its slice of the row's
//           causal prefix [0, pos + t] with an online softmax in fp32, four cache positions per
//           warp step so that four independent 16-byte K loads and V loads are in flight per
//           lane; a second kernel merges the NS partials, rounds o = bf16(O / L) and applies
//           bf16(sigmoid(gate)).
// Row independence: the slice boundaries of row t depend only on its own prefix length, so row t
// of an n-row call is bit-identical to a 1-row call at position pos + t.
#include "common.cuh"
#include "../../include/qengine_b200.h"

namespace qb {
namespace {

constexpr int kSplitWarps = 8, kStep = 4;

template <int HD>
__global__ void __launch_bounds__(HD)
attn_prep_kernel(const bf16* qg, const bf16* k, const bf16* v,
                 long ldp, const bf16* qnw, const bf16* knw,
                 const float* inv_freq, const int* pos_ptr,
                 bf16* q_out, bf16* kc, bf16* vc, int Hq,
                 int max_len, int rd, float eps) {
  dep_release();
  dep_wait();
  __shared__ float xn[HD];
  __shared__ float scratch[32];
  const int hb = blockIdx.x, c = threadIdx.x, t = blockIdx.y;
  const bool is_q = hb < Hq;
  const int h = is_q ? hb : hb - Hq;
  const int pos = pos_ptr[0] + t;
  const bf16* src = is_q ? qg + (long)t * ldp + (size_t)h * 2 * HD : k + (long)t * ldp + (size_t)h * HD;
  const float x = tofloat(src[c]);
  const float inv = rsqrtf(block_allsum(x * x, scratch) / (float)HD + eps);
  xn[c] = rnd(x * inv * (1.0f + tofloat(is_q ? qnw[c] : knw[c])));
  __syncthreads();
  float y = xn[c];
  if (c < rd) {
    const int half = rd >> 1;
    const float ang = (float)pos * inv_freq[c % half];
    const float cs = rnd(cosf(ang)), sn = rnd(sinf(ang));
    const float rot = c < half ? -xn[c + half] : xn[c - half];
    y = rnd(rnd(xn[c] * cs) + rnd(rot * sn));
  }
  if (is_q) {
    q_out[((size_t)t * Hq + h) * HD + c] = tobf16(y);
  } else if (pos >= 0 && pos < max_len) {
    const size_t at = ((size_t)h * max_len + pos) * HD + c;
    kc[at] = tobf16(y);
    vc[at] = v[(long)t * ldp + (size_t)h * HD + c];
  }
}

// HD / 32 consecutive elements of one cache row for this lane, widened to fp32.
template <int HD>
__device__ __forceinline__ void load_lane(const bf16* row, int lane, float (&f)[HD / 32]) {
  if constexpr (HD == 256) {
    widen8(reinterpret_cast<const uint4*>(row)[lane], f);
  } else if constexpr (HD == 128) {
    const uint2 p = reinterpret_cast<const uint2*>(row)[lane];
    f[0] = __uint_as_float(p.x << 16); f[1] = __uint_as_float(p.x & 0xffff0000u);
    f[2] = __uint_as_float(p.y << 16); f[3] = __uint_as_float(p.y & 0xffff0000u);
  } else {
    const uint32_t p = reinterpret_cast<const uint32_t*>(row)[lane];
    f[0] = __uint_as_float(p << 16); f[1] = __uint_as_float(p & 0xffff0000u);
  }
}

template <int HD>
__global__ void __launch_bounds__(kSplitWarps * 32)
attn_split_kernel(const bf16* q, const bf16* kc,
                  const bf16* vc, const int* pos_ptr,
                  float* part_o, float* part_ml, int Hq, int Hkv,
                  int max_len, float scale) {
  constexpr int E = HD / 32;
  dep_release();
  dep_wait();
  __shared__ float sm[kSplitWarps], sl[kSplitWarps];
  __shared__ float so[kSplitWarps][HD];
  const int h = blockIdx.x, s = blockIdx.y, NS = gridDim.y, t = blockIdx.z;
  const int g = h / (Hq / Hkv);
  const int len = min(max(pos_ptr[0] + t + 1, 0), max_len);  // causal prefix of row t
  const int chunk = (len + NS - 1) / NS;
  const int start = s * chunk, end = min(len, start + chunk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  float qf[E];
  load_lane<HD>(q + ((size_t)t * Hq + h) * HD, lane, qf);
  const bf16* kb = kc + (size_t)g * max_len * HD;
  const bf16* vb = vc + (size_t)g * max_len * HD;
  float m = -INFINITY, l = 0.f, acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;

  // warp w takes positions start + kStep * (w + kSplitWarps * i) + {0..kStep-1}
  for (int p0 = start + kStep * warp; p0 < end; p0 += kStep * kSplitWarps) {
    float kf[kStep][E], vf[kStep][E], sc[kStep];
#pragma unroll
    for (int u = 0; u < kStep; ++u)
      if (p0 + u < end) load_lane<HD>(kb + (size_t)(p0 + u) * HD, lane, kf[u]);
#pragma unroll
    for (int u = 0; u < kStep; ++u)
      if (p0 + u < end) load_lane<HD>(vb + (size_t)(p0 + u) * HD, lane, vf[u]);
#pragma unroll
    for (int u = 0; u < kStep; ++u) {
      float dsum = 0.f;
      if (p0 + u < end) {
#pragma unroll
        for (int e = 0; e < E; ++e) dsum = fmaf(qf[e], kf[u][e], dsum);
      }
      sc[u] = dsum;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int u = 0; u < kStep; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
    }
    float mn = m;
#pragma unroll
    for (int u = 0; u < kStep; ++u) {
      sc[u] = (p0 + u < end) ? sc[u] * scale : -INFINITY;
      mn = fmaxf(mn, sc[u]);
    }
    const float corr = expf(m - mn);  // first step: exp(-inf) = 0
    l *= corr;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] *= corr;
#pragma unroll
    for (int u = 0; u < kStep; ++u) {
      if (p0 + u < end) {
        const float pe = expf(sc[u] - mn);
        l += pe;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = fmaf(pe, vf[u][e], acc[e]);
      }
    }
    m = mn;
  }
  if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
  for (int e = 0; e < E; ++e) so[warp][lane * E + e] = acc[e];
  __syncthreads();
  // merge the warps in warp order; thread c owns output dim c
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < kSplitWarps; ++w) M = fmaxf(M, sm[w]);
  float L = 0.f;
  const size_t slot = ((size_t)t * Hq + h) * NS + s;
  for (int c = threadIdx.x; c < HD; c += blockDim.x) {
    float O = 0.f;
    L = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kSplitWarps; ++w) {
        const float f = expf(sm[w] - M);
        L += sl[w] * f;
        O += so[w][c] * f;
      }
    }
    part_o[slot * HD + c] = O;
  }
  if (threadIdx.x == 0) {
    // L as computed by thread 0 (same formula for every thread)
    part_ml[slot * 2] = M;
    part_ml[slot * 2 + 1] = L;
  }
}

// The same split for all GQ query heads of one KV head in one CTA: every K / V row of the slice is
// loaded once and used by the GQ heads that share it (grouped-query attention), instead of once
// per query head. With a long cache the KV stream is the whole cost of the layer (134 MB per layer
// at 32K positions of the 27B shape), so this divides the L2 / HBM traffic by GQ. Position-to-warp
// assignment, step size and the order of every sum are those of attn_split_kernel: per head the
// result is bit-identical to it.
template <int HD, int GQ>
__global__ void __launch_bounds__(kSplitWarps * 32)
attn_split_gqa_kernel(const bf16* q, const bf16* kc, const bf16* vc, const int* pos_ptr, float* part_o,
                      float* part_ml, int Hq, int max_len, float scale) {
  constexpr int E = HD / 32;
  dep_release();
  dep_wait();
  __shared__ float sm[kSplitWarps], sl[kSplitWarps];
  __shared__ float so[kSplitWarps][HD];
  const int g = blockIdx.x, s = blockIdx.y, NS = gridDim.y, t = blockIdx.z;
  const int len = min(max(pos_ptr[0] + t + 1, 0), max_len);
  const int chunk = (len + NS - 1) / NS;
  const int start = s * chunk, end = min(len, start + chunk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  float qf[GQ][E], acc[GQ][E], m[GQ], l[GQ];
#pragma unroll
  for (int j = 0; j < GQ; ++j) {
    load_lane<HD>(q + ((size_t)t * Hq + g * GQ + j) * HD, lane, qf[j]);
    m[j] = -INFINITY;
    l[j] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[j][e] = 0.f;
  }
  const bf16* kb = kc + (size_t)g * max_len * HD;
  const bf16* vb = vc + (size_t)g * max_len * HD;

  for (int p0 = start + kStep * warp; p0 < end; p0 += kStep * kSplitWarps) {
    float kf[kStep][E], vf[kStep][E];
#pragma unroll
    for (int u = 0; u < kStep; ++u)
      if (p0 + u < end) load_lane<HD>(kb + (size_t)(p0 + u) * HD, lane, kf[u]);
#pragma unroll
    for (int u = 0; u < kStep; ++u)
      if (p0 + u < end) load_lane<HD>(vb + (size_t)(p0 + u) * HD, lane, vf[u]);
#pragma unroll
    for (int j = 0; j < GQ; ++j) {
      float sc[kStep];
#pragma unroll
      for (int u = 0; u < kStep; ++u) {
        float dsum = 0.f;
        if (p0 + u < end) {
#pragma unroll
          for (int e = 0; e < E; ++e) dsum = fmaf(qf[j][e], kf[u][e], dsum);
        }
        sc[u] = dsum;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < kStep; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
      }
      float mn = m[j];
#pragma unroll
      for (int u = 0; u < kStep; ++u) {
        sc[u] = (p0 + u < end) ? sc[u] * scale : -INFINITY;
        mn = fmaxf(mn, sc[u]);
      }
      const float corr = expf(m[j] - mn);
      l[j] *= corr;
#pragma unroll
      for (int e = 0; e < E; ++e) acc[j][e] *= corr;
#pragma unroll
      for (int u = 0; u < kStep; ++u) {
        if (p0 + u < end) {
          const float pe = expf(sc[u] - mn);
          l[j] += pe;
#pragma unroll
          for (int e = 0; e < E; ++e) acc[j][e] = fmaf(pe, vf[u][e], acc[j][e]);
        }
      }
      m[j] = mn;
    }
  }
  // per head: merge the warps in warp order (thread c owns output dim c), as attn_split_kernel
#pragma unroll
  for (int j = 0; j < GQ; ++j) {
    if (lane == 0) { sm[warp] = m[j]; sl[warp] = l[j]; }
#pragma unroll
    for (int e = 0; e < E; ++e) so[warp][lane * E + e] = acc[j][e];
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kSplitWarps; ++w) M = fmaxf(M, sm[w]);
    float L = 0.f;
    const size_t slot = ((size_t)t * Hq + g * GQ + j) * NS + s;
    for (int c = threadIdx.x; c < HD; c += blockDim.x) {
      float O = 0.f;
      L = 0.f;
      if (M != -INFINITY) {
#pragma unroll
        for (int w = 0; w < kSplitWarps; ++w) {
          const float f = expf(sm[w] - M);
          L += sl[w] * f;
          O += so[w][c] * f;
        }
      }
      part_o[slot * HD + c] = O;
    }
    if (threadIdx.x == 0) {
      part_ml[slot * 2] = M;
      part_ml[slot * 2 + 1] = L;
    }
    __syncthreads();
  }
}

template <int HD>
__global__ void __launch_bounds__(HD)
attn_merge_kernel(const float* part_o, const float* part_ml,
                  const bf16* qg, long ldp, bf16* out, long ldo, int Hq,
                  int NS) {
  dep_release();
  dep_wait();
  const int h = blockIdx.x, c = threadIdx.x, t = blockIdx.y;
  const size_t base = ((size_t)t * Hq + h) * NS;
  float M = -INFINITY;
  for (int s = 0; s < NS; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  float L = 0.f, O = 0.f;
  for (int s = 0; s < NS; ++s) {
    const float ms = part_ml[(base + s) * 2];
    if (ms == -INFINITY) continue;
    const float f = expf(ms - M);
    L += part_ml[(base + s) * 2 + 1] * f;
    O += part_o[(base + s) * HD + c] * f;
  }
  const float o = rnd(O / L);
  const float gate = tofloat(qg[(long)t * ldp + (size_t)h * 2 * HD + HD + c]);
  out[(long)t * ldo + (size_t)h * HD + c] = tobf16(o * rnd(sigmoid_acc(gate)));
}

inline bool pdl_on() { return pdl_launch_enabled() && pdl_trigger_enabled(); }

}  // namespace
}  // namespace qb

using namespace qb;

extern "C" int qe_attn_prep(const void* qg, const void* k, const void* v, long ldp, const void* qnw,
                            const void* knw, const float* inv_freq, const int* pos, void* q_out,
                            void* kc, void* vc, int n, int Hq, int Hkv, int hd, int max_len, int rd,
                            float eps, void* stream) {
  if (n < 1 || n > QE_MAX_ROWS || Hq < 1 || Hkv < 1 || rd < 0 || rd > hd || (rd & 1)) return QE_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid(Hq + Hkv, n);
#define QB_PREP(HD)                                                                              \
  return (int)launch(attn_prep_kernel<HD>, grid, dim3(HD), 0, s, pdl_on(), (const bf16*)qg,       \
                     (const bf16*)k, (const bf16*)v, ldp, (const bf16*)qnw, (const bf16*)knw,     \
                     inv_freq, pos, (bf16*)q_out, (bf16*)kc, (bf16*)vc, Hq, max_len, rd, eps)
  if (hd == 256) QB_PREP(256);
  if (hd == 128) QB_PREP(128);
  if (hd == 64) QB_PREP(64);
#undef QB_PREP
  return QE_ERR_ARG;
}

extern "C" int qe_attn_decode(const void* q, const void* kc, const void* vc, const int* pos,
                              const void* qg, long ldp, float* part_o, float* part_ml, void* out,
                              long ldo, int n, int Hq, int Hkv, int hd, int max_len, int NS,
                              float scale, void* stream) {
  if (n < 1 || n > QE_MAX_ROWS || Hq < 1 || Hkv < 1 || Hq % Hkv || NS < 1) return QE_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid(Hq, NS, n);
  const int gq = Hq / Hkv;
  const dim3 ggrid(Hkv, NS, n);
#define QB_GQA(HD, GQ)                                                                            \
  launch(attn_split_gqa_kernel<HD, GQ>, ggrid, dim3(kSplitWarps * 32), 0, s, pdl_on(),            \
         (const bf16*)q, (const bf16*)kc, (const bf16*)vc, pos, part_o, part_ml, Hq, max_len, scale)
#define QB_DEC(HD)                                                                                \
  {                                                                                               \
    int e;                                                                                        \
    if (gq == 2) e = (int)QB_GQA(HD, 2);                                                          \
    else if (gq == 3) e = (int)QB_GQA(HD, 3);                                                     \
    else if (gq == 4) e = (int)QB_GQA(HD, 4);                                                     \
    else if (gq == 6) e = (int)QB_GQA(HD, 6);                                                     \
    else                                                                                          \
      e = (int)launch(attn_split_kernel<HD>, grid, dim3(kSplitWarps * 32), 0, s, pdl_on(),        \
                      (const bf16*)q, (const bf16*)kc, (const bf16*)vc, pos, part_o, part_ml,     \
                      Hq, Hkv, max_len, scale);                                                   \
    if (e) return e;                                                                              \
    return (int)launch(attn_merge_kernel<HD>, dim3(Hq, n), dim3(HD), 0, s, pdl_on(),              \
                       (const float*)part_o, (const float*)part_ml, (const bf16*)qg, ldp,         \
                       (bf16*)out, ldo, Hq, NS);                                                  \
  }
  if (hd == 256) QB_DEC(256)
  if (hd == 128) QB_DEC(128)
  if (hd == 64) QB_DEC(64)
#undef QB_DEC
#undef QB_GQA
  return QE_ERR_ARG;
}
