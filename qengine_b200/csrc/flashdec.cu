// Gated GQA attention for decode / verify: n = 1..8 query rows at positions pos + t, causal over
// the KV cache. Boundary: replaces launch_attn_prep and launch_attn_decode of the reference
// (csrc/ops.h:25-30, kernels csrc/attn.cu:17-149); the math follows attention_qkv_from_proj and
// attention_core of the reference torch model (python/qengine/reference.py:252-272).
//
//   prep    per head: xn = bf16(x * rsqrt(mean x^2 + eps) * (1 + w)); rotate-half RoPE on the
//           first rd dims with bf16 rounding after every elementwise op (cos/sin rounded to
//           bf16 first); q -> q_out, k and raw v -> cache row pos + t (skipped past max_len).
//   decode  split-KV flash decoding: the row's causal prefix [0, pos + t] is cut into NS slices; a
//           CTA (KV head, split, row) streams its slice through shared memory once for all query
//           heads of the group (attn_stream_kernel; attn_split_kernel, one CTA per query head with
//           direct loads, serves group sizes outside {2, 3, 4, 6}); online softmax in fp32, four
//           positions per step; a second kernel merges the NS partials, rounds o = bf16(O / L)
//           and applies bf16(sigmoid(gate)).
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

// Grouped-query split fed through shared memory. CTA (KV head, split, row) = GQ consumer warps, one
// per query head of the group, + one producer warp whose lane 0 streams the K and V rows of the
// slice into a ring of kRingStages stages of kRingPos positions with bulk copies (cp.async.bulk,
// completion on an mbarrier). Every row is fetched from L2 / HBM once per group instead of once per
// query head, and a CTA needs few registers and 32 KB of shared memory, so several CTAs (dozens of
// warps) are resident per SM: with a long cache the layer is a pure KV stream (134 MB per layer at
// 32K positions of the 27B shape) and needs that many copies in flight. A consumer warp walks the
// positions of the slice in order, four at a time (lane = 8 consecutive dims, butterfly reduction,
// online softmax in fp32), and writes its own partial (no cross-warp merge). Slice boundaries
// depend only on the row's prefix length: row t of an n-row call is bit-identical to a 1-row call.
// Waits are bounded; a wait that runs out sets g_attn_error and the warp leaves.
constexpr int kRingPos = 8, kRingStages = 4;
__device__ int g_attn_error = 0;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ bool bar_wait(uint64_t* b, uint32_t parity, int limit = 1 << 22) {
  const uint32_t addr = smem_addr(b);
  for (int it = 0; it < limit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

template <int HD, int GQ>
__global__ void __launch_bounds__((GQ + 1) * 32)
attn_stream_kernel(const bf16* q, const bf16* kc, const bf16* vc, const int* pos_ptr, float* part_o,
                   float* part_ml, int Hq, int max_len, float scale) {
  constexpr int E = HD / 32;
  constexpr uint32_t kStageBytes = kRingPos * HD * 2;  // K (or V) rows of one stage
  dep_release();
  extern __shared__ __align__(128) unsigned char ring[];  // [stage][K rows | V rows]
  __shared__ uint64_t full[kRingStages], empty[kRingStages];
  const int g = blockIdx.x, s = blockIdx.y, NS = gridDim.y, t = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kRingStages; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&full[i])), "r"(1));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&empty[i])), "r"(GQ));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  dep_wait();  // pos, q and the newest cache rows come from kernels just before this one
  const int len = min(max(pos_ptr[0] + t + 1, 0), max_len);
  const int chunk = (len + NS - 1) / NS;
  const int start = s * chunk, end = min(len, start + chunk);
  const int nstage = end > start ? (end - start + kRingPos - 1) / kRingPos : 0;

  if (warp == GQ) {  // producer
    if (lane == 0) {
      const bf16* kb = kc + ((size_t)g * max_len + start) * HD;
      const bf16* vb = vc + ((size_t)g * max_len + start) * HD;
      for (int st = 0; st < nstage; ++st) {
        const int slot = st % kRingStages;
        if (st >= kRingStages && !bar_wait(&empty[slot], ((st / kRingStages) - 1) & 1)) {
          atomicExch(&g_attn_error, 1);
          break;
        }
        const uint32_t cnt = (uint32_t)min(kRingPos, end - start - st * kRingPos);
        const uint32_t bytes = cnt * HD * 2;
        unsigned char* dst = ring + (size_t)slot * 2 * kStageBytes;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(&full[slot])),
                     "r"(2 * bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_addr(dst)), "l"(kb + (size_t)st * kRingPos * HD), "r"(bytes), "r"(smem_addr(&full[slot]))
                     : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_addr(dst + kStageBytes)), "l"(vb + (size_t)st * kRingPos * HD), "r"(bytes),
                     "r"(smem_addr(&full[slot]))
                     : "memory");
      }
    }
    return;
  }

  const int h = g * GQ + warp;
  float qf[E], acc[E], m = -INFINITY, l = 0.f;
  load_lane<HD>(q + ((size_t)t * Hq + h) * HD, lane, qf);
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;

  for (int st = 0; st < nstage; ++st) {
    const int slot = st % kRingStages;
    if (!bar_wait(&full[slot], (st / kRingStages) & 1)) {
      atomicExch(&g_attn_error, 2);
      break;
    }
    const bf16* ks = reinterpret_cast<const bf16*>(ring + (size_t)slot * 2 * kStageBytes);
    const bf16* vs = reinterpret_cast<const bf16*>(ring + (size_t)slot * 2 * kStageBytes + kStageBytes);
    const int cnt = min(kRingPos, end - start - st * kRingPos);
#pragma unroll
    for (int p0 = 0; p0 < kRingPos; p0 += kStep) {
      if (p0 < cnt) {
        float sc[kStep];
#pragma unroll
        for (int u = 0; u < kStep; ++u) {
          float dsum = 0.f;
          if (p0 + u < cnt) {
            float kf[E];
            load_lane<HD>(ks + (size_t)(p0 + u) * HD, lane, kf);
#pragma unroll
            for (int e = 0; e < E; ++e) dsum = fmaf(qf[e], kf[e], dsum);
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
          sc[u] = (p0 + u < cnt) ? sc[u] * scale : -INFINITY;
          mn = fmaxf(mn, sc[u]);
        }
        const float corr = expf(m - mn);  // first step: exp(-inf) = 0
        l *= corr;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] *= corr;
#pragma unroll
        for (int u = 0; u < kStep; ++u) {
          if (p0 + u < cnt) {
            const float pe = expf(sc[u] - mn);
            l += pe;
            float vf[E];
            load_lane<HD>(vs + (size_t)(p0 + u) * HD, lane, vf);
#pragma unroll
            for (int e = 0; e < E; ++e) acc[e] = fmaf(pe, vf[e], acc[e]);
          }
        }
        m = mn;
      }
    }
    __syncwarp();
    if (lane == 0)
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&empty[slot])) : "memory");
  }
  // one warp = one head of one split: its running (m, l, acc) is the partial (acc is not yet
  // divided by l, as in attn_split_kernel)
  const size_t slot_o = ((size_t)t * Hq + h) * NS + s;
  float* po = part_o + slot_o * HD + lane * E;
#pragma unroll
  for (int e = 0; e < E; ++e) po[e] = (m == -INFINITY) ? 0.f : acc[e];
  if (lane == 0) {
    part_ml[slot_o * 2] = m;
    part_ml[slot_o * 2 + 1] = (m == -INFINITY) ? 0.f : l;
  }
}

// Merge of the NS split partials of one (head, row): warp w folds splits w, w + 8, ... into a
// running (M, L, O) in ascending order (lane = HD / 32 consecutive dims), the 8 warps are combined
// in warp order, then o = bf16(O / L) * bf16(sigmoid(gate)). The order depends on NS only.
template <int HD>
__global__ void __launch_bounds__(kSplitWarps * 32)
attn_merge_kernel(const float* part_o, const float* part_ml, const bf16* qg, long ldp, bf16* out, long ldo,
                  int Hq, int NS) {
  constexpr int E = HD / 32;
  dep_release();
  dep_wait();
  __shared__ float sm[kSplitWarps], sl[kSplitWarps];
  __shared__ float so[kSplitWarps][HD];
  const int h = blockIdx.x, t = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t base = ((size_t)t * Hq + h) * NS;
  float m = -INFINITY, l = 0.f, o[E];
#pragma unroll
  for (int e = 0; e < E; ++e) o[e] = 0.f;
#pragma unroll 4
  for (int s = warp; s < NS; s += kSplitWarps) {
    const float ms = part_ml[(base + s) * 2];
    if (ms == -INFINITY) continue;
    const float ls = part_ml[(base + s) * 2 + 1];
    const float* po = part_o + (base + s) * HD + lane * E;
    const float mn = fmaxf(m, ms);
    const float c1 = expf(m - mn), c2 = expf(ms - mn);  // first split: exp(-inf) = 0
    l = l * c1 + ls * c2;
#pragma unroll
    for (int e = 0; e < E; ++e) o[e] = o[e] * c1 + po[e] * c2;
    m = mn;
  }
  if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
  for (int e = 0; e < E; ++e) so[warp][lane * E + e] = o[e];
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < kSplitWarps; ++w) M = fmaxf(M, sm[w]);
  for (int c = threadIdx.x; c < HD; c += blockDim.x) {
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kSplitWarps; ++w) {
      if (sm[w] == -INFINITY) continue;
      const float f = expf(sm[w] - M);
      L += sl[w] * f;
      O += so[w][c] * f;
    }
    const float ob = rnd(O / L);
    const float gate = tofloat(qg[(long)t * ldp + (size_t)h * 2 * HD + HD + c]);
    out[(long)t * ldo + (size_t)h * HD + c] = tobf16(ob * rnd(sigmoid_acc(gate)));
  }
}

inline bool pdl_on() { return pdl_launch_enabled() && pdl_trigger_enabled(); }

template <int HD, int GQ>
cudaError_t launch_stream(dim3 grid, cudaStream_t s, bool pdl, const bf16* q, const bf16* kc, const bf16* vc,
                          const int* pos, float* part_o, float* part_ml, int Hq, int max_len, float scale) {
  constexpr size_t smem = (size_t)kRingStages * 2 * kRingPos * HD * 2;
  return launch(attn_stream_kernel<HD, GQ>, grid, dim3((GQ + 1) * 32), smem, s, pdl, q, kc, vc, pos, part_o,
                part_ml, Hq, max_len, scale);
}

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

extern "C" int qe_attn_error(void) {
  int h = 0;
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(&h, g_attn_error, sizeof(int));
  return h;
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
  launch_stream<HD, GQ>(ggrid, s, pdl_on(), (const bf16*)q, (const bf16*)kc, (const bf16*)vc, pos,  \
                        part_o, part_ml, Hq, max_len, scale)
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
    return (int)launch(attn_merge_kernel<HD>, dim3(Hq, n), dim3(kSplitWarps * 32), 0, s, pdl_on(),              \
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
