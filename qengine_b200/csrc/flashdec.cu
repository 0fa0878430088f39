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

// Tensor-core split for head dim 256 and long caches. The query heads of a KV group are the M rows
// of mma.m16n8k16 (GQ <= 8 of 16 rows used): S = Q K^T and O += P V run on the tensor cores, which
// removes the per-(position, head) widening, FMAs and butterfly reductions that make the CUDA-core
// kernels issue-bound (72 warp-instructions per position and head there, about 2 here), so that the
// layer becomes what it should be: a stream of the KV cache.
//   CTA (row, KV head, 6 consecutive splits) = 6 warps, each a pipeline of its own on its own split
//   (sub-slice of the row's causal prefix): it streams 16 positions per stage (K rows, V rows,
//   512 B each, one bulk copy per row issued by lane = row, into a 528-byte pitch so that LDS.128 and ldmatrix are
//   conflict-free) into a warp-private ring of 2 stages (33 KB per warp, 198 KB per SM in flight).
//   Q K^T: the k index of the mma is permuted so that thread (g, t) feeds dims (4c + t) * 8 .. + 7
//   of its position / head from ONE 16-byte load per two k-steps -- a dot product does not care
//   about the order as long as A and B agree. P (bf16, as a flash-attention kernel keeps it) goes
//   from the score accumulators straight into A fragments; V^T fragments come from
//   ldmatrix.x4.trans. Online softmax state (m, l) is per head row; l is kept as per-thread partial
//   sums and reduced once at the end.
// The partial of a split is written like the other split kernels' (unnormalised O, m, l) and merged
// by attn_merge_kernel. Split boundaries depend on the row's prefix length and NS only: row t of an
// n-row call is bit-identical to a 1-row call. Waits are bounded (g_attn_error = 3).
constexpr int kMmaWarps = 6, kMmaPos = 16, kMmaStages = 2, kRowPitch = 528;
constexpr int kMmaStageBytes = 2 * kMmaPos * kRowPitch;  // K rows, then V rows

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int GQ>
__global__ void __launch_bounds__(kMmaWarps * 32, 1)
attn_mma_kernel(const bf16* q, const bf16* kc, const bf16* vc, const int* pos_ptr, float* part_o, float* part_ml,
                int Hq, int max_len, float scale) {
  constexpr int HD = 256;
  dep_release();
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ uint64_t full[kMmaWarps][kMmaStages];
  // the row is the fastest grid index: the CTAs of the rows of a verify pass that read the same
  // slice of the cache run at the same time, so the slice comes from HBM once and from L2 after
  const int t = blockIdx.x, g = blockIdx.y, NS = gridDim.z * kMmaWarps;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.z * kMmaWarps + warp;
  unsigned char* wring = ring + (size_t)warp * kMmaStages * kMmaStageBytes;
  if (lane == 0) {
    for (int i = 0; i < kMmaStages; ++i)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&full[warp][i])), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  dep_wait();
  const int len = min(max(pos_ptr[0] + t + 1, 0), max_len);
  const int chunk = (len + NS - 1) / NS;
  const int start = s * chunk, end = min(len, start + chunk);
  const int nstage = end > start ? (end - start + kMmaPos - 1) / kMmaPos : 0;
  const bf16* kb = kc + (size_t)g * max_len * HD;
  const bf16* vb = vc + (size_t)g * max_len * HD;

  // whole warp: lane 0 arms the barrier, then lane r issues the two row copies of position r
  // (32 copies issued by one lane would serialise into microseconds per stage)
  auto refill = [&](int st) {
    const int slot = st % kMmaStages;
    const int p0 = start + st * kMmaPos, cnt = min(kMmaPos, end - p0);
    unsigned char* dst = wring + (size_t)slot * kMmaStageBytes;
    const uint32_t bar = smem_addr(&full[warp][slot]);
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)cnt * 1024u) : "memory");
    __syncwarp();
    if (lane < cnt) {
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       smem_addr(dst + lane * kRowPitch)), "l"(kb + (size_t)(p0 + lane) * HD), "r"(512u), "r"(bar) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       smem_addr(dst + (kMmaPos + lane) * kRowPitch)), "l"(vb + (size_t)(p0 + lane) * HD), "r"(512u),
                   "r"(bar)
                   : "memory");
    }
  };
  for (int st = 0; st < min(kMmaStages, nstage); ++st) refill(st);

  // A fragments of Q: row = head g * GQ + gi, thread column tq; chunk 4c + tq of the row (8 dims)
  // serves k-steps 2c (words 0, 1) and 2c + 1 (words 2, 3). Rows >= GQ are zero.
  const int gi = lane >> 2, tq = lane & 3;
  uint32_t qa[8][4];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (gi < GQ) v = reinterpret_cast<const uint4*>(q + ((size_t)t * Hq + g * GQ + gi) * HD)[4 * c + tq];
    qa[c][0] = v.x; qa[c][1] = v.y; qa[c][2] = v.z; qa[c][3] = v.w;
  }
  float oacc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  float m = -INFINITY, lsum = 0.f;
  bool ok = true;

  for (int st = 0; st < nstage && ok; ++st) {
    const int slot = st % kMmaStages;
    if (!bar_wait(&full[warp][slot], (st / kMmaStages) & 1)) {
      atomicExch(&g_attn_error, 3);
      ok = false;
      break;
    }
    unsigned char* kst = wring + (size_t)slot * kMmaStageBytes;
    unsigned char* vst = kst + kMmaPos * kRowPitch;
    const int cnt = min(kMmaPos, end - start - st * kMmaPos);
    if (cnt < kMmaPos) {  // stale rows behind a short last stage must not reach the P V product
      for (int r = cnt; r < kMmaPos; ++r)
        reinterpret_cast<uint4*>(vst + r * kRowPitch)[lane] = make_uint4(0u, 0u, 0u, 0u);
      __syncwarp();
    }
    // S = Q K^T for the two 8-position blocks of the stage
    float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        const uint4 kw = *reinterpret_cast<const uint4*>(kst + (nb * 8 + gi) * kRowPitch + (4 * c + tq) * 16);
        mma_bf16(sacc[nb], qa[c][0], 0u, qa[c][1], 0u, kw.x, kw.y);
        mma_bf16(sacc[nb], qa[c][2], 0u, qa[c][3], 0u, kw.z, kw.w);
      }
    }
    // online softmax of head row gi over positions 8 nb + 2 tq + {0, 1}
    float sc[2][2], bm = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        sc[nb][j] = (nb * 8 + 2 * tq + j < cnt) ? sacc[nb][j] * scale : -INFINITY;
        bm = fmaxf(bm, sc[nb][j]);
      }
    }
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
    const float mn = fmaxf(m, bm);
    const float corr = expf(m - mn);  // first stage: exp(-inf) = 0
    float pr[2][2];
    lsum *= corr;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        pr[nb][j] = expf(sc[nb][j] - mn);
        lsum += pr[nb][j];
      }
    }
    m = mn;
    const uint32_t pa0 = pack2(pr[0][0], pr[0][1]), pa2 = pack2(pr[1][0], pr[1][1]);
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { oacc[i][0] *= corr; oacc[i][1] *= corr; }
    // O += P V: V^T fragments for two 8-dim blocks per ldmatrix.x4.trans
    const uint32_t vaddr = smem_addr(vst + (((lane >> 3) & 1) * 8 + (lane & 7)) * kRowPitch + (lane >> 4) * 16);
#pragma unroll
    for (int i = 0; i < HD / 8; i += 2) {
      uint32_t b0, b1, b2, b3;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(vaddr + i * 16));
      mma_bf16(oacc[i], pa0, 0u, pa2, 0u, b0, b1);
      mma_bf16(oacc[i + 1], pa0, 0u, pa2, 0u, b2, b3);
    }
    __syncwarp();
    if (st + kMmaStages < nstage) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      refill(st + kMmaStages);
    }
  }
  lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
  lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
  if (gi < GQ) {
    const bool none = m == -INFINITY;
    const size_t slot_o = ((size_t)t * Hq + g * GQ + gi) * NS + s;
    float2* po = reinterpret_cast<float2*>(part_o + slot_o * HD) + tq;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) po[i * 4] = none ? make_float2(0.f, 0.f) : make_float2(oacc[i][0], oacc[i][1]);
    if (tq == 0) {
      part_ml[slot_o * 2] = m;
      part_ml[slot_o * 2 + 1] = none ? 0.f : lsum;
    }
  }
}

// Merge of the NS split partials of one (head, row). Phase 1: the (m, l) pairs of all splits go to
// shared memory in one coalesced sweep, M = max m, weight f_s = exp(m_s - M), L = sum l_s f_s
// (block reduction in a fixed order). Phase 2: warp w adds O_s f_s over splits w, w + 8, ... in
// ascending order with independent 16-byte loads in flight (lane = HD / 32 consecutive dims), the 8
// warps are combined in warp order, then o = bf16(O / L) * bf16(sigmoid(gate)). With hundreds of
// splits (long caches) a loop whose loads wait for each other would cost as much as the split
// kernel itself. The order depends on NS only.
constexpr int kMergeMaxSplits = 1024;
template <int HD>
__global__ void __launch_bounds__(kSplitWarps * 32)
attn_merge_kernel(const float* part_o, const float* part_ml, const bf16* qg, long ldp, bf16* out, long ldo,
                  int Hq, int NS) {
  constexpr int E = HD / 32;
  dep_release();
  dep_wait();
  __shared__ float fs[kMergeMaxSplits];
  __shared__ float red[32];
  __shared__ float so[kSplitWarps][HD];
  const int h = blockIdx.x, t = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t base = ((size_t)t * Hq + h) * NS;
  const float2* ml = reinterpret_cast<const float2*>(part_ml) + base;
  // phase 1
  float mymax = -INFINITY;
  for (int s = threadIdx.x; s < NS; s += blockDim.x) mymax = fmaxf(mymax, ml[s].x);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mymax = fmaxf(mymax, __shfl_xor_sync(0xffffffffu, mymax, o));
  if (lane == 0) red[warp] = mymax;
  __syncthreads();
  float M = red[0];
#pragma unroll
  for (int w = 1; w < kSplitWarps; ++w) M = fmaxf(M, red[w]);
  float lpart = 0.f;
  for (int s = threadIdx.x; s < NS; s += blockDim.x) {
    const float2 v = ml[s];
    const float f = v.x == -INFINITY ? 0.f : expf(v.x - M);
    fs[s] = f;
    lpart += v.y * f;
  }
  const float L = block_allsum(lpart, red);  // barriers inside also publish fs
  // phase 2
  float o[E];
#pragma unroll
  for (int e = 0; e < E; ++e) o[e] = 0.f;
#pragma unroll 4
  for (int s = warp; s < NS; s += kSplitWarps) {
    const float f = fs[s];
    const float* po = part_o + (base + s) * HD + lane * E;
    float v[E];
    if constexpr (E == 8) {
      const float4 a = reinterpret_cast<const float4*>(po)[0], b = reinterpret_cast<const float4*>(po)[1];
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) v[e] = po[e];
    }
#pragma unroll
    for (int e = 0; e < E; ++e) o[e] = fmaf(v[e], f, o[e]);
  }
#pragma unroll
  for (int e = 0; e < E; ++e) so[warp][lane * E + e] = o[e];
  __syncthreads();
  for (int c = threadIdx.x; c < HD; c += blockDim.x) {
    float O = 0.f;
#pragma unroll
    for (int w = 0; w < kSplitWarps; ++w) O += so[w][c];
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
  if (n < 1 || n > QE_MAX_ROWS || Hq < 1 || Hkv < 1 || Hq % Hkv || NS < 1 || NS > kMergeMaxSplits) return QE_ERR_ARG;
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
  if (hd == 256 && NS % kMmaWarps == 0 && gq >= 1 && gq <= 8) {
    const dim3 mgrid(n, Hkv, NS / kMmaWarps);
    constexpr size_t msmem = (size_t)kMmaWarps * kMmaStages * kMmaStageBytes;
    int e = QE_ERR_ARG;
#define QB_MMA(GQ)                                                                                \
  {                                                                                               \
    static bool attr = false;                                                                     \
    if (!attr) {                                                                                  \
      cudaFuncSetAttribute(attn_mma_kernel<GQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)msmem); \
      attr = true;                                                                                \
    }                                                                                             \
    e = (int)launch(attn_mma_kernel<GQ>, mgrid, dim3(kMmaWarps * 32), msmem, s, pdl_on(), (const bf16*)q, \
                    (const bf16*)kc, (const bf16*)vc, pos, part_o, part_ml, Hq, max_len, scale);   \
  }
    switch (gq) {
      case 1: QB_MMA(1) break;
      case 2: QB_MMA(2) break;
      case 3: QB_MMA(3) break;
      case 4: QB_MMA(4) break;
      case 6: QB_MMA(6) break;
      case 8: QB_MMA(8) break;
      default: e = -1; break;
    }
#undef QB_MMA
    if (e == 0)
      return (int)launch(attn_merge_kernel<256>, dim3(Hq, n), dim3(kSplitWarps * 32), 0, s, pdl_on(),
                         (const float*)part_o, (const float*)part_ml, (const bf16*)qg, ldp, (bf16*)out, ldo, Hq, NS);
    if (e > 0) return e;
  }
  if (hd == 256) QB_DEC(256)
  if (hd == 128) QB_DEC(128)
  if (hd == 64) QB_DEC(64)
#undef QB_DEC
#undef QB_GQA
  return QE_ERR_ARG;
}
