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
#include <algorithm>

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

// Tensor-core split for head dim 256 and long caches. The (pass row, query head) pairs that share a
// KV head are the M rows of mma.m16n8k16, packed densely: pair e = row * GQ + head sits in tile
// e / 16 at tile row e % 16, so the 30 pairs of a 5-row verify pass over 6 heads fill two tiles and
// S = Q K^T and O += P V of all five rows cost the tensor-core work of two. The per-(position,
// head) widening, FMAs and butterfly reductions that make the CUDA-core kernels issue-bound (72
// warp-instructions per position and head there, about 2 here) are gone and the layer becomes
// what it should be: a stream of the KV cache.
//
// One K/V stream serves all rows of a pass. The cache positions are cut into splits of C
// consecutive positions, C = 16 * ceil(len / (16 NS)) with len the row's own prefix length: split
// s of a row is [s C, (s + 1) C) clipped to the prefix, whatever else is in the pass. The rows of
// one pass have prefix lengths pos + 1 .. pos + n and therefore the same C, except when a multiple
// of 16 NS lies between them; then the rows on either side are served one after the other (two
// phases over the same code, rows of the other phase masked out). Within a phase a GROUP of
// WPG = ceil(n GQ / 16) warps (one per tile) works on a split: the group streams the split's K and V rows, 16
// positions per stage (1 KB per position; nine bulk copies per stage, see v_row) through a ring that all
// warps of the group read, warp w applying them to the pairs of tile w. full[] barriers count the
// bytes of a stage, empty[] barriers the warps that are done with it; the warp whose turn it is
// refills a stage once it is empty. 198 KB of stages per SM: 6 groups x 2 stages (one tile),
// 4 x 3 (two), 2 x 6 (three or four). A CTA is (KV head, z); its groups take the splits
// z GPC + group, + Z GPC, ... one after the other, the ring running across split boundaries.
//
//   Q K^T: the k index of the mma is permuted so that thread (g, t) feeds dims (4c + t) * 8 .. + 7
//   of its position / head from ONE 16-byte load per two k-steps -- a dot product does not care
//   about the order as long as A and B agree; four accumulators (two position blocks x even / odd
//   k-steps) keep dependent mma instructions apart. P goes from the score accumulators straight
//   into A fragments. For rows with at most kExactLen cached positions it goes as TWO bf16 numbers
//   per probability, its bf16 rounding and the bf16 rounding of what that left over: one bf16
//   alone costs 2^-9 relative per term, which shows in the last bits of the output when few terms
//   carry the sum; over thousands of positions the errors average out and the second product per
//   V fragment is not spent. V^T fragments come from ldmatrix.x4.trans. Online softmax state (m, l) is per head row; l is kept as per-thread partial
//   sums and reduced once at the end of a split.
//
// Positions of a stage that lie beyond a row's prefix get probability 0; their V rows are read
// all the same (times 0), so cache rows up to 15 positions past the longest prefix must hold
// finite numbers -- they do: the cache starts zeroed and is only written by attn_prep_kernel.
// The partial of a split is written like the other split kernels' (unnormalised O, m, l) and merged
// by attn_merge_kernel. Nothing a row computes depends on n or on the other rows: row t of an
// n-row call is bit-identical to a 1-row call. Waits are bounded (g_attn_error = 3).
constexpr int kMmaPos = 16, kMmaRingStages = 12, kExactLen = 4096;
constexpr int kRowBytes = 512;                   // one cached position of one KV head (256 x bf16)
constexpr int kVPairPitch = 2 * kRowBytes + 16;  // two V rows, then 16 bytes of padding
constexpr int kMmaStageBytes = kMmaPos * kRowBytes + (kMmaPos / 2) * kVPairPitch;  // K rows, then V row pairs

// Stage layout. K rows are dense (one copy per stage; the 16-byte loads of Q K^T, two tile rows per
// quarter warp, are two-way bank conflicts either way). V rows go in pairs, each pair 16 bytes
// further round the banks than the last, so that the eight row addresses of an ldmatrix fall into
// four bank groups (two-way conflicts) with eight copies per stage; one row per copy would be
// conflict-free but costs sixteen copies, which the issuing warp pays one after the other.
__device__ __forceinline__ unsigned char* v_row(unsigned char* stage, int r) {
  return stage + kMmaPos * kRowBytes + (r >> 1) * kVPairPitch + (r & 1) * kRowBytes;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __host__ __forceinline__ int split_len(int len, int NS) {
  const int per = 16 * NS;
  return 16 * max(1, (len + per - 1) / per);
}

// Where a group stands in its list of (phase, split, stage) items; every warp of the group steps
// an identical copy, so no communication is needed to agree on the next item.
struct MmaCursor {
  int ph, s, st, nst;
};

// groups per CTA for WPG warps per group: 6 x 1, 4 x 2, 2 x 3, 2 x 4 warps (255 registers each)
__host__ __device__ constexpr int mma_groups(int wpg) { return wpg == 1 ? 6 : wpg == 2 ? 4 : 2; }

template <int WPG>
__global__ void __launch_bounds__(mma_groups(WPG) * WPG * 32, 1)
attn_mma_kernel(const bf16* q, const bf16* kc, const bf16* vc, const int* pos_ptr, float* part_o, float* part_ml,
                int Hq, int GQ, int max_len, int n, int NS, float scale) {
  constexpr int HD = 256;
  constexpr int GPC = mma_groups(WPG);         // groups per CTA
  constexpr int SPG = kMmaRingStages / GPC;    // ring stages per group
  dep_release();
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ uint64_t full[GPC][SPG], empty[GPC][SPG];
  const int g = blockIdx.x, stride = gridDim.y * GPC;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = warp / WPG, wig = warp % WPG;
  unsigned char* gring = ring + (size_t)grp * SPG * kMmaStageBytes;
  if (threadIdx.x == 0) {
    for (int a = 0; a < GPC; ++a)
      for (int i = 0; i < SPG; ++i) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&full[a][i])), "r"(1));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&empty[a][i])), "r"(WPG));
      }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  dep_wait();
  const int pos0 = pos_ptr[0];
  auto row_len = [&](int r) { return min(max(pos0 + r + 1, 0), max_len); };
  // phases: rows whose split length equals that of row 0, then (rarely) the rest
  const int c_first = split_len(row_len(0), NS), c_last = split_len(row_len(n - 1), NS);
  const int nphase = c_first == c_last ? 1 : 2;
  int lmax0 = 0;  // longest prefix among the rows of phase 0
  for (int r = 0; r < n; ++r)
    if (split_len(row_len(r), NS) == c_first) lmax0 = row_len(r);
  auto phase_c = [&](int ph) { return ph == 0 ? c_first : c_last; };
  auto phase_lmax = [&](int ph) { return ph == 0 ? lmax0 : row_len(n - 1); };
  auto stages_of = [&](int ph, int s) {
    const int C = phase_c(ph);
    return min(max((phase_lmax(ph) - s * C + kMmaPos - 1) / kMmaPos, 0), C / kMmaPos);
  };
  const int s_first = blockIdx.y * GPC + grp;
  // the producer's cursor: next stage to request
  MmaCursor pc{0, s_first, 0, 0};
  auto settle = [&](MmaCursor& c) {  // move to the next existing stage at or after (ph, s, st)
    while (c.ph < nphase) {
      if (c.s < NS) {
        c.nst = stages_of(c.ph, c.s);
        if (c.st < c.nst) return true;
        c.s += stride;
        c.st = 0;
      } else {
        ++c.ph;
        c.s = s_first;
        c.st = 0;
      }
    }
    return false;
  };
  const bf16* kb = kc + (size_t)g * max_len * HD;
  const bf16* vb = vc + (size_t)g * max_len * HD;
  int issued = 0, done = 0;  // stages requested / consumed by this group so far
  bool ok = true;
  // Requests the stage under the producer cursor if it is this warp's turn; every warp advances
  // the cursor. The warp whose turn it is first waits until the slot's previous stage was read by
  // all warps of the group.
  auto request_next = [&]() {
    if (!settle(pc)) return;
    const int slot = issued % SPG, use = issued / SPG;
    if (issued % WPG == wig) {
      if (use > 0 && WPG > 1) {
        if (!bar_wait(&empty[grp][slot], (use - 1) & 1)) {
          atomicExch(&g_attn_error, 3);
          ok = false;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      if (ok) {
        const int p0 = pc.s * phase_c(pc.ph) + pc.st * kMmaPos, cnt = min(kMmaPos, max_len - p0);
        unsigned char* dst = gring + (size_t)slot * kMmaStageBytes;
        const uint32_t bar = smem_addr(&full[grp][slot]);
        if (cnt < kMmaPos) {  // end of the cache: V rows nobody copies must still be numbers
          for (int r = cnt; r < kMmaPos; ++r)
            reinterpret_cast<uint4*>(v_row(dst, r))[lane] = make_uint4(0u, 0u, 0u, 0u);
          __syncwarp();
        }
        if (lane == 0)
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)cnt * 1024u) : "memory");
        __syncwarp();
        // nine copies per stage, one lane each (a bulk copy is a warp-uniform instruction: copies
        // with per-lane operands are issued one after the other, so fewer and larger is faster):
        // lane 0 the K rows in one piece, lanes 1..8 two V rows each
        if (lane == 0) {
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                           smem_addr(dst)), "l"(kb + (size_t)p0 * HD), "r"((uint32_t)cnt * 512u), "r"(bar) : "memory");
        } else if (lane <= kMmaPos / 2 && 2 * (lane - 1) < cnt) {
          const int r = 2 * (lane - 1);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                           smem_addr(v_row(dst, r))), "l"(vb + (size_t)(p0 + r) * HD), "r"((uint32_t)min(2, cnt - r) * 512u),
                       "r"(bar)
                       : "memory");
        }
      }
    }
    ++issued;
    ++pc.st;
  };
  for (int i = 0; i < SPG; ++i) request_next();

  // A fragments of Q. This thread serves pairs e[0] = 16 wig + gi (tile rows 0..7) and e[1] =
  // e[0] + 8 (tile rows 8..15), pair e = pass row e / GQ, head e % GQ, in thread column tq:
  // chunk 4c + tq of the query (8 dims) serves k-steps 2c (words 0, 1) and 2c + 1 (words 2, 3).
  // Tile rows past the last pair are zero.
  constexpr int NH = 2;  // halves of a tile: rows 0..7 and 8..15
  const int gi = lane >> 2, tq = lane & 3;
  const int npair = n * GQ;
  bool has[NH], ex[NH];
  int row[NH], head[NH], len[NH], cl[NH];
  uint32_t qa[NH][8][4];
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    const int e = 16 * wig + gi + 8 * h;
    has[h] = e < npair;
    row[h] = has[h] ? e / GQ : 0;
    head[h] = g * GQ + (has[h] ? e % GQ : 0);
    len[h] = has[h] ? row_len(row[h]) : 0;
    cl[h] = split_len(len[h], NS);
    ex[h] = len[h] <= kExactLen;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (has[h]) v = reinterpret_cast<const uint4*>(q + ((size_t)row[h] * Hq + head[h]) * HD)[4 * c + tq];
      qa[h][c][0] = v.x; qa[h][c][1] = v.y; qa[h][c][2] = v.z; qa[h][c][3] = v.w;
    }
  }
  // the remainder product is spent when a pair of this warp has a short prefix (warp-uniform)
  bool exact_lane = false;
#pragma unroll
  for (int h = 0; h < NH; ++h) exact_lane = exact_lane || (has[h] && ex[h]);
  const bool exact = __any_sync(0xffffffffu, exact_lane);
  constexpr int LAST = NH - 1;

  for (int ph = 0; ph < nphase && ok; ++ph) {
    const int C = phase_c(ph);
    for (int s = s_first; s < NS && ok; s += stride) {
      const int nst = stages_of(ph, s);
      bool act[NH];
      int lim[NH];  // positions below it are in the pair's prefix
      float m[NH], l[NH];
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        act[h] = has[h] && cl[h] == C;
        lim[h] = act[h] ? min(len[h], (s + 1) * C) : 0;
        m[h] = -INFINITY;
        l[h] = 0.f;
      }
      float oacc[HD / 8][2 * NH];
#pragma unroll
      for (int i = 0; i < HD / 8; ++i)
#pragma unroll
        for (int j = 0; j < 2 * NH; ++j) oacc[i][j] = 0.f;
      for (int st = 0; st < nst; ++st) {
        const int slot = done % SPG;
        if (!bar_wait(&full[grp][slot], (done / SPG) & 1)) {
          atomicExch(&g_attn_error, 3);
          ok = false;
          break;
        }
        unsigned char* kst = gring + (size_t)slot * kMmaStageBytes;
        const int p0 = s * C + st * kMmaPos;
        // S = Q K^T for the two 8-position blocks of the stage; even and odd k-steps accumulate
        // apart and are added at the end
        float sacc[2][2][2 * NH];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
          for (int j = 0; j < 2 * NH; ++j) sacc[nb][0][j] = sacc[nb][1][j] = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 k0 = *reinterpret_cast<const uint4*>(kst + gi * kRowBytes + (4 * c + tq) * 16);
          const uint4 k1 = *reinterpret_cast<const uint4*>(kst + (8 + gi) * kRowBytes + (4 * c + tq) * 16);
          mma_bf16(sacc[0][0], qa[0][c][0], qa[LAST][c][0], qa[0][c][1], qa[LAST][c][1], k0.x, k0.y);
          mma_bf16(sacc[1][0], qa[0][c][0], qa[LAST][c][0], qa[0][c][1], qa[LAST][c][1], k1.x, k1.y);
          mma_bf16(sacc[0][1], qa[0][c][2], qa[LAST][c][2], qa[0][c][3], qa[LAST][c][3], k0.z, k0.w);
          mma_bf16(sacc[1][1], qa[0][c][2], qa[LAST][c][2], qa[0][c][3], qa[LAST][c][3], k1.z, k1.w);
        }
        // online softmax of a pair over positions p0 + 8 nb + 2 tq + {0, 1}
        uint32_t pa[2][NH], pl[2][NH];  // P = pa + pl: bf16 head, bf16 remainder; [position block][half]
        float corr[NH];
        bool rescale = false;
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          float sc[2][2], bm = -INFINITY;
#pragma unroll
          for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const float sv = sacc[nb][0][2 * h + j] + sacc[nb][1][2 * h + j];
              sc[nb][j] = (p0 + nb * 8 + 2 * tq + j < lim[h]) ? sv * scale : -INFINITY;
              bm = fmaxf(bm, sc[nb][j]);
            }
          }
          bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
          bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
          const float mn = fmaxf(m[h], bm);
          // a stage without a position of this pair leaves its state alone (mn = -inf only then)
          const bool any = mn != -INFINITY;
          corr[h] = any ? expf(m[h] - mn) : 1.f;  // first stage: exp(-inf) = 0
          rescale = rescale || corr[h] != 1.f;
          float pr[2][2];
          l[h] *= corr[h];
#pragma unroll
          for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              pr[nb][j] = any ? expf(sc[nb][j] - mn) : 0.f;
              l[h] += pr[nb][j];
            }
          }
          m[h] = mn;
#pragma unroll
          for (int nb = 0; nb < 2; ++nb) {
            const uint32_t hi = pack2(pr[nb][0], pr[nb][1]);
            pa[nb][h] = hi;
            pl[nb][h] = (exact && ex[h]) ? pack2(pr[nb][0] - __uint_as_float(hi << 16),
                                                 pr[nb][1] - __uint_as_float(hi & 0xffff0000u))
                                         : 0u;
          }
        }
        // rescale only when some pair of the warp saw a new maximum (times 1 changes nothing)
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
          for (int i = 0; i < HD / 8; ++i)
#pragma unroll
            for (int j = 0; j < 2 * NH; ++j) oacc[i][j] *= corr[j >> 1];
        }
        // O += P V: V^T fragments for two 8-dim blocks per ldmatrix.x4.trans
        const uint32_t vaddr = smem_addr(v_row(kst, ((lane >> 3) & 1) * 8 + (lane & 7)) + (lane >> 4) * 16);
        if (exact) {
          // the remainder product of a block follows the head product of the next block, so that
          // no mma waits for the one issued just before it
          uint32_t p0r = 0u, p1r = 0u, p2r = 0u, p3r = 0u;
#pragma unroll
          for (int i = 0; i < HD / 8; i += 2) {
            uint32_t b0, b1, b2, b3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(vaddr + i * 16));
            mma_bf16(oacc[i], pa[0][0], pa[0][LAST], pa[1][0], pa[1][LAST], b0, b1);
            mma_bf16(oacc[i + 1], pa[0][0], pa[0][LAST], pa[1][0], pa[1][LAST], b2, b3);
            if (i > 0) {
              mma_bf16(oacc[i - 2], pl[0][0], pl[0][LAST], pl[1][0], pl[1][LAST], p0r, p1r);
              mma_bf16(oacc[i - 1], pl[0][0], pl[0][LAST], pl[1][0], pl[1][LAST], p2r, p3r);
            }
            p0r = b0; p1r = b1; p2r = b2; p3r = b3;
          }
          mma_bf16(oacc[HD / 8 - 2], pl[0][0], pl[0][LAST], pl[1][0], pl[1][LAST], p0r, p1r);
          mma_bf16(oacc[HD / 8 - 1], pl[0][0], pl[0][LAST], pl[1][0], pl[1][LAST], p2r, p3r);
        } else {
#pragma unroll
          for (int i = 0; i < HD / 8; i += 2) {
            uint32_t b0, b1, b2, b3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(vaddr + i * 16));
            mma_bf16(oacc[i], pa[0][0], pa[0][LAST], pa[1][0], pa[1][LAST], b0, b1);
            mma_bf16(oacc[i + 1], pa[0][0], pa[0][LAST], pa[1][0], pa[1][LAST], b2, b3);
          }
        }
        __syncwarp();
        if (WPG > 1 && lane == 0)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&empty[grp][slot])) : "memory");
        ++done;
        if (WPG == 1) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        request_next();
        if (!ok) break;
      }
      if (!ok) break;
      // the split's partials of this thread's pairs (pairs of the other phase are written there;
      // a split without a position of the pair's prefix is not written: the merge skips it)
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        float lh = l[h];
        lh += __shfl_xor_sync(0xffffffffu, lh, 1);
        lh += __shfl_xor_sync(0xffffffffu, lh, 2);
        if (!act[h] || s * C >= len[h]) continue;
        const bool none = m[h] == -INFINITY;
        const size_t slot_o = ((size_t)row[h] * Hq + head[h]) * NS + s;
        float2* po = reinterpret_cast<float2*>(part_o + slot_o * HD) + tq;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i)
          po[i * 4] = none ? make_float2(0.f, 0.f) : make_float2(oacc[i][2 * h], oacc[i][2 * h + 1]);
        if (tq == 0) {
          part_ml[slot_o * 2] = m[h];
          part_ml[slot_o * 2 + 1] = none ? 0.f : lh;
        }
      }
    }
  }
}

// Merge of the split partials of one (head, row). Phase 1: the (m, l) pairs of the splits go to
// shared memory in one coalesced sweep, M = max m, weight f_s = exp(m_s - M), L = sum l_s f_s
// (block reduction in a fixed order). Phase 2: warp w adds O_s f_s over splits w, w + 16, ... in
// ascending order, eight 16-byte loads per lane in flight (lane = HD / 32 consecutive dims), the
// 16 warps are combined in warp order, then o = bf16(O / L) * bf16(sigmoid(gate)). With hundreds
// of splits (long caches) a loop whose loads wait for each other costs as much as the split
// kernel itself: 8 warps with four loads in flight took 13 us for 222 splits. The order depends
// on the number of splits merged only. With `aligned` (partials of attn_mma_kernel) that number
// is the count of splits that hold a position of the row's prefix, ceil(len / split length);
// the others were not written and are not read.
constexpr int kMergeMaxSplits = 1024, kMergeWarps = 16;
template <int HD>
__global__ void __launch_bounds__(kMergeWarps * 32)
attn_merge_kernel(const float* part_o, const float* part_ml, const bf16* qg, long ldp, bf16* out, long ldo,
                  int Hq, int NS, const int* pos_ptr, int max_len, int aligned) {
  constexpr int E = HD / 32;
  dep_release();
  dep_wait();
  __shared__ float fs[kMergeMaxSplits];
  __shared__ float red[32];
  __shared__ float so[kMergeWarps][HD];
  const int h = blockIdx.x, t = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int ns = NS;
  if (aligned) {
    const int len = min(max(pos_ptr[0] + t + 1, 0), max_len);
    const int C = split_len(len, NS);
    ns = min(NS, (len + C - 1) / C);
  }
  const size_t base = ((size_t)t * Hq + h) * NS;
  const float2* ml = reinterpret_cast<const float2*>(part_ml) + base;
  // phase 1
  float mymax = -INFINITY;
  for (int s = threadIdx.x; s < ns; s += blockDim.x) mymax = fmaxf(mymax, ml[s].x);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mymax = fmaxf(mymax, __shfl_xor_sync(0xffffffffu, mymax, o));
  if (lane == 0) red[warp] = mymax;
  __syncthreads();
  float M = red[0];
#pragma unroll
  for (int w = 1; w < kMergeWarps; ++w) M = fmaxf(M, red[w]);
  float lpart = 0.f;
  for (int s = threadIdx.x; s < ns; s += blockDim.x) {
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
  constexpr int kFlight = 8;
  for (int s0 = warp; s0 < ns; s0 += kMergeWarps * kFlight) {
    float v[kFlight][E];
#pragma unroll
    for (int j = 0; j < kFlight; ++j) {
      const int sj = s0 + j * kMergeWarps;
      if (sj < ns) {
        const float* po = part_o + (base + sj) * HD + lane * E;
        if constexpr (E == 8) {
          const float4 a = reinterpret_cast<const float4*>(po)[0], b = reinterpret_cast<const float4*>(po)[1];
          v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w;
          v[j][4] = b.x; v[j][5] = b.y; v[j][6] = b.z; v[j][7] = b.w;
        } else {
#pragma unroll
          for (int e = 0; e < E; ++e) v[j][e] = po[e];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kFlight; ++j) {
      const int sj = s0 + j * kMergeWarps;
      if (sj < ns) {
        const float f = fs[sj];
#pragma unroll
        for (int e = 0; e < E; ++e) o[e] = fmaf(v[j][e], f, o[e]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < E; ++e) so[warp][lane * E + e] = o[e];
  __syncthreads();
  for (int c = threadIdx.x; c < HD; c += blockDim.x) {
    float O = 0.f;
#pragma unroll
    for (int w = 0; w < kMergeWarps; ++w) O += so[w][c];
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
    return (int)launch(attn_merge_kernel<HD>, dim3(Hq, n), dim3(kMergeWarps * 32), 0, s, pdl_on(), \
                       (const float*)part_o, (const float*)part_ml, (const bf16*)qg, ldp,         \
                       (bf16*)out, ldo, Hq, NS, pos, max_len, 0);                                 \
  }
  if (hd == 256 && NS % 6 == 0 && gq >= 1 && gq <= 8) {
    // one CTA per (KV head, z); z covers the splits of a group stride with about one CTA per SM
    constexpr size_t msmem = (size_t)kMmaRingStages * kMmaStageBytes;
    const int wpg = (n * gq + 15) / 16, gpc = mma_groups(wpg);  // one warp per tile of 16 (row, head) pairs
    const int per_head = std::max(1, (qe_sm_count() + Hkv - 1) / Hkv);
    const dim3 mgrid(Hkv, std::min((NS + gpc - 1) / gpc, per_head));
    int e;
#define QB_MMA(WPG)                                                                               \
  {                                                                                               \
    static bool attr[64] = {};                                                                    \
    int dv = 0;                                                                                   \
    if (cudaGetDevice(&dv) != cudaSuccess || dv < 0 || dv >= 64) return QE_ERR_ARG;               \
    if (!attr[dv]) {                                                                              \
      cudaFuncSetAttribute(attn_mma_kernel<WPG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)msmem); \
      attr[dv] = true;                                                                            \
    }                                                                                             \
    e = (int)launch(attn_mma_kernel<WPG>, mgrid, dim3(mma_groups(WPG) * WPG * 32), msmem, s, pdl_on(), \
                    (const bf16*)q, (const bf16*)kc, (const bf16*)vc, pos, part_o, part_ml, Hq, gq, \
                    max_len, n, NS, scale);                                                       \
  }
    switch (wpg) {
      case 1: QB_MMA(1) break;
      case 2: QB_MMA(2) break;
      case 3: QB_MMA(3) break;
      default: QB_MMA(4) break;
    }
#undef QB_MMA
    if (e) return e;
    return (int)launch(attn_merge_kernel<256>, dim3(Hq, n), dim3(kMergeWarps * 32), 0, s, pdl_on(),
                       (const float*)part_o, (const float*)part_ml, (const bf16*)qg, ldp, (bf16*)out, ldo, Hq, NS,
                       pos, max_len, 1);
  }
  if (hd == 256) QB_DEC(256)
  if (hd == 128) QB_DEC(128)
  if (hd == 64) QB_DEC(64)
#undef QB_DEC
#undef QB_GQA
  return QE_ERR_ARG;
}
