// Device-side core of the W4A16 GEMV kernels (w4_stream.cu): the unpack + mma k-step, tile
// epilogues, the deterministic finish of tiles cut across workers, and the mbarrier / bulk-copy
// helpers of the ring modes.
// See w4_stream.cu for the wire format and the determinism argument.
#pragma once
#include "../../include/qengine_b200.h"
#include "common.cuh"

namespace qb {
namespace {

struct W4Args {
  const uint4* qw;
  const __half* scales;
  const bf16* x;
  bf16* out;
  float* ws;
  int* counters;
  int M, K, N;
  int tiles, G;       // Mp / 16, Kp / 128
  long ldx, ldo;
  int ksplit;         // mode 0: gridDim.y
  int total;          // tiles * G
  int out_f32;        // plain epilogue only: store unrounded fp32 sums (tensor-parallel partials)
  int epi;            // QE_EPI_*, read by kernels instantiated with kEpiRuntime
};
// Template value "take the epilogue from W4Args::epi": lets one kernel function serve every
// matrix of a layer, so that consecutive launches run the same code (a launch of a different
// function starts with cold instruction caches, which costs microseconds on kernels this short).
constexpr int kEpiRuntime = 2;

__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// One k-step of 16: four A registers from one packed word, times two x pairs.
__device__ __forceinline__ void kstep(float (&c)[4], uint32_t w, uint32_t b0, uint32_t b1) {
  constexpr uint32_t kNib = 0x000F000Fu, k128 = 0x43004300u, k136 = 0x43084308u;
  const uint32_t a0 = sub_bf16x2(and_or(w, kNib, k128), k136);
  const uint32_t a1 = sub_bf16x2(and_or(w >> 4, kNib, k128), k136);
  const uint32_t a2 = sub_bf16x2(and_or(w >> 8, kNib, k128), k136);
  const uint32_t a3 = sub_bf16x2(and_or(w >> 12, kNib, k128), k136);
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same k-step for fp16 activations. fp16 has a 10-bit mantissa, so the magic number 1024
// (0x6400) takes a nibble either at bits 0..3 (value 1024 + u) or at bits 4..7 (1024 + 16 u) of a
// half-word: one shift by 8 serves all four A registers instead of three shifts, which matters
// because shifts and lop3 share the half-rate ALU pipe. 1024 + u - 1032 and
// (1024 + 16 u) / 16 - 72 are both exactly u - 8 in fp16.
__device__ __forceinline__ uint32_t fma_f16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ void kstep_f16(float (&c)[4], uint32_t w, uint32_t b0, uint32_t b1) {
  constexpr uint32_t kLo = 0x000F000Fu, kHi = 0x00F000F0u, k1024 = 0x64006400u;
  constexpr uint32_t k1032 = 0x64086408u;   // fp16x2 (1032, 1032)
  constexpr uint32_t kSixteenth = 0x2C002C00u;  // fp16x2 (1/16, 1/16)
  constexpr uint32_t kNeg72 = 0xD480D480u;      // fp16x2 (-72, -72)
  const uint32_t w8 = w >> 8;
  const uint32_t a0 = sub_f16x2(and_or(w, kLo, k1024), k1032);
  const uint32_t a1 = fma_f16x2(and_or(w, kHi, k1024), kSixteenth, kNeg72);
  const uint32_t a2 = sub_f16x2(and_or(w8, kLo, k1024), k1032);
  const uint32_t a3 = fma_f16x2(and_or(w8, kHi, k1024), kSixteenth, kNeg72);
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Streaming 16-byte weight load. V selects the cache flavour (A/B knob kept from the boundary):
// 0 = read-only path, no L1 allocation; 1 = plain read-only; 2 = no L1 + 256 B L2 sector hint;
// 3 = no L1 + L2 evict-first policy.
template <int V>
__device__ __forceinline__ uint4 ldw(const uint4* p, uint64_t pol) {
  uint4 r;
  if constexpr (V == 1) {
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  } else if constexpr (V == 2) {
    asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  } else if constexpr (V == 3) {
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p), "l"(pol));
  } else {
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  }
  return r;
}

// The 16 x values of lane (row r, quarter t) for chunk c, masked beyond K and beyond N.
__device__ __forceinline__ void load_x16(uint32_t (&xr)[8], const W4Args& a, int r, int t, int c,
                                         bool vec) {
  if (r >= a.N) {
#pragma unroll
    for (int i = 0; i < 8; ++i) xr[i] = 0u;
    return;
  }
  const int k = c * 64 + 16 * t;
  const bf16* xp = a.x + (long)r * a.ldx + k;
  if (vec && k + 16 <= a.K) {
    // plain (coherent) loads: x was written by a preceding kernel that may have overlapped this one
    const uint4 lo = reinterpret_cast<const uint4*>(xp)[0];
    const uint4 hi = reinterpret_cast<const uint4*>(xp)[1];
    xr[0] = lo.x; xr[1] = lo.y; xr[2] = lo.z; xr[3] = lo.w;
    xr[4] = hi.x; xr[5] = hi.y; xr[6] = hi.z; xr[7] = hi.w;
  } else {
    const unsigned short* xs = reinterpret_cast<const unsigned short*>(xp);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t e0 = (k + 2 * i < a.K) ? xs[2 * i] : 0u;
      const uint32_t e1 = (k + 2 * i + 1 < a.K) ? xs[2 * i + 1] : 0u;
      xr[i] = e0 | (e1 << 16);
    }
  }
}

__device__ __forceinline__ float silu_fast(float v) { return v / (1.0f + __expf(-v)); }

// Store one finished 16 x 8 tile held as the mma C fragment of warp 0.
template <int EPI>
__device__ __forceinline__ void store_tile(const W4Args& a, int tile, const float (&f)[4], int lane) {
  if constexpr (EPI == kEpiRuntime) {
    if (a.epi == QE_EPI_SWIGLU) store_tile<QE_EPI_SWIGLU>(a, tile, f, lane);
    else store_tile<QE_EPI_NONE>(a, tile, f, lane);
    return;
  }
  const int r = lane >> 2, t = lane & 3;
  const int n0 = 2 * t, n1 = n0 + 1;
  unsigned short* out = reinterpret_cast<unsigned short*>(a.out);
  auto bits = [](float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); };
  if constexpr (EPI == QE_EPI_NONE) {
    const int m0 = tile * 16 + r, m1 = m0 + 8;
    if (a.out_f32) {  // partial sums of a K-split matrix, rounded only after the ranks are added
      float* o32 = reinterpret_cast<float*>(a.out);
      if (n0 < a.N) {
        if (m0 < a.M) o32[(long)n0 * a.ldo + m0] = f[0];
        if (m1 < a.M) o32[(long)n0 * a.ldo + m1] = f[2];
      }
      if (n1 < a.N) {
        if (m0 < a.M) o32[(long)n1 * a.ldo + m0] = f[1];
        if (m1 < a.M) o32[(long)n1 * a.ldo + m1] = f[3];
      }
      return;
    }
    if (n0 < a.N) {
      if (m0 < a.M) out[(long)n0 * a.ldo + m0] = bits(f[0]);
      if (m1 < a.M) out[(long)n0 * a.ldo + m1] = bits(f[2]);
    }
    if (n1 < a.N) {
      if (m0 < a.M) out[(long)n1 * a.ldo + m0] = bits(f[1]);
      if (m1 < a.M) out[(long)n1 * a.ldo + m1] = bits(f[3]);
    }
  } else {
    // gate rows 0..7 and up rows 8..15 of the tile are the same 8 outputs (quantize_w4_gate_up,
    // python/qengine/quant.py:114-125): silu(gate) * up in fp32, one rounding.
    const int j = tile * 8 + r;
    if (j < a.M) {
      if (n0 < a.N) out[(long)n0 * a.ldo + j] = bits(silu_fast(f[0]) * f[2]);
      if (n1 < a.N) out[(long)n1 * a.ldo + j] = bits(silu_fast(f[1]) * f[3]);
    }
  }
}

// This warp's share (groups gb + warp, gb + warp + WARPS, ...) of tile `tile`, groups [gb, ge).
template <int WARPS, int U, int V>
__device__ __forceinline__ void accumulate(const W4Args& a, int tile, int gb, int ge, int warp,
                                           int lane, float (&acc)[4], bool& waited, uint64_t pol,
                                           bool vec) {
  const int r = lane >> 2, t = lane & 3;
  const uint4* wbase = a.qw + ((long)tile * a.G) * 64 + lane;       // 64 uint4 per unit
  const __half* sbase = a.scales + ((long)tile * a.G) * 16 + r;
  for (int g0 = gb + warp; g0 < ge; g0 += WARPS * U) {
    uint4 w[U][2];
    float slo[U], shi[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int g = g0 + u * WARPS;
      if (g < ge) {
        w[u][0] = ldw<V>(wbase + (long)g * 64, pol);
        w[u][1] = ldw<V>(wbase + (long)g * 64 + 32, pol);
        slo[u] = __half2float(__ldg(sbase + g * 16));
        shi[u] = __half2float(__ldg(sbase + g * 16 + 8));
      }
    }
    // Weights and scales never depend on the producer kernel; x does.
    if (!waited) { dep_wait(); waited = true; }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int g = g0 + u * WARPS;
      if (g < ge) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t xr[8];
          load_x16(xr, a, r, t, 2 * g + h, vec);
          kstep(c, w[u][h].x, xr[0], xr[1]);
          kstep(c, w[u][h].y, xr[2], xr[3]);
          kstep(c, w[u][h].z, xr[4], xr[5]);
          kstep(c, w[u][h].w, xr[6], xr[7]);
        }
        acc[0] = fmaf(slo[u], c[0], acc[0]);
        acc[1] = fmaf(slo[u], c[1], acc[1]);
        acc[2] = fmaf(shi[u], c[2], acc[2]);
        acc[3] = fmaf(shi[u], c[3], acc[3]);
      }
    }
  }
}

// Unit range of CTA b out of B over `total` units: equal shares, the first `total % B` one larger.
__device__ __host__ __forceinline__ int range_begin(int total, int B, int b) {
  const int per = total / B, rem = total % B;
  return b * per + (b < rem ? b : rem);
}
__device__ __forceinline__ int range_owner(int total, int B, int u) {
  const int per = total / B, rem = total % B;
  const int big = rem * (per + 1);
  return u < big ? u / (per + 1) : rem + (u - big) / per;
}

// A warp finishes a segment [gb, ge) of `tile` whose sums it holds: a whole tile is stored; a
// partial one is published to this worker's scratch slot and the contributor that completes the
// tile (integer arrival count of groups) adds all slots in a fixed order and stores.
// STREAM = true: workers (CTAs, or warps in mode 4) own contiguous unit ranges, two slots each
// (first / last tile of the range); false: grid (tiles, ksplit), slot = tile * ksplit + y.
template <int EPI, bool STREAM>
__device__ __forceinline__ void finish_segment(const W4Args& a, int tile, int gb, int ge,
                                               bool first_of_cta, const float (&acc)[4], int lane,
                                               int B, int b) {
  const int G = a.G;
  if (ge - gb == G) {
    store_tile<EPI>(a, tile, acc, lane);
    return;
  }
  const int slot = STREAM ? 2 * b + (first_of_cta ? 0 : 1) : tile * a.ksplit + blockIdx.y;
  float* mine = a.ws + (long)slot * 128;
#pragma unroll
  for (int i = 0; i < 4; ++i) __stcg(mine + i * 32 + lane, acc[i]);
  __threadfence();
  __syncwarp();
  int last = 0;
  if (lane == 0) {
    const int cnt = ge - gb;
    last = (atomicAdd(a.counters + tile, cnt) + cnt == G);
  }
  last = __shfl_sync(0xffffffffu, last, 0);
  if (!last) return;
  __threadfence();
  float f[4] = {0.f, 0.f, 0.f, 0.f};
  if constexpr (!STREAM) {
    for (int s = 0; s < a.ksplit; ++s) {
      const float* p = a.ws + (long)(tile * a.ksplit + s) * 128;
#pragma unroll
      for (int i = 0; i < 4; ++i) f[i] += __ldcg(p + i * 32 + lane);
    }
  } else {
    // Worker c contributed its first segment (slot 2c) if its range starts inside this tile,
    // otherwise (its range starts in an earlier tile) its last one (slot 2c + 1).
    const int first = range_owner(a.total, B, tile * G);
    const int lastb = range_owner(a.total, B, tile * G + G - 1);
#pragma unroll 1
    for (int c = first; c <= lastb; ++c) {
      const int cs = range_begin(a.total, B, c);
      const float* p = a.ws + (long)(2 * c + (cs >= tile * G ? 0 : 1)) * 128;
#pragma unroll
      for (int i = 0; i < 4; ++i) f[i] += __ldcg(p + i * 32 + lane);
    }
  }
  store_tile<EPI>(a, tile, f, lane);
  if (lane == 0) a.counters[tile] = 0;
}

// Two-level finish for kernels whose workers are warps with CTA-contiguous ids (worker = CTA *
// warps + warp): segments of a tile held by warps of one CTA are combined through shared memory
// (ascending warp order, last arriver by a shared-memory group count), and only a tile that
// crosses a CTA boundary goes through global memory, as one partial per CTA (ascending CTA order,
// last arriver by the global group count). With every matrix of the model a warp's range is
// shorter than a tile, so almost every tile is cut across several warps: the one-level scheme
// makes the last warp read all of them back from L2 one after the other at the very end of the
// kernel, this one reads shared memory and at most a neighbour CTA's partial.
// Slots: shared part[warps][2][128] floats + cnt[kCtaTiles] ints (zero on entry, left zero);
// global a.ws 2 x 128 floats per CTA, a.counters per tile (left zero).
constexpr int kCtaTiles = 128;
struct CtaFix {
  float* part;
  int* cnt;
  int warps;
};
// Whether the two-level scheme applies: every CTA span must cover at most kCtaTiles tiles.
__device__ __host__ __forceinline__ bool cta_fix_ok(int total, int G, int B, int warps) {
  const int ctas = (B + warps - 1) / warps;
  const long span = ((long)total + ctas - 1) / ctas + warps;  // upper bound of a CTA span in units
  return span / G + 2 <= kCtaTiles;
}
template <int EPI>
__device__ __forceinline__ void finish_segment_cta(const W4Args& a, const CtaFix& fx, int tile, int gb, int ge,
                                                   bool first_seg, const float (&acc)[4], int lane, int B, int b) {
  const int G = a.G;
  if (ge - gb == G) {
    store_tile<EPI>(a, tile, acc, lane);
    return;
  }
  const int c = b / fx.warps, w0 = c * fx.warps, w1 = min(B, w0 + fx.warps);
  const int s0 = range_begin(a.total, B, w0), s1 = range_begin(a.total, B, w1);  // this CTA's span
  const int t0 = tile * G, t1 = t0 + G;
  const int lo = max(s0, t0), hi = min(s1, t1);  // the CTA's share of the tile
  float* mine = fx.part + ((b - w0) * 2 + (first_seg ? 0 : 1)) * 128;
#pragma unroll
  for (int i = 0; i < 4; ++i) mine[i * 32 + lane] = acc[i];
  __threadfence_block();
  __syncwarp();
  const int ti = tile - s0 / G;
  int last = 0;
  if (lane == 0) {
    const int cnt = ge - gb;
    last = (atomicAdd(fx.cnt + ti, cnt) + cnt == hi - lo);
  }
  last = __shfl_sync(0xffffffffu, last, 0);
  if (!last) return;
  __threadfence_block();
  float f[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const int fw = max(w0, range_owner(a.total, B, lo)), lw = min(w1 - 1, range_owner(a.total, B, hi - 1));
    for (int w = fw; w <= lw; ++w) {
      const int ws = range_begin(a.total, B, w);
      const float* p = fx.part + ((w - w0) * 2 + (ws >= t0 ? 0 : 1)) * 128;
#pragma unroll
      for (int i = 0; i < 4; ++i) f[i] += p[i * 32 + lane];
    }
  }
  if (lane == 0) fx.cnt[ti] = 0;
  if (hi - lo == G) {  // the whole tile lives in this CTA
    store_tile<EPI>(a, tile, f, lane);
    return;
  }
  float* gm = a.ws + (long)(2 * c + (s0 >= t0 ? 0 : 1)) * 128;
#pragma unroll
  for (int i = 0; i < 4; ++i) __stcg(gm + i * 32 + lane, f[i]);
  __threadfence();
  __syncwarp();
  int glast = 0;
  if (lane == 0) glast = (atomicAdd(a.counters + tile, hi - lo) + (hi - lo) == G);
  glast = __shfl_sync(0xffffffffu, glast, 0);
  if (!glast) return;
  __threadfence();
  float s[4] = {0.f, 0.f, 0.f, 0.f};
  const int fc = range_owner(a.total, B, t0) / fx.warps, lc = range_owner(a.total, B, t1 - 1) / fx.warps;
#pragma unroll 1
  for (int cc = fc; cc <= lc; ++cc) {
    const int cs0 = range_begin(a.total, B, cc * fx.warps);
    const float* p = a.ws + (long)(2 * cc + (cs0 >= t0 ? 0 : 1)) * 128;
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] += __ldcg(p + i * 32 + lane);
  }
  store_tile<EPI>(a, tile, s, lane);
  if (lane == 0) a.counters[tile] = 0;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* b, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
// Bounded wait: false if the phase did not complete within the limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, int limit = 1 << 20) {
  const uint32_t addr = smem_u32(b);
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
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

}  // namespace
}  // namespace qb
