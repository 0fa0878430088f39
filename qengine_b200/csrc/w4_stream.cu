// W4A16 GEMV / skinny GEMM for 1..8 activation rows on B200 (sm_100a).
//
//   out[n, m] = bf16( sum_g fp32(scale[m, g]) * sum_{k in group g} (u[m, k] - 8) * x[n, k] )
//
// Boundary: replaces gemv_w4_tile / gemv_w4_bsk of the reference (csrc/gemv_w4.cu:291-362) behind
// qe_w4_gemv (reference launch_gemv_w4, csrc/gemv_w4.h:56). The packed wire format is the
// reference's (python/qengine/quant.py:1-30): the matrix is a stream of 1 KB "units", unit
// u = tile * G + g holding the int4 codes of 16 rows x 128 k (G = Kp / 128 groups per tile) as
// two 512-byte chunks of 32 lanes x 16 bytes, plus 32 bytes of fp16 scales at scales + 16 * u.
// Lane l = 4r + t of a chunk owns rows r and r + 8 and 16 consecutive k; word s of its 16 bytes
// carries k0 + {0,1,2,3} with k0 = 64 c + 16 t + 4 s, nibble j = row r + 8 (j & 1),
// k0 + 2 ((j >> 1) & 1) + (j >> 2). `(w >> 4j) & 0x000F000F | 0x43004300` is therefore the bf16
// pair (128 + u, 128 + u) for one A register of mma.m16n8k16, and subtracting 136 gives the
// signed code exactly. The k order inside the mma differs from memory order, which a dot product
// does not see as long as the x fragment uses the same order: lane (r, t) feeds x[n = r] at the
// same 16 consecutive k.
//
// Work split. The unit stream is cut into equal contiguous ranges, one per CTA, so every CTA reads
// one contiguous slab of HBM (weights are 97 % of the bytes of a decode step). A range is walked
// tile by tile; inside a tile the warps of the CTA take groups round-robin, each warp keeping
// `U` units (U KB) of loads in flight. Two grids exist:
//   mode 2: persistent, grid = min(SMs * occupancy, units / min work) CTAs over the whole stream;
//   mode 0: grid (tiles, ksplit): CTA (x, y) owns the y-th k-slice of tile x.
// Both are the same kernel body with a different range function.
//
// Determinism and row independence. Each (tile, group) product is accumulated by a fixed warp in
// fp32 with the scale applied once per group; warps are summed in warp order through shared
// memory; a tile cut across CTAs is finished by whichever CTA arrives last (integer arrival
// counter, counting groups) which adds the per-CTA partials in ascending CTA order. Nothing
// depends on timing or on N: the 8 columns of the mma are independent dot products, and no launch
// decision looks at N. Row r of an N-row call is therefore bit-identical to the 1-row call, which
// is what lets a speculative verify pass reproduce plain decode token for token.
//
// Why tensor-core mma also for one row: at 6.5 TB/s the SMs consume ~12.7e12 int4 weights per
// second, i.e. under 3 issued thread-instructions per weight. Unpack + convert + FMA on CUDA
// cores needs more than that; with the multiply-accumulate inside mma.sync the cost is 1.5
// (per 8 weights: 3 shifts, 4 lop3, 4 sub.bf16x2, 1 mma). It also makes the one-row and k+1-row
// sums the same instruction sequence, hence the same bits.
#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "w4_core.cuh"

namespace qb {
namespace {

// MODE 2: grid.x CTAs over the whole unit stream. MODE 0: grid (tiles, ksplit).
template <int WARPS, int U, int V, int EPI, int MODE>
__global__ void __launch_bounds__(WARPS * 32) w4_stream_kernel(const W4Args a) {
  dep_release();
  __shared__ float red[WARPS][4][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = a.G;
  const bool vec = ((a.ldx & 7) == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
  uint64_t pol = 0;
  if constexpr (V == 3) asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));

  int u0, u1;  // this CTA's units
  if constexpr (MODE == 0) {
    const int y = blockIdx.y, ks = a.ksplit;
    u0 = blockIdx.x * G + (int)((long)G * y / ks);
    u1 = blockIdx.x * G + (int)((long)G * (y + 1) / ks);
  } else {
    u0 = range_begin(a.total, gridDim.x, blockIdx.x);
    u1 = range_begin(a.total, gridDim.x, blockIdx.x + 1);
  }
  bool waited = false;
  for (int u = u0; u < u1;) {
    const int tile = u / G;
    const int gb = u - tile * G;
    const int ge = min(G, gb + (u1 - u));
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    accumulate<WARPS, U, V>(a, tile, gb, ge, warp, lane, acc, waited, pol, vec);
    if (!waited) { dep_wait(); waited = true; }  // a warp without groups still orders its writes
    if constexpr (WARPS > 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) red[warp][i][lane] = acc[i];
      __syncthreads();
      if (warp == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float s = red[0][i][lane];
#pragma unroll
          for (int w2 = 1; w2 < WARPS; ++w2) s += red[w2][i][lane];
          acc[i] = s;
        }
      }
      __syncthreads();
    }
    if (warp == 0) finish_segment<EPI, MODE == 2>(a, tile, gb, ge, u == u0, acc, lane, gridDim.x, blockIdx.x);
    u += ge - gb;
  }
}

// ---------------------------------------------------------------------------------------------
// MODE 3: the same unit stream fed through shared memory by the TMA engine. One producer warp
// issues bulk copies (cp.async.bulk global -> shared, completion on an mbarrier) of SU units
// (SU KB of codes + SU * 32 B of scales) per stage into a ring of STAGES stages, WARPS consumer
// warps read their units from the ring. The copies do not depend on the producer kernel of x, so
// the ring is filled before the programmatic-dependency wait: the whole ring (STAGES * SU KB per
// CTA) of weights is already on chip when x becomes available, and the stream never stops at tile
// boundaries. Consumer warp w owns the units u0 + w, u0 + w + WARPS, ... of the CTA's range
// (a function of the launch shape only), so results stay deterministic and independent of N.
// Every barrier wait is bounded; on expiry the kernel records an error code and drains.
// ---------------------------------------------------------------------------------------------
__device__ int g_ring_error = 0;

__device__ __forceinline__ void consumer_sync(int threads) {
  asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

template <int WARPS, int SU, int STAGES, int EPI>
__global__ void __launch_bounds__((WARPS + 1) * 32) w4_ring_kernel(const W4Args a) {
  static_assert(SU % WARPS == 0, "every consumer warp owns SU / WARPS units of each stage");
  constexpr int PER = SU / WARPS;
  dep_release();
  extern __shared__ __align__(128) unsigned char ring_raw[];
  uint4* wring = reinterpret_cast<uint4*>(ring_raw);                                  // [STAGES][SU][64]
  __half* sring = reinterpret_cast<__half*>(ring_raw + (size_t)STAGES * SU * 1024);   // [STAGES][SU][16]
  __shared__ uint64_t full[STAGES], empty[STAGES];
  __shared__ float red[2][WARPS][4][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = a.G;
  const int u0 = range_begin(a.total, gridDim.x, blockIdx.x);
  const int u1 = range_begin(a.total, gridDim.x, blockIdx.x + 1);
  const int nstage = (u1 - u0 + SU - 1) / SU;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == WARPS) {
    // ---- producer: one lane streams this CTA's slab, stage by stage ----
    if (lane == 0) {
      for (int st = 0; st < nstage; ++st) {
        const int slot = st % STAGES;
        if (st >= STAGES && !mbar_wait(&empty[slot], ((st / STAGES) - 1) & 1)) {
          atomicExch(&g_ring_error, 1);
          break;
        }
        const int ub = u0 + st * SU, cnt = min(SU, u1 - ub);
        mbar_expect_tx(&full[slot], (uint32_t)cnt * (1024 + 32));
        bulk_load(wring + (size_t)slot * SU * 64, a.qw + (size_t)ub * 64, (uint32_t)cnt * 1024, &full[slot]);
        bulk_load(sring + (size_t)slot * SU * 16, a.scales + (size_t)ub * 16, (uint32_t)cnt * 32, &full[slot]);
      }
    }
    dep_wait();
    return;
  }

  // ---- consumers ----
  const int r = lane >> 2, t = lane & 3;
  dep_wait();  // x, out, scratch: after the producer kernel
  // Lane (r, t) multiplies x row r. Rows >= N feed mma columns that are never stored, so those
  // lanes simply read row N - 1 again: no zero fill, no branch. (Host guarantees K % 128 == 0,
  // 16-byte aligned x and ldx % 8 == 0 for this mode.)
  const uint4* xlane = reinterpret_cast<const uint4*>(a.x + (long)min(r, a.N - 1) * a.ldx + 16 * t);  // coherent loads
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  int tile = u0 / G;          // tile of the segment being accumulated
  int seg_begin = u0;         // first unit of that segment
  int phase = 0;              // red[] double buffer
  bool ok = true;

  // Sum the warps' partial tiles in warp order and let warp 0 store / publish the segment.
  auto close_segment = [&](int seg_end) {
#pragma unroll
    for (int c = 0; c < 4; ++c) red[phase][warp][c][lane] = acc[c];
    consumer_sync(WARPS * 32);
    if (warp == 0) {
      float f[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float s = red[phase][0][c][lane];
#pragma unroll
        for (int w2 = 1; w2 < WARPS; ++w2) s += red[phase][w2][c][lane];
        f[c] = s;
      }
      finish_segment<EPI, true>(a, tile, seg_begin - tile * G, seg_end - tile * G, seg_begin == u0, f, lane,
                                gridDim.x, blockIdx.x);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[c] = 0.f;
    phase ^= 1;
    seg_begin = seg_end;
    ++tile;
  };

  // One unit: 16 rows x 128 k from the ring times this lane's 32 x values.
  auto unit = [&](int slot, int idx, int g) {
    const uint4* wp = wring + ((size_t)slot * SU + idx) * 64 + lane;
    const uint4 w0 = wp[0], w1 = wp[32];
    const __half* sp = sring + ((size_t)slot * SU + idx) * 16 + r;
    const float slo = __half2float(sp[0]), shi = __half2float(sp[8]);
    const uint4* xp = xlane + g * 16;  // 128 bf16 per group = 16 uint4
    const uint4 x0 = xp[0], x1 = xp[1], x2 = xp[8], x3 = xp[9];
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    auto ks = [&](uint32_t w, uint32_t b0, uint32_t b1) { kstep(c, w, b0, b1); };
    ks(w0.x, x0.x, x0.y);
    ks(w0.y, x0.z, x0.w);
    ks(w0.z, x1.x, x1.y);
    ks(w0.w, x1.z, x1.w);
    ks(w1.x, x2.x, x2.y);
    ks(w1.y, x2.z, x2.w);
    ks(w1.z, x3.x, x3.y);
    ks(w1.w, x3.z, x3.w);
    acc[0] = fmaf(slo, c[0], acc[0]);
    acc[1] = fmaf(slo, c[1], acc[1]);
    acc[2] = fmaf(shi, c[2], acc[2]);
    acc[3] = fmaf(shi, c[3], acc[3]);
  };

  for (int st = 0; st < nstage; ++st) {
    const int slot = st % STAGES;
    if (!mbar_wait(&full[slot], (st / STAGES) & 1, ok ? (1 << 20) : 64)) {
      ok = false;
      atomicExch(&g_ring_error, 2);
    }
    const int ub = u0 + st * SU;
    if (ok && ub + SU <= u1 && ub + SU <= (tile + 1) * G) {
      // Whole stage inside the current tile: no per-unit checks. Units are taken in pairs whose
      // operands are all fetched before the first mma, so two independent mma chains overlap.
      const int gb = ub - tile * G + warp;
#pragma unroll
      for (int i0 = 0; i0 < PER; i0 += 2) {
        constexpr int P2 = PER >= 2 ? 2 : 1;
        uint4 wq[P2][2], xq[P2][4];
        float slo[P2], shi[P2];
#pragma unroll
        for (int j = 0; j < P2; ++j) {
          const int idx = warp + (i0 + j) * WARPS;
          const uint4* wp = wring + ((size_t)slot * SU + idx) * 64 + lane;
          wq[j][0] = wp[0];
          wq[j][1] = wp[32];
          const __half* sp = sring + ((size_t)slot * SU + idx) * 16 + r;
          slo[j] = __half2float(sp[0]);
          shi[j] = __half2float(sp[8]);
          const uint4* xp = xlane + (gb + (i0 + j) * WARPS) * 16;
          xq[j][0] = xp[0]; xq[j][1] = xp[1]; xq[j][2] = xp[8]; xq[j][3] = xp[9];
        }
        float c[P2][4];
#pragma unroll
        for (int j = 0; j < P2; ++j) { c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f; }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int j = 0; j < P2; ++j) {
            kstep(c[j], wq[j][h].x, xq[j][2 * h].x, xq[j][2 * h].y);
            kstep(c[j], wq[j][h].y, xq[j][2 * h].z, xq[j][2 * h].w);
          }
#pragma unroll
          for (int j = 0; j < P2; ++j) {
            kstep(c[j], wq[j][h].z, xq[j][2 * h + 1].x, xq[j][2 * h + 1].y);
            kstep(c[j], wq[j][h].w, xq[j][2 * h + 1].z, xq[j][2 * h + 1].w);
          }
        }
#pragma unroll
        for (int j = 0; j < P2; ++j) {
          acc[0] = fmaf(slo[j], c[j][0], acc[0]);
          acc[1] = fmaf(slo[j], c[j][1], acc[1]);
          acc[2] = fmaf(shi[j], c[j][2], acc[2]);
          acc[3] = fmaf(shi[j], c[j][3], acc[3]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int idx = warp + i * WARPS;  // unit of this stage owned by this warp
        const int u = ub + idx;
        // Tile boundaries inside the range that lie at or before u: close them. Every consumer
        // warp closes every such boundary exactly once (here, or in the catch-up loop after the
        // last stage), so the k-th barrier of each warp always belongs to the k-th boundary.
        while (u >= (tile + 1) * G && (tile + 1) * G < u1) close_segment((tile + 1) * G);
        if (u < u1 && ok) unit(slot, idx, u - tile * G);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[slot]);
  }
  while ((tile + 1) * G < u1) close_segment((tile + 1) * G);  // boundaries this warp never reached
  close_segment(u1);                                          // the last segment of the range
}

// ---------------------------------------------------------------------------------------------
// MODE 4: warp-private rings. The unit stream is cut into one contiguous range per WARP (all
// warps of all CTAs); each warp is a pipeline of its own: its lane 0 issues the bulk copies
// (cp.async.bulk global -> shared, completion on an mbarrier) that keep STAGES stages of PERW
// units of ITS range in flight, all lanes consume. No CTA barrier, no producer warp: a warp walks
// the groups of a tile in order, stores a tile it owned entirely and publishes a partial one (at
// most the first and the last tile of its range). With the 27B matrices a warp's range is shorter
// than a tile, so nearly every tile is cut across warps; TWO = true finishes such tiles in two
// levels (finish_segment_cta: the warps of a CTA combine through shared memory in warp order, only
// a tile that crosses a CTA boundary exchanges one partial per CTA through global memory), which
// removes the serial read-back of every contributor from L2 at the end of the kernel (2-3 us per
// launch). TWO = false (CTA spans of more than 128 tiles) keeps the one-level global scheme.
// Inner loop per unit: 2 LDS.128 + 2 LDS.16 (weights, scales), 4 coherent LDG.128 (x), 8 mma, no
// branch but the tile-end test. Ranges depend on the launch shape only: deterministic and
// independent of N.
// ---------------------------------------------------------------------------------------------
template <int PERW, int STAGES, int EPI, bool XF16, int MINB, bool TWO>
__global__ void __launch_bounds__(256, MINB) w4_warp_ring_kernel(const W4Args a, int nworkers) {
  constexpr int WARPS = 8;
  constexpr uint32_t kStageW = PERW * 1024, kStageS = PERW * 32;
  dep_release();
  extern __shared__ __align__(128) unsigned char ring_raw[];
  __shared__ uint64_t full[WARPS][STAGES];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int worker = blockIdx.x * WARPS + warp;
  unsigned char* wbase = ring_raw + (size_t)warp * STAGES * (kStageW + kStageS);
  unsigned char* sbase = wbase + (size_t)STAGES * kStageW;
  const int G = a.G;
  // two-level finish of tiles cut across warps (shared memory inside the CTA, global across CTAs)
  CtaFix fx;
  fx.part = reinterpret_cast<float*>(ring_raw + (size_t)WARPS * STAGES * (kStageW + kStageS));
  fx.cnt = reinterpret_cast<int*>(fx.part + WARPS * 2 * 128);
  fx.warps = WARPS;
  if (TWO) {
    if (threadIdx.x < kCtaTiles) fx.cnt[threadIdx.x] = 0;
    __syncthreads();
  }
  int u0 = 0, u1 = 0;
  if (worker < nworkers) {
    u0 = range_begin(a.total, nworkers, worker);
    u1 = range_begin(a.total, nworkers, worker + 1);
  }
  const int nstage = (u1 - u0 + PERW - 1) / PERW;

  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&full[warp][s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  auto refill = [&](int st) {  // lane 0 only
    const int slot = st % STAGES;
    const int ub = u0 + st * PERW, cnt = min(PERW, u1 - ub);
    mbar_expect_tx(&full[warp][slot], (uint32_t)cnt * (1024 + 32));
    bulk_load(wbase + (size_t)slot * kStageW, a.qw + (size_t)ub * 64, (uint32_t)cnt * 1024, &full[warp][slot]);
    bulk_load(sbase + (size_t)slot * kStageS, a.scales + (size_t)ub * 16, (uint32_t)cnt * 32, &full[warp][slot]);
  };
  if (lane == 0)
    for (int st = 0; st < min(STAGES, nstage); ++st) refill(st);  // weights never depend on x
  dep_wait();
  if (nstage == 0) return;

  const int r = lane >> 2, t = lane & 3;
  const uint4* xlane = reinterpret_cast<const uint4*>(a.x + (long)min(r, a.N - 1) * a.ldx + 16 * t);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  int tile = u0 / G;
  int g = u0 - tile * G;       // group of the next unit inside its tile
  int seg_gb = g;              // first group of the segment being accumulated
  bool first_seg = true;
  bool ok = true;

  // One unit (group gg of the current tile) into acc. The tile-end handling is NOT in here: this
  // body is replicated by the unrolled fast path below, and the kernel is short enough for its
  // code size to show up as instruction-cache misses at the start of every launch.
  auto unit_core = [&](const uint4* wp, const __half* sp, int gg) {
    const uint4 w0 = wp[0], w1 = wp[32];
    const float slo = __half2float(sp[0]), shi = __half2float(sp[8]);
    const uint4* xp = xlane + gg * 16;
    const uint4 x0 = xp[0], x1 = xp[1], x2 = xp[8], x3 = xp[9];
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    auto ks = [&](uint32_t w, uint32_t b0, uint32_t b1) {
      if constexpr (XF16) kstep_f16(c, w, b0, b1); else kstep(c, w, b0, b1);
    };
    ks(w0.x, x0.x, x0.y);
    ks(w0.y, x0.z, x0.w);
    ks(w0.z, x1.x, x1.y);
    ks(w0.w, x1.z, x1.w);
    ks(w1.x, x2.x, x2.y);
    ks(w1.y, x2.z, x2.w);
    ks(w1.z, x3.x, x3.y);
    ks(w1.w, x3.z, x3.w);
    acc[0] = fmaf(slo, c[0], acc[0]);
    acc[1] = fmaf(slo, c[1], acc[1]);
    acc[2] = fmaf(shi, c[2], acc[2]);
    acc[3] = fmaf(shi, c[3], acc[3]);
  };

  for (int st = 0; st < nstage; ++st) {
    const int slot = st % STAGES;
    if (!mbar_wait(&full[warp][slot], (st / STAGES) & 1, ok ? (1 << 20) : 64)) {
      ok = false;
      atomicExch(&g_ring_error, 4);
    }
    const uint4* wp = reinterpret_cast<const uint4*>(wbase + (size_t)slot * kStageW) + lane;
    const __half* sp = reinterpret_cast<const __half*>(sbase + (size_t)slot * kStageS) + r;
    const int cnt = min(PERW, u1 - (u0 + st * PERW));
    if (ok) {
      int i = 0;
      while (i < cnt) {
        const int run = min(cnt - i, G - g);  // units of this stage that stay inside the tile
        if (run == PERW) {
#pragma unroll
          for (int j = 0; j < PERW; ++j) unit_core(wp + j * 64, sp + j * 16, g + j);
        } else {
#pragma unroll 1
          for (int j = 0; j < run; ++j) unit_core(wp + (i + j) * 64, sp + (i + j) * 16, g + j);
        }
        g += run;
        i += run;
        // the tile is complete, or the range ends inside it: the only call site of the finish
        if (g == G || (st == nstage - 1 && i == cnt)) {
          if constexpr (TWO) finish_segment_cta<EPI>(a, fx, tile, seg_gb, g, first_seg, acc, lane, nworkers, worker);
          else finish_segment<EPI, true>(a, tile, seg_gb, g, first_seg, acc, lane, nworkers, worker);
          acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
          g = (g == G) ? 0 : g;
          seg_gb = g; first_seg = false; ++tile;
        }
      }
    }
    __syncwarp();
    if (lane == 0 && st + STAGES < nstage) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      refill(st + STAGES);
    }
  }
}

using KernelFn = void (*)(const W4Args);

template <int WARPS, int U, int V>
KernelFn pick_tail(int epi, int mode) {
  if (mode == 2)
    return epi == QE_EPI_SWIGLU ? w4_stream_kernel<WARPS, U, V, QE_EPI_SWIGLU, 2>
                                : w4_stream_kernel<WARPS, U, V, QE_EPI_NONE, 2>;
  return epi == QE_EPI_SWIGLU ? w4_stream_kernel<WARPS, U, V, QE_EPI_SWIGLU, 0>
                              : w4_stream_kernel<WARPS, U, V, QE_EPI_NONE, 0>;
}
template <int WARPS, int U>
KernelFn pick_v(int v, int epi, int mode) {
  // Flavours 2 and 3 are accepted at the boundary and served by flavour 0 (kept out of the
  // build to bound the number of instantiations).
  return v == 1 ? pick_tail<WARPS, U, 1>(epi, mode) : pick_tail<WARPS, U, 0>(epi, mode);
}
template <int WARPS>
KernelFn pick_u(int u, int v, int epi, int mode) {
  switch (u) {
    case 1: return pick_v<WARPS, 1>(v, epi, mode);
    case 2: return pick_v<WARPS, 2>(v, epi, mode);
    default: return pick_v<WARPS, 4>(v, epi, mode);
  }
}
KernelFn pick(int warps, int u, int v, int epi, int mode) {
  switch (warps) {
    case 4: return pick_u<4>(u, v, epi, mode);
    case 16: return pick_u<16>(u, v, epi, mode);
    default: return pick_u<8>(u, v, epi, mode);
  }
}

int blocks_per_sm(KernelFn fn, int threads) {
  static std::mutex mu;
  static std::unordered_map<const void*, int> cache;
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find((const void*)fn);
  if (it != cache.end()) return it->second;
  int b = 1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, fn, threads, 0) != cudaSuccess) b = 1;
  b = std::max(b, 1);
  cache[(const void*)fn] = b;
  return b;
}

using WarpKernelFn = void (*)(const W4Args, int);

struct Resolved {
  qe_w4_plan plan;
  KernelFn fn;
  size_t smem = 0;
  WarpKernelFn wfn = nullptr;  // mode 4
  int nworkers = 0;            // mode 4: warps that own a range
};

// Geometries of mode 4 (8 warps per CTA, one private ring per warp), chosen by `unroll`:
//   unroll 0/4: 4 units per stage x 3 stages = 12.4 KB per warp, 99 KB per CTA, 2 CTAs per SM
//   unroll 2  : 2 units per stage x 6 stages = same bytes, finer refill
//   unroll 1  : 4 units per stage x 2 stages = 66 KB per CTA, 3 CTAs per SM
struct WarpGeom {
  WarpKernelFn fn[8];  // [epilogue + 2 * x_is_fp16 + 4 * two-level finish]
  size_t smem;
  int bps;
};
template <int PERW, int ST, int MINB>
WarpGeom warp_geom(int bps) {
  // one function per (activation type, finish scheme) serves both epilogues
  WarpGeom g{{w4_warp_ring_kernel<PERW, ST, kEpiRuntime, false, MINB, false>,
              w4_warp_ring_kernel<PERW, ST, kEpiRuntime, false, MINB, false>,
              w4_warp_ring_kernel<PERW, ST, kEpiRuntime, true, MINB, false>,
              w4_warp_ring_kernel<PERW, ST, kEpiRuntime, true, MINB, false>,
              w4_warp_ring_kernel<PERW, ST, kEpiRuntime, false, MINB, true>,
              w4_warp_ring_kernel<PERW, ST, kEpiRuntime, false, MINB, true>,
              w4_warp_ring_kernel<PERW, ST, kEpiRuntime, true, MINB, true>,
              w4_warp_ring_kernel<PERW, ST, kEpiRuntime, true, MINB, true>},
             (size_t)8 * ST * PERW * (1024 + 32) + 8 * 2 * 128 * sizeof(float) + kCtaTiles * sizeof(int), bps};
  for (WarpKernelFn f : g.fn) cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
  return g;
}
// variant 1 selects the half-SM geometries: 2 CTAs x 50 KB and at most 64 registers per thread, so
// that the CTAs of the next kernel of the stream fit beside the running ones and fill their rings
// before their programmatic-dependency wait ends.
const WarpGeom& warp_geom_for(int unroll, int variant) {
  static const WarpGeom g4 = warp_geom<4, 3, 1>(2), g2 = warp_geom<2, 6, 1>(2), g1 = warp_geom<4, 2, 3>(3);
  static const WarpGeom h2 = warp_geom<2, 3, 4>(2), h3 = warp_geom<3, 2, 4>(2);
  if (variant == 1) return unroll == 4 ? h3 : h2;
  return unroll == 2 ? g2 : unroll == 4 ? g4 : g1;  // default: 3 CTAs per SM
}

// Ring geometries of mode 3 (8 consumer warps + 1 producer warp per CTA), chosen by `unroll`:
//   unroll 0/2: 16 units (16.5 KB) per stage x 6 stages = 99 KB in flight per CTA, 2 CTAs per SM
//   unroll 4  : 32 units (33 KB) per stage x 3 stages   = 99 KB, 4 independent units per warp
//   unroll 1  : 16 units per stage x 4 stages           = 66 KB, 3 CTAs per SM
constexpr int kRingWarps = 8;
struct RingGeom {
  KernelFn fn[2];
  size_t smem;
  int bps;
};
template <int SU, int ST>
RingGeom ring_geom(int bps) {
  RingGeom g{{w4_ring_kernel<kRingWarps, SU, ST, QE_EPI_NONE>, w4_ring_kernel<kRingWarps, SU, ST, QE_EPI_SWIGLU>},
             (size_t)ST * SU * (1024 + 32), bps};
  for (KernelFn f : g.fn) cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
  return g;
}
const RingGeom& ring_for(int unroll) {
  static const RingGeom g2 = ring_geom<16, 6>(2), g4 = ring_geom<32, 3>(2), g1 = ring_geom<16, 4>(3);
  return unroll == 4 ? g4 : unroll == 1 ? g1 : g2;
}

// Shape-only policy (never N). B200: 148 SMs; every matrix of the 27B model except the tiniest
// runs as one persistent unit stream; small matrices (< 4096 units) use the (tile, ksplit) grid
// so that a launch still covers every SM.
Resolved resolve(const qe_w4_params& p, const qe_w4_cfg& in) {
  Resolved r{};
  qe_w4_cfg c = in;
  const long tiles = p.Mp / 16, G = p.Kp / 128, units = tiles * G;
  const int sms = qe_sm_count();
  const int auto_mode = units < 4096 ? 0 : 4;  // warp-private rings for every large matrix
  int mode = (c.mode == 0 || c.mode == 2 || c.mode == 3 || c.mode == 4) ? c.mode : auto_mode;
  if (units >= (1L << 30)) mode = 0;  // 32-bit unit arithmetic in the stream modes
  // The ring paths serve the aligned fast case only (every matrix of the model qualifies).
  if (mode >= 3 && (p.K != p.Kp || (p.ldx & 7) || (reinterpret_cast<uintptr_t>(p.x) & 15))) mode = 2;
  if (p.x_f16) mode = 4;  // fp16 activations are served by the warp-ring kernel only
  if (mode == 4) {
    const WarpGeom& wg = warp_geom_for(c.unroll, c.variant);
    r.smem = wg.smem;
    r.plan.mode = 4;
    r.plan.threads = 256;
    r.plan.counters = tiles;
    const int bps = c.blocks_per_sm > 0 ? c.blocks_per_sm : wg.bps;
    const long want = (units + std::max(1, c.min_units) - 1) / std::max(1, c.min_units);
    const long workers = std::max<long>(1, std::min<long>((long)sms * bps * 8, want));
    // tiles cut across warps are finished through shared memory when every CTA span is short enough
    const bool two = cta_fix_ok((int)units, (int)G, (int)workers, 8);
    r.wfn = wg.fn[(p.epilogue == QE_EPI_SWIGLU ? 1 : 0) + (p.x_f16 ? 2 : 0) + (two ? 4 : 0)];
    r.nworkers = (int)workers;
    r.plan.grid_x = (int)((workers + 7) / 8);
    r.plan.grid_y = 1;
    r.plan.ws_floats = workers * 2 * 128;
    return r;
  }
  if (mode == 3) {
    const RingGeom& rg = ring_for(c.unroll);
    r.fn = rg.fn[p.epilogue == QE_EPI_SWIGLU ? 1 : 0];
    r.smem = rg.smem;
    r.plan.mode = 3;
    r.plan.threads = (kRingWarps + 1) * 32;
    r.plan.counters = tiles;
    const int bps = c.blocks_per_sm > 0 ? c.blocks_per_sm : rg.bps;
    const long per_block = (long)std::max(1, c.min_units) * kRingWarps;
    const long blocks = std::max<long>(1, std::min<long>((long)sms * bps, (units + per_block - 1) / per_block));
    r.plan.grid_x = (int)blocks;
    r.plan.grid_y = 1;
    r.plan.ws_floats = blocks * 2 * 128;
    return r;
  }
  int warps = (c.warps == 4 || c.warps == 8 || c.warps == 16) ? c.warps : 8;
  int unroll = (c.unroll == 1 || c.unroll == 2 || c.unroll == 4) ? c.unroll : 4;
  const int variant = (c.variant >= 0 && c.variant <= 3) ? c.variant : 0;
  r.fn = pick(warps, unroll, variant, p.epilogue, mode);
  r.plan.mode = mode;
  r.plan.threads = warps * 32;
  r.plan.counters = tiles;
  if (mode == 2) {
    const int bps = c.blocks_per_sm > 0 ? c.blocks_per_sm : blocks_per_sm(r.fn, r.plan.threads);
    const long per_block = (long)std::max(1, c.min_units) * warps;
    const long blocks = std::max<long>(1, std::min<long>((long)sms * bps, (units + per_block - 1) / per_block));
    r.plan.grid_x = (int)blocks;
    r.plan.grid_y = 1;
    r.plan.ws_floats = blocks * 2 * 128;
  } else {
    long ks = c.ksplit > 0 ? c.ksplit : qe_w4_auto_ksplit(p.Mp, p.Kp, p.N, warps);
    ks = std::max<long>(1, std::min<long>(ks, G));
    r.plan.grid_x = (int)tiles;
    r.plan.grid_y = (int)ks;
    r.plan.ws_floats = ks > 1 ? tiles * ks * 128 : 0;
  }
  return r;
}

}  // namespace
}  // namespace qb

using namespace qb;

extern "C" void qe_w4_cfg_default(qe_w4_cfg* c) {
  c->warps = 0; c->unroll = 0; c->ksplit = 0; c->pdl = 1; c->variant = 0; c->mode = -1;
  c->blocks_per_sm = 0; c->min_units = 4;
}

extern "C" int qe_w4_auto_ksplit(int Mp, int Kp, int N, int warps) {
  (void)N;  // never a function of the row count
  if (warps <= 0) warps = 8;
  const long tiles = Mp / 16, G = Kp / 128;
  if (tiles * G >= 4096) return 1;
  // Small matrix: cut K until the grid has about two CTAs per SM, keeping one group per warp.
  const int want = 2 * qe_sm_count();
  int ks = 1;
  while (tiles * ks < want && G / (ks * 2) >= warps) ks *= 2;
  return ks;
}

extern "C" int qe_w4_plan_gemv(const qe_w4_params* p, const qe_w4_cfg* cfg, qe_w4_plan* plan) {
  if (!p || !cfg || !plan) return QE_ERR_ARG;
  if (p->Mp <= 0 || p->Kp <= 0 || p->Mp % 16 || p->Kp % 128) return QE_ERR_ARG;
  *plan = resolve(*p, *cfg).plan;
  return 0;
}

// Error word of the ring kernel's bounded waits (0 = none). Host-visible for tests and the engine.
extern "C" int qe_w4_ring_error(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ring_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

extern "C" int qe_w4_gemv(const qe_w4_params* p, const qe_w4_cfg* cfg, void* stream) {
  if (!p || !cfg) return QE_ERR_ARG;
  if (p->N < 1 || p->N > QE_MAX_ROWS || p->Mp % 16 || p->Kp % 128 || p->Mp <= 0 || p->Kp <= 0)
    return QE_ERR_ARG;
  if (p->K > p->Kp || p->K <= 0 || p->M <= 0) return QE_ERR_ARG;
  if (p->epilogue == QE_EPI_SWIGLU ? p->M > p->Mp / 2 : p->M > p->Mp) return QE_ERR_ARG;
  const Resolved r = resolve(*p, *cfg);
  W4Args a{};
  a.qw = reinterpret_cast<const uint4*>(p->qw);
  a.scales = reinterpret_cast<const __half*>(p->scales);
  a.x = reinterpret_cast<const bf16*>(p->x);
  a.out = reinterpret_cast<bf16*>(p->out);
  a.out_f32 = (p->out_f32 && p->epilogue == QE_EPI_NONE) ? 1 : 0;
  a.epi = p->epilogue;
  a.ws = p->ws;
  a.counters = p->counters;
  a.M = p->M; a.K = p->K; a.N = p->N;
  a.tiles = p->Mp / 16; a.G = p->Kp / 128;
  a.ldx = p->ldx; a.ldo = p->ldo;
  a.ksplit = r.plan.grid_y;

  a.total = a.tiles * a.G;
  const bool pdl = cfg->pdl && pdl_launch_enabled() && pdl_trigger_enabled();
  if (r.plan.mode == 4)
    return (int)launch(r.wfn, dim3(r.plan.grid_x, 1, 1), dim3(r.plan.threads), r.smem,
                       (cudaStream_t)stream, pdl, a, r.nworkers);
  return (int)launch(r.fn, dim3(r.plan.grid_x, r.plan.grid_y, 1), dim3(r.plan.threads), r.smem,
                     (cudaStream_t)stream, pdl, a);
}

// ---------------------------------------------------------------------------------------------
// qe_w4_gemv_static: the same GEMV for callers that cannot allocate device memory.
//
// qe_w4_gemv needs two scratch buffers from its caller (fp32 partial-tile slots and int32 arrival
// counters). Some hosts have no way to provide them: a plugin that runs inside another runtime's
// callback where cudaMalloc is forbidden, code that executes between the capture and the replay
// of a CUDA graph and must not touch the allocator, or an embedder whose memory pool is owned by
// a framework it may not call back into. For them the scratch lives in this library instead, in
// a file-scope device array of fixed size that every GPU loading the library holds until exit:
// QE_W4_STATIC_WS_FLOATS fp32 slots (4 MiB) + QE_W4_STATIC_COUNTERS counters (64 KiB).
//
// The array's name is only a host-side handle. Its device address is looked up with
// cudaGetSymbolAddress once per device, on the first call made while that device is current
// (so make that first call before any stream capture), and that pointer is what the kernel
// receives. No cudaMalloc, cudaFree or allocating library routine is called here.
// Every call uses the same array and finds in it whatever the previous call left; the counters,
// which must start at zero, are cleared on the stream before each launch. Two calls that overlap
// on the GPU (different streams) therefore race on the scratch: serialise them.
// ---------------------------------------------------------------------------------------------
namespace qb {
namespace {
static __device__ __align__(256) unsigned char
    g_w4_static_scratch[(size_t)QE_W4_STATIC_COUNTERS * 4 + (size_t)QE_W4_STATIC_WS_FLOATS * 4];

// Device address of the scratch array on the current device (looked up once per device).
cudaError_t static_scratch(unsigned char** out) {
  static unsigned char* per_dev[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!per_dev[dev]) {
    unsigned char* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_w4_static_scratch);
    if (e != cudaSuccess) return e;
    per_dev[dev] = ptr;
  }
  *out = per_dev[dev];
  return cudaSuccess;
}
}  // namespace
}  // namespace qb

extern "C" int qe_w4_gemv_static(const qe_w4_params* p, const qe_w4_cfg* cfg, void* stream) {
  if (!p || !cfg) return QE_ERR_ARG;
  if (p->N < 1 || p->N > QE_MAX_ROWS || p->Mp % 16 || p->Kp % 128 || p->Mp <= 0 || p->Kp <= 0)
    return QE_ERR_ARG;
  qe_w4_plan plan;
  int rc = qe_w4_plan_gemv(p, cfg, &plan);
  if (rc) return rc;
  if (plan.ws_floats > QE_W4_STATIC_WS_FLOATS || plan.counters > QE_W4_STATIC_COUNTERS)
    return QE_ERR_SCRATCH;  // this shape / launch configuration needs more than the fixed array
  unsigned char* base = nullptr;
  cudaError_t e = static_scratch(&base);
  if (e != cudaSuccess) return (int)e;
  int* counters = reinterpret_cast<int*>(base);
  float* ws = reinterpret_cast<float*>(base + (size_t)QE_W4_STATIC_COUNTERS * 4);
  e = cudaMemsetAsync(counters, 0, (size_t)plan.counters * 4, (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  qe_w4_params q = *p;
  q.ws = ws;
  q.counters = counters;
  qe_w4_cfg c = *cfg;
  c.pdl = 0;  // the launch follows a memset on the stream: plain stream order
  return qe_w4_gemv(&q, &c, stream);
}
