// W4A16 GEMV / skinny GEMM for 1..8 activation rows on B200 (sm_100a), optionally fused with the
// residual add + RMSNorm that produces its input.
//
//   out[n, m] = bf16( sum_g fp32(scale[m, g]) * sum_{k in group g} (code[m, k] - 8) * x[n, k] )
//
// Boundary: qe_w4_gemv replaces launch_gemv_w4 of the reference (csrc/gemv_w4.h:56, kernels
// csrc/gemv_w4.cu:291-362) on the reference's packed wire format (w4_dev.cuh); qe_w4_gemv_ex adds
// the fused prologue (no counterpart in the reference, which runs rmsnorm1p as its own kernel).
//
// Design. The matrix is a stream of 1 KB units (16 rows x 128 k); 97 % of the bytes of a decode
// step are such units, so the kernel is organised around streaming them at HBM rate with as few
// issued instructions per unit as the unpack allows:
//   * one CTA per SM, NW warps; the unit stream is cut into one contiguous range per CTA (equal
//     shares, to within four units) and that range into one contiguous range per warp, so every
//     warp reads one contiguous slab of HBM and every SM has the same amount of work;
//   * each warp owns a private ring in shared memory that its lane 0 keeps full with bulk copies
//     (cp.async.bulk global -> shared, completion on an mbarrier): STAGES x PERW units in flight
//     per warp, ~130 KB per SM, issued before the programmatic-dependency wait because weights
//     never depend on the producer of x;
//   * ranges start at multiples of a ring stage whenever a tile is a whole number of stages long,
//     so a stage never straddles two tiles and its PERW units run as straight-line code: 2 LDS.128
//     of codes, 2 scales and 4 x 16 B of x per unit at immediate offsets, then the unpack feeding
//     mma.sync.m16n8k16. The unpack (shift, lop3, bf16x2 subtract per pair of weights) is the cost
//     that matters: at HBM rate an SM sub-partition has about 190 issue slots per unit, the
//     unpack and its eight tensor-core products need 104 of them, so everything else in the
//     loop has to stay in the low tens;
//   * a tile (16 output rows) that lies inside one warp's range is stored from registers; the at
//     most two cut tiles per warp (first / last of its range) are parked in shared memory and
//     combined after ONE block barrier at the end of the kernel, each by the warp that holds the
//     head of the tile, in ascending warp order. Only a tile that crosses a CTA boundary goes
//     through global memory: one partial per CTA, integer arrival counter, ascending CTA order.
// No float atomics and no data-dependent order: results are bit-identical run to run. No decision
// depends on the number of activation rows N and the 8 mma columns are independent dot products,
// so row r of an N-row call equals the 1-row call bit for bit (what lets a speculative verify
// pass reproduce plain decoding token for token).
//
// Fused prologue (PRO): x = RMSNorm1p(h_in + delta) is recomputed by every CTA into shared memory
// (10 KB per row at hidden 5120: 148 redundant copies cost less than one dependent kernel launch
// plus a trip through L2), and CTA 0 writes the updated residual stream to h_out. h_out must not
// alias h_in: other CTAs may still be reading h_in.
//
// Every mbarrier wait is bounded; on expiry the warp records g_w4_error, drains and leaves.
#include <cuda/atomic>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

#include "w4_dev.cuh"

namespace qb {
// error word of the GEMM's bounded waits (w4_gemm.cu), reported together with the GEMV's
int gemm_error_read();
int gemm_error_clear();
namespace {

using namespace w4;

struct GemvArgs {
  const uint4* qw;
  const __half* scales;
  const bf16* x;   // activations (unused with the prologue)
  long ldx;
  OutDesc o;
  float* ws;       // 2 x 128 floats per CTA: partial tiles that cross a CTA boundary
  int* counters;   // one arrival counter per tile, zero on entry, left zero
  int K, G, total;
  int nctas;       // CTAs that own work (<= gridDim.x)
  int nwarps;      // warps of a CTA that own work (small matrices keep min_units per warp)
  int quantum;     // warp ranges start at multiples of this many units (4 when G % 4 == 0, else 1)
  int cta_quantum; // CTA ranges start at multiples of this many units: `quantum`, or G (whole tiles)
  int two_way;     // every CTA range holds at least one tile's worth of units: a cut tile has two owners
  int xf16;        // the activations are fp16: `x` points to fp16 rows, or the prologue leaves fp16
                   // in shared memory (the normalised rows, which fp16 holds exactly, see make_job)
  __half* xn16_out;  // norm_rows_kernel only: optional fp16 copy of the normalised rows
  long ldx16;
  int xvec;        // x rows are 16-byte aligned with ldx % 8 == 0
  // fused residual + RMSNorm prologue (h_in != nullptr)
  const bf16* h_in;
  const int* tok;  // optional: row r of h_in is table row tok[r] (h_in = embedding table)
  int vocab;
  const bf16* delta;
  const bf16* norm_w;
  bf16* h_out;
  bf16* xn_out;
  long ldh, ldd, ldho, ldxo;
  float eps;
};

__device__ int g_w4_error = 0;

constexpr int kWaitLimit = 1 << 20;

// The stream is dealt out in quanta of q units, in two levels: equal shares of quanta per CTA
// (so every SM has the same amount of work to within one quantum), and inside a CTA equal shares
// of its quanta per warp.
__device__ __host__ __forceinline__ int cta_begin(int total, int q, int nctas, int c) {
  return q * share_begin(total / q, nctas, c);
}
__device__ __forceinline__ void warp_range(int total, int q, int qc, int nctas, int nwarps, int cta, int warp,
                                           int& u0, int& u1) {
  if (cta >= nctas) { u0 = u1 = total; return; }
  const int b = cta_begin(total, qc, nctas, cta), e = cta_begin(total, qc, nctas, cta + 1);
  u0 = b + q * share_begin((e - b) / q, nwarps, min(warp, nwarps));
  u1 = b + q * share_begin((e - b) / q, nwarps, min(warp + 1, nwarps));
}

// x fragment of a lane for the ragged cases (misaligned rows, or the last group when K is not a
// multiple of 128): element loads, zeros beyond K. Kept out of line: it is never on the hot path.
__device__ __noinline__ void load_x_slow(UnitOps& o, const bf16* row, int gg, int t, int K) {
  const unsigned short* xs = reinterpret_cast<const unsigned short*>(row);
  uint32_t v[16];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int k0 = gg * 128 + 64 * h + 16 * t;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int k = k0 + 2 * e;
      const uint32_t lo = k < K ? xs[k] : 0u, hi = k + 1 < K ? xs[k + 1] : 0u;
      v[h * 8 + e] = lo | (hi << 16);
    }
  }
  o.x0 = make_uint4(v[0], v[1], v[2], v[3]);   o.x1 = make_uint4(v[4], v[5], v[6], v[7]);
  o.x2 = make_uint4(v[8], v[9], v[10], v[11]); o.x3 = make_uint4(v[12], v[13], v[14], v[15]);
}

// The fused prologue: x_s[r] = RMSNorm1p(h_in[r] + delta[r]) * (1 + w) for r < N, computed by the
// whole CTA. A thread owns packets (8 elements) p = tid, tid + NT, ... of EVERY row: the loads of
// all rows are issued before the first dependent instruction, so the prologue costs one trip to
// L2, not one per row. Statistics in fp32, fixed reduction order (warp shuffle tree, then warps in
// order): a row's result does not depend on how many rows there are.
template <int NW>
__device__ __forceinline__ void norm_prologue(const GemvArgs& a, unsigned char* x_s, long pitch,
                                              float (*s_red)[NW], int tid, int r_lo, int r_hi, bool writer) {
  // x_s + r * pitch receives row r (shared memory inside the GEMV, the caller's xn buffer in the
  // stand-alone kernel below, which runs this same code on one row per block)
  constexpr int NT = NW * 32, RB = 4;  // rows are handled RB at a time (register budget)
  constexpr int WP = 3;                 // norm-weight packets a thread keeps (K <= 8 * WP * NT)
  const int lane = tid & 31, warp = tid >> 5, N = r_hi, npk = a.K >> 3;
  // the weight packets this thread needs in the second pass: requested now, so that their trip to
  // L2 overlaps the one of the rows
  const bool w_held = npk <= WP * NT;
  uint4 wv[WP];
#pragma unroll
  for (int i = 0; i < WP; ++i) {
    const int p = tid + i * NT;
    if (w_held && p < npk) wv[i] = reinterpret_cast<const uint4*>(a.norm_w)[p];
  }
#pragma unroll 1
  for (int r0 = r_lo; r0 < N; r0 += RB) {
    float ss[RB];
    const bf16* hrow[RB];
#pragma unroll
    for (int i = 0; i < RB; ++i) {
      const int r = r0 + i;
      ss[i] = 0.f;
      hrow[i] = nullptr;
      if (r < N) {
        if (a.tok) {
          const int id = a.tok[r];
          if (id >= 0 && id < a.vocab) hrow[i] = a.h_in + (size_t)id * a.K;  // else: a row of zeros
        } else {
          hrow[i] = a.h_in + (long)r * a.ldh;
        }
      }
    }
    for (int p = tid; p < npk; p += NT) {
      uint4 hv[RB], dv[RB];
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        if (r0 + i < N) {
          hv[i] = hrow[i] ? reinterpret_cast<const uint4*>(hrow[i])[p] : make_uint4(0u, 0u, 0u, 0u);
          if (a.delta) dv[i] = reinterpret_cast<const uint4*>(a.delta + (long)(r0 + i) * a.ldd)[p];
        }
      }
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        const int r = r0 + i;
        if (r < N) {
          float v[8];
          widen8(hv[i], v);
          if (a.delta) {
            float d[8];
            widen8(dv[i], d);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = rnd(v[e] + d[e]);
            hv[i] = narrow8(v);
          }
          reinterpret_cast<uint4*>(x_s + r * pitch)[p] = hv[i];
          if (writer && a.h_out) reinterpret_cast<uint4*>(a.h_out + (long)r * a.ldho)[p] = hv[i];
#pragma unroll
          for (int e = 0; e < 8; ++e) ss[i] = fmaf(v[e], v[e], ss[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < RB; ++i) {
      if (r0 + i < N) {
        const float w = warp_allsum(ss[i]);
        if (lane == 0) s_red[r0 + i - r_lo][warp] = w;
      }
    }
  }
  __syncthreads();
#pragma unroll 1
  for (int r0 = r_lo; r0 < N; r0 += RB) {
    float inv[RB];
#pragma unroll
    for (int i = 0; i < RB; ++i) {
      inv[i] = 0.f;
      if (r0 + i < N) {
        float tot = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < NW; ++w2) tot += s_red[r0 + i - r_lo][w2];
        inv[i] = rsqrtf(tot / (float)a.K + a.eps);
      }
    }
    int pi = 0;
    for (int p = tid; p < npk; p += NT, ++pi) {  // same thread -> packet map as above: own data only
      float g[8];
      uint4 wq = wv[0];
      if (!w_held) wq = reinterpret_cast<const uint4*>(a.norm_w)[p];
      else if (pi == 1) wq = wv[1];
      else if (pi == 2) wq = wv[2];
      widen8(wq, g);
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        const int r = r0 + i;
        if (r < N) {
          uint4* xs = reinterpret_cast<uint4*>(x_s + r * pitch);
          float v[8], y[8];
          widen8(xs[p], v);
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] = v[e] * inv[i] * (1.0f + g[e]);
          const uint4 q = narrow8(y);
          const bool in_place = reinterpret_cast<unsigned char*>(a.xn_out) == x_s;  // stand-alone kernel
          if (a.xf16) {  // the bf16-rounded values again, as fp16 (exact for normalised rows)
            widen8(q, y);
            const uint4 q16 = half8(y);
            if (in_place) {
              xs[p] = q;
              if (a.xn16_out) reinterpret_cast<uint4*>(a.xn16_out + (long)r * a.ldx16)[p] = q16;
            } else {
              xs[p] = q16;
            }
          } else {
            xs[p] = q;
          }
          if (writer && a.xn_out && !in_place) reinterpret_cast<uint4*>(a.xn_out + (long)r * a.ldxo)[p] = q;
        }
      }
    }
  }
  __syncthreads();
}

// The prologue as a launch of its own: one block per row, the same thread -> packet map and the
// same reduction order as inside the GEMV, hence the same bits. A pass of several rows runs this
// (the rows in parallel on as many SMs) in front of a plain GEMV instead of letting every block
// of the GEMV repeat the work for all rows; h_out may alias h_in here (a thread reads and writes
// its own packets only).
template <int NW>
__global__ void __launch_bounds__(NW * 32) norm_rows_kernel(const GemvArgs a) {
  dep_release();
  dep_wait();
  __shared__ float s_red[QE_MAX_ROWS][NW];
  const int r = blockIdx.x;
  norm_prologue<NW>(a, reinterpret_cast<unsigned char*>(a.xn_out), a.ldxo * 2, s_red, threadIdx.x, r, r + 1, true);
}

// A chain is up to kMaxJobs GEMVs that depend on each other only through global memory (the
// output of one is the input, or the residual update, of the next). They run as ONE cooperative
// launch: the blocks meet at a grid-wide barrier between two jobs, and every warp asks the copy
// engine for the head of its slab of the next matrix BEFORE it goes to the barrier, so the
// memory pipeline never drains at a job boundary the way it does at a kernel boundary (a
// separate launch costs about 6.6 us here before its first byte is multiplied).
constexpr int kMaxJobs = 4;
struct ChainArgs {
  GemvArgs job[kMaxJobs];
  int njobs;
  int* gbar;  // [0] arrivals of the current barrier, [1] generation (never reset)
};

// Grid-wide barrier for co-resident blocks (cooperative launch). Release: every thread's writes,
// then a device-scope fence by the arriving thread; acquire: fence after the generation moved
// (which also drops stale L1 lines, so plain loads afterwards see the other blocks' output).
// The spin is bounded: on expiry the error word is set and the block goes on (wrong results,
// reported; never a hang).
__device__ __forceinline__ void grid_barrier(int* gbar, int nblocks) {
  __syncthreads();
  if (threadIdx.x == 0) {
    volatile int* vg = gbar;
    const int gen = vg[1];
    __threadfence();
    if (atomicAdd(gbar, 1) == nblocks - 1) {
      vg[0] = 0;
      __threadfence();
      atomicAdd(gbar + 1, 1);
    } else {
      int spins = 0;
      while (vg[1] == gen) {
        if (++spins > (1 << 24)) {
          atomicExch(&g_w4_error, 2);
          break;
        }
      }
    }
    __threadfence();
  }
  __syncthreads();
}

template <int NW, int PERW, int STAGES>
__global__ void __launch_bounds__(NW * 32, 1) w4_chain_kernel(const __grid_constant__ ChainArgs c) {
  constexpr uint32_t kStageW = PERW * 1024, kStageS = PERW * 32;
  constexpr uint32_t kRing = STAGES * (kStageW + kStageS);
  dep_release();
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[NW][STAGES];
  __shared__ int s_rb[NW + 1];
  __shared__ float s_red[QE_MAX_ROWS][NW];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, t = lane & 3;
  unsigned char* ring_w = smem + (size_t)warp * kRing;
  unsigned char* ring_s = ring_w + (size_t)STAGES * kStageW;
  float* part = reinterpret_cast<float*>(smem + (size_t)NW * kRing);  // [NW][2][128]
  unsigned char* x_s = smem + (size_t)NW * kRing + (size_t)NW * 2 * 128 * sizeof(float);

  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) bar_init(&full[warp][s], 1);
    bar_fence_init();
  }
  __syncwarp();

  // Ring position of the next stage to consume; it runs on across jobs (a slot's barrier
  // completes one phase per fill, whichever matrix the fill came from).
  int slot = 0, phase = 0;
  bool ok = true;

  // lane 0: request stages [st0, st1) of the range [u0, u1) of job `a`, into consecutive ring
  // slots starting at `at`
  auto fill = [&](const GemvArgs& a, int u0, int u1, int st0, int st1, int at) {
    for (int st = st0; st < st1; ++st) {
      const int ub = u0 + st * PERW, cnt = min(PERW, u1 - ub);
      bar_expect(&full[warp][at], (uint32_t)cnt * (1024 + 32));
      bulk_g2s(ring_w + (size_t)at * kStageW, a.qw + (size_t)ub * 64, (uint32_t)cnt * 1024, &full[warp][at]);
      bulk_g2s(ring_s + (size_t)at * kStageS, a.scales + (size_t)ub * 16, (uint32_t)cnt * 32, &full[warp][at]);
      if (++at == STAGES) at = 0;
    }
  };
  auto range_of = [&](const GemvArgs& a, int& u0, int& u1) {
    warp_range(a.total, a.quantum, a.cta_quantum, a.nctas, a.nwarps, blockIdx.x, warp, u0, u1);
  };

  // weights never depend on the producer of x: the first stages are requested before the
  // programmatic-dependency wait
  {
    int u0, u1;
    range_of(c.job[0], u0, u1);
    if (lane == 0) fill(c.job[0], u0, u1, 0, min(STAGES, (u1 - u0 + PERW - 1) / PERW), 0);
  }
  dep_wait();

#pragma unroll 1
  for (int j = 0; j < c.njobs; ++j) {
    const GemvArgs& a = c.job[j];
    const int G = a.G, total = a.total;
    int u0, u1;
    range_of(a, u0, u1);
    if (lane == 0) {
      s_rb[warp] = u0;
      if (warp == NW - 1) s_rb[NW] = u1;
    }
    const int n_units = u1 - u0;
    const int nstage = (n_units + PERW - 1) / PERW;

    // ---- where this lane's x fragments come from ----
    // Lane (r, t) multiplies activation row r; rows >= N feed mma columns that are never stored
    // and simply re-read row N - 1. With the prologue x lives in shared memory (pitch + 16 B so
    // that the rows of a quarter-warp fall into different banks); both cases are read through one
    // generic pointer so that the stage body below exists once.
    const int xrow = min(r, a.o.N - 1);
    const unsigned char* xbase;
    bool xfast;
    if (a.h_in) {
      const long pitch = (long)a.K * 2 + 16;
      norm_prologue<NW>(a, x_s, pitch, s_red, tid, 0, a.o.N, blockIdx.x == 0);
      xbase = x_s + xrow * pitch + 32 * t;
      xfast = true;
    } else {
      xbase = reinterpret_cast<const unsigned char*>(a.x + (long)xrow * a.ldx) + 32 * t;
      xfast = a.xvec != 0;
    }
    const bool tail_k = (a.K & 127) != 0;  // the last group reads past K unless guarded

    // ---- the stream ----
    int tile = u0 / G;
    int g = u0 - tile * G;   // group of the next unit
    int seg_gb = g;          // first group of the segment held in acc
    float acc[4] = {0.f, 0.f, 0.f, 0.f};

    // A segment [seg_gb, g) of `tile` is complete: a whole tile is stored, a cut one parked (slot
    // 0 if this range starts inside the tile, slot 1 if it holds the tile's head).
    auto close_segment = [&]() {
      if (seg_gb == 0 && g == G) {
        tile_out(a.o, tile, acc, lane);
      } else {
        float* p = part + (warp * 2 + (seg_gb != 0 ? 0 : 1)) * 128;
#pragma unroll
        for (int k = 0; k < 4; ++k) p[k * 32 + lane] = acc[k];
      }
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      if (g == G) { g = 0; ++tile; }
      seg_gb = g;
    };

    // The stream exists twice, once per activation type (a.xf16): two separate loops, each with
    // its own register allocation, in ONE kernel function -- both unpack flavours inlined side by
    // side in one loop spill, and two kernel functions that alternate from launch to launch cost
    // more in instruction fetch than the cheaper unpack saves.
    auto stream = [&](auto f16_tag) {
      constexpr bool F16 = decltype(f16_tag)::value;
      // Both loops below walk the ring stage by stage. The fast one serves ranges made of whole
      // stages that never straddle a tile (every matrix of the model): no per-unit decisions at
      // all, every operand at an immediate offset from three base pointers.
      const bool all_fast = xfast && !tail_k && (a.quantum % PERW) == 0;
      if (all_fast) {
        const unsigned char* xg = xbase + (size_t)g * 256;
        // the next stage to request from HBM: whole stages only in this loop, so the copy sizes are
        // constants and the global addresses advance by constants
        const unsigned char* gw = reinterpret_cast<const unsigned char*>(a.qw) + (size_t)(u0 + STAGES * PERW) * 1024;
        const unsigned char* gs = reinterpret_cast<const unsigned char*>(a.scales) + (size_t)(u0 + STAGES * PERW) * 32;
        int to_request = nstage - STAGES;  // stages not yet requested
  #pragma unroll 1
        for (int st = 0; st < nstage && ok; ++st) {
          uint64_t* bar = &full[warp][slot];
          if (!bar_wait(bar, phase, kWaitLimit)) {
            ok = false;
            atomicExch(&g_w4_error, 1);
            break;
          }
          unsigned char* stage_w = ring_w + (size_t)slot * kStageW;
          unsigned char* stage_s = ring_s + (size_t)slot * kStageS;
          const uint4* wp = reinterpret_cast<const uint4*>(stage_w) + lane;
          const unsigned short* sp = reinterpret_cast<const unsigned short*>(stage_s) + r;
          const uint4* xp = reinterpret_cast<const uint4*>(xg);
          UnitOps ops[PERW];
  #pragma unroll
          for (int i = 0; i < PERW; ++i) {
            ops[i].w0 = wp[i * 64];
            ops[i].w1 = wp[i * 64 + 32];
            ops[i].s_lo = sp[i * 16];
            ops[i].s_hi = sp[i * 16 + 8];
            ops[i].x0 = xp[i * 16];
            ops[i].x1 = xp[i * 16 + 1];
            ops[i].x2 = xp[i * 16 + 8];
            ops[i].x3 = xp[i * 16 + 9];
          }
  #pragma unroll
          for (int i = 0; i < PERW; ++i) {
            if constexpr (F16) unit_fma_f16(acc, ops[i]);
            else unit_fma(acc, ops[i]);
          }
          g += PERW;
          xg += PERW * 256;
          if (g == G || st == nstage - 1) {
            close_segment();
            xg = xbase + (size_t)g * 256;
          }
          __syncwarp();  // every lane has read this stage: hand its slot back to the copy engine
          if (to_request > 0) {
            if (lane == 0) {
              async_proxy_fence();
              bar_expect(bar, kStageW + kStageS);
              bulk_g2s(stage_w, gw, kStageW, bar);
              bulk_g2s(stage_s, gs, kStageS, bar);
            }
            gw += kStageW;
            gs += kStageS;
            --to_request;
          }
          if (++slot == STAGES) { slot = 0; phase ^= 1; }
        }
      } else {
  #pragma unroll 1
        for (int st = 0; st < nstage && ok; ++st) {
          if (!bar_wait(&full[warp][slot], phase, kWaitLimit)) {
            ok = false;
            atomicExch(&g_w4_error, 1);
            break;
          }
          const uint4* wp = reinterpret_cast<const uint4*>(ring_w + (size_t)slot * kStageW) + lane;
          const unsigned short* sp = reinterpret_cast<const unsigned short*>(ring_s + (size_t)slot * kStageS) + r;
          const int cnt = min(PERW, n_units - st * PERW);
  #pragma unroll 1
          for (int i = 0; i < cnt; ++i) {
            UnitOps o;
            o.w0 = wp[i * 64];
            o.w1 = wp[i * 64 + 32];
            o.s_lo = sp[i * 16];
            o.s_hi = sp[i * 16 + 8];
            if (xfast && !(tail_k && g == G - 1)) {
              const uint4* xp = reinterpret_cast<const uint4*>(xbase + (size_t)g * 256);
              o.x0 = xp[0]; o.x1 = xp[1]; o.x2 = xp[8]; o.x3 = xp[9];
            } else {
              load_x_slow(o, a.x + (long)xrow * a.ldx, g, t, a.K);
            }
            if constexpr (F16) unit_fma_f16(acc, o);
            else unit_fma(acc, o);
            ++g;
            if (g == G || (st == nstage - 1 && i == cnt - 1)) close_segment();
          }
          __syncwarp();
          if (lane == 0 && st + STAGES < nstage) {
            async_proxy_fence();
            fill(a, u0, u1, st + STAGES, st + STAGES + 1, slot);
          }
          if (++slot == STAGES) { slot = 0; phase ^= 1; }
        }
      }
    };
    if (a.xf16) stream(std::true_type{});
    else stream(std::false_type{});

    // This warp's ring is empty: ask for the head of its slab of the next matrix now, so that the
    // copies run while the blocks finish this job and meet at the barrier.
    if (ok && j + 1 < c.njobs) {
      int v0, v1;
      range_of(c.job[j + 1], v0, v1);
      __syncwarp();
      if (lane == 0) {
        async_proxy_fence();
        fill(c.job[j + 1], v0, v1, 0, min(STAGES, (v1 - v0 + PERW - 1) / PERW), slot);
      }
    }
    __syncthreads();  // every partial tile of this CTA is in shared memory, s_rb is complete

    // ---- cut tiles: combined by the warp holding the head, ascending warp order ----
    const int cta_b = s_rb[0], cta_e = s_rb[NW];
    const int my_cta = blockIdx.x;
    auto publish = [&](int T, const float (&f)[4], int units, int pslot) {
      if (a.two_way && a.o.epi != QE_EPI_SWIGLU) {
        // Two owners, one round trip: both swap their partial into the same slot (the lower
        // CTA's slot 1). Per element, whoever gets the other's value back is second: it adds,
        // writes the output and empties the slot again. The sum of two numbers does not depend
        // on who was first. Empty = +0.0, so a partial that is +0.0 travels as -0.0 (same sum).
        float* sl = a.ws + ((size_t)(pslot ? my_cta : my_cta - 1) * 2 + 1) * 128;
        unsigned old[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          unsigned bits = __float_as_uint(f[k]);
          if (bits == 0u) bits = 0x80000000u;
          old[k] = atomicExch(reinterpret_cast<unsigned*>(sl + k * 32 + lane), bits);
        }
        float sum[4];
        unsigned mask = 0u;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          sum[k] = __uint_as_float(old[k]) + f[k];
          if (old[k] != 0u) {
            mask |= 1u << k;
            __stcg(sl + k * 32 + lane, 0.f);
          }
        }
        if (mask) tile_out(a.o, T, sum, lane, mask);
        return;
      }
      // one partial per CTA through global memory; whoever completes the tile adds them all
      float* gm = a.ws + ((size_t)my_cta * 2 + pslot) * 128;
#pragma unroll
      for (int k = 0; k < 4; ++k) __stcg(gm + k * 32 + lane, f[k]);
      __syncwarp();  // orders the 32 lanes' stores before lane 0's release
      int done = 0;
      if (lane == 0) {
        cuda::atomic_ref<int, cuda::thread_scope_device> arrivals(a.counters[T]);
        done = arrivals.fetch_add(units, cuda::memory_order_acq_rel) + units == G;
      }
      done = __shfl_sync(0xffffffffu, done, 0);  // also orders lane 0's acquire before the loads below
      if (!done) return;
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      const int q = a.cta_quantum;
      const int c_lo = share_owner(total / q, a.nctas, (T * G) / q);
      const int c_hi = share_owner(total / q, a.nctas, (T * G + G - 1) / q);
#pragma unroll 1
      for (int cc = c_lo; cc <= c_hi; ++cc) {
        const int cb = cta_begin(total, q, a.nctas, cc);
        float* p = a.ws + ((size_t)cc * 2 + (cb > T * G ? 0 : 1)) * 128;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          sum[k] += __ldcg(p + k * 32 + lane);
          __stcg(p + k * 32 + lane, 0.f);  // the slots are left empty for the two-owner exchange
        }
      }
      tile_out(a.o, T, sum, lane);
      if (lane == 0) a.counters[T] = 0;
    };

    if (ok && n_units > 0 && (u1 % G) != 0) {
      const int T = (u1 - 1) / G;
      if (T * G >= u0) {  // the head of tile T is in this warp's slot 1
        const int tend = T * G + G;
        float f[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) f[k] = part[(warp * 2 + 1) * 128 + k * 32 + lane];
        for (int w2 = warp + 1; w2 < NW && s_rb[w2] < min(tend, cta_e); ++w2) {
#pragma unroll
          for (int k = 0; k < 4; ++k) f[k] += part[(w2 * 2) * 128 + k * 32 + lane];
        }
        if (tend <= cta_e) tile_out(a.o, T, f, lane);
        else publish(T, f, cta_e - T * G, 1);
      }
    }
    if (warp == 0 && ok && cta_e > cta_b && (cta_b % G) != 0) {  // tile that began in an earlier CTA
      const int T = cta_b / G, tend = T * G + G;
      float f[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) f[k] = part[k * 32 + lane];
      for (int w2 = 1; w2 < NW && s_rb[w2] < min(tend, cta_e); ++w2) {
#pragma unroll
        for (int k = 0; k < 4; ++k) f[k] += part[(w2 * 2) * 128 + k * 32 + lane];
      }
      publish(T, f, min(tend, cta_e) - cta_b, 0);
    }
    if (j + 1 < c.njobs) grid_barrier(c.gbar, gridDim.x);  // also separates the uses of part / s_rb
  }
  if (!ok) {
    // Give the copies that are still in flight a bounded chance to land before the CTA exits.
    __syncwarp();
    for (int s = 0; s < STAGES; ++s) bar_wait(&full[warp][s], 0, 1 << 10), bar_wait(&full[warp][s], 1, 1 << 10);
  }
}

// ---- host side -----------------------------------------------------------------------------------
using KernelFn = void (*)(const ChainArgs);

struct Geometry {
  KernelFn fn;
  int nw, perw, stages;
  size_t ring_bytes() const { return (size_t)nw * stages * perw * (1024 + 32) + (size_t)nw * 2 * 128 * sizeof(float); }
};
template <int NW, int PERW, int STAGES>
constexpr Geometry geometry() {
  return Geometry{w4_chain_kernel<NW, PERW, STAGES>, NW, PERW, STAGES};
}
// Selected by the reference's launch options. `warps`: 0 (auto) / 16 -> 16 warps per CTA, 4 / 8 -> 8;
// variant 1 -> 24 warps, variant 2 -> 20 warps. `unroll` picks the ring: 2 -> 3 stages of 2 units, 4 -> 2
// stages of 4 units, 1 -> 2 stages of 2 units (the smallest; leaves room for eight rows of
// prologue input), 0 -> the deepest of the three that fits beside the prologue's rows. Work is split by CTA size only, so every ring shape of one CTA size gives the
// same bits.
const Geometry kGeoms[] = {geometry<16, 2, 3>(), geometry<16, 4, 2>(), geometry<16, 2, 2>(),
                           geometry<20, 2, 3>(), geometry<20, 4, 2>(), geometry<20, 2, 2>(),
                           geometry<8, 2, 3>(),  geometry<8, 4, 2>(),  geometry<8, 2, 2>(),
                           geometry<24, 2, 3>()};

// `ring` < 0: whatever `unroll` says (0 -> the 3 x 2 ring); 0..2: that ring of the chosen CTA size.
const Geometry& pick_geometry(const qe_w4_cfg& c, int ring = -1) {
  if (c.variant == 1) return kGeoms[9];
  if (ring < 0) ring = c.unroll == 4 ? 1 : c.unroll == 1 ? 2 : 0;
  const int size = (c.warps == 4 || c.warps == 8) ? 2 : c.variant == 2 ? 1 : 0;
  return kGeoms[3 * size + ring];
}

// Largest dynamic shared memory a launch of `fn` may ask for on the current device (the opt-in
// maximum minus the kernel's static shared memory). Raising the per-function limit is a per-device
// setting: done once per (function, device). Returns < 0 (minus the CUDA error) on failure.
long dynamic_smem_limit(KernelFn fn) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, long> known;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return -(long)e;
  std::lock_guard<std::mutex> lk(mu);
  auto it = known.find({(const void*)fn, dev});
  if (it != known.end()) return it->second;
  int optin = 0;
  cudaFuncAttributes fa{};
  if ((e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess ||
      (e = cudaFuncGetAttributes(&fa, fn)) != cudaSuccess)
    return -(long)e;
  const long limit = (long)optin - (long)fa.sharedSizeBytes;
  if ((e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit)) != cudaSuccess)
    return -(long)e;
  known[{(const void*)fn, dev}] = limit;
  return limit;
}

// Experiment knob with the reference's syntax (csrc/gemv_w4.cu:427-449):
//   QE_W4_CFG="TxG:mode,warps,unroll,ksplit,bps,min_units;..."   (T = Mp / 16, G = Kp / 128)
// replaces the launch options for the named shapes (never keyed on N). Read once per process.
struct ShapeCfg {
  long T, G;
  qe_w4_cfg c;
};
const std::vector<ShapeCfg>& env_overrides() {
  static const std::vector<ShapeCfg> table = [] {
    std::vector<ShapeCfg> v;
    const char* env = std::getenv("QE_W4_CFG");
    if (!env) return v;
    std::string all(env);
    for (size_t at = 0; at < all.size();) {
      const size_t end = std::min(all.find(';', at), all.size());
      ShapeCfg e{};
      if (std::sscanf(all.substr(at, end - at).c_str(), "%ldx%ld:%d,%d,%d,%d,%d,%d", &e.T, &e.G, &e.c.mode,
                      &e.c.warps, &e.c.unroll, &e.c.ksplit, &e.c.blocks_per_sm, &e.c.min_units) == 8)
        v.push_back(e);
      at = end + 1;
    }
    return v;
  }();
  return table;
}

struct Resolved {
  qe_w4_plan plan;
  const Geometry* geom;
  int nctas, nwarps, quantum, cta_quantum, two_way;
};

// Shape-only launch policy (never N): as many warps as there are units / min_units, at most one
// CTA per SM; ksplit > 0 asks for at least that many warps per tile.
Resolved resolve(const qe_w4_params& p, const qe_w4_cfg& c_in) {
  Resolved r{};
  const long tiles = p.Mp / 16, G = p.Kp / 128, units = tiles * G;
  qe_w4_cfg c = c_in;
  for (const ShapeCfg& e : env_overrides())
    if (e.T == tiles && e.G == G) {
      c.mode = e.c.mode; c.warps = e.c.warps; c.unroll = e.c.unroll; c.ksplit = e.c.ksplit;
      c.blocks_per_sm = e.c.blocks_per_sm; c.min_units = e.c.min_units;
    }
  r.geom = &pick_geometry(c);
  long min_units = std::max(1, c.min_units);
  if (c.ksplit > 0) min_units = std::max<long>(1, std::min<long>(min_units, G / std::min<long>(c.ksplit, G)));
  const long sms = qe_sm_count();
  const long ctas_max = sms;  // one CTA per SM
  // ranges are dealt out in quanta of 4 units (a whole number of ring stages in every geometry)
  // when the tiles are a whole number of quanta long, so that a stage never straddles two tiles
  const long quantum = (G % 4 == 0) ? 4 : 1;  // the same for every ring geometry: same split, same bits
  const long want = (units + min_units - 1) / min_units;  // warps that would each get min_units
  // small matrices: as many CTAs as possible (every SM pulls from HBM), fewer warps in each
  const long ctas = std::max<long>(1, std::min<long>({ctas_max, want, units / quantum}));
  const long per_cta = (units + ctas - 1) / ctas;
  r.nwarps = (int)std::max<long>(1, std::min<long>(r.geom->nw, (per_cta + min_units - 1) / min_units));
  r.quantum = (int)quantum;
  // CTA ranges of whole tiles where that costs less than the exchange of cut tiles between CTAs
  // (two global round trips at the end of the launch, about a microsecond): the surplus of the
  // fullest CTA over the even share, at about 30 ns per unit, must stay well below that. Decided
  // from the shape alone, like everything else in the plan.
  const long tiles_max = (tiles + ctas - 1) / ctas;
  const bool whole_tiles = ctas > 1 && tiles >= ctas && (tiles_max * ctas - tiles) * G <= 26 * ctas;
  r.cta_quantum = whole_tiles ? (int)G : (int)quantum;
  // the smallest CTA range in units; at least a tile long means no tile has three owners
  r.two_way = ((units / r.cta_quantum) / ctas) * r.cta_quantum >= G ? 1 : 0;
  r.nctas = (int)ctas;
  r.plan.mode = 4;
  r.plan.grid_x = (int)ctas;
  r.plan.grid_y = 1;
  r.plan.threads = r.geom->nw * 32;
  r.plan.ws_floats = (long)r.plan.grid_x * 2 * 128;
  r.plan.counters = tiles;
  return r;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check_params(const qe_w4_params* p, const qe_w4_cfg* cfg) {
  if (!p || !cfg) return QE_ERR_ARG;
  if (p->N < 1 || p->N > QE_MAX_ROWS || p->Mp % 16 || p->Kp % 128 || p->Mp <= 0 || p->Kp <= 0) return QE_ERR_ARG;
  if (p->K > p->Kp || p->K <= p->Kp - 128 || p->M <= 0) return QE_ERR_ARG;
  if (p->epilogue == QE_EPI_SWIGLU ? p->M > p->Mp / 2 : p->M > p->Mp) return QE_ERR_ARG;
  if (p->epilogue != QE_EPI_NONE && p->epilogue != QE_EPI_SWIGLU) return QE_ERR_ARG;
  if ((long)(p->Mp / 16) * (p->Kp / 128) >= (1L << 30)) return QE_ERR_ARG;  // 32-bit unit arithmetic
  if (!aligned16(p->qw) || !aligned16(p->scales)) return QE_ERR_ARG;        // bulk copies need 16 B
  return 0;
}

// Fill the device-side description of one job; *smem_extra = shared memory its prologue needs.
int make_job(const qe_w4_params* p, const qe_w4_norm* nrm, const qe_w4_cfg* cfg, GemvArgs& a, Resolved& r,
             size_t* smem_extra) {
  int rc = check_params(p, cfg);
  if (rc) return rc;
  r = resolve(*p, *cfg);
  a = GemvArgs{};
  a.qw = reinterpret_cast<const uint4*>(p->qw);
  a.scales = reinterpret_cast<const __half*>(p->scales);
  a.x = reinterpret_cast<const bf16*>(p->x);
  a.ldx = p->ldx;
  a.o.out = p->out;
  a.o.ldo = p->ldo;
  a.o.M = p->M;
  a.o.N = p->N;
  a.o.epi = p->epilogue;
  a.o.out_f32 = (p->out_f32 && p->epilogue == QE_EPI_NONE) ? 1 : 0;
  a.ws = p->ws;
  a.counters = p->counters;
  a.K = p->K;
  a.G = p->Kp / 128;
  a.total = (p->Mp / 16) * a.G;
  a.nctas = r.nctas;
  a.nwarps = r.nwarps;
  a.quantum = r.quantum;
  a.cta_quantum = r.cta_quantum;
  a.two_way = r.two_way;
  a.xvec = ((p->ldx & 7) == 0 && aligned16(p->x)) ? 1 : 0;
  *smem_extra = 0;
  if (nrm && nrm->h_in) {
    // the prologue holds N rows of x in shared memory and reads / writes 16-byte packets
    if (p->K != p->Kp || !nrm->norm_w || !aligned16(nrm->h_in) || !aligned16(nrm->norm_w) || (nrm->ldh & 7) ||
        (nrm->delta && (!aligned16(nrm->delta) || (nrm->ldd & 7))) ||
        (nrm->h_out && (!aligned16(nrm->h_out) || (nrm->ldho & 7) || nrm->h_out == nrm->h_in)) ||
        (nrm->xn_out && (!aligned16(nrm->xn_out) || (nrm->ldxo & 7))) || (nrm->tok && nrm->vocab < 1))
      return QE_ERR_ARG;
    *smem_extra = (size_t)p->N * ((size_t)p->K * 2 + 16);
    a.h_in = reinterpret_cast<const bf16*>(nrm->h_in);
    a.tok = nrm->tok;
    a.vocab = nrm->vocab;
    a.delta = reinterpret_cast<const bf16*>(nrm->delta);
    a.norm_w = reinterpret_cast<const bf16*>(nrm->norm_w);
    a.h_out = reinterpret_cast<bf16*>(nrm->h_out);
    a.xn_out = reinterpret_cast<bf16*>(nrm->xn_out);
    a.ldh = nrm->ldh; a.ldd = nrm->ldd; a.ldho = nrm->ldho; a.ldxo = nrm->ldxo;
    a.eps = nrm->eps;
    a.xf16 = nrm->f16 ? 1 : 0;
  } else if (!p->x) {
    return QE_ERR_ARG;
  } else if (p->x_f16) {
    // fp16 activations are served by the vector path only: whole groups, aligned rows
    if (p->K != p->Kp || !a.xvec) return QE_ERR_ARG;
    a.xf16 = 1;
  }
  return 0;
}

int launch_chain(const qe_w4_params* const* ps, const qe_w4_norm* const* nrms, int njobs, const qe_w4_cfg* cfg,
                 int* gridbar, cudaStream_t stream) {
  if (!ps || !cfg || njobs < 1 || njobs > kMaxJobs || (njobs > 1 && !gridbar)) return QE_ERR_ARG;
  ChainArgs c{};
  c.njobs = njobs;
  c.gbar = gridbar;
  const Geometry* geom = nullptr;
  size_t extra = 0;
  int grid = 1;
  for (int j = 0; j < njobs; ++j) {
    Resolved r{};
    size_t e = 0;
    const int rc = make_job(ps[j], nrms ? nrms[j] : nullptr, cfg, c.job[j], r, &e);
    if (rc) return rc;
    geom = r.geom;
    extra = std::max(extra, e);
    grid = std::max(grid, r.plan.grid_x);
  }
  // unroll = 0 (auto): the deepest ring that still leaves room for the prologue's rows. The split of
  // the work depends on the CTA size only, so this choice never changes a result.
  if (cfg->unroll == 0 && cfg->variant != 1) {
    for (int ring : {1, 0, 2}) {
      const Geometry& cand = pick_geometry(*cfg, ring);
      const long lim = dynamic_smem_limit(cand.fn);
      if (lim < 0) return (int)-lim;
      geom = &cand;
      if ((long)(cand.ring_bytes() + extra) <= lim) break;
    }
  }
  const size_t smem = geom->ring_bytes() + extra;
  const long limit = dynamic_smem_limit(geom->fn);
  if (limit < 0) return (int)-limit;
  if ((long)smem > limit) return QE_ERR_ARG;  // prologue rows do not fit: run qe_rmsnorm1p + qe_w4_gemv
  const bool pdl = cfg->pdl && pdl_launch_enabled() && pdl_trigger_enabled();
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid, 1, 1);
  lc.blockDim = dim3(geom->nw * 32, 1, 1);
  lc.dynamicSmemBytes = smem;
  lc.stream = stream;
  cudaLaunchAttribute at[2];
  int na = 0;
  if (pdl) {
    at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (njobs > 1) {  // the blocks wait for each other: they must all be resident
    at[na].id = cudaLaunchAttributeCooperative;
    at[na].val.cooperative = 1;
    ++na;
  }
  lc.attrs = at;
  lc.numAttrs = na;
  return (int)cudaLaunchKernelEx(&lc, geom->fn, c);
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
  (void)warps;
  // Large matrices need no hint: the unit stream is cut per warp anyway. A small one is cut along
  // K until every SM has a couple of warps to run.
  const long tiles = Mp / 16, G = Kp / 128;
  if (tiles * G >= 4096) return 1;
  const long want = 2L * qe_sm_count();
  long ks = 1;
  while (tiles * ks < want && ks * 2 <= G) ks *= 2;
  return (int)ks;
}

extern "C" int qe_w4_plan_gemv(const qe_w4_params* p, const qe_w4_cfg* cfg, qe_w4_plan* plan) {
  if (!p || !cfg || !plan) return QE_ERR_ARG;
  if (p->Mp <= 0 || p->Kp <= 0 || p->Mp % 16 || p->Kp % 128) return QE_ERR_ARG;
  *plan = resolve(*p, *cfg).plan;
  return 0;
}

extern "C" int qe_w4_ring_error(void) {
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_w4_error, sizeof(int)) != cudaSuccess) return -1;
  const int m = gemm_error_read();
  if (m < 0) return -1;
  return v | (m ? 16 * m : 0);
}

extern "C" int qe_w4_clear_error(void) {
  const int z = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  const int rc = gemm_error_clear();
  if (rc) return rc;
  return (int)cudaMemcpyToSymbol(g_w4_error, &z, sizeof(int));
}

extern "C" int qe_w4_gemv(const qe_w4_params* p, const qe_w4_cfg* cfg, void* stream) {
  return launch_chain(&p, nullptr, 1, cfg, nullptr, (cudaStream_t)stream);
}

extern "C" int qe_w4_gemv_ex(const qe_w4_params* p, const qe_w4_norm* nrm, const qe_w4_cfg* cfg, void* stream) {
  return launch_chain(&p, &nrm, 1, cfg, nullptr, (cudaStream_t)stream);
}

extern "C" int qe_w4_norm_rows(const qe_w4_norm* nrm, int N, int K, const qe_w4_cfg* cfg, void* stream) {
  if (!nrm || !cfg || N < 1 || N > QE_MAX_GEMM_ROWS || K < 8 || (K & 7) || !nrm->h_in || !nrm->norm_w || !nrm->xn_out)
    return QE_ERR_ARG;
  if (!aligned16(nrm->h_in) || !aligned16(nrm->norm_w) || !aligned16(nrm->xn_out) || (nrm->ldh & 7) || (nrm->ldxo & 7) ||
      (nrm->xn16_out && (!aligned16(nrm->xn16_out) || (nrm->ldx16 & 7))) ||
      (nrm->delta && (!aligned16(nrm->delta) || (nrm->ldd & 7))) ||
      (nrm->h_out && (!aligned16(nrm->h_out) || (nrm->ldho & 7))) || (nrm->tok && nrm->vocab < 1))
    return QE_ERR_ARG;
  GemvArgs a{};
  a.K = K;
  a.o.N = N;
  a.h_in = reinterpret_cast<const bf16*>(nrm->h_in);
  a.tok = nrm->tok;
  a.vocab = nrm->vocab;
  a.delta = reinterpret_cast<const bf16*>(nrm->delta);
  a.norm_w = reinterpret_cast<const bf16*>(nrm->norm_w);
  a.h_out = reinterpret_cast<bf16*>(nrm->h_out);
  a.xn_out = reinterpret_cast<bf16*>(nrm->xn_out);
  a.ldh = nrm->ldh; a.ldd = nrm->ldd; a.ldho = nrm->ldho; a.ldxo = nrm->ldxo;
  a.eps = nrm->eps;
  if (nrm->xn16_out) {
    a.xf16 = 1;
    a.xn16_out = reinterpret_cast<__half*>(nrm->xn16_out);
    a.ldx16 = nrm->ldx16;
  }
  const bool pdl = cfg->pdl && pdl_launch_enabled() && pdl_trigger_enabled();
  const int nw = pick_geometry(*cfg).nw;  // the reduction order follows the CTA size of the GEMV
  cudaStream_t s = (cudaStream_t)stream;
  switch (nw) {
    case 8: return (int)launch(norm_rows_kernel<8>, dim3(N), dim3(256), 0, s, pdl, a);
    case 16: return (int)launch(norm_rows_kernel<16>, dim3(N), dim3(512), 0, s, pdl, a);
    case 24: return (int)launch(norm_rows_kernel<24>, dim3(N), dim3(768), 0, s, pdl, a);
    default: return (int)launch(norm_rows_kernel<20>, dim3(N), dim3(640), 0, s, pdl, a);
  }
}

extern "C" int qe_w4_gemv_chain(const qe_w4_params* const* p, const qe_w4_norm* const* nrm, int njobs,
                                const qe_w4_cfg* cfg, int* gridbar, void* stream) {
  return launch_chain(p, nrm, njobs, cfg, gridbar, (cudaStream_t)stream);
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
