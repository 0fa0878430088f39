// W4A16 GEMM for up to 64 activation rows on B200 (sm_100a): the weight matrix is streamed from
// HBM once for all rows of a prefill pass, where the GEMV (w4_gemv.cu, 1..8 rows) would stream it
// once per 8 rows.
//
//   out[n, m] = bf16( sum_g fp32(scale[m, g]) * sum_{k in group g} (code[m, k] - 8) * x[n, k] )
//
// No counterpart in the reference, which prefills in passes of at most 8 rows through its GEMV
// (python/qengine/engine.py:558-573). Same packed wire format (w4_dev.cuh) and the GEMV's
// arithmetic per group (exact products of 4-bit integers and bf16 activations, fp32 sums, the
// group scale applied once); the order in which the groups of a tile are added differs from the
// GEMV's, so a row agrees with the GEMV to fp32 rounding, not bit for bit.
//
// Two kernels behind qe_w4_gemm:
//   * w4_gemm_tc_kernel (the default): tcgen05.mma, operands in shared memory, accumulator in
//     tensor memory; described in front of it, further down.
//   * w4_gemm_kernel (cfg->variant == 1): mma.sync.m16n8k16 on register fragments, described
//     next. With 8 row tiles it issues eight times the mma.sync instructions of the GEMV per
//     unit and saturates near 130 TFLOP/s, the rate of the legacy tensor path on this part: 64
//     rows cost about as much as the eight GEMV passes they replace. It is kept as the measured
//     baseline of the tensor-memory kernel and as a second implementation the tests compare.
//
// w4_gemm_kernel. With R rows every unit (16 weight rows x 128 k, 1 KB) needs R x 256 B of
// activations: at 64 rows 16 KB per KB of weights, far more than L2 can deliver to 148 SMs at
// the rate the weights arrive. The activations therefore live in shared memory, one slab of GS
// groups (GS x 128 k) of all rows at a time, double-buffered and filled by bulk copies; all warps
// of a CTA walk K slab by slab together. Work is dealt out in whole tiles (16 output rows): a CTA
// owns a contiguous range of tiles, a warp owns one tile per round -- or, when the CTA has fewer
// tiles than warps, 1/2 or 1/4 of the groups of every slab of one tile -- and keeps that tile's
// R x 16 sums in registers across all slabs. Each warp has a private ring of weight stages (its
// units of one slab, contiguous in memory) fed by bulk copies, as in the GEMV. Warps that share
// a tile add their sums through shared memory in ascending warp order after the last slab: no
// atomics, results are bit-identical run to run.
//
// Every mbarrier wait of both kernels is bounded; on expiry the warp records the error word
// (reported by qe_w4_ring_error), stops working, keeps arriving where others wait for it, and the
// CTA frees its tensor memory and leaves.
#include <cuda/atomic>

#include <algorithm>

#include "w4_dev.cuh"

namespace qb {
namespace {

using namespace w4;

struct GemmArgs {
  const uint4* qw;
  const __half* scales;
  const bf16* x;
  long ldx;
  OutDesc o;  // o.N = all activation rows (1..8 RT)
  int G, tiles, nctas;
  int kparts;      // tensor-memory kernel: parts of K a super-tile is split into
  float* ws;       // ... their fp32 sums, [super-tile][part][64][128]
  int* counters;   // ... and one arrival counter per super-tile, zero between launches
};

__device__ int g_gemm_error = 0;

constexpr int kGemmWaitLimit = 1 << 20;

// A bounded wait whose verdict is the same in every lane of the (converged) warp.
__device__ __forceinline__ bool warp_wait(uint64_t* b, uint32_t parity) {
  return __all_sync(0xffffffffu, bar_wait(b, parity, kGemmWaitLimit));
}
__device__ __forceinline__ void bar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sa(b)) : "memory");
}

__device__ __forceinline__ void mma_acc(float (&c)[4], const AFrag& f, uint32_t xa, uint32_t xb) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(f.a0), "r"(f.a1), "r"(f.a2), "r"(f.a3), "r"(xa), "r"(xb));
}

// NW warps; RT row tiles of 8 activation rows; slabs of GS groups; STAGES weight stages per warp.
template <int NW, int RT, int GS, int STAGES>
__global__ void __launch_bounds__(NW * 32, 1) w4_gemm_kernel(const __grid_constant__ GemmArgs a) {
  constexpr uint32_t kStageW = GS * 1024, kStageS = GS * 32;
  constexpr uint32_t kRing = STAGES * (kStageW + kStageS);
  constexpr uint32_t kPitch = GS * 256 + 16;  // + 16: the rows of a quarter-warp hit different banks
  constexpr uint32_t kSlab = 8 * RT * kPitch;
  static_assert(2 * kSlab >= (uint32_t)NW * RT * 128 * sizeof(float), "partial sums reuse the slab buffers");
  dep_release();
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full_w[NW][STAGES];
  __shared__ uint64_t full_x[2], empty_x[2];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, t = lane & 3;
  unsigned char* ring_w = smem + (size_t)warp * kRing;
  unsigned char* ring_s = ring_w + (size_t)STAGES * kStageW;
  unsigned char* xs = smem + (size_t)NW * kRing;  // two slabs; partial sums after the last slab

  if (tid == 0) {
    for (int b = 0; b < 2; ++b) {
      bar_init(&full_x[b], 1);
      bar_init(&empty_x[b], NW);
    }
  }
  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) bar_init(&full_w[warp][s], 1);
    bar_fence_init();
  }
  __syncthreads();

  // ---- this CTA's tiles, this warp's share of them ----
  const int G = a.G, N = a.o.N;
  const int cta = blockIdx.x;
  int T0 = 0, nt = 0;
  if (cta < a.nctas) {
    T0 = share_begin(a.tiles, a.nctas, cta);
    nt = share_begin(a.tiles, a.nctas, cta + 1) - T0;
  }
  int wpt = 1;  // warps per tile: the largest of 1, 2, 4 (<= GS) that the CTA's tiles can keep busy
  while (wpt * 2 <= GS && nt * wpt * 2 <= NW) wpt *= 2;
  const int RS = NW / wpt;              // tiles per round
  const int rounds = (nt + RS - 1) / RS;
  const int SPT = G / GS;               // slabs per tile
  const int n_it = rounds * SPT;        // slabs this CTA walks through
  const int tl = warp / wpt, sub = warp - tl * wpt;
  const int upw = GS / wpt, j0 = sub * upw;  // this warp's groups of a slab
  const int my_rounds = tl < nt ? (nt - tl + RS - 1) / RS : 0;
  const int my_it = my_rounds * SPT;    // weight stages of this warp: the first my_it slabs

  auto unit_of = [&](int q) {  // first unit of weight stage q
    const int round = q / SPT, s = q - round * SPT;
    return (T0 + round * RS + tl) * G + s * GS + j0;
  };
  auto fill_w = [&](int q, int at) {  // lane 0
    const int u = unit_of(q);
    bar_expect(&full_w[warp][at], (uint32_t)upw * (1024 + 32));
    bulk_g2s(ring_w + (size_t)at * kStageW, a.qw + (size_t)u * 64, (uint32_t)upw * 1024, &full_w[warp][at]);
    bulk_g2s(ring_s + (size_t)at * kStageS, a.scales + (size_t)u * 16, (uint32_t)upw * 32, &full_w[warp][at]);
  };
  // warp 0: request slab `it` of the activations (GS groups of every row)
  auto fill_x = [&](int it) {
    const int b = it & 1, s = it % SPT;
    if (lane == 0) bar_expect(&full_x[b], (uint32_t)N * GS * 256);
    __syncwarp();
    for (int row = lane; row < N; row += 32)
      bulk_g2s(xs + (size_t)b * kSlab + (size_t)row * kPitch, a.x + (long)row * a.ldx + (long)s * GS * 128,
               GS * 256, &full_x[b]);
  };

  // weights never depend on the producer of x: the first stages are requested before the
  // programmatic-dependency wait
  if (lane == 0)
    for (int q = 0; q < min(STAGES, my_it); ++q) fill_w(q, q);
  dep_wait();
  if (warp == 0 && n_it > 0) fill_x(0);

  // Lane (r, t) multiplies activation rows 8 rt + r; rows >= N re-read row N - 1 (their mma
  // columns are never stored), row tiles at or beyond N are skipped.
  const int rtu = (N + 7) >> 3;
  uint32_t xoff[RT];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt) xoff[rt] = (uint32_t)min(8 * rt + r, N - 1) * kPitch + 32 * t;

  float acc[RT][4];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt) acc[rt][0] = acc[rt][1] = acc[rt][2] = acc[rt][3] = 0.f;

  auto store_tile = [&](int tile, int rt, const float (&f)[4]) {
    OutDesc d = a.o;
    const size_t esz = d.out_f32 ? 4 : 2;
    d.out = static_cast<unsigned char*>(a.o.out) + (size_t)(8 * rt) * a.o.ldo * esz;
    d.N = min(8, N - 8 * rt);
    tile_out(d, tile, f, lane);
  };

  int slot = 0, phase = 0;
  bool ok = true;
#pragma unroll 1
  for (int it = 0; it < n_it && ok; ++it) {
    const int b = it & 1;
    if (warp == 0 && it + 1 < n_it) {
      // the other buffer is free once every warp has left slab it - 1
      if (it >= 1 && !warp_wait(&empty_x[b ^ 1], ((it - 1) >> 1) & 1)) {
        ok = false;
        atomicExch(&g_gemm_error, 2);
        break;
      }
      if (lane == 0) async_proxy_fence();
      fill_x(it + 1);
    }
    if (!warp_wait(&full_x[b], (it >> 1) & 1)) {
      ok = false;
      atomicExch(&g_gemm_error, 3);
      break;
    }
    if (it < my_it) {
      uint64_t* bar = &full_w[warp][slot];
      if (!warp_wait(bar, phase)) {
        ok = false;
        atomicExch(&g_gemm_error, 1);
        break;
      }
      const uint4* wp = reinterpret_cast<const uint4*>(ring_w + (size_t)slot * kStageW) + lane;
      const unsigned short* sp = reinterpret_cast<const unsigned short*>(ring_s + (size_t)slot * kStageS) + r;
      const unsigned char* xb = xs + (size_t)b * kSlab + (size_t)j0 * 256;
#pragma unroll 1
      for (int i = 0; i < upw; ++i) {
        const uint4 w0 = wp[i * 64], w1 = wp[i * 64 + 32];
        const uint32_t word[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        float c[RT][4];
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) c[rt][0] = c[rt][1] = c[rt][2] = c[rt][3] = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          // 16 bytes of x per row tile serve two words: k = 64 (q / 2) + 16 t + 8 (q % 2) .. + 7
          const AFrag f0 = unpack_word(word[2 * q]), f1 = unpack_word(word[2 * q + 1]);
          const uint32_t qo = (uint32_t)i * 256 + (q >> 1) * 128 + (q & 1) * 16;
#pragma unroll
          for (int rt = 0; rt < RT; ++rt) {
            if (rt < rtu) {
              const uint4 xv = *reinterpret_cast<const uint4*>(xb + xoff[rt] + qo);
              mma_acc(c[rt], f0, xv.x, xv.y);
              mma_acc(c[rt], f1, xv.z, xv.w);
            }
          }
        }
        const float lo = __half2float(__ushort_as_half(sp[i * 16]));
        const float hi = __half2float(__ushort_as_half(sp[i * 16 + 8]));
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
          acc[rt][0] = fmaf(lo, c[rt][0], acc[rt][0]);
          acc[rt][1] = fmaf(lo, c[rt][1], acc[rt][1]);
          acc[rt][2] = fmaf(hi, c[rt][2], acc[rt][2]);
          acc[rt][3] = fmaf(hi, c[rt][3], acc[rt][3]);
        }
      }
      __syncwarp();  // every lane has read this stage: hand its slot back to the copy engine
      if (lane == 0 && it + STAGES < my_it) {
        async_proxy_fence();
        fill_w(it + STAGES, slot);
      }
      if (++slot == STAGES) { slot = 0; phase ^= 1; }
      // last slab of a tile that this warp owns alone: store it and start the next round's tile
      if (wpt == 1 && (it + 1) % SPT == 0) {
        const int tile = T0 + (it / SPT) * RS + tl;
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
          if (rt < rtu) store_tile(tile, rt, acc[rt]);
          acc[rt][0] = acc[rt][1] = acc[rt][2] = acc[rt][3] = 0.f;
        }
      }
    }
    __syncwarp();
    if (lane == 0) bar_arrive(&empty_x[b]);  // this warp has left slab `it`
  }

  if (!ok) {
    // Give the copies that are still in flight a bounded chance to land before the CTA exits.
    __syncwarp();
    for (int s = 0; s < STAGES; ++s) bar_wait(&full_w[warp][s], 0, 1 << 10), bar_wait(&full_w[warp][s], 1, 1 << 10);
    for (int b = 0; b < 2; ++b) bar_wait(&full_x[b], 0, 1 << 10), bar_wait(&full_x[b], 1, 1 << 10);
  }
  if (wpt == 1) return;  // (uniform over the CTA) every tile was stored by its warp

  // ---- tiles shared by wpt warps (one round): partial sums through shared memory ----
  __syncthreads();  // every warp has left the last slab: its buffers are free
  float* part = reinterpret_cast<float*>(xs);  // [NW][RT][4][32]
  if (ok && sub != 0 && tl < nt) {
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int k = 0; k < 4; ++k) part[((warp * RT + rt) * 4 + k) * 32 + lane] = acc[rt][k];
  }
  __syncthreads();
  if (ok && sub == 0 && tl < nt) {
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
      if (rt < rtu) {
        for (int w2 = warp + 1; w2 < warp + wpt; ++w2)
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[rt][k] += part[((w2 * RT + rt) * 4 + k) * 32 + lane];
        store_tile(T0 + tl, rt, acc[rt]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The tensor-core path proper: tcgen05.mma with the accumulator in tensor memory.
//
// A job is one super-tile, 128 weight rows (eight 16-row tiles of the wire format) over all of K;
// the CTAs take super-tiles round-robin. One step = one group g (128 k) of a super-tile:
//   * 16 warps in two halves: warps 0..7 prepare the even steps, warps 8..15 the odd ones, one
//     tile each. Preparing = pull the tile's 1 KB unit of the step through a private ring of bulk
//     copies, unpack it to the exact bf16 integers code - 8 (w4_dev.cuh) and store it as rows of
//     the A operand [128 rows x 128 k] in the K-major 128-byte-swizzle layout the tensor core
//     reads (row pitch 128 B, 16-byte chunk index XOR row % 8; 16-byte stores, conflict-free);
//     and copy the step's activations [64 rows x 128 k] from global memory (L2) into the same
//     layout as the B operand, one own step ahead through registers;
//   * a seventeenth warp waits for the 16 arrivals of a step and issues its 8 tcgen05.mma (M 128,
//     N 64, K 16), which leave the group's exact integer dot products D_g[m, n] in one of three
//     64-column accumulators in tensor memory;
//   * every one of the 16 warps, every step, reads its 16 columns of D_{g-2} for its row
//     (tcgen05.ld), multiplies by the row's group scale in fp32 and adds to 16 registers:
//     acc[m, n] += scale[m, g] * D_g[m, n], groups in ascending order -- the arithmetic of the GEMV
//     (exact products, fp32 sums inside a group, the scale applied once per group).
// A, B and the accumulators have three stages and the halves alternate, so one half unpacks
// step z + 1 while the products of steps z and z - 1 are under way; there is no block-wide barrier
// in the loop, the warps meet only through two kinds of mbarrier: "step z may be multiplied" (one
// arrival per warp: its share of the operands is stored, if it had one, and it has read the
// products of step z - 3 out of the accumulator) and "products of step z complete"
// (tcgen05.commit). After the last group the registers hold the super-tile's [128 x 64] result:
// rounded and stored (or combined into SwiGLU) from there. A matrix with fewer super-tiles than
// half the SMs (the 5,120-row out and down projections: 40) is also split along K, up to as many
// jobs as there are SMs; the parts of a super-tile meet in a caller-provided fp32 workspace.
// ---------------------------------------------------------------------------------------------
constexpr int kTcWarps = 16, kTcThreads = (kTcWarps + 1) * 32, kTcStages = 4, kTcDepth = 3, kTcCols = 256;
constexpr int kTcScales = 8;                   // buffers of group scales (see the loop)
constexpr uint32_t kTcStageBytes = 1024 + 32;  // one unit of codes + its 16 scales
constexpr uint32_t kTcRing = kTcStages * kTcStageBytes;
constexpr uint32_t kTcA = 128 * 256, kTcB = 64 * 256;  // one stage of A / B
constexpr uint32_t kTcSmem =
    kTcDepth * (kTcA + kTcB) + kTcWarps * kTcRing + kTcScales * 128 * sizeof(float) + 1024;

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, N = 64, M = 128.
constexpr uint32_t kTcIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(da), "l"(db), "r"(kTcIdesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sa(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t u[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
        "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int k = 0; k < 16; ++k) v[k] = __uint_as_float(u[k]);
}

__global__ void __launch_bounds__(kTcThreads, 1) w4_gemm_tc_kernel(const __grid_constant__ GemmArgs a) {
  dep_release();
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t full_w[kTcWarps][kTcStages];
  __shared__ uint64_t a_full[kTcDepth];  // step z may be multiplied: one arrival per unpacking warp
  __shared__ uint64_t d_full[kTcDepth];  // its products are in tensor memory (tcgen05.commit)
  __shared__ uint32_t tmem_slot;
  __shared__ int s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, t = lane & 3;
  unsigned char* base = smem_raw + ((1024u - (sa(smem_raw) & 1023u)) & 1023u);  // swizzle atoms: 1 KB aligned
  unsigned char* Bbase = base + kTcDepth * kTcA;
  float* sc = reinterpret_cast<float*>(Bbase + kTcDepth * kTcB + (size_t)kTcWarps * kTcRing);  // [kTcScales][128]

  if (tid == 0) {
    for (int b = 0; b < kTcDepth; ++b) {
      bar_init(&a_full[b], kTcWarps);
      bar_init(&d_full[b], 1);
    }
  }
  if (lane == 0 && warp < kTcWarps) {
    for (int s = 0; s < kTcStages; ++s) bar_init(&full_w[warp][s], 1);
  }
  if (lane == 0) bar_fence_init();
  __syncwarp();
  if (warp == kTcWarps) {  // tensor memory: three accumulators of 64 columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sa(&tmem_slot)), "r"(kTcCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  // ---- this CTA's jobs: (super-tile, part of K), dealt out round-robin ----
  const int G = a.G, N = a.o.N, KP = a.kparts;
  const int J = ((a.tiles + 7) >> 3) * KP;
  const int cta = blockIdx.x, nctas = gridDim.x;
  const int nj = cta < J ? (J - cta + nctas - 1) / nctas : 0;
  struct Cur {
    int j, g, gend, tile0, jidx;
  };
  auto cur_set = [&](Cur& c, int j) {
    c.j = j;
    if (j < nj) {
      c.jidx = cta + j * nctas;
      const int st = c.jidx / KP, part = c.jidx - st * KP;
      c.g = share_begin(G, KP, part);
      c.gend = share_begin(G, KP, part + 1);
      c.tile0 = st * 8;
    } else {
      c.jidx = 0; c.g = 0; c.gend = 1 << 30; c.tile0 = 0;
    }
  };
  auto cur_next = [&](Cur& c) {
    if (++c.g == c.gend) cur_set(c, c.j + 1);
  };
  int Z = 0;  // steps
  {
    Cur c;
    for (int j = 0; j < nj; ++j) {
      cur_set(c, j);
      Z += c.gend - c.g;
    }
  }

  if (warp == kTcWarps) {
    // ---- the issuing warp: 8 products per step as soon as the step may be multiplied ----
    // One thread issues: its instruction latency is what a step waits for, so the descriptors are
    // built once and only their start-address field (low word, 16-byte units) moves in the loop.
    const uint64_t da0 = tc_desc(sa(base)), db0 = tc_desc(sa(Bbase));
    bool ok = true;
    int s3 = 0, ph = 0;
#pragma unroll 1
    for (int z = 0; z < Z && ok; ++z) {
      if (!warp_wait(&a_full[s3], ph)) {
        ok = false;
        atomicExch(&g_gemm_error, 2);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint64_t da = da0 + (uint64_t)(s3 * (kTcA >> 4)), db = db0 + (uint64_t)(s3 * (kTcB >> 4));
        const uint32_t d = tmem + s3 * 64;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma(d, da + (uint64_t)(c2 * (16384 >> 4) + kk * 2), db + (uint64_t)(c2 * (8192 >> 4) + kk * 2),
                   (c2 | kk) ? 1u : 0u);
        tc_commit(&d_full[s3]);
      }
      __syncwarp();
      if (++s3 == kTcDepth) { s3 = 0; ph ^= 1; }
    }
  } else {
    // ---- the 16 unpacking warps ----
    unsigned char* ring = Bbase + kTcDepth * kTcB + (size_t)warp * kTcRing;
    const int par = warp >> 3, ti = warp & 7;  // prepares the steps of this parity; tile of the super-tile
    // the unit of this warp's tile in a step; false beyond the matrix (only the matrix's last
    // super-tile can lack tiles, and its jobs are the last ones of their CTAs)
    auto unit_of = [&](const Cur& c, size_t& u) {
      u = (size_t)(c.tile0 + ti) * G + c.g;
      return c.j < nj && c.tile0 + ti < a.tiles;
    };
    auto fill_w = [&](size_t u, int at) {  // lane 0
      unsigned char* dst = ring + (size_t)at * kTcStageBytes;
      bar_expect(&full_w[warp][at], kTcStageBytes);
      bulk_g2s(dst, reinterpret_cast<const unsigned char*>(a.qw) + u * 1024, 1024, &full_w[warp][at]);
      bulk_g2s(dst + 1024, a.scales + u * 16, 32, &full_w[warp][at]);
    };
    Cur cz, cr;  // the current step; the next own step to request from HBM
    cur_set(cz, 0);
    cur_set(cr, 0);
    if (par) cur_next(cr);
    for (int q = 0; q < kTcStages; ++q) {
      size_t u;
      if (!unit_of(cr, u)) break;
      if (lane == 0) fill_w(u, q);
      cur_next(cr);
      cur_next(cr);
    }
    dep_wait();

    // this thread's four 16-byte pieces of the activations of a group (64 rows x 16 pieces,
    // dealt out over the 256 threads of a half): rows n0 + 16 i, piece j16
    const int t256 = tid & 255, n0 = t256 >> 4, j16 = t256 & 15;
    const uint4* xsrc = reinterpret_cast<const uint4*>(a.x + (long)n0 * a.ldx) + j16;
    const long xstep = 2 * a.ldx;  // 16 rows on, in 16-byte units
    const uint32_t boff = (j16 >> 3) * 8192 + n0 * 128 + (((j16 & 7) ^ (n0 & 7)) << 4);  // + 2048 i
    uint4 xr[4];
    auto load_x = [&](int g) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        xr[i] = n0 + 16 * i < N ? xsrc[(long)i * xstep + g * 16] : make_uint4(0u, 0u, 0u, 0u);
    };
    {
      Cur c = cz;
      if (par) cur_next(c);
      if (c.j < nj) load_x(c.g);
    }

    const int m = 32 * (warp & 3) + lane;  // this thread's row of the super-tile (a tensor-memory lane)
    const int col0 = 16 * (warp >> 2);     // its 16 activation rows
    const uint32_t t_lane = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + col0;
    float acc[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) acc[k] = 0.f;

    bool ok = true;
    // acc += scale[m, group of step z] * D(z)
    auto drain = [&](int z) {
      const int s3 = z % kTcDepth, ph = (z / kTcDepth) & 1;
      if (ok && !warp_wait(&d_full[s3], ph)) {
        ok = false;
        atomicExch(&g_gemm_error, 4);
      }
      if (!ok) return;
      tc_fence_after();
      float v[16];
      tc_ld16(t_lane + s3 * 64, v);
      const float sm = sc[(z & (kTcScales - 1)) * 128 + m];
#pragma unroll
      for (int k = 0; k < 16; ++k) acc[k] = fmaf(sm, v[k], acc[k]);
    };
    auto store_out = [&](int tile0) {  // the finished sums of a super-tile, from registers
      const int tile = tile0 + (m >> 4), rr = m & 15;
      if (a.o.epi == QE_EPI_SWIGLU) {
        bf16* o = static_cast<bf16*>(a.o.out);
        const int jrow = tile * 8 + rr;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const float up = __shfl_down_sync(0xffffffffu, acc[k], 8);
          const int n = col0 + k;
          if (ok && rr < 8 && jrow < a.o.M && n < N) o[(long)n * a.o.ldo + jrow] = tobf16(silu_fast(acc[k]) * up);
        }
      } else {
        const int mrow = tile * 16 + rr;
        if (ok && mrow < a.o.M) {
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const int n = col0 + k;
            if (n >= N) continue;
            if (a.o.out_f32) static_cast<float*>(a.o.out)[(long)n * a.o.ldo + mrow] = acc[k];
            else static_cast<bf16*>(a.o.out)[(long)n * a.o.ldo + mrow] = tobf16(acc[k]);
          }
        }
      }
    };

    // Three stages of A, B and accumulator; a warp reads the products of step z two steps later.
    // Before it arrives for step z (and before it writes stage z % 3) it has read the products of
    // step z - 3, so they are complete, the stage is free, and the issuing warp may overwrite that
    // accumulator once all 16 have arrived. A writer of the scales of step z + L has seen the
    // products of step z + L - 3, issued after everybody arrived for that step; a reader still
    // busy with step z has arrived for z + 2 at most, so L <= 5: eight buffers of scales.
    int slot = 0, phase = 0, since = 0, s3 = 0;
#pragma unroll 1
    for (int z = 0; z < Z; ++z) {
      if ((z & 1) == par) {
        unsigned char* As = base + (size_t)s3 * kTcA;
        unsigned char* Bs = Bbase + (size_t)s3 * kTcB;
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(Bs + boff + 2048 * i) = xr[i];
        size_t u;
        if (unit_of(cz, u)) {
          if (ok && !warp_wait(&full_w[warp][slot], phase)) {
            ok = false;
            atomicExch(&g_gemm_error, 1);
          }
          if (ok) {
            const unsigned char* st = ring + (size_t)slot * kTcStageBytes;
            const uint4 w0 = reinterpret_cast<const uint4*>(st)[lane], w1 = reinterpret_cast<const uint4*>(st)[32 + lane];
            if (lane < 16)
              sc[(z & (kTcScales - 1)) * 128 + 16 * ti + lane] = __half2float(reinterpret_cast<const __half*>(st + 1024)[lane]);
            unsigned char* rowp = As + (16 * ti + r) * 128;  // row r of the tile; row r + 8 is 1 KB on
            const uint32_t c0 = (uint32_t)((2 * t) ^ r) << 4, c1 = (uint32_t)((2 * t + 1) ^ r) << 4;
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {  // the two 64-k chunks of the unit
              const uint4 wv = ch ? w1 : w0;
              const AFrag f0 = unpack_word(wv.x), f1 = unpack_word(wv.y), f2 = unpack_word(wv.z), f3 = unpack_word(wv.w);
              unsigned char* q = rowp + ch * 16384;
              *reinterpret_cast<uint4*>(q + c0) = make_uint4(f0.a0, f0.a2, f1.a0, f1.a2);
              *reinterpret_cast<uint4*>(q + c1) = make_uint4(f2.a0, f2.a2, f3.a0, f3.a2);
              *reinterpret_cast<uint4*>(q + 1024 + c0) = make_uint4(f0.a1, f0.a3, f1.a1, f1.a3);
              *reinterpret_cast<uint4*>(q + 1024 + c1) = make_uint4(f2.a1, f2.a3, f3.a1, f3.a3);
            }
          }
          __syncwarp();  // every lane has read this stage: hand its slot back to the copy engine
          size_t un;
          if (unit_of(cr, un)) {
            if (lane == 0 && ok) fill_w(un, slot);
            cur_next(cr);
            cur_next(cr);
          }
          if (++slot == kTcStages) { slot = 0; phase ^= 1; }
        }
        async_proxy_fence();  // the stores above become visible to the tensor core's reads
      }
      tc_fence_before();  // this thread's tensor-memory loads are ordered before the arrival
      __syncwarp();
      if (lane == 0) bar_arrive(&a_full[s3]);
      if (++s3 == kTcDepth) s3 = 0;
      if ((z & 1) == par) {
        // The activations of the next own step: requested after the proxy fence above (which
        // would wait for them), two steps ahead of their use.
        Cur c = cz;
        cur_next(c);
        cur_next(c);
        if (c.j < nj) load_x(c.g);
      }
      if (since >= 2) drain(z - 2);
      if (cz.g + 1 == cz.gend) {
        // last group of the job: two or three more drains complete its sums
        if (since >= 1) drain(z - 1);
        drain(z);
        since = 0;
        if (KP == 1) {
          store_out(cz.tile0);
        } else {
          // A super-tile split along K: every part leaves its fp32 sums in the workspace; the
          // CTA that delivers the last part adds them in ascending order of the parts (so the
          // result does not depend on who was last) and stores the tile.
          float* wsj = a.ws + (size_t)cz.jidx * (64 * 128);
#pragma unroll
          for (int k = 0; k < 16; ++k) __stcg(wsj + (col0 + k) * 128 + m, acc[k]);
          __threadfence();
          asm volatile("bar.sync 1, %0;" ::"n"(kTcWarps * 32) : "memory");
          const int st = cz.tile0 >> 3;
          if (tid == 0) {
            cuda::atomic_ref<int, cuda::thread_scope_device> arrivals(a.counters[st]);
            const int last = arrivals.fetch_add(1, cuda::memory_order_acq_rel) == KP - 1;
            if (last) a.counters[st] = 0;
            s_last = last;
          }
          asm volatile("bar.sync 1, %0;" ::"n"(kTcWarps * 32) : "memory");
          const int last = s_last;
          asm volatile("bar.sync 1, %0;" ::"n"(kTcWarps * 32) : "memory");  // s_last may be rewritten
          if (last) {
            __threadfence();
#pragma unroll
            for (int k = 0; k < 16; ++k) acc[k] = 0.f;
            for (int p2 = 0; p2 < KP; ++p2) {
              const float* wp = a.ws + (size_t)(st * KP + p2) * (64 * 128);
#pragma unroll
              for (int k = 0; k < 16; ++k) acc[k] += __ldcg(wp + (col0 + k) * 128 + m);
            }
            store_out(cz.tile0);
          }
        }
#pragma unroll
        for (int k = 0; k < 16; ++k) acc[k] = 0.f;
      } else {
        ++since;
      }
      cur_next(cz);
    }
    if (!ok) {  // give the copies that are still in flight a bounded chance to land
      __syncwarp();
      for (int s = 0; s < kTcStages; ++s) bar_wait(&full_w[warp][s], 0, 1 << 10), bar_wait(&full_w[warp][s], 1, 1 << 10);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kTcWarps) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTcCols) : "memory");
  }
}

using GemmFn = void (*)(const GemmArgs);

struct GemmGeom {
  GemmFn fn;
  int nw, rt, gs, stages;
  size_t smem() const {
    return (size_t)nw * stages * gs * (1024 + 32) + 2 * (size_t)8 * rt * (gs * 256 + 16);
  }
};
template <int NW, int RT, int GS, int STAGES>
constexpr GemmGeom gemm_geom() {
  return GemmGeom{w4_gemm_kernel<NW, RT, GS, STAGES>, NW, RT, GS, STAGES};
}
// up to 32 rows: slabs of 4 groups; up to 64 rows (or K / 128 not a multiple of 4): slabs of 2
const GemmGeom kGemmGeoms[] = {gemm_geom<16, 4, 4, 2>(), gemm_geom<16, 8, 2, 4>()};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Parts of K a super-tile is split into (tensor-memory kernel): 1 unless the matrix has fewer
// super-tiles than half the SMs; then as many as keep the job count within the SMs, at least 8
// groups each. Shape (and device) only, never the row count.
int gemm_kparts(int tiles, int G, int epilogue) {
  const int ST = (tiles + 7) / 8, sms = qe_sm_count();
  if (epilogue != QE_EPI_NONE || ST * 2 > sms) return 1;
  return std::max(1, std::min({sms / ST, G / 8, 16}));
}

// The opt-in limit of dynamic shared memory is a per-device, per-function setting: raised once.
cudaError_t allow_smem(const GemmGeom& g, int which) {
  static bool done[2][64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (done[which][dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(g.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem());
  if (e == cudaSuccess) done[which][dev] = true;
  return e;
}

}  // namespace

// Error word of the bounded waits above, for qe_w4_ring_error / qe_w4_clear_error (w4_gemv.cu).
int gemm_error_read() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}
int gemm_error_clear() {
  const int z = 0;
  return (int)cudaMemcpyToSymbol(g_gemm_error, &z, sizeof(int));
}

}  // namespace qb

using namespace qb;

extern "C" int qe_w4_plan_gemm(const qe_w4_params* p, const qe_w4_cfg* cfg, qe_w4_plan* plan) {
  if (!p || !cfg || !plan || p->Mp <= 0 || p->Kp <= 0 || p->Mp % 16 || p->Kp % 128) return QE_ERR_ARG;
  const int tiles = p->Mp / 16, ST = (tiles + 7) / 8;
  const int kp = cfg->variant == 1 ? 1 : gemm_kparts(tiles, p->Kp / 128, p->epilogue);
  plan->mode = cfg->variant == 1 ? 1 : 0;
  plan->grid_x = std::min(qe_sm_count(), cfg->variant == 1 ? tiles : ST * kp);
  plan->grid_y = 1;
  plan->threads = cfg->variant == 1 ? 512 : kTcThreads;
  plan->ws_floats = kp > 1 ? (long)ST * kp * 64 * 128 : 0;
  plan->counters = kp > 1 ? ST : 0;
  return 0;
}

extern "C" int qe_w4_gemm(const qe_w4_params* p, const qe_w4_cfg* cfg, void* stream) {
  if (!p || !cfg) return QE_ERR_ARG;
  if (p->N < 1 || p->N > QE_MAX_GEMM_ROWS || p->Mp % 16 || p->Kp % 128 || p->Mp <= 0 || p->Kp <= 0) return QE_ERR_ARG;
  if (p->K != p->Kp || p->M <= 0 || p->x_f16 || !p->x || !p->out) return QE_ERR_ARG;
  if (p->epilogue == QE_EPI_SWIGLU ? p->M > p->Mp / 2 : p->M > p->Mp) return QE_ERR_ARG;
  if (p->epilogue != QE_EPI_NONE && p->epilogue != QE_EPI_SWIGLU) return QE_ERR_ARG;
  if ((long)(p->Mp / 16) * (p->Kp / 128) >= (1L << 30)) return QE_ERR_ARG;
  // bulk copies: 16-byte aligned sources, row strides that keep them so
  if (!aligned16(p->qw) || !aligned16(p->scales) || !aligned16(p->x) || (p->ldx & 7)) return QE_ERR_ARG;
  const int G = p->Kp / 128;
  if (cfg->variant != 1) {  // tensor memory path (the default); variant 1: the mma.sync kernels below
    static bool allowed[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!allowed[dev]) {
      e = cudaFuncSetAttribute(w4_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem);
      if (e != cudaSuccess) return (int)e;
      allowed[dev] = true;
    }
    GemmArgs a{};
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
    a.G = G;
    a.tiles = p->Mp / 16;
    a.kparts = gemm_kparts(a.tiles, G, p->epilogue);
    if (a.kparts > 1 && (!p->ws || !p->counters)) a.kparts = 1;  // no scratch: whole K per job
    a.ws = p->ws;
    a.counters = p->counters;
    a.nctas = std::min(qe_sm_count(), ((a.tiles + 7) / 8) * a.kparts);
    const bool pdl = cfg->pdl && pdl_launch_enabled() && pdl_trigger_enabled();
    return (int)launch(w4_gemm_tc_kernel, dim3(a.nctas), dim3(kTcThreads), kTcSmem, (cudaStream_t)stream, pdl, a);
  }
  int which;
  if (p->N <= 32 && G % 4 == 0) which = 0;
  else if (G % 2 == 0) which = 1;
  else return QE_ERR_ARG;
  const GemmGeom& g = kGemmGeoms[which];
  cudaError_t e = allow_smem(g, which);
  if (e != cudaSuccess) return (int)e;
  GemmArgs a{};
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
  a.G = G;
  a.tiles = p->Mp / 16;
  a.nctas = std::min(qe_sm_count(), a.tiles);
  const bool pdl = cfg->pdl && pdl_launch_enabled() && pdl_trigger_enabled();
  return (int)launch(g.fn, dim3(a.nctas), dim3(g.nw * 32), g.smem(), (cudaStream_t)stream, pdl, a);
}
