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
//   * one CTA per SM, NW warps; the unit stream is cut into one contiguous range per warp (all
//     warps of all CTAs, equal shares), so every warp reads one contiguous slab of HBM;
//   * each warp owns a private ring in shared memory that its lane 0 keeps full with bulk copies
//     (cp.async.bulk global -> shared, completion on an mbarrier): STAGES x PERW units in flight
//     per warp, ~130 KB per SM, issued before the programmatic-dependency wait because weights
//     never depend on the producer of x;
//   * operands of unit i + 1 (2 LDS.128 of codes, 2 scales, 4 x 16 B of x) are fetched into
//     registers while unit i is unpacked and multiplied (mma.sync.m16n8k16, two independent
//     accumulator chains): the loop body is straight-line code without a wait in the common case;
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
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <set>
#include <string>
#include <utility>
#include <vector>

#include "w4_dev.cuh"

namespace qb {
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
  int K, G, total, nworkers;
  int xvec;        // x rows are 16-byte aligned with ldx % 8 == 0
  // fused residual + RMSNorm prologue
  const bf16* h_in;
  const int* tok;  // optional: row r of h_in is table row tok[r] (h_in = embedding table)
  int vocab;
  const bf16* delta;
  const bf16* norm_w;
  bf16* h_out;
  bf16* xn_out;
  long ldh, ldd, ldho, ldxo;
  float eps;
  // optional L2 prefetch of memory a later kernel will stream
  const unsigned char* pf;
  unsigned long long pf_bytes;
};

__device__ int g_w4_error = 0;

constexpr int kWaitLimit = 1 << 20;

template <int NW, int PERW, int STAGES, bool PRO>
__global__ void __launch_bounds__(NW * 32, 1) w4_gemv_kernel(const GemvArgs a) {
  constexpr uint32_t kStageW = PERW * 1024, kStageS = PERW * 32;
  constexpr uint32_t kRing = STAGES * (kStageW + kStageS);
  constexpr int NT = NW * 32;
  dep_release();
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[NW][STAGES];
  __shared__ int s_rb[NW + 1];
  __shared__ float s_red[QE_MAX_ROWS][NW];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, t = lane & 3;
  const int G = a.G, total = a.total, nwk = a.nworkers;
  unsigned char* ring_w = smem + (size_t)warp * kRing;
  unsigned char* ring_s = ring_w + (size_t)STAGES * kStageW;
  float* part = reinterpret_cast<float*>(smem + (size_t)NW * kRing);  // [NW][2][128]
  unsigned char* x_s = smem + (size_t)NW * kRing + (size_t)NW * 2 * 128 * sizeof(float);

  // ---- ranges: worker v of nwk owns units [share_begin(v), share_begin(v + 1)) ----
  const int w_first = blockIdx.x * NW;
  const int worker = w_first + warp;
  const int u0 = share_begin(total, nwk, min(worker, nwk));
  const int u1 = share_begin(total, nwk, min(worker + 1, nwk));
  if (lane == 0) {
    s_rb[warp] = u0;
    if (warp == NW - 1) s_rb[NW] = u1;
    for (int s = 0; s < STAGES; ++s) bar_init(&full[warp][s], 1);
    bar_fence_init();
  }
  __syncwarp();
  const int n_units = u1 - u0;
  const int nstage = (n_units + PERW - 1) / PERW;

  auto refill = [&](int st) {  // lane 0 only: stage st of this warp's range into its ring slot
    const int slot = st % STAGES;
    const int ub = u0 + st * PERW, cnt = min(PERW, u1 - ub);
    bar_expect(&full[warp][slot], (uint32_t)cnt * (1024 + 32));
    bulk_g2s(ring_w + (size_t)slot * kStageW, a.qw + (size_t)ub * 64, (uint32_t)cnt * 1024, &full[warp][slot]);
    bulk_g2s(ring_s + (size_t)slot * kStageS, a.scales + (size_t)ub * 16, (uint32_t)cnt * 32, &full[warp][slot]);
  };
  if (lane == 0) {
    for (int st = 0; st < min(STAGES, nstage); ++st) refill(st);  // weights never depend on x
    if (a.pf_bytes) {  // this warp's slice of the hinted range, 16 KB per request
      const unsigned long long nslices = (unsigned long long)gridDim.x * NW;
      const unsigned long long per = ((a.pf_bytes + nslices - 1) / nslices + 15) & ~15ull;
      unsigned long long b = per * (unsigned long long)(blockIdx.x * NW + warp);
      const unsigned long long e = min(a.pf_bytes & ~15ull, b + per);
      for (; b < e; b += 16384) l2_prefetch(a.pf + b, (uint32_t)min(16384ull, e - b));
    }
  }
  __syncthreads();  // s_rb visible to everyone
  dep_wait();

  // ---- prologue: x = RMSNorm1p(h_in + delta) into shared memory, one copy per CTA ----
  const int xrow = min(r, a.o.N - 1);  // rows >= N feed mma columns that are never stored
  const long pitch = (long)a.K * 2 + 16;  // + 16 B: rows of one quarter-warp hit different banks
  if constexpr (PRO) {
    const int npk = a.K >> 3;
    float ss[QE_MAX_ROWS];
#pragma unroll
    for (int rr = 0; rr < QE_MAX_ROWS; ++rr) {
      ss[rr] = 0.f;
      if (rr < a.o.N) {
        const bf16* hrow = a.h_in + (long)rr * a.ldh;
        bool zero = false;
        if (a.tok) {
          const int id = a.tok[rr];
          zero = id < 0 || id >= a.vocab;
          hrow = a.h_in + (size_t)(zero ? 0 : id) * a.K;
        }
        uint4* xs = reinterpret_cast<uint4*>(x_s + rr * pitch);
        for (int p = tid; p < npk; p += NT) {
          float v[8];
          uint4 raw = zero ? make_uint4(0u, 0u, 0u, 0u) : reinterpret_cast<const uint4*>(hrow)[p];
          widen8(raw, v);
          if (a.delta) {
            float d[8];
            widen8(reinterpret_cast<const uint4*>(a.delta + (long)rr * a.ldd)[p], d);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = rnd(v[e] + d[e]);
            raw = narrow8(v);
          }
          xs[p] = raw;
          if (blockIdx.x == 0 && a.h_out) reinterpret_cast<uint4*>(a.h_out + (long)rr * a.ldho)[p] = raw;
#pragma unroll
          for (int e = 0; e < 8; ++e) ss[rr] = fmaf(v[e], v[e], ss[rr]);
        }
        ss[rr] = warp_allsum(ss[rr]);
        if (lane == 0) s_red[rr][warp] = ss[rr];
      }
    }
    __syncthreads();
#pragma unroll
    for (int rr = 0; rr < QE_MAX_ROWS; ++rr) {
      if (rr < a.o.N) {
        float tot = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < NW; ++w2) tot += s_red[rr][w2];
        const float inv = rsqrtf(tot / (float)a.K + a.eps);
        uint4* xs = reinterpret_cast<uint4*>(x_s + rr * pitch);
        for (int p = tid; p < npk; p += NT) {  // same thread -> packet map as above
          float v[8], g[8], y[8];
          widen8(xs[p], v);
          widen8(reinterpret_cast<const uint4*>(a.norm_w)[p], g);
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] = v[e] * inv * (1.0f + g[e]);
          const uint4 q = narrow8(y);
          xs[p] = q;
          if (blockIdx.x == 0 && a.xn_out) reinterpret_cast<uint4*>(a.xn_out + (long)rr * a.ldxo)[p] = q;
        }
      }
    }
    __syncthreads();
  }

  // ---- x fragment of group gg: 16 consecutive k per 64-k chunk for activation row `xrow` ----
  const bool tail_k = (a.K & 127) != 0;  // the last group reads past K unless guarded
  auto load_x = [&](UnitOps& o, int gg) {
    if constexpr (PRO) {
      const uint4* xp = reinterpret_cast<const uint4*>(x_s + xrow * pitch + (size_t)gg * 256 + 32 * t);
      o.x0 = xp[0]; o.x1 = xp[1]; o.x2 = xp[8]; o.x3 = xp[9];
    } else {
      const bf16* row = a.x + (long)xrow * a.ldx;
      if (a.xvec && !(tail_k && gg == G - 1)) {
        const uint4* xp = reinterpret_cast<const uint4*>(row + (size_t)gg * 128 + 16 * t);  // coherent loads
        o.x0 = xp[0]; o.x1 = xp[1]; o.x2 = xp[8]; o.x3 = xp[9];
      } else {  // misaligned rows or the ragged end of K: element loads, zeros beyond K
        const unsigned short* xs = reinterpret_cast<const unsigned short*>(row);
        uint32_t v[16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int k0 = gg * 128 + 64 * h + 16 * t;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int k = k0 + 2 * e;
            const uint32_t lo = k < a.K ? xs[k] : 0u, hi = k + 1 < a.K ? xs[k + 1] : 0u;
            v[h * 8 + e] = lo | (hi << 16);
          }
        }
        o.x0 = make_uint4(v[0], v[1], v[2], v[3]);   o.x1 = make_uint4(v[4], v[5], v[6], v[7]);
        o.x2 = make_uint4(v[8], v[9], v[10], v[11]); o.x3 = make_uint4(v[12], v[13], v[14], v[15]);
      }
    }
  };

  // ---- the stream: load cursor runs one unit ahead of the compute cursor ----
  bool ok = true;
  int l_slot = 0, l_phase = 0, l_j = 0;  // ring slot / phase / index of the next unit to load
  int tile = u0 / G;
  int g = u0 - tile * G;                 // group of the unit being computed
  int l_g = g;                           // group of the next unit to load
  int seg_gb = g;                        // first group of the segment in `acc`
  int c_j = 0, c_st = 0;                 // index in stage / stage of the unit being computed
  float acc[4] = {0.f, 0.f, 0.f, 0.f};

  auto load_next = [&](UnitOps& o) {
    if (l_j == 0 && !bar_wait(&full[warp][l_slot], l_phase, kWaitLimit)) {
      ok = false;
      atomicExch(&g_w4_error, 1);
      return;
    }
    const uint4* wp = reinterpret_cast<const uint4*>(ring_w + (size_t)l_slot * kStageW + (size_t)l_j * 1024) + lane;
    const unsigned short* sp =
        reinterpret_cast<const unsigned short*>(ring_s + (size_t)l_slot * kStageS + (size_t)l_j * 32) + r;
    o.w0 = wp[0];
    o.w1 = wp[32];
    o.s_lo = sp[0];
    o.s_hi = sp[8];
    load_x(o, l_g);
    if (++l_g == G) l_g = 0;
    if (++l_j == PERW) {
      l_j = 0;
      if (++l_slot == STAGES) { l_slot = 0; l_phase ^= 1; }
    }
  };

  auto step = [&](const UnitOps& cur, UnitOps& nxt, int i) {
    if (i + 1 < n_units) load_next(nxt);
    unit_fma(acc, cur);
    ++g;
    const bool last = i == n_units - 1;
    if (g == G || last) {
      if (seg_gb == 0 && g == G) {
        tile_out(a.o, tile, acc, lane);
      } else {  // cut tile: slot 0 if this range starts inside the tile, slot 1 if it holds its head
        float* p = part + (warp * 2 + (seg_gb != 0 ? 0 : 1)) * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) p[c * 32 + lane] = acc[c];
      }
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      if (g == G) { g = 0; ++tile; }
      seg_gb = g;
    }
    if (++c_j == PERW || last) {  // this stage is consumed: hand its slot back to the copy engine
      __syncwarp();
      if (lane == 0 && c_st + STAGES < nstage) {
        async_proxy_fence();
        refill(c_st + STAGES);
      }
      c_j = 0;
      ++c_st;
    }
  };

  {
    UnitOps A, B;
    if (n_units > 0) load_next(A);
    for (int i = 0; i < n_units && ok; i += 2) {
      step(A, B, i);
      if (i + 1 < n_units && ok) step(B, A, i + 1);
    }
    if (!ok) {
      // Give the copies that are still in flight a bounded chance to land before the CTA exits.
      __syncwarp();
      for (int s = 0; s < STAGES; ++s) bar_wait(&full[warp][s], 0, 1 << 10), bar_wait(&full[warp][s], 1, 1 << 10);
    }
  }
  __syncthreads();  // every partial tile of this CTA is in shared memory

  // ---- cut tiles: combined by the warp holding the head, ascending warp order ----
  const int cta_b = s_rb[0], cta_e = s_rb[NW];
  const int my_cta = blockIdx.x;
  auto publish = [&](int T, const float (&f)[4], int units, int slot) {
    // one partial per CTA through global memory; whoever completes the tile adds them all
    float* gm = a.ws + ((size_t)my_cta * 2 + slot) * 128;
#pragma unroll
    for (int c = 0; c < 4; ++c) __stcg(gm + c * 32 + lane, f[c]);
    __threadfence();
    __syncwarp();
    int done = 0;
    if (lane == 0) done = atomicAdd(a.counters + T, units) + units == G;
    done = __shfl_sync(0xffffffffu, done, 0);
    if (!done) return;
    __threadfence();
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const int c_lo = share_owner(total, nwk, T * G) / NW, c_hi = share_owner(total, nwk, T * G + G - 1) / NW;
#pragma unroll 1
    for (int cc = c_lo; cc <= c_hi; ++cc) {
      const int cb = share_begin(total, nwk, min(cc * NW, nwk));
      const float* p = a.ws + ((size_t)cc * 2 + (cb > T * G ? 0 : 1)) * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) s[c] += __ldcg(p + c * 32 + lane);
    }
    tile_out(a.o, T, s, lane);
    if (lane == 0) a.counters[T] = 0;
  };

  if (ok && n_units > 0 && (u1 % G) != 0) {
    const int T = (u1 - 1) / G;
    if (T * G >= u0) {  // the head of tile T is in this warp's slot 1
      const int tend = T * G + G;
      float f[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) f[c] = part[(warp * 2 + 1) * 128 + c * 32 + lane];
      for (int w2 = warp + 1; w2 < NW && s_rb[w2] < tend; ++w2) {
#pragma unroll
        for (int c = 0; c < 4; ++c) f[c] += part[(w2 * 2) * 128 + c * 32 + lane];
      }
      if (tend <= cta_e) tile_out(a.o, T, f, lane);
      else publish(T, f, cta_e - T * G, 1);
    }
  }
  if (warp == 0 && ok && cta_e > cta_b && (cta_b % G) != 0) {  // tile that began in an earlier CTA
    const int T = cta_b / G, tend = T * G + G;
    float f[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) f[c] = part[c * 32 + lane];
    for (int w2 = 1; w2 < NW && s_rb[w2] < tend; ++w2) {
#pragma unroll
      for (int c = 0; c < 4; ++c) f[c] += part[(w2 * 2) * 128 + c * 32 + lane];
    }
    publish(T, f, min(tend, cta_e) - cta_b, 0);
  }
}

// ---- host side -----------------------------------------------------------------------------------
using KernelFn = void (*)(const GemvArgs);

struct Geometry {
  KernelFn fn[2];  // [prologue]
  int nw, perw, stages;
  size_t ring_bytes() const { return (size_t)nw * stages * perw * (1024 + 32) + (size_t)nw * 2 * 128 * sizeof(float); }
};
template <int NW, int PERW, int STAGES>
constexpr Geometry geometry() {
  return Geometry{{w4_gemv_kernel<NW, PERW, STAGES, false>, w4_gemv_kernel<NW, PERW, STAGES, true>}, NW, PERW, STAGES};
}
// Selected by the reference's launch options: `warps` picks the CTA size (4 / 8 -> 8 warps,
// 0 / 16 -> 16 warps, variant 1 -> 24 warps), `unroll` the ring shape (0 / 4 -> 2 stages of 4
// units, 1 / 2 -> 3 stages of 2 units).
const Geometry kGeoms[] = {geometry<16, 4, 2>(), geometry<16, 2, 3>(), geometry<8, 4, 2>(), geometry<8, 2, 3>(),
                           geometry<24, 2, 3>()};

const Geometry& pick_geometry(const qe_w4_cfg& c) {
  const bool fine = c.unroll == 1 || c.unroll == 2;
  if (c.variant == 1) return kGeoms[4];
  if (c.warps == 4 || c.warps == 8) return kGeoms[fine ? 3 : 2];
  return kGeoms[fine ? 1 : 0];
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is per device: remember where it has been set.
cudaError_t allow_smem(KernelFn fn, size_t bytes) {
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lk(mu);
  if (done.count({(const void*)fn, dev})) return cudaSuccess;
  e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e == cudaSuccess) done.insert({(const void*)fn, dev});
  (void)bytes;
  return e;
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
  int nworkers;
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
  const long want = (units + min_units - 1) / min_units;
  const long workers = std::max<long>(1, std::min<long>({ctas_max * r.geom->nw, want, units}));
  r.nworkers = (int)workers;
  r.plan.mode = 4;
  r.plan.grid_x = (int)((workers + r.geom->nw - 1) / r.geom->nw);
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

int launch_gemv(const qe_w4_params* p, const qe_w4_norm* nrm, const qe_w4_cfg* cfg, cudaStream_t stream) {
  int rc = check_params(p, cfg);
  if (rc) return rc;
  const Resolved r = resolve(*p, *cfg);
  GemvArgs a{};
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
  a.nworkers = r.nworkers;
  a.xvec = ((p->ldx & 7) == 0 && aligned16(p->x)) ? 1 : 0;
  size_t smem = r.geom->ring_bytes();
  bool pro = false;
  if (nrm && nrm->h_in) {
    // the prologue holds N rows of x in shared memory and reads / writes 16-byte packets
    if (p->K != p->Kp || !nrm->norm_w || !aligned16(nrm->h_in) || !aligned16(nrm->norm_w) || (nrm->ldh & 7) ||
        (nrm->delta && (!aligned16(nrm->delta) || (nrm->ldd & 7))) ||
        (nrm->h_out && (!aligned16(nrm->h_out) || (nrm->ldho & 7) || nrm->h_out == nrm->h_in)) ||
        (nrm->xn_out && (!aligned16(nrm->xn_out) || (nrm->ldxo & 7))) || (nrm->tok && nrm->vocab < 1))
      return QE_ERR_ARG;
    smem += (size_t)p->N * ((size_t)p->K * 2 + 16);
    if (smem > 227 * 1024) return QE_ERR_ARG;  // caller runs qe_rmsnorm1p + qe_w4_gemv instead
    pro = true;
    a.h_in = reinterpret_cast<const bf16*>(nrm->h_in);
    a.tok = nrm->tok;
    a.vocab = nrm->vocab;
    a.delta = reinterpret_cast<const bf16*>(nrm->delta);
    a.norm_w = reinterpret_cast<const bf16*>(nrm->norm_w);
    a.h_out = reinterpret_cast<bf16*>(nrm->h_out);
    a.xn_out = reinterpret_cast<bf16*>(nrm->xn_out);
    a.ldh = nrm->ldh; a.ldd = nrm->ldd; a.ldho = nrm->ldho; a.ldxo = nrm->ldxo;
    a.eps = nrm->eps;
  } else if (!p->x) {
    return QE_ERR_ARG;
  }
  if (nrm && nrm->prefetch && nrm->prefetch_bytes) {
    a.pf = reinterpret_cast<const unsigned char*>(nrm->prefetch);
    a.pf_bytes = nrm->prefetch_bytes;
  }
  KernelFn fn = r.geom->fn[pro ? 1 : 0];
  cudaError_t e = allow_smem(fn, smem);
  if (e != cudaSuccess) return (int)e;
  const bool pdl = cfg->pdl && pdl_launch_enabled() && pdl_trigger_enabled();
  return (int)launch(fn, dim3(r.plan.grid_x, 1, 1), dim3(r.plan.threads), smem, stream, pdl, a);
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
  return v;
}

extern "C" int qe_w4_clear_error(void) {
  const int z = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  return (int)cudaMemcpyToSymbol(g_w4_error, &z, sizeof(int));
}

extern "C" int qe_w4_gemv(const qe_w4_params* p, const qe_w4_cfg* cfg, void* stream) {
  return launch_gemv(p, nullptr, cfg, (cudaStream_t)stream);
}

extern "C" int qe_w4_gemv_ex(const qe_w4_params* p, const qe_w4_norm* nrm, const qe_w4_cfg* cfg, void* stream) {
  return launch_gemv(p, nrm, cfg, (cudaStream_t)stream);
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
