// Gated delta-rule (Gated DeltaNet) decode / verify step for n = 1..8 rows with per-position
// checkpoints for rollback. Boundary: replaces launch_gdn_step_n of the reference
// (csrc/ops.h:20-24, kernel csrc/gdn.cu:65-311); the math follows deltanet_core of the
// reference torch model (python/qengine/reference.py:211-242) including every bf16 rounding.
//
// Rollback scheme (same contract as the reference, csrc/gdn.cu:1-11): the committed state S in
// global memory is the state after position pos - pending. A pass first replays the `pending`
// rows that the previous pass staged and that were accepted -- from their checkpoint
// (k, v, decay, beta), 2 D + 2 floats per position and head -- and writes S back once. Its own
// n rows then run on the register copy of S and are only staged; S is not written for them. A
// rejected draft therefore costs nothing to undo, and a full-state snapshot per position
// (D * D floats) is never needed. Replayed and new rows use the same update routine, so the
// committed state is bit-identical to plain one-row decoding.
//
// Per value head j (q/k head j / (Hv / Hk)), per row at position p:
//   conv  c = w0 x[p-3] + w1 x[p-2] + w2 x[p-1] + w3 x[p] (fp32), y = bf16(silu(bf16(c)))
//   q = y_q * rsqrt(sum y_q^2 + 1e-6) / sqrt(D),  k = y_k * rsqrt(sum y_k^2 + 1e-6),  v = y_v
//   beta = bf16(sigmoid(b)),  decay = exp(-exp(A_log) * softplus(a + dt_bias))
//   S *= decay;  kv = S^T k;  delta = (v - kv) * beta;  S += k delta^T;  o = S^T q
//   out = bf16( bf16(norm_w * bf16(o_b * rsqrt(mean o_b^2 + eps))) * silu(z) ),  o_b = bf16(o)
// Conv history lives in a 16-slot ring keyed by absolute position (slot p & 15); with n <= 8 the
// slots read (p-3..p-1 of the first row) and written (p..p+n-1) never alias.
//
// Layout: one CTA per value head, 4 D threads. Thread (d, h) owns column d of S and the rows
// [h D/4, (h+1) D/4): S is read and written coalesced along d and stays in registers for the
// whole pass. Dot products over the D rows are finished through shared memory in a fixed order.
//
// Dependency handling: the state load, the staged checkpoints and the per-head constants do not
// depend on the producer of this pass's projections (they were written by this kernel one pass
// ago), so they are fetched before the programmatic-dependency wait and overlap the in_proj GEMV.
#include "common.cuh"
#include "../../include/qengine_b200.h"

namespace qb {
namespace {

constexpr int kRing = 16, kMaxRows = QE_MAX_ROWS, kRowGroups = 4;

struct GdnArgs {
  const bf16 *qkv, *z, *b, *a;
  long ldp;
  bf16* ring;
  const bf16 *conv_w, *A_log, *dt_bias, *norm_w;
  float *S, *st_k, *st_v, *st_g;
  const int* ctl;
  bf16* out;
  long ldo;
  int n, Hk, Hv;
  float eps;
  int early;
};

// S <- decay S + k (beta (v - (decay S)^T k))^T on this thread's rows of column d.
template <int D>
__device__ __forceinline__ void delta_update(float (&s)[D / kRowGroups], const float* k,
                                             const float* v, float decay, float beta,
                                             float (*part)[D], int d, int h) {
  constexpr int RP = D / kRowGroups;
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < RP; ++i) {
    s[i] *= decay;
    acc = fmaf(s[i], k[h * RP + i], acc);
  }
  part[h][d] = acc;
  __syncthreads();
  float kv = part[0][d];
#pragma unroll
  for (int g = 1; g < kRowGroups; ++g) kv += part[g][d];
  const float delta = (v[d] - kv) * beta;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < RP; ++i) s[i] = fmaf(k[h * RP + i], delta, s[i]);
}

template <int D>
__global__ void __launch_bounds__(kRowGroups * D) gdn_rows_kernel(const GdnArgs a) {
  constexpr int RP = D / kRowGroups, NT = kRowGroups * D;
  static_assert(NT >= 3 * D + kMaxRows, "one thread per conv channel plus one per row gate");
  dep_release();
  if (!a.early) dep_wait();

  __shared__ float q_s[kMaxRows][D], k_s[kMaxRows][D], v_s[kMaxRows][D];
  __shared__ float gate_s[kMaxRows][2];  // (decay, beta)
  __shared__ float part[kRowGroups][D];
  __shared__ float scratch[32];

  const int j = blockIdx.x;
  const int rep = a.Hv / a.Hk, i_qk = j / rep;
  const int C = 2 * a.Hk * D + a.Hv * D;
  const int tid = threadIdx.x, d = tid % D, h = tid / D;
  const int n = a.n;
  float* Sj = a.S + (size_t)j * D * D;

  // ---- independent of this pass's producer: state, per-head constants ----
  float s[RP];
#pragma unroll
  for (int i = 0; i < RP; ++i) s[i] = Sj[(h * RP + i) * D + d];
  int ch = 0;
  float cw[4] = {0.f, 0.f, 0.f, 0.f};
  if (tid < 3 * D) {
    const int part_id = tid / D, c = tid % D;
    ch = part_id == 0 ? i_qk * D + c : part_id == 1 ? a.Hk * D + i_qk * D + c : 2 * a.Hk * D + j * D + c;
#pragma unroll
    for (int w = 0; w < 4; ++w) cw[w] = tofloat(a.conv_w[ch * 4 + w]);
  }
  const float A_log = tofloat(a.A_log[j]), dt_bias = tofloat(a.dt_bias[j]);
  const float nw = tid < D ? tofloat(a.norm_w[tid]) : 0.f;
  if (a.early) dep_wait();

  const int P = a.ctl[0], pend = min(max(a.ctl[1], 0), kMaxRows);

  // ---- 1. replay the kept rows of the previous pass, write the committed state once ----
  for (int t = 0; t < pend; ++t) {
    if (tid < D) k_s[0][tid] = a.st_k[((size_t)t * a.Hv + j) * D + tid];
    else if (tid < 2 * D) v_s[0][tid - D] = a.st_v[((size_t)t * a.Hv + j) * D + tid - D];
    __syncthreads();
    delta_update<D>(s, k_s[0], v_s[0], a.st_g[(t * a.Hv + j) * 2], a.st_g[(t * a.Hv + j) * 2 + 1],
                    part, d, h);
    __syncthreads();
  }
  if (pend > 0) {
#pragma unroll
    for (int i = 0; i < RP; ++i) Sj[(h * RP + i) * D + d] = s[i];
  }

  // ---- 2a. causal conv + SiLU of every new row; conv ring update; gates ----
  if (tid < 3 * D) {
    const int part_id = tid / D, c = tid % D;
    float hist[3];
#pragma unroll
    for (int w = 0; w < 3; ++w) {
      const int p = P - 3 + w;
      hist[w] = p >= 0 ? tofloat(a.ring[(size_t)(p & (kRing - 1)) * C + ch]) : 0.f;
    }
    const bool owner = part_id == 2 || (j % rep) == 0;  // q/k channels are shared by `rep` heads
    float x0 = hist[0], x1 = hist[1], x2 = hist[2];
    for (int t = 0; t < n; ++t) {
      const bf16 xb = a.qkv[(long)t * a.ldp + ch];
      const float x3 = tofloat(xb);
      float acc = cw[0] * x0;
      acc = fmaf(cw[1], x1, acc);
      acc = fmaf(cw[2], x2, acc);
      acc = fmaf(cw[3], x3, acc);
      const float y = rnd(silu_acc(rnd(acc)));
      if (part_id == 0) q_s[t][c] = y;
      else if (part_id == 1) k_s[t][c] = y;
      else v_s[t][c] = y;
      if (owner) a.ring[(size_t)((P + t) & (kRing - 1)) * C + ch] = xb;
      x0 = x1; x1 = x2; x2 = x3;
    }
  } else if (tid < 3 * D + n) {
    const int t = tid - 3 * D;
    const float bt = rnd(sigmoid_acc(tofloat(a.b[(long)t * a.ldp + j])));
    const float x = tofloat(a.a[(long)t * a.ldp + j]) + dt_bias;
    const float sp = x > 20.f ? x : log1pf(expf(x));
    gate_s[t][0] = expf(-expf(A_log) * sp);
    gate_s[t][1] = bt;
  }
  float zr[kMaxRows];
  if (tid < D) {
#pragma unroll
    for (int t = 0; t < kMaxRows; ++t)
      if (t < n) zr[t] = tofloat(a.z[(long)t * a.ldp + j * D + tid]);
  }
  __syncthreads();

  // ---- 2b. l2norm of q and k of every row: one warp per vector, fixed summation order ----
  {
    const int lane = tid & 31, warp = tid >> 5, nwarps = NT / 32;
    for (int vec = warp; vec < 2 * n; vec += nwarps) {
      float* p = (vec & 1) ? k_s[vec >> 1] : q_s[vec >> 1];
      float e[D / 32], ss = 0.f;
#pragma unroll
      for (int u = 0; u < D / 32; ++u) {
        e[u] = p[lane + 32 * u];
        ss += warp_allsum(e[u] * e[u]);
      }
      const float inv = rsqrtf(ss + 1e-6f);
#pragma unroll
      for (int u = 0; u < D / 32; ++u)
        p[lane + 32 * u] = (vec & 1) ? e[u] * inv : (e[u] * inv) / sqrtf((float)D);
    }
  }
  __syncthreads();

  // ---- 2c. checkpoint every row for the next pass ----
  for (int t = 0; t < n; ++t) {
    if (tid < D) a.st_k[((size_t)t * a.Hv + j) * D + tid] = k_s[t][tid];
    else if (tid < 2 * D) a.st_v[((size_t)t * a.Hv + j) * D + tid - D] = v_s[t][tid - D];
    else if (tid == 2 * D) {
      a.st_g[(t * a.Hv + j) * 2] = gate_s[t][0];
      a.st_g[(t * a.Hv + j) * 2 + 1] = gate_s[t][1];
    }
  }

  // ---- 2d. the recurrence, row by row, on the register copy of S ----
  for (int t = 0; t < n; ++t) {
    delta_update<D>(s, k_s[t], v_s[t], gate_s[t][0], gate_s[t][1], part, d, h);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < RP; ++i) acc = fmaf(s[i], q_s[t][h * RP + i], acc);
    part[h][d] = acc;
    __syncthreads();
    float o = 0.f;
    if (tid < D) {
      o = part[0][tid];
#pragma unroll
      for (int g = 1; g < kRowGroups; ++g) o += part[g][tid];
      o = rnd(o);
    }
    const float ss = block_allsum(tid < D ? o * o : 0.f, scratch);
    if (tid < D) {
      const float nn = rnd(o * rsqrtf(ss / (float)D + a.eps));
      const float y = rnd(nw * nn);
      a.out[(long)t * a.ldo + j * D + tid] = tobf16(y * silu_acc(zr[t]));
    }
    __syncthreads();
  }
}

// Off by default: the early state load assumes that no launch on the same state is still in
// flight, which a caller that keeps other kernels between two steps of a layer guarantees.
bool g_gdn_early = false;

}  // namespace
}  // namespace qb

using namespace qb;

extern "C" void qe_set_gdn_early(int on) { g_gdn_early = on != 0; }
extern "C" void qe_set_gdn_phases(int) {}

extern "C" int qe_gdn_step_n(const void* qkv, const void* z, const void* b, const void* a, long ldp,
                             void* ring, const void* conv_w, const void* A_log, const void* dt_bias,
                             const void* norm_w, float* S, float* st_k, float* st_v, float* st_g,
                             const int* ctl, void* out, long ldo, int n, int Hk, int Hv, int D,
                             float eps, int q, void* stream) {
  (void)q;
  if (n < 1 || n > QE_MAX_ROWS || Hk < 1 || Hv < 1 || Hv % Hk) return QE_ERR_ARG;
  GdnArgs g{};
  g.qkv = (const bf16*)qkv; g.z = (const bf16*)z; g.b = (const bf16*)b; g.a = (const bf16*)a;
  g.ldp = ldp; g.ring = (bf16*)ring; g.conv_w = (const bf16*)conv_w; g.A_log = (const bf16*)A_log;
  g.dt_bias = (const bf16*)dt_bias; g.norm_w = (const bf16*)norm_w;
  g.S = S; g.st_k = st_k; g.st_v = st_v; g.st_g = st_g; g.ctl = ctl; g.out = (bf16*)out; g.ldo = ldo;
  g.n = n; g.Hk = Hk; g.Hv = Hv; g.eps = eps; g.early = g_gdn_early ? 1 : 0;
  const bool pdl = pdl_launch_enabled() && pdl_trigger_enabled();
  cudaStream_t s = (cudaStream_t)stream;
  if (D == 128) return (int)launch(gdn_rows_kernel<128>, dim3(Hv), dim3(512), 0, s, pdl, g);
  if (D == 64) return (int)launch(gdn_rows_kernel<64>, dim3(Hv), dim3(256), 0, s, pdl, g);
  return QE_ERR_ARG;
}
