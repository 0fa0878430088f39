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
//   S' = decay S + k delta^T with delta = beta (v - decay S^T k);  o = S'^T q
//   out = bf16( bf16(norm_w * bf16(o_b * rsqrt(mean o_b^2 + eps))) * silu(z) ),  o_b = bf16(o)
// Conv history lives in a 16-slot ring keyed by absolute position (slot p & 15); with n <= 8 the
// slots read (p-3..p-1 of the first row) and written (p..p+n-1) never alias.
//
// B200 layout. The columns of S are independent in the recurrence (column d only needs k, q,
// v[d]), so a head is split over a thread-block cluster of D / 32 CTAs, 32 columns each: 192 CTAs
// for the 48 heads of the 27B shape instead of 48. A CTA is 8 warps; warp w owns rows
// [w D/8, (w+1) D/8) of its 32 columns in registers (lane = column, S read and written coalesced).
// One pass over the register state per row gives both S^T k and S^T q of the pre-update state:
//   kv = decay (S^T k),  delta = beta (v - kv),  o = decay (S^T q) + delta (k . q)
// so a row costs one block barrier (partials are double-buffered) instead of several. The gated
// RMSNorm needs the sum of o_b^2 over all D columns of the head: every CTA pushes its partial sum
// into the shared memory of all CTAs of the cluster (distributed shared memory stores), one cluster
// barrier, and each CTA adds the partials in rank order.
//
// Dependency handling: the state, the per-head constants, ctl and the checkpoints of the previous
// pass do not depend on the producer of this pass's projections, so with `early` the state load
// and the whole replay (including the write-back of S) run before the programmatic-dependency
// wait and overlap the in_proj GEMV. `early` requires that the previous pass has completed when
// this pass starts (an engine launches the first kernel of a pass in plain stream order).
#include <cooperative_groups.h>

#include "common.cuh"
#include "../../include/qengine_b200.h"

namespace cg = cooperative_groups;

namespace qb {
namespace {

constexpr int kRing = 16, kMaxRows = QE_MAX_ROWS, kCols = 32, kWarps = 8;

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

template <int D>
__global__ void __launch_bounds__(kWarps * 32) gdn_cluster_kernel(const GdnArgs a) {
  constexpr int RP = D / kWarps;        // state rows per warp
  constexpr int NT = kWarps * 32;
  constexpr int NCTA = D / kCols;       // CTAs per head = cluster size
  dep_release();
  if (!a.early) dep_wait();
  cg::cluster_group cluster = cg::this_cluster();

  __shared__ float q_s[kMaxRows][D], k_s[kMaxRows][D];
  __shared__ float v_s[kMaxRows][kCols], o_s[kMaxRows][kCols];
  __shared__ float gate_s[kMaxRows][2];      // (decay, beta)
  __shared__ float kq_s[kMaxRows];           // k . q per row
  __shared__ float part[2][2][kWarps][kCols];  // [buffer][k or q][warp][column]
  __shared__ float ss_all[NCTA][kMaxRows];   // sum of o_b^2 per row of every CTA of the cluster (pushed)

  const int j = blockIdx.y;                  // value head
  const int cs = blockIdx.x;                 // column slice = rank in the cluster
  const int c0 = cs * kCols;
  const int rep = a.Hv / a.Hk, i_qk = j / rep;
  const int C = 2 * a.Hk * D + a.Hv * D;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = a.n;
  float* Sj = a.S + (size_t)j * D * D + c0 + lane;

  // ---- independent of this pass's producer: state slice, per-head constants, checkpoints ----
  // Every global load of this section is issued into registers before anything is used: a
  // "shared[i] = global[j]" loop stalls on each store until its load is back, one memory round
  // trip per iteration (that was 4 us in front of the replay). Loaded here: ctl, the state (3 MB
  // per layer, from HBM), all eight checkpoint slots (whether or not they are pending: that is
  // only known once ctl arrives), the per-head constants and the conv taps; the conv history
  // needs the position and follows as soon as ctl is there.
  const int ctl_pos = a.ctl[0], ctl_pending = a.ctl[1];
  float s[RP];
#pragma unroll
  for (int i = 0; i < RP; ++i) s[i] = Sj[(size_t)(warp * RP + i) * D];
  constexpr int KPT = kMaxRows * D / NT;  // checkpoint k values per thread
  float kreg[KPT];
#pragma unroll
  for (int u = 0; u < KPT; ++u) {
    const int idx = tid + u * NT, t = idx / D, i = idx - t * D;
    kreg[u] = a.st_k[((size_t)t * a.Hv + j) * D + i];
  }
  const float vreg = a.st_v[((size_t)warp * a.Hv + j) * D + c0 + lane];  // 8 warps = 8 slots, lane = column
  const float greg = lane < 2 ? a.st_g[(warp * a.Hv + j) * 2 + lane] : 0.f;
  const float A_log = tofloat(a.A_log[j]), dt_bias = tofloat(a.dt_bias[j]);
  const float nw = tofloat(a.norm_w[c0 + lane]);
  // conv channels of this thread (q and k: all D channels of the head's q/k head; v: own columns)
  constexpr int CPT = (2 * D + kCols + NT - 1) / NT;  // 2 for D = 128
  float cw[CPT][4], hx[CPT][3];
  int chn[CPT];
#pragma unroll
  for (int u = 0; u < CPT; ++u) {
    const int idx = tid + u * NT;
    chn[u] = -1;
    if (idx < 2 * D + kCols) {
      const int part_id = idx < D ? 0 : idx < 2 * D ? 1 : 2;
      const int c = part_id == 0 ? idx : part_id == 1 ? idx - D : idx - 2 * D;
      chn[u] = part_id == 0 ? i_qk * D + c : part_id == 1 ? a.Hk * D + i_qk * D + c : 2 * a.Hk * D + j * D + c0 + c;
#pragma unroll
      for (int w = 0; w < 4; ++w) cw[u][w] = tofloat(a.conv_w[chn[u] * 4 + w]);
    }
  }
  // ctl and the checkpoints were written by the previous pass, which has completed (the first
  // kernel of a pass is launched in plain stream order): with `early` the whole replay, including
  // the write-back of S, runs before the dependency wait and overlaps the tail of the in_proj GEMV.
  const int P = ctl_pos, pend = min(max(ctl_pending, 0), kMaxRows);
#pragma unroll
  for (int u = 0; u < CPT; ++u) {
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      const int p = P - 3 + b;
      hx[u][b] = (chn[u] >= 0 && p >= 0) ? tofloat(a.ring[(size_t)(p & (kRing - 1)) * C + chn[u]]) : 0.f;
    }
  }
#pragma unroll
  for (int u = 0; u < KPT; ++u) {
    const int idx = tid + u * NT, t = idx / D, i = idx - t * D;
    k_s[t][i] = kreg[u];
  }
  v_s[warp][lane] = vreg;
  if (lane < 2) gate_s[warp][lane] = greg;

  // S <- decay S + k (beta (v - decay S^T k))^T on this thread's rows of its column; with Q also
  // returns o = S'^T q for the column. Identical arithmetic for replayed and new rows.
  auto row_update = [&](const float* kk, const float* qq, float v, float decay, float beta, float kq,
                        int buf, bool want_o) -> float {
    float pk = 0.f, pq = 0.f;
#pragma unroll
    for (int i = 0; i < RP; ++i) {
      pk = fmaf(s[i], kk[warp * RP + i], pk);
      if (want_o) pq = fmaf(s[i], qq[warp * RP + i], pq);
    }
    part[buf][0][warp][lane] = pk;
    if (want_o) part[buf][1][warp][lane] = pq;
    __syncthreads();
    float kv = part[buf][0][0][lane];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) kv += part[buf][0][w][lane];
    const float delta = (v - decay * kv) * beta;
#pragma unroll
    for (int i = 0; i < RP; ++i) s[i] = fmaf(kk[warp * RP + i], delta, decay * s[i]);
    if (!want_o) return 0.f;
    float qs = part[buf][1][0][lane];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) qs += part[buf][1][w][lane];
    return fmaf(delta, kq, decay * qs);
  };

  // ---- 1. replay the kept rows of the previous pass, write the committed state once ----
  int buf = 0;
  __syncthreads();
  for (int t = 0; t < pend; ++t) {
    row_update(k_s[t], nullptr, v_s[t][lane], gate_s[t][0], gate_s[t][1], 0.f, buf, false);
    buf ^= 1;
  }
  if (pend > 0) {
#pragma unroll
    for (int i = 0; i < RP; ++i) Sj[(size_t)(warp * RP + i) * D] = s[i];
  }
  if (a.early) dep_wait();  // from here on: this pass's projections
  // the gate input of this warp's row is only needed at the very end: fetch it now; likewise the
  // decay / beta inputs of row tid, which the same thread would otherwise only request after its
  // share of the convolution (a second, dependent memory round trip)
  const float z_pre = warp < n ? tofloat(a.z[(long)warp * a.ldp + j * D + c0 + lane]) : 0.f;
  const float b_pre = tid < n ? tofloat(a.b[(long)tid * a.ldp + j]) : 0.f;
  const float a_pre = tid < n ? tofloat(a.a[(long)tid * a.ldp + j]) : 0.f;
  // and every projection value this thread convolves, all rows at once: independent loads in
  // flight together instead of one round trip per row and channel
  bf16 xr[CPT][kMaxRows];
#pragma unroll
  for (int u = 0; u < CPT; ++u)
#pragma unroll
    for (int t = 0; t < kMaxRows; ++t)
      if (chn[u] >= 0 && t < n) xr[u][t] = a.qkv[(long)t * a.ldp + chn[u]];
  __syncthreads();  // k_s / v_s are about to be overwritten by the new rows

  // ---- 2a. causal conv + SiLU of every new row (q, k: all D channels; v: own columns) ----
#pragma unroll
  for (int u = 0; u < CPT; ++u) {
    const int idx = tid + u * NT;
    if (chn[u] < 0) continue;
    const int part_id = idx < D ? 0 : idx < 2 * D ? 1 : 2;
    const int c = part_id == 0 ? idx : part_id == 1 ? idx - D : idx - 2 * D;
    const int ch = chn[u];
    float x0 = hx[u][0], x1 = hx[u][1], x2 = hx[u][2];
    // q/k channels are shared by `rep` heads and by the CTAs of a head: one CTA writes them
    const bool owner = part_id == 2 || ((j % rep) == 0 && cs == 0);
#pragma unroll
    for (int t = 0; t < kMaxRows; ++t) {
      if (t >= n) break;
      const bf16 xb = xr[u][t];
      const float x3 = tofloat(xb);
      float acc = cw[u][0] * x0;
      acc = fmaf(cw[u][1], x1, acc);
      acc = fmaf(cw[u][2], x2, acc);
      acc = fmaf(cw[u][3], x3, acc);
      const float y = rnd(silu_acc(rnd(acc)));
      if (part_id == 0) q_s[t][c] = y;
      else if (part_id == 1) k_s[t][c] = y;
      else v_s[t][c] = y;
      if (owner) a.ring[(size_t)((P + t) & (kRing - 1)) * C + ch] = xb;
      x0 = x1; x1 = x2; x2 = x3;
    }
  }
  if (tid < n) {
    const int t = tid;
    const float bt = rnd(sigmoid_acc(b_pre));
    const float x = a_pre + dt_bias;
    const float sp = x > 20.f ? x : log1pf(expf(x));
    gate_s[t][0] = expf(-expf(A_log) * sp);
    gate_s[t][1] = bt;
  }
  __syncthreads();

  // ---- 2b. l2norm of q and k of every row and k . q: warp t handles row t. Each lane first adds
  // up its own D / 32 elements, so a sum costs ONE butterfly, and the two independent butterflies
  // of q and k overlap (twelve dependent ones were 0.5 us of the step) ----
  for (int t = warp; t < n; t += kWarps) {
    float eq[D / 32], ek[D / 32], sq = 0.f, sk = 0.f;
#pragma unroll
    for (int u = 0; u < D / 32; ++u) {
      eq[u] = q_s[t][lane + 32 * u];
      ek[u] = k_s[t][lane + 32 * u];
      sq = fmaf(eq[u], eq[u], sq);
      sk = fmaf(ek[u], ek[u], sk);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
      sk += __shfl_xor_sync(0xffffffffu, sk, o);
    }
    const float iq = rsqrtf(sq + 1e-6f), ik = rsqrtf(sk + 1e-6f);
    float dot = 0.f;
#pragma unroll
    for (int u = 0; u < D / 32; ++u) {
      const float qn = (eq[u] * iq) / sqrtf((float)D), kn = ek[u] * ik;
      q_s[t][lane + 32 * u] = qn;
      k_s[t][lane + 32 * u] = kn;
      dot = fmaf(qn, kn, dot);
    }
    dot = warp_allsum(dot);
    if (lane == 0) kq_s[t] = dot;
  }
  __syncthreads();

  // ---- 2d. the recurrence, row by row, on the register copy of S ----
  for (int t = 0; t < n; ++t) {
    const float o = row_update(k_s[t], q_s[t], v_s[t][lane], gate_s[t][0], gate_s[t][1], kq_s[t], buf, true);
    buf ^= 1;
    if (warp == 0) o_s[t][lane] = rnd(o);  // the mixer output is a bf16 tensor in the model
  }
  __syncthreads();

  // ---- 2e. gated RMSNorm over the head's D outputs: every CTA pushes its partial sum of squares
  // into the shared memory of all CTAs of the cluster; one cluster barrier makes them visible ----
  for (int t = warp; t < n; t += kWarps) {
    const float ob = o_s[t][lane];
    const float ssum = warp_allsum(ob * ob);
    if (lane < NCTA) *cluster.map_shared_rank(&ss_all[cs][t], lane) = ssum;
  }
  cluster.sync();
  for (int t = warp; t < n; t += kWarps) {
    float total = 0.f;
#pragma unroll
    for (int rk = 0; rk < NCTA; ++rk) total += ss_all[rk][t];
    const float ob = o_s[t][lane];
    const float nn = rnd(ob * rsqrtf(total / (float)D + a.eps));
    const float y = rnd(nw * nn);
    const float zz = t == warp ? z_pre : tofloat(a.z[(long)t * a.ldp + j * D + c0 + lane]);
    a.out[(long)t * a.ldo + j * D + c0 + lane] = tobf16(y * silu_acc(zz));
  }
  // no second barrier: nobody reads remote shared memory after the one above, and every remote
  // store was issued before it
  // ---- 2f. checkpoint every row for the next pass (k, gates: one CTA per head; v: own slice).
  // Last, behind the output: nothing in this pass waits for these stores. The CTA with cs == 0
  // overwrites st_k / st_g, which its siblings read while replaying: the cluster barrier of 2e
  // lies in between, and every CTA passes it only after its replay ----
  for (int t = 0; t < n; ++t) {
    if (cs == 0) {
      for (int i = tid; i < D; i += NT) a.st_k[((size_t)t * a.Hv + j) * D + i] = k_s[t][i];
      if (tid == 0) {
        a.st_g[(t * a.Hv + j) * 2] = gate_s[t][0];
        a.st_g[(t * a.Hv + j) * 2 + 1] = gate_s[t][1];
      }
    }
    if (tid < kCols) a.st_v[((size_t)t * a.Hv + j) * D + c0 + tid] = v_s[t][tid];
  }
}

// Off by default: the early state load assumes that no launch on the same state is still in
// flight, which a caller that keeps other kernels between two steps of a layer guarantees.
bool g_gdn_early = false;

template <int D>
cudaError_t launch_gdn(const GdnArgs& g, int Hv, cudaStream_t s, bool pdl) {
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(D / kCols, Hv, 1);
  c.blockDim = dim3(kWarps * 32, 1, 1);
  c.dynamicSmemBytes = 0;
  c.stream = s;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = D / kCols;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  c.attrs = at;
  c.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&c, gdn_cluster_kernel<D>, g);
}

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
  if (D == 128) return (int)launch_gdn<128>(g, Hv, s, pdl);
  if (D == 64) return (int)launch_gdn<64>(g, Hv, s, pdl);
  return QE_ERR_ARG;
}
