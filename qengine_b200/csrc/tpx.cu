// Tensor-parallel exchanges of the decode path, fused with their consumers (no counterpart in the
// single-GPU reference).
//
// A matrix split along K over t ranks leaves every rank with fp32 partial rows [n, H]. The
// consumer is always "residual += sum of the partial rows; RMSNorm1p". tp_xnorm_kernel does the
// exchange and the norm in ONE kernel (a cluster of 8 CTAs per row) over peer memory: every rank stores its partial row straight
// into a slot of every peer's exchange block (NVLink peer stores), and reads the other ranks'
// rows from its own block as they land. Transport is a flag-in-data protocol: each 8-byte store
// carries 4 bytes of payload and the 4-byte sequence number of the exchange, 8-byte stores are
// single-copy atomic, so a reader that sees the expected sequence number also sees the payload --
// no fences, no separate flag round trip; the latency of an exchange is one NVLink store.
//
//   block of rank r (cudaMalloc'ed by qe_tp_alloc, mapped into every peer through CUDA IPC):
//     ints  [0..7]   sequence number of the last finished norm exchange, per row
//           [8..15]  same for the argmax exchange
//           [16..19] sticky error word, late source rank, row, kind
//     +256  argmax slots  [2][8 src][8 rows] x 16 B   {value, seq, index, seq}
//     +4096 norm slots    [2][world src][8 rows][H] x 8 B   {payload, seq}
//
// Slots are double-buffered on the parity of the sequence number: a rank can only start exchange
// e + 2 after it finished e + 1, for which every peer must have pushed e + 1, which a peer does
// only after it finished reading e. Sequence numbers live in device memory and advance once per
// exchange per row, identically on every rank (all ranks run the same passes), so CUDA-graph
// replays need no host-side argument.
//
// Every wait is bounded (wall-clock limit per wait, default 10 s; sticky: after the first timeout
// no later wait spins at all). A timed-out exchange produces garbage and sets the error word that
// qe_tp_error reads; it never hangs the GPU. The sum over ranks is taken in ascending rank order
// on every rank, so all ranks hold bit-identical activations. The same norm without the exchange
// (parts already gathered by a library collective) is qe_rmsnorm1p_parts; its sum of squares is
// taken in another order, so the two transports agree to rounding, not bit for bit.
#include <cooperative_groups.h>

#include <algorithm>
#include <cstring>

#include "../../include/qengine_b200.h"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace qb {
namespace {

constexpr int kMaxWorld = 8, kRows = QE_MAX_ROWS;
constexpr long kAmOff = 256, kNormOff = 4096;
constexpr int kErrWord = 16;
constexpr int kNone = 0x7fffffff;

struct TpView {
  char* base[kMaxWorld];  // every rank's block as mapped into this process; [rank] is our own
  int rank, world, H;
  unsigned long long timeout_ns;
};

struct Comm {
  TpView v;
  int device;
};

__device__ __forceinline__ uint4 ld_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Two {payload, seq} pairs; returns once both carry sequence number e, or on timeout / earlier
// error (then `dead` is set and whatever is in the slot is returned).
__device__ __forceinline__ uint4 ll_wait(const void* p, uint32_t e, int* hdr, const TpView& tv, int src, int row,
                                         int kind, bool& dead) {
  uint4 v = ld_v4(p);
  if ((v.y == e && v.w == e) || dead) return v;
  const unsigned long long t0 = now_ns();
  for (uint32_t spin = 1;; ++spin) {
    v = ld_v4(p);
    if (v.y == e && v.w == e) return v;
    if ((spin & 127u) == 0) {
      volatile int* err = hdr + kErrWord;
      if (err[0] != 0 || now_ns() - t0 > tv.timeout_ns) {
        if (atomicCAS(hdr + kErrWord, 0, 1) == 0) { err[1] = src; err[2] = row; err[3] = kind; }
        dead = true;
        return v;
      }
    }
  }
}

__device__ __forceinline__ char* norm_slot(char* base, const TpView& tv, uint32_t e, int src, int row) {
  return base + kNormOff + ((((long)(e & 1u) * tv.world + src) * kRows + row) * (long)tv.H) * 8;
}

// RMSNorm1p with residual delta = bf16(sum over p of parts[p]), parts = gathered fp32 partial rows
// [nparts, rows, H] contiguous, summed in ascending p. Thread layout and arithmetic follow
// rmsnorm1p_vec_kernel (rowops.cu), so one part gives its bits.
template <int PKT>
__global__ void __launch_bounds__(256)
tp_norm_kernel(bf16* x, const float* part, int nparts, const bf16* w, bf16* out, int rows, int H, long ldx,
               long ldo, float eps) {
  dep_release();
  dep_wait();
  __shared__ float scratch[32];
  const int row = blockIdx.x, npk = H >> 3;
  uint4* xr = reinterpret_cast<uint4*>(x + (long)row * ldx);
  float v[PKT][8];
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < PKT; ++p) {
    const int i = threadIdx.x + p * blockDim.x;
    if (i < npk) {
      float d[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) d[k] = 0.f;
      for (int src = 0; src < nparts; ++src) {
        const float4* pr = reinterpret_cast<const float4*>(part + ((size_t)src * rows + row) * H) + 2 * i;
        const float4 a = pr[0], b = pr[1];
        d[0] += a.x; d[1] += a.y; d[2] += a.z; d[3] += a.w;
        d[4] += b.x; d[5] += b.y; d[6] += b.z; d[7] += b.w;
      }
      widen8(xr[i], v[p]);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[p][k] = rnd(v[p][k] + rnd(d[k]));
      xr[i] = narrow8(v[p]);
#pragma unroll
      for (int k = 0; k < 8; ++k) ss = fmaf(v[p][k], v[p][k], ss);
    }
  }
  const float inv = rsqrtf(block_allsum(ss, scratch) / (float)H + eps);
  uint4* orow = reinterpret_cast<uint4*>(out + (long)row * ldo);
#pragma unroll
  for (int p = 0; p < PKT; ++p) {
    const int i = threadIdx.x + p * blockDim.x;
    if (i < npk) {
      float g[8], y[8];
      widen8(__ldg(reinterpret_cast<const uint4*>(w) + i), g);
#pragma unroll
      for (int k = 0; k < 8; ++k) y[k] = v[p][k] * inv * (1.0f + g[k]);
      orow[i] = narrow8(y);
    }
  }
}

// The exchange + norm kernel. A row is handled by a thread-block cluster of kCX CTAs, each owning
// a slice of PK packets (8 elements each) of the row; inside a CTA the threads form a [peer][packet]
// grid, so every (peer, packet) pair has a thread of its own: it pushes this rank's packet into
// that peer's block (4 x 16-byte flag-in-data stores) and polls this rank's block for the packet
// the peer pushes (4 x 16-byte loads per try). With 8 ranks and hidden 5120 that is 4,480 threads
// on 8 SMs per row, each with 64 bytes out and 64 bytes in -- the exchange is one NVLink store
// latency plus one poll, not a loop over peers and packets in one CTA. The packets land in shared
// memory; the first PK threads of the CTA add the ranks in ascending order (every rank the same
// order: bit-identical activations everywhere), round once to bf16, add the residual, and the sum
// of squares of the row is combined across the cluster through distributed shared memory in CTA
// order. Rows of a pass run in parallel (grid.y).
constexpr int kCX = 8;  // CTAs per row = cluster size (portable maximum)

__global__ void __launch_bounds__(1024)
tp_xnorm_kernel(TpView tv, bf16* x, const float* part, const bf16* w, bf16* out, __half* out16, int H, int PK,
                long ldx, long ldp, long ldo, long ld16, float eps) {
  dep_release();
  dep_wait();
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ float recv_s[];  // [world][PK][8]: the peers' packets of this CTA's slice
  __shared__ float scratch[32];
  __shared__ float ss_all[kCX];      // sum of squares of every CTA's slice (pushed by its owner)
  const int cs = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
  const int npk = H >> 3, npeers = tv.world - 1;
  const int pk = tid % PK, pj = tid / PK;  // packet inside the slice, peer slot
  const int i = cs * PK + pk;              // packet of the row
  int* hdr = reinterpret_cast<int*>(tv.base[tv.rank]);
  const uint32_t e = (uint32_t)(*(volatile int*)(hdr + row)) + 1u;
  bool dead = *(volatile int*)(hdr + kErrWord) != 0;

  float mine[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) mine[k] = 0.f;
  const bool has_packet = i < npk && pj < max(npeers, 1);
  if (has_packet) {
    const float4* pr = reinterpret_cast<const float4*>(part + (long)row * ldp) + 2 * i;
    const float4 a = pr[0], b = pr[1];
    mine[0] = a.x; mine[1] = a.y; mine[2] = a.z; mine[3] = a.w;
    mine[4] = b.x; mine[5] = b.y; mine[6] = b.z; mine[7] = b.w;
  }
  if (has_packet && pj < npeers) {
    const int peer = pj < tv.rank ? pj : pj + 1;  // the other ranks in ascending order
    char* d = norm_slot(tv.base[peer], tv, e, tv.rank, row) + (long)i * 64;
#pragma unroll
    for (int q = 0; q < 4; ++q)
      st_v4(d + 16 * q, __float_as_uint(mine[2 * q]), e, __float_as_uint(mine[2 * q + 1]), e);
    const char* sp = norm_slot(tv.base[tv.rank], tv, e, peer, row) + (long)i * 64;
    uint4 rv[4];
    const unsigned long long t0 = now_ns();
    for (unsigned tries = 1;; ++tries) {
      // all four loads of a try are issued together: one round trip per try, never one per word
#pragma unroll
      for (int q = 0; q < 4; ++q) rv[q] = ld_v4(sp + 16 * q);
      bool all = true;
#pragma unroll
      for (int q = 0; q < 4; ++q) all = all && rv[q].y == e && rv[q].w == e;
      if (all || dead) break;
      if ((tries & 63u) == 0) {
        volatile int* err = hdr + kErrWord;
        if (err[0] != 0 || now_ns() - t0 > tv.timeout_ns) {
          if (atomicCAS(hdr + kErrWord, 0, 1) == 0) { err[1] = peer; err[2] = row; err[3] = 0; }
          dead = true;
          break;
        }
      }
    }
    float* dst = recv_s + ((size_t)peer * PK + pk) * 8;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      dst[2 * q] = __uint_as_float(rv[q].x);
      dst[2 * q + 1] = __uint_as_float(rv[q].z);
    }
  }
  __syncthreads();

  float v[8];
  float ss = 0.f;
  const bool owner = pj == 0 && i < npk;
  if (owner) {
    float dsum[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) dsum[k] = 0.f;
    for (int src = 0; src < tv.world; ++src) {
      if (src == tv.rank) {
#pragma unroll
        for (int k = 0; k < 8; ++k) dsum[k] += mine[k];
      } else {
        const float* rp = recv_s + ((size_t)src * PK + pk) * 8;
#pragma unroll
        for (int k = 0; k < 8; ++k) dsum[k] += rp[k];
      }
    }
    uint4* xr = reinterpret_cast<uint4*>(x + (long)row * ldx);
    widen8(xr[i], v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = rnd(v[k] + rnd(dsum[k]));
    xr[i] = narrow8(v);
#pragma unroll
    for (int k = 0; k < 8; ++k) ss = fmaf(v[k], v[k], ss);
  }
  const float mine_ss = block_allsum(ss, scratch);
  if (tid < kCX) *cluster.map_shared_rank(&ss_all[cs], tid) = mine_ss;
  cluster.sync();
  float total = 0.f;
#pragma unroll
  for (int c = 0; c < kCX; ++c) total += ss_all[c];
  const float inv = rsqrtf(total / (float)H + eps);
  if (owner) {
    float g[8], y[8];
    widen8(__ldg(reinterpret_cast<const uint4*>(w) + i), g);
#pragma unroll
    for (int k = 0; k < 8; ++k) y[k] = v[k] * inv * (1.0f + g[k]);
    const uint4 q = narrow8(y);
    reinterpret_cast<uint4*>(out + (long)row * ldo)[i] = q;
    if (out16) {  // the same bf16-rounded numbers as fp16: input of the GEMV's fp16 flavour
      widen8(q, y);
      reinterpret_cast<uint4*>(out16 + (long)row * ld16)[i] = half8(y);
    }
  }
  // every CTA of the cluster read the sequence number before the cluster barrier above
  if (cs == 0 && tid == 0) *(volatile int*)(hdr + row) = (int)e;
}

__device__ __forceinline__ bool beats(float a, int ia, float b, int ib) {
  const bool an = a != a, bn = b != b;
  if (an != bn) return an;
  if (!an && a != b) return a > b;
  return ia < ib;
}

// Greedy token over a vocabulary split across ranks: every rank pushes its (value, index) per row
// to every peer and merges the t candidates in ascending rank order with the argmax ordering rule
// (NaN first, larger value, lower index). 64 threads: thread = (row, src).
__global__ void __launch_bounds__(64)
tp_argmax_kernel(TpView tv, const float* cand_v, const int* cand_i, int rows, int* out) {
  dep_release();
  dep_wait();
  const int row = threadIdx.x >> 3, src = threadIdx.x & 7;
  int* hdr = reinterpret_cast<int*>(tv.base[tv.rank]);
  const bool active = row < rows && src < tv.world;
  float v = -INFINITY;
  int i = kNone;
  uint32_t e = 0;
  if (active) {
    e = (uint32_t)(*(volatile int*)(hdr + 8 + row)) + 1u;
    bool dead = *(volatile int*)(hdr + kErrWord) != 0;
    const long slot = kAmOff + (((long)(e & 1u) * kMaxWorld + tv.rank) * kRows + row) * 16;
    const float mv = cand_v[row];
    const int mi = cand_i[row];
    if (src != tv.rank) {  // this thread serves peer `src`: push ours, then wait for theirs
      st_v4(tv.base[src] + slot, __float_as_uint(mv), e, (uint32_t)mi, e);
      const long theirs = kAmOff + (((long)(e & 1u) * kMaxWorld + src) * kRows + row) * 16;
      const uint4 t = ll_wait(tv.base[tv.rank] + theirs, e, hdr, tv, src, row, 1, dead);
      v = __uint_as_float(t.x);
      i = (int)t.z;
    } else {
      v = mv;
      i = mi;
    }
  }
  // ascending-rank merge inside the 8-lane group of the row
  float bv = __shfl_sync(0xffffffffu, v, (threadIdx.x & 24));
  int bi = __shfl_sync(0xffffffffu, i, (threadIdx.x & 24));
  for (int s = 1; s < kMaxWorld; ++s) {
    const float ov = __shfl_sync(0xffffffffu, v, (threadIdx.x & 24) + s);
    const int oi = __shfl_sync(0xffffffffu, i, (threadIdx.x & 24) + s);
    if (s < tv.world && beats(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if (active && src == 0) {
    out[row] = bi == kNone ? 0 : bi;
    *(volatile int*)(hdr + 8 + row) = (int)e;
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool pdl_on() { return pdl_launch_enabled(); }

int launch_parts_norm(void* x, const float* part, int nparts, const void* w, void* out, int rows, int H, long ldx,
                      long ldo, float eps, cudaStream_t s) {
  if (rows < 1 || rows > kRows || H < 8 || H % 8 || H > 8 * 256 * 4 || ldx % 8 || ldo % 8 || !aligned16(x) ||
      !aligned16(out) || !aligned16(w) || !aligned16(part))
    return QE_ERR_ARG;
  bf16* X = (bf16*)x;
  const bf16* W = (const bf16*)w;
  bf16* O = (bf16*)out;
  const int npk = H / 8;
  if (npk <= 256) {
    const int threads = std::max(32, (npk + 31) / 32 * 32);
    return (int)launch(tp_norm_kernel<1>, dim3(rows), dim3(threads), 0, s, pdl_on(), X, part, nparts, W, O, rows, H,
                       ldx, ldo, eps);
  }
  if (npk <= 512)
    return (int)launch(tp_norm_kernel<2>, dim3(rows), dim3(256), 0, s, pdl_on(), X, part, nparts, W, O, rows, H, ldx,
                       ldo, eps);
  return (int)launch(tp_norm_kernel<4>, dim3(rows), dim3(256), 0, s, pdl_on(), X, part, nparts, W, O, rows, H, ldx,
                     ldo, eps);
}

}  // namespace
}  // namespace qb

using namespace qb;

extern "C" int qe_rmsnorm1p_parts(void* x, const float* parts, int nparts, const void* w, void* out, int rows,
                                  int H, long ldx, long ldo, float eps, void* stream) {
  if (nparts < 1) return QE_ERR_ARG;
  return launch_parts_norm(x, parts, nparts, w, out, rows, H, ldx, ldo, eps, (cudaStream_t)stream);
}

extern "C" long qe_tp_block_bytes(int H, int world) {
  if (H < 8 || H % 8 || world < 1 || world > kMaxWorld) return QE_ERR_ARG;
  return kNormOff + 2L * world * kRows * (long)H * 8;
}

extern "C" int qe_tp_alloc(long bytes, void** ptr) {
  if (bytes < kNormOff || !ptr) return QE_ERR_ARG;
  cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(*ptr, 0, (size_t)bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  return (int)e;
}

extern "C" int qe_tp_free(void* ptr) { return (int)cudaFree(ptr); }

extern "C" int qe_tp_export(void* ptr, unsigned char* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e == cudaSuccess) memcpy(handle64, &h, 64);
  return (int)e;
}

extern "C" int qe_tp_import(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

extern "C" int qe_tp_unmap(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

extern "C" int qe_tp_comm_create(void* const* blocks, int rank, int world, int H, void** comm) {
  if (!blocks || !comm || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || H < 8 || H % 8)
    return QE_ERR_ARG;
  Comm* c = new Comm();
  for (int r = 0; r < world; ++r) {
    if (!blocks[r]) { delete c; return QE_ERR_ARG; }
    c->v.base[r] = static_cast<char*>(blocks[r]);
  }
  c->v.rank = rank;
  c->v.world = world;
  c->v.H = H;
  c->v.timeout_ns = 10ull * 1000 * 1000 * 1000;
  cudaGetDevice(&c->device);
  *comm = c;
  return 0;
}

extern "C" int qe_tp_comm_destroy(void* comm) {
  delete static_cast<Comm*>(comm);
  return 0;
}

extern "C" int qe_tp_set_timeout_ms(void* comm, long ms) {
  if (!comm || ms < 1) return QE_ERR_ARG;
  static_cast<Comm*>(comm)->v.timeout_ns = (unsigned long long)ms * 1000000ull;
  return 0;
}

extern "C" int qe_tp_exchange_norm(void* comm, void* x, const float* part, const void* w, void* out, void* out16,
                                   int rows, long ldx, long ldp, long ldo, long ld16, float eps, void* stream) {
  if (!comm || (out16 && (!aligned16(out16) || ld16 % 8))) return QE_ERR_ARG;
  const Comm* c = static_cast<Comm*>(comm);
  const int H = c->v.H, npk = H / 8;
  if (rows < 1 || rows > kRows || ldx % 8 || ldo % 8 || ldp % 4 || !aligned16(x) || !aligned16(out) ||
      !aligned16(w) || !aligned16(part))
    return QE_ERR_ARG;
  const int PK = (npk + kCX - 1) / kCX;                      // packets per CTA
  const int lanes = PK * std::max(1, c->v.world - 1);        // one thread per (peer, packet)
  const int threads = std::max(32, (lanes + 31) / 32 * 32);
  if (threads > 1024) return QE_ERR_ARG;                     // hidden sizes beyond 8 * 8 * 146 per rank pair
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(kCX, rows, 1);
  lc.blockDim = dim3(threads, 1, 1);
  lc.dynamicSmemBytes = (size_t)c->v.world * PK * 8 * sizeof(float);
  lc.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = kCX;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = pdl_on() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&lc, tp_xnorm_kernel, c->v, (bf16*)x, part, (const bf16*)w, (bf16*)out,
                                 (__half*)out16, H, PK, ldx, ldp, ldo, ld16, eps);
}

extern "C" int qe_tp_exchange_argmax(void* comm, const float* cand_v, const int* cand_i, int rows, int* out,
                                     void* stream) {
  if (!comm || rows < 1 || rows > kRows) return QE_ERR_ARG;
  const Comm* c = static_cast<Comm*>(comm);
  return (int)launch(tp_argmax_kernel, dim3(1), dim3(64), 0, (cudaStream_t)stream, pdl_on(), c->v, cand_v, cand_i,
                     rows, out);
}

extern "C" int qe_tp_error(void* comm, int* info4) {
  if (!comm) return QE_ERR_ARG;
  const Comm* c = static_cast<Comm*>(comm);
  int w[4] = {0, 0, 0, 0};
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess)
    e = cudaMemcpy(w, c->v.base[c->v.rank] + kErrWord * 4, sizeof(w), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return -(int)e;
  if (info4) memcpy(info4, w, sizeof(w));
  return w[0];
}

extern "C" int qe_tp_clear_error(void* comm) {
  if (!comm) return QE_ERR_ARG;
  const Comm* c = static_cast<Comm*>(comm);
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemset(c->v.base[c->v.rank] + kErrWord * 4, 0, 16);
  return (int)e;
}
