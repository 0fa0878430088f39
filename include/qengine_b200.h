/*
 * qengine_b200 -- C ABI of the batch-1 speculative-decode operator library for B200 (sm_100a).
 *
 * This header is the drop-in boundary. Every entry point replaces one host launcher of the
 * reference project (manaspros/qengine): `csrc/ops.h` (the launchers behind the python module
 * `qengine._C`, bound in `csrc/bindings.cpp`) and `csrc/gemv_w4.h` (the W4A16 GEMV behind
 * `qengine._w4`, bound in `csrc/gemv_w4_bind.cpp`). The reference exports these with C++ linkage;
 * here they are plain `extern "C"` symbols over raw device pointers, sizes and a stream handle, so
 * they can be bound from pybind11, ctypes, cgo or anything else that can call C.
 *
 * Conventions (same as the reference, csrc/ops.h:1-2, csrc/bindings.cpp:1-4):
 *   - all pointers are device pointers unless a comment says "host";
 *   - activations / outputs are bf16 (passed as void*), control buffers int32, state fp32;
 *   - `ld*` arguments are row strides in ELEMENTS; rows have unit inner stride;
 *   - `stream` is a cudaStream_t passed as void*; every call only enqueues work on it, never
 *     allocates and never synchronises, so a whole decode cycle can be captured in a CUDA graph;
 *   - n (rows per pass) is 1..8.
 * Unlike the reference launchers (which return void) every launcher returns the cudaError_t of
 * the launch as an int (0 = cudaSuccess), or QE_ERR_ARG for an argument the kernels cannot serve.
 *
 * Numerical contract kept from the reference: row r of an n-row call is bit-identical to the
 * 1-row call on that row, for every op; results are bit-identical run to run (no float atomics).
 */
#ifndef QENGINE_B200_H_
#define QENGINE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QE_ERR_ARG (-22)
#define QE_MAX_ROWS 8

/* Library / device information. Returns the ABI version (bumped on incompatible changes). */
int qe_abi_version(void);
/* Number of SMs of the current device (cached per device). */
int qe_sm_count(void);

/* ------------------------------------------------------------------------------------------
 * Row ops. Reference: csrc/ops.h:6-17 (launch_embed .. launch_argmax), kernels csrc/basic.cu.
 * ------------------------------------------------------------------------------------------ */

/* out[r, :] = table[tok[r], :] for r < n; token ids outside [0, V) give a zero row.
 * Replaces launch_embed (csrc/ops.h:6-7). */
int qe_embed(const void* table, const int* tok, void* out, int n, int H, int V, long ldo,
             void* stream);

/* Zero-centred RMSNorm with optional fused residual add. If delta != NULL, x = bf16(x + delta) is
 * written back in place first. out = bf16(x * rsqrt(mean(x^2) + eps) * (1 + w)).
 * Replaces launch_rmsnorm1p (csrc/ops.h:8-9). */
int qe_rmsnorm1p(void* x, const void* delta, const void* w, void* out, int rows, int H, long ldx,
                 long ldd, long ldo, float eps, void* stream);

/* out[r, j] = bf16(sum_k W[j, k] * x[r, k]); W bf16 [N, K] row-major, K % 8 == 0, 16-byte aligned
 * rows. Replaces launch_gemv_bf16 (csrc/ops.h:10-11). */
int qe_gemv_bf16(const void* W, const void* x, void* out, int nr, int N, int K, long ldx, long ldo,
                 void* stream);

/* gu rows are [gate(I) | up(I)]; out = bf16(bf16(silu(gate)) * up).
 * Replaces launch_swiglu (csrc/ops.h:12). */
int qe_swiglu(const void* gu, void* out, int n, int I, long ldg, long ldo, void* stream);

/* Per-row argmax with torch semantics (NaN is the maximum, ties go to the lowest index, an
 * all -inf row gives 0). pv/pi: scratch with rows*nb entries each. out[r] = idmap ? idmap[i] : i.
 * Replaces launch_argmax (csrc/ops.h:13-14). */
int qe_argmax(const void* x, int rows, int n, long ldx, float* pv, int* pi, int nb, int* out,
              const int* idmap, void* stream);

/* Tensor-parallel helpers, no counterpart in the reference (it is single-GPU).
 * qe_rmsnorm1p_parts: like qe_rmsnorm1p with delta = bf16(sum over p < nparts of parts[p]), parts
 * fp32 [nparts, rows, H] contiguous (the all-gathered partial sums of a K-split GEMV), added in
 * ascending p so that the result does not depend on the collective's algorithm.
 * qe_argmax_v: qe_argmax that also stores the winning value and adds `base` to the index (a rank's
 * slice of the vocabulary). qe_argmax_merge: best of nparts candidates per row, vals / idx
 * [nparts, rows], same ordering rule (NaN first, larger value, lower index). */
int qe_rmsnorm1p_parts(void* x, const float* parts, int nparts, const void* w, void* out, int rows,
                       int H, long ldx, long ldo, float eps, void* stream);
int qe_argmax_v(const void* x, int rows, int n, long ldx, float* pv, int* pi, int nb, int* out,
                float* out_v, const int* idmap, int base, void* stream);
int qe_argmax_merge(const float* vals, const int* idx, int nparts, int rows, int* out, void* stream);

/* Tensor-parallel exchange over peer memory, fused with its consumer (no counterpart in the
 * reference). Each rank owns one exchange block (qe_tp_alloc; size qe_tp_block_bytes) that every
 * other rank of the node maps through CUDA IPC (qe_tp_export -> 64-byte handle -> qe_tp_import in
 * the peer process). qe_tp_comm_create takes the world's block addresses as seen from this
 * process (blocks[rank] = own) and returns an opaque communicator.
 *   qe_tp_exchange_norm: part = this rank's fp32 partial rows [rows, H] (stride ldp) of a matrix
 *     split along K. One kernel stores them into every peer's block, collects the peers' rows and
 *     computes x = bf16(x + bf16(sum over ranks, ascending)), out = RMSNorm1p(x) * (1 + w): the
 *     all-reduce and qe_rmsnorm1p in one launch, bit-identical on every rank. out16 (optional,
 *     stride ld16): the same rows as fp16, the input of a qe_w4_gemv with x_f16 = 1.
 *   qe_tp_exchange_argmax: (value, index) candidates per row from qe_argmax_v are exchanged and
 *     merged with the argmax ordering rule; out[r] = greedy token over the whole vocabulary.
 * All ranks must issue the same sequence of exchanges with the same row counts. Waits are bounded
 * (qe_tp_set_timeout_ms, default 10 s per wait; after the first timeout later waits do not spin);
 * qe_tp_error synchronises the device and returns the sticky error word (0 = none), info4 =
 * {error, late source rank, row, kind 0 norm / 1 argmax}. Calls only enqueue work on `stream` and
 * can be captured in CUDA graphs (sequence numbers live in the block). */
long qe_tp_block_bytes(int H, int world);
int qe_tp_alloc(long bytes, void** ptr);
int qe_tp_free(void* ptr);
int qe_tp_export(void* ptr, unsigned char* handle64);
int qe_tp_import(const unsigned char* handle64, void** ptr);
int qe_tp_unmap(void* ptr);
int qe_tp_comm_create(void* const* blocks, int rank, int world, int H, void** comm);
int qe_tp_comm_destroy(void* comm);
int qe_tp_set_timeout_ms(void* comm, long ms);
int qe_tp_exchange_norm(void* comm, void* x, const float* part, const void* w, void* out, void* out16,
                        int rows, long ldx, long ldp, long ldo, long ld16, float eps, void* stream);
int qe_tp_exchange_argmax(void* comm, const float* cand_v, const int* cand_i, int rows, int* out,
                          void* stream);
int qe_tp_error(void* comm, int* info4);
int qe_tp_clear_error(void* comm);

/* ------------------------------------------------------------------------------------------
 * Device-side bookkeeping of one pass. ctl (int32[>=24]): [0] pos, [1] pending DeltaNet rows,
 * [2] mode (0 prefill, 1 decode/verify), [3] m, [4] cycles, [5] accepted drafts, [16+m] histogram.
 * Reference: csrc/ops.h:15-19, kernels csrc/basic.cu:256-307. Integer results are bit-exact.
 * ------------------------------------------------------------------------------------------ */

/* Greedy longest-prefix acceptance. Replaces launch_accept (csrc/ops.h:15-16). */
int qe_accept(const int* in_tok, const int* am, int n, int* ctl, int* next_tok, int* log,
              int max_len, void* stream);

/* Advance pos by m+1, pending = m+1, next input = [am[m], drafts[0..k)].
 * Replaces launch_commit (csrc/ops.h:17). */
int qe_commit(int* ctl, int* in_tok, const int* am, const int* drafts, int k, void* stream);

/* qe_accept followed by qe_commit in one launch, for passes that run nothing in between (plain
 * decode, prefill). No counterpart in the reference, which always launches the two kernels. */
int qe_accept_commit(int* in_tok, const int* am, int n, int* ctl, int* next_tok, int* log,
                     int max_len, const int* drafts, int k, void* stream);

/* End of a chained single-row draft pass: draft_out[0] = mtp_am[0] and dst[0..H) = src[0..H).
 * Replaces the two device-to-device copies the reference issues there
 * (python/qengine/engine.py:516-517). */
int qe_chain_draft(const int* mtp_am, int* draft_out, const void* src, void* dst, int H,
                   void* stream);

/* mpos[0] = off < 0 ? pos : pos + m + 1 + off; optional dst[:] = src[m, :]; optional
 * draft0[0] = mtp_am[m]. Replaces launch_mtp_select (csrc/ops.h:18-19). */
int qe_mtp_select(const int* ctl, int* mpos, int off, const void* src, long lds, void* dst, int H,
                  const int* mtp_am, int* draft0, void* stream);

/* Measurement hook, no counterpart in the reference: in verify mode (ctl[2] == 1) overwrite the k
 * drafts in_tok[1..k] so that exactly `a` are accepted: draft j (position pos + 1 + j) becomes
 * truth[pos + 1 + j] for j < a and (truth + 1) mod vocab otherwise. a < 0 does nothing. */
int qe_force_drafts(int* in_tok, const int* ctl, const int* truth, int truth_len, int a, int k,
                    int vocab, void* stream);

/* ------------------------------------------------------------------------------------------
 * Gated DeltaNet step for n new rows with lazy rollback (csrc/ops.h:20-24, csrc/gdn.cu).
 * D = key head dim = value head dim (64 or 128; the reference fixes 128, csrc/bindings.cpp:133).
 * S fp32 [Hv, D, D]; ring bf16 [16, C] with C = 2*Hk*D + Hv*D; st_k, st_v fp32 [8, Hv, D];
 * st_g fp32 [8, Hv, 2]. `q` (the reference's thread-split knob) is accepted and ignored.
 * ------------------------------------------------------------------------------------------ */
int qe_gdn_step_n(const void* qkv, const void* z, const void* b, const void* a, long ldp,
                  void* ring, const void* conv_w, const void* A_log, const void* dt_bias,
                  const void* norm_w, float* S, float* st_k, float* st_v, float* st_g,
                  const int* ctl, void* out, long ldo, int n, int Hk, int Hv, int D, float eps,
                  int q, void* stream);

/* ------------------------------------------------------------------------------------------
 * Gated GQA attention for n rows at positions pos[0] + t (csrc/ops.h:25-30, csrc/attn.cu).
 * hd = head dim (64, 128 or 256; the reference fixes 256, csrc/bindings.cpp:155).
 * ------------------------------------------------------------------------------------------ */

/* q/k RMSNorm1p per head, partial RoPE on the first rd dims, q -> q_out [n, Hq*hd] (contiguous),
 * k, v -> caches [Hkv, max_len, hd] at pos + t (skipped when pos + t >= max_len).
 * Replaces launch_attn_prep (csrc/ops.h:25-27). */
int qe_attn_prep(const void* qg, const void* k, const void* v, long ldp, const void* qnw,
                 const void* knw, const float* inv_freq, const int* pos, void* q_out, void* kc,
                 void* vc, int n, int Hq, int Hkv, int hd, int max_len, int rd, float eps,
                 void* stream);

/* Split-KV flash decoding + combine + sigmoid gate. part_o fp32 [>=n, Hq, NS, hd], part_ml fp32
 * [>=n, Hq, NS, 2], 1 <= NS <= 1024. hd == 256 with NS a multiple of 6 runs the tensor-core split
 * kernel (long caches), otherwise the shared-memory-ring kernel. Rows are independent: row t of an
 * n-row call equals the 1-row call at pos + t. Replaces launch_attn_decode (csrc/ops.h:28-30). */
int qe_attn_decode(const void* q, const void* kc, const void* vc, const int* pos, const void* qg,
                   long ldp, float* part_o, float* part_ml, void* out, long ldo, int n, int Hq,
                   int Hkv, int hd, int max_len, int NS, float scale, void* stream);
/* Sticky error word of the attention ring waits (0 = none, 1 producer, 2 consumer wait ran out);
 * synchronises. No counterpart in the reference. */
int qe_attn_error(void);

/* ------------------------------------------------------------------------------------------
 * Run-time switches and L2 controls (csrc/ops.h:31-36).
 * ------------------------------------------------------------------------------------------ */
void qe_set_pdl_trigger(int on); /* kernels signal griddepcontrol.launch_dependents */
void qe_set_pdl_launch(int on);  /* own kernels launch with programmatic stream serialization */
void qe_set_gdn_early(int on);   /* DeltaNet kernel: state replay before the dependency wait */
void qe_set_gdn_phases(int on);  /* accepted for compatibility; the kernel has a single path */
int qe_l2_persist_limit(size_t bytes);
int qe_stream_access_window(uintptr_t base, size_t bytes, float hit_ratio, void* stream);

/* ------------------------------------------------------------------------------------------
 * W4A16 GEMV / skinny GEMM: out[n, m] = bf16(sum_g scale[m, g] * sum_{k in g} (u[m,k]-8) x[n,k]).
 * Reference: csrc/gemv_w4.h:9-55 (GemvParams, LaunchCfg, LaunchPlan, plan_gemv_w4, auto_ksplit,
 * launch_gemv_w4). Packed layout (python/qengine/quant.py:1-30):
 *   qw     int32 [Mp/16, Kp/64, 32, 4]   (16-row tile, 64-k chunk, lane, word)
 *   scales fp16  [Mp/16, Kp/128, 16]
 * ------------------------------------------------------------------------------------------ */
enum { QE_EPI_NONE = 0, QE_EPI_SWIGLU = 1 };

typedef struct qe_w4_params {
  const void* qw;      /* packed int4 weights (16-byte aligned) */
  const void* scales;  /* fp16 group scales (16-byte aligned) */
  const void* x;       /* bf16 activations, N rows, stride ldx; any alignment (16-byte aligned rows
                          with ldx % 8 == 0 take the vector path). Ignored by qe_w4_gemv_ex when a
                          prologue is given. */
  void* out;           /* bf16 output, N rows, stride ldo */
  float* ws;           /* fp32 partial-sum slots, qe_w4_plan::ws_floats entries; zero before the
                          first call, left zero by every call (like `counters`) */
  int* counters;       /* int32 arrival counters, qe_w4_plan::counters entries, zero between calls */
  int M;               /* logical output rows (QE_EPI_SWIGLU: intermediate size I) */
  int K;               /* logical reduction length, Kp - 128 < K <= Kp */
  int Mp, Kp;          /* padded sizes (multiples of 16 / 128) */
  int N;               /* activation rows, 1..8 (qe_w4_gemm: 1..QE_MAX_GEMM_ROWS) */
  long ldx, ldo;
  int epilogue;        /* QE_EPI_* */
  int out_f32;         /* 0: out is bf16 (the reference's contract). 1 (plain epilogue only): out is
                          fp32, ldo in floats, sums stored unrounded -- the partial sums of a matrix
                          split along K over tensor-parallel ranks. No counterpart in the reference. */
  int x_f16;           /* 0: x is bf16 (the reference's contract). 1: x holds fp16 rows (same strides in
                          elements); needs K == Kp, 16-byte aligned rows and ldx % 8 == 0, else
                          QE_ERR_ARG. The kernel then unpacks the codes to fp16 (one shift per word
                          instead of three). For values that fp16 holds exactly -- bf16 numbers of
                          magnitude 2^-17 .. 65504, e.g. rows normalised by qe_w4_norm_rows -- the
                          result has the bits of the bf16 path. No counterpart in the reference. */
} qe_w4_params;

/* Launch options with the reference's names (csrc/gemv_w4.h:27-39). 0 / -1 mean "auto by shape".
 * One kernel family serves every shape, so most of them only steer its geometry; every accepted
 * combination is deterministic and independent of N. */
typedef struct qe_w4_cfg {
  int warps;         /* warps per block: 0 (auto) / 16 -> 16, 4 / 8 -> 8 */
  int unroll;        /* ring of 1-KB weight units per warp: 4 -> 2 stages of 4, 2 -> 3 stages of 2,
                        1 -> 2 stages of 2, 0 -> the deepest that fits (never changes the result) */
  int ksplit;        /* > 0: at least this many warps share a 16-row tile; 0 = by min_units */
  int pdl;           /* launch with programmatic stream serialization */
  int variant;       /* 1: 24 warps per block, 2: 20 warps; other values: as `warps` says */
  int mode;          /* accepted for compatibility (-1, 0, 2, 3, 4); the plan always reports 4 */
  int blocks_per_sm; /* accepted for compatibility; the kernel runs one block per SM */
  int min_units;     /* minimum 1-KB units per warp (fewer warps for small matrices) */
} qe_w4_cfg;

typedef struct qe_w4_plan {
  int mode;
  int grid_x, grid_y, threads;
  long ws_floats; /* required size of qe_w4_params::ws */
  long counters;  /* required size of qe_w4_params::counters */
} qe_w4_plan;

/* Optional work fused into the GEMV launch; no counterpart in the reference, whose engine runs
 * launch_rmsnorm1p (csrc/ops.h:8-9) and launch_embed (csrc/ops.h:6-7) as kernels of their own in
 * front of launch_gemv_w4 (python/qengine/engine.py:434-466).
 *   Prologue (h_in != NULL): the GEMV input is x = RMSNorm1p(h_in + delta) * (1 + norm_w), with
 *   the arithmetic of qe_rmsnorm1p (bf16 residual sum, fp32 statistics, one rounding), computed
 *   by every block into shared memory. h_out (optional) receives bf16(h_in + delta), xn_out
 *   (optional) receives x; both are written by one block. h_out must not alias h_in. With tok !=
 *   NULL, h_in is an embedding table [vocab, K] and row r is table[tok[r]] (zeros when out of
 *   range). Needs K == Kp, 16-byte aligned rows, row strides that are multiples of 8, and
 *   N * (2 K + 16) bytes of shared memory beside the weight rings (QE_ERR_ARG otherwise: run
 *   qe_rmsnorm1p and qe_w4_gemv instead).
 *   f16 != 0: the normalised rows (rounded to bf16 as always) are kept as fp16 in shared memory and
 *   the GEMV runs its fp16 flavour (see qe_w4_params::x_f16). A normalised element is at most
 *   sqrt(K) * |1 + norm_w| in magnitude: the caller checks its norm weights once. xn16_out
 *   (qe_w4_norm_rows only, optional): fp16 copy of the normalised rows [N, K], stride ldx16, the
 *   input of a qe_w4_gemv with x_f16 = 1 that then equals the fused launch bit for bit. */
typedef struct qe_w4_norm {
  const void* h_in;    /* bf16 [N, K] rows (stride ldh), or the embedding table when tok != NULL */
  const int* tok;      /* optional token ids [N] */
  int vocab;           /* rows of the table (tok != NULL) */
  const void* delta;   /* optional bf16 [N, K] residual update, stride ldd */
  const void* norm_w;  /* bf16 [K] */
  void* h_out;         /* optional bf16 [N, K], stride ldho */
  void* xn_out;        /* optional bf16 [N, K], stride ldxo */
  long ldh, ldd, ldho, ldxo;
  float eps;
  int f16;             /* fused prologue: fp16 activations, see above */
  void* xn16_out;      /* qe_w4_norm_rows: optional fp16 [N, K] */
  long ldx16;
} qe_w4_norm;

/* Default-initialise a cfg (all auto, pdl on, min_units 4). */
void qe_w4_cfg_default(qe_w4_cfg* cfg);
/* Resolve the launch for a shape; never depends on N. Replaces plan_gemv_w4 (gemv_w4.h:50). */
int qe_w4_plan_gemv(const qe_w4_params* p, const qe_w4_cfg* cfg, qe_w4_plan* plan);
/* Replaces auto_ksplit (gemv_w4.h:53). */
int qe_w4_auto_ksplit(int Mp, int Kp, int N, int warps);
/* Replaces launch_gemv_w4 (gemv_w4.h:56). */
int qe_w4_gemv(const qe_w4_params* p, const qe_w4_cfg* cfg, void* stream);
/* qe_w4_gemv with the fused prologue described at qe_w4_norm (nrm may be NULL). */
int qe_w4_gemv_ex(const qe_w4_params* p, const qe_w4_norm* nrm, const qe_w4_cfg* cfg, void* stream);
/* The prologue of qe_w4_gemv_ex as a launch of its own: xn_out[r] = RMSNorm1p(h_in[r] + delta[r]) *
 * (1 + norm_w) and h_out[r] = bf16(h_in[r] + delta[r]) for r < N, one block per row, with exactly
 * the arithmetic (thread map, reduction order) the GEMV selected by `cfg` uses in its prologue:
 * running this and then qe_w4_gemv on xn_out gives the bits of qe_w4_gemv_ex. For passes of
 * several rows, where N blocks in parallel beat every GEMV block repeating the work for all rows.
 * N = 1..QE_MAX_GEMM_ROWS (the rows of a qe_w4_gemm pass).
 * h_out may alias h_in here; xn_out is required. K % 8 == 0. Semantics of launch_rmsnorm1p
 * (csrc/ops.h:8-9). */
int qe_w4_norm_rows(const qe_w4_norm* nrm, int N, int K, const qe_w4_cfg* cfg, void* stream);
/* Up to QE_W4_MAX_CHAIN GEMVs that depend on one another only through device memory (the output
 * of one is the input or the residual update of the next) as ONE cooperative launch: job j + 1
 * starts after a grid-wide barrier that follows job j, and every warp requests the head of its
 * slab of the next matrix before it reaches the barrier, so the memory pipeline does not drain
 * between the jobs the way it does between two kernel launches. Same results, bit for bit, as the
 * same calls made one by one with the same cfg. All jobs use `cfg`; p[j]->ws / counters must cover
 * the largest plan of the chain (they are reused job after job). gridbar: two int32 words in
 * device memory, zero before the first use, owned by the library afterwards (one pair per stream
 * of launches). nrm may be NULL, and so may any nrm[j]. njobs == 1 is qe_w4_gemv_ex. No
 * counterpart in the reference, which launches every GEMV separately. */
#define QE_W4_MAX_CHAIN 4
int qe_w4_gemv_chain(const qe_w4_params* const* p, const qe_w4_norm* const* nrm, int njobs,
                     const qe_w4_cfg* cfg, int* gridbar, void* stream);
/* Has no counterpart in the reference. The same GEMV as qe_w4_gemv for callers that cannot
 * allocate device memory (a plugin inside another runtime's callback, code running between the
 * capture and the replay of a graph, an embedder that may not call its allocator): p->ws and
 * p->counters are ignored and the scratch comes from a fixed array inside the library instead,
 * QE_W4_STATIC_WS_FLOATS fp32 slots + QE_W4_STATIC_COUNTERS counters (about 4.1 MiB per GPU, held
 * until exit). A shape / configuration whose plan needs more returns QE_ERR_SCRATCH. The first
 * call on a device looks the array's device address up (make it before any stream capture);
 * nothing is ever allocated or freed. All calls share the array: calls that overlap on the GPU
 * race, so keep them on one stream. `cfg->pdl` is ignored (plain stream order). */
#define QE_W4_STATIC_WS_FLOATS (1L << 20)
#define QE_W4_STATIC_COUNTERS (1L << 14)
#define QE_ERR_SCRATCH (-28)
int qe_w4_gemv_static(const qe_w4_params* p, const qe_w4_cfg* cfg, void* stream);

/* Has no counterpart in the reference, which prefills in passes of at most 8 rows through its GEMV
 * (python/qengine/engine.py:558-573). The same product as qe_w4_gemv for p->N = 1..QE_MAX_GEMM_ROWS
 * activation rows with the matrix streamed from HBM once for all of them: a prefill pass of 64
 * rows reads the weights once instead of eight times. Same wire format, epilogues and out_f32 as
 * qe_w4_gemv. Default kernel (cfg->variant != 1): tcgen05.mma with the accumulator in tensor
 * memory -- per 128-k group the exact integer dot products, scaled in fp32 and added group by
 * group in ascending order, i.e. the GEMV's arithmetic with another order of additions, so a row
 * agrees with qe_w4_gemv to fp32 rounding (not bit for bit); results are bit-identical run to run
 * and row r does not depend on N. cfg->variant == 1: an mma.sync kernel (needs Kp / 128 even).
 * Needs K == Kp, bf16 x with 16-byte aligned rows and ldx % 8 == 0 (QE_ERR_ARG otherwise);
 * p->x_f16 must be 0. Matrices of few rows (fewer 128-row super-tiles than half the SMs) are also
 * split along K; their partial sums meet in p->ws / p->counters, sized by qe_w4_plan_gemm (any
 * contents in ws; counters zero before the first call, left zero). With either pointer NULL the
 * split is skipped (same result up to fp32 rounding of the order of additions, fewer SMs busy).
 * Of cfg only pdl and variant are read. */
#define QE_MAX_GEMM_ROWS 64
int qe_w4_plan_gemm(const qe_w4_params* p, const qe_w4_cfg* cfg, qe_w4_plan* plan);
int qe_w4_gemm(const qe_w4_params* p, const qe_w4_cfg* cfg, void* stream);

/* The weight rings are fed by bulk copies whose completion waits are bounded; this returns the
 * sticky error word those waits set on expiry (0 = none) and qe_w4_clear_error resets it. Both
 * synchronise with the device. No counterpart in the reference. */
int qe_w4_ring_error(void);
int qe_w4_clear_error(void);

#ifdef __cplusplus
}
#endif
#endif /* QENGINE_B200_H_ */
