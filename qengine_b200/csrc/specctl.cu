// Device-side bookkeeping of a decode / verify pass, so that a whole speculative cycle is one
// CUDA graph with no host round trip: greedy longest-prefix acceptance, commit, MTP position and
// row selection. Integer state only; results are a pure function of (in_tok, am, ctl) and must be
// bit-exact against the reference (csrc/basic.cu:241-307: accept_kernel, commit_kernel,
// mtp_select_kernel) and against the CPU restatement used by the tests.
//
// ctl (int32): [0] pos = position of in_tok[0]; [1] pending = DeltaNet rows staged by the last
// pass and kept; [2] mode (0 prefill, 1 decode/verify); [3] m = index of the last kept row;
// [4] cycles; [5] accepted drafts; [16 + m] histogram of m.
#include "common.cuh"
#include "../../include/qengine_b200.h"

namespace qb {
namespace {

// One thread: acceptance of a pass over n rows. Returns m, the index of the last kept row.
__device__ __forceinline__ int accept_rows(const int* in_tok, const int* am, int n, int* ctl, int* next_tok,
                                           int* log, int max_len) {
  const int pos = ctl[0], mode = ctl[2];
  int m;
  if (mode == 1) {
    // rows 0..m are correct: draft i+1 (= in_tok[i+1]) equals the target's token am[i]
    m = 0;
    while (m + 1 < n && in_tok[m + 1] == am[m]) ++m;
    for (int i = 0; i <= m; ++i)
      if (pos + 1 + i < max_len) log[pos + 1 + i] = am[i];
    ctl[4] += 1;
    ctl[5] += m;
    ctl[16 + m] += 1;
    for (int r = 0; r < n; ++r) next_tok[r] = am[r];
  } else {
    // prefill: every row is a given token; the last chunk (in_tok[n] < 0) emits the first token
    m = n - 1;
    const int follow = in_tok[n];
    if (follow < 0 && pos + n < max_len) log[pos + n] = am[n - 1];
    for (int r = 0; r + 1 < n; ++r) next_tok[r] = in_tok[r + 1];
    next_tok[n - 1] = follow >= 0 ? follow : am[n - 1];
  }
  ctl[3] = m;
  return m;
}

// One thread: the kept rows become the sequence, the next pass starts from the model's token.
__device__ __forceinline__ void commit_rows(int m, int* ctl, int* in_tok, const int* am, const int* drafts, int k) {
  ctl[0] += m + 1;
  ctl[1] = m + 1;
  in_tok[0] = am[m];
  for (int j = 0; j < k; ++j) in_tok[1 + j] = drafts[j];
}

__global__ void accept_rows_kernel(const int* in_tok, const int* am, int n, int* ctl, int* next_tok, int* log,
                                   int max_len) {
  dep_release();
  dep_wait();
  if (threadIdx.x == 0) accept_rows(in_tok, am, n, ctl, next_tok, log, max_len);
}

__global__ void commit_rows_kernel(int* ctl, int* in_tok, const int* am, const int* drafts, int k) {
  dep_release();
  dep_wait();
  if (threadIdx.x == 0) commit_rows(ctl[3], ctl, in_tok, am, drafts, k);
}

// A pass without draft rows (plain decode, prefill) has nothing between acceptance and commit:
// both in one launch.
__global__ void accept_commit_kernel(int* in_tok, const int* am, int n, int* ctl, int* next_tok, int* log,
                                     int max_len, const int* drafts, int k) {
  dep_release();
  dep_wait();
  if (threadIdx.x != 0) return;
  const int m = accept_rows(in_tok, am, n, ctl, next_tok, log, max_len);
  commit_rows(m, ctl, in_tok, am, drafts, k);
}

// End of a chained draft pass (one row): the drafted token joins the draft list and the draft
// layer's output row becomes the hidden input of the next chained pass.
__global__ void chain_draft_kernel(const int* mtp_am, int* draft_out, const bf16* src, bf16* dst, int H) {
  dep_release();
  dep_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) draft_out[0] = mtp_am[0];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

__global__ void mtp_select_rows_kernel(const int* ctl, int* mpos, int off,
                                       const bf16* src, long lds,
                                       bf16* dst, int H, const int* mtp_am,
                                       int* draft0) {
  dep_release();
  dep_wait();
  const int m = ctl[3];
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    mpos[0] = off < 0 ? ctl[0] : ctl[0] + m + 1 + off;
    if (draft0) draft0[0] = mtp_am[m];
  }
  if (src) {
    const bf16* row = src + (long)m * lds;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x)
      dst[i] = row[i];
  }
}

// Measurement hook (no counterpart in the reference): before a verify pass, overwrite the k
// drafts so that exactly `a` of them will be accepted. truth[p] is the known greedy token at
// position p; draft j sits at position pos + 1 + j and becomes truth[p] for j < a and
// (truth[p] + 1) mod vocab otherwise. a < 0 leaves the drafts alone. Only acts in verify mode.
__global__ void force_drafts_kernel(int* in_tok, const int* ctl,
                                    const int* truth, int truth_len, int a, int k,
                                    int vocab) {
  dep_release();
  dep_wait();
  if (threadIdx.x != 0 || a < 0 || ctl[2] != 1) return;
  const int pos = ctl[0];
  for (int j = 0; j < k; ++j) {
    const int p = pos + 1 + j;
    const int t = (p >= 0 && p < truth_len) ? truth[p] : 0;
    in_tok[1 + j] = j < a ? t : (t + 1) % vocab;
  }
}

inline bool pdl_on() { return pdl_launch_enabled() && pdl_trigger_enabled(); }

}  // namespace
}  // namespace qb

using namespace qb;

extern "C" int qe_accept(const int* in_tok, const int* am, int n, int* ctl, int* next_tok, int* log,
                         int max_len, void* stream) {
  if (n < 1 || n > QE_MAX_ROWS) return QE_ERR_ARG;
  return (int)launch(accept_rows_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, pdl_on(), in_tok,
                     am, n, ctl, next_tok, log, max_len);
}

extern "C" int qe_commit(int* ctl, int* in_tok, const int* am, const int* drafts, int k,
                         void* stream) {
  if (k < 0 || k >= QE_MAX_ROWS) return QE_ERR_ARG;
  return (int)launch(commit_rows_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, pdl_on(), ctl,
                     in_tok, am, drafts, k);
}

extern "C" int qe_accept_commit(int* in_tok, const int* am, int n, int* ctl, int* next_tok, int* log,
                                int max_len, const int* drafts, int k, void* stream) {
  if (n < 1 || n > QE_MAX_ROWS || k < 0 || k >= QE_MAX_ROWS) return QE_ERR_ARG;
  return (int)launch(accept_commit_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, pdl_on(), in_tok, am, n,
                     ctl, next_tok, log, max_len, drafts, k);
}

extern "C" int qe_chain_draft(const int* mtp_am, int* draft_out, const void* src, void* dst, int H,
                              void* stream) {
  if (H < 1) return QE_ERR_ARG;
  return (int)launch(chain_draft_kernel, dim3((H + 255) / 256), dim3(256), 0, (cudaStream_t)stream, pdl_on(),
                     mtp_am, draft_out, (const bf16*)src, (bf16*)dst, H);
}

extern "C" int qe_mtp_select(const int* ctl, int* mpos, int off, const void* src, long lds, void* dst,
                             int H, const int* mtp_am, int* draft0, void* stream) {
  const int blocks = src ? (H + 255) / 256 : 1;
  return (int)launch(mtp_select_rows_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream,
                     pdl_on(), ctl, mpos, off, (const bf16*)src, lds, (bf16*)dst, H, mtp_am, draft0);
}

extern "C" int qe_force_drafts(int* in_tok, const int* ctl, const int* truth, int truth_len, int a,
                               int k, int vocab, void* stream) {
  if (k < 0 || k >= QE_MAX_ROWS || vocab < 1) return QE_ERR_ARG;
  return (int)launch(force_drafts_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, pdl_on(), in_tok,
                     ctl, truth, truth_len, a, k, vocab);
}
