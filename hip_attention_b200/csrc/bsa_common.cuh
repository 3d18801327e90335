// Shared pieces of the block-sparse attention kernels: the key list of a query block and the
// per-(row, key) admission rule.
//
// A query block attends three groups of keys, concatenated into one virtual list
//   [ sink tokens | selected blocks (ks blocks of block_size_k tokens) | window tokens ]
// which the kernels walk in tiles.  For a query row at position p (the block's largest position is
// pmax) a key at position t is admitted when
//   sink / selected entry ("far" keys):  t <= p - window
//   window entry:                        p - window < t <= p
// and a selected entry must also satisfy sink <= t <= pmax and t < T; sink and window entries are cut at T
// as well (query positions beyond the keys set HIPATTN_STATUS_TOKEN_RANGE).  The two rules are disjoint,
// so a token that appears in two groups is counted once.
#pragma once
#include "common.cuh"

namespace hipattn {

struct KeyList {
  int n_sink, n_sel, n_win, w_start, total;
  int pmax, pmin;
  const int64_t* idx;  // selected block starts of this query block
  int block_k, sink, T;
  int block_k_shift;   // log2(block_k) when it is a power of two, else -1
  int sink_floor;      // sink rounded down to whole blocks: the rank of the first selected entry under in-kernel RoPE
};

__device__ __forceinline__ KeyList make_key_list(const hipattn_bsa_params_t& p, int b, int h, int d, int pmin, int pmax) {
  KeyList kl;
  const int64_t n = (int64_t)b * p.H + h;
  const int d_idx = (int)(((int64_t)d * p.block_size_q) / p.index_block_q);
  kl.idx = p.indices + n * p.idx_stride_n + (int64_t)d_idx * p.idx_stride_d;
  long long ks = p.ks[n * p.ks_stride_n + (int64_t)d_idx * p.ks_stride_d];
  ks = ks < 0 ? 0 : (ks > p.K ? p.K : ks);
  kl.block_k = p.block_size_k;
  kl.block_k_shift = (p.block_size_k & (p.block_size_k - 1)) == 0 ? 31 - __clz(p.block_size_k) : -1;
  kl.sink = p.sink;
  kl.sink_floor = (p.sink / p.block_size_k) * p.block_size_k;
  kl.T = p.T;
  kl.pmax = pmax;
  kl.pmin = pmin;
  // Sink and window entries are positions, not table entries: keep them below T.  With dense K / V a
  // query position at or beyond T would otherwise address rows past the end of the tensors (a paged
  // cache maps such positions to page 0 by itself).  The clamp is reported, not silent.
  const int t_end = min(pmax + 1, p.T);
  if (pmax >= p.T && p.k.cache == nullptr && p.status && threadIdx.x == 0) atomicOr(p.status, HIPATTN_STATUS_TOKEN_RANGE);
  kl.n_sink = max(0, min(p.sink, t_end));
  kl.n_sel = (int)ks * p.block_size_k;
  kl.w_start = max(0, pmin - p.window + 1);
  kl.n_win = p.window > 0 ? max(0, t_end - kl.w_start) : 0;
  kl.total = kl.n_sink + kl.n_sel + kl.n_win;
  return kl;
}

// Index into kl.idx of the selected block that holds entry j, or -1 when j is not a selected entry.
__device__ __forceinline__ int selected_block_of(const KeyList& kl, int j) {
  j -= kl.n_sink;
  if (j < 0 || j >= kl.n_sel) return -1;
  return kl.block_k_shift >= 0 ? (j >> kl.block_k_shift) : (j / kl.block_k);
}

// Position of entry j of the virtual list, or -1 when the entry admits no row.  *is_window tells
// which admission rule applies.  `start` is kl.idx[selected_block_of(kl, j)] for a selected entry (unused otherwise);
// callers that fetched it ahead of time pass it in, so that no global load sits in this function.
__device__ __forceinline__ int key_position_at(const KeyList& kl, int j, long long start, bool* is_window) {
  *is_window = false;
  if (j < 0 || j >= kl.total) return -1;
  if (j < kl.n_sink) return j;
  j -= kl.n_sink;
  if (j < kl.n_sel) {
    const int blk = kl.block_k_shift >= 0 ? (j >> kl.block_k_shift) : (j / kl.block_k);
    const long long t = start + (j - blk * kl.block_k);
    if (t < kl.sink || t > kl.pmax || t >= kl.T) return -1;
    return (int)t;
  }
  j -= kl.n_sel;
  *is_window = true;
  return kl.w_start + j;
}

__device__ __forceinline__ int key_position(const KeyList& kl, int j, bool* is_window) {
  const int blk = selected_block_of(kl, j);
  return key_position_at(kl, j, blk >= 0 ? kl.idx[blk] : 0, is_window);
}

// Table position the key at entry j (position t) is rotated to by the attention's in-kernel RoPE, backend
// "streaming" (attention_extend_bsa.py:256-270, 1120, 1359): window keys keep their own position; sink and selected
// keys get their rank in the list [sink | selected blocks] shifted by pmin - window - sink - (selected tokens) + 1,
// floored at 0 (pmin = smallest query position of the attention block).
__device__ __forceinline__ int rope_key_position(const KeyList& kl, int j, int t, int window) {
  if (j >= kl.n_sink + kl.n_sel) return t;
  const int shift = kl.pmin - window - kl.sink - kl.n_sel + 1;
  // a selected entry's rank is (its block + sink / block_k) * block_k + its place in the block = its place among the
  // selected entries + the sink rounded down to whole blocks
  const int rank = j < kl.n_sink ? t : (j - kl.n_sink) + kl.sink_floor;
  return max(0, rank + shift);
}

__device__ __forceinline__ bool admits(int p_row, int t, bool is_window, int window) {
  if (t < 0) return false;
  return is_window ? (t > p_row - window && t <= p_row) : (t <= p_row - window);
}

}  // namespace hipattn
