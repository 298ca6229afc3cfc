// One row of the top-k block selection, done by one warp.
#pragma once

#include "common.cuh"

namespace dfs {

// float -> unsigned key with the same order (larger score <-> larger key)
__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// `src`: the row's n_cols fp32 scores (global or shared memory; unused for a dense row); `keys`: n_rank words of
// shared memory private to the warp.  Writes the ascending list out[0 .. kmax), its count, and optionally the
// row of the bool mask.  Exact and deterministic:
//   1. the k-th largest score is found by building its order-preserving 32-bit key from the most significant
//      bit down: a bit stays set when at least k candidates are >= the key built so far (up to 32 counting
//      passes over the row's keys, warp-reduced; the search stops early once exactly k candidates are >= the
//      key built so far, which then separates the k largest from the rest as well as the full key would);
//   2. every candidate above that threshold is selected, plus as many candidates EQUAL to it as are still
//      needed, lowest column first (the tie rule);
//   3. columns at or past n_rank are always selected ("forced": the text / boundary key blocks); a dense row
//      selects every column: when kmax has room for every column they are listed, otherwise the row gets the
//      count -1 ("every key block") and no list;
//   4. the list is written in ascending column order by an ordered warp compaction (ballot + popc), padded
//      with -1.
__device__ __forceinline__ void select_row_warp(const float* src, uint32_t* keys, int n_cols, int n_rank,
                                                int k_select, bool dense, int kmax, int32_t* __restrict__ out,
                                                int32_t* __restrict__ cnt_out, uint8_t* __restrict__ mrow,
                                                int lane) {
  const unsigned lt_mask = (1u << lane) - 1u;
  if (dense && kmax < n_cols) {  // marker row: every key block, nothing listed
    for (int pos = lane; pos < kmax; pos += 32) out[pos] = -1;
    if (mrow)
      for (int c = lane; c < n_cols; c += 32) mrow[c] = 1;
    if (lane == 0) *cnt_out = -1;
    return;
  }

  uint32_t thr = 0;  // key of the k-th largest candidate
  int need_eq = 0;   // how many candidates equal to it are selected
  if (!dense && k_select > 0) {
    for (int c = lane; c < n_rank; c += 32) keys[c] = order_key(src[c]);
    __syncwarp();
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = thr | (1u << bit);
      int local = 0;
      for (int c = lane; c < n_rank; c += 32) local += keys[c] >= cand;
      const int at_least = __reduce_add_sync(0xffffffffu, local);
      if (at_least >= k_select) thr = cand;
      if (at_least == k_select) break;  // exactly the k largest are >= thr: the lower bits cannot change the set
    }
    int gt = 0;
    for (int c = lane; c < n_rank; c += 32) gt += keys[c] > thr;
    need_eq = k_select - __reduce_add_sync(0xffffffffu, gt);
  }

  int written = 0, eq_seen = 0;
  for (int c0 = 0; c0 < n_cols; c0 += 32) {
    const int c = c0 + lane;
    const bool in_row = c < n_cols;
    const bool ranked = in_row && !dense && c < n_rank && k_select > 0;
    const uint32_t kc = ranked ? keys[c] : 0u;
    const bool eq = ranked && kc == thr;
    const unsigned eq_ballot = __ballot_sync(0xffffffffu, eq);
    const bool sel = in_row && (dense || c >= n_rank ||
                                (ranked && (kc > thr || (eq && eq_seen + __popc(eq_ballot & lt_mask) < need_eq))));
    eq_seen += __popc(eq_ballot);
    if (in_row && mrow) mrow[c] = sel ? 1 : 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, sel);
    if (sel) {
      const int pos = written + __popc(ballot & lt_mask);
      if (pos < kmax) out[pos] = c;
    }
    written += __popc(ballot);
  }
  for (int pos = written + lane; pos < kmax; pos += 32) out[pos] = -1;
  if (lane == 0) *cnt_out = written < kmax ? written : kmax;
}

// The same selection with the row's keys held in registers (kPerLane per lane, column c <-> key c / 32 of lane
// c % 32), for rows of at most 32 * kPerLane ranked columns: the 32 counting passes then run without a
// memory access.  Results are identical to select_row_warp's.
template <int kPerLane>
__device__ __forceinline__ void select_row_warp_regs(const float* src, int n_cols, int n_rank, int k_select,
                                                     bool dense, int kmax, int32_t* __restrict__ out,
                                                     int32_t* __restrict__ cnt_out, uint8_t* __restrict__ mrow,
                                                     int lane) {
  const unsigned lt_mask = (1u << lane) - 1u;
  if (dense && kmax < n_cols) {
    for (int pos = lane; pos < kmax; pos += 32) out[pos] = -1;
    if (mrow)
      for (int c = lane; c < n_cols; c += 32) mrow[c] = 1;
    if (lane == 0) *cnt_out = -1;
    return;
  }
  const bool rank = !dense && k_select > 0;
  uint32_t key[kPerLane];  // 0 past the ranked columns: below every threshold candidate, never counted
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int c = i * 32 + lane;
    key[i] = (rank && c < n_rank) ? order_key(src[c]) : 0u;
  }
  uint32_t thr = 0;
  int need_eq = 0;
  if (rank) {
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = thr | (1u << bit);
      int local = 0;
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) local += key[i] >= cand;
      const int at_least = __reduce_add_sync(0xffffffffu, local);
      if (at_least >= k_select) thr = cand;
      if (at_least == k_select) break;  // exactly the k largest are >= thr: the lower bits cannot change the set
    }
    int gt = 0;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) gt += (i * 32 + lane < n_rank) && key[i] > thr;
    need_eq = k_select - __reduce_add_sync(0xffffffffu, gt);
  }

  int written = 0, eq_seen = 0;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    if (i * 32 < n_cols) {  // warp-uniform
      const int c = i * 32 + lane;
      const bool in_row = c < n_cols;
      const bool ranked = in_row && rank && c < n_rank;
      const bool eq = ranked && key[i] == thr;
      const unsigned eq_ballot = __ballot_sync(0xffffffffu, eq);
      const bool sel =
          in_row && (dense || c >= n_rank ||
                     (ranked && (key[i] > thr || (eq && eq_seen + __popc(eq_ballot & lt_mask) < need_eq))));
      eq_seen += __popc(eq_ballot);
      if (in_row && mrow) mrow[c] = sel ? 1 : 0;
      const unsigned ballot = __ballot_sync(0xffffffffu, sel);
      if (sel) {
        const int pos = written + __popc(ballot & lt_mask);
        if (pos < kmax) out[pos] = c;
      }
      written += __popc(ballot);
    }
  }
  for (int c0 = kPerLane * 32; c0 < n_cols; c0 += 32) {  // columns past the registers: all forced (or dense)
    const int c = c0 + lane;
    const bool sel = c < n_cols;
    if (sel && mrow) mrow[c] = 1;
    const unsigned ballot = __ballot_sync(0xffffffffu, sel);
    if (sel) {
      const int pos = written + __popc(ballot & lt_mask);
      if (pos < kmax) out[pos] = c;
    }
    written += __popc(ballot);
  }
  for (int pos = written + lane; pos < kmax; pos += 32) out[pos] = -1;
  if (lane == 0) *cnt_out = written < kmax ? written : kmax;
}

// Rows of up to kRegisterRankMax ranked columns are selected from registers, longer ones from `keys`
// (n_rank words of shared memory private to the warp; may be null for the short rows).
constexpr int kRegisterRankMax = 1024;

__device__ __forceinline__ void select_row(const float* src, uint32_t* keys, int n_cols, int n_rank, int k_select,
                                           bool dense, int kmax, int32_t* __restrict__ out,
                                           int32_t* __restrict__ cnt_out, uint8_t* __restrict__ mrow, int lane) {
  if (n_rank <= 256)
    select_row_warp_regs<8>(src, n_cols, n_rank, k_select, dense, kmax, out, cnt_out, mrow, lane);
  else if (n_rank <= 512)
    select_row_warp_regs<16>(src, n_cols, n_rank, k_select, dense, kmax, out, cnt_out, mrow, lane);
  else if (n_rank <= kRegisterRankMax)
    select_row_warp_regs<32>(src, n_cols, n_rank, k_select, dense, kmax, out, cnt_out, mrow, lane);
  else
    select_row_warp(src, keys, n_cols, n_rank, k_select, dense, kmax, out, cnt_out, mrow, lane);
}

// The argument rules of a selection (shared by both entry points); 0 or a DFS_ERR_* code.
static inline int dfs_check_selection(int heads, int score_rows, int q_rows, int n_cols, int n_rank, int k_select,
                                      int* dense_row_start, int kmax) {
  if (heads <= 0 || q_rows <= 0 || n_cols <= 0 || score_rows < 0) return DFS_ERR_SHAPE;
  if (n_rank < 0 || n_rank > n_cols) return DFS_ERR_RANGE;
  if (k_select < 0 || k_select > n_rank) return DFS_ERR_RANGE;
  if (*dense_row_start < 0) return DFS_ERR_RANGE;
  if (*dense_row_start > q_rows) *dense_row_start = q_rows;
  if (*dense_row_start > score_rows) return DFS_ERR_RANGE;  // a ranked row needs its scores
  // every ranked row's list must fit; dense rows are listed only when kmax >= n_cols (else count -1)
  const int sparse_cnt = k_select + (n_cols - n_rank);
  if (kmax < sparse_cnt || kmax <= 0) return DFS_ERR_RANGE;
  return 0;
}

}  // namespace dfs
