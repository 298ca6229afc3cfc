// Per-row top-k key-block selection -> ascending index lists.
//
// One warp per (query-block row, head).  Exact and deterministic:
//   1. the k-th largest score is found by building its order-preserving 32-bit
//      key from the most significant bit down: a bit stays set when at least
//      k candidates are >= the key built so far (32 counting passes over the
//      row held in shared memory, warp-reduced);
//   2. every candidate above that threshold is selected, plus as many
//      candidates EQUAL to it as are still needed, lowest column first (the
//      tie rule);
//   3. columns at or past n_rank are always selected ("forced": the text /
//      boundary key blocks); rows at or past dense_row_start select every
//      column: when kmax has room for every column they are listed, otherwise
//      the row gets the count -1 ("every key block") and no list, so that a few
//      dense rows do not set the list length of all the others;
//   4. the list is written in ascending column order by an ordered warp
//      compaction (ballot + popc), padded with -1.
#include "common.cuh"

namespace {

constexpr int kWarpsPerCta = 8;

// float -> unsigned key with the same order (larger score <-> larger key)
__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void __launch_bounds__(kWarpsPerCta * 32)
    select_topk_kernel(const float* __restrict__ scores, int score_rows, int q_rows, int n_cols, int n_rank,
                       int k_select, int dense_row_start, int32_t* __restrict__ idx, int32_t* __restrict__ cnt,
                       int kmax, uint8_t* __restrict__ mask_out, int warps_per_cta) {
  extern __shared__ uint32_t keys_all[];  // [warps_per_cta][n_rank]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp >= warps_per_cta) return;
  const int row = blockIdx.x * warps_per_cta + warp;
  const int head = blockIdx.y;
  if (row >= q_rows) return;
  uint32_t* __restrict__ keys = keys_all + static_cast<size_t>(warp) * n_rank;
  int32_t* __restrict__ out = idx + (static_cast<size_t>(head) * q_rows + row) * kmax;
  uint8_t* __restrict__ mrow =
      mask_out ? mask_out + (static_cast<size_t>(head) * q_rows + row) * n_cols : nullptr;
  const bool dense = row >= dense_row_start;
  const unsigned lt_mask = (1u << lane) - 1u;
  if (dense && kmax < n_cols) {  // marker row: every key block, nothing listed
    for (int pos = lane; pos < kmax; pos += 32) out[pos] = -1;
    if (mrow)
      for (int c = lane; c < n_cols; c += 32) mrow[c] = 1;
    if (lane == 0) cnt[static_cast<size_t>(head) * q_rows + row] = -1;
    return;
  }

  uint32_t thr = 0;  // key of the k-th largest candidate
  int need_eq = 0;   // how many candidates equal to it are selected
  if (!dense && k_select > 0) {
    const float* __restrict__ src = scores + (static_cast<size_t>(head) * score_rows + row) * n_cols;
    for (int c = lane; c < n_rank; c += 32) keys[c] = order_key(src[c]);
    __syncwarp();
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = thr | (1u << bit);
      int local = 0;
      for (int c = lane; c < n_rank; c += 32) local += keys[c] >= cand;
      if (__reduce_add_sync(0xffffffffu, local) >= k_select) thr = cand;
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
  if (lane == 0) cnt[static_cast<size_t>(head) * q_rows + row] = written < kmax ? written : kmax;
}

}  // namespace

extern "C" int dfs_select_topk(const float* scores, int heads, int score_rows, int q_rows, int n_cols,
                               int n_rank, int k_select, int dense_row_start, int32_t* idx, int32_t* cnt,
                               int kmax, uint8_t* mask_out, void* stream) {
  if (scores == nullptr || idx == nullptr || cnt == nullptr) return DFS_ERR_NULL;
  if (heads <= 0 || q_rows <= 0 || n_cols <= 0 || score_rows < 0) return DFS_ERR_SHAPE;
  if (n_rank < 0 || n_rank > n_cols) return DFS_ERR_RANGE;
  if (k_select < 0 || k_select > n_rank) return DFS_ERR_RANGE;
  if (dense_row_start < 0) return DFS_ERR_RANGE;
  if (dense_row_start > q_rows) dense_row_start = q_rows;
  if (dense_row_start > score_rows) return DFS_ERR_RANGE;  // a ranked row needs its scores
  // every ranked row's list must fit; dense rows are listed only when kmax >= n_cols (else count -1)
  const int sparse_cnt = k_select + (n_cols - n_rank);
  if (kmax < sparse_cnt || kmax <= 0) return DFS_ERR_RANGE;
  // one warp per row, its keys in shared memory: fewer warps per CTA for very long rows
  const size_t row_bytes = sizeof(uint32_t) * static_cast<size_t>(n_rank > 0 ? n_rank : 1);
  if (row_bytes > 200 * 1024) return DFS_ERR_SHAPE;
  int warps = kWarpsPerCta;
  while (warps > 1 && row_bytes * warps > 96 * 1024) warps >>= 1;
  const size_t smem = row_bytes * warps;
  if (smem > 48 * 1024)
    DFS_CUDA_CHECK(cudaFuncSetAttribute(select_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)));
  dim3 grid((q_rows + warps - 1) / warps, heads);
  select_topk_kernel<<<grid, kWarpsPerCta * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      scores, score_rows, q_rows, n_cols, n_rank, k_select, dense_row_start, idx, cnt, kmax, mask_out, warps);
  return static_cast<int>(cudaGetLastError());
}
