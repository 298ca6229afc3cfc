// Per-row top-k key-block selection -> ascending index lists.
//
// One CTA per (query-block row, head).  Exact and deterministic: the rank of a
// candidate is the number of candidates that beat it (larger score, or equal
// score and lower column), so ties at the k-th place go to the lowest column.
// Columns at or past n_rank are always selected ("forced": the text / boundary
// key blocks); rows at or past dense_row_start select every column.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads) select_topk_kernel(const float* __restrict__ scores, int score_rows,
                                                               int q_rows, int n_cols, int n_rank, int k_select,
                                                               int dense_row_start, int32_t* __restrict__ idx,
                                                               int32_t* __restrict__ cnt, int kmax,
                                                               uint8_t* __restrict__ mask_out) {
  extern __shared__ float vals[];  // [n_rank]
  __shared__ int warp_tot[kThreads / 32];
  __shared__ int base_shared;
  const int row = blockIdx.x;
  const int head = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t* __restrict__ out = idx + (static_cast<size_t>(head) * q_rows + row) * kmax;
  uint8_t* __restrict__ mrow =
      mask_out ? mask_out + (static_cast<size_t>(head) * q_rows + row) * n_cols : nullptr;
  const bool dense = row >= dense_row_start;

  if (!dense) {
    const float* __restrict__ src = scores + (static_cast<size_t>(head) * score_rows + row) * n_cols;
    for (int c = threadIdx.x; c < n_rank; c += kThreads) vals[c] = src[c];
  }
  if (threadIdx.x == 0) base_shared = 0;
  __syncthreads();

  // columns are visited in ascending chunks of kThreads; an ordered compaction
  // (ballot + warp totals) keeps the list ascending
  for (int c0 = 0; c0 < n_cols; c0 += kThreads) {
    const int c = c0 + threadIdx.x;
    bool sel = false;
    if (c < n_cols) {
      if (dense || c >= n_rank) {
        sel = true;
      } else {
        const float v = vals[c];
        int rank = 0;
        for (int j = 0; j < n_rank; ++j) {
          const float u = vals[j];  // same address for the whole warp: broadcast
          rank += (u > v) || (u == v && j < c);
        }
        sel = rank < k_select;
      }
      if (mrow) mrow[c] = sel ? 1 : 0;
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, sel);
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int before = base_shared;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (sel) {
      const int pos = before + __popc(ballot & ((1u << lane) - 1u));
      if (pos < kmax) out[pos] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int t = base_shared;
      for (int w = 0; w < kThreads / 32; ++w) t += warp_tot[w];
      base_shared = t;
    }
    __syncthreads();
  }
  const int total = base_shared;
  for (int p = total + threadIdx.x; p < kmax; p += kThreads) out[p] = -1;
  if (threadIdx.x == 0) cnt[static_cast<size_t>(head) * q_rows + row] = total < kmax ? total : kmax;
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
  // every list must fit
  const int sparse_cnt = k_select + (n_cols - n_rank);
  const int need = dense_row_start < q_rows ? n_cols : sparse_cnt;
  if (kmax < need || kmax < sparse_cnt) return DFS_ERR_RANGE;
  const size_t smem = sizeof(float) * static_cast<size_t>(n_rank > 0 ? n_rank : 1);
  if (smem > 200 * 1024) return DFS_ERR_SHAPE;
  if (smem > 48 * 1024)
    DFS_CUDA_CHECK(cudaFuncSetAttribute(select_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)));
  dim3 grid(q_rows, heads);
  select_topk_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      scores, score_rows, q_rows, n_cols, n_rank, k_select, dense_row_start, idx, cnt, kmax, mask_out);
  return static_cast<int>(cudaGetLastError());
}
