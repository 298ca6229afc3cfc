// Per-row top-k key-block selection -> ascending index lists, from fp32 block scores in global memory.
// One warp per (query-block row, head); the row logic is select_row (select.cuh).
#include "select.cuh"

namespace {

using namespace dfs;

constexpr int kWarpsPerCta = 8;

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
  const size_t at = static_cast<size_t>(head) * q_rows + row;
  const bool dense = row >= dense_row_start;
  select_row(dense ? nullptr : scores + (static_cast<size_t>(head) * score_rows + row) * n_cols,
             n_rank > kRegisterRankMax ? keys_all + static_cast<size_t>(warp) * n_rank : nullptr, n_cols, n_rank,
             k_select, dense, kmax, idx + at * kmax, cnt + at, mask_out ? mask_out + at * n_cols : nullptr, lane);
}

}  // namespace

extern "C" int dfs_select_topk(const float* scores, int heads, int score_rows, int q_rows, int n_cols,
                               int n_rank, int k_select, int dense_row_start, int32_t* idx, int32_t* cnt,
                               int kmax, uint8_t* mask_out, void* stream) {
  if (scores == nullptr || idx == nullptr || cnt == nullptr) return DFS_ERR_NULL;
  const int rc = dfs_check_selection(heads, score_rows, q_rows, n_cols, n_rank, k_select, &dense_row_start, kmax);
  if (rc != 0) return rc;
  // one warp per row; the keys of a row too long for registers sit in shared memory: fewer warps per CTA
  // for very long rows
  const size_t row_bytes = n_rank > kRegisterRankMax ? sizeof(uint32_t) * static_cast<size_t>(n_rank) : 0;
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
