// Row gather along the token axis: dst[h, i, :] = src[h, perm[i], :].
//
// HBM-bound byte copy.  One thread moves one 16-byte chunk; consecutive
// threads cover one row's chunks, so every row is read and written as whole
// 128/256/512-byte segments.  Algorithmic traffic = 2 * bytes(tensor) plus the
// 4-byte index per row.
#include "common.cuh"

namespace {

struct PermuteArgs {
  const uint4* src[3];
  uint4* dst[3];
};

__global__ void __launch_bounds__(256) permute_rows_kernel(PermuteArgs args, const int32_t* __restrict__ perm,
                                                           long long seq_len, int chunks_per_row,
                                                           long long chunks_per_head) {
  const int which = blockIdx.z;
  const int head = blockIdx.y;
  // selects instead of a dynamic index keep the argument struct out of local memory
  const uint4* __restrict__ src = which == 0 ? args.src[0] : (which == 1 ? args.src[1] : args.src[2]);
  uint4* __restrict__ dst = which == 0 ? args.dst[0] : (which == 1 ? args.dst[1] : args.dst[2]);
  const long long base = static_cast<long long>(head) * chunks_per_head;
  for (long long c = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; c < chunks_per_head;
       c += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = c / chunks_per_row;
    const int col = static_cast<int>(c - row * chunks_per_row);
    const long long from = static_cast<long long>(__ldg(perm + row));
    dst[base + c] = __ldg(src + base + from * chunks_per_row + col);
  }
}

int launch_permute(const void* const* srcs, void* const* dsts, int n, const int32_t* perm, int heads,
                   int64_t seq_len, int row_bytes, cudaStream_t stream) {
  if (perm == nullptr) return DFS_ERR_NULL;
  if (heads <= 0 || seq_len <= 0 || row_bytes <= 0 || (row_bytes & 15) != 0) return DFS_ERR_SHAPE;
  PermuteArgs args = {};
  int m = 0;
  for (int i = 0; i < n; ++i) {
    if ((srcs[i] == nullptr) != (dsts[i] == nullptr)) return DFS_ERR_NULL;
    if (srcs[i] == nullptr) continue;
    if (!dfs_aligned16(srcs[i]) || !dfs_aligned16(dsts[i])) return DFS_ERR_ALIGN;
    if (srcs[i] == dsts[i]) return DFS_ERR_RANGE;  // a gather cannot run in place
    args.src[m] = static_cast<const uint4*>(srcs[i]);
    args.dst[m] = static_cast<uint4*>(dsts[i]);
    ++m;
  }
  if (m == 0) return 0;
  const int chunks_per_row = row_bytes / 16;
  const long long chunks_per_head = static_cast<long long>(seq_len) * chunks_per_row;
  long long blocks = (chunks_per_head + 255) / 256;
  // a few waves of 148 SMs x 8 resident CTAs; the grid-stride loop covers the rest
  const long long cap = 148LL * 8 * 4;
  if (blocks > cap) blocks = cap;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(heads), static_cast<unsigned>(m));
  permute_rows_kernel<<<grid, 256, 0, stream>>>(args, perm, seq_len, chunks_per_row, chunks_per_head);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" int dfs_permute_qkv(const void* q, const void* k, const void* v, const int32_t* perm, void* q_out,
                               void* k_out, void* v_out, int heads, int64_t seq_len, int row_bytes,
                               void* stream) {
  const void* srcs[3] = {q, k, v};
  void* dsts[3] = {q_out, k_out, v_out};
  return launch_permute(srcs, dsts, 3, perm, heads, seq_len, row_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int dfs_unpermute(const void* src, const int32_t* inv_perm, void* dst, int heads, int64_t seq_len,
                             int row_bytes, void* stream) {
  if (src == nullptr || dst == nullptr) return DFS_ERR_NULL;
  const void* srcs[1] = {src};
  void* dsts[1] = {dst};
  return launch_permute(srcs, dsts, 1, inv_perm, heads, seq_len, row_bytes, static_cast<cudaStream_t>(stream));
}
