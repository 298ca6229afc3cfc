// Row gather along the token axis: dst[h, i, :] = src[h, perm[i], :].
//
// HBM-bound byte copy.  One thread moves 16-byte chunks; consecutive threads cover one row's
// chunks, so every row is read and written as whole 128/256/512-byte segments.  A thread handles
// four chunks (a grid stride apart) per trip: the four index loads go out together, then the four
// row loads, then the four stores, so that a warp keeps 2 KB of reads in flight instead of 512
// bytes.  Index arithmetic is 32-bit (a head has fewer than 2^31 chunks; checked by the launcher),
// with a shift when a row is a power-of-two number of chunks.  Algorithmic traffic =
// 2 * bytes(tensor) plus the 4-byte index per row.
#include "common.cuh"

namespace {

struct PermuteArgs {
  const uint4* src[3];
  uint4* dst[3];
};

constexpr int kPermuteBatch = 4;

// chunk index within a head -> (row, column) with chunks_per_row = 1 << shift, or a division
template <bool kPow2>
__device__ __forceinline__ void split_chunk(unsigned c, unsigned chunks_per_row, int shift, unsigned& row,
                                            unsigned& col) {
  if (kPow2) {
    row = c >> shift;
    col = c & (chunks_per_row - 1u);
  } else {
    row = c / chunks_per_row;
    col = c - row * chunks_per_row;
  }
}

template <bool kPow2>
__global__ void __launch_bounds__(256) permute_rows_kernel(PermuteArgs args, const int32_t* __restrict__ perm,
                                                           unsigned chunks_per_row, int shift,
                                                           unsigned chunks_per_head) {
  const int which = blockIdx.z;
  const int head = blockIdx.y;
  // selects instead of a dynamic index keep the argument struct out of local memory
  const uint4* __restrict__ src = which == 0 ? args.src[0] : (which == 1 ? args.src[1] : args.src[2]);
  uint4* __restrict__ dst = which == 0 ? args.dst[0] : (which == 1 ? args.dst[1] : args.dst[2]);
  const size_t base = static_cast<size_t>(head) * chunks_per_head;
  src += base;
  dst += base;
  const unsigned stride = gridDim.x * blockDim.x;
  unsigned c = blockIdx.x * blockDim.x + threadIdx.x;
  // chunks_per_head < 2^31 and stride < 2^21, so c + 3 * stride cannot wrap
  for (; c + (kPermuteBatch - 1) * stride < chunks_per_head; c += kPermuteBatch * stride) {
    unsigned col[kPermuteBatch];
    int from[kPermuteBatch];
    uint4 val[kPermuteBatch];
#pragma unroll
    for (int b = 0; b < kPermuteBatch; ++b) {
      unsigned row;
      split_chunk<kPow2>(c + b * stride, chunks_per_row, shift, row, col[b]);
      from[b] = __ldg(perm + row);
    }
#pragma unroll
    for (int b = 0; b < kPermuteBatch; ++b)
      val[b] = __ldcs(src + static_cast<size_t>(from[b]) * chunks_per_row + col[b]);
#pragma unroll
    for (int b = 0; b < kPermuteBatch; ++b) __stcs(dst + c + b * stride, val[b]);
  }
  for (; c < chunks_per_head; c += stride) {
    unsigned row, col;
    split_chunk<kPow2>(c, chunks_per_row, shift, row, col);
    const int from = __ldg(perm + row);
    __stcs(dst + c, __ldcs(src + static_cast<size_t>(from) * chunks_per_row + col));
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
  if (chunks_per_head >= (1LL << 31)) return DFS_ERR_SHAPE;
  long long blocks = (chunks_per_head + 256 * kPermuteBatch - 1) / (256 * kPermuteBatch);
  // a few waves of 148 SMs x 8 resident CTAs; the grid-stride loop covers the rest
  const long long cap = 148LL * 8 * 4;
  if (blocks > cap) blocks = cap;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(heads), static_cast<unsigned>(m));
  int shift = 0;
  while ((1 << shift) < chunks_per_row) ++shift;
  if ((1 << shift) == chunks_per_row)
    permute_rows_kernel<true><<<grid, 256, 0, stream>>>(args, perm, chunks_per_row, shift,
                                                        static_cast<unsigned>(chunks_per_head));
  else
    permute_rows_kernel<false><<<grid, 256, 0, stream>>>(args, perm, chunks_per_row, 0,
                                                         static_cast<unsigned>(chunks_per_head));
  return static_cast<int>(cudaGetLastError());
}

// ---- gather from sequence shards held by several GPUs ----------------------------------------
// Source token r lives in shard r / shard_rows (one shard per GPU, [H_total, shard_stride, D]) at
// local row r % shard_rows; this rank gathers the rows of its own heads [head0, head0 + heads).
// Peer shards are read with plain 16-byte loads over NVLink; nothing else touches peer memory.
constexpr int kMaxShards = 8;

struct ShardedArgs {
  const uint4* src[3][kMaxShards];
  uint4* dst[3];
};

__global__ void __launch_bounds__(256)
    permute_rows_sharded_kernel(const __grid_constant__ ShardedArgs args, const int32_t* __restrict__ perm,
                                int chunks_per_row, long long chunks_per_head, unsigned shard_rows,
                                long long shard_stride_chunks, int head0) {
  const int which = blockIdx.z;
  const int head = blockIdx.y;
  uint4* __restrict__ dst = args.dst[which] + static_cast<long long>(head) * chunks_per_head;
  const long long head_off = static_cast<long long>(head0 + head) * shard_stride_chunks;
  for (long long c = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; c < chunks_per_head;
       c += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = c / chunks_per_row;
    const int col = static_cast<int>(c - row * chunks_per_row);
    const unsigned from = perm ? static_cast<unsigned>(__ldg(perm + row)) : static_cast<unsigned>(row);
    const unsigned shard = from / shard_rows;
    const unsigned local = from - shard * shard_rows;
    const uint4* __restrict__ src = args.src[which][shard];
    dst[c] = __ldg(src + head_off + static_cast<long long>(local) * chunks_per_row + col);
  }
}

}  // namespace

extern "C" int dfs_permute_qkv_sharded(const void* const* q_shards, const void* const* k_shards,
                                       const void* const* v_shards, int world, int64_t shard_rows,
                                       int64_t shard_stride_rows, int head0, const int32_t* perm, void* q_out,
                                       void* k_out, void* v_out, int heads, int64_t seq_len, int row_bytes,
                                       void* stream) {
  if (q_shards == nullptr || k_shards == nullptr || v_shards == nullptr) return DFS_ERR_NULL;
  if (q_out == nullptr || k_out == nullptr || v_out == nullptr) return DFS_ERR_NULL;
  if (world <= 0 || world > kMaxShards) return DFS_ERR_RANGE;
  if (heads <= 0 || head0 < 0 || seq_len <= 0 || row_bytes <= 0 || (row_bytes & 15) != 0) return DFS_ERR_SHAPE;
  if (shard_rows <= 0 || shard_stride_rows < shard_rows || shard_rows * world < seq_len) return DFS_ERR_RANGE;
  if (seq_len > 0x7fffffffLL) return DFS_ERR_SHAPE;
  ShardedArgs args = {};
  const void* const* tabs[3] = {q_shards, k_shards, v_shards};
  void* dsts[3] = {q_out, k_out, v_out};
  for (int t = 0; t < 3; ++t) {
    if (!dfs_aligned16(dsts[t])) return DFS_ERR_ALIGN;
    args.dst[t] = static_cast<uint4*>(dsts[t]);
    for (int s = 0; s < world; ++s) {
      if (tabs[t][s] == nullptr) return DFS_ERR_NULL;
      if (!dfs_aligned16(tabs[t][s])) return DFS_ERR_ALIGN;
      args.src[t][s] = static_cast<const uint4*>(tabs[t][s]);
    }
  }
  const int chunks_per_row = row_bytes / 16;
  const long long chunks_per_head = static_cast<long long>(seq_len) * chunks_per_row;
  long long blocks = (chunks_per_head + 255) / 256;
  const long long cap = 148LL * 8 * 4;
  if (blocks > cap) blocks = cap;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(heads), 3);
  permute_rows_sharded_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      args, perm, chunks_per_row, chunks_per_head, static_cast<unsigned>(shard_rows),
      shard_stride_rows * chunks_per_row, head0);
  return static_cast<int>(cudaGetLastError());
}

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
