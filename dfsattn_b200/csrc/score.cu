// Hierarchical block scoring: 16-token mean pooling of Q and K, pooled
// Q.K^T logits, softmax over all key tiles, 8x8 tile sums -> block scores.
//
// The softmax-ed tile-score tensor of the reference ([H, 7432, 7448] at the
// 720p shape, several GB) is never materialised.  Three kernels:
//   1. pool_tiles_kernel : means of 16 consecutive (scoring-layout) tokens,
//                          written d-major so that the GEMM reads them coalesced.
//   2. tile_lse_kernel   : fp32 GEMM of pooled Q x pooled K; for every (query
//                          tile, key BLOCK) only log-sum-exp of the 8 logits
//                          of that block is kept  (H * Nq * Kb floats).
//   3. block_sum_kernel  : per query block, row max / normaliser over all key
//                          blocks from the stored LSEs, then
//                          B[c] = sum_i exp(lse_ic - M_i) / Z_i   (= the sum of
//                          the 64 softmax-ed tile scores of the 8x8 group).
// Everything is fp32; sums of softmax-ed scores equal the reference's up to
// fp32 rounding (different summation order).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kTile = 16;    // tokens per pooled tile
constexpr int kBlock = 128;  // tokens per block
constexpr int kTilesPerBlock = kBlock / kTile;
constexpr int kGemmTile = 64;  // pooled rows per GEMM tile (= 8 blocks)

struct ScoreShape {
  int heads;
  long long seq_len, video_len;
  int head_dim;
  int q_blocks;  // rows of the block-score matrix
  int k_blocks;
  int nq, nk;          // pooled tiles (q_blocks*8, k_blocks*8)
  int nq_pad, nk_pad;  // padded to kGemmTile
  long long video_padded;  // Vb*128: scoring position where the text part starts
};

__host__ ScoreShape make_shape(int heads, int64_t seq_len, int64_t video_len, int head_dim, int wan_layout) {
  ScoreShape s;
  s.heads = heads;
  s.seq_len = seq_len;
  s.video_len = wan_layout ? seq_len : video_len;
  s.head_dim = head_dim;
  s.k_blocks = static_cast<int>((seq_len + kBlock - 1) / kBlock);
  s.q_blocks = static_cast<int>((s.video_len + kBlock - 1) / kBlock);
  s.nq = s.q_blocks * kTilesPerBlock;
  s.nk = s.k_blocks * kTilesPerBlock;
  s.nq_pad = (s.nq + kGemmTile - 1) / kGemmTile * kGemmTile;
  s.nk_pad = (s.nk + kGemmTile - 1) / kGemmTile * kGemmTile;
  s.video_padded = static_cast<long long>(s.q_blocks) * kBlock;
  return s;
}

__host__ size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

struct Workspace {
  size_t qm_off, km_off, lse_off, total;
};
__host__ Workspace make_workspace(const ScoreShape& s) {
  Workspace w;
  w.qm_off = 0;
  w.km_off = align256(w.qm_off + sizeof(float) * s.heads * s.head_dim * static_cast<size_t>(s.nq_pad));
  w.lse_off = align256(w.km_off + sizeof(float) * s.heads * s.head_dim * static_cast<size_t>(s.nk_pad));
  w.total = align256(w.lse_off + sizeof(float) * s.heads * static_cast<size_t>(s.nq) * s.k_blocks);
  return w;
}

// scoring position -> row of the permuted tensor, or -1 for a zero row.
// Layout: [video | zeros up to a block multiple | text | zeros].
__device__ __forceinline__ long long scoring_row(long long p, long long video_len, long long video_padded,
                                                 long long seq_len) {
  if (p < video_len) return p;
  if (p < video_padded) return -1;
  const long long r = video_len + (p - video_padded);
  return r < seq_len ? r : -1;
}

template <typename T>
struct Vec16;
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  __device__ static void accumulate(const uint4& raw, float* acc) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(p[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
};
template <>
struct Vec16<float> {
  static constexpr int kElems = 4;
  __device__ static void accumulate(const uint4& raw, float* acc) {
    const float* p = reinterpret_cast<const float*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] += p[i];
  }
};

// One thread: one 16-byte column chunk of one pooled tile.  A CTA covers
// TILES_PER_CTA consecutive tiles; results go through shared memory so that the
// d-major output is written as runs of TILES_PER_CTA consecutive floats.
template <typename T>
__global__ void __launch_bounds__(256) pool_tiles_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                         float* __restrict__ qm_t, float* __restrict__ km_t,
                                                         ScoreShape s) {
  constexpr int E = Vec16<T>::kElems;
  const int chunks = s.head_dim / E;          // 16-byte chunks per row
  const int tiles_per_cta = blockDim.x / chunks;
  extern __shared__ float sm_pool[];          // [head_dim][tiles_per_cta + 1]
  const int which = blockIdx.z;               // 0: Q, 1: K
  const int head = blockIdx.y;
  const int n_tiles = which == 0 ? s.nq : s.nk;
  const int n_pad = which == 0 ? s.nq_pad : s.nk_pad;
  const T* __restrict__ src = (which == 0 ? q : k) + static_cast<size_t>(head) * s.seq_len * s.head_dim;
  float* __restrict__ dst = (which == 0 ? qm_t : km_t) + static_cast<size_t>(head) * s.head_dim * n_pad;

  const int tile0 = blockIdx.x * tiles_per_cta;
  if (tile0 >= n_pad) return;
  const int tl = threadIdx.x / chunks;
  const int ch = threadIdx.x % chunks;
  const int tile = tile0 + tl;
  float acc[E];
#pragma unroll
  for (int i = 0; i < E; ++i) acc[i] = 0.f;
  if (tl < tiles_per_cta && tile < n_tiles) {
    const long long p0 = static_cast<long long>(tile) * kTile;
#pragma unroll 4
    for (int r = 0; r < kTile; ++r) {
      const long long row = scoring_row(p0 + r, s.video_len, s.video_padded, s.seq_len);
      if (row >= 0) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + row * s.head_dim) + ch);
        Vec16<T>::accumulate(raw, acc);
      }
    }
  }
  const int ld = tiles_per_cta + 1;
  if (tl < tiles_per_cta) {
#pragma unroll
    for (int i = 0; i < E; ++i) sm_pool[(ch * E + i) * ld + tl] = acc[i] * (1.0f / kTile);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < s.head_dim * tiles_per_cta; e += blockDim.x) {
    const int d = e / tiles_per_cta;
    const int t = e - d * tiles_per_cta;
    if (tile0 + t < n_pad) dst[static_cast<size_t>(d) * n_pad + tile0 + t] = sm_pool[d * ld + t];
  }
}

// 64 x 64 pooled logits per step, 4 x 4 per thread, fp32 FMA.
template <int HD>
__global__ void __launch_bounds__(256) tile_lse_kernel(const float* __restrict__ qm_t,
                                                       const float* __restrict__ km_t,
                                                       float* __restrict__ lse, ScoreShape s, float scale) {
  extern __shared__ float sm_gemm[];
  float* As = sm_gemm;                   // [HD][64]
  float* Bs = sm_gemm + HD * kGemmTile;  // [HD][64]
  const int head = blockIdx.y;
  const int row0 = blockIdx.x * kGemmTile;
  const int tx = threadIdx.x & 15;
  const int ty = threadIdx.x >> 4;
  const float* __restrict__ a_src = qm_t + static_cast<size_t>(head) * HD * s.nq_pad + row0;
  const float* __restrict__ b_src = km_t + static_cast<size_t>(head) * HD * s.nk_pad;

  for (int e = threadIdx.x; e < HD * (kGemmTile / 4); e += 256) {
    const int d = e / (kGemmTile / 4);
    const int c4 = e - d * (kGemmTile / 4);
    reinterpret_cast<float4*>(As)[e] =
        __ldg(reinterpret_cast<const float4*>(a_src + static_cast<size_t>(d) * s.nq_pad) + c4);
  }

  for (int col0 = 0; col0 < s.nk_pad; col0 += kGemmTile) {
    __syncthreads();  // previous step's readers of Bs are done (also covers As on the first step)
    for (int e = threadIdx.x; e < HD * (kGemmTile / 4); e += 256) {
      const int d = e / (kGemmTile / 4);
      const int c4 = e - d * (kGemmTile / 4);
      reinterpret_cast<float4*>(Bs)[e] =
          __ldg(reinterpret_cast<const float4*>(b_src + static_cast<size_t>(d) * s.nk_pad + col0) + c4);
    }
    __syncthreads();

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

#pragma unroll 8
    for (int d = 0; d < HD; ++d) {
      const float4 a = reinterpret_cast<const float4*>(As + d * kGemmTile)[ty];
      const float4 b = reinterpret_cast<const float4*>(Bs + d * kGemmTile)[tx];
      const float av[4] = {a.x, a.y, a.z, a.w};
      const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }

    // log-sum-exp over the 8 key tiles of one key block: 4 here, 4 in lane^1
    const int kblock = (col0 + tx * 4) / kTilesPerBlock;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float m = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[i][j] *= scale;
        m = fmaxf(m, acc[i][j]);
      }
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) sum += expf(acc[i][j] - m);
      const float m2 = __shfl_xor_sync(0xffffffffu, m, 1);
      const float s2 = __shfl_xor_sync(0xffffffffu, sum, 1);
      const float mm = fmaxf(m, m2);
      const float tot = sum * expf(m - mm) + s2 * expf(m2 - mm);
      const int row = row0 + ty * 4 + i;
      if ((tx & 1) == 0 && row < s.nq && kblock < s.k_blocks)
        lse[(static_cast<size_t>(head) * s.nq + row) * s.k_blocks + kblock] = mm + logf(tot);
    }
  }
}

// One CTA per (query block, head): 8 pooled rows x Kb stored LSEs -> Kb block scores.
__global__ void __launch_bounds__(256) block_sum_kernel(const float* __restrict__ lse,
                                                        float* __restrict__ block_scores, ScoreShape s) {
  __shared__ float row_max[kTilesPerBlock];
  __shared__ float row_inv[kTilesPerBlock];
  const int head = blockIdx.y;
  const int qb = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* __restrict__ rows = lse + (static_cast<size_t>(head) * s.nq + qb * kTilesPerBlock) * s.k_blocks;
  {
    const float* __restrict__ r = rows + static_cast<size_t>(warp) * s.k_blocks;  // warp i <-> pooled row i
    float m = -INFINITY;
    for (int c = lane; c < s.k_blocks; c += 32) m = fmaxf(m, r[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float z = 0.f;
    for (int c = lane; c < s.k_blocks; c += 32) z += expf(r[c] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    if (lane == 0) {
      row_max[warp] = m;
      row_inv[warp] = 1.0f / z;
    }
  }
  __syncthreads();
  float* __restrict__ out = block_scores + (static_cast<size_t>(head) * s.q_blocks + qb) * s.k_blocks;
  for (int c = threadIdx.x; c < s.k_blocks; c += blockDim.x) {
    float b = 0.f;
#pragma unroll
    for (int i = 0; i < kTilesPerBlock; ++i)
      b += expf(rows[static_cast<size_t>(i) * s.k_blocks + c] - row_max[i]) * row_inv[i];
    out[c] = b;
  }
}

template <typename T>
int launch_pool(const void* q, const void* k, float* qm, float* km, const ScoreShape& s, cudaStream_t stream) {
  const int chunks = s.head_dim / Vec16<T>::kElems;
  const int tiles_per_cta = 256 / chunks;
  const int n_pad = s.nk_pad > s.nq_pad ? s.nk_pad : s.nq_pad;
  dim3 grid((n_pad + tiles_per_cta - 1) / tiles_per_cta, s.heads, 2);
  const size_t smem = sizeof(float) * s.head_dim * (tiles_per_cta + 1);
  pool_tiles_kernel<T><<<grid, 256, smem, stream>>>(static_cast<const T*>(q), static_cast<const T*>(k), qm, km, s);
  return static_cast<int>(cudaGetLastError());
}

template <int HD>
int launch_lse(const float* qm, const float* km, float* lse, const ScoreShape& s, float scale,
               cudaStream_t stream) {
  const size_t smem = sizeof(float) * 2 * HD * kGemmTile;
  DFS_CUDA_CHECK(cudaFuncSetAttribute(tile_lse_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
  dim3 grid(s.nq_pad / kGemmTile, s.heads);
  tile_lse_kernel<HD><<<grid, 256, smem, stream>>>(qm, km, lse, s, scale);
  return static_cast<int>(cudaGetLastError());
}

int check_shape(int heads, int64_t seq_len, int64_t video_len, int head_dim, int tile, int block,
                int wan_layout) {
  if (tile != kTile || block != kBlock) return DFS_ERR_SHAPE;
  if (head_dim != 64 && head_dim != 128) return DFS_ERR_SHAPE;
  if (heads <= 0 || seq_len <= 0) return DFS_ERR_SHAPE;
  if (!wan_layout) {
    if (video_len <= 0 || video_len > seq_len) return DFS_ERR_RANGE;
    // The scoring layout [video | zero gap | text] must fit in Kb blocks; the
    // reference's view() fails on shapes where it does not.
    const int64_t vb = (video_len + kBlock - 1) / kBlock, kb = (seq_len + kBlock - 1) / kBlock;
    if (vb * kBlock + (seq_len - video_len) > kb * kBlock) return DFS_ERR_SHAPE;
  }
  return 0;
}

}  // namespace

extern "C" int64_t dfs_score_workspace_bytes(int heads, int64_t seq_len, int64_t video_len, int head_dim,
                                             int tile, int block, int wan_layout) {
  const int rc = check_shape(heads, seq_len, video_len, head_dim, tile, block, wan_layout);
  if (rc != 0) return rc;
  return static_cast<int64_t>(make_workspace(make_shape(heads, seq_len, video_len, head_dim, wan_layout)).total);
}

extern "C" int dfs_block_scores(const void* q_perm, const void* k_perm, int dtype, int heads, int64_t seq_len,
                                int64_t video_len, int head_dim, int tile, int block, int wan_layout,
                                float* block_scores, void* workspace, int64_t workspace_bytes, void* stream_) {
  if (q_perm == nullptr || k_perm == nullptr || block_scores == nullptr || workspace == nullptr)
    return DFS_ERR_NULL;
  if (!dfs_aligned16(q_perm) || !dfs_aligned16(k_perm) || !dfs_aligned16(workspace)) return DFS_ERR_ALIGN;
  if (dtype != DFS_DTYPE_BF16 && dtype != DFS_DTYPE_F32) return DFS_ERR_DTYPE;
  const int rc = check_shape(heads, seq_len, video_len, head_dim, tile, block, wan_layout);
  if (rc != 0) return rc;
  const ScoreShape s = make_shape(heads, seq_len, video_len, head_dim, wan_layout);
  const Workspace w = make_workspace(s);
  if (workspace_bytes < static_cast<int64_t>(w.total)) return DFS_ERR_WORKSPACE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  char* base = static_cast<char*>(workspace);
  float* qm = reinterpret_cast<float*>(base + w.qm_off);
  float* km = reinterpret_cast<float*>(base + w.km_off);
  float* lse = reinterpret_cast<float*>(base + w.lse_off);

  int err = dtype == DFS_DTYPE_BF16 ? launch_pool<__nv_bfloat16>(q_perm, k_perm, qm, km, s, stream)
                                    : launch_pool<float>(q_perm, k_perm, qm, km, s, stream);
  if (err != 0) return err;
  const float scale = 1.0f / sqrtf(static_cast<float>(head_dim));
  err = head_dim == 128 ? launch_lse<128>(qm, km, lse, s, scale, stream)
                        : launch_lse<64>(qm, km, lse, s, scale, stream);
  if (err != 0) return err;
  dim3 grid(s.q_blocks, s.heads);
  block_sum_kernel<<<grid, 256, 0, stream>>>(lse, block_scores, s);
  return static_cast<int>(cudaGetLastError());
}

// --------------------------------------------------------------------------
// Scoring without any allocation by the caller or by the library.
//
// Some hosts of this library may not allocate device memory at the moment
// they need block scores: an inference server whose memory pool was sized and
// frozen at start-up, a plugin that runs inside another framework's step where
// a cudaMalloc would synchronise the whole device, or a process that has
// handed all remaining memory to its tensor allocator.  For them the scratch
// lives in a fixed array inside the loaded library image.  Every GPU that
// loads the library holds these kStaticScratchBytes until the process exits.
// --------------------------------------------------------------------------
namespace {
constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB
constexpr int kMaxDevices = 64;
}  // namespace

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
// Device address of g_static_scratch per device.  In host code the symbol's
// name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
char* g_static_scratch_addr[kMaxDevices] = {};

int static_scratch_for_current_device(char** out) {
  int dev = -1;
  DFS_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return DFS_ERR_RANGE;
  if (g_static_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    DFS_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (ptr == nullptr) return DFS_ERR_NULL;
    g_static_scratch_addr[dev] = static_cast<char*>(ptr);
  }
  *out = g_static_scratch_addr[dev];
  return 0;
}
}  // namespace

extern "C" int64_t dfs_block_scores_static_max_bytes(void) { return static_cast<int64_t>(kStaticScratchBytes); }

extern "C" int dfs_block_scores_static(const void* q_perm, const void* k_perm, int dtype, int heads,
                                       int64_t seq_len, int64_t video_len, int head_dim, int tile, int block,
                                       int wan_layout, float* block_scores, void* stream_) {
  if (q_perm == nullptr || k_perm == nullptr || block_scores == nullptr) return DFS_ERR_NULL;
  if (!dfs_aligned16(q_perm) || !dfs_aligned16(k_perm)) return DFS_ERR_ALIGN;
  if (dtype != DFS_DTYPE_BF16 && dtype != DFS_DTYPE_F32) return DFS_ERR_DTYPE;
  const int rc = check_shape(heads, seq_len, video_len, head_dim, tile, block, wan_layout);
  if (rc != 0) return rc;
  const ScoreShape s = make_shape(heads, seq_len, video_len, head_dim, wan_layout);
  const Workspace w = make_workspace(s);
  if (w.total > kStaticScratchBytes) return DFS_ERR_STATIC_SCRATCH;  // shape needs more than the fixed array
  char* base = nullptr;
  const int rs = static_scratch_for_current_device(&base);
  if (rs != 0) return rs;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // Nothing in the scratch has to start at zero: the pooling kernel writes every
  // element of both pooled matrices (padding included) and the block-sum kernel
  // reads only LSE entries the GEMM kernel has just written, so whatever the
  // previous call left behind is never read.
  float* qm = reinterpret_cast<float*>(base + w.qm_off);
  float* km = reinterpret_cast<float*>(base + w.km_off);
  float* lse = reinterpret_cast<float*>(base + w.lse_off);
  int err = dtype == DFS_DTYPE_BF16 ? launch_pool<__nv_bfloat16>(q_perm, k_perm, qm, km, s, stream)
                                    : launch_pool<float>(q_perm, k_perm, qm, km, s, stream);
  if (err != 0) return err;
  const float scale = 1.0f / sqrtf(static_cast<float>(head_dim));
  err = head_dim == 128 ? launch_lse<128>(qm, km, lse, s, scale, stream)
                        : launch_lse<64>(qm, km, lse, s, scale, stream);
  if (err != 0) return err;
  dim3 grid(s.q_blocks, s.heads);
  block_sum_kernel<<<grid, 256, 0, stream>>>(lse, block_scores, s);
  return static_cast<int>(cudaGetLastError());
}
