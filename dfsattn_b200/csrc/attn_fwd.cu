// Block-sparse attention forward for sm_100a: online softmax over the selected
// 128-token key blocks of each 128-token query block.
//
// One CTA per (query block, head), 6 warps:
//   warp 0     TMA producer: Q tile once, then the K and V tiles of every
//              listed key block into two shared-memory rings (mbarrier
//              full/empty pairs per stage).
//   warp 1     tcgen05.mma issuer (one lane): S = Q K^T into one of two TMEM
//              score buffers, O += P V with P read from TMEM; owns the TMEM
//              allocation.
//   warps 2-5  softmax: one thread per query row.  tcgen05.ld the 128 scores,
//              running max / sum in the log2 domain, P written back to TMEM as
//              packed bf16 (tcgen05.st); the accumulator O (in TMEM) is only
//              rescaled when the row max grew by more than 2^8 (the sum uses
//              the same reference max, so the result is exact); epilogue
//              normalises and stores bf16 rows, optionally through a row map
//              (fused inverse permutation).
//
// Shared memory (HD = 128): Q 32 KB + 3 x 32 KB K stages + 3 x 32 KB V stages.
// Tiles are stored as [128 rows][64 bf16] boxes with the 128-byte TMA swizzle,
// which is the canonical K-major (Q, K) and MN-major (V) tcgen05 operand layout.
// TMEM (512 columns): S0 | S1 | O | P0 | P1.
//
// Every wait is bounded; on expiry the CTA records DFS_STATUS_WAIT_TIMEOUT,
// drains its copies in flight, frees its TMEM and returns.
#include "common.cuh"

namespace {

using namespace dfs;

constexpr int kBlockM = 128;  // query rows per CTA
constexpr int kBlockN = 128;  // keys per tile
constexpr int kThreads = 192;
constexpr int kStages = 3;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO = 256, kColP0 = 384, kColP1 = 448;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

template <int HD>
struct SmemLayout {
  static constexpr int kBoxBytes = kBlockN * 64 * 2;          // one [128][64] bf16 box
  static constexpr int kTileBytes = kBoxBytes * (HD / 64);    // one Q / K / V tile
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kTileBytes;
  static constexpr int kVOff = kKOff + kStages * kTileBytes;
  static constexpr int kBarOff = kVOff + kStages * kTileBytes;
  static constexpr int kNumBars = 1 + 4 * kStages + 2 + 2 + 1 + 1;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;  // + tmem address + abort flag
  static constexpr int kAlloc = kTotal + 1024;                // slack for 1024-byte alignment
};

struct Params {
  const int32_t* idx;   // [H, Qb, kmax] or nullptr (all key blocks)
  const int32_t* cnt;   // [H, Qb]
  const int32_t* out_row_map;
  __nv_bfloat16* out;
  int32_t* status;
  float* debug;         // optional dump of CTA (0,0): S of the first tile, O, l, m
  long long seq_len;
  long long kv_len;
  int kmax;
  int q_blocks, k_blocks;
  float scale_log2;
  uint32_t v_lbo, v_sbo;  // V operand descriptor strides (bytes)
};

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
    bsattn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const Params p) {
  using L = SmemLayout<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_tile = smem + L::kQOff;
  uint8_t* k_ring = smem + L::kKOff;
  uint8_t* v_ring = smem + L::kVOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + kStages;
  uint64_t* v_full = k_empty + kStages;
  uint64_t* v_empty = v_full + kStages;
  uint64_t* s_full = v_empty + kStages;  // [2]
  uint64_t* p_full = s_full + 2;         // [2]
  uint64_t* o_done = p_full + 2;
  uint64_t* mma_drain = o_done + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heavy rows (the dense text rows sit at the end) are scheduled first
  const int qb = p.q_blocks - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y;
  const int n_tiles = p.idx ? p.cnt[static_cast<size_t>(head) * p.q_blocks + qb] : p.k_blocks;
  const int32_t* __restrict__ my_idx =
      p.idx ? p.idx + (static_cast<size_t>(head) * p.q_blocks + qb) * p.kmax : nullptr;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 128);
    }
    mbar_init(o_done, 1);
    mbar_init(mma_drain, 1);
    abort_flag[0] = 0;  // set by the first wait that expires
    abort_flag[1] = 0;  // separate limit for the drain waits of the give-up path
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_arrive_expect_tx(q_full, L::kTileBytes);
      for (int c = 0; c < HD / 64; ++c)
        tma_load_3d(q_tile + c * L::kBoxBytes, &tm_q, q_full, c * 64, qb * kBlockM, head);
      int issued_k = 0, issued_v = 0;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int kb = my_idx ? __ldg(my_idx + j) : j;
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        ok = mbar_wait_bounded(&k_empty[s], ph ^ 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&k_full[s], L::kTileBytes);
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d(k_ring + s * L::kTileBytes + c * L::kBoxBytes, &tm_k, &k_full[s], c * 64, kb * kBlockN,
                      head);
        ++issued_k;
        ok = mbar_wait_bounded(&v_empty[s], ph ^ 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&v_full[s], L::kTileBytes);
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d(v_ring + s * L::kTileBytes + c * L::kBoxBytes, &tm_v, &v_full[s], c * 64, kb * kBlockN,
                      head);
        ++issued_v;
      }
      if (!ok) {
        // drain: the copies already issued must land before the CTA may exit
        mbar_wait_bounded(q_full, 0, abort_flag + 1);
        for (int j = issued_k > kStages ? issued_k - kStages : 0; j < issued_k; ++j)
          mbar_wait_bounded(&k_full[j % kStages], (j / kStages) & 1, abort_flag + 1);
        for (int j = issued_v > kStages ? issued_v - kStages : 0; j < issued_v; ++j)
          mbar_wait_bounded(&v_full[j % kStages], (j / kStages) & 1, abort_flag + 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(kBlockM, kBlockN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kBlockM, HD, 0, 1);
      const uint32_t q_addr = smem_u32(q_tile);
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag);
      for (int j = 0; j <= n_tiles && ok; ++j) {
        if (j < n_tiles) {
          const int s = j % kStages;
          ok = mbar_wait_bounded(&k_full[s], (j / kStages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t k_addr = smem_u32(k_ring + s * L::kTileBytes);
          const uint32_t d_tmem = tmem_base + ((j & 1) ? kColS1 : kColS0);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t off = (ks / 4) * L::kBoxBytes + (ks % 4) * 32;
            umma_ss(d_tmem, umma_desc_sw128(q_addr + off, 16, 1024), umma_desc_sw128(k_addr + off, 16, 1024),
                    idesc_qk, ks > 0);
          }
          umma_commit(&k_empty[s]);
          umma_commit(&s_full[j & 1]);
        }
        if (j >= 1) {
          const int jj = j - 1;
          const int s = jj % kStages;
          ok = mbar_wait_bounded(&v_full[s], (jj / kStages) & 1, abort_flag);
          if (!ok) break;
          ok = mbar_wait_bounded(&p_full[jj & 1], (jj >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t v_addr = smem_u32(v_ring + s * L::kTileBytes);
          const uint32_t p_tmem = tmem_base + ((jj & 1) ? kColP1 : kColP0);
#pragma unroll
          for (int ks = 0; ks < kBlockN / 16; ++ks) {
            // 16 keys per step: 8 packed columns of P, 16 rows (2 KB) of V
            umma_ts(tmem_base + kColO, p_tmem + ks * 8,
                    umma_desc_sw128(v_addr + ks * 2048, p.v_lbo, p.v_sbo), idesc_pv, (jj > 0) || (ks > 0));
          }
          umma_commit(&v_empty[s]);
          umma_commit(o_done);
        }
      }
      if (!ok) {
        // give-up path: let the MMAs already issued finish before TMEM is freed
        umma_commit(mma_drain);
        mbar_wait_bounded(mma_drain, 0, abort_flag + 1);
      }
    }
  } else {
    // ------------------------------ softmax -------------------------------
    const int row = (warp & 3) * 32 + lane;                       // TMEM lane = query row in the tile
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float c = p.scale_log2;
    float m_ref = -INFINITY;  // reference max (raw score units)
    float l_sum = 0.f;
    bool ok = true;
    const bool dump = p.debug != nullptr && qb == 0 && head == 0 && n_tiles > 0;

    for (int j = 0; j < n_tiles; ++j) {
      const int kb = my_idx ? __ldg(my_idx + j) : j;
      ok = mbar_wait_bounded(&s_full[j & 1], (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sr[4][32];
      const uint32_t s_addr = tmem_base + lane_sel + ((j & 1) ? kColS1 : kColS0);
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_ld32(s_addr + g * 32, sr[g]);
      tmem_wait_ld();

      // keys past kv_len (partial last block, zero-filled by TMA) are masked
      const long long key0 = static_cast<long long>(kb) * kBlockN;
      if (key0 + kBlockN > p.kv_len) {
        const int valid = static_cast<int>(p.kv_len - key0);
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (g * 32 + i >= valid) sr[g][i] = __float_as_uint(-INFINITY);
      }
      if (dump && j == 0) {
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
          for (int i = 0; i < 32; ++i) p.debug[row * 128 + g * 32 + i] = __uint_as_float(sr[g][i]);
      }

      float m_tile = -INFINITY;
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int i = 0; i < 32; ++i) m_tile = fmaxf(m_tile, __uint_as_float(sr[g][i]));

      // the previous P.V must have landed in O before O may be rescaled, and
      // waiting for it here every iteration keeps this barrier's phases in step
      if (j > 0) {
        ok = mbar_wait_bounded(o_done, (j - 1) & 1, abort_flag);
        if (!ok) break;
      }
      const bool grow = (m_tile - m_ref) * c > kRescaleThreshold;  // also true for the first tile
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, m_tile);
        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f((m_ref - m_new) * c);
        m_ref = m_new;
        l_sum *= alpha;
        if (j > 0) {
          tc_fence_after_sync();
          const uint32_t o_addr = tmem_base + lane_sel + kColO;
#pragma unroll
          for (int g = 0; g < HD / 32; ++g) {
            uint32_t o[32];
            tmem_ld32(o_addr + g * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(o_addr + g * 32, o);
          }
        }
      }
      const float neg_mc = (m_ref == -INFINITY) ? 0.f : -m_ref * c;
      const uint32_t p_addr = tmem_base + lane_sel + ((j & 1) ? kColP1 : kColP0);
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int e = g * 64 + 2 * i;  // keys e, e+1
          const float p0 = exp2f(fmaf(__uint_as_float(sr[e >> 5][e & 31]), c, neg_mc));
          const float p1 = exp2f(fmaf(__uint_as_float(sr[(e + 1) >> 5][(e + 1) & 31]), c, neg_mc));
          l_sum += p0 + p1;
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);  // key e in the low half
          packed[i] = *reinterpret_cast<const uint32_t*>(&h2);
        }
        tmem_st32(p_addr + g * 32, packed);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_full[j & 1]);
    }

    if (ok && n_tiles > 0) ok = mbar_wait_bounded(o_done, (n_tiles - 1) & 1, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      const long long tok = static_cast<long long>(qb) * kBlockM + row;
      const float inv_l = l_sum > 0.f ? 1.0f / l_sum : 0.f;
      const bool live = tok < p.seq_len;  // a row with an empty list gets zeros
      long long dst_row = tok;
      if (live && p.out_row_map) dst_row = __ldg(p.out_row_map + tok);
      __nv_bfloat16* dst = p.out + (static_cast<size_t>(head) * p.seq_len + (live ? dst_row : 0)) * HD;
      const uint32_t o_addr = tmem_base + lane_sel + kColO;
#pragma unroll
      for (int g = 0; g < HD / 32; ++g) {
        uint32_t o[32];
        if (n_tiles > 0) {
          tmem_ld32(o_addr + g * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (dump) {
#pragma unroll
          for (int i = 0; i < 32; ++i) p.debug[128 * 128 + row * HD + g * 32 + i] = __uint_as_float(o[i]);
        }
        if (live) {
#pragma unroll
          for (int v8 = 0; v8 < 4; ++v8) {
            uint4 pk;
            uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(o[v8 * 8 + 2 * t]) * inv_l,
                                                              __uint_as_float(o[v8 * 8 + 2 * t + 1]) * inv_l);
              w[t] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            reinterpret_cast<uint4*>(dst + g * 32)[v8] = pk;
          }
        }
      }
      if (dump) {
        p.debug[128 * 128 + 128 * HD + row] = l_sum;
        p.debug[128 * 128 + 128 * HD + 128 + row] = m_ref;
      }
    }
  }

  // ------------------------------- tear-down -------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0 && p.status) atomicExch(p.status, DFS_STATUS_WAIT_TIMEOUT);
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// [H, L, D] bf16 as a 3-D tensor (D innermost), box = 64 x 128 x 1, 128-byte swizzle,
// rows past L read as zero.
int make_tile_map(CUtensorMap* map, const void* base, int heads, int64_t seq_len, int head_dim) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return DFS_ERR_DRIVER;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(seq_len),
                              static_cast<cuuint64_t>(heads)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2,
                                 static_cast<cuuint64_t>(seq_len) * head_dim * 2};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(kBlockN), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : DFS_ERR_DRIVER;
}

template <int HD>
int launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Params& p, int heads,
               cudaStream_t stream) {
  using L = SmemLayout<HD>;
  DFS_CUDA_CHECK(cudaFuncSetAttribute(bsattn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      L::kAlloc));
  dim3 grid(p.q_blocks, heads);
  bsattn_fwd_kernel<HD><<<grid, kThreads, L::kAlloc, stream>>>(mq, mk, mv, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// Testing hooks: optional dump buffer for CTA (0,0) and alternative V descriptor
// strides.  Not part of the public header.
static float* g_debug_buffer = nullptr;
static uint32_t g_v_lbo = 0, g_v_sbo = 0;
extern "C" void dfs_debug_set_dump(float* device_buffer) { g_debug_buffer = device_buffer; }
extern "C" void dfs_debug_set_v_desc(uint32_t lbo, uint32_t sbo) {
  g_v_lbo = lbo;
  g_v_sbo = sbo;
}

extern "C" int dfs_block_sparse_fwd(const void* q, const void* k, const void* v, const int32_t* idx,
                                    const int32_t* cnt, int kmax, const int32_t* out_row_map, void* out,
                                    int heads, int64_t seq_len, int64_t kv_len, int head_dim, float scale,
                                    int32_t* status, void* stream_) {
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return DFS_ERR_NULL;
  if ((idx == nullptr) != (cnt == nullptr)) return DFS_ERR_NULL;
  if (!dfs_aligned16(q) || !dfs_aligned16(k) || !dfs_aligned16(v) || !dfs_aligned16(out)) return DFS_ERR_ALIGN;
  if (head_dim != 64 && head_dim != 128) return DFS_ERR_SHAPE;
  if (heads <= 0 || heads > 65535 || seq_len <= 0) return DFS_ERR_SHAPE;
  if (kv_len <= 0 || kv_len > seq_len) return DFS_ERR_RANGE;
  if (idx != nullptr && kmax <= 0) return DFS_ERR_RANGE;
  if (!(scale > 0.f)) return DFS_ERR_RANGE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  CUtensorMap mq, mk, mv;
  int rc = make_tile_map(&mq, q, heads, seq_len, head_dim);
  if (rc == 0) rc = make_tile_map(&mk, k, heads, seq_len, head_dim);
  if (rc == 0) rc = make_tile_map(&mv, v, heads, seq_len, head_dim);
  if (rc != 0) return rc;

  Params p;
  p.idx = idx;
  p.cnt = cnt;
  p.out_row_map = out_row_map;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = status;
  p.debug = g_debug_buffer;
  p.seq_len = seq_len;
  p.kv_len = kv_len;
  p.kmax = kmax;
  p.q_blocks = static_cast<int>((seq_len + kBlockM - 1) / kBlockM);
  p.k_blocks = static_cast<int>((kv_len + kBlockN - 1) / kBlockN);
  p.scale_log2 = scale * 1.4426950408889634f;
  // V tile = HD/64 boxes of [128 keys][64 dims]: 16 KB between the 64-wide
  // groups along the head dimension, 1 KB between groups of 8 keys.
  p.v_lbo = g_v_lbo ? g_v_lbo : 16384;
  p.v_sbo = g_v_sbo ? g_v_sbo : 1024;
  return head_dim == 128 ? launch_fwd<128>(mq, mk, mv, p, heads, stream)
                         : launch_fwd<64>(mq, mk, mv, p, heads, stream);
}
