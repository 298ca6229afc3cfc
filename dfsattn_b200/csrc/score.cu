// Hierarchical block scoring: 16-token mean pooling of Q and K, pooled
// Q.K^T logits, softmax over all key tiles, 8x8 tile sums -> block scores.
//
// The softmax-ed tile-score tensor of the reference ([H, 7432, 7448] at the
// 720p shape, several GB) is never materialised.  Three kernels:
//   1. pool_tiles_kernel : fp32 means of 16 consecutive (scoring-layout)
//                          tokens, stored as TWO bf16 matrices per tensor: the
//                          rounded mean ("hi") and the rounded remainder
//                          ("lo"), 16 significant bits together.
//   2. tile_lse_kernel   : pooled logits on tcgen05 tensor cores, fp32
//                          accumulate in TMEM: Qhi.Khi + Qhi.Klo + Qlo.Khi (the
//                          dropped lo.lo term is below 2^-16 relative).  For
//                          every (query tile, key BLOCK) only the base-2
//                          log-sum-exp of the 8 scaled logits of that block is
//                          kept  (H * Nq * Kb floats).
//   3. block_sum_kernel  : per query block, row max / normaliser over all key
//                          blocks from the stored LSEs (read once, held in
//                          registers), then
//                          B[c] = sum_i 2^(lse_ic - M_i) / Z_i   (= the sum of
//                          the 64 softmax-ed tile scores of the 8x8 group).
// Sums of softmax-ed scores equal the reference's fp32 results up to rounding
// (different summation order, 2^-16 operand split).
#include <math.h>
#include <stdlib.h>

#include <atomic>

#include "common.cuh"

namespace {

using namespace dfs;

constexpr int kBlock = 128;     // tokens per block
constexpr int kGemmTile = 128;  // pooled rows / columns per MMA tile
// tokens per pooled tile: 16, 32 or 64 (8, 4 or 2 tiles per block)

struct ScoreShape {
  int heads;
  long long seq_len, video_len;
  int head_dim;
  int tile;      // tokens per pooled tile
  int tpb;       // pooled tiles per block
  int q_blocks;  // rows of the block-score matrix
  int k_blocks;
  int nq, nk;          // pooled tiles (q_blocks*8, k_blocks*8)
  int nq_pad, nk_pad;  // padded to kGemmTile
  int lse_stride;      // floats per row of the stored log-sum-exps: key blocks rounded up to whole column tiles
  long long video_padded;  // Vb*128: scoring position where the text part starts
};

__host__ ScoreShape make_shape(int heads, int64_t seq_len, int64_t video_len, int head_dim, int tile,
                               int wan_layout) {
  ScoreShape s;
  s.tile = tile;
  s.tpb = kBlock / tile;
  s.heads = heads;
  s.seq_len = seq_len;
  s.video_len = wan_layout ? seq_len : video_len;
  s.head_dim = head_dim;
  s.k_blocks = static_cast<int>((seq_len + kBlock - 1) / kBlock);
  s.q_blocks = static_cast<int>((s.video_len + kBlock - 1) / kBlock);
  s.nq = s.q_blocks * s.tpb;
  s.nk = s.k_blocks * s.tpb;
  s.nq_pad = (s.nq + kGemmTile - 1) / kGemmTile * kGemmTile;
  s.nk_pad = (s.nk + kGemmTile - 1) / kGemmTile * kGemmTile;
  s.video_padded = static_cast<long long>(s.q_blocks) * kBlock;
  s.lse_stride = s.nk_pad / s.tpb;
  return s;
}

__host__ size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

// scratch layout: pooled Q as bf16 [2H][nq_pad][D] (plane 2h = hi, 2h+1 = lo), pooled K likewise,
// then the per-(query tile, key block) log-sum-exp values fp32 [H][nq][lse_stride] (rows padded to whole
// column tiles, so that a thread stores its consecutive key blocks of a tile as aligned 16-byte vectors)
struct Workspace {
  size_t qm_off, km_off, lse_off, total;
};
__host__ Workspace make_workspace(const ScoreShape& s) {
  Workspace w;
  w.qm_off = 0;
  w.km_off = align256(w.qm_off + 2 * sizeof(__nv_bfloat16) * s.heads * s.head_dim * static_cast<size_t>(s.nq_pad));
  w.lse_off = align256(w.km_off + 2 * sizeof(__nv_bfloat16) * s.heads * s.head_dim * static_cast<size_t>(s.nk_pad));
  w.total = align256(w.lse_off + sizeof(float) * s.heads * static_cast<size_t>(s.nq) * s.lse_stride);
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

// One thread: one 16-byte column chunk of one pooled tile (its rows summed in fp32), written as
// bf16 hi / lo rows.  Padding tiles are written as zeros.
template <typename T>
__global__ void __launch_bounds__(256) pool_tiles_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                         __nv_bfloat16* __restrict__ qm,
                                                         __nv_bfloat16* __restrict__ km, ScoreShape s) {
  constexpr int E = Vec16<T>::kElems;
  const int chunks = s.head_dim / E;  // 16-byte chunks per input row
  const int tiles_per_cta = blockDim.x / chunks;
  const int which = blockIdx.z;       // 0: Q, 1: K
  const int head = blockIdx.y;
  const int n_tiles = which == 0 ? s.nq : s.nk;
  const int n_pad = which == 0 ? s.nq_pad : s.nk_pad;
  const T* __restrict__ src = (which == 0 ? q : k) + static_cast<size_t>(head) * s.seq_len * s.head_dim;
  __nv_bfloat16* __restrict__ dst_hi =
      (which == 0 ? qm : km) + static_cast<size_t>(2 * head) * n_pad * s.head_dim;
  __nv_bfloat16* __restrict__ dst_lo = dst_hi + static_cast<size_t>(n_pad) * s.head_dim;

  const int tile = blockIdx.x * tiles_per_cta + threadIdx.x / chunks;
  const int ch = threadIdx.x % chunks;
  if (tile >= n_pad) return;
  float acc[E];
#pragma unroll
  for (int i = 0; i < E; ++i) acc[i] = 0.f;
  if (tile < n_tiles) {
    const long long p0 = static_cast<long long>(tile) * s.tile;
    const long long first = scoring_row(p0, s.video_len, s.video_padded, s.seq_len);
    const long long last = scoring_row(p0 + s.tile - 1, s.video_len, s.video_padded, s.seq_len);
    if (first >= 0 && last == first + s.tile - 1) {
      // the tile lies wholly inside the video or the text part (all but a handful do): its rows are
      // consecutive, four loads in flight per thread
      const uint4* __restrict__ base = reinterpret_cast<const uint4*>(src + first * s.head_dim) + ch;
      for (int r0 = 0; r0 < s.tile; r0 += 4) {  // the tile size is a multiple of 16
        uint4 raw[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) raw[r] = __ldcs(base + static_cast<size_t>(r0 + r) * chunks);
#pragma unroll
        for (int r = 0; r < 4; ++r) Vec16<T>::accumulate(raw[r], acc);
      }
    } else {  // a tile across the end of the video or of the text: row by row, skipping the zero rows
      for (int r = 0; r < s.tile; ++r) {
        const long long row = scoring_row(p0 + r, s.video_len, s.video_padded, s.seq_len);
        if (row >= 0) {
          const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + row * s.head_dim) + ch);
          Vec16<T>::accumulate(raw, acc);
        }
      }
    }
  }
  __nv_bfloat16 hi[E], lo[E];
#pragma unroll
  for (int i = 0; i < E; ++i) {
    const float mean = acc[i] / static_cast<float>(s.tile);  // exact: the tile size is a power of two
    hi[i] = __float2bfloat16_rn(mean);
    lo[i] = __float2bfloat16_rn(mean - __bfloat162float(hi[i]));
  }
  const size_t at = static_cast<size_t>(tile) * s.head_dim + ch * E;
  if constexpr (E == 8) {
    *reinterpret_cast<uint4*>(dst_hi + at) = *reinterpret_cast<const uint4*>(hi);
    *reinterpret_cast<uint4*>(dst_lo + at) = *reinterpret_cast<const uint4*>(lo);
  } else {
    *reinterpret_cast<uint2*>(dst_hi + at) = *reinterpret_cast<const uint2*>(hi);
    *reinterpret_cast<uint2*>(dst_lo + at) = *reinterpret_cast<const uint2*>(lo);
  }
}

// --------------------------------------------------------------------------
// pooled logits on tcgen05 + per-block log-sum-exp epilogue
//
// One CTA per (128 pooled query rows, head, range of key tiles); it walks its 128-column tiles of pooled keys.
//   warp 0   TMA producer: Q hi/lo once, K hi/lo tiles through a ring (2 stages; 4 half-size stages in pairs)
//   warps 1, 10  MMA issuers (one lane each, even / odd column tiles): 3 x D/16 MMAs per column tile into
//            one of four logits buffers in tensor memory (the epilogue frees a buffer as soon as it has
//            the logits in registers)
//   warps 2-9 epilogue: one thread per pooled query row and half of the 128 logits of a column tile
//            (two warps share a TMEM lane quadrant and take two of its four 32-column groups each, so a
//            scheduler has two warps to cover each other's tcgen05.ld latency); each group of 8 logits
//            (one key block) is reduced to a base-2 log-sum-exp
// Every wait is bounded; an expired wait sets *status and the CTA leaves through the common tear-down.
// --------------------------------------------------------------------------
constexpr int kLseThreads = 352;
constexpr int kLseIssuerB = 10;  // warp of the second MMA issuer
constexpr int kLseBufs = 4;      // logits buffers in tensor memory (128 columns each: all 512)

// kPair: the CTA is one of a pair that shares every pooled-K tile (see the pair notes at the kernel).
template <int HD, bool kPair>
struct LseSmem {
  static constexpr int kStages = kPair ? 4 : 2;
  static constexpr int kBoxBytes = 128 * 64 * 2;
  static constexpr int kTileBytes = kBoxBytes * (HD / 64);   // one 128-row bf16 tile (hi or lo)
  static constexpr int kKBoxBytes = kPair ? kBoxBytes / 2 : kBoxBytes;     // one box of this CTA's part of a K tile
  static constexpr int kKPartBytes = kPair ? kTileBytes / 2 : kTileBytes;  // this CTA's part of a K tile (hi or lo)
  static constexpr int kQOff = 0;                            // hi, lo
  static constexpr int kKOff = 2 * kTileBytes;               // [stage][hi, lo]
  static constexpr int kBarOff = kKOff + kStages * 2 * kKPartBytes;
  static constexpr int kNumBars = 1 + 2 * kStages + 2 * kLseBufs + 2;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 32;
};

__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// kPair: two CTAs on neighbouring SMs, launched as a cluster, take two consecutive 128-row tiles of pooled
// queries and walk the same pooled-key tiles.  Every MMA is one tcgen05.mma.cta_group::2 over 256 query rows
// issued by the even CTA (the leader); each CTA keeps its own Q tiles and its own 128 rows of the logits and
// loads only HALF (64 pooled keys) of every K tile, which the tensor cores of both SMs read.  The pooled keys
// therefore cross from L2 into shared memory once per 256 query rows instead of once per 128: with single
// CTAs this kernel is bound by exactly that traffic (64 KB per 128 x 128 logits).  The loads of both CTAs
// count on the leader's full barriers, the leader's commits go to the barriers of both CTAs, the epilogue
// warps of the other CTA release a logits buffer on the leader's barrier through its shared::cluster address,
// set-up and tear-down are cluster-wide barriers.
template <int HD, int TPB, bool kPair>
__global__ void __launch_bounds__(kLseThreads, 1)
    tile_lse_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    float* __restrict__ lse, ScoreShape s, float scale_log2, int32_t* status) {
  using L = LseSmem<HD, kPair>;
  constexpr int kStages = L::kStages;
  extern __shared__ __align__(1024) uint8_t smem[];
  const bool misaligned = (smem_u32(smem) & 1023u) != 0;
  if constexpr (!kPair) {
    if (misaligned) {
      if (threadIdx.x == 0 && status) atomicExch(status, DFS_STATUS_BAD_SMEM_ALIGNMENT);
      return;
    }
    if (status != nullptr && *reinterpret_cast<volatile int32_t*>(status) != 0) return;
  }
  uint8_t* q_tiles = smem + L::kQOff;
  uint8_t* k_ring = smem + L::kKOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;            // [stages]
  uint64_t* k_empty = k_full + kStages;   // [stages]
  uint64_t* s_full = k_empty + kStages;   // [bufs]  logits of a column tile are in TMEM buffer b
  uint64_t* s_empty = s_full + kLseBufs;  // [bufs]  the epilogue has read buffer b
  uint64_t* mma_drain = s_empty + kLseBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile uint32_t* skip_flag = tmem_slot + 3;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // pairs: rank of this CTA in its cluster of two; the even one issues the MMAs for both
  uint32_t rank = 0;
  if constexpr (kPair) rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int head = blockIdx.y;
  const int row0 = blockIdx.x * kGemmTile;  // pairs: rows past the padded pooled queries read as zeros
  // Column tiles of this CTA: the key tiles are cut into gridDim.z contiguous ranges (every (query tile,
  // key block) value is independent of the others, so small head counts still fill the GPU).  `ct`
  // below counts this CTA's tiles from zero (ring stages and barrier phases); ct0 + ct is the tile.
  const int ct_total = s.nk_pad / kGemmTile;
  const int ct_per = (ct_total + static_cast<int>(gridDim.z) - 1) / static_cast<int>(gridDim.z);
  const int ct0 = static_cast<int>(blockIdx.z) * ct_per;
  const int n_ct = ct0 >= ct_total ? 0 : (ct_total - ct0 < ct_per ? ct_total - ct0 : ct_per);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int b = 0; b < kLseBufs; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_empty[b], kPair ? 16 : 8);  // one arrival per epilogue warp (of both CTAs of a pair)
    }
    mbar_init(&mma_drain[0], 1);
    mbar_init(&mma_drain[1], 1);
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    if constexpr (kPair)
      *skip_flag = (misaligned ? 2u : 0u) |
                   ((status != nullptr && *reinterpret_cast<volatile int32_t*>(status) != 0) ? 1u : 0u);
    fence_barrier_init();
  }
  if (warp == 1) {
    if constexpr (kPair) {
      tmem_alloc_pair(tmem_slot, 128 * kLseBufs);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 128 * kLseBufs);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (kPair) cluster_sync_all(); else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Pairs: neither CTA may leave while the other still signals its barriers, so "do not start" is decided
  // together: both CTAs skip their roles when either of them wants to, and both go through the tear-down.
  bool skip = false;
  if constexpr (kPair)
    skip = (*skip_flag | ld_cluster_u32(cluster_addr(const_cast<uint32_t*>(skip_flag), rank ^ 1u))) != 0u;

  if (skip) {
    // pairs only: nothing to do, straight to the tear-down
  } else if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      if constexpr (kPair) {
        // the Q tiles of both CTAs and both halves of every K tile are counted on the LEADER's barriers,
        // which the leader arms with the bytes of the two CTAs together
        if (leader) mbar_arrive_expect_tx(q_full, 2 * 2 * L::kTileBytes);
        for (int part = 0; part < 2; ++part)
          for (int c = 0; c < HD / 64; ++c)
            tma_load_3d_pair(q_tiles + part * L::kTileBytes + c * L::kBoxBytes, &tm_q, cluster_addr(q_full, 0), c * 64,
                             row0, 2 * head + part);
      } else {
        mbar_arrive_expect_tx(q_full, 2 * L::kTileBytes);
        for (int part = 0; part < 2; ++part)
          for (int c = 0; c < HD / 64; ++c)
            tma_load_3d(q_tiles + part * L::kTileBytes + c * L::kBoxBytes, &tm_q, q_full, c * 64, row0,
                        2 * head + part);
      }
      bool ok = true;
      int issued = 0;
      for (int ct = 0; ct < n_ct; ++ct) {
        const int st = ct % kStages;
        ok = mbar_wait_bounded(&k_empty[st], ((ct / kStages) & 1) ^ 1, abort_flag);
        if (!ok) break;
        if constexpr (kPair) {
          // this CTA's 64 pooled keys of the tile (all dims), hi and lo: HD / 64 boxes of [64 keys][64 dims] each
          if (leader) mbar_arrive_expect_tx(&k_full[st], 2 * 2 * L::kKPartBytes);
          for (int part = 0; part < 2; ++part)
            for (int c = 0; c < HD / 64; ++c)
              tma_load_3d_pair(k_ring + (st * 2 + part) * L::kKPartBytes + c * L::kKBoxBytes, &tm_k,
                               cluster_addr(&k_full[st], 0), c * 64,
                               (ct0 + ct) * kGemmTile + static_cast<int>(rank) * (kGemmTile / 2), 2 * head + part);
        } else {
          mbar_arrive_expect_tx(&k_full[st], 2 * L::kTileBytes);
          for (int part = 0; part < 2; ++part)
            for (int c = 0; c < HD / 64; ++c)
              tma_load_3d(k_ring + (st * 2 + part) * L::kTileBytes + c * L::kBoxBytes, &tm_k, &k_full[st], c * 64,
                          (ct0 + ct) * kGemmTile, 2 * head + part);
        }
        ++issued;
      }
      if (!ok) {
        // drain: the copies already issued must land before the CTA may exit
        if (!kPair || leader) {
          mbar_wait_bounded(q_full, 0, abort_flag + 1);
          for (int ct = issued > kStages ? issued - kStages : 0; ct < issued; ++ct)
            mbar_wait_bounded(&k_full[ct % kStages], (ct / kStages) & 1, abort_flag + 1);
        } else {
          // the other CTA of a pair has no barrier of its own for its copies (they count on the leader's):
          // it gives them a millisecond, a thousand times what a copy from L2 or HBM takes
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000LL) {
          }
        }
      }
    }
  } else if (warp == 1 || warp == kLseIssuerB) {
    // Two issuing threads, one for the even column tiles and one for the odd ones: the pipe's issue queue is
    // shallow, so the barrier waits and commits of one thread are idle gaps in its stream of MMAs, which the
    // other thread's stream fills.
    const int par = warp == 1 ? 0 : 1;
    if (lane == 0 && leader) {
      // pairs: one instruction covers the 256 pooled query rows of both CTAs; the descriptors name the same
      // offsets in the shared memory of both
      constexpr uint32_t idesc = umma_idesc_bf16(kPair ? 2 * kGemmTile : kGemmTile, kGemmTile, 0, 0);
      const uint64_t q_hi = umma_desc_sw128(smem_u32(q_tiles), 16, 1024);
      const uint64_t q_lo = q_hi + (L::kTileBytes >> 4);
      const uint64_t k_desc0 = umma_desc_sw128(smem_u32(k_ring), 16, 1024);
      auto mma = [&](uint32_t d, uint64_t a, uint64_t b, uint32_t acc) {
        if constexpr (kPair) umma_ss_pair(d, a, b, idesc, acc); else umma_ss(d, a, b, idesc, acc);
      };
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag);
      for (int ct = par; ct < n_ct && ok; ct += 2) {
        const int st = ct % kStages, b = ct % kLseBufs;
        ok = mbar_wait_bounded(&k_full[st], (ct / kStages) & 1, abort_flag);
        if (!ok) break;
        ok = mbar_wait_bounded(&s_empty[b], ((ct / kLseBufs) & 1) ^ 1, abort_flag);  // passes at once the first time
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t k_hi = k_desc0 + static_cast<uint64_t>(st * 2) * (L::kKPartBytes >> 4);
        const uint64_t k_lo = k_hi + (L::kKPartBytes >> 4);
        const uint32_t d_tmem = tmem_base + b * 128;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint64_t q_off = (ks / 4) * (L::kBoxBytes >> 4) + (ks % 4) * 2;
          const uint64_t k_off = (ks / 4) * (L::kKBoxBytes >> 4) + (ks % 4) * 2;
          mma(d_tmem, q_hi + q_off, k_hi + k_off, ks > 0);
          mma(d_tmem, q_hi + q_off, k_lo + k_off, 1);
          mma(d_tmem, q_lo + q_off, k_hi + k_off, 1);
        }
        if constexpr (kPair) {
          umma_commit_pair(smem_u32(&k_empty[st]));
          umma_commit_pair(cluster_addr(&k_empty[st], 1));
          umma_commit_pair(smem_u32(&s_full[b]));
          umma_commit_pair(cluster_addr(&s_full[b], 1));
        } else {
          umma_commit(&k_empty[st]);
          umma_commit(&s_full[b]);
        }
      }
      if (!ok) {
        // give-up path: let the MMAs already issued finish before TMEM is freed
        if constexpr (kPair) umma_commit_pair(smem_u32(&mma_drain[par])); else umma_commit(&mma_drain[par]);
        mbar_wait_bounded(&mma_drain[par], 0, abort_flag + 1);
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;   // which two of the four 32-column groups of a tile
    const int row = row0 + quad * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    float* __restrict__ out_row = lse + (static_cast<size_t>(head) * s.nq + (row < s.nq ? row : 0)) * s.lse_stride;
    bool ok = true;
    for (int ct = 0; ct < n_ct; ++ct) {
      const int b = ct % kLseBufs;
      ok = mbar_wait_bounded(&s_full[b], (ct / kLseBufs) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      // both 32-column groups of this warp are requested before either is used
      uint32_t r[2][32];
      tmem_ld32(tmem_base + lane_sel + b * 128 + (2 * half) * 32, r[0]);
      tmem_ld32(tmem_base + lane_sel + b * 128 + (2 * half + 1) * 32, r[1]);
      tmem_wait_ld();
      // the logits are in registers: the buffer can take the tile after the next one while they are reduced
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (kPair && !leader) mbar_arrive_cluster(cluster_addr(&s_empty[b], 0)); else mbar_arrive(&s_empty[b]);
      }
#pragma unroll
      for (int gg = 0; gg < 2; ++gg) {
        const int g = 2 * half + gg;
        float res[32 / TPB];   // this thread's consecutive key blocks of the 32-column group
#pragma unroll
        for (int grp = 0; grp < 32 / TPB; ++grp) {  // one key block = TPB consecutive pooled columns
          // max of the raw logits first, then one FMA per logit: 2^(scale * (x - max))
          float mx = __uint_as_float(r[gg][grp * TPB]);
#pragma unroll
          for (int i = 1; i < TPB; ++i) mx = fmaxf(mx, __uint_as_float(r[gg][grp * TPB + i]));
          const float m = mx * scale_log2;
          float sum = 0.f;
#pragma unroll
          for (int i = 0; i < TPB; ++i) sum += ex2_approx(fmaf(__uint_as_float(r[gg][grp * TPB + i]), scale_log2, -m));
          res[grp] = m + lg2_approx(sum);
        }
        // whole 16-byte vectors: a row is padded to whole column tiles (key blocks past the last one hold
        // the value of all-zero pooled keys and are never read)
        const int kb0 = (ct0 + ct) * (kGemmTile / TPB) + g * (32 / TPB);
        if (row < s.nq) {
#pragma unroll
          for (int q4 = 0; q4 < 32 / TPB / 4; ++q4)
            *reinterpret_cast<float4*>(out_row + kb0 + 4 * q4) =
                make_float4(res[4 * q4], res[4 * q4 + 1], res[4 * q4 + 2], res[4 * q4 + 3]);
        }
      }
    }
  }

  // pairs: a cluster-wide barrier, so that neither CTA frees its tensor memory or leaves while the other one
  // may still signal its barriers or have an MMA running on it
  tc_fence_before_sync();
  if constexpr (kPair) cluster_sync_all(); else __syncthreads();
  if (abort_flag[0] != 0 && threadIdx.x == 0 && status) atomicExch(status, DFS_STATUS_WAIT_TIMEOUT);
  if constexpr (kPair) {
    if (misaligned && threadIdx.x == 0 && status) atomicExch(status, DFS_STATUS_BAD_SMEM_ALIGNMENT);
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    if constexpr (kPair) tmem_dealloc_pair(tmem_base, 128 * kLseBufs); else tmem_dealloc(tmem_base, 128 * kLseBufs);
  }
}

// One CTA per (query block, head): its pooled rows (at most 8) x Kb stored base-2 LSEs -> Kb block scores.
// Warp i holds pooled row i in registers (up to kSumVecs 16-byte vectors per lane, all loads in flight at
// once), so the array is read from memory exactly once: row maximum and normaliser by warp shuffles, the
// normalised exponentials to shared memory, then one thread per key block adds the rows' contributions.
constexpr int kSumVecs = 8;                        // rows of up to 32 * 4 * kSumVecs = 1024 key blocks
constexpr int kSumRowMax = 32 * 4 * kSumVecs;

__global__ void __launch_bounds__(256) block_sum_kernel(const float* __restrict__ lse,
                                                        float* __restrict__ block_scores, ScoreShape s) {
  extern __shared__ float4 part4[];  // [tpb][lse_stride / 4]: 2^(lse - M_i) / Z_i
  const int head = blockIdx.y;
  const int qb = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = s.lse_stride >> 2;  // lse_stride is a multiple of 16 floats
  if (warp < s.tpb) {
    const float4* __restrict__ r = reinterpret_cast<const float4*>(
        lse + (static_cast<size_t>(head) * s.nq + qb * s.tpb + warp) * s.lse_stride);
    float4 v[kSumVecs];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < kSumVecs; ++j)
      if (j * 32 < nvec) {  // uniform over the warp: vectors past the row's end cost nothing
        const int at = j * 32 + lane;
        v[j] = at < nvec ? __ldcs(r + at) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
    for (int j = 0; j < kSumVecs; ++j)
      if (j * 32 < nvec) {
        const int c = (j * 32 + lane) * 4;
        if (c + 3 >= s.k_blocks) {  // the row's last vectors: columns past the last key block hold nothing defined
          if (c + 0 >= s.k_blocks) v[j].x = -INFINITY;
          if (c + 1 >= s.k_blocks) v[j].y = -INFINITY;
          if (c + 2 >= s.k_blocks) v[j].z = -INFINITY;
          v[j].w = -INFINITY;
        }
        m = fmaxf(m, fmaxf(fmaxf(v[j].x, v[j].y), fmaxf(v[j].z, v[j].w)));
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float z = 0.f;
#pragma unroll
    for (int j = 0; j < kSumVecs; ++j)
      if (j * 32 < nvec) {
        v[j].x = ex2_approx(v[j].x - m);
        v[j].y = ex2_approx(v[j].y - m);
        v[j].z = ex2_approx(v[j].z - m);
        v[j].w = ex2_approx(v[j].w - m);
        z += (v[j].x + v[j].y) + (v[j].z + v[j].w);
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    const float inv = 1.0f / z;
    float4* dst = part4 + static_cast<size_t>(warp) * nvec;
#pragma unroll
    for (int j = 0; j < kSumVecs; ++j) {
      const int at = j * 32 + lane;
      if (at < nvec) dst[at] = make_float4(v[j].x * inv, v[j].y * inv, v[j].z * inv, v[j].w * inv);
    }
  }
  __syncthreads();
  const float* part = reinterpret_cast<const float*>(part4);
  float* __restrict__ out = block_scores + (static_cast<size_t>(head) * s.q_blocks + qb) * s.k_blocks;
  for (int c = threadIdx.x; c < s.k_blocks; c += blockDim.x) {
    float b = 0.f;
    for (int i = 0; i < s.tpb; ++i) b += part[static_cast<size_t>(i) * s.lse_stride + c];
    out[c] = b;
  }
}

// The same for rows of more than kSumRowMax key blocks: three passes over the stored values.
__global__ void __launch_bounds__(256) block_sum_long_kernel(const float* __restrict__ lse,
                                                             float* __restrict__ block_scores, ScoreShape s) {
  __shared__ float row_max[8];
  __shared__ float row_inv[8];
  const int head = blockIdx.y;
  const int qb = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* __restrict__ rows = lse + (static_cast<size_t>(head) * s.nq + qb * s.tpb) * s.lse_stride;
  if (warp < s.tpb) {
    const float* __restrict__ r = rows + static_cast<size_t>(warp) * s.lse_stride;  // warp i <-> pooled row i
    float m = -INFINITY;
    for (int c = lane; c < s.k_blocks; c += 32) m = fmaxf(m, r[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float z = 0.f;
    for (int c = lane; c < s.k_blocks; c += 32) z += exp2f(r[c] - m);
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
    for (int i = 0; i < s.tpb; ++i)
      b += exp2f(rows[static_cast<size_t>(i) * s.lse_stride + c] - row_max[i]) * row_inv[i];
    out[c] = b;
  }
}

template <typename T>
int launch_pool(const void* q, const void* k, __nv_bfloat16* qm, __nv_bfloat16* km, const ScoreShape& s,
                cudaStream_t stream) {
  const int chunks = s.head_dim / Vec16<T>::kElems;
  const int tiles_per_cta = 256 / chunks;
  const int n_pad = s.nk_pad > s.nq_pad ? s.nk_pad : s.nq_pad;
  dim3 grid((n_pad + tiles_per_cta - 1) / tiles_per_cta, s.heads, 2);
  pool_tiles_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(q), static_cast<const T*>(k), qm, km, s);
  return static_cast<int>(cudaGetLastError());
}

// Whether the logits kernel runs as CTA pairs (default) or as single CTAs.
bool score_pairs_enabled() {
  static const int flag = [] {
    const char* e = getenv("DFSATTN_SCORE_PAIRS");
    return e == nullptr ? 1 : (e[0] != '0');
  }();
  return flag != 0;
}

template <int HD, int TPB>
int launch_lse(const __nv_bfloat16* qm, const __nv_bfloat16* km, float* lse, const ScoreShape& s, float scale_log2,
               int32_t* status, cudaStream_t stream) {
  const int q_tiles = s.nq_pad / kGemmTile;
  const bool pairs = q_tiles >= 2 && score_pairs_enabled();
  CUtensorMap mq, mk;
  int rc = dfs_make_bf16_tile_map(&mq, qm, 2 * s.heads, s.nq_pad, HD);
  if (rc == 0) rc = dfs_make_bf16_tile_map(&mk, km, 2 * s.heads, s.nk_pad, HD, pairs ? 64 : 128);
  if (rc != 0) return rc;
  // at least ~4 CTAs per SM's worth of work items: split the key tiles when heads x query tiles are few
  const int ctas = q_tiles * s.heads, ct_total = s.nk_pad / kGemmTile;
  int splits = (4 * 148 + ctas - 1) / ctas;
  splits = splits < 1 ? 1 : (splits > 8 ? 8 : splits);
  if (splits > ct_total) splits = ct_total;
  if (!pairs) {
    using L = LseSmem<HD, false>;
    DFS_CUDA_CHECK(cudaFuncSetAttribute(tile_lse_kernel<HD, TPB, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        L::kTotal));
    dim3 grid(q_tiles, s.heads, splits);
    tile_lse_kernel<HD, TPB, false><<<grid, kLseThreads, L::kTotal, stream>>>(mq, mk, lse, s, scale_log2, status);
    return static_cast<int>(cudaGetLastError());
  }
  using L = LseSmem<HD, true>;
  auto kernel = tile_lse_kernel<HD, TPB, true>;
  DFS_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((q_tiles + 1) / 2 * 2), static_cast<unsigned>(s.heads),
                     static_cast<unsigned>(splits));
  cfg.blockDim = dim3(kLseThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  DFS_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, mq, mk, lse, s, scale_log2, status));
  return static_cast<int>(cudaGetLastError());
}

int check_shape(int heads, int64_t seq_len, int64_t video_len, int head_dim, int tile, int block,
                int wan_layout) {
  if (block != kBlock || (tile != 16 && tile != 32 && tile != 64)) return DFS_ERR_SHAPE;
  if (head_dim != 64 && head_dim != 128) return DFS_ERR_SHAPE;
  if (heads <= 0 || heads > 32767 || seq_len <= 0) return DFS_ERR_SHAPE;
  if (!wan_layout) {
    if (video_len <= 0 || video_len > seq_len) return DFS_ERR_RANGE;
    // The scoring layout [video | zero gap | text] must fit in Kb blocks; the
    // reference's view() fails on shapes where it does not.
    const int64_t vb = (video_len + kBlock - 1) / kBlock, kb = (seq_len + kBlock - 1) / kBlock;
    if (vb * kBlock + (seq_len - video_len) > kb * kBlock) return DFS_ERR_SHAPE;
  }
  return 0;
}

// pool -> tensor-core logits + per-block LSE -> block sums, on scratch of make_workspace(s).total bytes
int run_block_scores(const void* q_perm, const void* k_perm, int dtype, const ScoreShape& s, float* block_scores,
                     char* base, int32_t* status, cudaStream_t stream) {
  const Workspace w = make_workspace(s);
  __nv_bfloat16* qm = reinterpret_cast<__nv_bfloat16*>(base + w.qm_off);
  __nv_bfloat16* km = reinterpret_cast<__nv_bfloat16*>(base + w.km_off);
  float* lse = reinterpret_cast<float*>(base + w.lse_off);
  int err = dtype == DFS_DTYPE_BF16 ? launch_pool<__nv_bfloat16>(q_perm, k_perm, qm, km, s, stream)
                                    : launch_pool<float>(q_perm, k_perm, qm, km, s, stream);
  if (err != 0) return err;
  const float scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(s.head_dim));
  if (s.head_dim == 128)
    err = s.tpb == 8   ? launch_lse<128, 8>(qm, km, lse, s, scale_log2, status, stream)
          : s.tpb == 4 ? launch_lse<128, 4>(qm, km, lse, s, scale_log2, status, stream)
                       : launch_lse<128, 2>(qm, km, lse, s, scale_log2, status, stream);
  else
    err = s.tpb == 8   ? launch_lse<64, 8>(qm, km, lse, s, scale_log2, status, stream)
          : s.tpb == 4 ? launch_lse<64, 4>(qm, km, lse, s, scale_log2, status, stream)
                       : launch_lse<64, 2>(qm, km, lse, s, scale_log2, status, stream);
  if (err != 0) return err;
  dim3 grid(s.q_blocks, s.heads);
  if (s.lse_stride <= kSumRowMax)
    block_sum_kernel<<<grid, 256, sizeof(float) * s.tpb * s.lse_stride, stream>>>(lse, block_scores, s);
  else
    block_sum_long_kernel<<<grid, 256, 0, stream>>>(lse, block_scores, s);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

extern "C" int64_t dfs_score_workspace_bytes(int heads, int64_t seq_len, int64_t video_len, int head_dim,
                                             int tile, int block, int wan_layout) {
  const int rc = check_shape(heads, seq_len, video_len, head_dim, tile, block, wan_layout);
  if (rc != 0) return rc;
  return static_cast<int64_t>(make_workspace(make_shape(heads, seq_len, video_len, head_dim, tile, wan_layout)).total);
}

extern "C" int dfs_block_scores(const void* q_perm, const void* k_perm, int dtype, int heads, int64_t seq_len,
                                int64_t video_len, int head_dim, int tile, int block, int wan_layout,
                                float* block_scores, void* workspace, int64_t workspace_bytes, int32_t* status,
                                void* stream_) {
  if (q_perm == nullptr || k_perm == nullptr || block_scores == nullptr || workspace == nullptr)
    return DFS_ERR_NULL;
  if (!dfs_aligned16(q_perm) || !dfs_aligned16(k_perm) || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return DFS_ERR_ALIGN;
  if (dtype != DFS_DTYPE_BF16 && dtype != DFS_DTYPE_F32) return DFS_ERR_DTYPE;
  const int rc = check_shape(heads, seq_len, video_len, head_dim, tile, block, wan_layout);
  if (rc != 0) return rc;
  const ScoreShape s = make_shape(heads, seq_len, video_len, head_dim, tile, wan_layout);
  const Workspace w = make_workspace(s);
  if (workspace_bytes < static_cast<int64_t>(w.total)) return DFS_ERR_WORKSPACE;
  return run_block_scores(q_perm, k_perm, dtype, s, block_scores, static_cast<char*>(workspace), status,
                          static_cast<cudaStream_t>(stream_));
}

// --------------------------------------------------------------------------
// Fine top-p inside the chosen block pairs ("kp" selector)
//
// For every listed (query block, key block) pair of the refinable region the 8 x 8 softmax-ed
// tile scores are recomputed from the pooled means and the stored log-sum-exps that the block
// scoring left in its scratch, ranked jointly (larger first), and a tile is kept while the scores ranked
// before it sum to less than top_p times the pair's total.  Result: one 64-bit map per list
// entry, bit 8 * (query tile) + (key tile).  One CTA per (query block, head), one warp per pair.
// --------------------------------------------------------------------------
namespace {

constexpr int kFineWarps = 8;

// D += A . B for a 16 x 8 x 16 bf16 tile with fp32 accumulation; rows 8..15 of A are zero (a1 = a3 = 0),
// so only c[0], c[1] (row lane / 4, columns 2 * (lane % 4) and + 1) carry results.
__device__ __forceinline__ void mma_16x8x16_bf16(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

template <int HD>
__global__ void __launch_bounds__(kFineWarps * 32, 3)
fine_top_p_kernel(const __nv_bfloat16* __restrict__ qm, const __nv_bfloat16* __restrict__ km,
                  const float* __restrict__ lse, const int32_t* __restrict__ idx, const int32_t* __restrict__ cnt,
                  unsigned long long* __restrict__ bits, ScoreShape s, int q_rows, int kmax, int n_rank,
                  int dense_row_start, float top_p, float scale_log2) {
  __shared__ float row_lse[8];
  __shared__ uint4 q_s[2][8][HD / 8 + 4];
  const int head = blockIdx.y, qb = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t list_at = (static_cast<size_t>(head) * q_rows + qb) * kmax;
  const int listed = cnt[static_cast<size_t>(head) * q_rows + qb];
  const int n_list = listed > 0 ? listed : 0;  // -1 (a row that attends every block) has no list: maps unused
  const bool dense_row = qb >= dense_row_start || qb >= s.q_blocks;
  if (dense_row) {  // rows from the first boundary block on keep whole blocks
    for (int slot = threadIdx.x; slot < kmax; slot += blockDim.x) bits[list_at + slot] = slot < n_list ? ~0ull : 0ull;
    return;
  }
  // normaliser of each of the 8 pooled query rows over ALL key tiles: log2 sum_c 2^lse[i][c]
  {
    const float* __restrict__ r = lse + (static_cast<size_t>(head) * s.nq + qb * 8 + warp) * s.lse_stride;
    float m = -INFINITY;
    for (int c = lane; c < s.k_blocks; c += 32) m = fmaxf(m, r[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float z = 0.f;
    for (int c = lane; c < s.k_blocks; c += 32) z += exp2f(r[c] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    if (lane == 0) row_lse[warp] = m + log2f(z);
  }
  __syncthreads();

  // The 8 x 8 logits of a pair are one 16 x 8 x HD warp-level MMA with the upper 8 rows unused.  In its
  // fragment layout lane (g = lane / 4, t = lane % 4) holds query row g and key row g at two column
  // pairs of every 16-column step, straight from the bf16 hi / lo planes, and receives the logits
  // (query tile g, key tiles 2t and 2t + 1).  Same three products as the block scoring:
  // hi.hi + hi.lo + lo.hi with fp32 accumulation.
  // The contraction does not care in which order the columns are visited as long as both operands
  // visit them in the same order, so a lane takes 16 contiguous bytes (columns 8t .. 8t + 7 of a
  // 32-column span) per row and plane with one load and feeds them to two MMA steps.
  constexpr int kSpans = HD / 32;
  const int g = lane >> 2, t = lane & 3;
  // The pooled query rows (both planes) wait in shared memory, 320-byte row pitch: the eight lanes of a
  // 16-byte access phase (two rows) then fall on different banks.
  for (int e = threadIdx.x; e < 2 * 8 * (HD / 8); e += blockDim.x) {
    const int plane = e / (8 * (HD / 8)), row = (e / (HD / 8)) % 8, c = e % (HD / 8);
    const __nv_bfloat16* src = qm + (static_cast<size_t>(2 * head + plane) * s.nq_pad + qb * 8 + row) * HD;
    q_s[plane][row][c] = __ldg(reinterpret_cast<const uint4*>(src) + c);
  }
  // Lists are ascending (dfs_select_topk writes them so): the refinable entries, key blocks below
  // n_rank, are a prefix of the list.
  int n_ref = 0;
  for (int base = 0; base < n_list; base += blockDim.x) {
    const int slot = base + threadIdx.x;
    n_ref += __syncthreads_count(slot < n_list && idx[list_at + slot] < n_rank);
  }
  __syncthreads();
  for (int slot = n_ref + threadIdx.x; slot < kmax; slot += blockDim.x)
    bits[list_at + slot] = slot < n_list ? ~0ull : 0ull;  // forced (text / boundary) blocks stay whole; unused slots

  const int qi = g;  // this lane's two tiles: (qi, 2t) and (qi, 2t + 1)
  const float my_lse = row_lse[qi];
  // operands of the NEXT pair are requested before the current pair is ranked
  uint4 nh[kSpans], nl[kSpans];
  auto request = [&](int slot) {
    const int kb = idx[list_at + slot];
    const __nv_bfloat16* __restrict__ hi = km + (static_cast<size_t>(2 * head) * s.nk_pad + kb * 8 + g) * HD;
    const __nv_bfloat16* __restrict__ lo = hi + static_cast<size_t>(s.nk_pad) * HD;
#pragma unroll
    for (int sp = 0; sp < kSpans; ++sp) {
      nh[sp] = __ldg(reinterpret_cast<const uint4*>(hi) + sp * 4 + t);
      nl[sp] = __ldg(reinterpret_cast<const uint4*>(lo) + sp * 4 + t);
    }
  };
  if (warp < n_ref) request(warp);
  for (int slot = warp; slot < n_ref; slot += kFineWarps) {
    uint4 kh[kSpans], kl[kSpans];
#pragma unroll
    for (int sp = 0; sp < kSpans; ++sp) {
      kh[sp] = nh[sp];
      kl[sp] = nl[sp];
    }
    if (slot + kFineWarps < n_ref) request(slot + kFineWarps);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int sp = 0; sp < kSpans; ++sp) {
      const uint4 qh = q_s[0][g][sp * 4 + t], ql = q_s[1][g][sp * 4 + t];
      mma_16x8x16_bf16(acc, qh.x, qh.y, kh[sp].x, kh[sp].y);
      mma_16x8x16_bf16(acc, qh.z, qh.w, kh[sp].z, kh[sp].w);
      mma_16x8x16_bf16(acc, qh.x, qh.y, kl[sp].x, kl[sp].y);
      mma_16x8x16_bf16(acc, qh.z, qh.w, kl[sp].z, kl[sp].w);
      mma_16x8x16_bf16(acc, ql.x, ql.y, kh[sp].x, kh[sp].y);
      mma_16x8x16_bf16(acc, ql.z, ql.w, kh[sp].z, kh[sp].w);
    }
    const float d0 = acc[0], d1 = acc[1];
    const float v0 = exp2f(fmaf(d0, scale_log2, -my_lse)), v1 = exp2f(fmaf(d1, scale_log2, -my_lse));
    // Rank the 64 scores, largest first, with a bitonic sort over the warp (two per lane) on their bit
    // patterns (non-negative floats order like unsigned integers).  Only the values travel: the kept
    // tiles are the ranks whose preceding mass is below the limit, i.e. all scores down to the
    // smallest kept one, which every lane then compares with the two scores it still holds.  (Scores
    // exactly equal to that smallest kept one are all kept.)
    const uint32_t u0 = __float_as_uint(v0), u1 = __float_as_uint(v1);
    uint32_t k0 = u0, k1 = u1;
#pragma unroll
    for (int k = 2; k <= 64; k <<= 1) {
      const bool desc = ((2 * lane) & k) == 0;  // direction of this element's block in this round
#pragma unroll
      for (int j = k >> 1; j > 0; j >>= 1) {
        if (j == 1) {  // the partner is the lane's other element
          const uint32_t big = max(k0, k1), small = min(k0, k1);
          k0 = desc ? big : small;
          k1 = desc ? small : big;
        } else {
          const uint32_t o0 = __shfl_xor_sync(0xffffffffu, k0, j >> 1);
          const uint32_t o1 = __shfl_xor_sync(0xffffffffu, k1, j >> 1);
          const bool take_max = (((lane & (j >> 1)) == 0) == desc);
          k0 = take_max ? max(k0, o0) : min(k0, o0);
          k1 = take_max ? max(k1, o1) : min(k1, o1);
        }
      }
    }
    // rank 2 * lane holds k0, rank 2 * lane + 1 holds k1: mass ranked before each of them
    const float a = __uint_as_float(k0), b = __uint_as_float(k1);
    float inc = a + b;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += up;
    }
    const float before0 = inc - (a + b), before1 = before0 + a;
    const float limit = __shfl_sync(0xffffffffu, inc, 31) * top_p;
    // smallest kept score (rank 0 is always kept: nothing precedes it)
    const uint32_t mine = before1 < limit ? k1 : (before0 < limit ? k0 : 0xffffffffu);
    const uint32_t cutoff = __reduce_min_sync(0xffffffffu, mine);
    const uint32_t pair_bits = (u0 >= cutoff ? 1u : 0u) | (u1 >= cutoff ? 2u : 0u);  // tiles 2 * lane, 2 * lane + 1
    const uint32_t half = __reduce_or_sync(lane < 16 ? 0x0000ffffu : 0xffff0000u, pair_bits << (2 * (lane & 15)));
    const uint32_t word = __shfl_sync(0xffffffffu, half, 0), hi_word = __shfl_sync(0xffffffffu, half, 16);
    if (lane == 0) bits[list_at + slot] = (static_cast<unsigned long long>(hi_word) << 32) | word;
  }
}

}  // namespace

extern "C" int dfs_fine_top_p(const void* workspace, int64_t workspace_bytes, int heads, int64_t seq_len,
                              int64_t video_len, int head_dim, int tile, int block, int wan_layout,
                              const int32_t* idx, const int32_t* cnt, int kmax, int q_rows, int n_rank,
                              int dense_row_start, float fine_top_p, uint64_t* fine_bits, void* stream_) {
  if (workspace == nullptr || idx == nullptr || cnt == nullptr || fine_bits == nullptr) return DFS_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 || (reinterpret_cast<uintptr_t>(fine_bits) & 7u) != 0)
    return DFS_ERR_ALIGN;
  const int rc = check_shape(heads, seq_len, video_len, head_dim, tile, block, wan_layout);
  if (rc != 0) return rc;
  if (tile != 16) return DFS_ERR_SHAPE;  // the maps are 8 x 8: 16-token tiles inside 128-token blocks
  const ScoreShape s = make_shape(heads, seq_len, video_len, head_dim, tile, wan_layout);
  const Workspace w = make_workspace(s);
  if (workspace_bytes < static_cast<int64_t>(w.total)) return DFS_ERR_WORKSPACE;
  if (kmax <= 0 || q_rows < s.q_blocks || q_rows > s.k_blocks || n_rank < 0 || n_rank > s.k_blocks ||
      dense_row_start < 0)
    return DFS_ERR_RANGE;
  if (!(fine_top_p > 0.f)) return DFS_ERR_RANGE;
  const char* base = static_cast<const char*>(workspace);
  const __nv_bfloat16* qm = reinterpret_cast<const __nv_bfloat16*>(base + w.qm_off);
  const __nv_bfloat16* km = reinterpret_cast<const __nv_bfloat16*>(base + w.km_off);
  const float* lse = reinterpret_cast<const float*>(base + w.lse_off);
  const float scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(head_dim));
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  dim3 grid(q_rows, heads);
  auto* out = reinterpret_cast<unsigned long long*>(fine_bits);
  if (head_dim == 128)
    fine_top_p_kernel<128><<<grid, kFineWarps * 32, 0, stream>>>(qm, km, lse, idx, cnt, out, s, q_rows, kmax, n_rank,
                                                                 dense_row_start, fine_top_p, scale_log2);
  else
    fine_top_p_kernel<64><<<grid, kFineWarps * 32, 0, stream>>>(qm, km, lse, idx, cnt, out, s, q_rows, kmax, n_rank,
                                                                dense_row_start, fine_top_p, scale_log2);
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
// cudaGetSymbolAddress, asked once per device with that device current.  The
// slots are atomics: two host threads that make the first call on one device at
// the same time both look the address up and store the same value.  The address
// belongs to the device's primary context: after cudaDeviceReset() the slot is
// stale (the process must not call this entry point again on that device).
std::atomic<char*> g_static_scratch_addr[kMaxDevices];

int static_scratch_for_current_device(char** out) {
  int dev = -1;
  DFS_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return DFS_ERR_RANGE;
  char* addr = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (addr == nullptr) {
    void* ptr = nullptr;
    DFS_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (ptr == nullptr) return DFS_ERR_NULL;
    addr = static_cast<char*>(ptr);
    g_static_scratch_addr[dev].store(addr, std::memory_order_release);
  }
  *out = addr;
  return 0;
}
}  // namespace

extern "C" int64_t dfs_block_scores_static_max_bytes(void) { return static_cast<int64_t>(kStaticScratchBytes); }

extern "C" int dfs_block_scores_static(const void* q_perm, const void* k_perm, int dtype, int heads,
                                       int64_t seq_len, int64_t video_len, int head_dim, int tile, int block,
                                       int wan_layout, float* block_scores, int32_t* status, void* stream_) {
  if (q_perm == nullptr || k_perm == nullptr || block_scores == nullptr) return DFS_ERR_NULL;
  if (!dfs_aligned16(q_perm) || !dfs_aligned16(k_perm)) return DFS_ERR_ALIGN;
  if (dtype != DFS_DTYPE_BF16 && dtype != DFS_DTYPE_F32) return DFS_ERR_DTYPE;
  const int rc = check_shape(heads, seq_len, video_len, head_dim, tile, block, wan_layout);
  if (rc != 0) return rc;
  const ScoreShape s = make_shape(heads, seq_len, video_len, head_dim, tile, wan_layout);
  const Workspace w = make_workspace(s);
  if (w.total > kStaticScratchBytes) return DFS_ERR_STATIC_SCRATCH;  // shape needs more than the fixed array
  char* base = nullptr;
  const int rs = static_scratch_for_current_device(&base);
  if (rs != 0) return rs;
  // Nothing in the scratch has to start at zero: the pooling kernel writes every
  // element of the pooled matrices (padding included) and the block-sum kernel
  // reads only LSE entries the logits kernel has just written, so whatever the
  // previous call left behind is never read.
  return run_block_scores(q_perm, k_perm, dtype, s, block_scores, base, status,
                          static_cast<cudaStream_t>(stream_));
}
