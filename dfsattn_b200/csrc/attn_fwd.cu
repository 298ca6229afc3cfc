// Block-sparse attention forward for sm_100a: online softmax over the selected
// 128-token key blocks of each 128-token query block.
//
// One CTA per (query block, head), 12 warps:
//   warp 0      TMA producer: the Q tile once, then the K and V tiles of every
//               listed key block into two 3-stage shared-memory rings
//               (full/empty mbarrier per stage; a K slot is released by the barrier that
//               announces its scores).
//   warps 1, 2  MMA issuers (one lane each), warp 1 for the even steps, warp 2 for the
//               odd ones.  For its step j a thread issues O += P(j) V(j)
//               (tcgen05.mma TS form: P read from TMEM, V as MN-major B operand)
//               and straight after it S = Q K(j+3)^T (SS form) into the score
//               tile that P(j) lives in; the MMAs of one thread execute in issue
//               order, so that tile is reused without a completion wait.  Three
//               score tiles, not two: every hand-over between the tensor pipe and
//               the softmax costs a few hundred cycles of latency, and with two
//               steps in flight the pipe ran out of independent work during
//               those gaps.  Two issuing threads instead of one: the tensor
//               pipe's issue queue is shallow, so every commit or barrier wait
//               of an issuing thread is an idle gap in its stream of MMAs; with
//               two independent streams one fills the other's gaps.  Warp 1
//               owns the TMEM allocation.
//   warps 4-11  softmax: every warp owns 16 query rows and all 128 score columns
//               (tcgen05.ld shape 16x256b: a row lives in four threads, so row
//               maxima and sums are two shuffles and no warp depends on another).
//               Per step: load the scores, exp2 in the log2 domain with packed
//               fp32x2 arithmetic against the current reference maximum of the
//               row (no maxima of the tile itself are taken), P as packed bf16
//               over the first half of the score buffer it came from (tcgen05.st
//               shape 16x128b).  The reference maximum moves, and O is rescaled in
//               TMEM, only when a partial row sum shows that some score lies 2^60
//               above it (then the tile is read again and redone); sum and P use
//               the same reference maximum, so the result is exact.
//               Epilogue: normalise, store bf16 rows, optionally through a row
//               map (fused inverse permutation).
//   warp 3      idle (keeps the softmax warps aligned to TMEM lane quadrants).
//
// Shared memory (HD = 128): Q 32 KB + 3 x 32 KB K stages + 3 x 32 KB V stages.
// Tiles are stored as [128 rows][64 bf16] boxes with the 128-byte TMA swizzle:
// the canonical K-major (Q, K) and MN-major (V) tcgen05 operand layout.
// TMEM (512 columns): S0 | S1 | S2 | O; P(j) lives in the first 64 columns of S[j % 3].
//
// Every wait is bounded; on expiry the CTA records DFS_STATUS_WAIT_TIMEOUT,
// drains its copies and MMAs in flight, frees its TMEM and returns.
#include <stdlib.h>

#include "common.cuh"

namespace {

using namespace dfs;

constexpr int kBlockM = 128;  // query rows per CTA
constexpr int kBlockN = 128;  // keys per tile
constexpr int kThreads = 384;
constexpr int kStagesSingle = 3;  // K and V ring depth, one CTA per query block
constexpr int kStagesPair = 3;    // the same for a CTA of a pair (its stages are half as large)
constexpr uint32_t kTmemCols = 512;
// Tensor memory: three score buffers of 128 fp32 columns and the output accumulator.  P(j) (packed
// bf16 pairs, 64 columns) is written over the first half of the score buffer it was computed from:
// a warp has read all 128 columns of its rows before it stores any, and Q.K^T(j+3) waits for P.V(j).
constexpr int kSBufs = 3;
constexpr uint32_t kColO = 384;
__device__ __forceinline__ uint32_t s_col(int j) { return static_cast<uint32_t>(j % kSBufs) * 128u; }
// The softmax takes its exponentials against the row's current reference maximum without looking at the tile's
// own maximum first.  The reference only has to keep the exponentials inside the range of fp32 and bf16 (both
// reach 2^127; relative precision does not depend on the scale), so it is moved only when a thread's partial
// row sum of the tile exceeds this bound (or is not finite): then some score lies far above the reference,
// and the tile is redone with the separate maximum pass.  A sum below the bound means every exponential is.
constexpr float kSumBound = 1.0e18f;  // ~2^60: room for 2^17 keys times 2^60 below 2^127

// kPair: the CTA is one of a pair that shares every K and V tile (see the pair notes at the kernel).
// It then holds HALF of each: 64 of the 128 keys of a K tile (all dims: boxes of [64 rows][64 bf16]) and 64
// of the 128 dims of a V tile (all keys: one [128 rows][64 bf16] box).
template <int HD, bool kPair>
struct SmemLayout {
  static constexpr int kStages = kPair ? kStagesPair : kStagesSingle;
  static constexpr int kBoxBytes = kBlockN * 64 * 2;        // one [128][64] bf16 box
  static constexpr int kTileBytes = kBoxBytes * (HD / 64);  // one whole Q / K / V tile
  static constexpr int kKBoxBytes = kPair ? kBoxBytes / 2 : kBoxBytes;   // one box of this CTA's part of a K tile
  static constexpr int kStageBytes = kPair ? kTileBytes / 2 : kTileBytes;  // this CTA's part of a K or V tile
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kTileBytes;
  static constexpr int kVOff = kKOff + kStages * kStageBytes;
  static constexpr int kBarOff = kVOff + kStages * kStageBytes;
  static constexpr int kNumBars = 1 + 3 * kStages + kSBufs + kSBufs + 2;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;      // tmem address, two give-up flags, skip flag
  static constexpr int kTotal = kMiscOff + 16;
};

struct Params {
  const int32_t* idx;   // [H, Qb, kmax] or nullptr (all key blocks)
  const int32_t* cnt;   // [H, Qb]; -1 = every key block
  // [H, Qb, kmax] or nullptr: per listed block a 64-bit map of its 16 x 16-token tiles, bit 8 * i + j =
  // (query tile i, key tile j) is attended; read only by the kFine instantiation
  const unsigned long long* fine;
  const int32_t* out_row_map;
  __nv_bfloat16* out;
  int32_t* status;
  long long seq_len;
  long long kv_len;
  long long out_head_stride;   // elements between heads of the output
  long long out_token_stride;  // elements between tokens of the output
  // Output scattered over sequence shards held by several GPUs (0 = off): token d goes to shard
  // d / out_shard_rows, which is [H_total, out_shard_stride rows, D]; this launch's head h is head
  // out_head0 + h there.  Peer shards are written with plain stores over NVLink.
  __nv_bfloat16* out_shard[8];
  long long out_shard_rows;
  long long out_shard_stride;
  int out_head0;
  // Batched launch: the grid's heads are `batch` groups of list_heads heads each; head h reads the
  // lists of head h % list_heads and writes group h / list_heads of the output.
  int list_heads;
  long long out_batch_stride;  // elements between two groups of the output
  int kmax;
  int q_blocks, k_blocks;
  float scale_log2;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint64_t add2_rm(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// exp2 of two values on the FMA pipe instead of the special-function unit, which is the
// scarcest resource of the softmax (16 results per clock per SM).  floor(x) through the
// 1.5 * 2^23 magic add rounded down, a degree-3 polynomial of the fraction (relative error
// below 1e-4, far under the bf16 rounding of P), the exponent added into the float's bits.
__device__ __forceinline__ void exp2_poly2(uint64_t x, float& y0, float& y1) {
  constexpr float kMagic = 12582912.f;
  float x0, x1;
  unpack2(x, x0, x1);
  x = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));  // keeps the exponent arithmetic in range; 2^-126 ~ 0
  const uint64_t j = add2_rm(x, pack2(kMagic, kMagic));
  const uint64_t fl = add2(j, pack2(-kMagic, -kMagic));
  const uint64_t f = fma2(fl, pack2(-1.f, -1.f), x);
  uint64_t q = fma2(f, pack2(0.07711909f, 0.07711909f), pack2(0.22756439f, 0.22756439f));
  q = fma2(q, f, pack2(0.69514614f, 0.69514614f));
  q = fma2(q, f, pack2(1.0f, 1.0f));
  float q0, q1, j0, j1;
  unpack2(q, q0, q1);
  unpack2(j, j0, j1);
  y0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(j0) << 23));
  y1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(j1) << 23));
}
__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// Columns past `valid` of a score tile held as a 16x256b fragment (thread t of a row's four holds
// columns 8i + 2t, 8i + 2t + 1 of every group i, for two rows) become -inf.
__device__ __forceinline__ void mask_tail(uint32_t (&r)[64], int valid, int t4) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int col = 8 * i + 2 * t4;
    if (col >= valid) r[4 * i] = r[4 * i + 2] = __float_as_uint(-INFINITY);
    if (col + 1 >= valid) r[4 * i + 1] = r[4 * i + 3] = __float_as_uint(-INFINITY);
  }
}

// One pass over a thread's share of a score tile (two rows a and b): P = exp2(S*c - m*c) packed as
// bf16 pairs (P column 4i + t of a row = keys 8i + 2t, 8i + 2t + 1) and the tile's partial row sums.
// The first kPoly groups take their exponentials on the FMA pipe.  With kFine, key tile t (columns
// 16t .. 16t + 15: groups 2t and 2t + 1) takes part only if bit t of `keep` is set; the 16 rows of a
// softmax warp are one query tile, so the test is uniform over the warp and a dropped tile costs two
// stores of zero.
template <int kPoly, bool kFine>
__device__ __forceinline__ void exp_pass(const uint32_t (&r)[64], uint64_t c2, uint64_t nma2, uint64_t nmb2,
                                         uint32_t (&packed)[32], uint64_t& ta0, uint64_t& ta1, uint64_t& tb0,
                                         uint64_t& tb1, uint32_t keep) {
  ta0 = ta1 = tb0 = tb1 = pack2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (kFine && !((keep >> (i >> 1)) & 1u)) {
      packed[2 * i] = packed[2 * i + 1] = 0u;
      continue;
    }
    const float sa0 = __uint_as_float(r[4 * i]), sa1 = __uint_as_float(r[4 * i + 1]);
    const float sb0 = __uint_as_float(r[4 * i + 2]), sb1 = __uint_as_float(r[4 * i + 3]);
    const uint64_t xa = fma2(pack2(sa0, sa1), c2, nma2);
    const uint64_t xb = fma2(pack2(sb0, sb1), c2, nmb2);
    float a0, a1, b0, b1;
    if (i < kPoly) {
      exp2_poly2(xa, a0, a1);
      exp2_poly2(xb, b0, b1);
    } else {
      unpack2(xa, a0, a1);
      unpack2(xb, b0, b1);
      a0 = ex2(a0);
      a1 = ex2(a1);
      b0 = ex2(b0);
      b1 = ex2(b1);
    }
    if (i & 1) {
      ta1 = add2(ta1, pack2(a0, a1));
      tb1 = add2(tb1, pack2(b0, b1));
    } else {
      ta0 = add2(ta0, pack2(a0, a1));
      tb0 = add2(tb0, pack2(b0, b1));
    }
    packed[2 * i] = cvt_bf16x2(a0, a1);      // row a (even key in the low half)
    packed[2 * i + 1] = cvt_bf16x2(b0, b1);  // row b
  }
}

// Of the 16 column groups of a score tile, how many have their exp2 evaluated by the polynomial
// on the FMA pipe instead of the special-function unit.  Measured (same box, alternated): for D = 128, 1 and 2
// are equal in short bursts and 1 is 0.5-0.8 % faster in a sustained loop at the power cap (none: 3-5 %
// slower; 3 and 4: 1-2 % slower); 3 for D = 64 (2 to 5 within 2 %, 6 and 8 slower).
#ifndef DFS_POLY_GROUPS_D128
#define DFS_POLY_GROUPS_D128 1
#endif
#ifndef DFS_POLY_GROUPS_D64
#define DFS_POLY_GROUPS_D64 3
#endif

// kPair (dense calls, HD = 128): two CTAs on neighbouring SMs, launched as a cluster, take two
// consecutive query blocks and walk the same key blocks.  Every MMA is one tcgen05.mma.cta_group::2 over
// 256 query rows issued by the even CTA (the leader): each CTA contributes its own Q tile (or its own P in
// tensor memory) and receives its own 128 rows of the result in its own tensor memory, and each CTA loads
// only HALF of every K and V tile, which the tensor cores of both SMs read.  K and V therefore cross from
// L2 into shared memory once per 256 query rows instead of once per 128.  What changes against the
// single-CTA form: the TMA loads of both CTAs count on the leader's full barriers; the leader's commits go
// to the barriers of both CTAs (two commits, one per CTA); the softmax warps of the other CTA arrive on the
// leader's P barrier through its shared::cluster address (a plain arrive: with cluster-scope release
// semantics on it every softmax warp lost ~700 cycles per step, and what it publishes, P in tensor memory,
// is ordered by the tcgen05 fences anyway); set-up and tear-down are cluster-wide barriers.  Everything a
// softmax warp waits on is a barrier of its own CTA.  Measured against single CTAs on the dense call:
// 1 239 against 1 200 TFLOP/s in bursts (Wan 480p, 8 heads), 157.6 against 162.5 ms sustained at the
// HunyuanVideo 720p shape.  Listed (sparse) rows stay single: neighbouring query blocks share only a
// third of their key blocks.
template <int HD, bool kFine, bool kPair>
__global__ void __launch_bounds__(kThreads, 1)
    bsattn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const Params p) {
  static_assert(!kPair || (HD == 128 && !kFine), "pairs: dense calls with 128-wide heads");
  using L = SmemLayout<HD, kPair>;
  constexpr int kStages = L::kStages;
  constexpr int kPolyGroups = HD == 128 ? DFS_POLY_GROUPS_D128 : DFS_POLY_GROUPS_D64;
  extern __shared__ __align__(1024) uint8_t smem[];
  const bool misaligned = (smem_u32(smem) & 1023u) != 0;  // the swizzled tiles need 1024-byte alignment
  if constexpr (!kPair) {
    if (misaligned) {
      if (threadIdx.x == 0 && p.status) atomicExch(p.status, DFS_STATUS_BAD_SMEM_ALIGNMENT);
      return;
    }
    // a CTA that starts after another one has given up does no work: one expired wait must not
    // cost a wait limit per remaining CTA
    if (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) return;
  }
  uint8_t* q_tile = smem + L::kQOff;
  uint8_t* k_ring = smem + L::kKOff;
  uint8_t* v_ring = smem + L::kVOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;            // [3]  TMA -> Q.K^T issuer
  uint64_t* v_full = k_full + kStages;    // [3]  TMA -> P.V issuer
  uint64_t* v_empty = v_full + kStages;   // [3]  P.V(j) completed: V slot j%3 is free and O holds step j
  uint64_t* s_full = v_empty + kStages;   // [3]  Q.K^T issuer -> softmax: scores of step j are in S[j%3] (and K slot j%3 is free)
  uint64_t* p_full = s_full + kSBufs;     // [3]  softmax -> P.V issuer: P(j) is in the first half of S[j%3]
  uint64_t* mma_drain = p_full + kSBufs;  // [2]  give-up path of the two issuers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* skip_flag = tmem_slot + 3;  // pairs only: this CTA would rather not start (see below)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // pairs: rank of this CTA in its cluster of two; the even one issues the MMAs for both
  uint32_t rank = 0;
  if constexpr (kPair) rank = cluster_ctarank();
  const bool leader = rank == 0;
  // single CTAs: heavy rows (the dense text rows sit at the end) are scheduled first.  Pairs: CTA r of
  // pair i takes query block 2 i + r; with an odd number of blocks the last CTA has no rows (its Q tile
  // reads as zeros and nothing is stored), but it still loads its halves of K and V for its partner.
  const int qb = kPair ? static_cast<int>(blockIdx.x) : p.q_blocks - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y;                 // row of the Q/K/V tensors
  const int group = head / p.list_heads;       // batch element
  const int lhead = head - group * p.list_heads;  // head within the batch element: lists and output
  // a negative count marks a row that attends every key block (no list is read for it)
  const int listed = p.idx ? p.cnt[static_cast<size_t>(lhead) * p.q_blocks + qb] : -1;
  const int n_tiles = listed >= 0 ? listed : p.k_blocks;
  const int32_t* __restrict__ my_idx =
      listed >= 0 ? p.idx + (static_cast<size_t>(lhead) * p.q_blocks + qb) * p.kmax : nullptr;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < kSBufs; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], kPair ? 16 : 8);  // one arrival per softmax warp (of both CTAs of a pair)
    }
    for (int b = 0; b < 2; ++b) mbar_init(&mma_drain[b], 1);
    abort_flag[0] = 0;  // set by the first wait that expires
    abort_flag[1] = 0;  // separate limit for the drain waits of the give-up path
    if constexpr (kPair)
      *skip_flag = (misaligned ? 2u : 0u) |
                   ((p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) ? 1u : 0u);
    fence_barrier_init();
  }
  if (warp == 1) {
    if constexpr (kPair) {
      tmem_alloc_pair(tmem_slot, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (kPair) cluster_sync_all(); else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Pairs: neither CTA may leave while the other still signals its barriers, so "do not start" (a failure
  // was recorded earlier, or the shared memory is misaligned) is decided together: both CTAs skip their
  // roles when either of them wants to, and both still go through the common tear-down.
  bool skip = false;
  if constexpr (kPair) skip = (*skip_flag | ld_cluster_u32(cluster_addr(skip_flag, rank ^ 1u))) != 0u;

  if (skip) {
    // pairs only: nothing to do, straight to the tear-down
  } else if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      if constexpr (kPair) {
        // both Q tiles and both halves of every K and V tile are counted on the LEADER's barriers, which
        // the leader arms with the bytes of the two CTAs together
        if (leader) mbar_arrive_expect_tx(q_full, 2 * L::kTileBytes);
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d_pair(q_tile + c * L::kBoxBytes, &tm_q, cluster_addr(q_full, 0), c * 64, qb * kBlockM, head);
      } else {
        mbar_arrive_expect_tx(q_full, L::kTileBytes);
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d(q_tile + c * L::kBoxBytes, &tm_q, q_full, c * 64, qb * kBlockM, head);
      }
      bool ok = true;
      int issued_k = 0, issued_v = 0;
      int s = 0;
      uint32_t ph = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int kb = my_idx ? __ldg(my_idx + j) : j;
        // The K ring is as deep as there are score tiles, so "Q.K^T(j) has completed" (the K slot is
        // free) and "the scores of step j are there" are the same event: one commit signals both (every
        // commit is an idle gap in the issuing thread's stream of MMAs).
        static_assert(kStages == kSBufs, "K slots are released through the score barriers");
        ok = mbar_wait_bounded(&s_full[s], ph ^ 1, abort_flag);  // passes at once in the first round
        if (!ok) break;
        if constexpr (kPair) {
          // this CTA's 64 keys of the tile (all dims): HD / 64 boxes of [64 keys][64 dims]
          if (leader) mbar_arrive_expect_tx(&k_full[s], L::kTileBytes);
          for (int c = 0; c < HD / 64; ++c)
            tma_load_3d_pair(k_ring + s * L::kStageBytes + c * L::kKBoxBytes, &tm_k, cluster_addr(&k_full[s], 0), c * 64,
                             kb * kBlockN + static_cast<int>(rank) * (kBlockN / 2), head);
        } else {
          mbar_arrive_expect_tx(&k_full[s], L::kTileBytes);
          for (int c = 0; c < HD / 64; ++c)
            tma_load_3d(k_ring + s * L::kTileBytes + c * L::kBoxBytes, &tm_k, &k_full[s], c * 64, kb * kBlockN,
                        head);
        }
        ++issued_k;
        ok = mbar_wait_bounded(&v_empty[s], ph ^ 1, abort_flag);
        if (!ok) break;
        if constexpr (kPair) {
          // this CTA's 64 dims of the tile (all keys): one box of [128 keys][64 dims]
          if (leader) mbar_arrive_expect_tx(&v_full[s], L::kTileBytes);
          tma_load_3d_pair(v_ring + s * L::kStageBytes, &tm_v, cluster_addr(&v_full[s], 0), static_cast<int>(rank) * 64,
                           kb * kBlockN, head);
        } else {
          mbar_arrive_expect_tx(&v_full[s], L::kTileBytes);
          for (int c = 0; c < HD / 64; ++c)
            tma_load_3d(v_ring + s * L::kTileBytes + c * L::kBoxBytes, &tm_v, &v_full[s], c * 64, kb * kBlockN,
                        head);
        }
        ++issued_v;
        if (++s == kStages) {
          s = 0;
          ph ^= 1;
        }
      }
      if (!ok) {
        // drain: the copies already issued must land before the CTA may exit
        if (!kPair || leader) {
          mbar_wait_bounded(q_full, 0, abort_flag + 1);
          for (int j = issued_k > kStages ? issued_k - kStages : 0; j < issued_k; ++j)
            mbar_wait_bounded(&k_full[j % kStages], (j / kStages) & 1, abort_flag + 1);
          for (int j = issued_v > kStages ? issued_v - kStages : 0; j < issued_v; ++j)
            mbar_wait_bounded(&v_full[j % kStages], (j / kStages) & 1, abort_flag + 1);
        } else {
          // the other CTA of a pair has no barrier of its own for its copies (they count on the leader's):
          // it gives them a millisecond, a thousand times what a copy from L2 or HBM takes
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000LL) {
          }
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ------------------------------ MMA issuers ----------------------------
    // Two issuing threads, warp 1 for the even steps and warp 2 for the odd ones.  For its step j a
    // thread issues P.V(j) and, straight after it, Q.K^T(j+3) into the score tile that P(j) lives
    // in: tcgen05.mma instructions of one thread execute in the order they were issued, so the
    // reader of P(j) is ordered before the next writer of that tile without a completion wait (a
    // wait there left the pipe idle for the ~300 cycles an MMA group needs to report completion).
    // Two threads because the pipe's issue queue is shallow: the commits and barrier waits of one
    // thread are idle gaps in its stream of MMAs, which the other thread's stream fills.
    // Pairs: the leader's two threads issue for both CTAs (a third issuing thread changed nothing).
    constexpr int kIssuers = 2;
    if (lane == 0 && leader) {
      const int par = warp - 1;
      // pairs: one instruction covers the 256 query rows of both CTAs
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kPair ? 2 * kBlockM : kBlockM, HD, 0, 1);
      constexpr uint32_t idesc_qk = umma_idesc_bf16(kPair ? 2 * kBlockM : kBlockM, kBlockN, 0, 0);
      // Descriptors are built once; per stage and per 16-element step they are one 64-bit add
      // (the start-address field counts 16-byte units).
      // V tile = HD/64 boxes of [128 keys][64 dims], used as an MN-major operand: 16 KB between
      // the 64-wide groups along the head dimension, 1 KB between groups of 8 keys.
      // Pairs: the descriptors name the same offsets in the shared memory of both CTAs; each CTA's
      // part of a K tile is [64 keys][HD] (boxes of 8 KB), of a V tile [128 keys][64 dims] (one box).
      const uint64_t v_desc0 = umma_desc_sw128(smem_u32(v_ring), L::kBoxBytes, 1024);
      const uint64_t q_desc = umma_desc_sw128(smem_u32(q_tile), 16, 1024);
      const uint64_t k_desc0 = umma_desc_sw128(smem_u32(k_ring), 16, 1024);
      constexpr uint64_t kStageStep = L::kStageBytes >> 4;
      const uint32_t o_tmem = tmem_base + kColO;
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag);

      auto issue_qk = [&](int j) {   // S[j%3] = Q K(j)^T, K from ring slot j%3
        const int s = j % kStages;
        if (!mbar_wait_bounded(&k_full[s], (j / kStages) & 1, abort_flag)) return false;
        tc_fence_after_sync();
        const uint64_t k_desc = k_desc0 + kStageStep * s;
        const uint32_t d_tmem = tmem_base + s_col(j);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          // 32 bytes per 16-element step inside a 64-wide box, then the next box
          const uint64_t q_off = (ks / 4) * (L::kBoxBytes >> 4) + (ks % 4) * 2;
          const uint64_t k_off = (ks / 4) * (L::kKBoxBytes >> 4) + (ks % 4) * 2;
          if constexpr (kPair)
            umma_ss_pair(d_tmem, q_desc + q_off, k_desc + k_off, idesc_qk, ks > 0);
          else
            umma_ss(d_tmem, q_desc + q_off, k_desc + k_off, idesc_qk, ks > 0);
        }
        if constexpr (kPair) {
          umma_commit_pair(smem_u32(&s_full[j % kSBufs]));   // also releases K slot s of this CTA
          umma_commit_pair(cluster_addr(&s_full[j % kSBufs], 1));
        } else {
          umma_commit(&s_full[j % kSBufs]);   // also releases K slot s
        }
        return true;
      };

      // the first three score tiles: 0 and 2 from the even thread, 1 from the odd one
      for (int j = par; j < kSBufs && j < n_tiles && ok; j += kIssuers) ok = issue_qk(j);
      for (int j = par; j < n_tiles && ok; j += kIssuers) {
        const int s = j % kStages;
        // What this step needs besides P(j) -- V(j) and the completion of P.V(j-1) -- is waited for FIRST: it
        // normally is there long before the softmax warps are done, and a barrier wait costs ~100 cycles even
        // when it passes at once, cycles that would otherwise sit between the arrival of P and the first MMA.
        // (Not so the K tile of the Q.K^T that follows: the producer requests it only after V(j+2), i.e.
        // after P.V(j-1) has completed, and waiting for it here would put its latency in front of P.V(j).)
        ok = mbar_wait_bounded(&v_full[s], (j / kStages) & 1, abort_flag);
        if (!ok) break;
        if (j > 0) {
          // O += P(j) V(j) follows P.V(j-1), which the other thread issued: wait until that one
          // has completed (its barrier's next phase is P.V(j+2), issued by this thread later on, so the
          // parity wait cannot be fooled).
          ok = mbar_wait_bounded(&v_empty[(j - 1) % kStages], ((j - 1) / kStages) & 1, abort_flag);
          if (!ok) break;
        }
        ok = mbar_wait_bounded(&p_full[j % kSBufs], (j / kSBufs) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t v_desc = v_desc0 + kStageStep * s;
        const uint32_t p_tmem = tmem_base + s_col(j);
        // 16 keys per step: 8 packed columns of P, 16 rows (2 KB = 128 address units) of V
        if constexpr (kPair) {
          umma_ts_pair(o_tmem, p_tmem, v_desc, idesc_pv, j > 0);
#pragma unroll
          for (int ks = 1; ks < kBlockN / 16; ++ks)
            umma_ts_pair(o_tmem, p_tmem + ks * 8, v_desc + static_cast<uint64_t>(ks * 128), idesc_pv, 1);
          umma_commit_pair(smem_u32(&v_empty[s]));
          umma_commit_pair(cluster_addr(&v_empty[s], 1));
        } else {
          umma_ts(o_tmem, p_tmem, v_desc, idesc_pv, j > 0);
#pragma unroll
          for (int ks = 1; ks < kBlockN / 16; ++ks)
            umma_ts(o_tmem, p_tmem + ks * 8, v_desc + static_cast<uint64_t>(ks * 128), idesc_pv, 1);
          umma_commit(&v_empty[s]);
        }
        if (j + kSBufs < n_tiles) ok = issue_qk(j + kSBufs);
      }
      if (!ok) {
        // give-up path: let the MMAs already issued finish before TMEM is freed
        if constexpr (kPair) umma_commit_pair(smem_u32(&mma_drain[par])); else umma_commit(&mma_drain[par]);
        mbar_wait_bounded(&mma_drain[par], 0, abort_flag + 1);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ softmax -------------------------------
    // Warp w owns 16 query rows: TMEM lanes 32*(w%4) + 16*((w-4)/4) .. +15, all 128 score columns.
    // In the 16x256b fragment a thread holds, for its two rows (a = lane/4, b = a + 8), the columns
    // 8i + 2t and 8i + 2t + 1 (t = lane%4) of every group i of eight: a row lives in four threads,
    // so row reductions are two shuffles and no other warp is involved.
    const int quad = warp & 3;
    const int sub = (warp - 4) >> 2;
    const int lane_base = quad * 32 + sub * 16;
    const uint32_t lane_sel = static_cast<uint32_t>(lane_base) << 16;
    const int t4 = lane & 3;
    const int row_a = lane_base + (lane >> 2);  // first of this thread's two rows of the tile (the other: + 8)
    const float c = p.scale_log2;
    const uint64_t c2 = pack2(c, c);
    float m_a = -INFINITY, m_b = -INFINITY;  // reference maxima (raw score units) of the two rows
    uint64_t la0 = pack2(0.f, 0.f), la1 = la0, lb0 = la0, lb1 = la0;  // partial row sums (this thread's columns)
    bool ok = true;
    const uint32_t o_addr = tmem_base + lane_sel + kColO;
    int kb_next = n_tiles > 0 ? (my_idx ? __ldg(my_idx) : 0) : 0;
    // tile map byte of this warp's query tile for the current and the next listed block
    const unsigned long long* __restrict__ my_fine =
        (kFine && p.fine != nullptr && my_idx != nullptr)
            ? p.fine + (static_cast<size_t>(lhead) * p.q_blocks + qb) * p.kmax : nullptr;
    const int fine_shift = 8 * (lane_base >> 4);
    uint32_t keep_next = 0xffu;
    if (kFine && my_fine != nullptr && n_tiles > 0) keep_next = static_cast<uint32_t>(__ldg(my_fine) >> fine_shift) & 0xffu;

    for (int j = 0; j < n_tiles; ++j) {
      const int kb = kb_next;
      if (j + 1 < n_tiles) kb_next = my_idx ? __ldg(my_idx + j + 1) : j + 1;
      const uint32_t keep = keep_next;
      if (kFine && my_fine != nullptr && j + 1 < n_tiles)
        keep_next = static_cast<uint32_t>(__ldg(my_fine + j + 1) >> fine_shift) & 0xffu;
      // keys past kv_len (partial last block, zero-filled by TMA) are masked
      const long long key0 = static_cast<long long>(kb) * kBlockN;
      const int valid = key0 + kBlockN > p.kv_len ? static_cast<int>(p.kv_len - key0) : kBlockN;
      ok = mbar_wait_bounded(&s_full[j % kSBufs], (j / kSBufs) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();

      const uint32_t s_addr = tmem_base + lane_sel + s_col(j);
      const uint32_t p_addr = s_addr;  // P goes over the first half of the scores it came from
      if (kFine && keep == 0u) {
        // no key tile of this block is kept for this warp's query tile: P = 0, nothing else to do
        uint32_t zeros[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) zeros[i] = 0u;
        tmem_st_16x128b_x16(p_addr, zeros);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[j % kSBufs]);   // (tile maps: never a pair)
        continue;
      }
      uint32_t r[64];
      tmem_ld_16x256b_x16(s_addr, r);
      tmem_wait_ld();
      if (valid < kBlockN) mask_tail(r, valid, t4);

      // After the first tile the exponentials are taken against the row's current reference maximum straight
      // away, without the tile's own maxima (no max instructions and no shuffles in the common case); only
      // when a partial row sum shows that some score lies far above the reference (kSumBound), or a row
      // that had no reference yet sees its first keys, is the tile read again, its maxima found, the
      // reference moved (O rescaled in tensor memory) and the pass redone.  Sum and P always use the same
      // reference, so the result is exact.
      uint32_t packed[32];
      uint64_t ta0, ta1, tb0, tb1;  // this tile's partial row sums
      bool redo = true;             // the exp2 pass against the final reference is still to be done
      if (j > 0) {
        // a row may still be without a reference (-inf): every key it has seen so far was dropped by a
        // tile map or lies past kv_len
        const float nma = (m_a == -INFINITY) ? 0.f : -m_a * c;
        const float nmb = (m_b == -INFINITY) ? 0.f : -m_b * c;
        exp_pass<kPolyGroups, kFine>(r, c2, pack2(nma, nma), pack2(nmb, nmb), packed, ta0, ta1, tb0, tb1, keep);
        // did any exponential leave the safe range?  (!(x <= bound) also catches inf and NaN)
        float sa0, sa1, sb0, sb1;
        unpack2(add2(ta0, ta1), sa0, sa1);
        unpack2(add2(tb0, tb1), sb0, sb1);
        const float pa = sa0 + sa1, pb = sb0 + sb1;
        const bool grow = !(pa <= kSumBound) || !(pb <= kSumBound) || (m_a == -INFINITY && pa > 0.f) ||
                          (m_b == -INFINITY && pb > 0.f);
        redo = __any_sync(0xffffffffu, grow) != 0;
        if (redo) {   // rare: read the tile again
          tmem_ld_16x256b_x16(s_addr, r);
          tmem_wait_ld();
          if (valid < kBlockN) mask_tail(r, valid, t4);
        }
      }
      if (redo) {
        // the tile's row maxima: this thread's columns, then the row's four threads
        float xa0 = -INFINITY, xa1 = -INFINITY, xb0 = -INFINITY, xb1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          if (kFine && !((keep >> (i >> 1)) & 1u)) continue;  // a dropped key tile
          xa0 = max3(xa0, __uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]));
          xb0 = max3(xb0, __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
          xa1 = max3(xa1, __uint_as_float(r[4 * i + 4]), __uint_as_float(r[4 * i + 5]));
          xb1 = max3(xb1, __uint_as_float(r[4 * i + 6]), __uint_as_float(r[4 * i + 7]));
        }
        float mt_a = fmaxf(xa0, xa1), mt_b = fmaxf(xb0, xb1);
        mt_a = fmaxf(mt_a, __shfl_xor_sync(0xffffffffu, mt_a, 1));
        mt_b = fmaxf(mt_b, __shfl_xor_sync(0xffffffffu, mt_b, 1));
        mt_a = fmaxf(mt_a, __shfl_xor_sync(0xffffffffu, mt_a, 2));
        mt_b = fmaxf(mt_b, __shfl_xor_sync(0xffffffffu, mt_b, 2));
        const float na = fmaxf(m_a, mt_a), nb = fmaxf(m_b, mt_b);
        const float alpha_a = (m_a == -INFINITY) ? 0.f : ex2((m_a - na) * c);
        const float alpha_b = (m_b == -INFINITY) ? 0.f : ex2((m_b - nb) * c);
        m_a = na;
        m_b = nb;
        const uint64_t aa = pack2(alpha_a, alpha_a), ab = pack2(alpha_b, alpha_b), zero2 = pack2(0.f, 0.f);
        la0 = fma2(la0, aa, zero2);
        la1 = fma2(la1, aa, zero2);
        lb0 = fma2(lb0, ab, zero2);
        lb1 = fma2(lb1, ab, zero2);
        if (j > 0) {
          // P.V of step j-1 must have landed in O.  Its barrier completes one phase every
          // three steps and its next phase needs P(j+2), so the parity wait cannot be fooled.
          ok = mbar_wait_bounded(&v_empty[(j - 1) % kStages], ((j - 1) / kStages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int h = 0; h < HD / 64; ++h) {
            uint32_t o[32];
            tmem_ld_16x256b_x8(o_addr + h * 64, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              o[4 * i] = __float_as_uint(__uint_as_float(o[4 * i]) * alpha_a);
              o[4 * i + 1] = __float_as_uint(__uint_as_float(o[4 * i + 1]) * alpha_a);
              o[4 * i + 2] = __float_as_uint(__uint_as_float(o[4 * i + 2]) * alpha_b);
              o[4 * i + 3] = __float_as_uint(__uint_as_float(o[4 * i + 3]) * alpha_b);
            }
            tmem_st_16x256b_x8(o_addr + h * 64, o);
          }
        }
        // a row whose keys are all masked keeps the reference -inf: its exponentials are exp2(-inf) = 0
        const float nma = (m_a == -INFINITY) ? 0.f : -m_a * c, nmb = (m_b == -INFINITY) ? 0.f : -m_b * c;
        exp_pass<kPolyGroups, kFine>(r, c2, pack2(nma, nma), pack2(nmb, nmb), packed, ta0, ta1, tb0, tb1, keep);
      }
      // only now: the scores are not needed any more
      tmem_st_16x128b_x16(p_addr, packed);
      la0 = add2(la0, ta0);
      la1 = add2(la1, ta1);
      lb0 = add2(lb0, tb0);
      lb1 = add2(lb1, tb1);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        // pairs: the P barrier that counts is the leader's (sixteen warps arrive on it)
        if (kPair && !leader) mbar_arrive_cluster(cluster_addr(&p_full[j % kSBufs], 0)); else mbar_arrive(&p_full[j % kSBufs]);
      }
    }

    // row sums: this thread's columns, then the row's four threads
    float sa0, sa1, sb0, sb1;
    unpack2(add2(la0, la1), sa0, sa1);
    unpack2(add2(lb0, lb1), sb0, sb1);
    float l_a = sa0 + sa1, l_b = sb0 + sb1;
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    if (ok && n_tiles > 0)
      ok = mbar_wait_bounded(&v_empty[(n_tiles - 1) % kStages], ((n_tiles - 1) / kStages) & 1, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      // a row that never saw an unmasked key still has no reference maximum; its sum is not exactly
      // zero (masked scores on the polynomial exp2 come out as 2^-126), its result is
      const float inv_a = (l_a > 0.f && m_a != -INFINITY) ? 1.0f / l_a : 0.f;
      const float inv_b = (l_b > 0.f && m_b != -INFINITY) ? 1.0f / l_b : 0.f;
      const long long tok_a = static_cast<long long>(qb) * kBlockM + row_a, tok_b = tok_a + 8;
      const bool live_a = tok_a < p.seq_len, live_b = tok_b < p.seq_len;  // a row with an empty list gets zeros
      long long dst_a = tok_a, dst_b = tok_b;
      if (p.out_row_map) {
        if (live_a) dst_a = __ldg(p.out_row_map + tok_a);
        if (live_b) dst_b = __ldg(p.out_row_map + tok_b);
      }
      __nv_bfloat16 *out_a, *out_b;
      if (p.out_shard_rows > 0) {
        const long long ra = live_a ? dst_a : 0, rb = live_b ? dst_b : 0;
        const long long sa = ra / p.out_shard_rows, sb = rb / p.out_shard_rows;
        const long long head_row = static_cast<long long>(p.out_head0 + head) * p.out_shard_stride;
        out_a = p.out_shard[sa] + (head_row + ra - sa * p.out_shard_rows) * HD;
        out_b = p.out_shard[sb] + (head_row + rb - sb * p.out_shard_rows) * HD;
      } else {
        __nv_bfloat16* base = p.out + group * p.out_batch_stride + lhead * p.out_head_stride;
        out_a = base + (live_a ? dst_a : 0) * p.out_token_stride;
        out_b = base + (live_b ? dst_b : 0) * p.out_token_stride;
      }
#pragma unroll
      for (int h = 0; h < HD / 64; ++h) {
        uint32_t o[32];
        if (n_tiles > 0) {
          tmem_ld_16x256b_x8(o_addr + h * 64, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int col = h * 64 + 8 * i + 2 * t4;
          if (live_a)
            *reinterpret_cast<uint32_t*>(out_a + col) =
                cvt_bf16x2(__uint_as_float(o[4 * i]) * inv_a, __uint_as_float(o[4 * i + 1]) * inv_a);
          if (live_b)
            *reinterpret_cast<uint32_t*>(out_b + col) =
                cvt_bf16x2(__uint_as_float(o[4 * i + 2]) * inv_b, __uint_as_float(o[4 * i + 3]) * inv_b);
        }
      }
    }
  }

  // ------------------------------- tear-down -------------------------------
  // pairs: a cluster-wide barrier, so that neither CTA frees its tensor memory or leaves while the
  // other one may still signal its barriers or have an MMA running on it
  tc_fence_before_sync();
  if constexpr (kPair) cluster_sync_all(); else __syncthreads();
  if (abort_flag[0] != 0 && threadIdx.x == 0 && p.status) atomicExch(p.status, DFS_STATUS_WAIT_TIMEOUT);
  if constexpr (kPair) {
    if (misaligned && threadIdx.x == 0 && p.status) atomicExch(p.status, DFS_STATUS_BAD_SMEM_ALIGNMENT);
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    if constexpr (kPair) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------
// [H, L, D] bf16 as a 3-D tensor (D innermost), box = 64 x 128 x 1, 128-byte swizzle,
// rows past L read as zero.
int make_tile_map(CUtensorMap* map, const void* base, int heads, int64_t seq_len, int head_dim,
                  int box_rows = 128) {
  return dfs_make_bf16_tile_map(map, base, heads, seq_len, head_dim, box_rows);
}

template <int HD, bool kFine>
int launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Params& p, int heads,
               cudaStream_t stream) {
  using L = SmemLayout<HD, false>;
  DFS_CUDA_CHECK(cudaFuncSetAttribute(bsattn_fwd_kernel<HD, kFine, false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
  dim3 grid(p.q_blocks, heads);
  bsattn_fwd_kernel<HD, kFine, false><<<grid, kThreads, L::kTotal, stream>>>(mq, mk, mv, p);
  return static_cast<int>(cudaGetLastError());
}

// Dense call with 128-wide heads: clusters of two CTAs, each pair on two consecutive query blocks
// (mk: K with boxes of 64 rows, the half tile one CTA loads).
int launch_fwd_pairs(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Params& p, int heads,
                     cudaStream_t stream) {
  using L = SmemLayout<128, true>;
  auto kernel = bsattn_fwd_kernel<128, false, true>;
  DFS_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((p.q_blocks + 1) / 2 * 2), static_cast<unsigned>(heads), 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  DFS_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, mq, mk, mv, p));
  return static_cast<int>(cudaGetLastError());
}

// Whether dense calls with 128-wide heads run as CTA pairs.
bool dense_pairs_enabled() {
  static const int flag = [] {
    const char* e = getenv("DFSATTN_DENSE_PAIRS");
    return e == nullptr ? 1 : (e[0] != '0');
  }();
  return flag != 0;
}

}  // namespace

namespace {
struct ShardedOut {
  void* const* shards = nullptr;  // host array of `world` device pointers, or null
  int world = 0;
  int64_t shard_rows = 0, shard_stride_rows = 0;
  int head0 = 0;
};

int block_sparse_fwd_impl(const void* q, const void* k, const void* v, const int32_t* idx, const int32_t* cnt,
                          const uint64_t* fine, int kmax, const int32_t* out_row_map, void* out, int out_token_major,
                          const ShardedOut& sh, int batch, int heads, int64_t seq_len, int64_t kv_len,
                          int head_dim, float scale, int32_t* status, void* stream_) {
  // `heads` = heads of one batch element (what the lists cover); the tensors hold batch * heads heads
  if (batch <= 0 || heads <= 0 || static_cast<int64_t>(batch) * heads > 65535) return DFS_ERR_SHAPE;
  const int all_heads = batch * heads;
  if (sh.shards != nullptr) {
    if (batch != 1) return DFS_ERR_RANGE;
    if (sh.world <= 0 || sh.world > 8 || sh.head0 < 0) return DFS_ERR_RANGE;
    if (sh.shard_rows <= 0 || sh.shard_stride_rows < sh.shard_rows || sh.shard_rows * sh.world < seq_len)
      return DFS_ERR_RANGE;
    for (int s = 0; s < sh.world; ++s) {
      if (sh.shards[s] == nullptr) return DFS_ERR_NULL;
      if (!dfs_aligned16(sh.shards[s])) return DFS_ERR_ALIGN;
    }
    out = sh.shards[0];  // only for the shared argument checks below
  }
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return DFS_ERR_NULL;
  if ((idx == nullptr) != (cnt == nullptr)) return DFS_ERR_NULL;
  if (fine != nullptr && idx == nullptr) return DFS_ERR_NULL;  // tile maps belong to list entries
  if ((reinterpret_cast<uintptr_t>(fine) & 7u) != 0) return DFS_ERR_ALIGN;
  if (!dfs_aligned16(q) || !dfs_aligned16(k) || !dfs_aligned16(v) || !dfs_aligned16(out)) return DFS_ERR_ALIGN;
  if (head_dim != 64 && head_dim != 128) return DFS_ERR_SHAPE;
  if (seq_len <= 0) return DFS_ERR_SHAPE;
  if (kv_len <= 0 || kv_len > seq_len) return DFS_ERR_RANGE;
  if (idx != nullptr && kmax <= 0) return DFS_ERR_RANGE;
  if (!(scale > 0.f)) return DFS_ERR_RANGE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  const bool pairs = idx == nullptr && head_dim == 128 && dense_pairs_enabled();
  CUtensorMap mq, mk, mv;
  int rc = make_tile_map(&mq, q, all_heads, seq_len, head_dim);
  if (rc == 0) rc = make_tile_map(&mk, k, all_heads, seq_len, head_dim, pairs ? 64 : 128);
  if (rc == 0) rc = make_tile_map(&mv, v, all_heads, seq_len, head_dim);
  if (rc != 0) return rc;

  Params p;
  p.idx = idx;
  p.cnt = cnt;
  p.fine = reinterpret_cast<const unsigned long long*>(fine);
  p.out_row_map = out_row_map;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = status;
  p.seq_len = seq_len;
  p.kv_len = kv_len;
  // per batch element [H, L, D] or, token-major, [L, H*D]
  p.out_head_stride = out_token_major ? head_dim : seq_len * head_dim;
  p.out_token_stride = out_token_major ? static_cast<long long>(heads) * head_dim : head_dim;
  p.list_heads = heads;
  p.out_batch_stride = static_cast<long long>(heads) * seq_len * head_dim;
  for (int s = 0; s < 8; ++s)
    p.out_shard[s] = (sh.shards != nullptr && s < sh.world) ? static_cast<__nv_bfloat16*>(sh.shards[s]) : nullptr;
  p.out_shard_rows = sh.shards != nullptr ? sh.shard_rows : 0;
  p.out_shard_stride = sh.shard_stride_rows;
  p.out_head0 = sh.head0;
  p.kmax = kmax;
  p.q_blocks = static_cast<int>((seq_len + kBlockM - 1) / kBlockM);
  p.k_blocks = static_cast<int>((kv_len + kBlockN - 1) / kBlockN);
  p.scale_log2 = scale * 1.4426950408889634f;
  if (pairs) return launch_fwd_pairs(mq, mk, mv, p, all_heads, stream);
  if (fine != nullptr)
    return head_dim == 128 ? launch_fwd<128, true>(mq, mk, mv, p, all_heads, stream)
                           : launch_fwd<64, true>(mq, mk, mv, p, all_heads, stream);
  return head_dim == 128 ? launch_fwd<128, false>(mq, mk, mv, p, all_heads, stream)
                         : launch_fwd<64, false>(mq, mk, mv, p, all_heads, stream);
}
}  // namespace

namespace {
// One warp waits on a barrier that nothing completes and leaves as the attention kernel does after
// an expired wait: flag in shared memory, CTA-wide barrier, one thread reports to the status word.
__global__ void wait_timeout_selftest_kernel(int32_t* status, long long limit_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag[2];
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag[0] = abort_flag[1] = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait_bounded(&bar, 0, abort_flag, limit_cycles);
  __syncthreads();
  if (abort_flag[0] != 0 && threadIdx.x == 0 && status) atomicExch(status, DFS_STATUS_WAIT_TIMEOUT);
}
}  // namespace

namespace {
__global__ void status_snapshot_kernel(const int32_t* __restrict__ status, volatile int32_t* mirror) {
  *mirror = *reinterpret_cast<const volatile int32_t*>(status);
  __threadfence_system();
}
}  // namespace

extern "C" int dfs_status_snapshot(const int32_t* status, int32_t* mirror, void* stream) {
  if (status == nullptr || mirror == nullptr) return DFS_ERR_NULL;
  status_snapshot_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(status, mirror);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dfs_selftest_wait_timeout(int64_t limit_cycles, int32_t* status, void* stream) {
  if (status == nullptr) return DFS_ERR_NULL;
  if (limit_cycles < 1 || limit_cycles >= (1LL << 31)) return DFS_ERR_RANGE;
  wait_timeout_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_cycles);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dfs_block_sparse_fwd_ex(const void* q, const void* k, const void* v, const int32_t* idx,
                                       const int32_t* cnt, int kmax, const int32_t* out_row_map, void* out,
                                       int out_token_major, int heads, int64_t seq_len, int64_t kv_len,
                                       int head_dim, float scale, int32_t* status, void* stream) {
  return block_sparse_fwd_impl(q, k, v, idx, cnt, nullptr, kmax, out_row_map, out, out_token_major, ShardedOut(), 1, heads,
                               seq_len, kv_len, head_dim, scale, status, stream);
}

extern "C" int dfs_block_sparse_fwd_batched(const void* q, const void* k, const void* v, const int32_t* idx,
                                            const int32_t* cnt, int kmax, const int32_t* out_row_map, void* out,
                                            int out_token_major, int batch, int heads, int64_t seq_len,
                                            int64_t kv_len, int head_dim, float scale, int32_t* status,
                                            void* stream) {
  return block_sparse_fwd_impl(q, k, v, idx, cnt, nullptr, kmax, out_row_map, out, out_token_major, ShardedOut(), batch,
                               heads, seq_len, kv_len, head_dim, scale, status, stream);
}

extern "C" int dfs_block_sparse_fwd_fine(const void* q, const void* k, const void* v, const int32_t* idx,
                                         const int32_t* cnt, const uint64_t* fine_bits, int kmax,
                                         const int32_t* out_row_map, void* out, int out_token_major, int heads,
                                         int64_t seq_len, int64_t kv_len, int head_dim, float scale,
                                         int32_t* status, void* stream) {
  if (fine_bits == nullptr) return DFS_ERR_NULL;
  return block_sparse_fwd_impl(q, k, v, idx, cnt, fine_bits, kmax, out_row_map, out, out_token_major, ShardedOut(),
                               1, heads, seq_len, kv_len, head_dim, scale, status, stream);
}

extern "C" int dfs_block_sparse_fwd_sharded(const void* q, const void* k, const void* v, const int32_t* idx,
                                            const int32_t* cnt, int kmax, const int32_t* out_row_map,
                                            void* const* out_shards, int world, int64_t shard_rows,
                                            int64_t shard_stride_rows, int head0, int heads, int64_t seq_len,
                                            int64_t kv_len, int head_dim, float scale, int32_t* status,
                                            void* stream) {
  if (out_shards == nullptr) return DFS_ERR_NULL;
  ShardedOut sh;
  sh.shards = out_shards;
  sh.world = world;
  sh.shard_rows = shard_rows;
  sh.shard_stride_rows = shard_stride_rows;
  sh.head0 = head0;
  return block_sparse_fwd_impl(q, k, v, idx, cnt, nullptr, kmax, out_row_map, nullptr, 0, sh, 1, heads, seq_len, kv_len,
                               head_dim, scale, status, stream);
}

extern "C" int dfs_block_sparse_fwd(const void* q, const void* k, const void* v, const int32_t* idx,
                                    const int32_t* cnt, int kmax, const int32_t* out_row_map, void* out,
                                    int heads, int64_t seq_len, int64_t kv_len, int head_dim, float scale,
                                    int32_t* status, void* stream) {
  return dfs_block_sparse_fwd_ex(q, k, v, idx, cnt, kmax, out_row_map, out, 0, heads, seq_len, kv_len, head_dim,
                                 scale, status, stream);
}
