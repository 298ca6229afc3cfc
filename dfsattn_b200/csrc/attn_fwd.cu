// Block-sparse attention forward for sm_100a: online softmax over the selected
// 128-token key blocks of each 128-token query block.
//
// One CTA works on TWO adjacent query blocks of one head (tiles "a" and "b"),
// each with its own key-block list, so that the softmax of one tile runs while
// the tensor cores work for the other.  12 warps:
//   warp 0      TMA producer: both Q tiles once, then the K / V tiles of both
//               lists, interleaved in exactly the order the MMA warp consumes
//               them, through one 5-slot shared-memory ring (full/empty
//               mbarrier per slot).
//   warp 1      tcgen05.mma issuer (one lane): S_t = Q_t K^T into tile t's TMEM
//               score buffer (SS form), O_t += P_t V (TS form, P read from
//               TMEM, V as MN-major B operand); owns the TMEM allocation.
//   warps 4-7   softmax of tile a, warps 8-11 softmax of tile b: one thread per
//               query row.  Pass 1 reads the 128 scores for the row maximum,
//               pass 2 reads them again, computes exp2 in the log2 domain and
//               writes P as packed bf16 over the first 64 columns of the score
//               buffer it has just consumed.  The accumulator O_t is rescaled
//               in TMEM only when a row maximum grew by more than 2^8 (sum and
//               P use the same reference maximum, so the result is exact).
//               Epilogue: normalise, store bf16 rows, optionally through a row
//               map (fused inverse permutation).
//   warps 2-3   idle (they keep the softmax warps aligned to TMEM lane quadrants).
//
// Shared memory (HD = 128): 2 x 32 KB Q + 5 x 32 KB ring.  Tiles are stored as
// [128 rows][64 bf16] boxes with the 128-byte TMA swizzle: the canonical
// K-major (Q, K) and MN-major (V) tcgen05 operand layout.
// TMEM (512 columns): S_a | S_b | O_a | O_b, P_t aliasing S_t.
//
// Every wait is bounded; on expiry the CTA records DFS_STATUS_WAIT_TIMEOUT,
// drains its copies and MMAs in flight, frees its TMEM and returns.
#include "common.cuh"

namespace {

using namespace dfs;

constexpr int kBlockM = 128;  // query rows per tile
constexpr int kBlockN = 128;  // keys per tile
constexpr int kThreads = 384;
constexpr int kRing = 5;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 384;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

template <int HD>
struct SmemLayout {
  static constexpr int kBoxBytes = kBlockN * 64 * 2;        // one [128][64] bf16 box
  static constexpr int kTileBytes = kBoxBytes * (HD / 64);  // one Q / K / V tile
  static constexpr int kQOff = 0;
  static constexpr int kRingOff = 2 * kTileBytes;
  static constexpr int kBarOff = kRingOff + kRing * kTileBytes;
  static constexpr int kNumBars = 1 + 2 * kRing + 2 + 2 + 2 + 1;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;  // + tmem address + two give-up flags
  static constexpr int kAlloc = kTotal + 1024;                // slack for 1024-byte alignment
};

struct Params {
  const int32_t* idx;   // [H, Qb, kmax] or nullptr (all key blocks)
  const int32_t* cnt;   // [H, Qb]
  const int32_t* out_row_map;
  __nv_bfloat16* out;
  int32_t* status;
  float* debug;         // optional dump for (query block 0, head 0): S of the first tile, O, l, m
  long long seq_len;
  long long kv_len;
  int kmax;
  int q_blocks, k_blocks;
  float scale_log2;
  uint32_t v_lbo, v_sbo;  // V operand descriptor strides (bytes)
};

// ---- packed fp32x2 arithmetic (halves the instruction count of the softmax) ----
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
    bsattn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const Params p) {
  using L = SmemLayout<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_tiles = smem + L::kQOff;
  uint8_t* ring = smem + L::kRingOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;
  uint64_t* full = bars + 1;         // [kRing]
  uint64_t* empty = full + kRing;    // [kRing]
  uint64_t* s_full = empty + kRing;  // [2]  MMA -> softmax: scores of tile t are in TMEM
  uint64_t* p_full = s_full + 2;     // [2]  softmax -> MMA: P of tile t is in TMEM
  uint64_t* o_final = p_full + 2;    // [2]  last P.V of tile t has completed
  uint64_t* mma_drain = o_final + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heavy rows (the dense text rows sit at the end) are scheduled first
  const int pair = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y;
  const int qb_a = 2 * pair, qb_b = 2 * pair + 1;
  const bool has_b = qb_b < p.q_blocks;
  const size_t at_a = static_cast<size_t>(head) * p.q_blocks + qb_a;
  const size_t at_b = has_b ? at_a + 1 : at_a;
  const int n_a = p.idx ? p.cnt[at_a] : p.k_blocks;
  const int n_b = !has_b ? 0 : (p.idx ? p.cnt[at_b] : p.k_blocks);
  const int32_t* __restrict__ list_a = p.idx ? p.idx + at_a * p.kmax : nullptr;
  const int32_t* __restrict__ list_b = p.idx ? p.idx + at_b * p.kmax : nullptr;
  const int n_max = n_a > n_b ? n_a : n_b;
  // per-tile values are picked with selects (t is 0 or 1) so that nothing lands in local memory
#define TILE_SEL(t, a, b) ((t) == 0 ? (a) : (b))

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
      mbar_init(&o_final[t], 1);
    }
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
      mbar_arrive_expect_tx(q_full, L::kTileBytes * (has_b ? 2 : 1));
      for (int t = 0; t < (has_b ? 2 : 1); ++t)
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d(q_tiles + t * L::kTileBytes + c * L::kBoxBytes, &tm_q, q_full, c * 64,
                      TILE_SEL(t, qb_a, qb_b) * kBlockM, head);
      int it = 0;
      bool ok = true;
      // one ring entry: wait for the slot, arm its barrier, issue the boxes of one tile
      auto push = [&](const CUtensorMap* tm, int kb) {
        if (!ok) return;
        const int s = it % kRing;
        ok = mbar_wait_bounded(&empty[s], ((it / kRing) & 1) ^ 1, abort_flag);
        if (!ok) return;
        mbar_arrive_expect_tx(&full[s], L::kTileBytes);
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d(ring + s * L::kTileBytes + c * L::kBoxBytes, tm, &full[s], c * 64, kb * kBlockN, head);
        ++it;
      };
      int cur_a = n_a > 0 && list_a ? __ldg(list_a) : 0;
      int cur_b = n_b > 0 && list_b ? __ldg(list_b) : 0;
      if (n_a > 0) push(&tm_k, cur_a);
      if (n_b > 0) push(&tm_k, cur_b);
      for (int j = 0; j < n_max && ok; ++j) {
        if (j < n_a) push(&tm_v, cur_a);
        if (j + 1 < n_a) {
          cur_a = list_a ? __ldg(list_a + j + 1) : j + 1;
          push(&tm_k, cur_a);
        }
        if (j < n_b) push(&tm_v, cur_b);
        if (j + 1 < n_b) {
          cur_b = list_b ? __ldg(list_b + j + 1) : j + 1;
          push(&tm_k, cur_b);
        }
      }
      if (!ok) {
        // drain: the copies already issued must land before the CTA may exit
        mbar_wait_bounded(q_full, 0, abort_flag + 1);
        for (int j = it > kRing ? it - kRing : 0; j < it; ++j)
          mbar_wait_bounded(&full[j % kRing], (j / kRing) & 1, abort_flag + 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(kBlockM, kBlockN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kBlockM, HD, 0, 1);
      int it = 0;
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag);
      auto take = [&]() -> int {  // next ring entry, in production order
        const int s = it % kRing;
        ok = ok && mbar_wait_bounded(&full[s], (it / kRing) & 1, abort_flag);
        ++it;
        return s;
      };
      auto issue_qk = [&](int t) {
        const int s = take();
        if (!ok) return;
        tc_fence_after_sync();
        const uint32_t q_addr = smem_u32(q_tiles + t * L::kTileBytes);
        const uint32_t k_addr = smem_u32(ring + s * L::kTileBytes);
        const uint32_t d_tmem = tmem_base + (t ? kColS1 : kColS0);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = (ks / 4) * L::kBoxBytes + (ks % 4) * 32;
          umma_ss(d_tmem, umma_desc_sw128(q_addr + off, 16, 1024), umma_desc_sw128(k_addr + off, 16, 1024),
                  idesc_qk, ks > 0);
        }
        umma_commit(&empty[s]);
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int j) {
        const int s = take();
        ok = ok && mbar_wait_bounded(&p_full[t], j & 1, abort_flag);
        if (!ok) return;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(ring + s * L::kTileBytes);
        const uint32_t p_tmem = tmem_base + (t ? kColS1 : kColS0);  // P aliases S
        const uint32_t o_tmem = tmem_base + (t ? kColO1 : kColO0);
#pragma unroll
        for (int ks = 0; ks < kBlockN / 16; ++ks) {
          // 16 keys per step: 8 packed columns of P, 16 rows (2 KB) of V
          umma_ts(o_tmem, p_tmem + ks * 8, umma_desc_sw128(v_addr + ks * 2048, p.v_lbo, p.v_sbo), idesc_pv,
                  (j > 0) || (ks > 0));
        }
        umma_commit(&empty[s]);
        if (j == TILE_SEL(t, n_a, n_b) - 1) umma_commit(&o_final[t]);
      };
      if (n_a > 0 && ok) issue_qk(0);
      if (n_b > 0 && ok) issue_qk(1);
      for (int j = 0; j < n_max && ok; ++j) {
        // Q.K^T of step j+1 overwrites S_t / P_t: it is issued after the P.V that reads P_t
        if (j < n_a) issue_pv(0, j);
        if (ok && j + 1 < n_a) issue_qk(0);
        if (ok && j < n_b) issue_pv(1, j);
        if (ok && j + 1 < n_b) issue_qk(1);
      }
      if (!ok) {
        // give-up path: let the MMAs already issued finish before TMEM is freed
        umma_commit(mma_drain);
        mbar_wait_bounded(mma_drain, 0, abort_flag + 1);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ softmax -------------------------------
    const int t = (warp - 4) >> 2;                                // tile a or b
    const int row = (warp & 3) * 32 + lane;                       // TMEM lane = query row in the tile
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_sel + (t ? kColS1 : kColS0);
    const uint32_t o_addr = tmem_base + lane_sel + (t ? kColO1 : kColO0);
    const int nt = TILE_SEL(t, n_a, n_b);
    const int my_qb = TILE_SEL(t, qb_a, qb_b);
    const int32_t* __restrict__ my_list = TILE_SEL(t, list_a, list_b);
    const float c = p.scale_log2;
    const uint64_t c2 = pack2(c, c);
    float m_ref = -INFINITY;  // reference max (raw score units)
    uint64_t l2a = pack2(0.f, 0.f), l2b = l2a, l2c = l2a, l2d = l2a;  // eight partial row sums (independent chains)
    bool ok = true;
    const bool dump = p.debug != nullptr && my_qb == 0 && head == 0 && nt > 0;

    for (int j = 0; j < nt; ++j) {
      const int kb = my_list ? __ldg(my_list + j) : j;
      // keys past kv_len (partial last block, zero-filled by TMA) are masked
      const long long key0 = static_cast<long long>(kb) * kBlockN;
      const int valid = key0 + kBlockN > p.kv_len ? static_cast<int>(p.kv_len - key0) : kBlockN;
      ok = mbar_wait_bounded(&s_full[t], j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();

      // pass 1: row maximum of this tile (four independent chains; the loop over the two
      // 64-column halves is kept rolled to bound the code size)
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t r0[32], r1[32];
        tmem_ld32(s_addr + h * 64, r0);
        tmem_ld32(s_addr + h * 64 + 32, r1);
        tmem_wait_ld();
        if (valid < kBlockN) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (h * 64 + i >= valid) r0[i] = __float_as_uint(-INFINITY);
            if (h * 64 + 32 + i >= valid) r1[i] = __float_as_uint(-INFINITY);
          }
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = max3(mx0, __uint_as_float(r0[i]), __uint_as_float(r0[i + 1]));
          mx1 = max3(mx1, __uint_as_float(r0[i + 2]), __uint_as_float(r0[i + 3]));
          mx2 = max3(mx2, __uint_as_float(r1[i]), __uint_as_float(r1[i + 1]));
          mx3 = max3(mx3, __uint_as_float(r1[i + 2]), __uint_as_float(r1[i + 3]));
        }
      }
      const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));

      // S_t(j) being ready implies that the previous P.V of this tile has landed in O_t
      // (it was issued before this tile's Q.K^T), so O_t may be rescaled right here.
      const bool grow = (m_tile - m_ref) * c > kRescaleThreshold;  // also true for the first tile
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, m_tile);
        const float alpha = (m_ref == -INFINITY) ? 0.f : ex2((m_ref - m_new) * c);
        m_ref = m_new;
        const uint64_t alpha2 = pack2(alpha, alpha), zero2 = pack2(0.f, 0.f);
        l2a = fma2(l2a, alpha2, zero2);
        l2b = fma2(l2b, alpha2, zero2);
        l2c = fma2(l2c, alpha2, zero2);
        l2d = fma2(l2d, alpha2, zero2);
        if (j > 0) {
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
      const uint64_t neg_mc2 = pack2(neg_mc, neg_mc);

      // pass 2: P = exp2(S*c - m*c) as packed bf16, written over the columns just read
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t r0[32], r1[32];
        tmem_ld32(s_addr + h * 64, r0);
        tmem_ld32(s_addr + h * 64 + 32, r1);
        tmem_wait_ld();
        if (valid < kBlockN) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (h * 64 + i >= valid) r0[i] = __float_as_uint(-INFINITY);
            if (h * 64 + 32 + i >= valid) r1[i] = __float_as_uint(-INFINITY);
          }
        }
        if (dump && j == 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            p.debug[row * 128 + h * 64 + i] = __uint_as_float(r0[i]);
            p.debug[row * 128 + h * 64 + 32 + i] = __uint_as_float(r1[i]);
          }
        }
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          float a0, a1, b0, b1, e0, e1, f0, f1;
          unpack2(fma2(pack2(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1])), c2, neg_mc2), a0, a1);
          unpack2(fma2(pack2(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1])), c2, neg_mc2), b0, b1);
          unpack2(fma2(pack2(__uint_as_float(r0[2 * i + 2]), __uint_as_float(r0[2 * i + 3])), c2, neg_mc2), e0, e1);
          unpack2(fma2(pack2(__uint_as_float(r1[2 * i + 2]), __uint_as_float(r1[2 * i + 3])), c2, neg_mc2), f0, f1);
          a0 = ex2(a0);
          a1 = ex2(a1);
          b0 = ex2(b0);
          b1 = ex2(b1);
          e0 = ex2(e0);
          e1 = ex2(e1);
          f0 = ex2(f0);
          f1 = ex2(f1);
          l2a = add2(l2a, pack2(a0, a1));
          l2b = add2(l2b, pack2(b0, b1));
          l2c = add2(l2c, pack2(e0, e1));
          l2d = add2(l2d, pack2(f0, f1));
          packed[i] = cvt_bf16x2(a0, a1);            // keys h*64 + 2i, +1   (even key in the low half)
          packed[16 + i] = cvt_bf16x2(b0, b1);       // keys h*64 + 32 + 2i, +1
          packed[i + 1] = cvt_bf16x2(e0, e1);
          packed[16 + i + 1] = cvt_bf16x2(f0, f1);
        }
        tmem_st32(s_addr + h * 32, packed);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_full[t]);
    }

    if (ok && nt > 0) ok = mbar_wait_bounded(&o_final[t], 0, abort_flag);
    if (ok && (t == 0 || has_b)) {
      tc_fence_after_sync();
      float l_lo, l_hi;
      unpack2(add2(add2(l2a, l2b), add2(l2c, l2d)), l_lo, l_hi);
      const float l_sum = l_lo + l_hi;
      const long long tok = static_cast<long long>(my_qb) * kBlockM + row;
      const float inv_l = l_sum > 0.f ? 1.0f / l_sum : 0.f;
      const bool live = tok < p.seq_len;  // a row with an empty list gets zeros
      long long dst_row = tok;
      if (live && p.out_row_map) dst_row = __ldg(p.out_row_map + tok);
      __nv_bfloat16* dst = p.out + (static_cast<size_t>(head) * p.seq_len + (live ? dst_row : 0)) * HD;
#pragma unroll
      for (int g = 0; g < HD / 32; ++g) {
        uint32_t o[32];
        if (nt > 0) {
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
            pk.x = cvt_bf16x2(__uint_as_float(o[v8 * 8 + 0]) * inv_l, __uint_as_float(o[v8 * 8 + 1]) * inv_l);
            pk.y = cvt_bf16x2(__uint_as_float(o[v8 * 8 + 2]) * inv_l, __uint_as_float(o[v8 * 8 + 3]) * inv_l);
            pk.z = cvt_bf16x2(__uint_as_float(o[v8 * 8 + 4]) * inv_l, __uint_as_float(o[v8 * 8 + 5]) * inv_l);
            pk.w = cvt_bf16x2(__uint_as_float(o[v8 * 8 + 6]) * inv_l, __uint_as_float(o[v8 * 8 + 7]) * inv_l);
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

#undef TILE_SEL
  // ------------------------------- tear-down -------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag[0] != 0 && threadIdx.x == 0 && p.status) atomicExch(p.status, DFS_STATUS_WAIT_TIMEOUT);
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
  dim3 grid((p.q_blocks + 1) / 2, heads);  // two adjacent query blocks per CTA
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
