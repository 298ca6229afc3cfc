// Fused pre-attention step: the Q/K/V projections of a token-major activation [rows, H*D] become
// head-major, normalised, rotated and already token-permuted tensors [H, L, D] in ONE pass.
//
//   out[h, out_row0 + i, :] = rope( rmsnorm( src[row(i), h*D : (h+1)*D] ) ),  row(i) = perm ? perm[i] : i
//
// It stands for what the reference does in five to eleven separate passes over Q and K:
// unflatten/transpose/contiguous (replace_hyvideo.py:247-249, replace_wan.py:174-176), RMSNorm per
// head (kernels/include/norm/narrow_rms_norm.cuh:22-71: y = (x * rsqrt(mean(x^2) + eps)) * gamma, fp32,
// rounded to the tensor type) or over the whole H*D row (kernels/triton/rmsnorm.py:8-49, used by
// replace_wan.py:162-166 before the transpose), the rotary embedding of the video tokens
// (kernels/include/rope/rope_enc.cuh:17-36: out[i] = x[i]*cos[i] + (i even ? -x[i^1] : x[i^1])*sin[i],
// fp32, on the rounded result of the norm; text rows are left alone, rope_enc_txtlast.cuh:46-50), and
// the Hilbert gather of attention_hyvideo.py:1034-1036.  V is only transposed and gathered.
//
// HBM-bound: every element is read once and written once (2 x 3 x rows x H x D x 2 bytes).  One warp
// owns one token: its lanes walk the token's 16-byte chunks, so a head's 128 (or 64) elements sit in
// 16 (8) neighbouring lanes and the per-head sum of squares is a sub-warp shuffle reduction.  The
// chunk a lane holds is at the same offset inside every head, so its slice of gamma and of the
// cos/sin row is loaded once per token.  Source rows (H*D*2 bytes, contiguous) and destination rows
// (D*2 bytes per head) are both touched as whole 128-byte-aligned segments.
#include "common.cuh"

namespace {

constexpr int kWarpsPerCta = 8;

struct PrepareParams {
  const uint4* src[3];  // Q, K, V projections [src_rows, H*D] bf16; any may be null
  uint4* dst[3];        // [H, out_len, D] bf16
  const __nv_bfloat16* gamma[2];  // Q, K norm weights ([D] per head / [H*D] across heads) or null
  float eps[2];
  const float* cos_tab;  // [rope_rows, rope_dim] fp32 or null
  const float* sin_tab;
  const int32_t* perm;   // [n_rows] source row of output row out_row0 + i, or null (identity)
  long long rope_rows;   // source rows below this are rotated with table row = source row
  long long n_rows, out_row0, out_len;
  int heads;
  int norm_across_heads;  // 0: one RMS per (token, head); 1: one RMS per token over H*D
  int rope_pairs;         // 1: tables hold one value per element pair ([.., D/2]); 0: one per element ([.., D])
};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <int HD>
__global__ void __launch_bounds__(kWarpsPerCta * 32) qkv_prepare_kernel(const PrepareParams p) {
  constexpr int kLanesPerHead = HD / 8;  // 16-byte chunks per head row
  const int lane = threadIdx.x & 31;
  const long long i = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  if (i >= p.n_rows) return;
  const long long src_row = p.perm ? static_cast<long long>(__ldg(p.perm + i)) : i;
  const int chunks = p.heads * kLanesPerHead;  // per token
  const int in_head = lane % kLanesPerHead;    // this lane's chunk offset inside every head
  const bool rotate = p.cos_tab != nullptr && src_row < p.rope_rows;

  // this lane's slice of the rotary row: c[j], s[j] multiply element 8*in_head + j
  float cs[8], sn[8];
  if (rotate) {
    if (p.rope_pairs) {
      const float4 c4 = __ldg(reinterpret_cast<const float4*>(p.cos_tab + src_row * (HD / 2)) + in_head);
      const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.sin_tab + src_row * (HD / 2)) + in_head);
      cs[0] = cs[1] = c4.x, cs[2] = cs[3] = c4.y, cs[4] = cs[5] = c4.z, cs[6] = cs[7] = c4.w;
      sn[0] = sn[1] = s4.x, sn[2] = sn[3] = s4.y, sn[4] = sn[5] = s4.z, sn[6] = sn[7] = s4.w;
    } else {
      const float4* c4 = reinterpret_cast<const float4*>(p.cos_tab + src_row * HD) + 2 * in_head;
      const float4* s4 = reinterpret_cast<const float4*>(p.sin_tab + src_row * HD) + 2 * in_head;
      const float4 ca = __ldg(c4), cb = __ldg(c4 + 1), sa = __ldg(s4), sb = __ldg(s4 + 1);
      cs[0] = ca.x, cs[1] = ca.y, cs[2] = ca.z, cs[3] = ca.w, cs[4] = cb.x, cs[5] = cb.y, cs[6] = cb.z, cs[7] = cb.w;
      sn[0] = sa.x, sn[1] = sa.y, sn[2] = sa.z, sn[3] = sa.w, sn[4] = sb.x, sn[5] = sb.y, sn[6] = sb.z, sn[7] = sb.w;
    }
  }

#pragma unroll
  for (int t = 0; t < 3; ++t) {
    const uint4* __restrict__ src = p.src[t];
    if (src == nullptr) continue;
    uint4* __restrict__ dst = p.dst[t];
    const uint4* __restrict__ row = src + src_row * chunks;
    const __nv_bfloat16* __restrict__ gamma = t < 2 ? p.gamma[t] : nullptr;
    const bool rot = t < 2 && rotate;

    float rstd_all = 0.f;
    float g[8];
    if (gamma != nullptr) {
      if (p.norm_across_heads) {
        // first pass over the token: sum of squares of the whole row (the second read hits L1/L2)
        float ss = 0.f;
        for (int c = lane; c < chunks; c += 32) {
          float x[8];
          unpack8(__ldg(row + c), x);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss = fmaf(x[j], x[j], ss);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        rstd_all = rsqrtf(ss / static_cast<float>(p.heads * HD) + p.eps[t]);
      } else {
        unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + in_head), g);
      }
    }

    // All lanes take part in every round (the shuffles below need the full warp).  Rounds go in
    // batches of four whose loads are issued together: the kernel lives on memory-level parallelism.
    const int rounds = (chunks + 31) / 32;
    for (int r0 = 0; r0 < rounds; r0 += 4) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = (r0 + u) * 32 + lane;
        raw[u] = c < chunks ? __ldg(row + c) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (r0 + u >= rounds) break;  // warp-uniform
        const int c = (r0 + u) * 32 + lane;
        const bool live = c < chunks;
        float x[8];
        unpack8(raw[u], x);
        if (gamma != nullptr) {
          float rstd = rstd_all;
          if (!p.norm_across_heads) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(x[j], x[j], ss);
#pragma unroll
            for (int o = kLanesPerHead / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            rstd = rsqrtf(ss / static_cast<float>(HD) + p.eps[t]);
          } else if (live) {
            unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + c), g);
          }
          // the reference stores the normalised tensor in its own type before the rotation reads it
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] = round_bf16((x[j] * rstd) * g[j]);
        }
        if (rot) {
          float y[8];
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            y[j] = fmaf(-x[j + 1], sn[j], x[j] * cs[j]);
            y[j + 1] = fmaf(x[j], sn[j + 1], x[j + 1] * cs[j + 1]);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] = y[j];
        }
        if (live) {
          const int head = c / kLanesPerHead;
          dst[(static_cast<long long>(head) * p.out_len + p.out_row0 + i) * kLanesPerHead + in_head] = pack8(x);
        }
      }
    }
  }
}

}  // namespace

extern "C" int dfs_qkv_prepare(const void* q_src, const void* k_src, const void* v_src, const void* gamma_q,
                               const void* gamma_k, float eps_q, float eps_k, int norm_across_heads,
                               const float* cos_tab, const float* sin_tab, int rope_dim, int64_t rope_rows,
                               const int32_t* perm, void* q_out, void* k_out, void* v_out, int heads,
                               int64_t n_rows, int64_t out_row0, int64_t out_len, int head_dim, void* stream) {
  const void* srcs[3] = {q_src, k_src, v_src};
  void* dsts[3] = {q_out, k_out, v_out};
  if (head_dim != 64 && head_dim != 128) return DFS_ERR_SHAPE;
  if (heads <= 0 || n_rows < 0 || out_row0 < 0 || out_len < out_row0 + n_rows) return DFS_ERR_SHAPE;
  if ((cos_tab == nullptr) != (sin_tab == nullptr)) return DFS_ERR_NULL;
  if (cos_tab != nullptr) {
    if (rope_dim != head_dim && rope_dim != head_dim / 2) return DFS_ERR_SHAPE;
    if (rope_rows < 0) return DFS_ERR_RANGE;
    if (!dfs_aligned16(cos_tab) || !dfs_aligned16(sin_tab)) return DFS_ERR_ALIGN;
  }
  PrepareParams p = {};
  bool any = false;
  for (int t = 0; t < 3; ++t) {
    if ((srcs[t] == nullptr) != (dsts[t] == nullptr)) return DFS_ERR_NULL;
    if (srcs[t] == nullptr) continue;
    if (!dfs_aligned16(srcs[t]) || !dfs_aligned16(dsts[t])) return DFS_ERR_ALIGN;
    if (srcs[t] == dsts[t]) return DFS_ERR_RANGE;  // a transpose cannot run in place
    p.src[t] = static_cast<const uint4*>(srcs[t]);
    p.dst[t] = static_cast<uint4*>(dsts[t]);
    any = true;
  }
  if (!any || n_rows == 0) return 0;
  if ((gamma_q != nullptr && !dfs_aligned16(gamma_q)) || (gamma_k != nullptr && !dfs_aligned16(gamma_k)))
    return DFS_ERR_ALIGN;
  p.gamma[0] = static_cast<const __nv_bfloat16*>(gamma_q);
  p.gamma[1] = static_cast<const __nv_bfloat16*>(gamma_k);
  p.eps[0] = eps_q;
  p.eps[1] = eps_k;
  p.cos_tab = cos_tab;
  p.sin_tab = sin_tab;
  p.perm = perm;
  p.rope_rows = cos_tab ? rope_rows : 0;
  p.n_rows = n_rows;
  p.out_row0 = out_row0;
  p.out_len = out_len;
  p.heads = heads;
  p.norm_across_heads = norm_across_heads ? 1 : 0;
  p.rope_pairs = (cos_tab != nullptr && rope_dim == head_dim / 2) ? 1 : 0;
  const long long blocks = (n_rows + kWarpsPerCta - 1) / kWarpsPerCta;
  if (blocks > 0x7fffffffLL) return DFS_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (head_dim == 128)
    qkv_prepare_kernel<128><<<static_cast<unsigned>(blocks), kWarpsPerCta * 32, 0, s>>>(p);
  else
    qkv_prepare_kernel<64><<<static_cast<unsigned>(blocks), kWarpsPerCta * 32, 0, s>>>(p);
  return static_cast<int>(cudaGetLastError());
}
