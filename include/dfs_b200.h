/*
 * dfs_b200.h -- C ABI of the B200 (sm_100a) DFS sparse-attention kernels.
 *
 * Drop-in boundary for the native DFS attention path of codesiena/DFSattn:
 * Hilbert permute -> pooled block scoring -> per-row top-k block selection ->
 * 128x128 block-sparse attention -> inverse permute.  The reference performs
 * these steps with PyTorch ops and a third-party CUDA extension; a binding
 * (ctypes / pybind / cffi) replaces those calls with the entry points below.
 * Citations are paths inside the reference repository.
 *
 * Conventions
 *  - Every function returns an int status: 0 = ok, negative = rejected
 *    argument (nothing was launched), positive = CUDA runtime error code.
 *  - Unless stated otherwise pointers are DEVICE pointers; tensors are dense,
 *    row-major, "head-major" [H, L, D] (the reference's [1,H,L,D] with the
 *    batch of one dropped; attention_hyvideo.py:399 asserts batch 1).
 *  - `stream` is a cudaStream_t passed as void*.  No call synchronises and none
 *    allocates device memory.  State kept between calls: host-side lookups that
 *    are made once (the driver's tensor-map encoder, the per-device address of
 *    the fixed scratch array of dfs_block_scores_static, the environment
 *    switches DFSATTN_DENSE_PAIRS and DFSATTN_SCORE_PAIRS: "0" runs dense
 *    attention calls, or the logits kernel of the block scoring, on single
 *    CTAs instead of CTA pairs; same results); nothing else.
 *  - Kernels never trap: every wait inside a kernel is bounded; a kernel that
 *    gives up writes a non-zero code to `*status` (device int32, caller
 *    zero-initialised, may be NULL for kernels that have no waits).  The word
 *    is sticky: while it is non-zero, CTAs that start later return at once, so
 *    the caller must read it back (asynchronously is enough), discard the
 *    results produced since its last look and zero it before going on.
 */
#ifndef DFS_B200_H
#define DFS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DFS_B200_VERSION 1

/* element types of Q/K/V/O */
#define DFS_DTYPE_BF16 0
#define DFS_DTYPE_F32 1

/* argument-rejection codes (negative return values) */
#define DFS_ERR_NULL -1        /* required pointer is NULL                   */
#define DFS_ERR_ALIGN -2       /* pointer not 16-byte aligned                */
#define DFS_ERR_SHAPE -3       /* unsupported shape (D, block, tile, sizes)  */
#define DFS_ERR_DTYPE -4       /* unsupported element type                   */
#define DFS_ERR_RANGE -5       /* k / count / length out of range            */
#define DFS_ERR_WORKSPACE -6   /* workspace too small                        */
#define DFS_ERR_DRIVER -7      /* tensor-map encode entry point unavailable  */
#define DFS_ERR_STATIC_SCRATCH -8 /* shape needs more scratch than the fixed
                                     in-library array of the _static entry point */

/* device status codes written by kernels to *status */
#define DFS_STATUS_OK 0
#define DFS_STATUS_WAIT_TIMEOUT 1 /* a bounded barrier wait expired           */
#define DFS_STATUS_BAD_SMEM_ALIGNMENT 2 /* dynamic shared memory not 1 KB aligned */

int dfs_version(void);
const char* dfs_status_string(int code);

/* ---- host-side helpers (no GPU needed) --------------------------------- */

/* 3-D Hilbert token order over an f x h x w latent grid.
 * Replaces hilbert3d_perm(), dfsattn/utils/order.py:206-258 (curve over the
 * enclosing 2^b cube, points outside the grid dropped; coordinates ordered
 * [x, y, z]; raster index z*h*w + y*w + x).  perm_out: HOST int64[f*h*w]. */
int dfs_hilbert3d_perm(int f, int h, int w, int64_t* perm_out);

/* Refresh flag and current sparsity for a denoising step.
 * Replaces _compute_cache_schedule(), dfsattn/attention_hyvideo.py:40-65.
 * Returns DFS_ERR_RANGE when cache_interval <= 0 (the reference raises). */
int dfs_cache_schedule(int step_idx, int skip_steps, int cache_interval, double sparsity,
                       double sparsity_dcrt, int* is_cache_step, double* current_sparsity);

/* Selected (q,k) token pairs of index lists, with partial last blocks.
 * Replaces _block_interaction_count(), dfsattn/attention_hyvideo.py:521-546.
 * idx/cnt are HOST copies of the lists (idx may be NULL for "all blocks"). */
int64_t dfs_interaction_count(const int32_t* idx_host, const int32_t* cnt_host, int heads,
                              int q_blocks, int k_blocks, int kmax, int64_t seq_len, int block);

/* ---- permutation -------------------------------------------------------- */

/* dst[h, i, :] = src[h, perm[i], :] for three tensors in one launch.
 * Replaces _apply_permutation_in_place() x3, dfsattn/attention_hyvideo.py:177-184
 * as called at :1034-1036.  row_bytes = D * sizeof(element), multiple of 16.
 * Any of the three (src,dst) pairs may be NULL/NULL to skip it. */
int dfs_permute_qkv(const void* q, const void* k, const void* v, const int32_t* perm,
                    void* q_out, void* k_out, void* v_out, int heads, int64_t seq_len,
                    int row_bytes, void* stream);

/* dst[h, i, :] = src[h, inv_perm[i], :].
 * Replaces _apply_inverse_permutation(), dfsattn/attention_hyvideo.py:187-194
 * (call site :1086).  The attention entry point can write un-permuted rows
 * itself (out_row_map), which makes this call unnecessary on the hot path. */
int dfs_unpermute(const void* src, const int32_t* inv_perm, void* dst, int heads,
                  int64_t seq_len, int row_bytes, void* stream);

/* ---- sequence shards on several GPUs (fused with the exchange) -------------- */

/* dfs_permute_qkv for inputs that are sharded along the sequence over `world` GPUs of one node:
 * the gather reads every row it needs straight from the shard that holds it (plain loads from
 * peer memory over NVLink), so the Q/K/V all-to-all that would otherwise bring the sequence
 * together (what Ulysses-style sequence parallelism does before attention) and the Hilbert
 * gather of dfsattn/attention_hyvideo.py:1034-1036 are one pass.  The reference has no multi-GPU
 * path for this operator; this is the entry point for callers whose activations are sequence-sharded.
 *  q/k/v_shards : HOST arrays of `world` DEVICE pointers; shard s holds tokens
 *                 [s*shard_rows, min((s+1)*shard_rows, L)) of ALL heads as
 *                 [heads_total, shard_stride_rows, D] (shard_stride_rows >= shard_rows).  Pointers
 *                 of other GPUs must be peer-accessible (CUDA IPC / symmetric memory).
 *  head0, heads : this GPU gathers heads [head0, head0 + heads) into q/k/v_out [heads, L, D].
 *  perm         : int32 [L] (global token order) or NULL for the identity.
 * The caller orders the launch after every GPU has written its shard (a barrier across GPUs). */
int dfs_permute_qkv_sharded(const void* const* q_shards, const void* const* k_shards,
                            const void* const* v_shards, int world, int64_t shard_rows,
                            int64_t shard_stride_rows, int head0, const int32_t* perm, void* q_out,
                            void* k_out, void* v_out, int heads, int64_t seq_len, int row_bytes,
                            void* stream);

/* dfs_block_sparse_fwd whose result goes back to sequence shards on `world` GPUs: the row of
 * token d (after out_row_map) of local head h is stored in shard d / shard_rows at
 * [head0 + h, d % shard_rows, :] (plain stores to peer memory), which replaces the output
 * all-to-all.  out_shards as the input tables above.  The caller makes the other GPUs wait
 * (a barrier across GPUs) before they read their shard. */
int dfs_block_sparse_fwd_sharded(const void* q, const void* k, const void* v, const int32_t* idx,
                                 const int32_t* cnt, int kmax, const int32_t* out_row_map,
                                 void* const* out_shards, int world, int64_t shard_rows,
                                 int64_t shard_stride_rows, int head0, int heads, int64_t seq_len,
                                 int64_t kv_len, int head_dim, float scale, int32_t* status, void* stream);

/* ---- fused pre-attention step (processor side) --------------------------- */

/* Token-major projections [rows, H*D] (bf16) -> head-major, normalised, rotated and
 * token-permuted [H, out_len, D] in one pass:
 *   out[h, out_row0 + i, :] = rope(rmsnorm(src[row(i), h*D:(h+1)*D])),  row(i) = perm ? perm[i] : i.
 * Replaces, for Q and K, unflatten/transpose/contiguous (dfsattn/replace_hyvideo.py:247-249,
 * replace_wan.py:174-176), the RMSNorm (per head: kernels/include/norm/narrow_rms_norm.cuh:22-71 as
 * called from kernels/__init__.py:34-52; over the whole H*D row: kernels/triton/rmsnorm.py:8-49 as
 * called at replace_wan.py:162-166), the rotary embedding of the leading rope_rows tokens
 * (kernels/include/rope/rope_enc.cuh:17-36 and rope_enc_txtlast.cuh:33-75; complex form:
 * replace_wan.py:207-215) and the Hilbert gather of dfsattn/attention_hyvideo.py:1034-1036; V is
 * transposed and gathered only.  Arithmetic as in those kernels: fp32, y = (x*rsqrt(mean(x^2)+eps))*gamma
 * rounded to bf16, then out[i] = y[i]*cos[i] + (i even ? -y[i+1] : y[i-1])*sin[i] rounded to bf16.
 *  q_src/k_src/v_src : bf16 [src_rows, H*D]; any may be NULL together with its output.
 *  gamma_q/gamma_k   : bf16 [D] (norm_across_heads == 0) or [H*D] (!= 0); NULL = no norm.
 *  cos_tab/sin_tab   : fp32 [rope_rows, rope_dim], rope_dim == D (one value per element, pairs hold the
 *                      same value twice) or D/2 (one value per pair: real and imaginary part of the
 *                      complex frequencies); NULL = no rotation.  Source rows >= rope_rows (text) are
 *                      not rotated.
 *  perm              : int32 [n_rows] or NULL (identity).
 *  Two calls assemble a tensor whose text rows come from separate projections
 *  (replace_hyvideo.py:292-312): video rows with out_row0 = 0, text rows with out_row0 = video_len. */
int dfs_qkv_prepare(const void* q_src, const void* k_src, const void* v_src, const void* gamma_q,
                    const void* gamma_k, float eps_q, float eps_k, int norm_across_heads,
                    const float* cos_tab, const float* sin_tab, int rope_dim, int64_t rope_rows,
                    const int32_t* perm, void* q_out, void* k_out, void* v_out, int heads,
                    int64_t n_rows, int64_t out_row0, int64_t out_len, int head_dim, void* stream);

/* ---- scoring + selection ------------------------------------------------ */

/* Bytes of scratch dfs_block_scores needs for this shape. */
int64_t dfs_score_workspace_bytes(int heads, int64_t seq_len, int64_t video_len, int head_dim,
                                  int tile, int block, int wan_layout);

/* Pooled block scores, fp32 [H, Rb, Kb] with Kb = ceil(L/block) and
 * Rb = ceil(video_len/block) (hyvideo layout) or Kb (wan layout).
 * Replaces _compute_tile_score() + the 8x8 tile sums,
 * dfsattn/attention_hyvideo.py:310-385,419-422 (hyvideo layout: zero gap
 * between video and text, query tiles cover the video part only) and
 * dfsattn/attention_wan.py:157-209,243-246 (wan_layout != 0: zero pad at the
 * end only, query tiles cover everything).  q, k are the PERMUTED tensors
 * [H, L, D] (bf16 or f32).  Means are fp32, carried into the tensor-core
 * product as a bf16 hi + lo pair (16 significant bits), logits accumulate in
 * fp32, softmax and sums are fp32.  tile is 16, 32 or 64 and block 128; workspace
 * 256-byte aligned; status: device int32, zero-initialised by the caller. */
int dfs_block_scores(const void* q_perm, const void* k_perm, int dtype, int heads,
                     int64_t seq_len, int64_t video_len, int head_dim, int tile, int block,
                     int wan_layout, float* block_scores, void* workspace,
                     int64_t workspace_bytes, int32_t* status, void* stream);

/* dfs_block_scores for callers that cannot allocate device memory.
 * No counterpart in the reference: the reference lets PyTorch allocate its
 * temporaries freely.  This variant exists for hosts that must not call
 * cudaMalloc (or any allocating routine) when scores are needed -- a server
 * whose device memory pool is sized once and then frozen, a plugin invoked
 * from inside another framework's step where an allocation would stall the
 * device, a process that has already given all free memory to its tensor
 * allocator.  Same arguments and results as dfs_block_scores minus the
 * workspace: the scratch is a fixed array of
 * dfs_block_scores_static_max_bytes() bytes (32 MiB) inside the library image,
 * resident on every GPU that loads the library until the process exits.
 *  - Shapes whose scratch need (dfs_score_workspace_bytes) exceeds that size
 *    are rejected with DFS_ERR_STATIC_SCRATCH; nothing is launched.
 *  - The first call on each device looks up the array's device address (with
 *    that device current); make that first call outside any stream capture.
 *    The address is kept per device ordinal for the life of the process:
 *    after cudaDeviceReset() on a device this entry point must not be used on
 *    it again.  Concurrent first calls from several host threads are safe.
 *  - The call allocates nothing and frees nothing.
 *  - All calls on a device share the one array, which keeps the previous
 *    call's contents; nothing in it needs to be cleared between calls (every
 *    element that is read has been written earlier in the same call), but two
 *    calls whose kernels overlap on the GPU (different streams) race on it:
 *    serialise them on one stream or with events. */
int64_t dfs_block_scores_static_max_bytes(void);
int dfs_block_scores_static(const void* q_perm, const void* k_perm, int dtype, int heads,
                            int64_t seq_len, int64_t video_len, int head_dim, int tile, int block,
                            int wan_layout, float* block_scores, int32_t* status, void* stream);

/* Per (head, row): the k_select largest of scores[h, r, 0:n_rank) (ties: lowest
 * column first), plus every column in [n_rank, n_cols) ("forced" columns),
 * written in ascending order to idx[h, r, 0:cnt) and padded with -1 up to
 * kmax (>= k_select + n_cols - n_rank); rows r >= dense_row_start select every
 * column: listed like the others when kmax >= n_cols, otherwise the row gets
 * cnt = -1 ("every key block", understood by the attention and counting entry
 * points) and no list, so that a few dense rows do not set kmax for all rows.
 * Replaces torch.topk + scatter_ and the dense text rules,
 * dfsattn/attention_hyvideo.py:431-443,491-501 and attention_wan.py:248-253.
 * scores: fp32 [H, score_rows, n_cols]; idx: int32 [H, q_rows, kmax];
 * cnt: int32 [H, q_rows]; mask_out (optional): uint8 [H, q_rows, n_cols].
 * Rows r >= score_rows must be dense rows. */
int dfs_select_topk(const float* scores, int heads, int score_rows, int q_rows, int n_cols,
                    int n_rank, int k_select, int dense_row_start, int32_t* idx, int32_t* cnt,
                    int kmax, uint8_t* mask_out, void* stream);

/* ---- block-sparse attention forward ------------------------------------- */

/* O[h, map(i), :] = softmax_j( q_i . k_j * scale ) v_j over the keys j of the
 * 128-token key blocks listed for query block i/128, bf16 in / fp32
 * accumulate / bf16 out, on tcgen05 tensor cores.
 * Replaces block_sparse_attn_func(..., base_blockmask, ...) as called at
 * dfsattn/attention_hyvideo.py:1075-1082 and attention_wan.py:379-386, and,
 * with idx == NULL (every key block), flash_attn_varlen_func at
 * dfsattn/fullattention.py:108-116 (with D = 128 that dense call runs as
 * clusters of two CTAs sharing every K and V tile; same results).
 *  q, k, v : bf16 [H, L, D], already permuted; D = 64 or 128.
 *  idx/cnt : int32 [H, Qb, kmax] / [H, Qb] ascending block lists (Qb = ceil(L/128));
 *            cnt = -1 marks a row that attends every key block (its list is not read).
 *  kv_len  : keys j >= kv_len are masked out (L when there is no padding).
 *  out_row_map : int32 [L] or NULL; row i of the result is stored at row
 *            out_row_map[i] (pass the forward permutation to fuse the
 *            inverse permute of attention_hyvideo.py:1086).
 *  scale   : softmax scale (the reference uses D^-0.5).
 *  status  : device int32, zero-initialised by the caller. */
int dfs_block_sparse_fwd(const void* q, const void* k, const void* v, const int32_t* idx,
                         const int32_t* cnt, int kmax, const int32_t* out_row_map, void* out,
                         int heads, int64_t seq_len, int64_t kv_len, int head_dim, float scale,
                         int32_t* status, void* stream);

/* dfs_block_sparse_fwd with a choice of output layout: out_token_major == 0 stores [H, L, D] as
 * above; != 0 stores token-major [L, H*D], which is what the output projection reads, so that the
 * transpose(1, 2).flatten(2, 3) copy after the attention call (dfsattn/replace_hyvideo.py:443,
 * replace_wan.py:311) disappears together with the inverse permute. */
int dfs_block_sparse_fwd_ex(const void* q, const void* k, const void* v, const int32_t* idx,
                            const int32_t* cnt, int kmax, const int32_t* out_row_map, void* out,
                            int out_token_major, int heads, int64_t seq_len, int64_t kv_len,
                            int head_dim, float scale, int32_t* status, void* stream);

/* The "kp" selector: fine top-p inside the chosen block pairs.  Replaces
 * _refine_topk_mask_with_subblock_top_p (dfsattn/attention_hyvideo.py:211-302, reached from
 * _compute_block_mask :481-489 when selector_mode == "kp").  Call it right after dfs_block_scores
 * with the SAME shape arguments and workspace (it reads the pooled means and log-sum-exps left
 * there) and after dfs_select_topk (it walks the lists).  For every list entry (head, query block,
 * slot) it writes a 64-bit map, bit 8 * i + j = the 16 x 16-token tile (query tile i, key tile j)
 * of that 128 x 128 pair is attended: the pair's 64 softmax-ed tile scores are ranked jointly,
 * largest first, and a tile is kept while the scores ranked before it sum to less than fine_top_p
 * times the pair's total (scores exactly equal to the smallest kept one are all kept).  Key
 * blocks >= n_rank (text / boundary columns) and query rows >= dense_row_start keep whole pairs (all ones, :298-301; rows with cnt = -1 attend every block
 * anyway and get 0, their maps are not read); slots >= cnt get 0.  tile must be 16.
 *  idx/cnt   : the lists, int32 [H, q_rows, kmax] / [H, q_rows], each list ascending (as
 *              dfs_select_topk writes them: the refinable entries are then a prefix).
 *  fine_bits : uint64 [H, q_rows, kmax]. */
int dfs_fine_top_p(const void* workspace, int64_t workspace_bytes, int heads, int64_t seq_len,
                   int64_t video_len, int head_dim, int tile, int block, int wan_layout,
                   const int32_t* idx, const int32_t* cnt, int kmax, int q_rows, int n_rank,
                   int dense_row_start, float fine_top_p, uint64_t* fine_bits, void* stream);

/* dfs_block_sparse_fwd_ex restricted further to the 16 x 16-token tiles named by the maps of
 * dfs_fine_top_p (fine_bits: uint64 [H, Qb, kmax], one map per list entry): scores of dropped
 * tiles are excluded from the softmax.  Replaces kp_fine_sparse_attention as called at
 * dfsattn/attention_hyvideo.py:968-982 (the reference's Triton kernel over compact 16 x 16 masks,
 * dfsattn/kernels/triton/kp_flex_attention.py).  The tensor-core work is that of the listed
 * 128 x 128 blocks; dropped tiles save softmax work only.  A row left without any key gets zeros. */
int dfs_block_sparse_fwd_fine(const void* q, const void* k, const void* v, const int32_t* idx,
                              const int32_t* cnt, const uint64_t* fine_bits, int kmax,
                              const int32_t* out_row_map, void* out, int out_token_major, int heads,
                              int64_t seq_len, int64_t kv_len, int head_dim, float scale,
                              int32_t* status, void* stream);

/* Several batch elements that share ONE set of block lists, in one launch: the two
 * classifier-free-guidance passes of a Wan denoising step.  The reference runs them as two
 * successive calls (its processor counts two calls per step, dfsattn/replace_wan.py:253,320-323,
 * and its operator refuses batch > 1, dfsattn/attention_wan.py:219); the second call reuses the
 * mask the first one cached, because the Wan cache key carries no step or sparsity term
 * (attention_wan.py:147-154, :792-800).
 *  q, k, v : bf16 [batch * H, L, D] (batch-major: element b holds heads b*H .. b*H+H-1).
 *  idx/cnt : int32 [H, Qb, kmax] / [H, Qb]; head h of EVERY element uses list h.
 *  out     : [batch, H, L, D] or, token-major, [batch, L, H*D].
 * Everything else as dfs_block_sparse_fwd_ex; batch == 1 is the same call. */
int dfs_block_sparse_fwd_batched(const void* q, const void* k, const void* v, const int32_t* idx,
                                 const int32_t* cnt, int kmax, const int32_t* out_row_map, void* out,
                                 int out_token_major, int batch, int heads, int64_t seq_len,
                                 int64_t kv_len, int head_dim, float scale, int32_t* status,
                                 void* stream);

/* ---- diagnostics ----------------------------------------------------------- */

/* Copies the status word to *mirror behind the work already queued on `stream`, with a one-thread
 * kernel.  mirror is any address the device can write: device memory, or page-locked host memory
 * (with unified addressing its host pointer is the device pointer), which the host can then poll
 * without synchronising and without putting a copy into the queue of a DMA engine, where it would
 * wait behind large transfers of other streams.  No counterpart in the reference. */
int dfs_status_snapshot(const int32_t* status, int32_t* mirror, void* stream);

/* Exercises the give-up path of the kernels' bounded waits without any other work: one small
 * CTA waits, for at most limit_cycles SM clock cycles, on a barrier that nothing ever completes,
 * then leaves through the same tear-down as the attention kernel and writes
 * DFS_STATUS_WAIT_TIMEOUT to *status.  No counterpart in the reference (which has no bounded
 * waits); it lets a host verify its handling of the status word on a healthy GPU.
 * limit_cycles must be in [1, 2^31). */
int dfs_selftest_wait_timeout(int64_t limit_cycles, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DFS_B200_H */
