"""Torch-facing wrappers over the C ABI (include/dfs_b200.h).

Torch is used only for device memory and the current stream; every operator
below is one call into libdfs_b200.so.  Tensors are head-major [H, L, D].
"""
import math
from typing import Optional, Tuple

import torch

from ._lib import check, lib

BLOCK = 128
TILE = 16

_DTYPE_CODE = {torch.bfloat16: 0, torch.float32: 1}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("dfsattn_b200 operators need CUDA tensors (there is no CPU path)")


# ---- status word ------------------------------------------------------------
# One int32 per device that a kernel sets when one of its bounded waits ran out.  The word is
# sticky: once it is set, CTAs that start later return at once, so an operator must not go on
# handing out results.  Every operator call therefore polls it (below) without stalling the stream.
_status = {}
_monitors = {}


def _device_key(device) -> int:
    device = torch.device(device)
    return device.index if device.index is not None else torch.cuda.current_device()


def status_tensor(device) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait expired."""
    key = _device_key(device)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _status[key]


_STATUS_NAMES = {1: "a bounded wait inside a kernel expired", 2: "dynamic shared memory was not 1 KB aligned"}


def _raise_status(word: torch.Tensor, code: int):
    word.zero_()
    raise RuntimeError(f"dfsattn_b200 kernel reported device status {code} "
                       f"({_STATUS_NAMES.get(code, 'unknown code')}); results since the last check are invalid")


def check_status(device=None):
    """Synchronise and raise if any kernel on ``device`` reported a give-up."""
    device = torch.device("cuda" if device is None else device)
    word = status_tensor(device)
    code = int(word.item())
    mon = _monitors.get(_device_key(device))
    if mon is not None:
        mon["event"] = None
    if code != 0:
        _raise_status(word, code)


def poll_status(device):
    """Called at the start of every operator call: look at the copy of the status word that the
    PREVIOUS call queued (if that copy has finished; no wait otherwise), raise ``RuntimeError`` and
    clear the word if it was set, then queue a fresh snapshot into pinned host memory
    behind the work already on the current stream.  A give-up is therefore reported one call late
    at the latest once the stream has drained, and without any synchronisation on the fast path."""
    key = _device_key(device)
    word = status_tensor(device)
    mon = _monitors.get(key)
    if mon is None:
        mon = {"host": torch.zeros(1, dtype=torch.int32).pin_memory(), "event": None}
        _monitors[key] = mon
    ev = mon["event"]
    if ev is not None and ev.query():
        mon["event"] = None
        code = int(mon["host"][0])
        if code != 0:
            mon["host"][0] = 0
            _raise_status(word, code)
    if mon["event"] is None:
        # a one-thread kernel writes the word into the pinned host int: unlike a copy it does not queue
        # behind the large transfers a DMA engine may be busy with for other streams
        check(lib.dfs_status_snapshot(word.data_ptr(), mon["host"].data_ptr(), _stream(torch.device("cuda", key))),
              "dfs_status_snapshot")
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(torch.device("cuda", key)))
        mon["event"] = ev


# ---- host helpers -------------------------------------------------------------
def hilbert3d_perm(f: int, h: int, w: int) -> torch.Tensor:
    out = torch.empty(f * h * w, dtype=torch.int64)
    check(lib.dfs_hilbert3d_perm(f, h, w, out.data_ptr()), "dfs_hilbert3d_perm")
    return out


def cache_schedule(step_idx, skip_steps, cache_interval, sparsity, sparsity_dcrt) -> Tuple[bool, float]:
    import ctypes
    flag, cur = ctypes.c_int(0), ctypes.c_double(0.0)
    rc = lib.dfs_cache_schedule(int(step_idx), int(skip_steps), int(cache_interval), float(sparsity),
                                float(sparsity_dcrt), ctypes.byref(flag), ctypes.byref(cur))
    if rc == -5:  # DFS_ERR_RANGE: the reference raises ValueError here
        raise ValueError("cache_interval must be greater than 0.")
    check(rc, "dfs_cache_schedule")
    return bool(flag.value), float(cur.value)


def interaction_count(idx: Optional[torch.Tensor], cnt: Optional[torch.Tensor], heads, seq_len,
                      block=BLOCK) -> int:
    qb = kb = math.ceil(seq_len / block)
    if idx is None:
        r = lib.dfs_interaction_count(None, None, heads, qb, kb, 0, seq_len, block)
    else:
        idx_h = idx.detach().to("cpu", torch.int32).contiguous()
        cnt_h = cnt.detach().to("cpu", torch.int32).contiguous()
        r = lib.dfs_interaction_count(idx_h.data_ptr(), cnt_h.data_ptr(), heads, qb, kb, idx_h.shape[-1],
                                      seq_len, block)
    if r < 0:
        check(int(r), "dfs_interaction_count")
    return int(r)


# ---- permutation ----------------------------------------------------------------
def permute_qkv(q, k, v, perm_i32):
    """Gather rows of three [H, L, D] tensors by ``perm_i32`` in one launch."""
    _need_cuda(q, k, v, perm_i32)
    outs = [torch.empty_like(t) if t is not None else None for t in (q, k, v)]
    first = next(t for t in (q, k, v) if t is not None)
    H, L, D = first.shape
    for t in (q, k, v):
        if t is not None and (not t.is_contiguous() or t.shape != first.shape or t.dtype != first.dtype):
            raise ValueError("q, k, v must be contiguous [H, L, D] tensors of one dtype")
    check(lib.dfs_permute_qkv(_ptr(q), _ptr(k), _ptr(v), perm_i32.data_ptr(), _ptr(outs[0]), _ptr(outs[1]),
                              _ptr(outs[2]), H, L, D * first.element_size(), _stream(first.device)),
          "dfs_permute_qkv")
    return tuple(outs)


def unpermute(x, inv_perm_i32):
    _need_cuda(x, inv_perm_i32)
    if not x.is_contiguous():
        raise ValueError("x must be contiguous [H, L, D]")
    H, L, D = x.shape
    out = torch.empty_like(x)
    check(lib.dfs_unpermute(x.data_ptr(), inv_perm_i32.data_ptr(), out.data_ptr(), H, L,
                            D * x.element_size(), _stream(x.device)), "dfs_unpermute")
    return out


# ---- scoring + selection ----------------------------------------------------------
def block_scores(q_perm, k_perm, video_len: int, wan_layout: bool, tile=TILE, block=BLOCK,
                 workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 block scores [H, Rb, Kb] from permuted [H, L, D] tensors."""
    _need_cuda(q_perm, k_perm)
    if q_perm.dtype not in _DTYPE_CODE or k_perm.dtype != q_perm.dtype:
        raise ValueError("scores need bf16 or fp32 inputs")
    if not (q_perm.is_contiguous() and k_perm.is_contiguous()):
        raise ValueError("q, k must be contiguous")
    H, L, D = q_perm.shape
    need = lib.dfs_score_workspace_bytes(H, L, video_len, D, tile, block, int(wan_layout))
    if need < 0:
        check(int(need), "dfs_score_workspace_bytes")
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=q_perm.device)
    kb = math.ceil(L / block)
    rb = kb if wan_layout else math.ceil(video_len / block)
    out = torch.empty((H, rb, kb), dtype=torch.float32, device=q_perm.device)
    check(lib.dfs_block_scores(q_perm.data_ptr(), k_perm.data_ptr(), _DTYPE_CODE[q_perm.dtype], H, L,
                               video_len, D, tile, block, int(wan_layout), out.data_ptr(),
                               workspace.data_ptr(), workspace.numel() * workspace.element_size(),
                               status_tensor(q_perm.device).data_ptr(), _stream(q_perm.device)),
          "dfs_block_scores")
    return out


def fine_top_p(workspace: torch.Tensor, heads: int, seq_len: int, video_len: int, head_dim: int,
               wan_layout: bool, idx: torch.Tensor, cnt: torch.Tensor, n_rank: int, dense_row_start: int,
               top_p: float, tile=TILE, block=BLOCK) -> torch.Tensor:
    """64-bit tile maps int64 [H, Qb, kmax] for the lists (``dfs_fine_top_p``): which 16 x 16-token
    tiles of each listed 128 x 128 pair are attended.  ``workspace`` is the scratch ``block_scores``
    has just filled for the same shape."""
    _need_cuda(workspace, idx, cnt)
    if idx.dtype != torch.int32 or cnt.dtype != torch.int32 or not (idx.is_contiguous() and cnt.is_contiguous()):
        raise ValueError("idx, cnt must be contiguous int32")
    H, q_rows, kmax = idx.shape
    if H != heads or tuple(cnt.shape) != (H, q_rows):
        raise ValueError("lists do not match the head count")
    bits = torch.empty((H, q_rows, kmax), dtype=torch.int64, device=idx.device)
    check(lib.dfs_fine_top_p(workspace.data_ptr(), workspace.numel() * workspace.element_size(), heads, seq_len,
                             video_len, head_dim, tile, block, int(wan_layout), idx.data_ptr(), cnt.data_ptr(),
                             kmax, q_rows, int(n_rank), int(dense_row_start), float(top_p), bits.data_ptr(),
                             _stream(idx.device)), "dfs_fine_top_p")
    return bits


def block_scores_static(q_perm, k_perm, video_len: int, wan_layout: bool, out: torch.Tensor,
                        tile=TILE, block=BLOCK) -> torch.Tensor:
    """Block scores into the caller's ``out`` [H, Rb, Kb] fp32 without allocating
    anything: scratch is the 32 MiB array built into the library (see
    ``dfs_block_scores_static`` in include/dfs_b200.h for who needs this and the
    limits).  Raises ValueError when the shape needs more scratch than that."""
    _need_cuda(q_perm, k_perm, out)
    if q_perm.dtype not in _DTYPE_CODE or k_perm.dtype != q_perm.dtype:
        raise ValueError("scores need bf16 or fp32 inputs")
    if not (q_perm.is_contiguous() and k_perm.is_contiguous() and out.is_contiguous()):
        raise ValueError("q, k, out must be contiguous")
    H, L, D = q_perm.shape
    kb = math.ceil(L / block)
    rb = kb if wan_layout else math.ceil(video_len / block)
    if out.dtype != torch.float32 or tuple(out.shape) != (H, rb, kb):
        raise ValueError(f"out must be fp32 of shape {(H, rb, kb)}")
    check(lib.dfs_block_scores_static(q_perm.data_ptr(), k_perm.data_ptr(), _DTYPE_CODE[q_perm.dtype], H, L,
                                      video_len, D, tile, block, int(wan_layout), out.data_ptr(),
                                      status_tensor(q_perm.device).data_ptr(), _stream(q_perm.device)),
          "dfs_block_scores_static")
    return out


def select_topk(scores, q_rows: int, n_rank: int, k_select: int, dense_row_start: int,
                want_mask: bool = False):
    """Index lists (idx int32 [H, q_rows, kmax], cnt int32 [H, q_rows]) from fp32
    block scores [H, score_rows, n_cols]; optional uint8 mask [H, q_rows, n_cols]."""
    _need_cuda(scores)
    if scores.dtype != torch.float32 or not scores.is_contiguous():
        raise ValueError("scores must be contiguous fp32")
    H, score_rows, n_cols = scores.shape
    # lists are as long as a ranked row needs; rows from dense_row_start on get the count -1 ("every key
    # block") instead of a list of all of them
    kmax = max(1, k_select + (n_cols - n_rank))
    idx = torch.empty((H, q_rows, kmax), dtype=torch.int32, device=scores.device)
    cnt = torch.empty((H, q_rows), dtype=torch.int32, device=scores.device)
    mask = torch.empty((H, q_rows, n_cols), dtype=torch.uint8, device=scores.device) if want_mask else None
    check(lib.dfs_select_topk(scores.data_ptr(), H, score_rows, q_rows, n_cols, n_rank, k_select,
                              dense_row_start, idx.data_ptr(), cnt.data_ptr(), kmax, _ptr(mask),
                              _stream(scores.device)), "dfs_select_topk")
    return idx, cnt, mask


# ---- attention -----------------------------------------------------------------------
class ShardTable:
    """Where one tensor's sequence shards live on the GPUs of a node: device pointers (one per
    GPU, peer-accessible), tokens per shard and the row stride of a head inside a shard
    ([heads_total, stride_rows, D] each).  Passed to the *_sharded entry points as a host array."""

    def __init__(self, ptrs, shard_rows: int, stride_rows: int):
        import ctypes
        self.world = len(ptrs)
        self.array = (ctypes.c_void_p * self.world)(*[int(p) for p in ptrs])
        self.shard_rows = int(shard_rows)
        self.stride_rows = int(stride_rows)


def permute_qkv_sharded(q_tab: ShardTable, k_tab: ShardTable, v_tab: ShardTable, head0: int, heads: int,
                        seq_len: int, head_dim: int, perm, device):
    """Gather this GPU's heads [head0, head0 + heads) of Q, K, V from sequence shards on several GPUs
    into permuted bf16 [heads, L, D] tensors (``dfs_permute_qkv_sharded``)."""
    outs = [torch.empty((heads, seq_len, head_dim), dtype=torch.bfloat16, device=device) for _ in range(3)]
    check(lib.dfs_permute_qkv_sharded(q_tab.array, k_tab.array, v_tab.array, q_tab.world, q_tab.shard_rows,
                                      q_tab.stride_rows, head0, _ptr(perm), outs[0].data_ptr(),
                                      outs[1].data_ptr(), outs[2].data_ptr(), heads, seq_len, head_dim * 2,
                                      _stream(outs[0].device)), "dfs_permute_qkv_sharded")
    return outs


def block_sparse_fwd(q_perm, k_perm, v_perm, idx, cnt, out_row_map=None, kv_len=None, scale=None,
                     out=None, token_major=False, out_shards: Optional[ShardTable] = None, out_head0: int = 0,
                     batch: int = 1, fine: Optional[torch.Tensor] = None):
    """bf16 block-sparse attention over permuted [H, L, D] tensors; ``idx=None``
    attends every key block (dense).  ``token_major=True`` stores the result as
    [L, H, D] (the layout the output projection reads) instead of [H, L, D].

    ``batch`` > 1: the tensors are [batch * H, L, D], the lists [H, Qb, kmax] are shared by all
    batch elements, and the result is [batch, H, L, D] or, token-major, [batch, L, H, D]
    (``dfs_block_sparse_fwd_batched``).  ``fine``: int64 tile maps [H, Qb, kmax] from ``fine_top_p``
    (``dfs_block_sparse_fwd_fine``); not combined with ``batch`` or ``out_shards``."""
    _need_cuda(q_perm, k_perm, v_perm)
    for t in (q_perm, k_perm, v_perm):
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.shape != q_perm.shape:
            raise ValueError("q, k, v must be contiguous bf16 [H, L, D] tensors of one shape")
    H, L, D = q_perm.shape
    batch = int(batch)
    if batch < 1 or H % batch:
        raise ValueError("the leading dimension must be batch * heads")
    if fine is not None:
        if batch != 1 or out_shards is not None or idx is None:
            raise ValueError("tile maps go with plain lists of one batch element on one GPU")
        if fine.dtype != torch.int64 or not fine.is_contiguous() or tuple(fine.shape) != tuple(idx.shape) \
                or not fine.is_cuda:
            raise ValueError("fine must be a contiguous CUDA int64 tensor shaped like idx")
    if batch > 1:
        if out_shards is not None:
            raise ValueError("batched launches do not scatter to sequence shards")
        H //= batch
        if idx is not None and idx.shape[0] != H:
            raise ValueError("batched launches take one list per head of ONE batch element")
        want = (batch, L, H, D) if token_major else (batch, H, L, D)
        if out is None:
            out = torch.empty(want, dtype=q_perm.dtype, device=q_perm.device)
        elif tuple(out.shape) != want or not out.is_contiguous() or out.dtype != torch.bfloat16:
            raise ValueError(f"out must be a contiguous bf16 tensor of shape {want}")
        check(lib.dfs_block_sparse_fwd_batched(
            q_perm.data_ptr(), k_perm.data_ptr(), v_perm.data_ptr(), _ptr(idx), _ptr(cnt),
            0 if idx is None else idx.shape[-1], _ptr(out_row_map), out.data_ptr(), int(token_major), batch, H, L,
            L if kv_len is None else int(kv_len), D, D ** -0.5 if scale is None else float(scale),
            status_tensor(q_perm.device).data_ptr(), _stream(q_perm.device)), "dfs_block_sparse_fwd_batched")
        return out
    if out_shards is not None:
        # rows go straight to the sequence shards of the GPUs that own them; nothing is returned
        check(lib.dfs_block_sparse_fwd_sharded(
            q_perm.data_ptr(), k_perm.data_ptr(), v_perm.data_ptr(), _ptr(idx), _ptr(cnt),
            0 if idx is None else idx.shape[-1], _ptr(out_row_map), out_shards.array, out_shards.world,
            out_shards.shard_rows, out_shards.stride_rows, int(out_head0), H, L,
            L if kv_len is None else int(kv_len), D, D ** -0.5 if scale is None else float(scale),
            status_tensor(q_perm.device).data_ptr(), _stream(q_perm.device)), "dfs_block_sparse_fwd_sharded")
        return None
    want = (L, H, D) if token_major else (H, L, D)
    if out is None:
        out = torch.empty(want, dtype=q_perm.dtype, device=q_perm.device)
    elif tuple(out.shape) != want or not out.is_contiguous() or out.dtype != torch.bfloat16:
        raise ValueError(f"out must be a contiguous bf16 tensor of shape {want}")
    kv_len = L if kv_len is None else int(kv_len)
    scale = D ** -0.5 if scale is None else float(scale)
    kmax = 0 if idx is None else idx.shape[-1]
    if fine is not None:
        check(lib.dfs_block_sparse_fwd_fine(q_perm.data_ptr(), k_perm.data_ptr(), v_perm.data_ptr(), _ptr(idx),
                                            _ptr(cnt), fine.data_ptr(), kmax, _ptr(out_row_map), out.data_ptr(),
                                            int(token_major), H, L, kv_len, D, scale,
                                            status_tensor(q_perm.device).data_ptr(), _stream(q_perm.device)),
              "dfs_block_sparse_fwd_fine")
        return out
    check(lib.dfs_block_sparse_fwd_ex(q_perm.data_ptr(), k_perm.data_ptr(), v_perm.data_ptr(), _ptr(idx),
                                      _ptr(cnt), kmax, _ptr(out_row_map), out.data_ptr(), int(token_major),
                                      H, L, kv_len, D, scale, status_tensor(q_perm.device).data_ptr(),
                                      _stream(q_perm.device)), "dfs_block_sparse_fwd_ex")
    return out


# ---- fused pre-attention step ----------------------------------------------------------
def qkv_prepare(q_src, k_src, v_src, heads: int, *, gamma_q=None, gamma_k=None, eps_q=1e-6, eps_k=1e-6,
                norm_across_heads=False, cos=None, sin=None, rope_rows=None, perm=None,
                out=None, out_row0=0, out_len=None):
    """Projections [rows, H*D] (bf16, token-major) -> (q, k, v) head-major [H, out_len, D], with the
    RMSNorm, the rotary embedding of the first ``rope_rows`` source rows and the token gather
    ``perm`` applied on the way (``dfs_qkv_prepare`` in include/dfs_b200.h).  ``out`` is an
    optional (q, k, v) triple of [H, out_len, D] tensors to fill rows [out_row0, out_row0 + n)."""
    srcs = (q_src, k_src, v_src)
    first = next(t for t in srcs if t is not None)
    _need_cuda(first)
    for t in srcs:
        if t is not None and (t.dtype != torch.bfloat16 or not t.is_contiguous() or t.shape != first.shape
                              or t.dim() != 2):
            raise ValueError("projections must be contiguous bf16 [rows, H*D] tensors of one shape")
    rows, hd = first.shape
    if hd % heads:
        raise ValueError("row width is not a multiple of the head count")
    D = hd // heads
    n = rows if perm is None else perm.numel()
    out_len = out_row0 + n if out_len is None else int(out_len)
    if out is None:
        out = tuple(torch.empty((heads, out_len, D), dtype=torch.bfloat16, device=first.device)
                    if t is not None else None for t in srcs)
    for t, o in zip(srcs, out):
        if (t is None) != (o is None):
            raise ValueError("out must match the given projections")
        if o is not None and (tuple(o.shape) != (heads, out_len, D) or not o.is_contiguous()
                              or o.dtype != torch.bfloat16):
            raise ValueError(f"outputs must be contiguous bf16 {(heads, out_len, D)}")
    for g in (gamma_q, gamma_k):
        if g is not None and (g.dtype != torch.bfloat16 or not g.is_contiguous()
                              or g.numel() != (hd if norm_across_heads else D)):
            raise ValueError("norm weights must be contiguous bf16 of D (per head) or H*D elements")
    rope_dim = 0
    if cos is not None:
        if sin is None or cos.shape != sin.shape or cos.dtype != torch.float32 or sin.dtype != torch.float32 \
                or not (cos.is_contiguous() and sin.is_contiguous()) or cos.dim() != 2:
            raise ValueError("cos/sin must be contiguous fp32 [rows, D] or [rows, D/2] tables of one shape")
        rope_dim = cos.shape[1]
        rope_rows = cos.shape[0] if rope_rows is None else int(rope_rows)
        if rope_rows > cos.shape[0]:
            raise ValueError("rope_rows exceeds the table")
    if perm is not None and (perm.dtype != torch.int32 or not perm.is_contiguous()):
        raise ValueError("perm must be contiguous int32")
    check(lib.dfs_qkv_prepare(_ptr(q_src), _ptr(k_src), _ptr(v_src), _ptr(gamma_q), _ptr(gamma_k),
                              float(eps_q), float(eps_k), int(norm_across_heads), _ptr(cos), _ptr(sin),
                              rope_dim, int(rope_rows or 0), _ptr(perm), _ptr(out[0]), _ptr(out[1]),
                              _ptr(out[2]), heads, n, int(out_row0), out_len, D, _stream(first.device)),
          "dfs_qkv_prepare")
    return out
