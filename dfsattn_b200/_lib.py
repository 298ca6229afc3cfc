"""ctypes binding of libdfs_b200.so (the C ABI declared in include/dfs_b200.h).

There is no fallback: if the library is missing or a symbol is absent the
import fails loudly.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdfs_b200.so")

c_void_p, c_int, c_int64, c_float, c_double = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64,
                                               ctypes.c_float, ctypes.c_double)
c_uint32 = ctypes.c_uint32

# name -> (restype, argtypes); mirrors include/dfs_b200.h
SIGNATURES = {
    "dfs_version": (c_int, []),
    "dfs_status_string": (ctypes.c_char_p, [c_int]),
    "dfs_hilbert3d_perm": (c_int, [c_int, c_int, c_int, c_void_p]),
    "dfs_cache_schedule": (c_int, [c_int, c_int, c_int, c_double, c_double,
                                   ctypes.POINTER(c_int), ctypes.POINTER(c_double)]),
    "dfs_interaction_count": (c_int64, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int]),
    "dfs_permute_qkv": (c_int, [c_void_p] * 7 + [c_int, c_int64, c_int, c_void_p]),
    "dfs_unpermute": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_void_p]),
    "dfs_score_workspace_bytes": (c_int64, [c_int, c_int64, c_int64, c_int, c_int, c_int, c_int]),
    "dfs_block_scores": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_int, c_int,
                                 c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "dfs_block_scores_static_max_bytes": (c_int64, []),
    "dfs_block_scores_static": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_int, c_int,
                                        c_int, c_void_p, c_void_p, c_void_p]),
    "dfs_fine_top_p": (c_int, [c_void_p, c_int64, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]),
    "dfs_select_topk": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                c_void_p, c_int, c_void_p, c_void_p]),
    "dfs_block_sparse_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                     c_void_p, c_int, c_int64, c_int64, c_int, c_float, c_void_p, c_void_p]),
    "dfs_block_sparse_fwd_ex": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                        c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_float, c_void_p,
                                        c_void_p]),
    "dfs_block_sparse_fwd_fine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                          c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_float,
                                          c_void_p, c_void_p]),
    "dfs_block_sparse_fwd_batched": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                             c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int, c_float,
                                             c_void_p, c_void_p]),
    "dfs_permute_qkv_sharded": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_void_p]),
    "dfs_block_sparse_fwd_sharded": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                             c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int64, c_int64,
                                             c_int, c_float, c_void_p, c_void_p]),
    "dfs_qkv_prepare": (c_int, [c_void_p] * 5 + [c_float, c_float, c_int, c_void_p, c_void_p, c_int, c_int64,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int,
                                c_void_p]),
    "dfs_selftest_wait_timeout": (c_int, [c_int64, c_void_p, c_void_p]),
    "dfs_status_snapshot": (c_int, [c_void_p, c_void_p, c_void_p]),
}


class DfsLibraryError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise DfsLibraryError(
            f"{LIB_PATH} is missing: build it with `python dfsattn_b200/build.py` "
            "(there is no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise DfsLibraryError(f"{LIB_PATH} does not export {name}") from exc
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(code, what):
    """Raise for a non-zero status returned by a C-ABI call."""
    if code == 0:
        return
    msg = lib.dfs_status_string(int(code)).decode()
    if code < 0:
        raise ValueError(f"{what}: {msg} (code {code})")
    raise RuntimeError(f"{what}: {msg} (cudaError {code})")
