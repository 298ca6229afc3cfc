"""B200-native (sm_100a) DFS sparse attention behind the reference's processor API.

Public surface (names follow codesiena/DFSattn):
  dfsattn_b200.attention_hyvideo : DFS_Attention, dfs_attention, _compute_cache_schedule
  dfsattn_b200.attention_wan     : DFS_Attention, dfs_attention
  dfsattn_b200.replace_hyvideo   : HunyuanVideo_DFSAttn_Processor2_0
  dfsattn_b200.replace_wan       : Wan_DFSAttn_Processor2_0
  dfsattn_b200.order             : hilbert3d_perm, build_video_perm
  dfsattn_b200.ops               : one wrapper per C-ABI entry point

Importing the package loads libdfs_b200.so and fails loudly when it is missing.
"""
from . import _lib  # noqa: F401  (loads the shared library)

__version__ = "0.1.0"
