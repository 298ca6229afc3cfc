"""Golden fine masks of the "kp" selector, made by running the REFERENCE's own code on CPU.

    python tests/golden/make_golden_kp.py /path/to/reference

For every case of ``tests/golden_cases.py`` it calls the reference's
``DFS_Attention(..., selector_mode="kp", fine_top_p=p)._compute_block_mask`` (which ends in
``_refine_topk_mask_with_subblock_top_p``, dfsattn/attention_hyvideo.py:211-302) on the seeded
synthetic inputs and stores the resulting 16 x 16-token mask, bit-packed, for p = 0.9 and p = 0.5 in
``tests/golden/kp_<case>.npz``.  Only outputs are stored, no reference source.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from golden_cases import CASES, inputs  # noqa: E402

FINE_TOP_P = (0.9, 0.5)


def main():
    if len(sys.argv) < 2:
        raise SystemExit(f"usage: python {sys.argv[0]} <checkout of codesiena/DFSattn>")
    sys.path.insert(0, sys.argv[1])
    import dfsattn.attention_hyvideo as ref_hy
    torch.set_num_threads(8)
    for name, spec in CASES.items():
        q, k, v, vperm = inputs(name)
        L = q.shape[2]
        video_len = L - spec["text"]
        out = {}
        for p in FINE_TOP_P:
            att = ref_hy.DFS_Attention(0, 0, spec["sparsity"], True, video_len, vperm, 128, 16, 16,
                                       selector_mode="kp", fine_top_p=p)
            perm, _ = att._compute_permutation(vperm, L, torch.device("cpu"))
            fine = att._compute_block_mask(q, k, perm, spec["sparsity"])
            tag = f"p{int(round(p * 100)):02d}"
            out[f"fine_shape_{tag}"] = np.array(fine.shape)
            out[f"fine_bits_{tag}"] = np.packbits(fine.numpy().reshape(-1))
            print(name, tag, tuple(fine.shape), "density", float(fine.float().mean()))
        np.savez_compressed(os.path.join(HERE, "kp_" + name + ".npz"), **out)


if __name__ == "__main__":
    main()
