"""Generate golden fixtures by running the REFERENCE's own Python code on CPU.

Run in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports ``dfsattn.attention_hyvideo`` / ``dfsattn.attention_wan`` from the
reference checkout, feeds them seeded synthetic inputs and stores the results
(schedule table, block score sums, block masks, interaction counts, attention
outputs of the reference's packed CPU loop) as ``tests/golden/*.npz`` together
with a checksum of the inputs.  Only outputs are stored, no reference source.

The Hilbert permutation fed to the reference functions comes from
``oracle.hilbert`` because the reference's own builder needs a third-party
package that is not available offline; to the functions exercised here the
permutation is plain input data.
"""

import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

CASES = {
    # name: grid, text_len, heads, dim, sparsity, order
    "cfg0_4x16x16": dict(grid=(4, 16, 16), text=0, heads=2, dim=64, sparsity=0.3, order="hilbert3d"),
    "hy_text_4x12x20_t100": dict(grid=(4, 12, 20), text=100, heads=2, dim=128, sparsity=0.5, order="hilbert3d"),
    "hy_text_5x11x17_t256": dict(grid=(5, 11, 17), text=256, heads=3, dim=128, sparsity=0.45, order="hilbert3d"),
    "ragged_5x11x17": dict(grid=(5, 11, 17), text=0, heads=2, dim=128, sparsity=0.3, order="hilbert3d"),
    "raster_3x16x16": dict(grid=(3, 16, 16), text=0, heads=2, dim=64, sparsity=0.34, order="raster"),
}

# attention outputs are stored for every ROW_STRIDE-th token only (fixture size)
ROW_STRIDE = 5

SCHEDULES = [
    dict(skip_steps=12, cache_interval=12, sparsity=0.3, sparsity_dcrt=0.1, steps=50),
    dict(skip_steps=12, cache_interval=12, sparsity=0.25, sparsity_dcrt=0.1, steps=50),
    dict(skip_steps=0, cache_interval=5, sparsity=0.5, sparsity_dcrt=0.0, steps=30),
    dict(skip_steps=24, cache_interval=24, sparsity=0.3, sparsity_dcrt=0.1, steps=100),
    dict(skip_steps=3, cache_interval=7, sparsity=0.4, sparsity_dcrt=0.15, steps=40),
]


def checksum(*tensors):
    m = hashlib.sha256()
    for t in tensors:
        m.update(t.contiguous().numpy().tobytes())
    return m.hexdigest()


def case_inputs(spec, seed=0):
    from dfsattn_b200.synthetic import structured_qkv
    from oracle.hilbert import hilbert3d_perm
    f, h, w = spec["grid"]
    q, k, v = structured_qkv(spec["grid"], spec["heads"], spec["dim"], text_len=spec["text"],
                             dtype=torch.float32, device="cpu", seed=seed)
    vperm = torch.from_numpy(hilbert3d_perm(f, h, w)) if spec["order"] == "hilbert3d" else None
    return q, k, v, vperm


def main():
    if len(sys.argv) < 2:
        raise SystemExit(f"usage: python {sys.argv[0]} <checkout of codesiena/DFSattn>")
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    import dfsattn.attention_hyvideo as ref_hy
    import dfsattn.attention_wan as ref_wan

    # ---- schedule tables --------------------------------------------------
    sched = {}
    for i, s in enumerate(SCHEDULES):
        flags, vals = [], []
        for step in range(s["steps"]):
            f_, v_ = ref_hy._compute_cache_schedule(step, s["skip_steps"], s["cache_interval"],
                                                    s["sparsity"], s["sparsity_dcrt"])
            f2, v2 = ref_wan._compute_cache_schedule(step, s["skip_steps"], s["cache_interval"],
                                                     s["sparsity"], s["sparsity_dcrt"])
            assert (f_, v_) == (f2, v2)
            flags.append(f_)
            vals.append(v_)
        sched[f"flags_{i}"] = np.array(flags)
        sched[f"vals_{i}"] = np.array(vals, dtype=np.float64)
        sched[f"params_{i}"] = np.array([s["skip_steps"], s["cache_interval"], s["sparsity"],
                                         s["sparsity_dcrt"], s["steps"]], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "schedule.npz"), **sched)

    # ---- scoring / mask / attention --------------------------------------
    for name, spec in CASES.items():
        q, k, v, vperm = case_inputs(spec)
        L = q.shape[2]
        video_len = L - spec["text"]
        out = {"input_sha256": np.array(checksum(q, k, v))}

        hy = ref_hy.DFS_Attention(0, 0, spec["sparsity"], True, video_len, vperm, 128, 16, 16)
        perm, inv = hy._compute_permutation(vperm, L, torch.device("cpu"))
        ts = hy._compute_tile_score(q, k, 16, 16, 128, perm)
        vb, kb = -(-video_len // 128), -(-L // 128)
        out["hy_block_sums"] = ts.view(1, spec["heads"], vb, 8, kb, 8).sum(dim=(3, 5))[0].numpy()
        mask = hy._compute_block_mask(q, k, perm, spec["sparsity"])
        out["hy_mask"] = mask.numpy()
        out["hy_pairs"] = np.array(hy._block_interaction_count(mask, L))
        frontier = torch.zeros_like(mask)
        o, _ = hy._run_oracle_hybrid_attention(q, k, v, perm, inv, mask, frontier)
        out["hy_attn"] = o[:, :, ::ROW_STRIDE].numpy()
        dense = torch.ones_like(mask)
        o, _ = hy._run_oracle_hybrid_attention(q, k, v, perm, inv, dense, frontier)
        out["dense_attn"] = o[:, :, ::ROW_STRIDE].numpy()

        if spec["text"] == 0:
            wan = ref_wan.DFS_Attention(0, 0, spec["sparsity"], True, vperm, 128, 16, 16)
            wperm, _ = wan._compute_permutation(vperm, L, torch.device("cpu"))
            ts = wan._compute_tile_score(q, k, 16, 16, 128, wperm)
            out["wan_block_sums"] = ts.view(1, spec["heads"], kb, 8, kb, 8).sum(dim=(3, 5))[0].numpy()
            wmask = wan._compute_block_mask(q, k, wperm, spec["sparsity"])
            out["wan_mask"] = wmask.numpy()
            o, _ = hy._run_oracle_hybrid_attention(q, k, v, perm, inv, wmask, frontier)
            out["wan_attn"] = o[:, :, ::ROW_STRIDE].numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "L", L, "Kb", kb, "pairs", int(out["hy_pairs"]))


if __name__ == "__main__":
    main()
