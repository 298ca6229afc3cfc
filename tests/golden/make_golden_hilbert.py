"""Golden Hilbert permutations from the third-party package the reference calls.

    python tests/golden/make_golden_hilbert.py OUT_DIR

``dfsattn/utils/order.py:4,250`` takes its Hilbert codes from ``hilbert.encode``
of the ``numpy-hilbert-curve`` package.  Where that package is installed this
script calls it exactly as the reference does (coordinates ordered [x, y, z],
``num_dims=3``, ``num_bits = max(1, ceil(log2(max(w, h, f))))``, order.py:228-256)
and stores the resulting permutations as ``hilbert_<f>x<h>x<w>.npy`` (outputs, not
source).  Where it is not installed the script says so and writes nothing; the
tests then pin the order by its properties only.  It also reports whether the two
other packages the reference's processors and sparse kernel need are present.
"""
import importlib
import json
import math
import os
import sys

import numpy as np

GRIDS = [(4, 16, 16), (3, 5, 7), (21, 30, 52), (33, 45, 80), (21, 45, 80)]


def reference_order(encode, f, h, w):
    max_dim = max(w, h, f)
    num_bits = max(1, math.ceil(math.log2(max_dim))) if max_dim > 1 else 1
    X = np.repeat(np.arange(w, dtype=np.int64), h * f)
    Y = np.tile(np.repeat(np.arange(h, dtype=np.int64), f), w)
    Z = np.tile(np.arange(f, dtype=np.int64), w * h)
    linear = Z * (h * w) + Y * w + X
    codes = np.asarray(encode(np.column_stack([X, Y, Z]), 3, num_bits)).astype(np.int64)
    return linear[np.argsort(codes, kind="stable")]


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    report = {}
    for name in ("hilbert", "diffusers", "block_sparse_attn"):
        try:
            mod = importlib.import_module(name)
            report[name] = "importable: " + str(getattr(mod, "__version__", getattr(mod, "__file__", "?")))
        except Exception as exc:  # noqa: BLE001  (the report wants the reason, whatever it is)
            report[name] = f"unavailable: {type(exc).__name__}: {exc}"
    if report["hilbert"].startswith("importable"):
        from hilbert import encode
        for f, h, w in GRIDS:
            np.save(os.path.join(out_dir, f"hilbert_{f}x{h}x{w}.npy"), reference_order(encode, f, h, w))
    with open(os.path.join(out_dir, "package_probe.json"), "w") as fh:
        json.dump(report, fh, indent=1)
    print(json.dumps(report))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else ".")
