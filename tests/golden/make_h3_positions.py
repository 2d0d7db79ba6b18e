"""Generates tests/golden/h3_positions.npz from the REFERENCE's own host code.

Runs mx::h3_build_layout (src/models/minimax_h3/layout.cpp:68-118) through
oracle/_ref/libmx_ref_layout.so, which oracle/Makefile compiles from the reference tree; needs that
tree, no GPU.    python tests/golden/make_h3_positions.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import binding as orc  # noqa: E402

CASES = [
    # T, F_lat, H, W, A, anchors
    (512, 21, 60, 104, 0, []),
    (37, 7, 30, 52, 25, ["first", "last"]),
    (5, 2, 4, 6, 3, ["last"]),
    (226, 12, 44, 80, 93, ["first"]),
    (0, 1, 2, 2, 0, []),
]

if __name__ == "__main__":
    orc.build(ref=True)
    out = {}
    for i, (T, F, H, W, A, anchors) in enumerate(CASES):
        pos = orc.h3_positions(T, F, H, W, A, anchors, use_reference=True)
        out[f"case{i}_args"] = np.array([T, F, H, W, A] + [0 if a == "first" else 1 for a in anchors], np.int64)
        out[f"case{i}_pos"] = pos
    np.savez_compressed(Path(__file__).with_name("h3_positions.npz"), **out)
    print("wrote", len(CASES), "cases")
