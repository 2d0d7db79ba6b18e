"""Generates tests/golden/h3_ref2va_positions.npz: rotary positions of the reference-conditioned layout
from the REFERENCE's own host code (mx::h3_build_ref2va_layout, src/models/minimax_h3/layout.cpp:121-188,
built into oracle/_ref/libmx_ref_layout.so by oracle/Makefile).  Runs on the CPU where the reference tree
is present:

    python tests/golden/make_h3_ref2va_positions.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import binding as orc  # noqa: E402

# name -> (T, refs, F_lat, H, W, A)
CASES = {
    "no_refs": (7, [], 4, 6, 10, 11),
    "image_only": (5, [dict(kind="image", h=8, w=12)], 2, 6, 10, 3),
    "audio_only": (3, [dict(kind="audio", audio=9)], 7, 4, 4, 5),
    "video_with_track": (5, [dict(kind="video", frames=7, h=6, w=10, audio=13)], 12, 6, 10, 20),
    "video_longer_than_track": (4, [dict(kind="video", frames=11, h=4, w=6, audio=2)], 3, 8, 6, 4),
    "mixed": (5, [dict(kind="image", h=8, w=12), dict(kind="video", frames=7, h=6, w=10, audio=13),
                  dict(kind="audio", audio=9), dict(kind="video", frames=3, h=4, w=4, audio=0),
                  dict(kind="image", h=6, w=10)], 4, 6, 10, 11),
    "no_text": (0, [dict(kind="video", frames=2, h=2, w=2, audio=1)], 1, 2, 2, 1),
    # the headline video shape: 21 latent frames of 60 x 104, 512 text rows, one reference image
    "h3_480p_one_image": (512, [dict(kind="image", h=60, w=104)], 21, 60, 104, 203),
}

if __name__ == "__main__":
    out = {name: orc.h3_ref2va_positions(*c, use_reference=True) for name, c in CASES.items()}
    dst = Path(__file__).with_name("h3_ref2va_positions.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})
