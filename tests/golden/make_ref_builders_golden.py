"""Generates tests/golden/ref_builders.npz from the REFERENCE's own statements for the host-side
builders: the MSRoPE table of QwenImageDit::prepare (src/models/qwen_image/dit.cpp:128-183), the
timestep embedding of QwenImageDit::time_mod (:221-230), H3Dit::time_basis
(src/models/minimax_h3/dit.cpp:167-176) and the cos / sin table of H3Dit::prepare (:254-262), run
through oracle/_ref/libmx_ref_builders.so (built by oracle/Makefile from the reference tree; no GPU).

    python tests/golden/make_ref_builders_golden.py
"""
import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))
from oracle import binding as orc  # noqa: E402
import ref_builder_cases as cases  # noqa: E402


def digest(*arrays) -> np.ndarray:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest(), np.uint8).copy()


if __name__ == "__main__":
    orc.build(ref=True)
    out = {}
    for i, (T, H, W, conds) in enumerate(cases.QWEN_ROPE_FULL):
        out[f"qwen_rope_full{i}_cos"], out[f"qwen_rope_full{i}_sin"] = orc.ref_qwen_rope_table(T, H, W, conds)
    for i, (T, H, W, conds) in enumerate(cases.QWEN_ROPE_DIGEST):
        cos, sin = orc.ref_qwen_rope_table(T, H, W, conds)
        out[f"qwen_rope_digest{i}"] = digest(cos, sin)
        out[f"qwen_rope_digest{i}_rows"] = np.array([cos.shape[0]], np.int64)
    out["timestep_full"] = np.stack([orc.ref_qwen_timestep_embedding(float(t)) for t in cases.TIMESTEPS_FULL])
    out["timestep_digest"] = digest(*[orc.ref_qwen_timestep_embedding(float(t)) for t in cases.timesteps_digest()])
    table, ts, small = cases.h3_basis_inputs()
    out["h3_basis"] = orc.ref_h3_time_basis(ts, table)
    out["h3_basis_small"] = orc.ref_h3_time_basis(ts, small)
    invf = cases.h3_inv_freq()
    for name, pos in cases.h3_rope_positions():
        cos, sin = orc.ref_h3_rope_table(pos, invf)
        if pos.shape[0] <= 64:
            out[f"h3_rope_{name}_cos"], out[f"h3_rope_{name}_sin"] = cos, sin
        out[f"h3_rope_{name}_digest"] = digest(cos, sin)
    np.savez_compressed(Path(__file__).with_name("ref_builders.npz"), **out)
    print("wrote", len(out), "arrays")
