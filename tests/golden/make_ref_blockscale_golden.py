"""Generates tests/golden/ref_blockscale_sm100a.npz: outputs of the REFERENCE's own quantiser.

Runs src/kernels/blockscale.cu of the reference - compiled unmodified for sm_100a into
oracle/_ref/libmx_ref_blockscale.so by oracle/Makefile - on the seeded cases of
ref_blockscale_cases.py.  Needs a B200 and that library (built where the reference tree is present):

    python tests/golden/make_ref_blockscale_golden.py [out.npz]
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))
from oracle import binding as orc  # noqa: E402
import ref_blockscale_cases  # noqa: E402


def run_reference(L, mode, x_bits, K):
    """x_bits: uint16 [rows, ldx] on the host.  Returns (q, sf, amax) as numpy."""
    rows, ldx = x_bits.shape
    P, I64 = C.c_void_p, C.c_int64
    L.ref_qscale_bytes.restype = I64
    L.ref_qscale_bytes.argtypes = [C.c_int, I64, I64]
    L.ref_quantize_blockscaled.argtypes = [C.c_int, P, I64, I64, I64, P, P, P, P]
    L.ref_bs_last_error.restype = C.c_char_p
    x = torch.from_numpy(np.ascontiguousarray(x_bits)).cuda()
    q = torch.zeros(rows * K // (2 if mode == 2 else 1), dtype=torch.uint8, device="cuda")
    sf = torch.full((L.ref_qscale_bytes(mode, rows, K),), 0xAA, dtype=torch.uint8, device="cuda")
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    rc = L.ref_quantize_blockscaled(mode, x.data_ptr(), ldx, rows, K, q.data_ptr(), sf.data_ptr(), amax.data_ptr(), None)
    torch.cuda.synchronize()
    if rc:
        raise RuntimeError(L.ref_bs_last_error().decode())
    return q.cpu().numpy(), sf.cpu().numpy(), amax.cpu().numpy()


if __name__ == "__main__":
    L = orc.ref_blockscale()
    outs = {}
    for name, c in ref_blockscale_cases.cases().items():
        q, sf, amax = run_reference(L, c["mode"], c["x"], c["K"])
        outs[name + ".q"], outs[name + ".sf"], outs[name + ".amax"] = q, sf, amax
    dst = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).with_name("ref_blockscale_sm100a.npz")
    np.savez_compressed(dst, **outs)
    print("wrote", dst, len(outs), "arrays", sum(v.nbytes for v in outs.values()), "bytes")
