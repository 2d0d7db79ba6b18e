"""Seeded inputs for the activation block-scale quantiser, shared by make_ref_blockscale_golden.py
(which runs the REFERENCE's kernel on them on a GPU) and by the tests that replay them through the CPU
oracle and through libmxk.  Every case: mode (1 MXFP8, 2 NVFP4), x = bf16 bits [rows, ldx], K."""
import numpy as np

from ref_cases import _bf16, _n, all_finite_bf16


def _log_uniform(g, shape, lo, hi):
    mag = np.exp(g.uniform(np.log(lo), np.log(hi), shape))
    return (mag * g.choice([-1.0, 1.0], shape)).astype(np.float32)


def cases():
    out = {}
    g = np.random.default_rng(4480)
    for tag, mode in (("mx", 1), ("fp4", 2)):
        # two row tiles of the scale layout (130 > 128), 12 scale columns
        out[f"{tag}_dense"] = dict(mode=mode, x=_bf16(_n(g, (130, 384), 1.7)), K=384)
        # row stride wider than K, scale columns padded (K / 32 = 5 -> 8, K / 16 = 10 -> 12)
        out[f"{tag}_strided"] = dict(mode=mode, x=_bf16(_n(g, (37, 168), 0.4, 0.2)), K=160)
        # magnitudes over 30 decades inside one block: most elements flush to zero codes
        out[f"{tag}_wide"] = dict(mode=mode, x=_bf16(_log_uniform(g, (33, 256), 1e-15, 1e15)), K=256)
        # post-activation look: a few outlier channels, many small values, exact zeros
        a = _n(g, (64, 512), 0.5)
        a[:, ::97] *= 40.0
        a[g.uniform(size=a.shape) < 0.2] = 0.0
        a[5] = 0.0
        out[f"{tag}_outliers"] = dict(mode=mode, x=_bf16(a), K=512)
    # every finite bf16 value, in bit order (blocks of near-equal magnitude) and shuffled
    allv = all_finite_bf16()
    assert allv.size == 65280
    out["mx_every_bf16"] = dict(mode=1, x=allv.reshape(255, 256).copy(), K=256)
    out["mx_every_bf16_shuffled"] = dict(mode=1, x=g.permutation(allv).reshape(255, 256).copy(), K=256)
    # a tensor of values up to the bf16 limit (scale exponent clamp) and one of zeros only
    out["mx_huge"] = dict(mode=1, x=_bf16(_log_uniform(g, (4, 64), 1e36, 3e38)), K=64)
    out["mx_tiny"] = dict(mode=1, x=_bf16(_log_uniform(g, (4, 64), 1e-40, 1e-37)), K=64)
    out["mx_zeros"] = dict(mode=1, x=np.zeros((3, 32), np.uint16), K=32)
    out["fp4_zeros"] = dict(mode=2, x=np.zeros((3, 32), np.uint16), K=32)
    # unit-range values: many products land exactly on the e2m1 rounding thresholds
    grid = (g.integers(-24, 25, (40, 128)) * 0.25).astype(np.float32)
    grid[0, 0] = 6.0
    out["fp4_grid"] = dict(mode=2, x=_bf16(grid), K=128)
    return out
