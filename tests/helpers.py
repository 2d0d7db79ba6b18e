"""Shared test helpers: seeded inputs, bf16 comparison, guarded device buffers."""
from __future__ import annotations

import numpy as np

from oracle import binding as orc

# Acceptance for bf16 outputs against the fp32 oracle: every element is within one bf16 unit in
# the last place of the oracle's bf16 value, or - for values near zero, where cancellation makes
# the last place meaningless - within 2^-8 * max(|ref|, 2^-6) absolutely.
BF16_REL = 2.0 ** -8
BF16_FLOOR = 2.0 ** -6
# fp32 outputs (residual stream, axpy): |err| <= 2^-20 * max(|ref|, 1).  The operands are O(1), so a
# result that cancels to a small value still carries rounding noise of a few fp32 ulps of 1.
F32_REL = 2.0 ** -20


def rng(seed):
    return np.random.default_rng(seed)


def normal_f32(g, shape, std=1.0, mean=0.0):
    return (g.standard_normal(shape, dtype=np.float32) * np.float32(std) + np.float32(mean)).astype(np.float32)


def normal_bf16(g, shape, std=1.0):
    return orc.f32_to_bf16_bits(normal_f32(g, shape, std))


def ordered(bits):
    b = bits.astype(np.int32)
    mag = b & 0x7FFF
    return np.where(b & 0x8000, -mag, mag)


def bf16_report(got_bits, ref_bits):
    got_bits = np.asarray(got_bits).reshape(-1)
    ref_bits = np.asarray(ref_bits).reshape(-1)
    ulp = np.abs(ordered(got_bits) - ordered(ref_bits))
    got, ref = orc.bf16_bits_to_f32(got_bits), orc.bf16_bits_to_f32(ref_bits)
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    tol = BF16_REL * np.maximum(np.abs(ref.astype(np.float64)), BF16_FLOOR)
    bad = (ulp > 1) & (err > tol)
    bad |= ~np.isfinite(got) & np.isfinite(ref)
    return dict(n=got.size, bad=int(bad.sum()), max_ulp=int(ulp.max()) if ulp.size else 0,
                mismatch=float((ulp > 0).mean()) if ulp.size else 0.0,
                worst=int(np.argmax(np.where(bad, err, 0))) if bad.any() else -1)


def assert_bf16_close(got_bits, ref_bits, what=""):
    r = bf16_report(got_bits, ref_bits)
    assert r["bad"] == 0, f"{what}: {r}"
    return r


def assert_f32_close(got, ref, what="", rel=F32_REL, floor=1.0):
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    err = np.abs(got - ref)
    tol = rel * np.maximum(np.abs(ref), floor)
    bad = err > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {got.size} beyond tolerance, worst err {err.max():.3e}"


GUARD = 64  # elements of guard band on each side


class Guarded:
    """A device tensor with poisoned guard bands before and after the payload."""

    def __init__(self, torch, shape, dtype, fill=None):
        import math
        n = int(math.prod(shape)) if len(shape) else 1
        self.torch = torch
        self.full = torch.empty(n + 2 * GUARD, dtype=dtype, device="cuda")
        self.raw = self.full.view(torch.uint8)
        self.raw.fill_(0xA5)
        self.t = self.full[GUARD:GUARD + n].view(shape)
        self.nbytes = self.full.element_size() * GUARD
        if fill is not None:
            self.t.copy_(fill)

    def check(self, what=""):
        a = self.raw[:self.nbytes]
        b = self.raw[-self.nbytes:]
        assert bool((a == 0xA5).all()) and bool((b == 0xA5).all()), f"{what}: guard band overwritten"


def to_dev(torch, a):
    """numpy -> CUDA tensor; uint16 arrays become bfloat16 tensors with the same bits."""
    t = torch.from_numpy(np.ascontiguousarray(a))
    if a.dtype == np.uint16:
        t = t.view(torch.bfloat16)
    return t.cuda()


def bits(t):
    """CUDA bf16 tensor -> numpy uint16 bit patterns."""
    import torch
    return t.detach().contiguous().view(torch.uint16).cpu().numpy()
