"""The CPU oracle's latent layout functions against the formulas and inputs of the reference's own tests
(tests/qwen_latent_test.cpp:17-46: uniform values in [-4, 4], scales in [0.25, 4], N = 37 and 1031;
tests/h3_latent_test.cpp:11-36: the deterministic ramps, F, H, W, A = 2, 6, 10, 37)."""
import numpy as np
import pytest

from oracle import binding as orc


def qwen_inputs(n, seed):
    g = np.random.default_rng(seed)
    mean = g.uniform(-4, 4, 64).astype(np.float32)
    std = g.uniform(0.25, 4, 64).astype(np.float32)
    x = g.uniform(-4, 4, (64, n)).astype(np.float32)
    return x, mean, std


def h3_inputs(F, H, W, A):
    """The ramps of tests/h3_latent_test.cpp:15-16, without its 288-float offset."""
    nv, na = 24 * F * H * W, 64 * A
    rows = ((np.arange(288, 288 + nv) % 10007 - 5003) / 16).astype(np.float32)
    audio = ((np.arange(288, 288 + na) % 1009 - 503) / 8).astype(np.float32)
    return rows, audio


@pytest.mark.parametrize("n", [1, 37, 1031])
def test_qwen_latent_matches_two_step_float_arithmetic(n):
    x, mean, std = qwen_inputs(n, n)
    enc = orc.qwen_latent_encode(x, mean, std)
    want = ((x - mean[:, None]).astype(np.float32) / std[:, None]).astype(np.float32).T
    assert np.array_equal(enc.view(np.uint32), np.ascontiguousarray(want).view(np.uint32))
    dec = orc.qwen_latent_decode(enc, mean, std)
    want = ((enc * std[None, :]).astype(np.float32) + mean[None, :]).astype(np.float32).T
    assert np.array_equal(dec.view(np.uint32), np.ascontiguousarray(want).view(np.uint32))
    # decode(encode(x)) is x up to the two roundings each way
    assert np.abs(dec - x).max() <= 4e-6 * 16


@pytest.mark.parametrize("F,H,W,A", [(2, 6, 10, 37), (1, 2, 2, 1), (3, 4, 66, 70)])
def test_h3_latent_is_the_patch_and_channel_permutation(F, H, W, A):
    rows, audio = h3_inputs(F, H, W, A)
    z = orc.h3_latent_video(rows, F, H, W)
    want = rows.reshape(F, H // 2, W // 2, 24, 2, 2).transpose(3, 0, 1, 4, 2, 5).reshape(24, F, H, W)
    assert np.array_equal(z, want)
    za = orc.h3_latent_audio(audio, A)
    assert np.array_equal(za, audio.reshape(2, A, 32).transpose(0, 2, 1))
