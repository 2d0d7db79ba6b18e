"""Cases of tests/golden/ref_builders.npz (shared by the generator and the tests)."""
import numpy as np

# QwenImageDit::prepare layouts: (T text rows incl. placeholders, H, W, [(slot0, h, w), ...])
QWEN_ROPE_FULL = [       # small: the whole table is stored
    (7, 4, 6, []),
    (0, 2, 2, []),
    (12, 6, 4, [(3, 4, 4)]),
    (20, 8, 8, [(0, 2, 4), (9, 4, 2)]),
]
QWEN_ROPE_DIGEST = [     # benchmark-sized: a SHA-256 of the bytes is stored
    (128, 32, 32, []),                      # BASELINE.json configs[0]
    (256, 64, 64, []),                      # configs[1]
    (512, 128, 128, []),                    # configs[3]
    (1600, 64, 48, [(14, 64, 64), (1100, 32, 48)]),   # an edit layout with two condition images
]

TIMESTEPS_FULL = [0.0, 1.0, 0.5, 0.001, 0.999, 0.25, 1e-6, 0.7071, 0.0314159, 0.96875, 0.123456, 0.875, 0.3333333, 0.0625,
                  0.9999999, 0.5019531]


def timesteps_digest():
    g = np.random.default_rng(77)
    return np.concatenate([np.arange(1001, dtype=np.float32) / np.float32(1000.0), g.random(1047, dtype=np.float32)])


def h3_basis_inputs():
    g = np.random.default_rng(78)
    table = g.standard_normal((1025, 8)).astype(np.float32)
    ts = np.concatenate([np.array([0.0, 1.0, 0.5, -0.25, 1.5, 1.0 / 1024, 1023.0 / 1024, 0.99999994, 1e-8], np.float32),
                         g.random(247, dtype=np.float32)])
    small = g.standard_normal((2, 3)).astype(np.float32)   # the smallest grid the formula allows
    return table, ts, small


def h3_inv_freq(n=16, theta=10000.0):
    # the checkpoint's inv_freq vector follows 1 / theta^(2k / 2n) (tools/ref/h3_dit_ref.py:101); any fp32 vector serves
    return (1.0 / np.power(np.float32(theta), np.arange(n, dtype=np.float32) * np.float32(2.0) / np.float32(2 * n))).astype(np.float32)


def h3_rope_positions():
    """(name, positions fp32 [S, 3]) built from the committed reference positions fixture."""
    from pathlib import Path
    z = np.load(Path(__file__).with_name("h3_positions.npz"))
    return [("case2", z["case2_pos"]), ("case1", z["case1_pos"]), ("case0", z["case0_pos"])]
