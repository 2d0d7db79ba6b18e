"""Which kernel family a norm call takes is decided by pure host arithmetic on pointer values and
sizes (mxk_norm_path_probe).  These checks run without a GPU on made-up addresses, which nothing
dereferences: a row the bulk-copy kernel would fetch with cp.async.bulk must start on a 16-byte
boundary, whatever the element type, because callers pass offset pointers (the reference's callers
hand the launchers views such as `x + s0*D`, src/models/minimax_h3/dit_sp.cpp:91,153-163, out of
a 256-byte aligned arena, src/core/tensor.cpp:122-129)."""
import itertools

import pytest

GENERIC, VECTOR, BULK = 0, 1, 2
LN, RMS, RMS_BF16, RES_LN, RES_RMS, RES_LN_Q, RES_RMS_Q = range(7)
BASE = 0x7F0000000000  # a 256-byte aligned made-up device address


@pytest.fixture(scope="module")
def L():
    from miroxen_b200 import _lib, build
    if not _lib.lib_path().exists():
        build.build()
    return _lib


def probe(L, op, x=BASE, y=BASE + (1 << 30), out=BASE + (2 << 30), w=None, rows=64, dim=3072,
          scale=None, shift=None, gate=None):
    none = L.RowMod(None, None, 0)
    return L.lib().mxk_norm_path_probe(op, x, y, out, w, scale or none, shift or none, gate or none, rows, dim)


def test_aligned_model_shapes_take_the_bulk_copy_kernel(L):
    for dim in (1152, 3072, 4096, 5120, 5376):
        for op in (LN, RMS, RMS_BF16, RES_LN, RES_RMS, RES_LN_Q, RES_RMS_Q):
            assert probe(L, op, dim=dim) == BULK, (op, dim)


def test_bf16_input_offset_by_four_elements_leaves_the_bulk_copy_kernel(L):
    # 4 bf16 elements = 8 bytes: fine for the 64-bit loads of the register kernel, not for a bulk copy
    assert probe(L, RMS_BF16, x=BASE + 8) == VECTOR
    assert probe(L, RMS_BF16, x=BASE + 16) == BULK
    assert probe(L, RMS_BF16, x=BASE + 2) == GENERIC
    assert probe(L, RMS_BF16, x=BASE + 4) == GENERIC


def test_residual_row_offset_by_four_elements_leaves_the_bulk_copy_kernel(L):
    y0 = BASE + (1 << 30)
    for op in (RES_LN, RES_RMS):
        assert probe(L, op, y=y0 + 8) == VECTOR
        assert probe(L, op, y=y0 + 16) == BULK
        assert probe(L, op, y=y0 + 2) == GENERIC
    # the one-pass MXFP8 forms exist for the bulk-copy kernel only: they refuse instead
    for op in (RES_LN_Q, RES_RMS_Q):
        assert probe(L, op, y=y0 + 8) == -1
        assert probe(L, op, y=y0 + 16) == BULK
        assert probe(L, op, x=BASE + 4) == -1


def test_fp32_input_needs_sixteen_bytes_for_either_vector_kernel(L):
    for off, want in ((4, GENERIC), (8, GENERIC), (12, GENERIC), (16, BULK), (256, BULK)):
        assert probe(L, LN, x=BASE + off) == want, off
        assert probe(L, RMS, x=BASE + off) == want, off


def test_row_pitch_must_be_a_multiple_of_sixteen_bytes(L):
    # dim % 4 == 0 but dim % 8 != 0: fp32 rows still start on 16 bytes, bf16 rows only every second row
    assert probe(L, LN, dim=3076) == BULK
    assert probe(L, RMS_BF16, dim=3076) == VECTOR
    assert probe(L, RES_LN, dim=3076) == VECTOR
    assert probe(L, LN, dim=3074) == GENERIC
    assert probe(L, RMS_BF16, dim=3073) == GENERIC


def test_no_combination_reaches_the_bulk_copy_kernel_with_a_misaligned_row(L):
    y0 = BASE + (1 << 30)
    for op, xoff, yoff, dim in itertools.product(range(7), (0, 2, 4, 8, 12, 16, 24, 32), (0, 2, 4, 8, 16, 24),
                                                 (64, 100, 1152, 3072, 3076, 3080)):
        got = probe(L, op, x=BASE + xoff, y=y0 + yoff, dim=dim)
        if got != BULK:
            continue
        esz = 2 if op == RMS_BF16 else 4
        assert xoff % 16 == 0 and (dim * esz) % 16 == 0, (op, xoff, yoff, dim)
        if op >= RES_LN:
            assert yoff % 16 == 0 and (dim * 2) % 16 == 0, (op, xoff, yoff, dim)


def test_single_rows_and_unaligned_vectors(L):
    assert probe(L, LN, rows=1) == VECTOR
    assert probe(L, LN, w=BASE + (3 << 30)) == BULK  # op 0 ignores w (layernorm_mod has no affine weight)
    assert probe(L, RMS, w=BASE + (3 << 30) + 4) == GENERIC
    sc = L.RowMod(BASE + (3 << 30) + 8, None, 0)
    assert probe(L, LN, scale=sc) == GENERIC
    assert probe(L, LN, out=BASE + (2 << 30) + 4) == GENERIC
    assert probe(L, LN, out=BASE + (2 << 30) + 8) == BULK
    assert probe(L, LN, rows=0) == -1
