"""mxk_dit_block_ops_host_static - the host-buffer block runner for callers that must not allocate
device memory (an engine that sized its arena once at start-up, a plugin inside a process that
forbids cudaMalloc on its threads).  Its staging is a fixed array inside the library instead of the
buffers mxk_host_pipeline_create allocates.

Checked here, through the C ABI: on the same inputs it returns exactly what mxk_dit_block_ops_host
returns, on two calls in a row (the second call finds the first call's bytes in the shared array),
for a block whose rows span several staging chunks; and a block too wide for the array is refused
with MXK_ERR_TOO_LARGE.  The file name makes pytest collect it last.
"""
import numpy as np
import pytest

import helpers as H

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mx():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import miroxen_b200 as m
    m.lib()
    return m


def host_bits(t):
    return t.view(torch.uint16).numpy().copy() if t.dtype == torch.bfloat16 else t.numpy().copy()


CASES = [
    # rows, dim, H, D, F, norm_mode, act_mode, rot, rope_mode, packed, n_prefix
    (1000, 3072, 24, 128, 12288, 0, 0, 128, 1, False, 700),  # about 2.6 chunks of the 32 MiB array
    (300, 5120, 40, 128, 13824, 1, 1, 128, 2, True, 0),
]


@pytest.mark.parametrize("cfg", CASES)
def test_static_staging_matches_allocating_pipeline(mx, cfg):
    from test_gpu_tables_chain import make_block
    rows = cfg[0]
    outs = ("h1", "q_out", "k_out", "h2", "act", "x") + (("v_out",) if cfg[9] else ())
    # reference: the allocating pipeline
    _, tr, ar = make_block(mx, H.rng(rows), *cfg, host=True)
    pipe = mx.HostPipeline(128, cfg[1], cfg[4], cfg[2], cfg[3], cfg[7], with_v=cfg[9], act_mode=cfg[6])
    up_ref, down_ref = pipe.run(ar)
    pipe.close()
    want = {k: host_bits(tr[k]) for k in outs}
    assert mx.lib().mxk_static_stage_bytes() == 32 << 20
    for call in range(2):  # the second call runs over what the first left in the array
        _, ts, a = make_block(mx, H.rng(rows), *cfg, host=True)
        up, down = mx.dit_block_ops_host_static(a)
        assert (up, down) == (up_ref, down_ref)
        for k in outs:
            assert np.array_equal(host_bits(ts[k]), want[k]), f"call {call}: {k} differs from mxk_dit_block_ops_host"
    torch.cuda.synchronize()
    assert mx.device_error() == 0


def test_static_staging_rejects_a_block_that_does_not_fit(mx):
    from test_gpu_tables_chain import make_block
    # 64 rows of a block this wide need more than 32 MiB of staging
    cfg = (8, 8192, 64, 128, 200000, 0, 0, 128, 1, False, 0)
    _, t, a = make_block(mx, H.rng(1), *cfg, host=True)
    rc = mx.lib().mxk_dit_block_ops_host_static(a, None, None, None)
    assert rc == -3
    msg = mx.lib().mxk_last_error().decode()
    assert "static" in msg and "fit" in msg
