"""libmxk's latent layout kernels through the C ABI: bit-exact against the CPU oracle on the inputs of the
reference's own tests and at pipeline sizes, and - where oracle/_ref/libmx_ref_latent.so travelled with the
tree - against the reference's kernels run on the same device buffers."""
import ctypes as C

import numpy as np
import pytest

from oracle import binding as orc
from test_cpu_latent import h3_inputs, qwen_inputs

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mx():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import miroxen_b200 as m
    m.lib()
    return m


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def same_bits(t, want):
    return np.array_equal(t.cpu().numpy().view(np.uint32).ravel(), np.ascontiguousarray(want).view(np.uint32).ravel())


# 3772 = a 736 x 1312 image / 256, 16384 = 2048 x 2048 / 256 (tests/qwen_latent_test.cpp:106-107)
@pytest.mark.parametrize("n", [1, 31, 37, 1031, 3772, 16384])
def test_qwen_latent_encode_decode_bits(mx, n):
    x, mean, std = qwen_inputs(n, n)
    xd, md, sd = dev(x), dev(mean), dev(std)
    y = torch.full((n, 64), float("nan"), device="cuda")
    mx.ops.qwen_latent_encode(xd, y, n, md, sd)
    enc = orc.qwen_latent_encode(x, mean, std)
    assert same_bits(y, enc)
    z = torch.full((64, n), float("nan"), device="cuda")
    mx.ops.qwen_latent_decode(y, z, n, md, sd)
    assert same_bits(z, orc.qwen_latent_decode(enc, mean, std))
    if orc.have_ref_latent():
        L = orc.ref_latent()
        P, I64 = C.c_void_p, C.c_int64
        L.ref_qwen_latent_encode.argtypes = L.ref_qwen_latent_decode.argtypes = [P, P, I64, P, P, P]
        ry, rz = torch.empty_like(y), torch.empty_like(z)
        assert L.ref_qwen_latent_encode(xd.data_ptr(), ry.data_ptr(), n, md.data_ptr(), sd.data_ptr(), None) == 0
        assert L.ref_qwen_latent_decode(ry.data_ptr(), rz.data_ptr(), n, md.data_ptr(), sd.data_ptr(), None) == 0
        torch.cuda.synchronize()
        assert torch.equal(ry.view(torch.int32), y.view(torch.int32)) and torch.equal(rz.view(torch.int32), z.view(torch.int32))


# (72, 80, 46, 405) is the reference benchmark's size (tests/h3_latent_test.cpp:73)
@pytest.mark.parametrize("F,H,W,A", [(2, 6, 10, 37), (1, 2, 2, 1), (3, 4, 66, 70), (5, 8, 130, 33), (72, 80, 46, 405)])
def test_h3_latent_video_audio_bits(mx, F, H, W, A):
    rows, audio = h3_inputs(F, H, W, A)
    rd, ad = dev(rows), dev(audio)
    z = torch.full((24, F, H, W), float("nan"), device="cuda")
    za = torch.full((2, 32, A), float("nan"), device="cuda")
    mx.ops.h3_latent_video(rd, z, F, H, W)
    mx.ops.h3_latent_audio(ad, za, A)
    assert same_bits(z, orc.h3_latent_video(rows, F, H, W))
    assert same_bits(za, orc.h3_latent_audio(audio, A))
    if orc.have_ref_latent():
        L = orc.ref_latent()
        P, I64 = C.c_void_p, C.c_int64
        L.ref_h3_latent_video.argtypes = [P, P, I64, I64, I64, P]
        L.ref_h3_latent_audio.argtypes = [P, P, I64, P]
        rz, rza = torch.empty_like(z), torch.empty_like(za)
        assert L.ref_h3_latent_video(rd.data_ptr(), rz.data_ptr(), F, H, W, None) == 0
        assert L.ref_h3_latent_audio(ad.data_ptr(), rza.data_ptr(), A, None) == 0
        torch.cuda.synchronize()
        assert torch.equal(rz, z) and torch.equal(rza, za)


def test_latent_argument_errors(mx):
    """The reference rejects these (tests/h3_latent_test.cpp:69-71; src/kernels/qwen_latent.cu:43)."""
    t = torch.zeros(64 * 4, device="cuda")
    with pytest.raises(mx.MxkError):
        mx.ops.h3_latent_video(None, None, 1, 3, 2)
    with pytest.raises(mx.MxkError):
        mx.ops.h3_latent_video(t, t, 1, 3, 2)
    with pytest.raises(mx.MxkError):
        mx.ops.h3_latent_audio(t, t, 0)
    with pytest.raises(mx.MxkError):
        mx.ops.qwen_latent_encode(t, t, 0, t, t)
    with pytest.raises(mx.MxkError):
        mx.ops.qwen_latent_decode(t, t, 4, None, t)
