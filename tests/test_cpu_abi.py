"""CPU-side checks of the drop-in boundary: the library loads, exports every symbol the header
declares, and rejects bad arguments with a status and a message before touching a GPU."""
import ctypes as C
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def L():
    from miroxen_b200 import _lib, build
    if not _lib.lib_path().exists():
        build.build()
    return _lib


def test_library_exports_every_declared_symbol(L):
    lib = L.lib()
    names = L.header_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mxk.h but not exported"
    assert set(names) == set(L.PROTOTYPES), set(names) ^ set(L.PROTOTYPES)
    assert lib.mxk_version() >= 100


def test_struct_layouts_match_header(L):
    # RowMod must have the reference's layout: two pointers and an int64.
    assert C.sizeof(L.RowMod) == 24
    assert C.sizeof(L.HeadTensor) == 48
    assert C.sizeof(L.RopeRun) == 72


def test_missing_library_fails_loudly(tmp_path):
    code = ("import miroxen_b200._lib as l, pathlib; l.lib_path = lambda: pathlib.Path('%s/nope.so');\n"
            "import sys\n"
            "try:\n    l.lib()\nexcept l.MxkError as e:\n    print('RAISED', e); sys.exit(0)\nsys.exit(1)") % tmp_path
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert r.returncode == 0 and "RAISED" in r.stdout, r.stdout + r.stderr


def test_argument_validation_returns_status(L):
    lib = L.lib()
    none = L.RowMod(None, None, 0)
    # the reference's own head_norm_rope check: D even, <= 256, rot even and <= D
    for D, rot in ((7, 4), (258, 2), (128, 130), (128, 3)):
        rc = lib.mxk_head_norm_rope(1, 4, 1024, 0, 8, D, None, 1e-6, 1, 1, rot, 1, 1, None)
        assert rc == -1 and b"head_norm_rope" in lib.mxk_last_error()
    assert lib.mxk_head_norm_rope(1, 4, 1024, 0, 8, 128, None, 1e-6, 1, 1, 128, 9, 1, None) == -1
    assert lib.mxk_head_norm_rope(1, 4, 1024, 0, 8, 128, None, 1e-6, None, None, 128, 1, 1, None) == -1  # rope without tables
    assert lib.mxk_layernorm_mod(None, 4, 3072, 1e-6, none, none, None, None) == -1
    assert lib.mxk_layernorm_mod(1, 4, 0, 1e-6, none, none, 1, None) == -1
    bad = L.RowMod(1, None, 5)  # prefix rows without a prefix vector
    assert lib.mxk_rmsnorm_mod(1, 4, 64, 1e-6, None, bad, none, 1, None) == -1
    assert lib.mxk_gated_residual(None, None, 3, 64, none, 0, None) == -1
    assert lib.mxk_gated_residual_norm(1, 1, 3, 64, none, 0, 2, 1e-6, None, none, none, 1, None) == -1
    assert lib.mxk_qkv_norm_rope(None, 4, 3, 8, 128, 1e-6, None, None, None) == -1
    assert lib.mxk_set_tuning(b"no_such_knob", 1) == -1
    assert b"no_such_knob" in lib.mxk_last_error()
    assert lib.mxk_dit_block_ops(None, None) == -1


def test_zero_and_negative_sizes_are_silent_noops(L):
    lib = L.lib()
    none = L.RowMod(None, None, 0)
    assert lib.mxk_layernorm_mod(None, 0, 3072, 1e-6, none, none, None, None) == 0
    assert lib.mxk_rmsnorm_mod(None, -3, 3072, 1e-6, None, none, none, None, None) == 0
    assert lib.mxk_rmsnorm_bf16(None, 0, 3072, 1e-6, None, None, None) == 0
    assert lib.mxk_gated_residual(None, None, 0, 3072, none, 1, None) == 0
    assert lib.mxk_head_norm_rope(None, 0, 0, 0, 24, 128, None, 0.0, None, None, 128, 1, None, None) == 0
    assert lib.mxk_silu_mul(None, 0, 12288, None, None) == 0
    for f in (lib.mxk_gelu_tanh_inplace, lib.mxk_gelu_erf_inplace, lib.mxk_silu_inplace_f32):
        assert f(None, 0, None) == 0
    assert lib.mxk_axpy_f32(None, None, 1.0, 0, None) == 0
    assert lib.mxk_scatter_rows(None, 64, None, None, 0, 0, None) == 0


def test_host_builders_match_oracle(L):
    """The host-side builders are plain libm code and run without a GPU."""
    import numpy as np
    from oracle import binding as orc
    lib = L.lib()
    for t in (0.0, 0.5, 0.25, 0.999, 1.0, 0.3337):
        out = np.empty((2, 256), np.float32)
        assert lib.mxk_qwen_timestep_embedding_host(t, out.ctypes.data) == 0
        assert np.array_equal(out.view(np.uint32), orc.qwen_timestep_embedding(t).view(np.uint32))
    axes = (C.c_int32 * 3)(16, 56, 56)
    invf = np.empty(64, np.float32)
    assert lib.mxk_msrope_inv_freq_host(axes, 3, 10000.0, invf.ctypes.data) == 0
    assert invf[0] == 1.0 and invf[8] == 1.0 and invf[36] == 1.0 and 0 < invf[63] < invf[62]
    ft = np.empty(21, np.float32)
    assert lib.mxk_h3_frame_times_host(512, 21, ft.ctypes.data) == 0
    pos = orc.h3_positions(512, 21, 60, 104, 0, [])
    assert np.array_equal(ft, pos[512::30 * 52, 0])
    hg = np.empty(30, np.float32)
    assert lib.mxk_h3_spatial_grid_host(60, 60, 104, hg.ctypes.data) == 0
    assert np.array_equal(hg, pos[512:512 + 30 * 52:52, 1])


def test_cpp_shim_compiles_and_links(tmp_path, L):
    """include/mx_ops.h and include/mx_latent.h (the reference's namespace mx signatures over the C ABI) build with g++ against
    libmxk and reports a bad argument as std::runtime_error, like the reference's MX_CHECK."""
    import shutil
    if not shutil.which("g++") or not Path("/usr/local/cuda/include/cuda_runtime.h").exists():
        pytest.skip("no g++ / CUDA headers")
    src = tmp_path / "shim.cpp"
    src.write_text(r'''
#include <cstdio>
#include <cstring>
#include "mx_ops.h"
#include "mx_latent.h"
int main() {
  try {  // the reference's own negative test (tests/h3_latent_test.cpp:69-71)
    mx::h3_latent::video(nullptr, nullptr, 1, 3, 2, nullptr);
    return 3;
  } catch (const std::runtime_error& e) {
    if (!std::strstr(e.what(), "h3_latent_video")) return 4;
  }
  try {
    mx::qwen_latent::encode(nullptr, nullptr, 0, nullptr, nullptr, nullptr);
    return 5;
  } catch (const std::runtime_error&) {
  }
  mx::layernorm_mod(nullptr, 0, 3072, 1e-6f, mx::RowMod{}, mx::RowMod{}, nullptr, nullptr);   // rows == 0: no-op
  mx::gated_residual(nullptr, nullptr, -1, 3072, mx::RowMod{}, 1, nullptr);
  try {
    mx::head_norm_rope((const mx::bf16*)16, 4, 1024, 0, 8, 7, nullptr, 1e-6f, nullptr, nullptr, 4, mx::ROPE_HALF,
                       (mx::bf16*)16, nullptr);
  } catch (const std::runtime_error& e) {
    std::printf("THROWN %s\n", e.what());
    return std::strstr(e.what(), "head_norm_rope") ? 0 : 2;
  }
  return 1;
}
''')
    exe = tmp_path / "shim"
    lib = L.lib_path()
    r = subprocess.run(["g++", "-std=c++17", str(src), "-I", str(ROOT / "include"), "-I", "/usr/local/cuda/include",
                        "-L", str(lib.parent), "-lmxk", f"-Wl,-rpath,{lib.parent}", "-o", str(exe)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "THROWN" in r.stdout, r.stdout + r.stderr
