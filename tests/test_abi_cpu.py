"""CPU-side checks of the C ABI: the library loads, exports every symbol the
header declares, and rejects bad arguments with the documented status codes
before touching a device (no compute calls here)."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from ddfnet_b200.csrc import build
    build.build()
    from ddfnet_b200 import _lib
    return _lib.load()


def _declared_symbols():
    with open(os.path.join(ROOT, "include", "ddf_b200.h")) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ddf_b200_\w+)\s*\(", text)))


def test_header_symbols_exported(L):
    from ddfnet_b200 import _lib
    declared = _declared_symbols()
    assert declared, "no declarations found in include/ddf_b200.h"
    assert sorted(_lib.SYMBOLS) == declared
    for name in declared:
        assert getattr(L, name) is not None


def test_header_cites_reference():
    with open(os.path.join(ROOT, "include", "ddf_b200.h")) as f:
        text = f.read()
    for cite in ("ddf/src/ddf_mul_ext.cpp:21-34", "ddf/src/ddf_mul_ext.cpp:36-55",
                 "ddf/src/cuda/ddf_mul_cuda_kernel.cu:423-527"):
        assert cite in text


def test_version_and_strerror(L):
    assert L.ddf_b200_version() >= 100
    assert L.ddf_b200_strerror(0) == b"success"
    for code in range(-10, 0):
        assert L.ddf_b200_strerror(code).startswith(b"ddf_b200:")


def test_argument_checks(L):
    fwd = lambda *a: L.ddf_b200_forward(None, None, None, None, *a, None)
    # B, C, H, W, k, d, s, combine, dtype, variant
    assert fwd(0, 4, 8, 8, 3, 1, 1, 0, 0, 0) == -2
    assert fwd(1, 4, 8, 8, 4, 1, 1, 0, 0, 0) == -3   # even kernel (ddf/ddf.py:63)
    assert fwd(1, 4, 8, 8, 3, 0, 1, 0, 0, 0) == -3
    assert fwd(1, 4, 8, 8, 3, 1, 0, 0, 0, 0) == -3
    assert fwd(1, 4, 1, 8, 3, 1, 2, 0, 0, 0) == -2   # H/s == 0
    assert fwd(1, 4, 8, 8, 3, 1, 1, 2, 0, 0) == -4
    assert fwd(1, 4, 8, 8, 3, 1, 1, 0, 9, 0) == -5
    assert fwd(1, 4, 8, 8, 3, 1, 1, 0, 0, 5) == -6
    assert fwd(1, 4, 8, 8, 3, 1, 1, 0, 0, 0) == -1   # NULL pointers
    assert L.ddf_b200_backward(None, None, None, None, None, None, None, None, 0,
                               1, 4, 8, 8, 3, 1, 1, 0, 0, 0, None) == -1
    assert L.ddf_b200_backward_workspace(1, 4, 8, 8, 4, 1, 1, 0, 0, 0) == 0


def test_argument_checks_of_the_adjacent_entry_points(L):
    """Fused FilterNorm forward, layout adapters, front end, channel branch: every refusal
    below happens before a device is touched (pointers are NULL or never dereferenced)."""
    import ctypes
    fake = ctypes.c_void_p(4096)   # non-NULL, 16-byte aligned, never dereferenced on these paths
    # fused FilterNorm: k*k must exceed 1
    assert L.ddf_b200_forward_sfnorm(fake, fake, fake, fake, 1, 4, 8, 8, 1, 1, 1, 0, 0, 0, 1.0, None) == -3
    assert L.ddf_b200_forward_sfnorm(None, None, None, None, 1, 4, 8, 8, 3, 1, 1, 0, 0, 0, 1.0, None) == -1
    # layout adapters
    assert L.ddf_b200_nhwc_to_nchw(None, None, 1, 4, 8, 8, 0, None) == -1
    assert L.ddf_b200_nhwc_to_nchw(fake, fake, 0, 4, 8, 8, 0, None) == -2
    assert L.ddf_b200_nhwc_to_nchw(fake, fake, 1, 4, 8, 8, 3, None) == -5          # float64 not built
    assert L.ddf_b200_nchw_to_nhwc(fake, fake, 1, 4, 8, 8, 0, fake, None, 0, None) == -1   # scale without shift
    assert L.ddf_b200_nhwc_to_nchw_affine(fake, fake, 1, 9, 8, 8, 4, 0, None, None, 0, None) == -2  # source narrower
    assert L.ddf_b200_nhwc_to_nchw(ctypes.c_void_p(4098), fake, 1, 4, 8, 8, 1, None) == -7  # misaligned
    # front end
    assert L.ddf_b200_frontend_tiles(56, 56) == 49 and L.ddf_b200_frontend_tiles(7, 7) == 1
    assert L.ddf_b200_pack_frontend(None, None, None, 1, 4, 8, 8, 0, None) == -1
    assert L.ddf_b200_pack_frontend(fake, fake, fake, 1, 0, 8, 8, 0, None) == -2
    assert L.ddf_b200_pack_frontend(fake, fake, fake, 1, 4096, 8, 8, 0, None) == -7
    assert L.ddf_b200_pack_frontend(fake, fake, fake, 1, 4, 8, 8, 3, None) == -5
    # channel branch
    cf = lambda *a: L.ddf_b200_channel_filter(fake, 1, 1.0, fake, fake, fake, fake, fake, fake, *a, None)
    assert L.ddf_b200_channel_filter(None, 1, 1.0, fake, fake, fake, fake, fake, fake, 1, 64, 12, 3, 0, None) == -1
    assert cf(0, 64, 12, 3, 0) == -2
    assert cf(1, 64, 12, 7, 0) == -7       # k = 3 or 5 only
    assert cf(1, 4096, 12, 3, 0) == -7     # C <= 2048
    assert cf(1, 20, 4, 3, 0) == -7        # C a multiple of 8
    assert cf(1, 300, 60, 3, 0) == -7      # above 256: a multiple of the 256-channel slice
    assert cf(1, 64, 1000, 3, 0) == -7     # mid <= 512
    assert L.ddf_b200_channel_filter_slice(64) == 64 and L.ddf_b200_channel_filter_slice(1024) == 256


def test_plan_prefers_streaming_at_benchmark_shapes(L):
    from ddfnet_b200 import _lib
    for C, H, s in [(64, 56, 1), (128, 28, 1), (256, 14, 1), (512, 7, 1), (128, 56, 2), (256, 28, 2), (512, 14, 2)]:
        assert L.ddf_b200_plan(128, C, H, H, 3, 1, s, 0, _lib.BF16, 0) == _lib.VARIANT_STREAM
    assert L.ddf_b200_plan(2, 3, 9, 11, 7, 1, 1, 0, _lib.F32, 0) == _lib.VARIANT_GENERIC
    assert L.ddf_b200_plan(128, 64, 56, 56, 3, 1, 1, 0, _lib.F64, 0) == _lib.VARIANT_GENERIC


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import ddfnet_b200._lib as lib
    monkeypatch.setenv("DDF_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(lib, "_lib", None)
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        lib.load()
