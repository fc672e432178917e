"""The backward entry point that allocates nothing (ddf_b200_backward_noalloc).

It serves hosts that may not call cudaMalloc on this path (a runtime with a
fixed device arena, a plugin running where allocation is forbidden): the
scratch of the filter-gradient kernel is a fixed array inside the library
instead of a caller-provided workspace.  Here it is called through the C ABI,
twice in a row (the array is shared and keeps the previous call's contents),
and must reproduce the regular entry point's gradients; a problem whose scratch
need exceeds the built-in array must be refused.

Collected last on purpose, so that a run that stops at the first failure has
already run every other test.
"""
import pytest
import torch

from tests.util import check_close, make_inputs, oracle_backward

pytestmark = pytest.mark.gpu


def _call(L, fn_noalloc, tensors, shape, comb, dtc, lib):
    go, x, cf, sf = tensors
    B, C, H, W, k, d, s = shape
    gx, gcf, gsf = torch.empty_like(x), torch.empty_like(cf), torch.empty_like(sf)
    stream = torch.cuda.current_stream().cuda_stream
    if fn_noalloc:
        rc = L.ddf_b200_backward_noalloc(go.data_ptr(), x.data_ptr(), cf.data_ptr(), sf.data_ptr(),
                                         gx.data_ptr(), gcf.data_ptr(), gsf.data_ptr(),
                                         B, C, H, W, k, d, s, comb, dtc, stream)
    else:
        ws_bytes = int(L.ddf_b200_backward_workspace(B, C, H, W, k, d, s, comb, dtc, lib.VARIANT_AUTO))
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
        rc = L.ddf_b200_backward(go.data_ptr(), x.data_ptr(), cf.data_ptr(), sf.data_ptr(),
                                 gx.data_ptr(), gcf.data_ptr(), gsf.data_ptr(), ws.data_ptr(), ws_bytes,
                                 B, C, H, W, k, d, s, comb, dtc, lib.VARIANT_AUTO, stream)
    assert rc == 0, L.ddf_b200_strerror(rc)
    torch.cuda.synchronize()
    return gx, gcf, gsf


@pytest.mark.parametrize("dt,dtc", [("f32", 0), ("bf16", 2)])
@pytest.mark.parametrize("mode,comb", [("mul", 0), ("add", 1)])
def test_noalloc_backward_matches_regular_entry_point(dt, dtc, mode, comb):
    from ddfnet_b200 import _lib
    from tests.util import DTYPES
    L = _lib.load()
    dev = torch.device("cuda:0")
    dtype = DTYPES[dt]
    # big enough that AUTO takes the streaming kernels (the ones that use scratch)
    shapes = [(32, 128, 28, 28, 3, 1, 1), (64, 256, 14, 14, 3, 1, 1)]
    for shape in shapes:
        B, C, H, W, k, d, s = shape
        assert L.ddf_b200_plan(B, C, H, W, k, d, s, comb, dtc, 1) == _lib.VARIANT_STREAM
        need = int(L.ddf_b200_backward_workspace(B, C, H, W, k, d, s, comb, dtc, _lib.VARIANT_AUTO))
        assert 0 < need <= int(L.ddf_b200_backward_noalloc_limit())
        x, cf, sf, go = make_inputs(B, C, H, W, k, s, dtype, seed=900 + H)
        tensors = tuple(t.to(dev) for t in (go, x, cf, sf))
        want = _call(L, False, tensors, shape, comb, dtc, _lib)
        oracle = oracle_backward(go, x, cf, sf, k, d, s, mode)
        for attempt in range(2):          # two calls in a row share the built-in scratch
            got = _call(L, True, tensors, shape, comb, dtc, _lib)
            for name, g, w, o in zip(("grad_x", "grad_cf", "grad_sf"), got, want, oracle):
                assert torch.equal(g, w), f"{name} differs from ddf_b200_backward (call {attempt})"
                check_close(g, o, dtype, f"noalloc {name} {shape} {dt} {mode}", reduction=name != "grad_x")
    assert L.ddf_b200_take_fault() == 0


def test_noalloc_small_problems_and_single_gradients():
    """Small problems, where both entry points choose the generic kernels, and calls that ask
    for one gradient only (the limit and the scratch concern the spatial-filter gradient
    alone): still bit-identical to ddf_b200_backward."""
    from ddfnet_b200 import _lib
    L = _lib.load()
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    shape = (2, 6, 9, 11, 3, 1, 1)
    B, C, H, W, k, d, s = shape
    assert L.ddf_b200_plan(B, C, H, W, k, d, s, 0, 0, 1) == _lib.VARIANT_GENERIC
    x, cf, sf, go = make_inputs(B, C, H, W, k, s, torch.float32, seed=41)
    tensors = tuple(t.to(dev) for t in (go, x, cf, sf))
    want = _call(L, False, tensors, shape, 0, 0, _lib)
    for attempt in range(2):
        got = _call(L, True, tensors, shape, 0, 0, _lib)
        for name, g, w in zip(("grad_x", "grad_cf", "grad_sf"), got, want):
            assert torch.equal(g, w), f"{name} differs from ddf_b200_backward on a small problem"
    # grad_cf only, on a problem whose grad_sf scratch would exceed the built-in array
    big = (128, 64, 28, 28, 5, 1, 1)
    B, C, H, W, k, d, s = big
    x, cf, sf, go = (t.to(dev) for t in make_inputs(B, C, H, W, k, s, torch.float32, seed=6))
    gcf_a, gcf_b = torch.empty_like(cf), torch.empty_like(cf)
    rc = L.ddf_b200_backward_noalloc(go.data_ptr(), x.data_ptr(), cf.data_ptr(), sf.data_ptr(), None,
                                     gcf_a.data_ptr(), None, B, C, H, W, k, d, s, 0, 0, stream)
    assert rc == 0, L.ddf_b200_strerror(rc)
    rc = L.ddf_b200_backward(go.data_ptr(), x.data_ptr(), cf.data_ptr(), sf.data_ptr(), None, gcf_b.data_ptr(),
                             None, None, 0, B, C, H, W, k, d, s, 0, 0, _lib.VARIANT_AUTO, stream)
    assert rc == 0, L.ddf_b200_strerror(rc)      # no workspace needed without grad_sf
    torch.cuda.synchronize()
    assert torch.equal(gcf_a, gcf_b)
    assert L.ddf_b200_take_fault() == 0


def test_noalloc_refuses_problems_beyond_its_scratch():
    from ddfnet_b200 import _lib
    L = _lib.load()
    dev = torch.device("cuda:0")
    shape = (128, 64, 28, 28, 5, 1, 1)   # k = 5, 128 samples: needs more than the built-in 16 MiB
    B, C, H, W, k, d, s = shape
    need = int(L.ddf_b200_backward_workspace(B, C, H, W, k, d, s, 0, 0, _lib.VARIANT_AUTO))
    assert need > int(L.ddf_b200_backward_noalloc_limit())
    x, cf, sf, go = (t.to(dev) for t in make_inputs(B, C, H, W, k, s, torch.float32, seed=5))
    gx, gcf, gsf = torch.empty_like(x), torch.empty_like(cf), torch.empty_like(sf)
    rc = L.ddf_b200_backward_noalloc(go.data_ptr(), x.data_ptr(), cf.data_ptr(), sf.data_ptr(),
                                     gx.data_ptr(), gcf.data_ptr(), gsf.data_ptr(),
                                     B, C, H, W, k, d, s, 0, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -11
    assert b"16 MiB" in L.ddf_b200_strerror(rc)
    torch.cuda.synchronize()
