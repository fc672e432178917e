"""Backward parity on the GPU: all three input gradients from the CUDA kernels
(through autograd and the C ABI) against the float64 CPU oracle."""
import pytest
import torch

from tests.util import DTYPES, check_close, make_inputs, oracle_backward

pytestmark = pytest.mark.gpu


def _grads(x, cf, sf, go, k, d, s, m, version=""):
    from ddfnet_b200 import ddf
    dev = torch.device("cuda:0")
    xd, cfd, sfd = (t.to(dev).requires_grad_() for t in (x, cf, sf))
    out = ddf(xd, cfd, sfd, k, d, s, m, version)
    out.backward(go.to(dev))
    return xd.grad, cfd.grad, sfd.grad


def _check(shape, dt, version, seed):
    B, C, H, W, k, d, s = shape
    dtype = DTYPES[dt]
    x, cf, sf, go = make_inputs(B, C, H, W, k, s, dtype, seed)
    for m in ("mul", "add"):
        got = _grads(x, cf, sf, go, k, d, s, m, version)
        want = oracle_backward(go, x, cf, sf, k, d, s, m)
        for name, g, w in zip(("grad_x", "grad_cf", "grad_sf"), got, want):
            assert g.dtype == dtype
            check_close(g, w, dtype, f"{name} {shape} {dt} {m} '{version}'", reduction=name != "grad_x")
    from ddfnet_b200 import _lib
    assert _lib.load().ddf_b200_take_fault() == 0


GENERIC = []
for k, d in [(1, 1), (3, 1), (3, 2), (5, 1), (5, 2), (7, 1)]:
    for s in (1, 2):
        GENERIC.append((2, 3, 9, 11, k, d, s))
GENERIC += [(1, 70, 10, 10, 3, 1, 1), (35, 1, 10, 10, 3, 2, 2), (1, 1, 50, 50, 3, 1, 1),
            (1, 70, 10, 10, 5, 1, 2), (20, 1, 10, 10, 5, 2, 1), (1, 1, 40, 40, 5, 1, 1),
            (2, 5, 13, 9, 3, 1, 2), (1, 2, 4, 30, 3, 1, 3),
            # even planes at k=3, d=1, s=2: the dedicated stride-2 grad-x kernel
            (2, 5, 12, 10, 3, 1, 2), (1, 20, 6, 8, 3, 1, 2), (3, 17, 14, 14, 3, 1, 2), (1, 3, 2, 2, 3, 1, 2)]


@pytest.mark.parametrize("shape", GENERIC)
@pytest.mark.parametrize("dt", ["f32", "f64", "f16", "bf16"])
def test_generic_backward(shape, dt):
    _check(shape, dt, "o", seed=300 + shape[4] + shape[5] + shape[6])


STREAM = [
    (3, 64, 28, 28, 3, 1, 1),
    (4, 16, 56, 56, 3, 1, 1),
    (8, 32, 14, 14, 3, 1, 1),
    (8, 64, 7, 7, 3, 1, 1),
    (40, 8, 7, 7, 3, 1, 1),
    (3, 32, 28, 28, 3, 2, 1),
    (3, 32, 28, 28, 5, 1, 1),
    (3, 32, 28, 28, 5, 2, 1),
    (3, 32, 56, 56, 3, 1, 2),
    (3, 32, 28, 28, 3, 1, 2),
    (2, 24, 20, 24, 3, 1, 1),
    (300, 8, 28, 28, 3, 1, 1),   # grad-x in the row kernel: a new sample every chunk, filter buffers reused
    (400, 64, 7, 7, 3, 1, 1),
    (40, 6, 56, 56, 3, 1, 1),
]


@pytest.mark.parametrize("shape", STREAM)
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_stream_backward(shape, dt):
    """version '' here: every gradient takes the streaming kernel where one
    exists for the shape and the generic kernel otherwise."""
    from ddfnet_b200 import ddf
    B, C, H, W, k, d, s = shape
    dtype = DTYPES[dt]
    x, cf, sf, go = make_inputs(B, C, H, W, k, s, dtype, 400 + H + k + d + s)
    dev = torch.device("cuda:0")
    from ddfnet_b200 import _lib
    L = _lib.load()
    for m in ("mul", "add"):
        want = oracle_backward(go, x, cf, sf, k, d, s, m)
        xd, cfd, sfd, god = (t.to(dev) for t in (x, cf, sf, go))
        gx, gcf, gsf = torch.empty_like(xd), torch.empty_like(cfd), torch.empty_like(sfd)
        comb = {"mul": 0, "add": 1}[m]
        dtc = {"f32": 0, "f16": 1, "bf16": 2}[dt]
        # STREAM where it exists, per gradient group; fall back to AUTO otherwise
        ws_bytes = int(L.ddf_b200_backward_workspace(B, C, H, W, k, d, s, comb, dtc, _lib.VARIANT_STREAM))
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        rc = L.ddf_b200_backward(god.data_ptr(), xd.data_ptr(), cfd.data_ptr(), sfd.data_ptr(),
                                 gx.data_ptr(), gcf.data_ptr(), gsf.data_ptr(), ws.data_ptr(), ws_bytes,
                                 B, C, H, W, k, d, s, comb, dtc, _lib.VARIANT_STREAM,
                                 torch.cuda.current_stream().cuda_stream)
        if rc == -7:  # some gradient has no streaming kernel for this shape: mixed path
            gx, gcf, gsf = _grads(x, cf, sf, go, k, d, s, m, "")
        else:
            assert rc == 0, L.ddf_b200_strerror(rc)
        for name, g, w in zip(("grad_x", "grad_cf", "grad_sf"), (gx, gcf, gsf), want):
            check_close(g, w, dtype, f"{name} {shape} {dt} {m}", reduction=name != "grad_x")
    assert L.ddf_b200_take_fault() == 0


@pytest.mark.parametrize("k", [3, 5])
@pytest.mark.parametrize("d", [1, 2])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_config3_full_size(k, d, dt):
    # forward + backward, B=64, C=256, 28x28, stride 1, both modes
    _check((64, 256, 28, 28, k, d, 1), dt, "", seed=3000 + k + d)


def test_partial_gradients():
    from ddfnet_b200 import ddf
    dev = torch.device("cuda:0")
    x, cf, sf, go = make_inputs(2, 8, 12, 12, 3, 1, torch.float32, 77)
    want = oracle_backward(go, x, cf, sf, 3, 1, 1, "mul")
    for need in [(True, False, False), (False, True, False), (False, False, True), (True, False, True)]:
        ts = [t.to(dev).requires_grad_(n) for t, n in zip((x, cf, sf), need)]
        ddf(*ts, 3, 1, 1, "mul").backward(go.to(dev))
        for t, n, w in zip(ts, need, want):
            if n:
                check_close(t.grad, w, torch.float32, f"partial {need}")
            else:
                assert t.grad is None


GRADCHECK = [(1, 7, 6, 6, 3), (5, 1, 6, 6, 3), (1, 1, 12, 12, 3), (1, 7, 6, 6, 5), (4, 1, 6, 6, 5),
             (1, 1, 10, 10, 5)]


@pytest.mark.parametrize("shape", GRADCHECK)
@pytest.mark.parametrize("s", [1, 2])
@pytest.mark.parametrize("m", ["mul", "add"])
def test_gradcheck_float64(shape, s, m):
    """The reference's own test protocol (grad_check.py:139-299): float64
    gradcheck with eps 1e-3, atol 1e-5, dilation 1 and 2."""
    from ddfnet_b200 import ddf
    B, C, H, W, k = shape
    dev = torch.device("cuda:0")
    for d in (1, 2):
        g = torch.Generator().manual_seed(5)
        x = torch.randn(B, C, H, W, generator=g, dtype=torch.float64).to(dev).requires_grad_()
        cf = torch.randn(B, C, k, k, generator=g, dtype=torch.float64).to(dev).requires_grad_()
        sf = torch.randn(B, k * k, H // s, W // s, generator=g, dtype=torch.float64).to(dev).requires_grad_()
        assert torch.autograd.gradcheck(lambda a, b, c: ddf(a, b, c, k, d, s, m), (x, cf, sf),
                                        eps=1e-3, atol=1e-5)
