"""ddf_b200_forward_sfnorm / ddf_sfnorm (spatial FilterNorm fused into the forward kernel)
against the oracle: FilterNorm restated in float64 (pinned to the reference's module by
tests/golden/filternorm_*.pt) followed by the oracle's DDF forward."""
import glob
import os

import pytest
import torch

from oracle import ddf_oracle as O
from tests.util import DTYPES, check_close

pytestmark = pytest.mark.gpu

SCALE = 2.0 ** 0.5 / 3  # calculate_gain('relu') / k for k = 3


def _inputs(B, C, H, W, k, s, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, C, H, W, generator=g).relu_().to(dtype)
    cf = (torch.randn(B, C, k, k, generator=g) / 3).to(dtype)
    raw = (torch.randn(B, k * k, H // s, W // s, generator=g) * 1.3 + 0.4).to(dtype)  # conv output: not centred
    return x, cf, raw


def _expected(x, cf, raw, k, d, s, comb, scale):
    sfn = O.filter_norm_spatial(raw.double(), 1, k, scale)
    return O.forward(x.double(), cf.double(), sfn, k, d, s, comb)


CASES = [
    # B, C, H, k, d, s, version     (streaming kernel paths: P = 8, 4x2 planes, 7, 7 at stride 2, 2; generic)
    (8, 64, 56, 3, 1, 1, "f"),
    (8, 128, 28, 3, 1, 1, "f"),
    (16, 256, 14, 3, 1, 1, "f"),
    (16, 512, 7, 3, 1, 1, "f"),
    (8, 128, 56, 3, 1, 2, "f"),
    (8, 256, 28, 3, 1, 2, "f"),
    (8, 64, 28, 3, 2, 1, "f"),
    (8, 64, 28, 5, 1, 1, "f"),
    (8, 32, 12, 3, 1, 1, "f"),
    (2, 6, 13, 3, 1, 1, "o"),
    (2, 5, 12, 5, 2, 2, "o"),
    (3, 7, 9, 3, 1, 1, ""),
]


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("comb", ["mul", "add"])
@pytest.mark.parametrize("case", CASES)
def test_fused_forward_matches_oracle(case, comb, dt):
    from ddfnet_b200 import ddf_sfnorm
    B, C, H, k, d, s, ver = case
    dtype = DTYPES[dt]
    scale = 2.0 ** 0.5 / k
    x, cf, raw = _inputs(B, C, H, H, k, s, dtype, 77 + C + H)
    dev = torch.device("cuda:0")
    out = ddf_sfnorm(x.to(dev), cf.to(dev), raw.to(dev), k, d, s, comb, scale, ver)
    assert out.dtype == dtype
    check_close(out, _expected(x, cf, raw, k, d, s, comb, scale), dtype, f"fused fwd {case} {comb} {dt}")


def test_fused_forward_float64_generic():
    from ddfnet_b200 import ddf_sfnorm
    x, cf, raw = _inputs(2, 5, 11, 10, 3, 1, torch.float64, 5)
    dev = torch.device("cuda:0")
    out = ddf_sfnorm(x.to(dev), cf.to(dev), raw.to(dev), 3, 1, 1, "mul", SCALE)
    check_close(out, _expected(x, cf, raw, 3, 1, 1, "mul", SCALE), torch.float64, "fused fwd f64")


def test_fused_equals_unfused_on_reference_module_output():
    """The kernel's normalisation against the reference FilterNorm's own output (golden)."""
    from ddfnet_b200 import ddf, ddf_sfnorm
    f = torch.load(os.path.join(os.path.dirname(__file__), "golden", "filternorm_spatial_k3_h1_relu.pt"))
    raw, sfn, k = f["raw"], f["out"], f["k"]
    B, _, H, W = raw.shape
    g = torch.Generator().manual_seed(1)
    x = torch.randn(B, 6, H, W, generator=g, dtype=torch.float64)
    cf = torch.randn(B, 6, k, k, generator=g, dtype=torch.float64)
    dev = torch.device("cuda:0")
    for comb in ("mul", "add"):
        fused = ddf_sfnorm(x.to(dev), cf.to(dev), raw.to(dev), k, 1, 1, comb, f["scale"])
        plain = ddf(x.to(dev), cf.to(dev), sfn.to(dev), k, 1, 1, comb)
        assert (fused - plain).abs().max().item() <= 1e-10


def test_fused_rejects_k1():
    from ddfnet_b200 import _lib
    L = _lib.load()
    t = torch.zeros(64, device="cuda:0")
    rc = L.ddf_b200_forward_sfnorm(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                   1, 1, 4, 4, 1, 1, 1, 0, 0, 0, 1.0, None)
    assert rc == -3


@pytest.mark.parametrize("comb", ["mul", "add"])
def test_fused_gradcheck_float64(comb):
    """The reference's gradcheck protocol (grad_check.py:139-299: float64, eps 1e-3, atol 1e-5)
    through the fused function, raw spatial filter included."""
    from ddfnet_b200 import ddf_sfnorm
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(11)
    x = torch.randn(1, 3, 6, 6, generator=g, dtype=torch.float64).to(dev).requires_grad_()
    cf = torch.randn(1, 3, 3, 3, generator=g, dtype=torch.float64).to(dev).requires_grad_()
    raw = torch.randn(1, 9, 6, 6, generator=g, dtype=torch.float64).to(dev).requires_grad_()
    assert torch.autograd.gradcheck(lambda a, b, c: ddf_sfnorm(a, b, c, 3, 1, 1, comb, SCALE),
                                    (x, cf, raw), eps=1e-3, atol=1e-5)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_fused_backward_matches_unfused_chain(dt):
    """Gradients of the fused op against autograd through torch FilterNorm ops + the plain op."""
    from ddfnet_b200 import ddf, ddf_sfnorm
    from ddfnet_b200.op import spatial_filter_norm
    dtype = DTYPES[dt]
    dev = torch.device("cuda:0")
    x, cf, raw = (t.to(dev) for t in _inputs(8, 128, 28, 28, 3, 1, dtype, 21))
    go = torch.randn(8, 128, 28, 28, device=dev).to(dtype)
    a = [t.clone().requires_grad_() for t in (x, cf, raw)]
    ddf_sfnorm(a[0], a[1], a[2], 3, 1, 1, "mul", SCALE).backward(go)
    b = [t.clone().requires_grad_() for t in (x, cf, raw)]
    ddf(b[0], b[1], spatial_filter_norm(b[2], 3, SCALE).to(dtype), 3, 1, 1, "mul").backward(go)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    for name, p, q in zip(("gx", "gcf", "graw"), a, b):
        num = (p.grad.double() - q.grad.double()).norm().item()
        den = q.grad.double().norm().item()
        assert num <= tol * den, (name, num / den)
