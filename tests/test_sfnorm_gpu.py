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


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("comb", ["mul", "add"])
def test_fused_backward_matches_oracle(dt, comb):
    """Gradients of the fused op (recomputed filter by ddf_b200_sfnorm, DDF backward, norm
    Jacobian by ddf_b200_sfnorm_backward) against the float64 oracle: the CPU oracle's DDF
    gradients on the float64-normalised filter, carried through a float64 autograd of the
    normalisation written out from its definition (ddf/ddf.py:146-152)."""
    from ddfnet_b200 import ddf_sfnorm
    from oracle import ddf_oracle
    dtype = DTYPES[dt]
    dev = torch.device("cuda:0")
    B, C, H = 4, 48, 14
    x, cf, raw = _inputs(B, C, H, H, 3, 1, dtype, 21)
    go = torch.randn(B, C, H, H, generator=torch.Generator().manual_seed(5)).to(dtype)
    a = [t.to(dev).requires_grad_() for t in (x, cf, raw)]
    ddf_sfnorm(a[0], a[1], a[2], 3, 1, 1, comb, SCALE).backward(go.to(dev))
    v = raw.double().requires_grad_()
    c = v - v.mean(dim=1, keepdim=True)
    normed = c / ((c * c).sum(dim=1, keepdim=True) / 8).sqrt().add(1e-10) * SCALE
    assert torch.allclose(normed.detach(), ddf_oracle.filter_norm_spatial(raw.double(), 1, 3, SCALE), atol=1e-12)
    gx, gcf, gsf = ddf_oracle.backward(go.double(), x.double(), cf.double(), normed.detach(), 3, 1, 1, comb)
    (graw,) = torch.autograd.grad(normed, v, gsf)
    # float32: the project's 1e-5 bound.  2-byte types: the backward stores the recomputed filter
    # and the filter gradient in the element type (as the unfused module sequence does), so the
    # aggregate bound is that type's rounding: relative L2 of 2**-9 (f16: 2**-11) times a small factor.
    for name, got, want in zip(("gx", "gcf", "graw"), (a[0].grad, a[1].grad, a[2].grad), (gx, gcf, graw)):
        if dtype == torch.float32:
            check_close(got, want, dtype, f"fused backward {name} {comb}", reduction=name != "gx")
        else:
            rel = ((got.double().cpu() - want).norm() / want.norm()).item()
            assert rel <= (6e-3 if dtype == torch.bfloat16 else 1e-3), (name, rel)


def test_sfnorm_kernels_float64():
    """ddf_b200_sfnorm / ddf_b200_sfnorm_backward in float64 against autograd, k = 3 and 5, including
    a pixel whose values are all equal (zero spread: the gradient of the spread term is dropped)."""
    from ddfnet_b200 import _lib
    L = _lib.load()
    dev = torch.device("cuda:0")
    for k in (3, 5):
        kk = k * k
        g = torch.Generator().manual_seed(k)
        raw = torch.randn(3, kk, 6, 5, generator=g, dtype=torch.float64)
        raw[0, :, 0, 0] = 0.25
        gy = torch.randn(3, kk, 6, 5, generator=g, dtype=torch.float64)
        rd, gd = raw.to(dev), gy.to(dev)
        out, gr = torch.empty_like(rd), torch.empty_like(rd)
        assert L.ddf_b200_sfnorm(rd.data_ptr(), out.data_ptr(), 3, k, 6, 5, _lib.F64, 0.4, None) == 0
        assert L.ddf_b200_sfnorm_backward(rd.data_ptr(), gd.data_ptr(), gr.data_ptr(), 3, k, 6, 5, _lib.F64, 0.4, None) == 0
        torch.cuda.synchronize()
        v = raw.clone().requires_grad_()
        c = v - v.mean(dim=1, keepdim=True)
        y = c / ((c * c).sum(dim=1, keepdim=True) / (kk - 1)).sqrt().add(1e-10) * 0.4
        mask = torch.ones(3, 1, 6, 5, dtype=torch.bool)
        mask[0, 0, 0, 0] = False
        (want,) = torch.autograd.grad(y, v, gy * mask)
        assert torch.allclose(out.cpu(), y.detach(), atol=1e-12)
        keep = mask.expand_as(want)
        assert torch.allclose(gr.cpu()[keep], want[keep], atol=1e-10)
        assert torch.isfinite(gr).all()
