"""Shared helpers for the parity tests: seeded inputs, the oracle call, and the
tolerance rule.

Tolerances (stated by the project's target):
  float64  : 1e-10 absolute/relative (the reference's own forward check,
             grad_check.py:44, uses 1e-10)
  float32  : max abs/rel error <= 1e-5.  For the two gradients that are long
             sums (grad_cf over H'W' pixels, grad_sf over C channels; pass
             reduction=True) the absolute part scales with the tensor's RMS: the
             rounding error of a float32 sum follows the size of its summands and
             partial sums, not of a result that may have cancelled to near zero.
  float16  : <= 2e-3 relative (a correctly rounded float16 is within 4.9e-4)
  bfloat16 : <= 2e-3 relative *on top of the final rounding to bfloat16*: a
             correctly rounded bfloat16 value is itself up to 2**-8 = 3.9e-3
             away from the exact one (1.6e-3 .. 2.3e-3 in the RMS), so a bare
             2e-3 bound against the exact value cannot be met by any
             implementation.  In exchange every element must lie within one
             bfloat16 ulp of the oracle result rounded to bfloat16 (plus the
             same 2e-3 relative slack for long float32 sums).
  Both 2-byte types are also held, in the aggregate, to a relative L2 distance
  of 2e-3 from the oracle result rounded to the storage type.
"""
from __future__ import annotations

import torch

from oracle import ddf_oracle

DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "f64": torch.float64}


def make_inputs(B, C, H, W, k, s, dtype, seed, with_go=True):
    """x ~ relu(N(0,1)), cf, sf ~ N(0,1/9), go ~ N(0,1); generated on the CPU in
    float32 from a seeded generator, rounded to `dtype`.  Returns CPU tensors of
    `dtype` (feed `.double()` of them to the oracle: same values)."""
    g = torch.Generator().manual_seed(seed)
    OH, OW = H // s, W // s
    x = torch.randn(B, C, H, W, generator=g).relu_()
    cf = torch.randn(B, C, k, k, generator=g) / 3
    sf = torch.randn(B, k * k, OH, OW, generator=g) / 3
    out = [x.to(dtype), cf.to(dtype), sf.to(dtype)]
    if with_go:
        out.append(torch.randn(B, C, OH, OW, generator=g).to(dtype))
    return out


def oracle_forward(x, cf, sf, k, d, s, combine):
    return ddf_oracle.forward(x.double(), cf.double(), sf.double(), k, d, s, combine)


def oracle_backward(go, x, cf, sf, k, d, s, combine):
    return ddf_oracle.backward(go.double(), x.double(), cf.double(), sf.double(), k, d, s, combine)


def check_close(actual, expected64, dtype, what="", reduction=False):
    """actual: tensor of `dtype` (any device); expected64: CPU float64 oracle result."""
    a = actual.detach().to("cpu", torch.float64)
    b = expected64
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    assert torch.isfinite(a).all(), f"{what}: non-finite values"
    err = (a - b).abs()
    if dtype == torch.float64:
        bound = 1e-10 * b.abs().clamp_min(1.0)
    elif dtype == torch.float32:
        floor = max(1.0, b.pow(2).mean().sqrt().item()) if reduction else 1.0
        bound = 1e-5 * b.abs().clamp_min(floor)
    elif dtype == torch.float16:
        bound = 2e-3 * b.abs() + 1e-5
    else:  # bfloat16
        bound = (2e-3 + 2.0 ** -8) * b.abs() + 1e-5
    bad = err > bound
    if bad.any():
        i = torch.nonzero(bad)[0].tolist()
        worst = (err / bound).max().item()
        raise AssertionError(
            f"{what}: {int(bad.sum())} of {b.numel()} elements out of tolerance; first at {i}: "
            f"got {a[tuple(i)].item()!r} want {b[tuple(i)].item()!r}; worst err/bound {worst:.3g}")
    if dtype == torch.bfloat16:
        # element-wise: within one bfloat16 ulp of the correctly rounded oracle value
        b_r = b.to(dtype).to(torch.float64)
        ulp = torch.pow(2.0, torch.floor(torch.log2(b_r.abs().clamp_min(2.0 ** -126))) - 7)
        off = (a - b_r).abs()
        lim = ulp + 2e-3 * b.abs() + 1e-5
        if (off > lim).any():
            i = torch.nonzero(off > lim)[0].tolist()
            raise AssertionError(f"{what}: {int((off > lim).sum())} elements more than one bfloat16 ulp from the "
                                 f"rounded oracle; first at {i}: got {a[tuple(i)].item()!r} want {b_r[tuple(i)].item()!r}")
    if dtype in (torch.float16, torch.bfloat16):
        b_rounded = b.to(dtype).to(torch.float64)
        rel_l2 = ((a - b_rounded).pow(2).sum() / b.pow(2).sum().clamp_min(1e-30)).sqrt().item()
        assert rel_l2 <= 2e-3, f"{what}: relative L2 distance {rel_l2:.3e} > 2e-3"
