"""Seeded random sweep over the shapes the row kernel takes (square planes 7, 14, 28 or 56 wide,
stride 1 or 2, channel counts that are small multiples of its chunk, small batches): forward and
all three gradients against the float64 oracle."""
import random

import pytest
import torch

from tests.util import DTYPES, check_close, make_inputs, oracle_backward, oracle_forward

pytestmark = pytest.mark.gpu


def _cases(n, seed):
    rnd = random.Random(seed)
    out = []
    for it in range(n):
        ow = rnd.choice([7, 14, 28, 56])
        s = rnd.choice([1, 1, 2])
        dt = rnd.choice(["bf16", "f16", "f32"])
        if ow == 56 or dt == "f32":
            s = 1                      # stride 2 is built for outputs up to 28 wide, 2-byte types
        # threads per plane of the kernel's geometry -> planes it covers at once
        if dt == "f32":
            tpp = ow * (ow // 7)
        elif ow == 7:
            tpp = 7
        elif s == 1:
            tpp = ow * (ow // 14)
        else:
            tpp = ow * (ow // 7)
        cht = 448 // tpp
        c = cht * rnd.choice([1, 1, 2, 3, 5])
        if ow == 56 and c > 16:
            c = rnd.choice([2, 4, 6])
        out.append((rnd.choice([1, 2, 3, 5, 9]), c, ow * s, s, dt, rnd.choice(["mul", "add"]), 1000 + it))
    return out


@pytest.mark.parametrize("case", _cases(48, 7))
def test_forward_and_gradients(case):
    from ddfnet_b200 import _lib, ddf
    B, C, H, s, dt, mode, seed = case
    dtype = DTYPES[dt]
    dev = torch.device("cuda:0")
    x, cf, sf, go = make_inputs(B, C, H, H, 3, s, dtype, seed=seed)
    xs = [t.to(dev).requires_grad_() for t in (x, cf, sf)]
    out = ddf(*xs, 3, 1, s, mode, "f")
    check_close(out, oracle_forward(x, cf, sf, 3, 1, s, mode), dtype, f"forward {case}")
    out.backward(go.to(dev))
    gx, gcf, gsf = oracle_backward(go, x, cf, sf, 3, 1, s, mode)
    check_close(xs[0].grad, gx, dtype, f"grad-x {case}")
    check_close(xs[1].grad, gcf, dtype, f"grad-cf {case}", reduction=True)
    check_close(xs[2].grad, gsf, dtype, f"grad-sf {case}", reduction=True)
    assert _lib.load().ddf_b200_take_fault() == 0
