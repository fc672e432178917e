"""Our CUDA op against the reference project's OWN CUDA op on identical seeded inputs.

oracle/build_ref.py compiles the reference's extension modules, unmodified, for sm_100a
into oracle/_ref/ (done where the reference sources are present; the built modules travel
with the repository snapshot).  oracle/ref_op.py calls them the way the reference's Python
wrapper does.  Tolerances: float32 max abs/rel 1e-5 (gradients that are long sums: absolute
part scaled by the tensor's RMS, as in tests/util.py), float64 1e-10.
Shapes: benchmark configuration 1, configuration 3 (k 3/5 x d 1/2 x mul/add, at a reduced
batch so that the reference's backward stays within seconds) and the four stride-1 stage
shapes of the reference's own consistency check (grad_check.py:77-135).
"""
import pytest
import torch

from tests.util import make_inputs

pytestmark = pytest.mark.gpu


def _ref():
    from oracle import ref_op
    if not ref_op.available():
        pytest.skip("oracle/_ref is not built: the reference sources were not present when "
                    "__graft_entry__.build() ran (python oracle/build_ref.py builds it)")
    return ref_op


def _close(got, want, dtype, what, reduction=False):
    a, b = got.double().cpu(), want.double().cpu()
    assert a.shape == b.shape, what
    if dtype == torch.float64:
        bound = 1e-10 * b.abs().clamp_min(1.0)
    else:
        floor = max(1.0, b.pow(2).mean().sqrt().item()) if reduction else 1.0
        bound = 1e-5 * b.abs().clamp_min(floor)
    err = (a - b).abs()
    assert (err <= bound).all(), f"{what}: max err/bound {(err / bound).max().item():.3g}"


CASES = [(2, 64, 56, 3, 1, "mul")]                                    # configuration 1
CASES += [(4, 256, 28, k, d, m) for k in (3, 5) for d in (1, 2) for m in ("mul", "add")]   # configuration 3
CASES += [(6, 64, 56, 3, 1, "mul"), (6, 128, 28, 3, 1, "mul"), (6, 256, 14, 3, 1, "mul"), (6, 512, 7, 3, 1, "mul")]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dt", [torch.float32, torch.float64])
def test_forward_and_gradients_match_the_reference_cuda_op(case, dt):
    from ddfnet_b200 import ddf
    ref = _ref()
    B, C, H, k, d, mode = case
    dev = torch.device("cuda:0")
    x, cf, sf, go = (t.to(dev) for t in make_inputs(B, C, H, H, k, 1, dt, seed=4000 + C + k + d))
    xs = [t.detach().clone().requires_grad_() for t in (x, cf, sf)]
    out = ddf(*xs, k, d, 1, mode)
    out.backward(go)
    want = ref.forward(x, cf, sf, k, d, 1, mode)
    _close(out.detach(), want, dt, f"forward {case}")
    gx, gcf, gsf = ref.backward(go, x, cf, sf, k, d, 1, mode)
    _close(xs[0].grad, gx, dt, f"grad_x {case}")
    _close(xs[1].grad, gcf, dt, f"grad_cf {case}", reduction=True)
    _close(xs[2].grad, gsf, dt, f"grad_sf {case}", reduction=True)
