"""ddf_b200_channel_filter (the channel branch after its average pool, one kernel) against
the oracle: the two 1x1 convolutions restated as float64 matrix products followed by the
FilterNorm restatement that tests/golden/filternorm_channel_*.pt pin to the reference module."""
import pytest
import torch

from oracle import ddf_oracle as O
from tests.util import DTYPES

pytestmark = pytest.mark.gpu


def _expected(pooled, w1, b1, w2, b2, gain, c, k):
    g = pooled.double()
    h = torch.relu(g @ w1.double().t() + b1.double())
    r = h @ w2.double().t() + b2.double()
    return O.filter_norm_channel(r, c, k, gain.double()).reshape(-1, c, k, k)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("cfg", [(8, 64, 3), (5, 128, 3), (16, 512, 3), (3, 24, 3), (6, 96, 5), (1, 768, 3), (7, 256, 5)])
def test_channel_filter_matches_oracle(cfg, dt):
    from ddfnet_b200 import DDFPack
    from ddfnet_b200.modules import channel_filter_fused
    B, C, k = cfg
    dtype = DTYPES[dt]
    dev = torch.device("cuda:0")
    torch.manual_seed(B * 1000 + C)
    m = DDFPack(C, kernel_size=k).to(dev).to(dtype).eval()
    x = torch.randn(B, C, 14, 14, device=dev).relu_().to(dtype)
    with torch.no_grad():
        got = channel_filter_fused(m.channel_branch, x, k)
    assert got is not None and got.shape == (B, C, k, k) and got.dtype == dtype
    br = m.channel_branch
    pooled = x.float().mean(dim=(2, 3)).cpu()
    want = _expected(pooled, br[1].weight.detach().cpu().reshape(-1, C), br[1].bias.detach().cpu(),
                     br[3].weight.detach().cpu().reshape(C * k * k, -1), br[3].bias.detach().cpu(),
                     br[4].std.detach().cpu(), C, k)
    err = (got.cpu().double() - want).abs()
    tol = {"f32": 2e-5, "f16": 2e-3, "bf16": 1e-2}[dt]   # final rounding of the stored type included
    bound = tol * want.abs() + tol * want.abs().max()
    assert (err <= bound).all(), (err / bound).max().item()


def test_fused_branch_equals_module_sequence_in_ddfpack(monkeypatch):
    from ddfnet_b200 import DDFPack
    dev = torch.device("cuda:0")
    torch.manual_seed(2)
    # the module sequence's float32 convolutions would otherwise run in TF32
    monkeypatch.setattr(torch.backends.cudnn, "allow_tf32", False)
    monkeypatch.setattr(torch.backends.cuda.matmul, "allow_tf32", False)
    for head in (1, 4):
        m = DDFPack(64, kernel_size=3, head=head).to(dev).eval()
        x = torch.randn(6, 64, 28, 28, device=dev)
        with torch.no_grad():
            m.fuse_channel_branch = True
            a = m(x)
            m.fuse_channel_branch = False
            b = m(x)
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)


def test_gradients_fall_back_to_the_module_sequence():
    from ddfnet_b200 import DDFPack
    from ddfnet_b200.modules import channel_filter_fused
    m = DDFPack(32, kernel_size=3).to("cuda:0")
    x = torch.randn(2, 32, 14, 14, device="cuda:0")
    assert channel_filter_fused(m.channel_branch, x, 3) is None  # parameters require grad
    m(x).sum().backward()
    assert m.channel_branch[3].weight.grad is not None


def test_unsupported_channel_counts_use_the_module_sequence():
    from ddfnet_b200 import DDFPack
    from ddfnet_b200.modules import channel_filter_fused
    for C in (20, 300):  # not a multiple of 8 / of the 256-channel slice
        m = DDFPack(C).to("cuda:0").eval()
        x = torch.randn(2, C, 7, 7, device="cuda:0")
        with torch.no_grad():
            assert channel_filter_fused(m.channel_branch, x, 3) is None
            assert m(x).shape == x.shape


def test_out_of_range_is_refused():
    from ddfnet_b200 import _lib
    L = _lib.load()
    t = torch.zeros(64, device="cuda:0")
    p = t.data_ptr()
    assert L.ddf_b200_channel_filter(p, 1, 1.0, p, p, p, p, p, p, 1, 4096, 8, 3, 0, None) == -7
    assert L.ddf_b200_channel_filter(p, 1, 1.0, p, p, p, p, p, p, 1, 16, 8, 7, 0, None) == -7
    assert L.ddf_b200_channel_filter(p, 1, 1.0, p, p, p, p, p, p, 1, 20, 8, 3, 0, None) == -7
    assert L.ddf_b200_channel_filter_slice(64) == 64 and L.ddf_b200_channel_filter_slice(512) == 256
