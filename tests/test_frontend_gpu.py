"""ddf_b200_pack_frontend (one pass over a channels_last x: NCHW copy and pooled partial sums)
against plain torch arithmetic in float64 on the same rounded values."""
import pytest
import torch

from tests.util import DTYPES

pytestmark = pytest.mark.gpu

CASES = [  # B, C, H, W
    (2, 64, 56, 56), (2, 128, 28, 28), (3, 256, 14, 14), (2, 512, 7, 7), (1, 72, 10, 12), (2, 128, 56, 56),
]


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("case", CASES)
def test_frontend_matches_torch(case, dt):
    from ddfnet_b200.modules import pack_frontend
    B, C, H, W = case
    dtype = DTYPES[dt]
    dev = torch.device("cuda:0")
    torch.manual_seed(C + H)
    x = torch.randn(B, C, H, W, device=dev).to(dtype).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        got = pack_frontend(x)
    assert got is not None
    x_nchw, pooled = got
    assert x_nchw.is_contiguous() and torch.equal(x_nchw, x)
    xd = x.double().cpu()
    nt = (H * W + 63) // 64
    assert pooled.shape == (B, nt, C) and pooled.dtype == torch.float32
    want_sum = xd.sum(dim=(2, 3))
    got_sum = pooled.double().cpu().sum(dim=1)
    assert (got_sum - want_sum).abs().max().item() <= 1e-4 * max(1.0, want_sum.abs().max().item())


def test_pooled_sums_of_half_input():
    from ddfnet_b200.modules import pack_frontend
    dev = torch.device("cuda:0")
    x = torch.randn(3, 128, 28, 28, device=dev).half().contiguous(memory_format=torch.channels_last)
    x_nchw, pooled = pack_frontend(x)
    assert torch.equal(x_nchw, x)
    want = x.double().sum(dim=(2, 3))
    assert (pooled.double().sum(dim=1) - want).abs().max().item() <= 1e-3


def test_nchw_input_or_gradients_decline():
    from ddfnet_b200.modules import pack_frontend
    dev = torch.device("cuda:0")
    x = torch.randn(2, 32, 8, 8, device=dev)
    with torch.no_grad():
        assert pack_frontend(x) is None                            # contiguous NCHW: nothing to convert
    xcl = x.contiguous(memory_format=torch.channels_last).requires_grad_()
    assert pack_frontend(xcl) is None                              # gradients are being recorded


@pytest.mark.parametrize("cfg", [
    dict(in_channels=64, kernel_size=3, stride=1, head=1, kernel_combine="mul"),
    dict(in_channels=128, kernel_size=3, stride=2, head=1, kernel_combine="add"),
    dict(in_channels=64, kernel_size=3, stride=1, head=2, kernel_combine="mul"),
])
def test_ddfpack_channels_last_inference_equals_module_sequence(cfg, monkeypatch):
    """The whole fused inference route (front end, channel-branch kernel, op with fused
    FilterNorm) on a channels_last tensor against the reference's module sequence on NCHW."""
    from ddfnet_b200 import DDFPack
    monkeypatch.setattr(torch.backends.cudnn, "allow_tf32", False)
    monkeypatch.setattr(torch.backends.cuda.matmul, "allow_tf32", False)
    dev = torch.device("cuda:0")
    torch.manual_seed(4)
    m = DDFPack(**cfg).to(dev).eval()
    x = torch.randn(4, cfg["in_channels"], 28, 28, device=dev)
    with torch.no_grad():
        a = m(x.contiguous(memory_format=torch.channels_last))
        m.fuse_channel_branch = False
        m.fuse_filter_norm = False
        b = m(x)
    torch.testing.assert_close(a, b, rtol=1e-4, atol=2e-5)
