"""ddf_b200_nhwc_to_nchw / ddf_b200_nchw_to_nhwc (layout adapters around the NCHW op) against
torch's own permutes: moving data must be bit-exact; the optional affine + ReLU is compared
with the same arithmetic in float32."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(2, 64, 56, 56), (3, 128, 28, 28), (2, 256, 14, 14), (2, 512, 7, 7), (1, 5, 7, 7),
          (2, 9, 28, 28), (1, 70, 9, 11), (2, 3, 224, 224)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_round_trip_is_exact(shape, dtype):
    from ddfnet_b200.layout import to_channels_last, to_nchw
    dev = torch.device("cuda:0")
    x = torch.randn(*shape, device=dev).to(dtype)
    cl = to_channels_last(x)
    assert cl.is_contiguous(memory_format=torch.channels_last) and cl.shape == x.shape
    assert torch.equal(cl, x)                       # same logical values
    assert torch.equal(cl.permute(0, 2, 3, 1).contiguous(), x.permute(0, 2, 3, 1).contiguous())
    back = to_nchw(x.contiguous(memory_format=torch.channels_last))
    assert back.is_contiguous() and torch.equal(back, x)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 64, 28, 28), (1, 70, 9, 11), (2, 512, 7, 7)])
def test_affine_relu_on_the_way(shape, dtype):
    from ddfnet_b200.layout import to_channels_last
    dev = torch.device("cuda:0")
    x = torch.randn(*shape, device=dev).to(dtype)
    scale = torch.randn(shape[1], device=dev)
    shift = torch.randn(shape[1], device=dev)
    got = to_channels_last(x, scale, shift, relu=True)
    want = torch.relu(torch.addcmul(shift.reshape(1, -1, 1, 1), x.float(), scale.reshape(1, -1, 1, 1))).to(dtype)
    assert got.is_contiguous(memory_format=torch.channels_last)
    # fmaf in the kernel against torch's float32 ops: allow one rounding step of the type
    torch.testing.assert_close(got.float(), want.float(), rtol=2 ** -7 if dtype != torch.float32 else 1e-6,
                               atol=1e-6)
    got2 = to_channels_last(x, relu=True)
    assert torch.equal(got2, torch.relu(x))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_nhwc_to_nchw_takes_leading_channels_and_adds_a_shift(dtype):
    from ddfnet_b200.layout import to_nchw_affine
    dev = torch.device("cuda:0")
    for (B, SC, C, H, W) in ((2, 16, 9, 28, 28), (3, 32, 18, 7, 7), (1, 16, 16, 10, 6)):
        x = torch.randn(B, SC, H, W, device=dev).to(dtype).contiguous(memory_format=torch.channels_last)
        shift = torch.randn(C, device=dev)
        ones = torch.ones(C, device=dev)
        got = to_nchw_affine(x, C, ones, shift)
        want = (x[:, :C].float() + shift.reshape(1, -1, 1, 1)).to(dtype)
        assert got.is_contiguous() and got.shape == (B, C, H, W)
        torch.testing.assert_close(got.float(), want.float(), rtol=2 ** -7 if dtype != torch.float32 else 1e-6,
                                   atol=1e-6)


def test_misaligned_pointer_is_refused():
    from ddfnet_b200 import _lib
    L = _lib.load()
    t = torch.zeros(4096, device="cuda:0", dtype=torch.float16)
    rc = L.ddf_b200_nhwc_to_nchw(t.data_ptr() + 2, t.data_ptr() + 2048, 1, 8, 4, 4, _lib.F16, None)
    assert rc == -7


def test_channels_last_model_matches_nchw_model():
    """The fused inference harness in channels_last (library transposes, BatchNorm + ReLU on
    the way back) against the plain module-by-module NCHW network."""
    from ddfnet_b200.resnet import DDFResNet, fold_batchnorm
    dev = torch.device("cuda:0")
    torch.manual_seed(7)
    m = DDFResNet([1, 1, 1, 1], "mul").to(dev).eval()
    for mod in m.modules():
        if isinstance(mod, torch.nn.BatchNorm2d):
            mod.running_mean.normal_(0, 0.1)
            mod.running_var.uniform_(0.5, 2)
            mod.weight.data.normal_(1, 0.2)
            mod.bias.data.normal_(0, 0.1)
    x = torch.randn(4, 3, 224, 224, device=dev)
    with torch.no_grad():
        y0 = m(x)
        fold_batchnorm(m, fuse_activations=True)
        m = m.to(memory_format=torch.channels_last)
        y1 = m(x.contiguous(memory_format=torch.channels_last))
    rel = ((y0 - y1).norm() / y0.norm()).item()
    assert rel < 1e-3, rel
