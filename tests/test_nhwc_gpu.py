"""The channels_last (NHWC) forward, ddf_b200_forward_nhwc, against the float64 CPU oracle on
identical seeded inputs: plain, with the spatial filter in both layouts it accepts, with the
fused bias + spatial FilterNorm, and with the affine + ReLU epilogue; and the pooled partial
sums that feed the channel branch."""
import pytest
import torch

from tests.util import DTYPES, check_close, make_inputs, oracle_forward

pytestmark = pytest.mark.gpu

# B, C, H, W, stride -- the ddf_resnet stage shapes at small batch, odd output widths (one
# pixel per thread), channel counts on both sides of a warp, stride 2 with an odd height
SHAPES = [(3, 64, 56, 56, 1), (2, 128, 28, 28, 1), (3, 256, 14, 14, 1), (5, 512, 7, 7, 1),
          (2, 128, 56, 56, 2), (3, 256, 28, 28, 2), (3, 512, 14, 14, 2), (2, 8, 9, 6, 1),
          (2, 16, 11, 10, 2), (1, 1024, 5, 4, 1)]


def _cl(t):
    return t.contiguous(memory_format=torch.channels_last)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_nhwc_forward(shape, dt):
    from ddfnet_b200.nhwc import ddf_nhwc
    B, C, H, W, s = shape
    dtype = DTYPES[dt]
    dev = torch.device("cuda:0")
    x, cf, sf = make_inputs(B, C, H, W, 3, s, dtype, seed=600 + C + s, with_go=False)
    xd, cfd = _cl(x.to(dev)), cf.to(dev)
    for m in ("mul", "add"):
        want = oracle_forward(x, cf, sf, 3, 1, s, m)
        # spatial filter in the reference's planar layout
        out = ddf_nhwc(xd, cfd, sf.to(dev), 3, 1, s, m)
        assert out.is_contiguous(memory_format=torch.channels_last) and out.shape == want.shape
        check_close(out, want, dtype, f"nhwc {shape} {dt} {m} planar sf")
        # ... and as 16 channels_last maps of which the first 9 count
        sf16 = torch.zeros(B, 16, H // s, W // s, dtype=dtype)
        sf16[:, :9] = sf
        sf16[:, 9:] = 7.0   # must be ignored
        out = ddf_nhwc(xd, cfd, _cl(sf16.to(dev)), 3, 1, s, m)
        check_close(out, want, dtype, f"nhwc {shape} {dt} {m} channels_last sf")


@pytest.mark.parametrize("shape", [(3, 64, 28, 28, 1), (2, 128, 14, 14, 2), (3, 32, 7, 7, 1)])
@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_nhwc_fused_norm_bias_and_epilogue(shape, dt):
    """Raw filter + bias -> FilterNorm inside the kernel; BatchNorm-style affine + ReLU on the
    store.  The oracle applies the same steps in float64."""
    from ddfnet_b200.nhwc import ddf_nhwc
    from oracle import ddf_oracle
    B, C, H, W, s = shape
    dtype = DTYPES[dt]
    dev = torch.device("cuda:0")
    x, cf, raw = make_inputs(B, C, H, W, 3, s, dtype, seed=650 + C, with_go=False)
    g = torch.Generator().manual_seed(9)
    bias = torch.randn(9, generator=g) * 0.2
    scale = torch.rand(C, generator=g) + 0.5
    shift = torch.randn(C, generator=g) * 0.3
    gain = 2.0 ** 0.5 / 3
    sfn = ddf_oracle.filter_norm_spatial(raw.double() + bias.double().view(1, 9, 1, 1), 1, 3, gain)
    for m in ("mul", "add"):
        sf_used = sfn.to(dtype).double() if m == "add" else sfn   # add mode rounds the normalised filter
        want = ddf_oracle.forward(x.double(), cf.double(), sf_used, 3, 1, s, m)
        want = torch.relu(want * scale.double().view(1, C, 1, 1) + shift.double().view(1, C, 1, 1))
        out = ddf_nhwc(x.to(dev).contiguous(memory_format=torch.channels_last), cf.to(dev), raw.to(dev), 3, 1, s, m,
                       sf_bias=bias.to(dev), sf_norm_scale=gain, out_scale=scale.to(dev), out_shift=shift.to(dev),
                       relu=True)
        if m == "mul":
            check_close(out, want, dtype, f"nhwc fused {shape} {dt} {m}")
        else:
            # add mode stores the normalised filter in the element type (as the reference's module
            # sequence does): the kernel rounds its float value, the oracle its float64 value, and
            # the two can land one unit in the last place apart on any tap.  Allow exactly that:
            # one ulp of the filter times the sum of |x| under the window, times the epilogue scale.
            ulp = 2.0 ** (-11 if dtype == torch.float16 else -8)
            sum_abs = torch.nn.functional.avg_pool2d(x.double().abs(), 3, s, 1, divisor_override=1)[..., :H // s, :W // s]
            slack = ulp * sfn.abs().max() * sum_abs * scale.double().abs().view(1, C, 1, 1)
            got = out.detach().cpu().double()
            bound = (2e-3 + (2.0 ** -8 if dtype == torch.bfloat16 else 0.0)) * want.abs() + 1e-5 + slack
            assert ((got - want).abs() <= bound).all(), f"nhwc fused {shape} {dt} {m}"


def test_nhwc_pool_partials_and_refusals():
    from ddfnet_b200 import _lib
    from ddfnet_b200.nhwc import nhwc_supported, pool_partials
    dev = torch.device("cuda:0")
    for (B, C, H, W) in [(3, 64, 56, 56), (2, 512, 7, 7), (2, 8, 5, 3)]:
        x = torch.randn(B, C, H, W, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
        p = pool_partials(x.to(dev).contiguous(memory_format=torch.channels_last))
        assert p.shape[0] == B and p.shape[2] == C
        got = p.sum(dim=1).cpu().double()
        want = x.double().sum(dim=(2, 3))
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-3)
    # outside the kernel's range: the helper says so and the C entry point refuses
    x = torch.zeros(1, 12, 8, 8, dtype=torch.bfloat16, device=dev).contiguous(memory_format=torch.channels_last)
    assert not nhwc_supported(x, 3, 1, 1)          # C not a multiple of 8
    assert not nhwc_supported(x.float(), 3, 1, 1)
    L = _lib.load()
    z = torch.zeros(64, dtype=torch.float32, device=dev)
    rc = L.ddf_b200_forward_nhwc(x.data_ptr(), z.data_ptr(), z.data_ptr(), None, z.data_ptr(), None, None, 0,
                                 1, 12, 8, 8, 3, 1, 1, 0, _lib.BF16, 0, 0, 0, 0, 1.0, None)
    assert rc == -7


@pytest.mark.parametrize("cfg", [
    dict(in_channels=64, kernel_size=3, stride=1, head=1, kernel_combine="mul"),
    dict(in_channels=128, kernel_size=3, stride=2, head=1, kernel_combine="add"),
])
@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_ddfpack_channels_last_path_uses_no_layout_copy_and_matches_float32(cfg, dt):
    """DDFPack on a channels_last half-precision tensor takes the channels-innermost route
    (pooled sums, channel-branch kernel, padded convolution, NHWC DDF kernel): the result is
    channels_last, no transposing kernel of the library runs, and it agrees with the
    reference's module sequence evaluated in float32 on the same (rounded) weights."""
    import copy
    from ddfnet_b200 import DDFPack, _lib
    dtype = DTYPES[dt]
    dev = torch.device("cuda:0")
    torch.manual_seed(11)
    m = DDFPack(**cfg).to(dev).eval().to(dtype)
    ref = copy.deepcopy(m).float()
    ref.fuse_channel_branch = False
    ref.fuse_filter_norm = False
    x = torch.randn(4, cfg["in_channels"], 28, 28, device=dev).to(dtype)
    scale = (torch.rand(cfg["in_channels"], device=dev) + 0.5)
    shift = torch.randn(cfg["in_channels"], device=dev) * 0.2
    L = _lib.load()
    with torch.no_grad():
        n0 = L.ddf_b200_launch_count()
        a = m.forward_channels_last(x.contiguous(memory_format=torch.channels_last), scale, shift, relu=True)
        launches = L.ddf_b200_launch_count() - n0
        b = torch.relu(ref(x.float()) * scale.view(1, -1, 1, 1) + shift.view(1, -1, 1, 1))
    assert a is not None and a.is_contiguous(memory_format=torch.channels_last)
    assert launches == 3          # pooled sums, channel branch, DDF: no transposes
    rel = ((a.float() - b).norm() / b.norm()).item()
    assert rel < (1.5e-2 if dtype == torch.bfloat16 else 3e-3), rel
    # the ordinary forward takes the same route for channels_last input
    with torch.no_grad():
        c = m(x.contiguous(memory_format=torch.channels_last))
        d = ref(x.float())
    assert c.is_contiguous(memory_format=torch.channels_last)
    assert ((c.float() - d).norm() / d.norm()).item() < (1.5e-2 if dtype == torch.bfloat16 else 3e-3)


def test_channels_last_half_model_matches_float32_model():
    from ddfnet_b200.resnet import DDFResNet, fold_batchnorm
    import copy
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
        h = copy.deepcopy(m)
        fold_batchnorm(h, fuse_activations=True)
        h = h.half().to(memory_format=torch.channels_last)
        y1 = h(x.half().contiguous(memory_format=torch.channels_last))
    rel = ((y0 - y1.float()).norm() / y0.norm()).item()
    assert rel < 2e-2, rel
