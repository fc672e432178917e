"""The DDF forward on channels_last tensors (``ddf_b200_forward_nhwc``): inference helpers
for networks that keep their activations channels-innermost.  No autograd history is
recorded; callers that need gradients use ``ddf`` on contiguous NCHW tensors.
"""
from __future__ import annotations

import torch

from . import _lib
from .op import _DTYPES


def _is_cl(t: torch.Tensor) -> bool:
    return t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last)


def nhwc_supported(x: torch.Tensor, kernel_size: int, dilation: int, stride: int) -> bool:
    """True when ``ddf_nhwc`` covers this input (else convert to NCHW and use ``ddf``)."""
    b, c, h, w = x.shape
    return (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and _is_cl(x) and kernel_size == 3
            and dilation == 1 and stride in (1, 2) and c % 8 == 0 and c <= 2048 and 256 % (c // 8) == 0
            and w % stride == 0 and b <= 65535
            and not (torch.is_grad_enabled() and x.requires_grad))


def pool_partials(x: torch.Tensor) -> torch.Tensor:
    """Float partial sums (B, tiles, C) of a channels_last ``x`` over tiles of pixels, the form
    ``ddf_b200_channel_filter`` takes for the channel branch's average pool."""
    b, c, h, w = x.shape
    lib = _lib.load()
    nt = int(lib.ddf_b200_pool_nhwc_tiles(h, w))
    out = torch.empty((b, nt, c), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.ddf_b200_pool_nhwc(x.data_ptr(), out.data_ptr(), b, c, h, w, _DTYPES[x.dtype],
                                          torch.cuda.current_stream().cuda_stream))
    return out


def ddf_nhwc(x: torch.Tensor, channel_filter: torch.Tensor, spatial_filter: torch.Tensor,
             kernel_size: int = 3, dilation: int = 1, stride: int = 1, kernel_combine: str = "mul",
             sf_bias: torch.Tensor | None = None, sf_norm_scale: float | None = None,
             out_scale: torch.Tensor | None = None, out_shift: torch.Tensor | None = None,
             relu: bool = False) -> torch.Tensor:
    """DDF forward on a channels_last ``x`` (B, C, H, W); returns a channels_last tensor.

    ``channel_filter`` (B, C, k, k) contiguous.  ``spatial_filter`` (B, G, H/s, W/s) with
    G >= k*k maps, channels_last or contiguous; only the first k*k maps are read.  With
    ``sf_norm_scale`` given, ``spatial_filter`` is the raw convolution output: ``sf_bias``
    (k*k float32 values) is added and the spatial FilterNorm applied inside the kernel.
    ``out_scale`` / ``out_shift`` (C float32 values each) and ``relu`` are applied on the store.
    """
    assert kernel_combine in ("mul", "add")
    b, c, h, w = x.shape
    k = kernel_size
    oh, ow = h // stride, w // stride
    assert nhwc_supported(x, k, dilation, stride), "outside ddf_b200_forward_nhwc's range"
    assert channel_filter.shape == (b, c, k, k) and channel_filter.is_contiguous() and channel_filter.dtype == x.dtype
    g = spatial_filter.shape[1]
    assert spatial_filter.shape == (b, g, oh, ow) and g >= k * k and spatial_filter.dtype == x.dtype
    # a tensor can satisfy both layouts (one map or one pixel); prefer the planar reading then
    if spatial_filter.is_contiguous():
        strides = (g * oh * ow, 1, oh * ow)
    elif _is_cl(spatial_filter):
        strides = (g * oh * ow, g, 1)
    else:
        spatial_filter = spatial_filter.contiguous()
        strides = (g * oh * ow, 1, oh * ow)
    for t in (sf_bias, out_scale, out_shift):
        assert t is None or (t.dtype == torch.float32 and t.is_cuda and t.is_contiguous())
    assert (out_scale is None) == (out_shift is None)
    out = torch.empty((b, c, oh, ow), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    ptr = lambda t: t.data_ptr() if t is not None else None
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().ddf_b200_forward_nhwc(
            x.data_ptr(), channel_filter.data_ptr(), spatial_filter.data_ptr(), ptr(sf_bias), out.data_ptr(),
            ptr(out_scale), ptr(out_shift), int(relu), b, c, h, w, k, dilation, stride,
            _lib.MUL if kernel_combine == "mul" else _lib.ADD, _DTYPES[x.dtype], strides[0], strides[1], strides[2],
            int(sf_norm_scale is not None), float(sf_norm_scale or 1.0), torch.cuda.current_stream().cuda_stream))
    return out
