"""Layout adapters between a channels_last (NHWC) network and the contiguous NCHW tensors
the DDF op works on, backed by the tiled-transpose kernels of libddf_b200.so
(``ddf_b200_nhwc_to_nchw`` / ``ddf_b200_nchw_to_nhwc``).  Inference helpers: they do not
record autograd history (a tensor that requires grad goes through plain torch ops instead).
"""
from __future__ import annotations

import torch

from . import _lib
from .op import _DTYPES


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dim() == 4 and t.dtype in _DTYPES and t.dtype != torch.float64 \
        and not (torch.is_grad_enabled() and t.requires_grad)


def to_nchw(x: torch.Tensor) -> torch.Tensor:
    """A contiguous (NCHW) copy of a channels_last tensor; NCHW input is returned as is."""
    if x.is_contiguous():
        return x
    if not (_native(x) and x.is_contiguous(memory_format=torch.channels_last)):
        return x.contiguous()
    b, c, h, w = x.shape
    out = torch.empty((b, c, h, w), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().ddf_b200_nhwc_to_nchw(
            x.data_ptr(), out.data_ptr(), b, c, h, w, _DTYPES[x.dtype],
            torch.cuda.current_stream().cuda_stream))
    return out


def to_nchw_affine(x: torch.Tensor, channels: int, scale: torch.Tensor, shift: torch.Tensor,
                   relu: bool = False) -> torch.Tensor:
    """Contiguous NCHW tensor of the first ``channels`` channels of a channels_last ``x``, with
    ``x * scale[c] + shift[c]`` (float32 tensors of ``channels`` values) applied on the way."""
    b, sc, h, w = x.shape
    assert channels <= sc and scale.numel() == channels and shift.numel() == channels
    if not (_native(x) and x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous()):
        y = x[:, :channels] * scale.to(x.dtype).reshape(1, -1, 1, 1) + shift.to(x.dtype).reshape(1, -1, 1, 1)
        return (torch.relu(y) if relu else y).contiguous()
    out = torch.empty((b, channels, h, w), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().ddf_b200_nhwc_to_nchw_affine(
            x.data_ptr(), out.data_ptr(), b, channels, h, w, sc, _DTYPES[x.dtype],
            scale.data_ptr(), shift.data_ptr(), int(relu), torch.cuda.current_stream().cuda_stream))
    return out


def to_channels_last(x: torch.Tensor, scale: torch.Tensor | None = None,
                     shift: torch.Tensor | None = None, relu: bool = False) -> torch.Tensor:
    """channels_last copy of a contiguous NCHW tensor, optionally with
    ``relu(x * scale[c] + shift[c])`` applied on the way (``scale`` / ``shift``: float32
    tensors of C values, e.g. an eval-mode BatchNorm folded to an affine map)."""
    assert (scale is None) == (shift is None)
    if not (_native(x) and x.is_contiguous()):
        y = x
        if scale is not None:
            y = y * scale.to(y.dtype).reshape(1, -1, 1, 1) + shift.to(y.dtype).reshape(1, -1, 1, 1)
        if relu:
            y = torch.relu(y)
        return y.contiguous(memory_format=torch.channels_last)
    b, c, h, w = x.shape
    out = torch.empty((b, c, h, w), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    if scale is not None:
        assert scale.dtype == torch.float32 and shift.dtype == torch.float32
        assert scale.numel() == c and shift.numel() == c and scale.is_cuda and shift.is_cuda
        scale, shift = scale.contiguous(), shift.contiguous()
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().ddf_b200_nchw_to_nhwc(
            x.data_ptr(), out.data_ptr(), b, c, h, w, _DTYPES[x.dtype],
            scale.data_ptr() if scale is not None else None,
            shift.data_ptr() if shift is not None else None, int(relu),
            torch.cuda.current_stream().cuda_stream))
    return out
