"""``ddf(features, channel_filter, spatial_filter, kernel_size, dilation, stride,
kernel_combine, version)`` -- drop-in for the reference autograd op
(``DDFFunction`` / ``ddf`` in ddf/ddf.py:27-122).

Same positional signature, same assertion checks (ddf/ddf.py:32-65), same
8-tuple of gradients (ddf/ddf.py:119).  Differences, all deliberate:

* float16 and bfloat16 tensors are computed natively (float accumulation) and
  the result has the input's type; the reference up-casts float16 to float32
  (ddf/ddf.py:36-42) and cannot take bfloat16.
* inputs are saved for the backward when autograd asks for any input gradient
  (``ctx.needs_input_grad``); the reference tests ``requires_grad`` on its
  up-cast copies (ddf/ddf.py:88-89), which loses the graph under float16.
* ``version``: '' picks a kernel automatically, 'o' forces the generic kernel,
  'f' forces the plane-streaming kernel (the reference's 'o' / 'f' select its
  generic / tiled forward, ddf/ddf.py:77-84).
* non-contiguous inputs raise RuntimeError, as the reference's native
  CHECK_CONTIGUOUS does (ddf/src/cuda/ddf_mul_cuda.cpp:28-40).

The arithmetic runs in hand-written CUDA kernels reached through the C ABI of
libddf_b200.so; there is no CPU path.
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16,
           torch.float64: _lib.F64}
_COMBINE = {"mul": _lib.MUL, "add": _lib.ADD}
_VARIANT = {"": _lib.VARIANT_AUTO, "o": _lib.VARIANT_GENERIC, "f": _lib.VARIANT_STREAM}


def _common_dtype(*tensors):
    dt = tensors[0].dtype
    for t in tensors[1:]:
        dt = torch.promote_types(dt, t.dtype)
    if dt not in _DTYPES:
        raise TypeError(f"ddf: unsupported dtype {dt}")
    return dt


def _require_contiguous(t, name):
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous ")


def _backward_launch(ctx, grad_output, features, channel_filter, spatial_filter, need):
    """All requested gradients of the op through ddf_b200_backward; tensors are contiguous
    and of one dtype.  Returns (gx, gcf, gsf), None where not requested."""
    dt = features.dtype
    grad_output = grad_output.to(dt).contiguous()
    b, c, h, w = features.size()
    k, d, s = ctx.kernel_size, ctx.dilation, ctx.stride
    need_x, need_cf, need_sf = need
    dev = features.device
    gx = torch.empty_like(features) if need_x else None
    gcf = torch.empty_like(channel_filter) if need_cf else None
    gsf = torch.empty_like(spatial_filter) if need_sf else None

    lib = _lib.load()
    comb, dtc = _COMBINE[ctx.op_type], _DTYPES[dt]
    with torch.cuda.device(dev):
        ws_bytes = int(lib.ddf_b200_backward_workspace(b, c, h, w, k, d, s, comb, dtc, ctx.bwd_variant))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
        stream = torch.cuda.current_stream().cuda_stream
        ptr = lambda t: t.data_ptr() if t is not None else None
        _lib.check(lib.ddf_b200_backward(
            grad_output.data_ptr(), features.data_ptr(), channel_filter.data_ptr(),
            spatial_filter.data_ptr(), ptr(gx), ptr(gcf), ptr(gsf), ptr(ws), ws_bytes,
            b, c, h, w, k, d, s, comb, dtc, ctx.bwd_variant, stream))
    return gx, gcf, gsf


def _check_shapes(features, channel_filter, spatial_filter, kernel_size, dilation, stride,
                  kernel_combine, version):
    """The reference's argument checks (ddf/ddf.py:32-65)."""
    assert features.is_cuda, 'input feature must be a CUDA tensor.'
    assert channel_filter.is_cuda, 'channel_filter must be a CUDA tensor.'
    assert spatial_filter.is_cuda, 'spatial_filter must be a CUDA tensor.'
    b, c, h, w = features.size()
    bc, cc, hc, wc = channel_filter.size()
    assert bc == b and cc == c, \
        "channel_filter size {} does not match feature size {}".format(
            channel_filter.size(), features.size())
    assert hc == kernel_size and wc == kernel_size, \
        "channel_filter size {} does not match kernel size {}".format(
            channel_filter.size(), kernel_size)
    bs, cs, hs, ws = spatial_filter.size()
    assert bs == b and hs == h // stride and ws == w // stride, \
        "spatial_filter size {} does not match feature size {} with stride {}".format(
            spatial_filter.size(), features.size(), stride)
    assert cs == kernel_size ** 2, \
        "spatial_filter size {} does not match kernel size {}".format(
            spatial_filter.size(), kernel_size)
    assert (kernel_size - 1) % 2 == 0 and kernel_size >= 1 and dilation >= 1 and stride >= 1
    assert kernel_combine in {'mul', 'add'}, \
        'only support mul or add combination, instead of {}'.format(kernel_combine)
    assert version in _VARIANT, "version must be '', 'o' or 'f'"
    assert channel_filter.device == features.device and spatial_filter.device == features.device


def spatial_filter_norm(raw, kernel_size, scale):
    """FilterNorm(filter_type='spatial') without running statistics (ddf/ddf.py:146-157) on a
    (B, k*k, H, W) tensor whose heads are already folded into B: each pixel's k*k values are
    centred, divided by their unbiased std + 1e-10 and multiplied by ``scale``.  Plain torch
    ops, float32 statistics for 2-byte inputs; used to recompute the filter for the backward
    of the fused op."""
    v = raw.float() if raw.dtype in (torch.float16, torch.bfloat16) else raw
    v = v - v.mean(dim=1, keepdim=True)
    v = v / (v.std(dim=1, keepdim=True) + 1e-10)
    return v * scale


class DDFSpatialNormFunction(Function):
    """``ddf`` with the spatial FilterNorm fused into the forward kernel:
    ``ddf_sfnorm(x, cf, raw, k, d, s, combine, scale, version)`` equals
    ``ddf(x, cf, FilterNorm_spatial(raw), k, d, s, combine, version)`` with the normalised
    filter never written to memory (it is kept in float inside the kernel).  The backward
    recomputes the normalised filter with the library's ``ddf_b200_sfnorm``, runs the ordinary
    DDF backward on it and carries the filter gradient back through the normalisation with
    ``ddf_b200_sfnorm_backward``: no torch arithmetic on either path."""

    @staticmethod
    def forward(ctx, features, channel_filter, spatial_raw, kernel_size=3, dilation=1, stride=1,
                kernel_combine='mul', scale=1.0, version=''):
        _check_shapes(features, channel_filter, spatial_raw, kernel_size, dilation, stride,
                      kernel_combine, version)
        assert kernel_size >= 3, 'the fused filter norm needs kernel_size >= 3'
        ctx.in_dtypes = (features.dtype, channel_filter.dtype, spatial_raw.dtype)
        dt = _common_dtype(features, channel_filter, spatial_raw)
        features, channel_filter, spatial_raw = (t.to(dt) for t in (features, channel_filter, spatial_raw))
        _require_contiguous(features, "features")
        _require_contiguous(channel_filter, "channel_filter")
        _require_contiguous(spatial_raw, "spatial_filter")
        ctx.kernel_size, ctx.dilation, ctx.stride = kernel_size, dilation, stride
        ctx.op_type = kernel_combine
        ctx.scale = float(scale)
        ctx.bwd_variant = _lib.VARIANT_GENERIC if version == 'o' else _lib.VARIANT_AUTO
        b, c, h, w = features.size()
        output = torch.empty((b, c, h // stride, w // stride), dtype=dt, device=features.device)
        lib = _lib.load()
        with torch.cuda.device(features.device):
            _lib.check(lib.ddf_b200_forward_sfnorm(
                features.data_ptr(), channel_filter.data_ptr(), spatial_raw.data_ptr(),
                output.data_ptr(), b, c, h, w, kernel_size, dilation, stride,
                _COMBINE[kernel_combine], _DTYPES[dt], _VARIANT[version], ctx.scale,
                torch.cuda.current_stream().cuda_stream))
        if any(ctx.needs_input_grad[:3]):
            ctx.save_for_backward(features, channel_filter, spatial_raw)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        features, channel_filter, spatial_raw = ctx.saved_tensors
        need_x, need_cf, need_sf = ctx.needs_input_grad[:3]
        lib = _lib.load()
        b, kk, oh, ow = spatial_raw.shape
        dtc = _DTYPES[spatial_raw.dtype]
        # the normalised filter, recomputed once by the library for the gradient kernels
        normed = torch.empty_like(spatial_raw)
        with torch.cuda.device(features.device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.ddf_b200_sfnorm(spatial_raw.data_ptr(), normed.data_ptr(), b, ctx.kernel_size, oh, ow,
                                           dtc, ctx.scale, stream))
        gx, gcf, gsf = _backward_launch(ctx, grad_output, features, channel_filter, normed,
                                        (need_x, need_cf, need_sf))
        graw = None
        if need_sf:
            # ... and the filter gradient carried back through the normalisation
            graw = torch.empty_like(spatial_raw)
            gsf = gsf.contiguous()
            with torch.cuda.device(features.device):
                _lib.check(lib.ddf_b200_sfnorm_backward(
                    spatial_raw.data_ptr(), gsf.data_ptr(), graw.data_ptr(), b, ctx.kernel_size, oh, ow, dtc,
                    ctx.scale, torch.cuda.current_stream().cuda_stream))
        dx, dcf, dsf = ctx.in_dtypes
        gx = gx.to(dx) if gx is not None else None
        gcf = gcf.to(dcf) if gcf is not None else None
        graw = graw.to(dsf) if graw is not None else None
        return gx, gcf, graw, None, None, None, None, None, None


class DDFFunction(Function):
    @staticmethod
    def forward(ctx, features, channel_filter, spatial_filter,
                kernel_size=3, dilation=1, stride=1, kernel_combine='mul', version=''):
        _check_shapes(features, channel_filter, spatial_filter, kernel_size, dilation, stride,
                      kernel_combine, version)
        b, c, h, w = features.size()

        ctx.in_dtypes = (features.dtype, channel_filter.dtype, spatial_filter.dtype)
        dt = _common_dtype(features, channel_filter, spatial_filter)
        features = features.to(dt)
        channel_filter = channel_filter.to(dt)
        spatial_filter = spatial_filter.to(dt)
        _require_contiguous(features, "features")
        _require_contiguous(channel_filter, "channel_filter")
        _require_contiguous(spatial_filter, "spatial_filter")

        ctx.kernel_size = kernel_size
        ctx.dilation = dilation
        ctx.stride = stride
        ctx.op_type = kernel_combine
        ctx.variant = _VARIANT[version]
        # as in the reference, 'f' selects a forward kernel only (its backward always
        # runs the non-"faster" module, ddf/ddf.py:71,103,114)
        ctx.bwd_variant = _lib.VARIANT_GENERIC if version == 'o' else _lib.VARIANT_AUTO

        output = torch.empty((b, c, h // stride, w // stride), dtype=dt, device=features.device)
        lib = _lib.load()
        with torch.cuda.device(features.device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.ddf_b200_forward(
                features.data_ptr(), channel_filter.data_ptr(), spatial_filter.data_ptr(),
                output.data_ptr(), b, c, h, w, kernel_size, dilation, stride,
                _COMBINE[kernel_combine], _DTYPES[dt], ctx.variant, stream))
        if any(ctx.needs_input_grad[:3]):
            ctx.save_for_backward(features, channel_filter, spatial_filter)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.is_cuda
        features, channel_filter, spatial_filter = ctx.saved_tensors
        gx, gcf, gsf = _backward_launch(ctx, grad_output, features, channel_filter, spatial_filter,
                                        ctx.needs_input_grad[:3])
        dx, dcf, dsf = ctx.in_dtypes
        if gx is not None and gx.dtype != dx:
            gx = gx.to(dx)
        if gcf is not None and gcf.dtype != dcf:
            gcf = gcf.to(dcf)
        if gsf is not None and gsf.dtype != dsf:
            gsf = gsf.to(dsf)
        return gx, gcf, gsf, None, None, None, None, None


ddf = DDFFunction.apply
ddf_sfnorm = DDFSpatialNormFunction.apply
