"""``ddf_host``: the DDF forward for callers whose tensors live in host memory.

Inputs are CPU tensors (pinned memory gives full PCIe speed); the result is a
pinned CPU tensor.  The batch is cut into chunks that are pipelined over three CUDA
streams so that the upload of one chunk, the kernels of another and the download
of a third overlap (the op is independent per sample, so chunking is exact).
"""
from __future__ import annotations

import torch

from .op import ddf


_STREAMS = {}


def _streams(dev, n):
    key = (dev.index, n)
    if key not in _STREAMS:
        _STREAMS[key] = [torch.cuda.Stream(device=dev) for _ in range(n)]
    return _STREAMS[key]


def ddf_host(features, channel_filter, spatial_filter, kernel_size=3, dilation=1, stride=1,
             kernel_combine='mul', out=None, device=None, chunks=None):
    assert not features.is_cuda and not channel_filter.is_cuda and not spatial_filter.is_cuda
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    b, c, h, w = features.shape
    if out is None:
        out = torch.empty((b, c, h // stride, w // stride), dtype=features.dtype, pin_memory=True)
    if chunks is None:
        # about 24 MB of input per chunk: enough chunks to overlap the two copy
        # directions with the kernels, few enough that host launch cost stays small
        nbytes = features.numel() * features.element_size()
        chunks = max(1, min(8, nbytes // (24 << 20)))
    chunks = max(1, min(chunks, b))
    streams = _streams(dev, min(3, chunks))
    cur = torch.cuda.current_stream(dev)
    for st in streams:
        st.wait_stream(cur)
    keep = []
    with torch.no_grad():
        for i in range(chunks):
            lo, hi = i * b // chunks, (i + 1) * b // chunks
            if lo == hi:
                continue
            st = streams[i % len(streams)]
            with torch.cuda.stream(st):
                xd = features[lo:hi].to(dev, non_blocking=True)
                cfd = channel_filter[lo:hi].to(dev, non_blocking=True)
                sfd = spatial_filter[lo:hi].to(dev, non_blocking=True)
                od = ddf(xd, cfd, sfd, kernel_size, dilation, stride, kernel_combine)
                out[lo:hi].copy_(od, non_blocking=True)
                keep.append((xd, cfd, sfd, od))
    for st in streams:
        cur.wait_stream(st)
        st.synchronize()
    return out
