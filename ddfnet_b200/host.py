"""``ddf_host`` / ``ddf_host_async``: the DDF forward for callers whose tensors live in host
memory.

Inputs are CPU tensors (pinned memory gives full PCIe speed); the result is a pinned CPU
tensor.  The batch is cut into chunks that travel over a small set of persistent CUDA streams
taken in rotation -- across calls too -- so that the upload of one chunk, the kernel of another
and the download of a third overlap (the op is independent per sample, so chunking is exact).
PCIe is full duplex: with uploads and downloads in flight together a sequence of calls costs
about max(upload, download), not their sum.  ``ddf_host_async`` returns without waiting, which
is what lets consecutive calls overlap; ``ddf_host`` is the same followed by a wait.
"""
from __future__ import annotations

import torch

from .op import ddf

_N_STREAMS = 4
_STREAMS = {}
_NEXT = {}


def _streams(dev):
    if dev.index not in _STREAMS:
        _STREAMS[dev.index] = [torch.cuda.Stream(device=dev) for _ in range(_N_STREAMS)]
        _NEXT[dev.index] = 0
    return _STREAMS[dev.index]


class HostResult:
    """Handle of an asynchronous ``ddf_host_async`` call: ``out`` holds the result once
    ``wait()`` has returned (or once the streams it names have been synchronised)."""

    def __init__(self, out, events):
        self.out = out
        self._events = events

    def wait(self):
        for e in self._events:
            e.synchronize()
        return self.out


def ddf_host_async(features, channel_filter, spatial_filter, kernel_size=3, dilation=1, stride=1,
                   kernel_combine='mul', out=None, device=None, chunks=None) -> HostResult:
    assert not features.is_cuda and not channel_filter.is_cuda and not spatial_filter.is_cuda
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    b, c, h, w = features.shape
    if out is None:
        out = torch.empty((b, c, h // stride, w // stride), dtype=features.dtype, pin_memory=True)
    if chunks is None:
        # about 16 MB of input per chunk: enough pieces to overlap the two copy directions
        # with the kernels, few enough that the host's launch cost stays small
        nbytes = features.numel() * features.element_size()
        chunks = max(1, min(8, nbytes // (16 << 20)))
    chunks = max(1, min(chunks, b))
    streams = _streams(dev)
    cur = torch.cuda.current_stream(dev)
    used = {}
    with torch.no_grad():
        for i in range(chunks):
            lo, hi = i * b // chunks, (i + 1) * b // chunks
            if lo == hi:
                continue
            k = _NEXT[dev.index]
            _NEXT[dev.index] = (k + 1) % _N_STREAMS
            st = streams[k]
            if k not in used:
                st.wait_stream(cur)  # ordered after whatever the caller queued before
            with torch.cuda.stream(st):
                # tensors allocated here belong to `st`: the caching allocator reuses their
                # memory in stream order, so they need not outlive this block
                xd = features[lo:hi].to(dev, non_blocking=True)
                cfd = channel_filter[lo:hi].to(dev, non_blocking=True)
                sfd = spatial_filter[lo:hi].to(dev, non_blocking=True)
                od = ddf(xd, cfd, sfd, kernel_size, dilation, stride, kernel_combine)
                out[lo:hi].copy_(od, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(st)
                used[k] = ev
    return HostResult(out, list(used.values()))


def ddf_host(features, channel_filter, spatial_filter, kernel_size=3, dilation=1, stride=1,
             kernel_combine='mul', out=None, device=None, chunks=None):
    """Synchronous form: the returned pinned tensor holds the result."""
    return ddf_host_async(features, channel_filter, spatial_filter, kernel_size, dilation, stride,
                          kernel_combine, out, device, chunks).wait()
