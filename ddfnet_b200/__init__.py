"""ddfnet_b200 -- the Decoupled Dynamic Filter (DDF) operator for NVIDIA B200.

``ddf`` is a drop-in for the reference's autograd op; ``DDFPack`` / ``DDFUpPack``
/ ``FilterNorm`` mirror the modules that call it (reference: ddf/ddf.py).  The
arithmetic runs in hand-written sm_100a CUDA kernels behind the C ABI declared
in include/ddf_b200.h.
"""
from .op import DDFFunction, DDFSpatialNormFunction, ddf, ddf_sfnorm
from .modules import (DDFPack, DDFUpPack, FilterNorm, build_channel_branch,
                      build_spatial_branch)
from ._lib import take_fault
from .host import ddf_host, ddf_host_async
from .layout import to_channels_last, to_nchw

__all__ = ["ddf", "ddf_sfnorm", "DDFFunction", "DDFSpatialNormFunction", "DDFPack", "DDFUpPack", "FilterNorm",
           "build_spatial_branch", "build_channel_branch", "ddf_host", "ddf_host_async", "to_nchw",
           "to_channels_last", "take_fault"]
