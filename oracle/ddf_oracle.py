"""ctypes wrapper around the CPU oracle (``oracle/ddf_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU-baseline legs of ``bench.py``.  The shipped package
(``ddfnet_b200``) never imports this module and has no CPU fallback.

The arithmetic restates the reference op (see the header of ``ddf_oracle.c`` for
the file:line map).  ``forward`` / ``backward`` take and return torch CPU tensors
(float64 -> golden instance, float32 -> timed baseline instance).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "ddf_oracle.c")
_SO = os.path.join(_HERE, "libddf_oracle.so")
_lock = threading.Lock()
_lib = None

COMBINE = {"mul": 0, "add": 1}


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (x86-64-v3 so the binary runs on any AVX2 host)."""
    with _lock:
        stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(_SRC)
        if force or stale:
            cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC",
                   "-Wall", "-o", _SO + ".tmp", _SRC]
            subprocess.run(cmd, check=True, cwd=_HERE)
            os.replace(_SO + ".tmp", _SO)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        ip = ctypes.c_int
        vp = ctypes.c_void_p
        for sfx in ("f64", "f32"):
            f = getattr(L, f"ddf_oracle_forward_{sfx}")
            f.argtypes = [vp, vp, vp, vp] + [ip] * 8
            f.restype = None
            g = getattr(L, f"ddf_oracle_backward_{sfx}")
            g.argtypes = [vp] * 7 + [ip] * 8
            g.restype = None
        L.ddf_oracle_max_threads.restype = ip
        L.ddf_oracle_set_threads.argtypes = [ip]
        _lib = L
    return _lib


def max_threads() -> int:
    return int(lib().ddf_oracle_max_threads())


def set_threads(n: int) -> None:
    lib().ddf_oracle_set_threads(int(n))


def _sfx(t: torch.Tensor) -> str:
    if t.dtype == torch.float64:
        return "f64"
    if t.dtype == torch.float32:
        return "f32"
    raise TypeError("oracle takes float64 or float32 CPU tensors")


def _prep(*ts):
    dt = ts[0].dtype
    out = []
    for t in ts:
        assert t.device.type == "cpu" and t.dtype == dt
        out.append(t.contiguous())
    return out


def forward(x, cf, sf, k=3, d=1, s=1, combine="mul"):
    x, cf, sf = _prep(x, cf, sf)
    B, C, H, W = x.shape
    assert cf.shape == (B, C, k, k)
    assert sf.shape == (B, k * k, H // s, W // s)
    out = torch.empty(B, C, H // s, W // s, dtype=x.dtype)
    fn = getattr(lib(), f"ddf_oracle_forward_{_sfx(x)}")
    fn(x.data_ptr(), cf.data_ptr(), sf.data_ptr(), out.data_ptr(),
       B, C, H, W, k, d, s, COMBINE[combine])
    return out


def backward(go, x, cf, sf, k=3, d=1, s=1, combine="mul", need=(True, True, True)):
    """Returns (grad_x, grad_cf, grad_sf); entries not needed are None."""
    go, x, cf, sf = _prep(go, x, cf, sf)
    B, C, H, W = x.shape
    assert go.shape == (B, C, H // s, W // s)
    gx = torch.empty_like(x) if need[0] else None
    gcf = torch.empty_like(cf) if need[1] else None
    gsf = torch.empty_like(sf) if need[2] else None
    fn = getattr(lib(), f"ddf_oracle_backward_{_sfx(x)}")
    p = lambda t: t.data_ptr() if t is not None else None
    fn(go.data_ptr(), x.data_ptr(), cf.data_ptr(), sf.data_ptr(),
       p(gx), p(gcf), p(gsf), B, C, H, W, k, d, s, COMBINE[combine])
    return gx, gcf, gsf


# --------------------------------------------------------------------------------------
# Independent derivation used to pin the C oracle: unfold-based composite whose
# gradients come from torch autograd (no hand-written backward involved).
# --------------------------------------------------------------------------------------
def composite_forward(x, cf, sf, k=3, d=1, s=1, combine="mul"):
    """out = sum_t unfold(x)[.., t, ..] * (cf (.) sf), on any device/dtype torch supports."""
    import torch.nn.functional as F

    B, C, H, W = x.shape
    OH, OW = H // s, W // s
    pad = (k - 1) // 2 * d
    cols = F.unfold(x, kernel_size=k, dilation=d, padding=pad, stride=s)
    fh = (H + 2 * pad - d * (k - 1) - 1) // s + 1
    fw = (W + 2 * pad - d * (k - 1) - 1) // s + 1
    cols = cols.view(B, C, k * k, fh, fw)[:, :, :, :OH, :OW]
    cfv = cf.reshape(B, C, k * k, 1, 1)
    sfv = sf.reshape(B, 1, k * k, OH, OW)
    w = cfv * sfv if combine == "mul" else cfv + sfv
    return (cols * w).sum(dim=2)


def py_forward_restatement(feat, channel_att, spatial_att, kernel_size, dilation, stride,
                           kernel_combine):
    """Six-deep loop with the structure of the reference's test oracle
    (grad_check.py:11-30, stride 1 only).  Small cases only."""
    assert stride == 1
    B, C, H, W = feat.shape
    out = torch.zeros(B, C, H, W, dtype=torch.float64)
    half = kernel_size // 2
    for b in range(B):
        for c in range(C):
            for y in range(H):
                for x in range(W):
                    acc = 0.0
                    for iy in range(kernel_size):
                        for ix in range(kernel_size):
                            yy = y + (iy - half) * dilation
                            xx = x + (ix - half) * dilation
                            if yy < 0 or yy >= H or xx < 0 or xx >= W:
                                continue
                            ca = float(channel_att[b, c, iy, ix])
                            sa = float(spatial_att[b, iy * kernel_size + ix, y, x])
                            wgt = ca * sa if kernel_combine == "mul" else ca + sa
                            acc += wgt * float(feat[b, c, yy, xx])
                    out[b, c, y, x] = acc
    return out


def filter_norm_spatial(raw: torch.Tensor, head: int, k: int, scale: float) -> torch.Tensor:
    """FilterNorm(filter_type='spatial') with neither running std nor running mean, restated
    from ddf/ddf.py:146-152 with explicit loops over the taps (float64): for every sample,
    head and pixel, the k*k values are centred, divided by (unbiased std + 1e-10) and
    multiplied by ``scale`` (= calculate_gain(nonlinearity) / k, ddf/ddf.py:135)."""
    v = raw.double()
    b, ch, h, w = v.shape
    kk = k * k
    assert ch == head * kk
    v = v.reshape(b, head, kk, h, w)
    out = torch.empty_like(v)
    mean = torch.zeros(b, head, h, w, dtype=torch.float64)
    for t in range(kk):
        mean += v[:, :, t]
    mean /= kk
    var = torch.zeros_like(mean)
    for t in range(kk):
        var += (v[:, :, t] - mean) ** 2
    std = (var / (kk - 1)).sqrt()
    for t in range(kk):
        out[:, :, t] = (v[:, :, t] - mean) / (std + 1e-10) * scale
    return out.reshape(b, ch, h, w)


def filter_norm_channel(raw: torch.Tensor, c: int, k: int, std_param: torch.Tensor) -> torch.Tensor:
    """FilterNorm(filter_type='channel', running_std=True) restated from ddf/ddf.py:158-170:
    per sample and channel, the k*k values are centred, divided by (unbiased std + 1e-10)
    and multiplied by the learnable per-(channel, tap) std.  Returns (B, C*k*k), float64."""
    kk = k * k
    v = raw.double().reshape(raw.shape[0], c, kk)
    mean = v.sum(dim=2, keepdim=True) / kk
    d = v - mean
    std = ((d * d).sum(dim=2, keepdim=True) / (kk - 1)).sqrt()
    return (d / (std + 1e-10)).reshape(raw.shape[0], c * kk) * std_param.double()[None, :]
