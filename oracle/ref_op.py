"""Calls the reference project's own compiled CUDA extension modules (built by
oracle/build_ref.py into oracle/_ref/).  TEST INFRASTRUCTURE ONLY: used to
produce the fixtures under tests/golden/ and to time the reference's kernels
beside ours; never imported by the shipped package.

The call protocol restates what the reference's Python wrapper does around the
native calls: zero-filled caller-allocated output (ddf/ddf.py:74), the variant
rule (ddf/ddf.py:77-84), float16 up-cast (ddf/ddf.py:36-42, 97-98) and the six
zero-filled tensors of the backward (ddf/ddf.py:106-117).
"""
from __future__ import annotations

import importlib
import os
import sys

import torch

_REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_mods = None


def available() -> bool:
    return all(os.path.exists(os.path.join(_REF, m + ".so"))
               for m in ("ddf_mul_ext", "ddf_mul_faster_ext", "ddf_add_ext", "ddf_add_faster_ext"))


def _load():
    global _mods
    if _mods is None:
        if not available():
            raise RuntimeError("reference extension modules are not built (oracle/build_ref.py)")
        if _REF not in sys.path:
            sys.path.insert(0, _REF)
        _mods = {
            "mul": importlib.import_module("ddf_mul_ext"),
            "mul_faster": importlib.import_module("ddf_mul_faster_ext"),
            "add": importlib.import_module("ddf_add_ext"),
            "add_faster": importlib.import_module("ddf_add_faster_ext"),
        }
    return _mods


def _up(t):
    return t.float() if t.dtype == torch.float16 else t


def forward(x, cf, sf, k=3, d=1, s=1, combine="mul", version=""):
    mods = _load()
    x, cf, sf = _up(x), _up(cf), _up(sf)
    b, c, h, w = x.shape
    out = x.new_zeros((b, c, h // s, w // s))
    if version == "f":
        op = combine + "_faster"
    elif version == "o":
        op = combine
    elif k <= 4 and h >= 14 and w >= 14 and s == 1:
        op = combine + "_faster"
    else:
        op = combine
    mods[op].forward(x, cf, sf, k, d, s, out)
    return out


def backward(go, x, cf, sf, k=3, d=1, s=1, combine="mul"):
    mods = _load()
    go, x, cf, sf = _up(go).contiguous(), _up(x), _up(cf), _up(sf)
    r_go = torch.zeros_like(go)
    r_gx = torch.zeros_like(x)
    r_gsf = torch.zeros_like(sf)
    gx = torch.zeros_like(x)
    gcf = torch.zeros_like(cf)
    gsf = torch.zeros_like(sf)
    mods[combine].backward(go, x, cf, sf, k, d, s, r_go, r_gx, r_gsf, gx, gcf, gsf)
    return gx, gcf, gsf
