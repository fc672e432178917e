"""Generates filternorm_*.pt in this directory by running the REFERENCE project's own
``FilterNorm`` module (ddf/ddf.py:125-173, pure PyTorch) on the CPU in float64 on seeded
inputs.  The reference package imports its four CUDA extension modules at import time
(ddf/ddf.py:17); they are not needed by FilterNorm, so empty stand-ins are registered
for them before the import.

    python tests/golden/make_golden_filternorm.py /path/to/reference [outdir]
"""
import os
import sys
import types

import torch


def main(ref_root, outdir):
    for name in ("ddf_mul_ext", "ddf_mul_faster_ext", "ddf_add_ext", "ddf_add_faster_ext"):
        sys.modules["ddf." + name] = types.ModuleType("ddf." + name)
    sys.path.insert(0, ref_root)
    from ddf.ddf import FilterNorm  # the reference's class

    g = torch.Generator().manual_seed(9090)
    cases = {}
    # spatial: (B, head*k*k, H, W), no running statistics (build_spatial_branch)
    for name, (B, head, k, H, W, nl) in {
        "spatial_k3_h1_relu": (2, 1, 3, 7, 9, "relu"),
        "spatial_k3_h2_linear": (2, 2, 3, 6, 5, "linear"),
        "spatial_k5_h1_relu": (1, 1, 5, 4, 6, "relu"),
    }.items():
        raw = torch.randn(B, head * k * k, H, W, generator=g, dtype=torch.float64) * 1.7 + 0.3
        m = FilterNorm(head, k, "spatial", nl)
        cases[name] = {"type": "spatial", "head": head, "k": k, "nonlinearity": nl, "raw": raw,
                       "scale": float(m.std), "out": m(raw)}
    # channel: (B, C*k*k, 1, 1) with the learnable std (build_channel_branch)
    for name, (B, C, k, nl) in {
        "channel_k3_relu": (3, 6, 3, "relu"),
        "channel_k5_relu": (2, 4, 5, "relu"),
    }.items():
        raw = torch.randn(B, C * k * k, 1, 1, generator=g, dtype=torch.float64) * 0.8 - 0.1
        m = FilterNorm(C, k, "channel", nl, running_std=True)
        with torch.no_grad():
            m.std.copy_((torch.randn(C * k * k, generator=g) * float(torch.nn.init.calculate_gain(nl)) / k))
        m = m.double()
        cases[name] = {"type": "channel", "C": C, "k": k, "nonlinearity": nl, "raw": raw,
                       "std": m.std.detach().clone(), "out": m(raw).detach()}
    for name, c in cases.items():
        c["source"] = "reference FilterNorm (theFoxofSky/ddfnet ddf/ddf.py), float64, CPU"
        torch.save(c, os.path.join(outdir, "filternorm_" + name + ".pt"))
        print("wrote", name, tuple(c["out"].shape))


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else os.path.dirname(os.path.abspath(__file__)))
