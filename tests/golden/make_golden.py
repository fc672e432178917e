"""Generates the fixtures in this directory by running the REFERENCE project's
own CUDA kernels (compiled unmodified into oracle/_ref/ by oracle/build_ref.py)
on a CUDA device, on seeded inputs, in float64.  Needs a GPU:

    python tests/golden/make_golden.py [outdir]

Each fixture holds the inputs and the reference's forward output and three
gradients, so tests/test_oracle.py can pin the CPU oracle to the reference's
results without the reference being present.
"""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_op  # noqa: E402

# name: B, C, H, W, k, d, s, combine, forward version
CASES = {
    "mul_k3_d1_s1_f": (2, 6, 16, 18, 3, 1, 1, "mul", "f"),
    "mul_k3_d2_s1_o": (1, 10, 15, 15, 3, 2, 1, "mul", "o"),
    "add_k3_d1_s1_f": (2, 5, 14, 14, 3, 1, 1, "add", "f"),
    "add_k3_d1_s2_o": (2, 4, 13, 16, 3, 1, 2, "add", "o"),
    "mul_k3_d1_s2_o": (1, 7, 14, 14, 3, 1, 2, "mul", "o"),
    "mul_k5_d1_s1_o": (1, 6, 12, 10, 5, 1, 1, "mul", "o"),
    "add_k5_d2_s2_o": (2, 3, 11, 12, 5, 2, 2, "add", "o"),
    "mul_k3_d1_s1_7x7": (3, 8, 7, 7, 3, 1, 1, "mul", "o"),
}


def main(outdir):
    dev = torch.device("cuda:0")
    for i, (name, (B, C, H, W, k, d, s, m, ver)) in enumerate(sorted(CASES.items())):
        g = torch.Generator().manual_seed(4242 + i)
        x = torch.randn(B, C, H, W, generator=g, dtype=torch.float64).relu_()
        cf = torch.randn(B, C, k, k, generator=g, dtype=torch.float64) / 3
        sf = torch.randn(B, k * k, H // s, W // s, generator=g, dtype=torch.float64) / 3
        go = torch.randn(B, C, H // s, W // s, generator=g, dtype=torch.float64)
        xd, cfd, sfd, god = (t.to(dev) for t in (x, cf, sf, go))
        out = ref_op.forward(xd, cfd, sfd, k, d, s, m, ver)
        gx, gcf, gsf = ref_op.backward(god, xd, cfd, sfd, k, d, s, m)
        torch.cuda.synchronize()
        torch.save({"k": k, "d": d, "s": s, "combine": m, "version": ver, "tol": 1e-9,
                    "x": x, "cf": cf, "sf": sf, "go": go,
                    "out": out.cpu(), "gx": gx.cpu(), "gcf": gcf.cpu(), "gsf": gsf.cpu(),
                    "source": "reference CUDA kernels (theFoxofSky/ddfnet), float64, sm_100a"},
                   os.path.join(outdir, name + ".pt"))
        print("wrote", name)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
