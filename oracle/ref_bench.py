"""Times the REFERENCE project's own CUDA kernels (oracle/_ref/, built unmodified
by oracle/build_ref.py) beside this repository's kernels, on the same GPU, the
same seeded inputs and the same CUDA-event protocol.  TEST/MEASUREMENT
INFRASTRUCTURE ONLY.

The reference has no bfloat16 path and up-casts float16 to float32
(ddf/ddf.py:36-42), so it is timed in float32; ours is timed in float32 and in
bfloat16.  Every number is the mean over rotating buffer sets larger than L2.

    python oracle/ref_bench.py [--out results.json] [--backward]
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import ref_op  # noqa: E402

L2 = 126 * 1024 * 1024
SHAPES = [(64, 56, 1), (128, 28, 1), (256, 14, 1), (512, 7, 1), (128, 56, 2), (256, 28, 2), (512, 14, 2)]


def fwd_bytes(B, C, H, s, es, k=3):
    oh = H // s
    return es * (B * C * H * H + B * C * k * k + B * k * k * oh * oh + B * C * oh * oh)


def time_calls(fn, sets, reps=3):
    for st in sets:
        fn(*st)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        for st in sets:
            fn(*st)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (reps * len(sets))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--batch", type=int, default=128)
    args = ap.parse_args()
    from ddfnet_b200 import ddf
    dev = torch.device("cuda:0")
    B = args.batch
    rows = []
    for (C, H, s) in SHAPES:
        g = torch.Generator().manual_seed(C + H + s)
        oh = H // s
        x = torch.randn(B, C, H, H, generator=g).relu_().to(dev)
        cf = (torch.randn(B, C, 3, 3, generator=g) / 3).to(dev)
        sf = (torch.randn(B, 9, oh, oh, generator=g) / 3).to(dev)
        nb32 = fwd_bytes(B, C, H, s, 4)
        nsets = min(16, max(3, 2 * L2 // nb32 + 2))
        sets32 = [(x.clone(), cf.clone(), sf.clone()) for _ in range(nsets)]
        sets16 = [(a.bfloat16(), b.bfloat16(), c.bfloat16()) for a, b, c in sets32] * 2
        for mode in ("mul", "add"):
            with torch.no_grad():
                ref_us = time_calls(lambda a, b, c: ref_op.forward(a, b, c, 3, 1, s, mode), sets32)
                our32 = time_calls(lambda a, b, c: ddf(a, b, c, 3, 1, s, mode), sets32)
                our16 = time_calls(lambda a, b, c: ddf(a, b, c, 3, 1, s, mode), sets16)
                err = (ref_op.forward(*sets32[0], 3, 1, s, mode) - ddf(*sets32[0], 3, 1, s, mode)).abs().max().item()
            rows.append({"C": C, "H": H, "stride": s, "combine": mode,
                         "reference_f32_us": round(ref_us, 2), "ours_f32_us": round(our32, 2),
                         "ours_bf16_us": round(our16, 2),
                         "reference_f32_gbs": round(nb32 / ref_us / 1e3, 1),
                         "ours_f32_gbs": round(nb32 / our32 / 1e3, 1),
                         "ours_bf16_gbs": round(nb32 / 2 / our16 / 1e3, 1),
                         "max_abs_diff_f32": err})
            print(rows[-1], flush=True)
        del sets32, sets16
    # backward at the B=64, C=256, 28x28 configuration, float32
    Bb, C, H = 64, 256, 28
    g = torch.Generator().manual_seed(9)
    mk = lambda *shape: torch.randn(*shape, generator=g).to(dev)
    for k, d in ((3, 1), (5, 1)):
        x, cf, sf, go = mk(Bb, C, H, H).relu_(), mk(Bb, C, k, k) / 3, mk(Bb, k * k, H, H) / 3, mk(Bb, C, H, H)
        for mode in ("mul", "add"):
            def ours(go_, x_, cf_, sf_):
                xs = [t.detach().requires_grad_() for t in (x_, cf_, sf_)]
                out = ddf(*xs, k, d, 1, mode)
                out.backward(go_)
            ref_us = time_calls(lambda *a: ref_op.backward(*a, k, d, 1, mode), [(go, x, cf, sf)] * 3)
            our_us = time_calls(ours, [(go, x, cf, sf)] * 3)
            rows.append({"backward": True, "k": k, "d": d, "combine": mode,
                         "reference_bwd_f32_us": round(ref_us, 1),
                         "ours_fwd_plus_bwd_f32_us": round(our_us, 1)})
            print(rows[-1], flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
