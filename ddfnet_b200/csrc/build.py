"""Builds libddf_b200.so from the CUDA sources in this directory with nvcc for
sm_100a (cross-compiles without a GPU).  The library links the CUDA runtime
statically and has no other dependency, so it loads in any process.

    python -m ddfnet_b200.csrc.build [--force] [-DNAME=VALUE ...] [--out NAME]
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
SOURCES = ["abi.cu", "bwd_stream.cu", "layout.cu", "channel_branch.cu", "probe.cu", "nhwc.cu", "sfnorm.cu", "stream_inst_f32.cu", "stream_inst_f16.cu",
           "stream_inst_bf16.cu", "ring_inst_f16.cu", "ring_inst_bf16.cu", "row_inst_f16.cu", "row_inst_bf16.cu", "row_inst_f32.cu", "bwd_inst_f32.cu", "bwd_inst_f16.cu", "bwd_inst_bf16.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _deps() -> list[str]:
    return sorted(os.path.join(HERE, f) for f in os.listdir(HERE)
                  if f.endswith((".cu", ".cuh", ".inc"))) + [
        os.path.join(os.path.dirname(PKG), "include", "ddf_b200.h")]


def _fingerprint(defines: list[str]) -> str:
    h = hashlib.sha256()
    for p in _deps():
        h.update(p.encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + defines).encode())
    return h.hexdigest()


def build(force: bool = False, defines: list[str] | None = None,
          out_name: str = "libddf_b200.so", verbose: bool = False) -> str:
    defines = list(defines or [])
    out = os.path.join(PKG, out_name)
    stamp = out + ".stamp"
    fp = _fingerprint(defines)
    if not force and os.path.exists(out) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == fp:
                return out
    bdir = os.path.join(HERE, "build", out_name.replace(".so", ""))
    os.makedirs(bdir, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: str) -> str:
        obj = os.path.join(bdir, src.replace(".cu", ".o"))
        cmd = [nvcc] + NVCC_FLAGS + defines + ["-c", os.path.join(HERE, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    link = [nvcc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
            "-o", out + ".tmp"] + objs
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(out + ".tmp", out)
    with open(stamp, "w") as f:
        f.write(fp)
    return out


if __name__ == "__main__":
    args = sys.argv[1:]
    force = "--force" in args
    verbose = "-v" in args
    defs = [a for a in args if a.startswith("-D")]
    name = "libddf_b200.so"
    if "--out" in args:
        name = args[args.index("--out") + 1]
    print(build(force=force, defines=defs, out_name=name, verbose=verbose))
