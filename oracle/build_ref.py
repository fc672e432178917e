"""Builds the reference project's own CUDA extension modules (ddf_mul_ext,
ddf_mul_faster_ext, ddf_add_ext, ddf_add_faster_ext) from the sources where they
lie under the reference checkout, for sm_100a, into oracle/_ref/ .

TEST INFRASTRUCTURE ONLY.  No reference source is copied or modified: the
sources are compiled in place with one force-included header (ref_shim.h) that
restores a PyTorch dispatch overload they rely on.  The reference's own build
(ddf/setup.py:8-67, torch CUDAExtension) is not run; this is the same list of
translation units and the same three -D__CUDA_NO_HALF* flags, passed to nvcc /
g++ directly.

Only runs where the reference checkout exists; the built modules travel.

    python oracle/build_ref.py [/path/to/reference]
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

MODULES = {
    "ddf_mul_ext": ["src/ddf_mul_ext.cpp", "src/cuda/ddf_mul_cuda.cpp", "src/cuda/ddf_mul_cuda_kernel.cu"],
    "ddf_mul_faster_ext": ["src/ddf_mul_faster_ext.cpp", "src/cuda/ddf_mul_faster_cuda.cpp",
                           "src/cuda/ddf_mul_faster_cuda_kernel.cu"],
    "ddf_add_ext": ["src/ddf_add_ext.cpp", "src/cuda/ddf_add_cuda.cpp", "src/cuda/ddf_add_cuda_kernel.cu"],
    "ddf_add_faster_ext": ["src/ddf_add_faster_ext.cpp", "src/cuda/ddf_add_faster_cuda.cpp",
                           "src/cuda/ddf_add_faster_cuda_kernel.cu"],
}


def build(ref_root: str = "/root/reference", force: bool = False) -> bool:
    ddf_dir = os.path.join(ref_root, "ddf")
    if not os.path.isdir(ddf_dir):
        return False
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT, exist_ok=True)
    inc = ce.include_paths() + [sysconfig.get_paths()["include"]]
    incs = sum((["-I", i] for i in inc), [])
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    shim = os.path.join(HERE, "ref_shim.h")

    def compile_one(job):
        mod, src = job
        obj = os.path.join(OUT, f"{mod}__{os.path.basename(src)}.o")
        common = ["-DWITH_CUDA", f"-DTORCH_EXTENSION_NAME={mod}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                  abi, "-include", shim] + incs
        if src.endswith(".cu"):
            cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
                   "-Xcompiler", "-fPIC", "-w", "-D__CUDA_NO_HALF_OPERATORS__",
                   "-D__CUDA_NO_HALF_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"] + common
        else:
            cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-w", "-I", "/usr/local/cuda/include"] + common
        cmd += ["-c", os.path.join(ddf_dir, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)}\n{r.stderr[-4000:]}")
        return mod, obj

    todo = [m for m in MODULES if force or not os.path.exists(os.path.join(OUT, m + ".so"))]
    jobs = [(m, s) for m in todo for s in MODULES[m]]
    objs: dict[str, list[str]] = {m: [] for m in todo}
    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        for mod, obj in ex.map(compile_one, jobs):
            objs[mod].append(obj)
    for mod in todo:
        so = os.path.join(OUT, mod + ".so")
        cmd = ["g++", "-shared", "-o", so] + objs[mod] + [
            "-L", torch_lib, "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda",
            "-ltorch_cuda", "-L", "/usr/local/cuda/lib64", "-lcudart",
            f"-Wl,-rpath,{torch_lib}"]
        subprocess.run(cmd, check=True)
        for o in objs[mod]:
            os.remove(o)
    return True


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    print("built" if build(root, force="--force" in sys.argv) else "reference checkout not found")
