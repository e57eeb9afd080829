"""Builds the reference's own two CUDA kernels (attn_k4_q28.cu, packbits.cu) as GPU-side checkers.
TEST INFRASTRUCTURE ONLY.

The sources are compiled where they lie in a checkout of the reference (never copied): the
directory named by the environment variable SPOTLIGHT_REFERENCE_DIR, else a `reference` directory
beside this repository. Outputs go to oracle/_ref/ only (git-ignored): two pybind11/torch
extension modules for sm_100a, importable on a machine with a B200. Without a checkout this
script does nothing. The kernels are the unmodified reference; the reference passes no arch flag
of its own (spotlight/kernel/setup.py:4-21), so the only addition is -gencode for sm_100a.

    python oracle/build_ref.py
"""
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
KERNELS = ("attn_k4_q28", "packbits")


def reference_dir():
    cand = os.environ.get("SPOTLIGHT_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "spotlight", "kernel")) else None


def build_one(ref, name):
    import torch
    from torch.utils import cpp_extension as ce
    src = os.path.join(ref, "spotlight", "kernel", name + ".cu")
    out = os.path.join(OUT, name + ".so")
    if os.path.exists(out) and os.path.getmtime(out) > os.path.getmtime(src):
        return out
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["nvcc", "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
           f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *inc, src, "-o", out, f"-L{libdir}", "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
           "-Xlinker", f"-rpath={libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the reference kernel {name} failed:\n{r.stderr[-2000:]}")
    return out


def main():
    ref = reference_dir()
    if ref is None:
        print("no reference checkout found; oracle/_ref not (re)built")
        return
    os.makedirs(OUT, exist_ok=True)
    with ThreadPoolExecutor(max_workers=2) as ex:
        for out in ex.map(lambda n: build_one(ref, n), KERNELS):
            print(out)


if __name__ == "__main__":
    main()
