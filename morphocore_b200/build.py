"""Build the native parts of the package in-tree, for sm_100a only:

  morphocore_b200/libmorphocore_b200.so   CUDA kernels + the C-ABI of include/morphocore_b200.h (nvcc)
  morphocore_b200/_C.so                   thin PyTorch C++ extension registering torch.ops.morphocore.* (g++)

Usage: python morphocore_b200/build.py [--force] [--verbose]   (run by path: it must work before the libraries exist)
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
BUILD = os.path.join(PKG, "csrc", "build")
LIB = os.path.join(PKG, "libmorphocore_b200.so")
EXT = os.path.join(PKG, "_C.so")
CUDA_UNITS = ["api.cu", "morpho_forward_f32.cu", "morpho_forward_f64.cu", "morpho_backward_f32.cu", "morpho_backward_f64.cu",
              "smorph_f32.cu", "smorph_f64.cu", "noalloc.cu", "morpho_pair_f32.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _newer(target, sources):
    return os.path.exists(target) and all(os.path.getmtime(target) > os.path.getmtime(s) for s in sources)


def _headers():
    inc = os.path.join(os.path.dirname(PKG), "include", "morphocore_b200.h")
    return [inc] + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]


def _includes(path, seen=None):
    """Files a source reaches through #include "..." (transitively): what its object depends on."""
    import re
    seen = set() if seen is None else seen
    if path in seen or not os.path.exists(path):
        return seen
    seen.add(path)
    with open(path) as f:
        for name in re.findall(r'^\s*#\s*include\s+"([^"]+)"', f.read(), flags=re.M):
            _includes(os.path.normpath(os.path.join(os.path.dirname(path), name)), seen)
    return seen


def build_cuda(force=False, verbose=False):
    os.makedirs(BUILD, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    headers = _headers()
    units = [u for u in CUDA_UNITS if os.path.exists(os.path.join(CSRC, u))]

    def compile_unit(unit):
        src, obj = os.path.join(CSRC, unit), os.path.join(BUILD, unit + ".o")
        if not force and _newer(obj, sorted(_includes(src))):
            return obj
        cmd = [nvcc, "-c", src, "-o", obj] + NVCC_FLAGS
        proc = subprocess.run(cmd, capture_output=True, text=True)
        with open(obj + ".log", "w") as f:
            f.write(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {unit}:\n{proc.stdout}\n{proc.stderr}")
        if verbose:
            print(f"compiled {unit}", flush=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(len(units), os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_unit, units))
    if force or not _newer(LIB, objects):
        subprocess.run([nvcc, "-shared", "-o", LIB] + objects + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "shared"], check=True)
    return LIB


def build_ext(force=False, verbose=False):
    import torch
    from torch.utils import cpp_extension

    src = os.path.join(CSRC, "torch_ext.cpp")
    if not force and _newer(EXT, [src, LIB] + _headers()):
        return EXT
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    includes = cpp_extension.include_paths("cuda") + [sysconfig.get_paths()["include"], os.path.join(os.path.dirname(PKG), "include")]
    cmd = [cxx, "-shared", "-fPIC", "-O2", "-std=c++17", "-o", EXT, src, "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    cmd += [f"-I{p}" for p in includes]
    cmd += [f"-L{PKG}", "-lmorphocore_b200", "-Wl,-rpath,$ORIGIN", f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}",
            "-lc10", "-lc10_cuda", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-L/usr/local/cuda/lib64", "-lcudart"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return EXT


def build_probe(force=False, verbose=False):
    """The instruction-rate probe bench.py runs for its roofline denominators (a stand-alone executable)."""
    root = os.path.dirname(PKG)
    src, out = os.path.join(root, "probe_rates.cu"), os.path.join(root, "probe_rates")
    if not force and _newer(out, [src]):
        return out
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-o", out, src], check=True)
    return out


def build(force=False, verbose=False):
    build_cuda(force, verbose)
    build_ext(force, verbose)
    build_probe(force, verbose)


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("--cuda-only", action="store_true")
    args = parser.parse_args()
    if args.cuda_only:
        print(build_cuda(args.force, args.verbose))
    else:
        build(args.force, args.verbose)
        print(LIB, EXT)
