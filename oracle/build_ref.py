"""Compile the reference's own CPU implementation into oracle/_ref/_C.so.

TEST INFRASTRUCTURE ONLY. The library built here is the unmodified reference (its five C++
translation units, CPU path, no CUDA) compiled from the sources where they lie; nothing is copied
into this repository and the output folder is git-ignored. It registers the reference's operators
under torch.ops.morphocore when loaded with torch.ops.load_library, so it must never be loaded in a
process that also imports morphocore_b200 (both own that operator namespace): the golden-vector
generator and the CPU-baseline runner each use it in a process of their own.

Usage: python oracle/build_ref.py --reference /path/to/reference [--force]
(or set MORPHOCORE_REFERENCE to the root of the reference checkout)
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_LIB = os.path.join(OUT_DIR, "_C.so")
CPP_DIR = "morphocore/functional/csrc/cpp"
UNITS = ["morpho_op.cpp", "reshaper.cpp", "smorph.cpp", "bindings.cpp", "smorph_scm.cpp"]


def reference_root(explicit=None):
    """Root of the reference checkout: the argument, else the MORPHOCORE_REFERENCE environment variable, else a
    folder named `reference` beside this repository; None when none of them holds the sources."""
    candidates = [explicit, os.environ.get("MORPHOCORE_REFERENCE"),
                  os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for root in candidates:
        if root and os.path.isdir(os.path.join(root, CPP_DIR)):
            return root
    return None


def build(reference=None, force=False, verbose=True):
    """Return the path of the built library, or None when neither the reference sources nor an earlier build exist."""
    reference = reference_root(reference)
    src_dir = os.path.join(reference, CPP_DIR) if reference else None
    if src_dir is None:
        return OUT_LIB if os.path.exists(OUT_LIB) else None
    if os.path.exists(OUT_LIB) and not force:
        newest = max(os.path.getmtime(os.path.join(src_dir, f)) for f in os.listdir(src_dir))
        if os.path.getmtime(OUT_LIB) > newest:
            return OUT_LIB

    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    includes = [os.path.join(reference, "morphocore/functional/csrc"), src_dir,
                os.path.join(reference, "morphocore/functional/csrc/cuda"),
                sysconfig.get_paths()["include"]] + cpp_extension.include_paths()
    # Same optimisation flags as the reference's CPU-only build (its setup.py, linux branch).
    flags = ["-O3", "-DNDEBUG", "-fopenmp", "-Wno-unused-variable", "-Wno-psabi", "-g0", "-fPIC", "-std=c++17",
             "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    inc = [f"-I{p}" for p in includes]

    def compile_unit(unit):
        obj = os.path.join(OUT_DIR, unit.replace(".cpp", ".o"))
        cmd = [cxx, "-c", os.path.join(src_dir, unit), "-o", obj] + flags + inc
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(len(UNITS), os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_unit, UNITS))

    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    link = [cxx, "-shared", "-o", OUT_LIB] + objects + ["-fopenmp", f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}",
                                                         "-lc10", "-ltorch", "-ltorch_cpu"]
    if verbose:
        print(" ".join(link), flush=True)
    subprocess.run(link, check=True)
    for obj in objects:
        os.remove(obj)
    return OUT_LIB


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=None)
    parser.add_argument("--force", action="store_true")
    args = parser.parse_args()
    path = build(args.reference, args.force)
    print(path if path else "reference sources not found; nothing built")
    sys.exit(0 if path else 1)
