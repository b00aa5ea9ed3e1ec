"""Builds the CUDA shared library in-tree (``bps_nav_b200/libbpsn.so``) with nvcc for sm_100a.

Run as ``python -m bps_nav_b200.build``.  nvcc cross-compiles without a GPU.
FMA contraction is disabled (``-fmad=false``): the navigation-mesh queries and
the GAE scan must round every operation like the scalar CPU reference does.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libbpsn.so")
SOURCES = ["bpsn.cu", "navmesh_host.cpp", "dataset_host.cpp"]


def _nvcc():
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build libbpsn.so")
    return cand


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)
            if f.endswith((".cu", ".cuh", ".cpp", ".h"))]
    deps.append(os.path.join(HERE, "..", "include", "bpsn.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def _ext_path():
    import sysconfig
    return os.path.join(HERE, "_bpsn_fast" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_pyext(force=False):
    """The CPython binding of the per-step calls (csrc/pyext.c), linked against libbpsn.so in
    this directory.  Optional: without Python's headers or a C compiler the package uses ctypes
    for those calls too.  Returns the module's path or None."""
    import sysconfig
    out = _ext_path()
    src = os.path.join(CSRC, "pyext.c")
    inc = sysconfig.get_paths()["include"]
    cc = shutil.which("gcc") or shutil.which("cc")
    if not cc or not os.path.exists(os.path.join(inc, "Python.h")):
        return None
    if not force and os.path.exists(out) and os.path.getmtime(out) >= max(
            os.path.getmtime(src), os.path.getmtime(LIB)):
        return out
    cmd = [cc, "-O2", "-fPIC", "-shared", f"-I{inc}", src, f"-L{HERE}", "-l:libbpsn.so",
           "-Wl,-rpath,$ORIGIN", "-o", out]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write("could not build the _bpsn_fast module (ctypes will be used):\n" +
                         res.stderr)
        return None
    return out


def build(force=False, verbose=False):
    lib = _build_lib(force, verbose)
    build_pyext(force)
    return lib


def _build_lib(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    cmd = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-fmad=false", "-Xcompiler", "-fPIC", "-shared",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-lz", "-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
