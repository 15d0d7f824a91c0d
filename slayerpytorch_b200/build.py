"""In-tree build of the native parts (no GPU needed; nvcc cross-compiles for sm_100a).

Products, all under ``slayerpytorch_b200/lib/``:

* ``libslayer_b200.so``   the CUDA kernels behind the C ABI of ``include/slayer_b200.h``
* ``slayerCuda.*.so``     Python extension module with the reference's operator names
* ``slayerLoihiCuda.*.so``

Run ``python -m slayerpytorch_b200.build`` (add ``-v`` for ptxas resource usage, ``-f`` to
force a rebuild).
"""
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")
INCLUDE = os.path.join(ROOT, "include")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC]

# Per-file arithmetic flags.  The FIR and SRM kernels flush denormals like the reference's
# -use_fast_math build (setup.py:19) so that results can be compared bit for bit with it;
# everything else keeps IEEE behaviour.  Division and square root stay IEEE everywhere.
CUDA_SOURCES = {
    "common.cu": [],
    "shift.cu": [],
    "fir.cu": ["-ftz=true"],
    "fir_sparse.cu": ["-ftz=true"],
    "srm_spike.cu": ["-ftz=true"],
    "loihi_spike.cu": [],
    "spike_grad.cu": [],
    "delay_grad.cu": [],
    "packed.cu": [],
    "events.cu": [],
    "loss.cu": ["-ftz=true"],
    "tma.cu": [],
}
HEADERS = ["common.cuh", "tile.cuh", "tma.cuh", "fir_sparse.cuh", os.path.join(INCLUDE, "slayer_b200.h")]

MODULES = {"slayerCuda": "bindings_slayer.cpp", "slayerLoihiCuda": "bindings_loihi.cpp"}


def _newer(target, deps):
    if not os.path.isfile(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), res.stdout))
    if verbose and res.stdout.strip():
        print(res.stdout)
    return res.stdout


def nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.isfile(cand)):
            return cand
    return "nvcc"


def build_library(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    relink = force
    for src, extra in CUDA_SOURCES.items():
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src.replace(".cu", ".o"))
        if force or _newer(o, [s] + hdrs + [os.path.abspath(__file__)]):
            flags = ["-Xptxas", "-v"] if verbose else []
            _run([nvcc()] + ARCH + NVCC_COMMON + extra + flags + ["-c", s, "-o", o], verbose)
            relink = True
        objs.append(o)
    lib = os.path.join(LIBDIR, "libslayer_b200.so")
    if relink or not os.path.isfile(lib):
        _run([nvcc()] + ARCH + ["-shared", "-o", lib] + objs, verbose)
    return lib


def build_modules(force=False, verbose=False):
    """The pybind11 shims, compiled by g++ against the installed torch headers."""
    import torch
    from torch.utils import cpp_extension as ce

    ext = sysconfig.get_config_var("EXT_SUFFIX")
    inc = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], INCLUDE, CSRC, "/usr/local/cuda/include"]:
        inc += ["-isystem" if "torch" in p or "python" in p else "-I", p]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    built = []
    for name, src in MODULES.items():
        s = os.path.join(CSRC, src)
        target = os.path.join(LIBDIR, name + ext)
        deps = [s, os.path.join(CSRC, "bindings_common.h"), os.path.join(INCLUDE, "slayer_b200.h")]
        if force or _newer(target, deps):
            cmd = (["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
                    "-DTORCH_EXTENSION_NAME=" + name, "-DTORCH_API_INCLUDE_EXTENSION_H",
                    "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi]
                   + inc + [s, "-o", target,
                            "-L", LIBDIR, "-lslayer_b200", "-Wl,-rpath,$ORIGIN",
                            "-L", tlib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
                            "-ltorch_python", "-Wl,-rpath," + tlib])
            _run(cmd, verbose)
        built.append(target)
    return built


def build_all(force=False, verbose=False):
    lib = build_library(force, verbose)
    mods = build_modules(force, verbose)
    return [lib] + mods


if __name__ == "__main__":
    for path in build_all(force="-f" in sys.argv, verbose="-v" in sys.argv):
        print("built", path)
