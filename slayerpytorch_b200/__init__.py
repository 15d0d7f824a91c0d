"""slayerpytorch_b200 — Blackwell (sm_100a) implementation of SLAYER's spiking-neuron hot path.

The package holds

* ``csrc/``    hand-written CUDA kernels behind a C ABI (``include/slayer_b200.h``) and the
               pybind11 shims that export them under the reference's module names;
* ``lib/``     the built binaries (``libslayer_b200.so``, ``slayerCuda``, ``slayerLoihiCuda``);
* ``layer``    a host-side mirror of the reference's ``spikeLayer`` hot-path methods
               (psp, spike, delay, delayShift, spikeLoihi) with fused backward passes;
* ``capi``     a ctypes view of the C ABI for callers that hold raw device pointers.

``import slayerpytorch_b200`` makes ``import slayerCuda`` / ``import slayerLoihiCuda`` resolve
to the new binaries, which is all the reference's own ``slayer.py`` / ``slayerLoihi.py`` need
to run on them unchanged.  There is no CPU fallback: if the binaries are missing, importing
the operators fails.
"""
import os
import sys

__version__ = "0.1.0"

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(PKG_DIR, "lib")


def lib_dir():
    return LIB_DIR


def install():
    """Put the built extension modules first on ``sys.path`` (idempotent)."""
    if LIB_DIR not in sys.path:
        sys.path.insert(0, LIB_DIR)
    return LIB_DIR


def load_ops():
    """Import and return ``(slayerCuda, slayerLoihiCuda)``; raises if they are not built or
    if the names resolve to some other implementation."""
    install()
    import torch  # noqa: F401  (the extension modules link against libtorch)
    try:
        import slayerCuda
        import slayerLoihiCuda
    except ImportError as e:
        raise ImportError(
            "slayerpytorch_b200: the CUDA extension modules are not built "
            "(run `python -m slayerpytorch_b200.build`); there is no CPU fallback") from e
    for m in (slayerCuda, slayerLoihiCuda):
        if getattr(m, "backend", None) != "slayer_b200":
            raise ImportError("module %s at %s is not the slayer_b200 build"
                              % (m.__name__, getattr(m, "__file__", "?")))
    return slayerCuda, slayerLoihiCuda


install()
