"""Locate and import the optional reference artefacts used as a second opinion by GPU tests.

``oracle/_ref/`` (git-ignored, produced by ``oracle/build_ref.py`` where a reference checkout
exists) may hold the reference's CUDA operators compiled for sm_100 (``slayerCuda_ref``,
``slayerLoihiCuda_ref``) and its installed pure-Python package (``slayerSNN``).  Tests that
need them skip when they are absent.
"""
import importlib
import importlib.machinery
import importlib.util
import os
import sys
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def load_ref_extension(name):
    path = os.path.join(REF, name + ".so")
    if not os.path.isfile(path):
        return None
    if name in sys.modules:
        return sys.modules[name]
    import torch  # noqa: F401
    loader = importlib.machinery.ExtensionFileLoader(name, path)
    spec = importlib.util.spec_from_loader(name, loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    sys.modules[name] = mod
    return mod


def load_reference_python(slayer_cuda, slayer_loihi_cuda, alias):
    """Import the reference's slayer.py / slayerLoihi.py / spikeLoss.py UNCHANGED, bound to the
    given operator modules, under the package name `alias` (the package __init__ is not run: it
    needs matplotlib and an older NumPy)."""
    src = os.path.join(REF, "slayerSNN")
    if not os.path.isfile(os.path.join(src, "slayer.py")):
        return None
    saved = {k: sys.modules.get(k) for k in ("slayerCuda", "slayerLoihiCuda")}
    sys.modules["slayerCuda"], sys.modules["slayerLoihiCuda"] = slayer_cuda, slayer_loihi_cuda
    try:
        pkg = types.ModuleType(alias)
        pkg.__path__ = [src]
        sys.modules[alias] = pkg
        mods = types.SimpleNamespace(
            slayer=importlib.import_module(alias + ".slayer"),
            loihi=importlib.import_module(alias + ".slayerLoihi"),
            loss=importlib.import_module(alias + ".spikeLoss"))
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    return mods
