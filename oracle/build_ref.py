"""Build the reference's own CUDA operators as a second opinion for the parity tests.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file or what it
produces; only ``tests/``, the ``build()`` step and the reference-kernel column of the
benchmark use it.

What it does, and only when the reference checkout is present (``SLAYER_REFERENCE_ROOT``
or the default location given on the command line):

* compiles ``src/cuda/slayerKernels.cu`` and ``src/cuda/slayerLoihiKernels.cu`` of the
  reference *where they lie*, unmodified, with the reference's own nvcc flags
  (``-O2 -use_fast_math``, setup.py:17-21 and :37-41) but for sm_100, under the module
  names ``slayerCuda_ref`` and ``slayerLoihiCuda_ref``;
* installs the reference's pure-Python package the way the third ``setup()`` call of its
  setup.py does (``package_dir={'slayerSNN': 'src'}``, setup.py:46-50) so that the
  "reference autograd code runs unchanged on the new operators" tests can import it.

Every output goes to ``oracle/_ref/``, which is git-ignored: no reference source is ever
committed.  The GPU machine has no reference checkout; it only uses what was built here.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def reference_root(default=None):
    root = os.environ.get("SLAYER_REFERENCE_ROOT", default)
    if root and os.path.isfile(os.path.join(root, "src", "cuda", "slayerKernels.cu")):
        return root
    return None


def build_cuda_ops(root, verbose=False):
    """Compile the two reference extensions into oracle/_ref/ (a few minutes each)."""
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    from torch.utils.cpp_extension import load

    built = []
    for name, src in (("slayerCuda_ref", "slayerKernels.cu"),
                      ("slayerLoihiCuda_ref", "slayerLoihiKernels.cu")):
        target = os.path.join(OUT, name + ".so")
        source = os.path.join(root, "src", "cuda", src)
        if os.path.isfile(target) and os.path.getmtime(target) >= os.path.getmtime(source):
            built.append(target)
            continue
        bdir = os.path.join(OUT, "build_" + name)
        os.makedirs(bdir, exist_ok=True)
        load(name=name, sources=[source], build_directory=bdir,
             extra_cflags=["-g"], extra_cuda_cflags=["-O2", "-use_fast_math"],
             extra_include_paths=[os.path.join(root, "src", "cuda")],
             is_python_module=False, verbose=verbose)
        shutil.copy2(os.path.join(bdir, name + ".so"), target)
        shutil.rmtree(bdir)          # keep only the binary
        built.append(target)
    return built


def install_python_package(root):
    """Install the reference's pure-Python package as oracle/_ref/slayerSNN/."""
    dst = os.path.join(OUT, "slayerSNN")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(dst)
    for name in sorted(os.listdir(os.path.join(root, "src"))):
        if name.endswith(".py"):
            shutil.copy2(os.path.join(root, "src", name), os.path.join(dst, name))
    return dst


def main(argv):
    root = reference_root(argv[1] if len(argv) > 1 else None)
    if root is None:
        print("reference checkout not found; nothing built")
        return 0
    os.makedirs(OUT, exist_ok=True)
    print("installed", install_python_package(root))
    for so in build_cuda_ops(root, verbose="-v" in argv):
        print("built", so)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
