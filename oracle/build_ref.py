"""Build recipe for the GPU witness: the reference's own ``fast_jl`` extension.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this.

The reference kernel (``fast_jl/fast_jl.cu`` and the ``.cuh`` headers next to
it) is compiled *where it lies* in the reference checkout, with one explicit
``nvcc`` command (the reference's ``setup.py`` is not run), and its only
output is ``oracle/_ref/fast_jl.so``.  No reference source is copied into
tracked files.

The resulting module is the bit-exactness witness for the projection matrix:
GPU tests project one-hot rows through it and through the new kernel and
compare the bits, and ``tests/golden/make_fastjl_golden.py`` uses it to
produce the committed golden vectors.

``install_python_package`` is the second recipe: the reference's pure-Python
package, installed by pip into the git-ignored ``baseline/_ref``, which lets one
GPU test run the unmodified ``TRAKer`` on top of this library.

The reference checkout is found through ``--reference``, the environment variable
``TRAK_REFERENCE_DIR`` or, failing both, a directory named ``reference`` next to this
repository.

Usage:  python oracle/build_ref.py [--reference /path/to/reference]
"""
import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "fast_jl.so")


def default_reference() -> str:
    """Where the reference checkout is expected when no path is given."""
    env = os.environ.get("TRAK_REFERENCE_DIR")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference: str = None, force: bool = False) -> str | None:
    """Compile the reference extension; returns the path or None if the
    reference checkout is absent (e.g. on a machine that only has the
    prebuilt file)."""
    reference = reference or default_reference()
    src = os.path.join(reference, "fast_jl", "fast_jl.cu")
    if not os.path.exists(src):
        return OUT if os.path.exists(OUT) else None
    if os.path.exists(OUT) and not force and os.path.getmtime(OUT) >= os.path.getmtime(src):
        return OUT
    import torch  # noqa: F401  (only to locate headers and libraries)
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT_DIR, exist_ok=True)
    inc = ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    libdirs = ce.library_paths("cuda")
    cmd = ["nvcc", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-DTORCH_EXTENSION_NAME=fast_jl", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=1",
           "--expt-relaxed-constexpr",
           # the reference ships PTX for sm_70; build that plus native sm_100
           "-gencode", "arch=compute_70,code=compute_70",
           "-gencode", "arch=compute_100,code=sm_100"]
    for i in inc:
        cmd += ["-isystem", i]
    for l in libdirs:
        cmd += ["-L" + l, "-Xlinker", "-rpath=" + l]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-lcudart", src, "-o", OUT]
    print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return OUT


PY_DIR = os.path.join(os.path.dirname(HERE), "baseline", "_ref")


def install_python_package(reference: str = None, force: bool = False) -> str | None:
    """Install the reference's pure-Python package (``trak``) with pip, offline and without
    dependencies, into the git-ignored ``baseline/_ref`` directory, so that a GPU test can drive
    this library through the unmodified ``TRAKer``.  Returns the directory, or None when neither
    the checkout nor an earlier install is there."""
    reference = reference or default_reference()
    done = os.path.isdir(os.path.join(PY_DIR, "trak"))
    if not os.path.exists(os.path.join(reference, "setup.py")) or (done and not force):
        return PY_DIR if done else None
    cmd = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
           "--upgrade", "--target", PY_DIR, reference]
    print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return PY_DIR


def load():
    """Import the built witness as module ``fast_jl`` (None when not built)."""
    if not os.path.exists(OUT):
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location("fast_jl", OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference())
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    p = build(a.reference, a.force)
    print("built:" if p else "reference not present; nothing built", p)
    q = install_python_package(a.reference, a.force)
    print("python package:" if q else "reference not present; nothing installed", q)
    sys.exit(0)
