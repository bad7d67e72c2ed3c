"""Compiles the reference project's OWN extension sources, unmodified, for sm_100a -- TEST INFRASTRUCTURE ONLY.

    QVB8_REFERENCE_ROOT=<checkout of the reference project> python oracle/build_ref.py [--force] [qvb8_cuda|qvb8r_cuda ...]

Outputs go to ``oracle/_ref/`` (git-ignored) and nowhere else:

    oracle/_ref/qvb8_cuda.so     src/qv_band/formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu          (-O3 --use_fast_math)
    oracle/_ref/qvb8r_cuda.so    src/qv_band/formats/qvb8r/backends/cuda_qvb8r/qvb8r_cuda.cu + qvb8r_cpu.cpp  (-O3, OpenMP)

with the flags the reference's own loaders pass (formats/qvb8/module.py:35-36, formats/qvb8r/module.py:30-33); the
sources are compiled where they lie, nothing is copied.  The two modules are torch extensions (pybind11 + ATen), so the
build goes through ``torch.utils.cpp_extension.load`` with the arch forced to 10.0a; each takes 4-5 minutes.  The tests
use them as the second parity target (the reference's own kernels on the same GPU) and the benchmark as a same-box speed
baseline; the CPU functions of ``qvb8r_cuda`` (embed_rows / encode / row_hist) also generate the QVB8R golden fixtures.

Without the reference checkout (for instance on a GPU box) this script does nothing and prebuilt files are used as is.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

MODULES = {
    "qvb8_cuda": dict(
        sources=["src/qv_band/formats/qvb8/backends/cuda_qvb8/qvb8_cuda.cu"],
        cflags=["-O3"], cuda_cflags=["-O3", "--use_fast_math"], ldflags=[]),
    "qvb8r_cuda": dict(
        sources=["src/qv_band/formats/qvb8r/backends/cuda_qvb8r/qvb8r_cuda.cu",
                 "src/qv_band/formats/qvb8r/backends/cuda_qvb8r/qvb8r_cpu.cpp"],
        cflags=["-O3", "-fopenmp"], cuda_cflags=["-O3"], ldflags=["-fopenmp"]),
}


def reference_root() -> str | None:
    """The reference checkout: $QVB8_REFERENCE_ROOT, else a directory named ``reference`` beside this repository."""
    cands = [os.environ.get("QVB8_REFERENCE_ROOT"), os.path.join(os.path.dirname(HERE), os.pardir, "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "src", "qv_band")):
            return os.path.abspath(c)
    return None


def _key(root: str, spec: dict) -> str:
    import torch
    h = hashlib.sha256()
    for s in spec["sources"]:
        with open(os.path.join(root, s), "rb") as fh:
            h.update(fh.read())
    h.update(json.dumps([spec["cflags"], spec["cuda_cflags"], spec["ldflags"], torch.__version__]).encode())
    return h.hexdigest()


def build_one(name: str, root: str, force: bool = False, verbose: bool = False) -> str:
    spec = MODULES[name]
    so = os.path.join(OUT, name + ".so")
    stamp = os.path.join(OUT, name + ".key")
    key = _key(root, spec)
    if not force and os.path.exists(so) and os.path.exists(stamp) and open(stamp).read().strip() == key:
        return so
    os.makedirs(OUT, exist_ok=True)
    work = os.path.join(OUT, "_obj_" + name)
    os.makedirs(work, exist_ok=True)
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    if os.path.isfile("/usr/bin/g++"):          # the distribution's compiler carries libgomp
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    from torch.utils import cpp_extension
    cpp_extension.load(name=name, sources=[os.path.join(root, s) for s in spec["sources"]],
                       extra_cflags=spec["cflags"], extra_cuda_cflags=spec["cuda_cflags"],
                       extra_ldflags=spec["ldflags"], build_directory=work, verbose=verbose, is_python_module=False)
    built = os.path.join(work, name + ".so")
    os.replace(built, so)
    with open(stamp, "w") as fh:
        fh.write(key)
    return so


def build(names=None, force: bool = False, verbose: bool = False) -> list[str]:
    root = reference_root()
    if root is None:
        return []
    return [build_one(n, root, force, verbose) for n in (names or list(MODULES))]


def load(name: str):
    """Import a built reference module from oracle/_ref (None when it is not there)."""
    so = os.path.join(OUT, name + ".so")
    if not os.path.exists(so):
        return None
    import importlib.util
    import torch  # noqa: F401  (the module links against torch)
    spec = importlib.util.spec_from_file_location(name, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    done = build(args or None, force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print("\n".join(done) if done else "reference checkout not found: nothing built")
