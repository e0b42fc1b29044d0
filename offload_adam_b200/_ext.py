"""Build and load the native extension ``offload_adam_b200._C``.

The extension is compiled in-tree for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and imported from the package
directory.  Every build records a digest of all files under ``csrc/`` next to the
binary; ``load()`` imports a prebuilt ``_C*.so`` only when that digest matches the
sources it finds, and rebuilds (one process at a time, under a file lock) otherwise,
so an edited kernel can never run from an old binary.  On a machine with a CUDA
device a missing extension is an error: nothing silently falls back to eager
PyTorch there.
"""

from __future__ import annotations

import glob
import hashlib
import importlib
import importlib.util
import os
import sys
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG_DIR, "csrc")
_NAME = "_C"
_lock = threading.Lock()
_module = None

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--fmad=false",  # explicit rounding everywhere; kernels are memory bound
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
    "-U__CUDA_NO_HALF_OPERATORS__",
    "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC"]


def sources():
    out = sorted(glob.glob(os.path.join(_CSRC, "*.cu")) + glob.glob(os.path.join(_CSRC, "*.cpp")))
    return out


def _so_path():
    # the in-tree build writes _C.so, setup.py build_ext --inplace _C.<abi>.so: newest wins
    cands = sorted(glob.glob(os.path.join(_PKG_DIR, _NAME + "*.so")), key=os.path.getmtime, reverse=True)
    return cands[0] if cands else None


_DIGEST_FILE = os.path.join(_PKG_DIR, _NAME + ".digest")


def source_digest():
    """SHA-256 over the names and contents of every file under ``csrc/`` and the flags."""
    h = hashlib.sha256()
    deps = sorted(sources() + glob.glob(os.path.join(_CSRC, "*.h")) + glob.glob(os.path.join(_CSRC, "*.cuh")))
    for path in deps:
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()


def _stale(so):
    """True when there is no binary or it was not built from the sources present now."""
    if so is None:
        return True
    try:
        with open(_DIGEST_FILE) as f:
            return f.read().strip() != source_digest()
    except OSError:
        return True


def _import_so(path):
    spec = importlib.util.spec_from_file_location(f"{__package__}.{_NAME}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[f"{__package__}.{_NAME}"] = mod
    return mod


def build(verbose=False, force=False):
    """Compile every CUDA/C++ source of the package into ``_C.so`` (sm_100a)."""
    global _module
    import torch  # noqa: F401  (must be imported before the extension)
    from torch.utils import cpp_extension

    import fcntl

    with _lock, open(os.path.join(_PKG_DIR, "." + _NAME + ".lock"), "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)  # ranks of one job build one at a time; the others reuse
        so = _so_path()
        if so is not None and not force and not _stale(so):
            if _module is None:
                _module = _import_so(so)
            return _module
        if _module is not None:
            raise RuntimeError("offload_adam_b200: the sources under csrc/ changed after the extension was "
                               "imported; restart the process to rebuild")
        build_dir = os.path.join(_PKG_DIR, "build")
        os.makedirs(build_dir, exist_ok=True)
        os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 4)))
        cpp_extension.load(
            name=_NAME,
            sources=sources(),
            extra_cflags=CXX_FLAGS,
            extra_cuda_cflags=NVCC_FLAGS,
            extra_include_paths=[_CSRC],
            build_directory=build_dir,
            verbose=verbose,
            is_python_module=False,
        )
        built = os.path.join(build_dir, _NAME + ".so")
        target = os.path.join(_PKG_DIR, _NAME + ".so")
        if os.path.exists(target):
            os.remove(target)
        import shutil

        shutil.copy2(built, target)
        with open(_DIGEST_FILE, "w") as f:
            f.write(source_digest())
        _module = _import_so(target)
        return _module


def load(required=None):
    """Return the extension module, or None when it is absent and not required.

    ``required`` defaults to "a CUDA device is visible": GPU code paths must
    never run without the native kernels.
    """
    global _module
    if _module is not None:
        return _module
    import torch

    if required is None:
        required = torch.cuda.is_available()
    so = _so_path()
    if so is not None and not _stale(so):
        try:
            with _lock:
                if _module is None:
                    _module = _import_so(so)
            return _module
        except Exception as e:  # pragma: no cover - depends on the machine
            if required:
                raise RuntimeError(f"offload_adam_b200: failed to import {so}: {e}") from e
    try:
        return build()
    except Exception as e:
        if required:
            raise RuntimeError(
                "offload_adam_b200: the native extension is missing and could not be built "
                f"({e}); run `python -c 'import __graft_entry__ as g; g.build()'` at the repo root"
            ) from e
        return None


def loaded_path():
    return getattr(_module, "__file__", None)
