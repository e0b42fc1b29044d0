"""Build and load the native extension ``offload_adam_b200._C``.

The extension is compiled in-tree for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and imported from the package
directory.  ``load()`` imports a prebuilt ``_C*.so`` when one is present and
builds it otherwise; ``build()`` always (re)builds when a source is newer than
the binary.  On a machine with a CUDA device a missing extension is an error:
nothing silently falls back to eager PyTorch there.
"""

from __future__ import annotations

import glob
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


def _stale(so):
    if so is None:
        return True
    t = os.path.getmtime(so)
    deps = sources() + glob.glob(os.path.join(_CSRC, "*.h")) + glob.glob(os.path.join(_CSRC, "*.cuh"))
    return any(os.path.getmtime(s) > t for s in deps)


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

    with _lock:
        so = _so_path()
        if so is not None and not force and not _stale(so):
            if _module is None:
                _module = _import_so(so)
            return _module
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
    if so is not None:
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
