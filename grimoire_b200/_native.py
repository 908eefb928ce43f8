"""ctypes loaders for the two in-tree native libraries.

``cuda()`` returns ``libgrimoire_cuda.so`` (sm_100a kernels, flat C ABI taking raw device pointers
and a stream), ``host()`` returns ``libgrimoire_host.so`` (C++ runtime: codecs, readers, tokenizer,
scheduler core).  Both are built by ``grimoire_b200.build``; a missing CUDA library on a machine
that has a GPU is an error, never a silent fallback to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIBDIR = Path(__file__).resolve().parent / "lib"
_cuda = None
_host = None


class NativeLibraryMissing(RuntimeError):
    pass


def _load(name: str, builder: str):
    path = _LIBDIR / name
    if not path.exists():
        if os.environ.get("GRIMOIRE_NO_AUTOBUILD") == "1":
            raise NativeLibraryMissing(f"{path} is missing; run `python -m grimoire_b200.build`")
        from . import build as _build

        getattr(_build, builder)()
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)


def cuda() -> ctypes.CDLL:
    global _cuda
    if _cuda is None:
        _cuda = _load("libgrimoire_cuda.so", "build_cuda")
    return _cuda


def host() -> ctypes.CDLL:
    """The host runtime.  GRIMOIRE_HOST_LIB names another build of it (the sanitizer build of ``build_host(sanitize=True)``)."""
    global _host
    if _host is None:
        alt = os.environ.get("GRIMOIRE_HOST_LIB")
        if alt:
            _host = ctypes.CDLL(alt, mode=ctypes.RTLD_GLOBAL)
        else:
            _host = _load("libgrimoire_host.so", "build_host")
    return _host


def cuda_available() -> bool:
    """True when this process can launch the sm_100a kernels (GPU present and library built)."""
    try:
        import torch

        return torch.cuda.is_available() and (_LIBDIR / "libgrimoire_cuda.so").exists()
    except Exception:  # pragma: no cover
        return False


class KernelError(RuntimeError):
    pass


launch_count = 0   # kernel launches issued through this module (every check() follows one launch)


def check(code: int, what: str) -> None:
    """Raise on a non-zero launcher return (cudaError_t value, or -2 = unsupported shape)."""
    global launch_count
    if code == 0:
        launch_count += 1
        return
    if code == -2:
        raise KernelError(f"{what}: unsupported shape / arguments")
    if code == -1:
        raise KernelError(f"{what}: unsupported variant")
    raise KernelError(f"{what}: CUDA error {code}")


def ptr(t) -> ctypes.c_void_p:
    """Device (or host) pointer of a torch tensor, or NULL for None."""
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream_ptr() -> ctypes.c_void_p:
    import torch

    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
