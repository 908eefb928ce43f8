"""In-tree native build: nvcc for the sm_100a kernels, g++ for the host runtime.

Two shared libraries are produced under ``grimoire_b200/lib/``:

* ``libgrimoire_cuda.so``  every ``csrc/kernels/*.cu`` translation unit, compiled with
  ``-gencode arch=compute_100a,code=sm_100a`` (arch-specific target: tcgen05 / TMEM / TMA).
* ``libgrimoire_host.so``  every ``csrc/host/*.cpp`` file (codecs, safetensors, GGUF, tokenizer,
  scheduler core, page pool, request parsing) with plain g++ -std=c++17.

Both expose a flat ``extern "C"`` ABI and are loaded with ctypes (``grimoire_b200._native``), so
neither needs the PyTorch headers and a full rebuild takes seconds.  Objects are cached under
``build/`` keyed by a hash of the source, its local includes and the flags.

The reference builds its kernels with a shell script per target (build_b70.sh:186-238); this is
the equivalent for one target, sm_100a.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = ROOT / "build"

NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", shutil.which("g++") or "g++")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
    "-DGRM_SM100A=1",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-pthread", "-Wall", "-Wno-unused-function"]


def _hash_inputs(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    # local headers: anything under csrc/ (cheap: a few dozen small files)
    for hdr in sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.hpp")) + list(CSRC.rglob("*.h"))):
        h.update(hdr.name.encode())
        h.update(hdr.read_bytes())
    return h.hexdigest()[:24]


def _compile(src: Path, compiler: str, flags: list[str], verbose: bool) -> Path:
    OBJDIR.mkdir(exist_ok=True)
    tag = _hash_inputs(src, flags)
    obj = OBJDIR / f"{src.stem}.{tag}.o"
    if obj.exists():
        return obj
    for old in OBJDIR.glob(f"{src.stem}.*.o"):
        old.unlink()
    cmd = [compiler, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"compile failed: {src}")
    if verbose and res.stderr.strip():
        print(res.stderr, flush=True)
    return obj


def _link(objs: list[Path], out: Path, compiler: str, extra: list[str]) -> None:
    LIBDIR.mkdir(exist_ok=True)
    tmp = out.with_suffix(".tmp.so")
    cmd = [compiler, "-shared", "-o", str(tmp), *[str(o) for o in objs], *extra]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"link failed: {out}")
    tmp.replace(out)


def _stale(out: Path, objs: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(o.stat().st_mtime > t for o in objs)


def build_cuda(verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every kernel translation unit for sm_100a and link libgrimoire_cuda.so."""
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    flags = list(NVCC_FLAGS)
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile(s, NVCC, flags, verbose or ptxas_info), srcs))
    out = LIBDIR / "libgrimoire_cuda.so"
    if _stale(out, objs):
        _link(objs, out, NVCC, ["-Xcompiler", "-fPIC", "-cudart", "static"])
    return out


SANITIZE_FLAGS = ["-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-fno-sanitize-recover=undefined", "-g", "-O1"]


def sanitizer_toolchain():
    """(g++ path, libasan.so path) of a compiler that ships the AddressSanitizer runtime, or None."""
    for cxx in dict.fromkeys([CXX, "/usr/bin/g++", shutil.which("g++") or "g++"]):
        try:
            out = subprocess.run([cxx, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
        except OSError:
            continue
        if out and os.path.sep in out and os.path.exists(out):
            return cxx, os.path.realpath(out)
    return None


def build_host(verbose: bool = False, sanitize: bool = False) -> Path:
    """Compile the host-side C++ runtime (no CUDA needed) and link libgrimoire_host.so.  ``sanitize`` builds
    libgrimoire_host_asan.so with AddressSanitizer + UndefinedBehaviorSanitizer instead (the parsers of untrusted files
    run under it in the tests; load it with GRIMOIRE_HOST_LIB and the ASan runtime preloaded)."""
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    if not srcs:
        raise RuntimeError("no host sources under csrc/host")
    flags = [f for f in CXX_FLAGS if f != "-O2"] + SANITIZE_FLAGS if sanitize else CXX_FLAGS
    objdir_tag = "asan." if sanitize else ""
    cxx = CXX
    if sanitize:
        tc = sanitizer_toolchain()
        if tc is None:
            raise RuntimeError("no compiler with the AddressSanitizer runtime on this machine")
        cxx = tc[0]

    def comp(src: Path) -> Path:
        if not sanitize:
            return _compile(src, CXX, flags, verbose)
        OBJDIR.mkdir(exist_ok=True)
        obj = OBJDIR / f"{src.stem}.{objdir_tag}{_hash_inputs(src, flags)}.o"
        if not obj.exists():
            for old in OBJDIR.glob(f"{src.stem}.{objdir_tag}*.o"):
                old.unlink()
            res = subprocess.run([cxx, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
            if res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
                raise RuntimeError(f"compile failed: {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(comp, srcs))
    out = LIBDIR / ("libgrimoire_host_asan.so" if sanitize else "libgrimoire_host.so")
    if _stale(out, objs):
        _link(objs, out, cxx, ["-pthread"] + (["-fsanitize=address,undefined"] if sanitize else []))
    return out


def build_all(verbose: bool = False) -> dict[str, Path]:
    return {"host": build_host(verbose), "cuda": build_cuda(verbose)}


if __name__ == "__main__":
    v = "-v" in sys.argv
    if "--ptxas" in sys.argv:
        # registers / spills / shared memory per kernel; forces a recompile of everything
        shutil.rmtree(OBJDIR, ignore_errors=True)
        build_cuda(verbose=True, ptxas_info=True)
    else:
        for k, p in build_all(v).items():
            print(k, p)
