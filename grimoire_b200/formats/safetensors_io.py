"""safetensors files: zero-copy reader over the C++ mmap parser, a writer for synthetic checkpoints
and converted artifacts, and sharded-checkpoint discovery (``model.safetensors.index.json``).

Reference: SafeTensors / HFModel::discover (include/b70/safetensors.hpp:64-119,
src/safetensors.cpp:252-478)."""
from __future__ import annotations

import ctypes
import json
import struct
from pathlib import Path
from typing import Iterable, Optional

import torch

from .. import _native

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
    "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafeTensorsFile:
    def __init__(self, path: str | Path):
        self.path = str(path)
        lib = _native.host()
        lib.grm_st_open.restype = ctypes.c_void_p
        lib.grm_st_data.restype = ctypes.c_void_p
        lib.grm_st_data_len.restype = ctypes.c_int64
        err = ctypes.create_string_buffer(512)
        self._h = lib.grm_st_open(self.path.encode(), err, 512)
        if not self._h:
            raise ValueError(f"{self.path}: {err.value.decode(errors='replace')}")
        self._h = ctypes.c_void_p(self._h)
        self._lib = lib
        self.tensors: dict[str, tuple[str, tuple[int, ...], int, int]] = {}
        name = ctypes.create_string_buffer(1024)
        dt = ctypes.create_string_buffer(32)
        shape = (ctypes.c_int64 * 8)()
        b, e = ctypes.c_int64(), ctypes.c_int64()
        for i in range(lib.grm_st_count(self._h)):
            nd = lib.grm_st_info(self._h, i, name, 1024, dt, 32, shape, ctypes.byref(b), ctypes.byref(e))
            if nd < 0:
                raise ValueError(f"{self.path}: unreadable tensor record {i}")
            self.tensors[name.value.decode()] = (dt.value.decode(), tuple(shape[d] for d in range(nd)), b.value, e.value)
        self._base = lib.grm_st_data(self._h)
        self._len = lib.grm_st_data_len(self._h)

    def keys(self):
        return self.tensors.keys()

    def info(self, name: str):
        return self.tensors[name]

    def get(self, name: str) -> torch.Tensor:
        """Copy one tensor out of the mapping (the mapping itself stays read-only)."""
        dt, shape, b, e = self.tensors[name]
        if dt not in _DTYPES:
            raise ValueError(f"{name}: unsupported dtype {dt}")
        n = e - b
        if n == 0:
            return torch.empty(shape, dtype=_DTYPES[dt])
        buf = (ctypes.c_ubyte * n).from_address(self._base + b)
        t = torch.frombuffer(buf, dtype=torch.uint8).clone()
        return t.view(_DTYPES[dt]).reshape(shape)

    def metadata(self) -> dict:
        out = ctypes.create_string_buffer(1 << 20)
        n = self._lib.grm_st_metadata(self._h, out, 1 << 20)
        return json.loads(out.value.decode()) if n > 0 else {}

    def close(self):
        if self._h:
            self._lib.grm_st_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def save_file(tensors: dict[str, torch.Tensor], path: str | Path, metadata: Optional[dict] = None) -> None:
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ValueError(f"{name}: dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class CheckpointDir:
    """All shards of a HF model directory behind one name -> tensor lookup."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        idx = self.path / "model.safetensors.index.json"
        self.files: dict[str, SafeTensorsFile] = {}
        self.where: dict[str, str] = {}
        if idx.exists():
            wm = json.loads(idx.read_text())["weight_map"]
            for name, shard in wm.items():
                # a shard is a plain file name inside this directory: no separators, no parent references
                if not isinstance(shard, str) or shard in ("", ".", "..") or "/" in shard or "\\" in shard or Path(shard).name != shard:
                    raise ValueError(f"index names a shard outside the checkpoint directory: {shard!r}")
                self.where[name] = shard
        else:
            shards = sorted(p.name for p in self.path.glob("*.safetensors"))
            if not shards:
                raise FileNotFoundError(f"no safetensors files under {self.path}")
            for s in shards:
                f = self._open(s)
                for name in f.keys():
                    self.where[name] = s

    def _open(self, shard: str) -> SafeTensorsFile:
        if shard not in self.files:
            self.files[shard] = SafeTensorsFile(self.path / shard)
        return self.files[shard]

    def keys(self) -> Iterable[str]:
        return self.where.keys()

    def __contains__(self, name: str) -> bool:
        return name in self.where

    def get(self, name: str) -> torch.Tensor:
        return self._open(self.where[name]).get(name)

    def info(self, name: str):
        return self._open(self.where[name]).info(name)
