"""The host C++ runtime (GGUF / safetensors parsers, tokenizer, scheduler core) under AddressSanitizer and
UndefinedBehaviorSanitizer: the format, tokenizer and scheduler-core tests plus a set of damaged files run in a child
interpreter that loads the sanitizer build (the reference builds its GGUF tests the same way, Makefile:72-77)."""
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _asan_runtime():
    from grimoire_b200.build import sanitizer_toolchain

    tc = sanitizer_toolchain()
    return tc[1] if tc else None


@pytest.mark.skipif(_asan_runtime() is None, reason="no AddressSanitizer runtime on this machine")
def test_host_runtime_is_clean_under_asan_ubsan(tmp_path):
    from grimoire_b200.build import build_host

    lib = build_host(sanitize=True)
    env = dict(os.environ, LD_PRELOAD=_asan_runtime(), GRIMOIRE_HOST_LIB=str(lib), PYTHONPATH=str(ROOT),
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1:verify_asan_link_order=0", UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    # 1) the ordinary tests of everything that lives in the host library
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", "tests/test_gguf.py", "tests/test_tokenizer.py",
                        "tests/test_formats.py", "tests/test_checkpoint.py", "tests/test_scheduler.py::test_core_hold_then_batched_admission_then_interleave",
                        "tests/test_scheduler.py::test_core_cancel_and_retire_free_slots"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    # 2) damaged containers: every one must be refused with an error, never crash or read out of bounds
    fuzz = tmp_path / "fuzz.py"
    fuzz.write_text('''
import json, random, struct, sys
from pathlib import Path
import torch
from grimoire_b200.formats import gguf
from grimoire_b200.formats.safetensors_io import SafeTensorsFile, save_file
d = Path(sys.argv[1])
save_file({"a": torch.arange(64, dtype=torch.float32).reshape(8, 8), "b": torch.ones(5, dtype=torch.bfloat16)}, d / "ok.safetensors")
good = (d / "ok.safetensors").read_bytes()
rng = random.Random(0)
refused = 0
for i in range(200):
    b = bytearray(good)
    for _ in range(rng.randint(1, 6)):
        b[rng.randrange(0, min(len(b), 200))] = rng.randrange(256)
    if i % 5 == 0:
        b = b[: rng.randrange(8, len(b))]
    (d / "bad.safetensors").write_bytes(bytes(b))
    try:
        f = SafeTensorsFile(d / "bad.safetensors")
        for k in list(f.keys()):
            f.get(k)
    except Exception:
        refused += 1
# GGUF: huge dims (element count overflow), absurd alignment, truncated records
def gguf_bytes(dims, align, off=0, typ=0):
    s = b"GGUF" + struct.pack("<IQQ", 3, 1, 1)
    k = b"general.alignment"
    s += struct.pack("<Q", len(k)) + k + struct.pack("<II", 4, align)
    n = b"t"
    s += struct.pack("<Q", len(n)) + n + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", x) for x in dims)
    s += struct.pack("<IQ", typ, off)
    return s + b"\\0" * 256
cases = [gguf_bytes([2**33, 2**33], 32), gguf_bytes([2**62, 8], 32), gguf_bytes([4, 4], 0), gguf_bytes([4, 4], 3), gguf_bytes([4, 4], 2**31),
         gguf_bytes([4, 4], 32, off=2**63), gguf_bytes([4, 4], 32, off=2**64 - 8), gguf_bytes([4, 4], 32)[:40], gguf_bytes([4, 4], 32, typ=999)]
for i, c in enumerate(cases):
    (d / "bad.gguf").write_bytes(c)
    try:
        g = gguf.GGUFFile(str(d / "bad.gguf"))
        for name in list(g.tensors):
            g.tensor(name)
        g.close()
    except Exception:
        refused += 1
print("refused", refused)
''')
    r = subprocess.run([sys.executable, str(fuzz), str(tmp_path)], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "refused" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-4000:]
