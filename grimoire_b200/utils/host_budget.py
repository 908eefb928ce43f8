"""Host memory budget: how much RAM this process may still take, container limits included, and how many per-conversation
host buffers fit beside what every local rank already holds.  Used before host-resident experts are pinned.

Reference: include/b70/host_history_budget.hpp (MemAvailable capped by the cgroup limit; slots shared by all local ranks)."""
from __future__ import annotations

from typing import Iterable, Optional

_CGROUPS = (("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory.current"),
            ("/sys/fs/cgroup/memory/memory.limit_in_bytes", "/sys/fs/cgroup/memory/memory.usage_in_bytes"))


def _read_int(path: str) -> Optional[int]:
    try:
        with open(path) as f:
            return int(f.read().split()[0])
    except (OSError, ValueError, IndexError):
        return None                      # missing file, or "max"


def host_available_ram(meminfo: str = "/proc/meminfo", cgroups: Iterable[tuple[str, str]] = _CGROUPS) -> int:
    """Bytes available to this process: MemAvailable of the machine, capped by (limit - usage) of the container's memory
    cgroup (v2 or v1) when there is one -- /proc/meminfo alone describes the whole host."""
    available = 0
    try:
        with open(meminfo) as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    available = int(line.split()[1]) * 1024
                    break
    except (OSError, ValueError, IndexError):
        available = 0
    for lim_path, cur_path in cgroups:
        cap, used = _read_int(lim_path), _read_int(cur_path)
        if cap is not None and used is not None:
            available = min(available, max(0, cap - used))
    return available


def host_slot_limit(available: int, reserve: int, slot_bytes: int, ranks: int, requested: int) -> int:
    """How many of ``requested`` host buffers of ``slot_bytes`` fit: the first one on every local rank exists already, the
    others must fit all ``ranks`` at once in what is available above ``reserve``."""
    if requested <= 1 or slot_bytes <= 0:
        return max(0, requested)
    ranks = max(1, ranks)
    extra = (available - reserve) // (slot_bytes * ranks) if available > reserve else 0
    return 1 + int(min(requested - 1, extra))
