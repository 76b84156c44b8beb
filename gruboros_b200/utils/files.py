"""Small file helpers."""
from __future__ import annotations

import os


def read_last_line(path: str, max_line: int = 1 << 16) -> str:
    """Last non-empty line of a text file without reading the whole file (the reference carries the same helper,
    train.py:365-384, for peeking at a metrics TSV).  Returns "" for a missing or empty file."""
    try:
        size = os.path.getsize(path)
    except OSError:
        return ""
    if size == 0:
        return ""
    with open(path, "rb") as f:
        block = min(size, max_line)
        f.seek(size - block)
        tail = f.read(block)
    lines = [ln for ln in tail.splitlines() if ln.strip()]
    return lines[-1].decode("utf-8", errors="replace") if lines else ""
