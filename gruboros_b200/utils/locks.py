"""Advisory file lock with a timeout (reference train.py:260-282, gossip/evolutionary_node.py:26-46)."""
from __future__ import annotations

import contextlib
import fcntl
import time


@contextlib.contextmanager
def file_lock(lock_path: str, timeout: float = 30.0, poll: float = 0.01):
    """Exclusive flock on `lock_path`; raises TimeoutError if it cannot be taken within `timeout` seconds."""
    handle = open(lock_path, "w")
    deadline = time.monotonic() + timeout
    try:
        while True:
            try:
                fcntl.flock(handle.fileno(), fcntl.LOCK_EX | fcntl.LOCK_NB)
                break
            except BlockingIOError:
                if time.monotonic() >= deadline:
                    raise TimeoutError(f"could not acquire lock {lock_path} within {timeout}s") from None
                time.sleep(min(poll, max(0.0, deadline - time.monotonic())))
        try:
            yield handle
        finally:
            fcntl.flock(handle.fileno(), fcntl.LOCK_UN)
    finally:
        handle.close()
