"""Side channel for multi-process runs (one process per GPU): ranks read RANK / WORLD_SIZE /
LOCAL_RANK from the environment (torchrun's variables) and exchange the NCCL unique id
through a file in a directory all ranks can see."""
from __future__ import annotations

import os
import time


def dist_env():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def exchange_bytes(payload: bytes | None, rank: int, path: str, timeout_s: float = 60.0) -> bytes:
    """Rank 0 publishes ``payload`` at ``path`` (atomic rename); every rank returns it."""
    if rank == 0:
        tmp = f"{path}.tmp.{os.getpid()}"
        with open(tmp, "wb") as f:
            f.write(payload)
        os.replace(tmp, path)
        return payload
    t0 = time.time()
    while not os.path.exists(path):
        if time.time() - t0 > timeout_s:
            raise TimeoutError(f"rank {rank}: nothing published at {path} after {timeout_s} s")
        time.sleep(0.01)
    with open(path, "rb") as f:
        return f.read()
