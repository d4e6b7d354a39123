"""Side channel for multi-process runs (one process per GPU): ranks read RANK / WORLD_SIZE /
LOCAL_RANK from the environment (torchrun's variables) and exchange the NCCL unique id
through a file in a directory all ranks can see."""
from __future__ import annotations

import os
import time


def dist_env():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def run_token(explicit: str | None = None) -> str:
    """A string every rank of ONE launch agrees on and no other launch shares: the launcher's
    run id, rendezvous port and restart count plus the launcher's process id (all ranks are its
    children).  Files of the side channel carry it in their names, so whatever an earlier run -
    or an earlier attempt of this run - left in the directory is never read."""
    if explicit is not None:
        return str(explicit)
    e = os.environ
    return "-".join([e.get("TORCHELASTIC_RUN_ID", "run"), e.get("MASTER_PORT", "0"),
                     e.get("TORCHELASTIC_RESTART_COUNT", "0"), str(os.getppid())])


def publish(path: str, payload: bytes) -> None:
    """Writes ``payload`` at ``path`` so that a reader sees either nothing or all of it."""
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(payload)
    os.replace(tmp, path)


def wait_for(path: str, timeout_s: float = 60.0, who: str = "") -> bytes:
    """Blocks until ``path`` exists (published with ``publish``) and returns its bytes."""
    t0 = time.time()
    while not os.path.exists(path):
        if time.time() - t0 > timeout_s:
            raise TimeoutError(f"{who}nothing published at {path} after {timeout_s} s")
        time.sleep(0.01)
    with open(path, "rb") as f:
        return f.read()


def exchange_bytes(payload: bytes | None, rank: int, path: str, timeout_s: float = 60.0,
                   token: str | None = None) -> bytes:
    """Rank 0 publishes ``payload`` at ``path.<token>`` (atomic rename); every rank returns it.
    ``token`` (default ``run_token()``) ties the file to this launch: a file an earlier run left
    at ``path`` has another name and is ignored."""
    full = f"{path}.{run_token(token)}"
    if rank == 0:
        publish(full, payload)
        return payload
    return wait_for(full, timeout_s, f"rank {rank}: ")


def allgather_bytes(payload: bytes, rank: int, world: int, path: str, timeout_s: float = 60.0,
                    token: str | None = None) -> list[bytes]:
    """Every rank publishes ``payload`` at ``path.<token>.<rank>`` and returns the payloads of all
    ranks in rank order (the side channel for the IPC handles of ``train.PeerGroup``, and a host
    rendezvous when the payload is empty)."""
    full = f"{path}.{run_token(token)}"
    publish(f"{full}.{rank}", payload)
    return [payload if r == rank else wait_for(f"{full}.{r}", timeout_s, f"rank {rank}: ")
            for r in range(world)]


class PeerLost(RuntimeError):
    """A rank did not announce the step in time, or announced that it left."""


class StepGate:
    """Host-side gate in front of a collective step (failure detection without touching the GPU).

    Before a rank enqueues step ``k`` (whose kernels wait on the other ranks inside NCCL), it
    announces ``k`` in a file and waits until every rank has announced ``k``.  A rank that
    crashed, hung on the host or left on purpose never announces, the others give up after
    ``timeout_s`` and raise ``PeerLost`` BEFORE launching anything, so no kernel is ever left
    spinning on a partner that will not come.  Files live in a directory all ranks can see and
    carry the launch's ``token`` (``run_token()``) in their names: after a restart in the same
    directory - the recovery case that follows ``PeerLost`` - the previous run's announcements
    (a stale ``7`` or ``left 7``) have other names and cannot let a step pass with the peer
    absent.  A gate also removes its own rank's file when it is created.
    """

    def __init__(self, directory: str, rank: int, world: int, timeout_s: float = 10.0,
                 token: str | None = None):
        self.dir, self.rank, self.world, self.timeout_s = directory, rank, world, timeout_s
        self.token = run_token(token)
        self._last = 0
        os.makedirs(directory, exist_ok=True)
        try:
            os.remove(self._path(rank))
        except OSError:
            pass

    def _path(self, rank: int) -> str:
        return os.path.join(self.dir, f"step_gate.{self.token}.{rank}")

    def _write(self, text: str) -> None:
        tmp = self._path(self.rank) + f".tmp.{os.getpid()}"
        with open(tmp, "w") as f:
            f.write(text)
        os.replace(tmp, self._path(self.rank))

    def _read(self, rank: int):
        try:
            with open(self._path(rank)) as f:
                return f.read().strip()
        except OSError:
            return None

    def leave(self) -> None:
        """Announce a clean exit (call between steps, with nothing in flight).  The marker
        carries the last step this rank entered, so a slower peer still inside that step's
        rendezvous sees that this rank did reach it."""
        self._write(f"left {self._last}")

    def enter(self, step: int) -> None:
        """Announce ``step`` and wait for every rank to do the same; raises ``PeerLost``."""
        self._write(str(step))
        self._last = step
        t0 = time.time()
        pending = set(range(self.world)) - {self.rank}
        while pending:
            for r in list(pending):
                v = self._read(r)
                if v is not None and v.startswith("left"):
                    parts = v.split()
                    if len(parts) == 2 and parts[1].isdigit() and int(parts[1]) >= step:
                        pending.discard(r)          # it made this step and left afterwards
                        continue
                    raise PeerLost(f"rank {r} left before step {step}")
                if v is not None and v.isdigit() and int(v) >= step:
                    pending.discard(r)
            if pending and time.time() - t0 > self.timeout_s:
                raise PeerLost(f"ranks {sorted(pending)} did not reach step {step} within "
                               f"{self.timeout_s} s")
            if pending:
                time.sleep(0.002)
