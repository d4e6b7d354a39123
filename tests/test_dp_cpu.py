"""Host-side logic of the multi-GPU paths on CPU with world_size 2 (gloo): row sharding, the
flat gradient bucket, and the data-parallel gradient rule (sum over ranks x 1/world equals
the global-batch gradient because the reference divides by the LOCAL batch size).  The
arithmetic here is the CPU oracle's; the collective is gloo standing in for NCCL."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from novann_b200 import workloads
    from novann_b200.launch import exchange_bytes
    from novann_b200.train import flatten_params, shard_rows, unflatten_params
    from oracle import oracle_np as o

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dims = (32, 16, 8, 10)
    x, y, params = workloads.mlp_inputs(16, dims, seed=1)
    lo, hi = shard_rows(16, rank, world)
    r = o.mlp_train_step(params, x[lo:hi], y[lo:hi], 0.01)
    bucket = torch.from_numpy(flatten_params(r["grads"]))
    dist.all_reduce(bucket, op=dist.ReduceOp.SUM)
    avg = unflatten_params((bucket.numpy() * np.float32(1.0 / world)).astype(np.float32), dims)
    full = o.mlp_train_step(params, x, y, 0.01)
    for a, b in zip(avg, full["grads"]):
        assert a.shape == b.shape
        assert np.max(np.abs(a - b)) <= 1e-6 * max(1e-30, np.max(np.abs(b))) + 1e-9
    # per-tensor FP8 over row shards: max of the partial amax values == amax of the whole tensor
    t = workloads.fp8_input(8, 64, seed=3)
    part = torch.tensor([float(o.amax_f32(t[rank * 4:(rank + 1) * 4]))])
    dist.all_reduce(part, op=dist.ReduceOp.MAX)
    assert np.float32(part.item()) == o.amax_f32(t)
    # the unique-id side channel
    got = exchange_bytes(b"x" * 128 if rank == 0 else None, rank, os.path.join(tmpdir, "id"))
    assert got == b"x" * 128
    dist.destroy_process_group()


def test_world_size_2_gloo(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)


def test_shard_rows_and_bucket_layout():
    sys.path.insert(0, ROOT)
    from novann_b200 import workloads
    from novann_b200.train import flatten_params, shard_rows, unflatten_params
    assert [shard_rows(16384, r, 8) for r in (0, 7)] == [(0, 2048), (14336, 16384)]
    with pytest.raises(ValueError):
        shard_rows(10, 0, 4)
    _, _, params = workloads.mlp_inputs(4, (784, 256, 128, 10), seed=0)
    flat = flatten_params(params)
    assert flat.size == 235146                       # the bucket the all-reduce moves
    back = unflatten_params(flat, (784, 256, 128, 10))
    assert all(np.array_equal(a, b) for a, b in zip(back, params))
    assert [b.shape for b in back] == [(256, 784), (1, 256), (128, 256), (1, 128), (10, 128), (1, 10)]


def _gate_worker(rank, tmpdir, q):
    sys.path.insert(0, ROOT)
    from novann_b200.launch import PeerLost, StepGate
    gate = StepGate(tmpdir, rank, 2, timeout_s=60.0)   # generous: process start-up times differ
    gate.enter(1)                      # both ranks make step 1
    gate.timeout_s = 2.0
    if rank == 1:
        gate.leave()                   # rank 1 leaves between steps, nothing in flight
        q.put((rank, "left"))
        return
    try:
        gate.enter(2)
        q.put((rank, "no error"))
    except PeerLost as e:
        q.put((rank, f"PeerLost: {e}"))


def _silent_worker(rank, tmpdir, q):
    sys.path.insert(0, ROOT)
    from novann_b200.launch import PeerLost, StepGate
    gate = StepGate(tmpdir, rank, 2, timeout_s=1.0)
    if rank == 1:
        return                         # never joins (a rank that died before the first step)
    import time
    t0 = time.time()
    try:
        gate.enter(1)
        q.put((rank, "no error"))
    except PeerLost as e:
        q.put((rank, f"PeerLost after {time.time() - t0:.1f}s: {e}"))


def test_step_gate_detects_a_rank_that_left_or_never_joined(tmp_path):
    """Failure detection happens on the host, before a collective step is enqueued: no kernel
    is ever left waiting for a partner that will not come."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    for worker, sub in ((_gate_worker, "a"), (_silent_worker, "b")):
        q = ctx.Queue()
        d = str(tmp_path / sub)
        ps = [ctx.Process(target=worker, args=(r, d, q)) for r in range(2)]
        for p in ps:
            p.start()
        for p in ps:
            p.join(30)
            assert p.exitcode == 0
        msgs = dict(q.get(timeout=5) for _ in range(1 if worker is _silent_worker else 2))
        assert msgs[0].startswith("PeerLost"), msgs


def test_step_gate_peer_that_left_right_after_a_step_still_counts_for_that_step(tmp_path):
    """A fast rank may finish step k and leave before a slow rank has looked: the slow rank must
    still pass step k's rendezvous and only fail at step k + 1."""
    from novann_b200.launch import PeerLost, StepGate
    fast = StepGate(str(tmp_path), 1, 2, timeout_s=0.5)
    slow = StepGate(str(tmp_path), 0, 2, timeout_s=0.5)
    fast._write("1")
    fast._last = 1
    fast.leave()
    slow.enter(1)
    with pytest.raises(PeerLost, match="left before step 2"):
        slow.enter(2)


def test_step_gate_ignores_what_an_earlier_run_left_in_the_directory(tmp_path):
    """Restart in the same directory (the recovery case after PeerLost): the first run reached
    step 3 and one rank even left cleanly; the second run has only rank 0 alive.  Neither the
    stale ``3`` nor the stale ``left 3`` may let rank 0 pass step 1."""
    from novann_b200.launch import PeerLost, StepGate, exchange_bytes
    d = str(tmp_path)
    a, b = StepGate(d, 0, 2, timeout_s=0.5, token="run1"), StepGate(d, 1, 2, timeout_s=0.5, token="run1")
    for step in (1, 2, 3):
        a._write(str(step)); a._last = step
        b._write(str(step)); b._last = step
        a.enter(step)
        b.enter(step)
    b.leave()
    again = StepGate(d, 0, 2, timeout_s=0.5, token="run2")
    with pytest.raises(PeerLost, match="did not reach step 1"):
        again.enter(1)
    # same token, new gate object (a worker restarted by the same launcher): its own stale
    # announcement is removed on creation
    a2 = StepGate(d, 0, 2, timeout_s=0.2, token="run1")
    assert a2._read(0) is None
    # the id side channel: a file of an earlier launch is not returned to the other ranks
    exchange_bytes(b"old" * 8, 0, os.path.join(d, "nccl_id"), token="run1")
    with pytest.raises(TimeoutError):
        exchange_bytes(None, 1, os.path.join(d, "nccl_id"), timeout_s=0.3, token="run2")
    exchange_bytes(b"new" * 8, 0, os.path.join(d, "nccl_id"), token="run2")
    assert exchange_bytes(None, 1, os.path.join(d, "nccl_id"), timeout_s=0.3, token="run2") == b"new" * 8


def _allgather_worker(rank, world, tmpdir, q):
    sys.path.insert(0, ROOT)
    from novann_b200.launch import allgather_bytes
    got = allgather_bytes(bytes([rank]) * 64, rank, world, os.path.join(tmpdir, "handles"), token="t1")
    again = allgather_bytes(b"", rank, world, os.path.join(tmpdir, "rendezvous"), token="t1")
    q.put((rank, got, again))


def test_allgather_bytes_returns_every_ranks_payload_in_rank_order(tmp_path):
    """The side channel of the peer-memory step (64-byte IPC handles, and an empty payload as a
    host rendezvous): three processes, every rank gets the same list."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_allgather_worker, args=(r, 3, str(tmp_path), q)) for r in range(3)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=60) for _ in range(3))
    for p in ps:
        p.join(timeout=30)
    for rank, got, again in res:
        assert got == [bytes([r]) * 64 for r in range(3)]
        assert again == [b"", b"", b""]
