"""Data-parallel training step on two GPUs: one process per GPU, row-sharded batch, one NCCL
all-reduce of the flat gradient bucket, 1/world folded into the SGD kernel.  The result must
equal the single-process step on the whole batch (the reference's semantics).  Needs two
devices; on a one-GPU box the test reports itself skipped (there is no other path to fall to).
"""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, tmpdir):
    sys.path.insert(0, ROOT)
    from novann_b200 import workloads
    from novann_b200.launch import exchange_bytes
    from novann_b200.train import Communicator, MLPTrainStep, shard_rows
    from oracle import oracle_np as o

    uid = Communicator.make_unique_id() if rank == 0 else None
    uid = exchange_bytes(uid, rank, os.path.join(tmpdir, "nccl_id"))
    comm = Communicator(uid, rank, world, device=rank)
    dims = (784, 256, 128, 10)
    x, y, params = workloads.mlp_inputs(128, dims, seed=0)
    lo, hi = shard_rows(128, rank, world)
    st = MLPTrainStep(params, hi - lo, 0.01, device=rank, comm=comm)
    cur = params
    for s in range(3):
        xs, ys, _ = workloads.mlp_inputs(128, dims, seed=20 + s)
        st.step(xs[lo:hi], ys[lo:hi])
        cur = o.mlp_train_step(cur, xs, ys, 0.01)["params"]
    for a, b in zip(st.params(), cur):
        err = np.max(np.abs(a - b)) / max(1e-30, np.max(np.abs(b)))
        assert err <= 1e-5, (rank, err)
    # the same step with forward / loss / backward replayed from a CUDA graph and the all-reduce
    # and the SGD kernel enqueued after it (the collective itself is never captured)
    st.capture()
    assert st._graph_is_partial
    for s in range(2):
        xs, ys, _ = workloads.mlp_inputs(128, dims, seed=40 + s)
        st.step(xs[lo:hi], ys[lo:hi])
        cur = o.mlp_train_step(cur, xs, ys, 0.01)["params"]
    for a, b in zip(st.params(), cur):
        err = np.max(np.abs(a - b)) / max(1e-30, np.max(np.abs(b)))
        assert err <= 2e-5, (rank, err)
    comm.close()


def test_two_rank_step_equals_global_batch_step(gpu, tmp_path):
    from novann_b200.device import device_count
    if device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, str(tmp_path)), nprocs=2, join=True)


def _fp8_shard_worker(rank, world, tmpdir):
    sys.path.insert(0, ROOT)
    from novann_b200 import quant, workloads
    from novann_b200.device import DeviceBuffer
    from novann_b200.launch import publish, wait_for
    from novann_b200.train import shard_rows
    from oracle import oracle_np as o

    x = workloads.fp8_input(1024, 2048, seed=9)               # every rank can rebuild the tensor
    lo, hi = shard_rows(1024, rank, world)
    shard = np.ascontiguousarray(x[lo:hi])
    part = quant.amax(shard, device=rank)                     # this rank's partial amax (one float)
    # the one scalar exchange of the path: max-combine on the host, no collective
    publish(os.path.join(tmpdir, f"amax.{rank}"), np.float32(part).tobytes())   # atomic: all 4 bytes or no file
    vals = []
    for r in range(world):
        vals.append(np.frombuffer(wait_for(os.path.join(tmpdir, f"amax.{r}")), np.float32)[0])
    amax = np.float32(max(vals))
    for fmt in ("e4m3", "e5m2"):
        d = DeviceBuffer.from_numpy(shard, rank)
        q = DeviceBuffer(shard.size, rank)
        asi = DeviceBuffer(12, rank)
        a_in = DeviceBuffer.from_numpy(np.array([amax], np.float32), rank)
        quant.quantize_fp8_tensor_device(q, asi, d, shard.size, fmt, amax_in=a_in)
        codes = q.to_numpy(np.uint8, shard.shape)
        want, scale, inv = o.quantize_fp8_tensor(x, fmt)      # the one-GPU (whole tensor) result
        assert np.array_equal(codes, want[lo:hi]), (rank, fmt)
        assert asi.to_numpy(np.float32, (3,))[1] == scale
        back = quant.dequantize_fp8(codes, scale, fmt, device=rank)
        assert np.array_equal(back.view(np.uint32), o.dequantize_fp8(want[lo:hi], scale, fmt).view(np.uint32))


def test_two_rank_fp8_row_shards_equal_whole_tensor(gpu, tmp_path):
    """FP8 per-tensor quantisation over row shards on two GPUs: each rank reduces its own amax,
    the two floats are max-combined on the host, and the codes equal the one-GPU result bit for
    bit (no collective on the data path)."""
    from novann_b200.device import device_count
    if device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_fp8_shard_worker, args=(2, str(tmp_path)), nprocs=2, join=True)


def _gated_worker(rank, world, tmpdir, q):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"        # a rank leaves in this test: no multicast bindings
    from novann_b200 import _lib, workloads
    from novann_b200.launch import PeerLost, StepGate, exchange_bytes
    from novann_b200.train import Communicator, MLPTrainStep, shard_rows

    uid = Communicator.make_unique_id() if rank == 0 else None
    uid = exchange_bytes(uid, rank, os.path.join(tmpdir, "nccl_id"), token="gated")
    comm = Communicator(uid, rank, world, device=rank)
    gate = StepGate(tmpdir, rank, world, timeout_s=120.0, token="gated")
    dims = (784, 256, 128, 10)
    x, y, params = workloads.mlp_inputs(128, dims, seed=0)
    lo, hi = shard_rows(128, rank, world)
    st = MLPTrainStep(params, hi - lo, 0.01, device=rank, comm=comm, gate=gate, collective_timeout_ms=60000)
    for _ in range(2):
        st.step(x[lo:hi], y[lo:hi])             # both ranks: gate, all-reduce, watchdog wait
    gate.timeout_s = 3.0
    if rank == 1:
        gate.leave()                            # between steps, nothing in flight
        comm.close()
        q.put((rank, "left"))
        return
    before = _lib.lib().nvq_launch_count()
    try:
        st.step(x[lo:hi], y[lo:hi])
        q.put((rank, "no error"))
    except PeerLost as e:
        launched = _lib.lib().nvq_launch_count() - before
        q.put((rank, f"PeerLost launched={launched} step_no={st._step_no}: {e}"))
    comm.abort()                                # the partner is gone: tear down without waiting


def test_gated_step_raises_before_anything_is_launched_when_a_rank_left(gpu, tmp_path):
    """The ``gate=`` hook of the data-parallel step together with the collective: both ranks run
    two gated steps, rank 1 leaves between steps (nothing in flight) and closes its
    communicator, and rank 0's third step must raise PeerLost with no kernel launched and the
    step counter unchanged - no kernel is left waiting for the partner."""
    from novann_b200.device import device_count
    if device_count() < 2:
        pytest.skip("needs two GPUs")
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_gated_worker, args=(r, 2, str(tmp_path), q)) for r in range(2)]
    for p in ps:
        p.start()
    msgs = dict(q.get(timeout=240) for _ in range(2))
    for p in ps:
        p.join(60)
        assert p.exitcode == 0
    assert msgs[1] == "left"
    assert msgs[0].startswith("PeerLost launched=0 step_no=2"), msgs
