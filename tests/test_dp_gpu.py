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


def _peer_worker(rank, world, tmpdir):
    sys.path.insert(0, ROOT)
    import functools
    from novann_b200 import workloads
    from novann_b200.launch import allgather_bytes
    from novann_b200.train import MLPTrainStep, PeerGroup, shard_rows
    from oracle import oracle_np as o

    dims = (784, 256, 128, 10)
    x, y, params = workloads.mlp_inputs(128, dims, seed=0)
    n = sum(p.size for p in params)
    counter = [0]

    def gather(payload):
        counter[0] += 1
        return allgather_bytes(payload, rank, world, os.path.join(tmpdir, f"peer{counter[0]}"), token="peer")

    peer = PeerGroup(rank, world, n, device=rank, allgather=gather, timeout_ms=20000)
    lo, hi = shard_rows(128, rank, world)
    st = MLPTrainStep(params, hi - lo, 0.01, device=rank, peer=peer)
    cur = params
    for s in range(3):                       # eager: nine kernels + the fused all-reduce / update
        xs, ys, _ = workloads.mlp_inputs(128, dims, seed=60 + s)
        st.step(xs[lo:hi], ys[lo:hi])
        cur = o.mlp_train_step(cur, xs, ys, 0.01)["params"]
    st.capture()                             # two graphs, one per gradient buffer
    for s in range(3):
        xs, ys, _ = workloads.mlp_inputs(128, dims, seed=70 + s)
        st.step(xs[lo:hi], ys[lo:hi])
        cur = o.mlp_train_step(cur, xs, ys, 0.01)["params"]
    mine = st.params()
    for a, b in zip(mine, cur):
        err = np.max(np.abs(a - b)) / max(1e-30, np.max(np.abs(b)))
        assert err <= 2e-5, (rank, err)
    # every rank adds the gradients in the same order: the parameters agree bit for bit
    blob = np.concatenate([p.ravel() for p in mine]).tobytes()
    everyone = gather(blob)
    assert all(e == everyone[0] for e in everyone)
    peer.close()


def test_two_rank_peer_memory_step_equals_global_batch_step(gpu, tmp_path):
    """The data-parallel step with the all-reduce and the SGD update fused into one kernel over
    NVLink peer memory (no NCCL): equal to the whole-batch step, and bit-identical across ranks."""
    from novann_b200.device import device_count
    if device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_peer_worker, args=(2, str(tmp_path)), nprocs=2, join=True)


def test_peer_step_on_one_rank_equals_the_plain_step(gpu):
    """world = 1: the fused kernel is the SGD update (sum of one gradient, 1 / 1)."""
    from novann_b200 import workloads
    from novann_b200.train import MLPTrainStep, PeerGroup
    dims = (784, 256, 128, 10)
    x, y, params = workloads.mlp_inputs(128, dims, seed=3)
    n = sum(p.size for p in params)
    peer = PeerGroup(0, 1, n, device=gpu)
    a = MLPTrainStep(params, 128, 0.01, device=gpu, peer=peer)
    b = MLPTrainStep(params, 128, 0.01, device=gpu)
    for s in range(3):
        xs, ys, _ = workloads.mlp_inputs(128, dims, seed=80 + s)
        a.step(xs, ys)
        b.step(xs, ys)
    for pa, pb in zip(a.params(), b.params()):
        np.testing.assert_array_equal(pa, pb)
    peer.close()


def test_peer_step_gives_up_when_a_rank_never_announces(gpu):
    """A group of two whose second rank is absent: nothing ever sets its flag, the kernel's wait
    runs out after the time limit, the parameters stay as they were, the error flag reports it and
    the context stays usable (no fault, no hang)."""
    from novann_b200 import _lib, workloads
    from novann_b200.train import MLPTrainStep, PeerGroup
    dims = (784, 256, 128, 10)
    x, y, params = workloads.mlp_inputs(128, dims, seed=4)
    n = sum(p.size for p in params)
    peer = PeerGroup(0, 2, n, device=gpu, timeout_ms=50, absent=(1,))
    st = MLPTrainStep(params, 64, 0.01, device=gpu, peer=peer)
    before = st.params()
    with pytest.raises(_lib.NvqError):
        st.step(x[:64], y[:64])
    for pa, pb in zip(st.params(), before):
        np.testing.assert_array_equal(pa, pb)
    # the device still works
    plain = MLPTrainStep(params, 64, 0.01, device=gpu)
    plain.step(x[:64], y[:64])
    assert np.isfinite(plain.loss())
    peer.close()


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
