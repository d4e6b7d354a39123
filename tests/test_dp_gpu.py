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
    comm.close()


def test_two_rank_step_equals_global_batch_step(gpu, tmp_path):
    from novann_b200.device import device_count
    if device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, str(tmp_path)), nprocs=2, join=True)
