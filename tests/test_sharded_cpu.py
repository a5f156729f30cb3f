"""CPU-only: column sharding + all-gather plumbing on world_size-2 gloo ranks.

The CUDA operator is replaced by the oracle as the per-rank solver (test stand-in only), so
what is checked here is the host logic: slab arithmetic, slab extraction, and that gathering
every rank's slab reproduces the unsharded result bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import harness
from texo_b200 import sharded


def test_slab_arithmetic():
    assert sharded.slab_width(8192, 8) == 1024
    assert sharded.slab_width(10240, 8) == 1280
    assert sharded.slab_width(57344, 8) == 7168
    assert sharded.slab_width(28672, 8) == 3584
    assert sharded.slab_width(1000, 3) == 384
    # slabs tile [0, N) exactly, in order, also when N does not divide evenly
    for N, world in [(8192, 8), (1000, 3), (100, 4), (130, 2), (16, 8)]:
        edges = [sharded.column_slab(N, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == N
        for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
            assert a1 == b0 and a0 <= a1
    with pytest.raises(ValueError):
        sharded.column_slab(10, 2, 2)


def _oracle_solver(A, B, sa, sb, sc, za, zb, zc):
    o = harness.load_oracle()
    M, K = A.shape
    N = B.shape[1]
    out = o.mm_int8(A.numpy(), B.numpy(), M, N, K, (sa, sb, sc, za, zb, zc))
    return torch.from_numpy(out)


def _worker(rank, world, port, N, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K = 24, 96
        rows, cols_k = np.arange(M), np.arange(K)
        A = torch.from_numpy(harness.hashed_int8(1, 0, rows, cols_k))
        # every rank materialises only its own slab of the logical B
        n0, n1 = sharded.column_slab(N, world, rank)
        B_slab = torch.from_numpy(harness.hashed_int8(1, 1, np.arange(K), np.arange(n0, n1)))
        q = (0.02, 0.03, 4.0, 3, -5, 1)
        C = sharded.mm_int8_sharded(A, B_slab, N, *q, gather=True, solver=_oracle_solver)
        C_slab = sharded.mm_int8_sharded(A, B_slab, N, *q, gather=False, solver=_oracle_solver)
        assert tuple(C_slab.shape) == (M, n1 - n0)
        assert torch.equal(C[:, n0:n1], C_slab)
        np.save(os.path.join(result_dir, f"c{rank}.npy"), C.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N", [256, 200])
def test_two_rank_gather_equals_unsharded(tmp_path, oracle, N):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, N, str(tmp_path)), nprocs=2, join=True)
    M, K = 24, 96
    A = harness.hashed_int8(1, 0, np.arange(M), np.arange(K))
    B = harness.hashed_int8(1, 1, np.arange(K), np.arange(N))
    want = oracle.mm_int8(A, B, M, N, K, (0.02, 0.03, 4.0, 3, -5, 1))
    for r in range(2):
        assert np.array_equal(np.load(tmp_path / f"c{r}.npy"), want)


def _oracle_w4a8_solver(A, w, sa, sb, sc, za, zb, zc):
    o = harness.load_oracle()
    M, K = A.shape
    out = o.mm_int4a8(A.numpy(), w.numpy(), M, w.shape[0], K, (sa, sb, sc, za, zb, zc))
    return torch.from_numpy(out)


def _w4a8_worker(rank, world, port, N, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K = 24, 96
        A = torch.from_numpy(harness.hashed_int8(1, 0, np.arange(M), np.arange(K)))
        n0, n1 = sharded.column_slab(N, world, rank)
        w_slab = torch.from_numpy(harness.hashed_int8(1, 2, np.arange(n0, n1), np.arange(K // 2)).view(np.uint8))
        q = (0.02, 0.03, 0.4, 3, -5, 1)
        C = sharded.mm_int4a8_sharded(A, w_slab, N, *q, gather=True, solver=_oracle_w4a8_solver)
        np.save(os.path.join(result_dir, f"w{rank}.npy"), C.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N", [256, 200])
def test_two_rank_w4a8_gather_equals_unsharded(tmp_path, oracle, N):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_w4a8_worker, args=(2, port, N, str(tmp_path)), nprocs=2, join=True)
    M, K = 24, 96
    A = harness.hashed_int8(1, 0, np.arange(M), np.arange(K))
    w = harness.hashed_int8(1, 2, np.arange(N), np.arange(K // 2)).view(np.uint8)
    want = oracle.mm_int4a8(A, w, M, N, K, (0.02, 0.03, 0.4, 3, -5, 1))
    for r in range(2):
        assert np.array_equal(np.load(tmp_path / f"w{r}.npy"), want)


def _upload_worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        for M in (24, 25):  # divisible by the world size (split upload) and not (whole upload)
            host = torch.from_numpy(harness.hashed_int8(3, 0, np.arange(M), np.arange(40)))
            dev = torch.full((M, 40), 99, dtype=torch.int8)  # a CPU tensor stands in for device memory
            sharded.upload_replicated_rows(host, dev)
            assert torch.equal(dev, host), (rank, M)
        with open(os.path.join(result_dir, f"up{rank}.txt"), "w") as fh:
            fh.write("ok")
    finally:
        dist.destroy_process_group()


def test_replicated_upload_in_row_shares(tmp_path):
    """Each rank carries 1/world of the rows of a replicated matrix and an all-gather completes
    it: every rank ends with the whole matrix."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_upload_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "up0.txt").exists() and (tmp_path / "up1.txt").exists()


def _failing_worker(rank, world, port, result_dir):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=10))
    M, K, N = 8, 32, 256
    A = torch.zeros((M, K), dtype=torch.int8)
    n0, n1 = sharded.column_slab(N, world, rank)
    B_slab = torch.zeros((K, n1 - n0), dtype=torch.int8)
    if rank == 1:
        os._exit(0)  # this rank disappears between steps, before the collective
    try:
        sharded.mm_int8_sharded(A, B_slab, N, 1.0, 1.0, 1.0, 0, 0, 0, gather=True, solver=_oracle_solver)
        outcome = "completed"
    except Exception as exc:  # the surviving rank must get an error, not hang
        outcome = "error:" + type(exc).__name__
    with open(os.path.join(result_dir, "outcome.txt"), "w") as fh:
        fh.write(outcome)
    os._exit(0)


def test_lost_rank_surfaces_as_an_error_on_the_survivor(tmp_path):
    """Host-side failure injection: one of two gloo ranks exits before the all-gather; the
    other one's collective must end with an error within the process-group timeout."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_failing_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "outcome.txt").read_text().startswith("error:")


def test_operators_refuse_cpu_tensors():
    from texo_b200 import ops

    with pytest.raises(ValueError):
        ops.mm_int8(torch.zeros((2, 2), dtype=torch.int8), torch.zeros((2, 2), dtype=torch.int8),
                    1.0, 1.0, 1.0, 0, 0, 0)
