"""GPU test of the column-sharded mm_int8 on two ranks (one process per GPU, NCCL).

Every rank materialises the same logical A and only its own column slab of B from the
counter-based generator, runs the single-GPU operator on it, and the gathered C must equal
the oracle's unsharded result bit for bit - once with an NCCL all-gather after the matmul and
with the gather fused into the matmul's epilogue (stores into the peers' copies of C in
symmetric memory: per-peer stores, and multimem stores through the NVLink multicast mapping).  Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest

from tests import harness

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _worker(rank, world, port, M, N, K, q, out_dir):
    import torch.distributed as dist

    from texo_b200 import sharded

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        A = torch.from_numpy(harness.hashed_int8(7, 0, np.arange(M), np.arange(K))).cuda()
        n0, n1 = sharded.column_slab(N, world, rank)
        B_slab = torch.from_numpy(harness.hashed_int8(7, 1, np.arange(K), np.arange(n0, n1))).cuda()
        C = sharded.mm_int8_sharded(A, B_slab, N, *q, gather=True)
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, f"c{rank}.npy"), C.cpu().numpy())
        # the same with the gather fused into the matmul's epilogue (no collective): once with
        # per-peer stores, once through the NVLink multicast mapping where the platform has one
        for tag, multicast in (("f", False), ("m", True)):
            out = sharded.GatheredOutput(M, N, torch.device("cuda", rank), multicast=multicast)
            out.tensor.fill_(99)
            out.wait()
            sharded.mm_int8_allgather(A, B_slab, out, *q)
            out.wait()
            torch.cuda.synchronize()
            np.save(os.path.join(out_dir, f"{tag}{rank}.npy"), out.tensor.cpu().numpy())
            if multicast:
                np.save(os.path.join(out_dir, f"mc{rank}.npy"), np.array([int(out.multicast_ptr != 0)]))
        # decode-shaped rows take the skinny kernel, which stores to the peers as well
        out16 = sharded.GatheredOutput(16, N, torch.device("cuda", rank))
        out16.tensor.fill_(99)
        out16.wait()
        sharded.mm_int8_allgather(A[:16].contiguous(), B_slab, out16, *q)
        out16.wait()
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, f"g{rank}.npy"), out16.tensor.cpu().numpy())
    finally:
        dist.destroy_process_group()


def test_two_gpu_slabs_gather_to_the_unsharded_result(tmp_path, oracle):
    if not torch.cuda.is_available():
        pytest.fail("no CUDA device: GPU tests need a B200")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    M, N, K = 384, 1280, 1024
    q = (0.02, 0.03, 12.0, 3, -5, 1)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, M, N, K, q, str(tmp_path)), nprocs=2, join=True)
    A = harness.hashed_int8(7, 0, np.arange(M), np.arange(K))
    B = harness.hashed_int8(7, 1, np.arange(K), np.arange(N))
    want = oracle.mm_int8(A, B, M, N, K, q)
    for r in range(2):
        assert np.array_equal(np.load(tmp_path / f"c{r}.npy"), want)
        assert np.array_equal(np.load(tmp_path / f"f{r}.npy"), want), "fused all-gather, peer stores"
        assert np.array_equal(np.load(tmp_path / f"m{r}.npy"), want), (
            "fused all-gather, multicast=%d" % int(np.load(tmp_path / f"mc{r}.npy")[0]))
        assert np.array_equal(np.load(tmp_path / f"g{r}.npy"), want[:16]), "fused all-gather, decode rows"
