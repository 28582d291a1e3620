"""The N>1 path on CPU: two gloo ranks shard each operator family with the package's index
logic, compute their shard with an FP64 stand-in for the native call, and reassemble /
reduce with the package's collectives.  Checks the partition + collective plumbing that
bench.py uses on GPUs."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    pkg = entry.load_package()
    sh = pkg.shard
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(3)
        # --- matMul: rows of A and C sharded, B replicated, all-gather of row blocks
        N, M, K = 52, 24, 40
        A = torch.rand((N, K), generator=g, dtype=torch.float64)
        B = torch.rand((K, M), generator=g, dtype=torch.float64)
        r0, r1 = sh.shard_rows(N, world, rank)
        local = A[r0:r1] @ B
        counts = [sh.shard_rows(N, world, r)[1] - sh.shard_rows(N, world, r)[0] for r in range(world)]
        C = torch.cat(sh.all_gather_rows(dist, local, counts), 0)
        ok_mm = torch.allclose(C, A @ B, rtol=0, atol=1e-12)
        # --- batchMatMul: batch sharded
        Batch = 5
        Ab = torch.rand((Batch, 6, 8), generator=g, dtype=torch.float64)
        Bb = torch.rand((Batch, 8, 4), generator=g, dtype=torch.float64)
        b0, b1 = sh.shard_batch(Batch, world, rank)
        counts = [sh.shard_batch(Batch, world, r)[1] - sh.shard_batch(Batch, world, r)[0] for r in range(world)]
        Cb = torch.cat(sh.all_gather_rows(dist, torch.matmul(Ab[b0:b1], Bb[b0:b1]), counts), 0)
        ok_bmm = torch.allclose(Cb, torch.matmul(Ab, Bb), rtol=0, atol=1e-12)
        # --- conv: images sharded (NHWC slabs are contiguous)
        Nimg = 8
        i0, i1 = sh.shard_images(Nimg, world, rank)
        ok_img = (i1 - i0) % 4 == 0 and i0 % 4 == 0
        # --- long-K A^T B: K sharded, partials summed on rank 0
        Kl = 256
        At = torch.rand((Kl, 12), generator=g, dtype=torch.float64)
        Bt = torch.rand((Kl, 8), generator=g, dtype=torch.float64)
        k0, k1 = sh.shard_k(Kl, world, rank)
        part = At[k0:k1].T @ Bt[k0:k1]
        sh.reduce_partials(dist, part, dst=0)
        ok_k = True
        if rank == 0:
            ok_k = torch.allclose(part, At.T @ Bt, rtol=0, atol=1e-10)
        # --- convolution weight gradient: images sharded, each rank's partial deltaW summed (data-parallel training)
        Xi = torch.rand((Nimg, 5, 5, 4), generator=g, dtype=torch.float64)
        dYi = torch.rand((Nimg, 5, 5, 4), generator=g, dtype=torch.float64)

        def dw(X, dY):   # 3x3, stride 1, pad 1: deltaW[oc, fh, fw, ic]
            Xp = torch.nn.functional.pad(X, (0, 0, 1, 1, 1, 1))
            return torch.stack([torch.stack([torch.einsum("nhwo,nhwi->oi", dY, Xp[:, fh:fh + 5, fw:fw + 5, :])
                                             for fw in range(3)], 1) for fh in range(3)], 1)
        part_w = dw(Xi[i0:i1], dYi[i0:i1]).contiguous()
        sh.reduce_partials(dist, part_w, dst=0)
        ok_dw = True
        if rank == 0:
            ok_dw = torch.allclose(part_w, dw(Xi, dYi), rtol=0, atol=1e-10)
        # --- max-over-ranks timing reduction used by the benchmark
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ok_t = t.item() == float(world)
        results[rank] = bool(ok_mm and ok_bmm and ok_img and ok_k and ok_dw and ok_t)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_rank_sharding_and_collectives():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}
