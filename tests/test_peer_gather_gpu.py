"""Row-sharded matMul reassembled by the kernel's own stores, on two GPUs of one box: each rank multiplies its rows
and the contraction kernel writes them into its own copy of the full product and into the peer's (peer memory mapped
through PyTorch symmetric memory, plain mappings, no multicast).  After one barrier every rank holds the whole
product, bit for bit what a single GPU computes.  Both ways of writing the copies are run (blocks carried over
between drains; every store repeated at once).  Skipped on a box with one GPU.

The ranks are child processes that only ever stop between steps, with nothing in flight."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    import __graft_entry__ as entry
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok = True
    try:
        pkg = entry.load_package()
        mm = pkg.cu32.Cuda_matMul
        stream = torch.cuda.current_stream().cuda_stream
        rows, M, K = 2308, 2304, 160          # per rank: more tiles than CTA pairs, ragged last tile row
        g = torch.Generator(device="cuda").manual_seed(11)
        A_all = torch.rand((world * rows, K), generator=g, device="cuda") * 2 - 1    # same on every rank
        B = torch.rand((K, M), generator=g, device="cuda") * 2 - 1
        whole = torch.empty((world * rows, M), device="cuda")
        mm.matMul([stream], 1, A_all.data_ptr(), B.data_ptr(), whole.data_ptr(), world * rows, M, K)
        pg = pkg.shard.PeerGather(dist, world, rank, (rows, M), torch.device("cuda", rank))
        A = A_all[rank * rows:(rank + 1) * rows].contiguous()
        for lazy in (1, 0):
            pkg.cu32.tune("rep_lazy", lazy)
            pg.full.zero_()
            pg.barrier()
            mm.matMul_replicated([stream], 1, A.data_ptr(), B.data_ptr(), pg.local.data_ptr(), pg.replicas, rows, M, K)
            pg.barrier()
            for r in range(world):
                ok = ok and bool(torch.equal(pg.block(r), whole[r * rows:(r + 1) * rows]))
            pg.barrier()
        pkg.cu32.tune("rep_lazy", 1)
        ok = ok and pkg.cu32.read_status() == 0
    finally:
        torch.cuda.synchronize()
        dist.destroy_process_group()
    results[rank] = ok


def test_two_ranks_write_each_others_copies():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on one box")
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():
            p.kill()      # the exact child this test started
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {0: True, 1: True}
