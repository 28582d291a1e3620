"""Sharding of the three operator families over the GPUs of one box, one process per GPU.

The reference is single-GPU; sharding is layered outside its native API.  Every operator on
this path decomposes into independent output blocks, so each rank calls the same native on
its own slice and no data-path collective is needed to *compute*; a collective only
reassembles outputs (all-gather) or, for the long-K weight-gradient shape, sums one small
partial result (reduce).  This module holds the index arithmetic; it is pure Python so the
multi-rank logic can be tested with ``gloo`` ranks on CPU.

  batchMatMul*      shard the batch axis            -> all-gather of C slabs (optional)
  conv3D            shard the image axis N (NHWC)   -> all-gather of Y slabs (optional)
  matMul, matMulT2  shard the rows of A and C       -> all-gather of C row blocks (optional)
  matMulT1, long K  shard K (rows of A and B)       -> sum of the [N, M] partials
"""
from __future__ import annotations


def split_range(total: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """Contiguous [begin, end) of `total` units owned by `rank`.  Boundaries are multiples
    of `multiple` (the Java engine's pad-to-4 contract) except the last end, which is
    `total`; earlier ranks get the larger shares."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    groups = -(-total // multiple)
    base, extra = divmod(groups, world)
    g0 = rank * base + min(rank, extra)
    g1 = g0 + base + (1 if rank < extra else 0)
    return min(g0 * multiple, total), min(g1 * multiple, total)


def shard_rows(N: int, world: int, rank: int) -> tuple[int, int]:
    """Rows of A / C for matMul and matMulT2 (row counts stay multiples of 4)."""
    return split_range(N, world, rank, 4)


def shard_batch(Batch: int, world: int, rank: int) -> tuple[int, int]:
    return split_range(Batch, world, rank, 1)


def shard_images(N: int, world: int, rank: int) -> tuple[int, int]:
    """Images of an NHWC batch (the native contract wants N % 4 == 0 per call)."""
    return split_range(N, world, rank, 4)


def shard_k(K: int, world: int, rank: int) -> tuple[int, int]:
    """Reduction rows for the long-K A^T B shape; multiples of 32 keep k-blocks whole."""
    return split_range(K, world, rank, 32)


def all_gather_rows(dist, local, counts):
    """Reassemble blocks of unequal height along the first axis: returns the list of per-rank
    tensors.  `dist` is torch.distributed.  Equal-size collectives are the portable form, so
    shorter blocks are padded to the tallest for the transfer and trimmed afterwards; with
    equal counts (the benchmark configurations) no copy is made."""
    import torch
    tallest = max(counts)
    if local.shape[0] == tallest:
        send = local.contiguous()
    else:
        send = torch.zeros((tallest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        send[: local.shape[0]] = local
    outs = [torch.empty_like(send) for _ in counts]
    dist.all_gather(outs, send)
    return [o[:c] for o, c in zip(outs, counts)]


def reduce_partials(dist, partial, dst: int = 0):
    """Sum the per-rank [N, M] partial products of a K-sharded A^T B onto `dst`."""
    dist.reduce(partial, dst=dst, op=dist.ReduceOp.SUM)
    return partial


class PeerGather:
    """Gathered output of a row-sharded product without a collective after it: every rank holds a copy of the full
    output in memory that its peers can address (one allocation per rank, exchanged once over the process group),
    and each rank's product is stored by the contraction kernel itself into its own block of every copy
    (``cu32_matMul_replicated``).  Only stores cross NVLink; nothing is loaded from a peer.

    ``block(r)`` is rank r's block inside this rank's copy; ``local`` is this rank's own block (the kernel's C),
    ``replicas`` the device addresses of this rank's block inside the peers' copies."""

    def __init__(self, dist, world: int, rank: int, block_shape, device):
        import os
        # plain peer mappings only: no NVLink multicast object is bound to this memory (a rank that exits early
        # must not leave one behind)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch
        import torch.distributed._symmetric_memory as symm
        self.world, self.rank = world, rank
        n = 1
        for d in block_shape:
            n *= int(d)
        self.block_elems = n
        self.full = symm.empty((world, n), dtype=torch.float32, device=device)
        self.handle = symm.rendezvous(self.full, dist.group.WORLD)
        self.block_shape = tuple(block_shape)
        self.local = self.full[rank].view(self.block_shape)
        self.replicas = []
        self._keep = []
        for r in range(world):
            if r == rank:
                continue
            peer = self.handle.get_buffer(r, (world, n), torch.float32)
            self._keep.append(peer)
            self.replicas.append(peer[rank].data_ptr())

    def block(self, r: int):
        return self.full[r].view(self.block_shape)

    def barrier(self):
        """All ranks' kernels have drained and their stores are visible everywhere."""
        import torch
        torch.cuda.synchronize()
        self.handle.barrier()
