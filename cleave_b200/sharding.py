"""Multi-GPU use of the kernels, one process per GPU (``torch.distributed``).

The reference is single-GPU. Its operators shard naturally: decode requests are independent, so
a batch is partitioned by request with NO collective on the data path; a large GEMM shards its
weight along N, every rank recomputes the per-row RMSNorm statistics locally, and one all-gather
over NVLink reassembles Y only when the caller wants the full matrix on every rank.
"""

from __future__ import annotations

import heapq


def partition_requests(kv_lens, world: int, tile: int = 64, balance: bool = True):
    """Request indices per rank. ``balance=True``: longest-processing-time-first over KV tile counts
    (skewed lengths would leave a contiguous split far from even); each rank's list is sorted so
    that results can be put back in request order. Empty requests cost one unit of bookkeeping."""
    n = len(kv_lens)
    if world <= 0:
        raise ValueError("world must be positive")
    if not balance:
        per = -(-n // world)
        return [list(range(r * per, min(n, (r + 1) * per))) for r in range(world)]
    cost = [max(1, -(-int(l) // tile)) for l in kv_lens]
    heap = [(0, r) for r in range(world)]
    heapq.heapify(heap)
    out = [[] for _ in range(world)]
    for i in sorted(range(n), key=lambda i: -cost[i]):
        load, r = heapq.heappop(heap)
        out[r].append(i)
        heapq.heappush(heap, (load + cost[i], r))
    return [sorted(x) for x in out]


def shard_paged_tables(kv_indptr, kv_indices, kv_last_page_len, requests, keep_order: bool = False):
    """Page tables of one rank's requests over a private pool: ``(indptr, indices, last, pages)``
    where ``pages`` lists the global page ids the rank must hold, in its local numbering (local page
    ``i`` holds global page ``pages[i]``). By default local ids follow the walk of the requests (page
    tables become sequential); ``keep_order=True`` numbers the rank's pages by the rank of their global
    id instead, so that a scattered global table stays as scattered on the rank (a subset of a random
    permutation, order kept, is again a random permutation)."""
    ptr = [int(x) for x in kv_indptr]
    new_ptr, walk = [0], []
    for b in requests:
        walk.extend(int(x) for x in kv_indices[ptr[b]:ptr[b + 1]])
        new_ptr.append(len(walk))
    if keep_order:
        pages = sorted(set(walk))
        local = {g: i for i, g in enumerate(pages)}
        new_idx = [local[g] for g in walk]
    else:
        pages, local, new_idx = [], {}, []
        for g in walk:  # a page shared by two requests is held once
            if g not in local:
                local[g] = len(pages)
                pages.append(g)
            new_idx.append(local[g])
    last = None if kv_last_page_len is None else [int(kv_last_page_len[b]) for b in requests]
    return new_ptr, new_idx, last, pages


def gather_by_request(local_out, requests_per_rank, group=None):
    """All ranks' per-request outputs back in request order (only for callers that need every
    request everywhere; the decode data path itself has no collective)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    counts = [len(r) for r in requests_per_rank]
    width = max(counts) if counts else 0
    pad = torch.zeros((width,) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    pad[:local_out.shape[0]] = local_out
    bufs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(bufs, pad, group=group)
    total = sum(counts)
    full = torch.empty((total,) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    for r, reqs in enumerate(requests_per_rank):
        if reqs:
            full[torch.tensor(reqs, device=local_out.device)] = bufs[r][:len(reqs)]
    return full


def n_shard(n: int, rank: int, world: int, align: int = 8):
    """Column range ``[lo, hi)`` of rank's weight shard; boundaries are multiples of ``align``."""
    blocks = -(-n // align)
    lo = min(n, (blocks * rank // world) * align)
    hi = min(n, (blocks * (rank + 1) // world) * align)
    return lo, hi


def gemm_n_sharded(local_gemm, x, w_shards, n_total, *, gather=True, group=None):
    """``Y = op(X, W)`` with W sharded along N. ``local_gemm(x, *w_shards)`` computes this rank's
    columns (any of the GEMM family; RMSNorm statistics are per row over K and need no exchange).
    With ``gather`` the shards are all-gathered and concatenated along N."""
    import torch
    import torch.distributed as dist

    y_local = local_gemm(x, *w_shards)
    if not gather:
        return y_local
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    bounds = [n_shard(n_total, r, world) for r in range(world)]
    assert bounds[rank][1] - bounds[rank][0] == y_local.shape[1]
    widths = {hi - lo for lo, hi in bounds}
    if len(widths) == 1:
        # equal shards (the usual case): one collective straight from the kernel's output into a
        # (world, M, N / world) buffer, then one strided copy into the row-major (M, N) result
        m = y_local.shape[0]
        stacked = torch.empty((world, m, y_local.shape[1]), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(stacked, y_local.contiguous(), group=group)
        return stacked.permute(1, 0, 2).reshape(m, n_total)
    width = max(widths)
    pad = torch.zeros((y_local.shape[0], width), dtype=y_local.dtype, device=y_local.device)
    pad[:, :y_local.shape[1]] = y_local
    bufs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(bufs, pad, group=group)
    return torch.cat([b[:, :hi - lo] for b, (lo, hi) in zip(bufs, bounds)], dim=1)


def symmetric_result(m: int, n_total: int, dtype, device, group=None):
    """An (M, N_total) result tensor in symmetric memory - one copy per GPU of the group, every copy mapped into
    every process - and its handle. Allocate once and reuse: the rendezvous is a collective."""
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem

    y = symm_mem.empty((m, n_total), dtype=dtype, device=device)
    return y, symm_mem.rendezvous(y, group=group if group is not None else dist.group.WORLD)


def gemm_n_sharded_fused(local_gemm, x, w_shards, n_total, y, handle, group=None):
    """``Y = op(X, W)`` with W sharded along N and the all-gather fused into the product: ``local_gemm(x, *w_shards,
    out=..., peers=...)`` (one of ``ops.matmul`` / ``rmsnorm_matmul`` / ``swiglu``) writes this rank's columns
    into its own copy of ``y`` (from :func:`symmetric_result`) and, tile by tile while it computes the next one, into
    every other rank's copy through NVLink. The barrier at the end orders the ranks; after it ``y`` holds the whole
    result on every rank. No NCCL collective and no reassembly copy."""
    import torch.distributed as dist

    from . import _lib, ops

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    lo, hi = n_shard(n_total, rank, world)
    itemsize = y.element_size()
    peers = [int(handle.buffer_ptrs[r]) + lo * itemsize for r in range(world) if r != rank]
    key = (tuple(x.shape), tuple(w_shards[0].shape), x.dtype, len(w_shards))
    if _IN_KERNEL.get(key, True):
        try:
            local_gemm(x, *w_shards, out=y[:, lo:hi], peers=peers)
            handle.barrier()
            return y
        except _lib.Cb200Error as exc:
            if exc.status != _lib.ERR_UNSUPPORTED:
                raise
            _IN_KERNEL[key] = False  # remembered: the refusal costs a host round trip every time
    # shapes the CTA-pair kernel does not take (few rows): the product into a dense block, then one kernel that
    # copies the block into this rank's slice of every copy - still no collective and no reassembly pass
    block = local_gemm(x, *w_shards)
    ops.peer_scatter_cols(block, n_total, [y.data_ptr() + lo * itemsize] + peers)
    handle.barrier()
    return y


_IN_KERNEL: dict = {}  # (shapes, dtype) -> False once cb200_gemm has refused to send that product's tiles itself
