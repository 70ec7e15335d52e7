"""Multi-process host logic on CPU (gloo, world size 2): request partition with no data-path
collective, N-sharded GEMM with one all-gather. The local compute is the torch checker - the
kernels themselves need a GPU; what is tested is partitioning, renumbering and reassembly."""

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cleave_b200 import sharding
from cleave_b200.runtime import reference as R


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_partition_is_balanced_and_complete():
    lens = [512, 32768, 700, 1, 129, 64, 20000, 0, 4096, 9000]
    parts = sharding.partition_requests(lens, 4)
    assert sorted(i for p in parts for i in p) == list(range(len(lens)))
    cost = lambda p: sum(max(1, -(-lens[i] // 64)) for i in p)  # noqa: E731
    loads = [cost(p) for p in parts]
    assert max(loads) <= max(-(-max(lens) // 64), 1.34 * sum(loads) / 4)
    assert sharding.partition_requests(lens, 2, balance=False) == [[0, 1, 2, 3, 4], [5, 6, 7, 8, 9]]
    bounds = [sharding.n_shard(11008, r, 8) for r in range(8)]
    assert bounds[0][0] == 0 and bounds[-1][1] == 11008 and all(a[1] == b[0] for a, b in zip(bounds, bounds[1:]))
    assert all(lo % 8 == 0 for lo, _ in bounds)


def _fused_host_logic(rank, world, x, w):
    """The host side of the fused all-gather (sharding.gemm_n_sharded_fused) with stand-ins for the symmetric-memory
    handle and the GEMM: which slice of the result the kernel is given, which peer addresses, one barrier per call;
    and, when the GEMM answers "unsupported", the dense block and one scatter over all copies - remembered, so that
    the refusal is not asked for again."""
    from cleave_b200 import _lib, ops

    n = w.shape[1]
    lo, hi = sharding.n_shard(n, rank, world)

    class Handle:
        buffer_ptrs = [10_000 * (r + 1) for r in range(world)]
        barriers = 0

        def barrier(self):
            Handle.barriers += 1

    y = torch.zeros(x.shape[0], n)
    calls = []

    def gemm(x_, w_, out=None, peers=None):
        calls.append((None if out is None else tuple(out.shape), peers))
        res = R.rmsnorm_matmul(x_, w_, 1e-6)
        if out is None:
            return res
        out.copy_(res)
        return out

    sharding._IN_KERNEL.clear()
    got = sharding.gemm_n_sharded_fused(gemm, x, (w[:, lo:hi].contiguous(),), n, y, Handle())
    want_peers = [Handle.buffer_ptrs[r] + lo * 4 for r in range(world) if r != rank]
    ok = got is y and calls == [((x.shape[0], hi - lo), want_peers)] and Handle.barriers == 1
    ok = ok and torch.allclose(y[:, lo:hi], R.rmsnorm_matmul(x, w, 1e-6)[:, lo:hi], rtol=1e-5, atol=1e-5)

    def refusing(x_, w_, out=None, peers=None):
        if peers is not None:
            calls.append("refused")
            raise _lib.Cb200Error(_lib.ERR_UNSUPPORTED, "unsupported")
        calls.append("dense")
        return R.rmsnorm_matmul(x_, w_, 1e-6)

    scattered = []
    real = ops.peer_scatter_cols
    ops.peer_scatter_cols = lambda block, ld, dsts: scattered.append((tuple(block.shape), ld, list(dsts)))
    try:
        calls.clear()
        sharding._IN_KERNEL.clear()
        for _ in range(2):
            sharding.gemm_n_sharded_fused(refusing, x, (w[:, lo:hi].contiguous(),), n, y, Handle())
    finally:
        ops.peer_scatter_cols = real
    ok = ok and calls == ["refused", "dense", "dense"] and Handle.barriers == 3
    ok = ok and scattered == [((x.shape[0], hi - lo), n, [y.data_ptr() + lo * 4] + want_peers)] * 2
    return bool(ok)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        lens = [300, 5, 0, 1000, 64, 129]
        ps, hq, hkv, d = 16, 8, 2, 64
        pages = [-(-n // ps) for n in lens]
        num_pages = sum(pages) + 2
        idx = torch.randperm(num_pages, generator=g)[:sum(pages)].int()
        ptr = torch.tensor([0] + np.cumsum(pages).tolist(), dtype=torch.int32)
        last = torch.tensor([n - (p - 1) * ps if p else 0 for n, p in zip(lens, pages)], dtype=torch.int32)
        q_ = torch.randn(len(lens), hq, d, generator=g).bfloat16()
        kc = torch.randn(num_pages, ps, hkv, d, generator=g).bfloat16()
        vc = torch.randn(num_pages, ps, hkv, d, generator=g).bfloat16()
        want_out, want_lse = R.gqa_paged_decode(q_, kc, vc, ptr, idx, last, d ** -0.5)
        # each rank holds only its requests' pages, renumbered into a private pool
        parts = sharding.partition_requests(lens, world, tile=16)
        mine = parts[rank]
        lptr, lidx, llast, held = sharding.shard_paged_tables(ptr, idx, last, mine)
        sel = torch.tensor(held, dtype=torch.long)
        out, lse = R.gqa_paged_decode(q_[mine], kc[sel], vc[sel], torch.tensor(lptr, dtype=torch.int32),
                                      torch.tensor(lidx, dtype=torch.int32), torch.tensor(llast, dtype=torch.int32),
                                      d ** -0.5)
        full_out = sharding.gather_by_request(out.float(), parts)
        full_lse = sharding.gather_by_request(lse, parts)
        ok1 = torch.equal(full_out, want_out.float()) and torch.equal(full_lse, want_lse)
        # N-sharded RMSNorm @ W with one all-gather
        x = torch.randn(8, 64, generator=g)
        w = torch.randn(64, 104, generator=g)
        lo, hi = sharding.n_shard(104, rank, world)
        y = sharding.gemm_n_sharded(lambda x_, w_: R.rmsnorm_matmul(x_, w_, 1e-6), x, [w[:, lo:hi].contiguous()], 104)
        ok2 = torch.allclose(y, R.rmsnorm_matmul(x, w, 1e-6), rtol=1e-5, atol=1e-5)
        ok2 = ok2 and _fused_host_logic(rank, world, x, w)
        q.put((rank, bool(ok1), bool(ok2)))
    finally:
        dist.destroy_process_group()


def test_request_sharding_and_n_sharded_gemm_world_size_2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True, True), (1, True, True)]
