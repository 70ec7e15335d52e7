"""Two GPUs, one process each, NCCL over 127.0.0.1: decode sharded by request with no collective on
the data path (results gathered only to be checked), and a GEMM sharded along N with one all-gather - as an NCCL
collective after the product, and fused into the product's kernel over peer memory.
Skipped on a single-GPU box; the CPU (gloo) form of the same logic is tests/test_sharding_cpu.py."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path[:0] = [os.path.dirname(here), here, os.path.join(here, "golden")]
    import torch.distributed as dist

    import cases
    from cleave_b200 import ops, sharding
    from oracle import cleave_oracle as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        # ---- paged decode, requests dealt longest-first; every rank holds only its own requests' pages
        kv_lens = [700, 1, 129, 64, 2000, 0, 333, 65]
        inp = cases.gqa_paged_inputs(7, kv_lens, 32, 8, 128, 64, "bf16")
        parts = sharding.partition_requests(kv_lens, world)
        mine = parts[rank]
        indptr, indices, last, held = sharding.shard_paged_tables(inp["kv_indptr"], inp["kv_indices"],
                                                                  inp["kv_last_page_len"], mine)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
        bf = lambda a: dev(a).to(torch.bfloat16)  # noqa: E731
        i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")  # noqa: E731
        held = held if held else [0]  # a rank without live pages still passes a valid pool
        out = torch.empty(len(mine), 32, 128, dtype=torch.bfloat16, device="cuda")
        lse = torch.empty(len(mine), 32, dtype=torch.float32, device="cuda")
        ops.gqa_paged_decode(bf(inp["q"][mine]), bf(inp["k_cache"][held]), bf(inp["v_cache"][held]), i32(indptr),
                             i32(indices), i32(last), inp["sm_scale"], out=out, lse=lse)
        full = sharding.gather_by_request(out.float(), parts)
        want, _ = orc.gqa_paged_decode(inp["q"], inp["k_cache"], inp["v_cache"], inp["kv_indptr"], inp["kv_indices"],
                                       inp["kv_last_page_len"], inp["sm_scale"])
        ok1 = bool(np.allclose(full.cpu().numpy(), want, rtol=2e-2, atol=2e-2))
        # ---- RMSNorm(X) @ W with W sharded along N and one all-gather
        g = cases.gemm_inputs(3, 64, 1000, 512, "f16", gamma=True)
        lo, hi = sharding.n_shard(1000, rank, world)
        f16 = lambda a: dev(a).to(torch.float16)  # noqa: E731
        gm = f16(g["gamma"])
        y = sharding.gemm_n_sharded(lambda x_, w_: ops.rmsnorm_matmul(x_, w_, eps=1e-6, gamma=gm), f16(g["x"]),
                                    [f16(g["w0"][:, lo:hi])], 1000)
        ok2 = bool(np.allclose(y.float().cpu().numpy(), orc.rmsnorm_matmul(g["x"], g["w0"], 1e-6, g["gamma"], "f16"),
                               rtol=2e-2, atol=2e-2))
        # ---- the same kind of product with the all-gather fused into the kernel: every rank writes its columns into
        # its own copy of the full result (symmetric memory) and, tile by tile, into the other rank's copy; no NCCL
        # collective. Unequal shards, a partial last tile, rows that do not fill a tile; the result must equal the
        # shards computed one by one on every rank.
        ok3 = True
        # (64 rows: the product runs on the single-CTA kernels and one scatter kernel sends the block to the copies)
        for op, mm, nn, kk in (("matmul", 512, 1288, 1024), ("rmsnorm", 300, 2048, 512), ("swiglu", 256, 520, 256),
                               ("rmsnorm", 64, 1000, 512)):
            gen = torch.Generator(device="cpu").manual_seed(5)
            xs = torch.randn(mm, kk, generator=gen).to(torch.float16).cuda()
            ws = (torch.randn(kk, nn, generator=gen) / kk ** 0.5).to(torch.float16).cuda()
            w1 = (torch.randn(kk, nn, generator=gen) / kk ** 0.5).to(torch.float16).cuda()
            bounds = [sharding.n_shard(nn, r, world) for r in range(world)]
            if op == "matmul":
                fn = lambda a, b, **kw: ops.matmul(a, b, **kw)  # noqa: E731
            elif op == "rmsnorm":
                fn = lambda a, b, **kw: ops.rmsnorm_matmul(a, b, eps=1e-6, **kw)  # noqa: E731
            else:
                fn = lambda a, b, c, **kw: ops.swiglu(a, b, c, **kw)  # noqa: E731
            shards = lambda a0, a1: (ws[:, a0:a1].contiguous(),) + ((w1[:, a0:a1].contiguous(),) if op == "swiglu" else ())  # noqa: E731
            ys, handle = sharding.symmetric_result(mm, nn, torch.float16, "cuda")
            ys.fill_(float("nan"))
            handle.barrier()
            got = sharding.gemm_n_sharded_fused(fn, xs, shards(*bounds[rank]), nn, ys, handle)
            torch.cuda.synchronize()
            want = torch.cat([fn(xs, *shards(a0, a1)) for a0, a1 in bounds], dim=1)
            # the shards on their own may run under another plan (split K in a cluster) than the pair kernel the fused
            # form takes, so equality is up to the operators' tolerance; a cell nobody wrote would still be NaN
            ok3 = ok3 and not bool(torch.isnan(got).any()) and bool(torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2))
        torch.cuda.synchronize()
        q.put((rank, ok1, ok2 and ok3))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_request_sharded_decode_and_n_sharded_gemm_on_two_gpus():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True, True), (1, True, True)]
