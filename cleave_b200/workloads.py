"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

The reference evaluates its paged operators on axis tuples captured from a public benchmark
suite (python/cleave/dynamic/workloads.py:19-326) whose trace files are not redistributable
here; these generators stand in for them: lengths uniform in a range, a random permutation as
the page table, N(0,1) tensors.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class PagedDecodeWorkload:
    q: torch.Tensor                 # (batch, HQ, D)
    k_cache: torch.Tensor           # (num_pages, page, HKV, D)
    v_cache: torch.Tensor
    kv_indptr: torch.Tensor         # (batch + 1) int32, pages
    kv_indices: torch.Tensor        # (num_pages) int32
    kv_last_page_len: torch.Tensor  # (batch) int32
    sm_scale: float
    kv_lens: torch.Tensor           # (batch) int64, CPU

    @property
    def tokens(self) -> int:
        return int(self.kv_lens.sum())

    def algorithmic_bytes(self) -> int:
        """Bytes any implementation must move: live K and V tokens, Q, O, lse and the tables."""
        hkv, d = self.k_cache.shape[2], self.k_cache.shape[3]
        esz = self.k_cache.element_size()
        kv = self.tokens * 2 * hkv * d * esz
        qo = 2 * self.q.numel() * esz
        lse = self.q.shape[0] * self.q.shape[1] * 4
        tables = 4 * (self.kv_indices.numel() + self.kv_indptr.numel() + self.kv_last_page_len.numel())
        return kv + qo + lse + tables

    def flops(self) -> int:
        return 4 * self.q.shape[1] * self.q.shape[2] * self.tokens

    def args(self):
        return (self.q, self.k_cache, self.v_cache, self.kv_indptr, self.kv_indices,
                self.kv_last_page_len, self.sm_scale)


def paged_decode_tables(batch, page_size, lo, hi, seed):
    """CPU tensors ``(kv_lens, kv_indptr, kv_indices, kv_last_page_len, num_pages)``:
    ``kv_len ~ randint(lo, hi + 1)``, pool sized to the total page count, block table a random
    permutation of the page ids."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    kv_lens = torch.randint(lo, hi + 1, (batch,), generator=g)
    pages = (kv_lens + page_size - 1) // page_size
    num_pages = int(pages.sum())
    kv_indices = torch.randperm(num_pages, generator=g).to(torch.int32)
    kv_indptr = torch.cat([torch.zeros(1, dtype=torch.int64), pages.cumsum(0)]).to(torch.int32)
    last = (kv_lens - (pages - 1) * page_size).to(torch.int32)
    return kv_lens, kv_indptr, kv_indices, last, num_pages


def paged_decode_workload(batch=128, hq=32, hkv=8, d=128, page_size=64, lo=512, hi=32768, seed=0,
                          dtype=torch.float16, device="cuda") -> PagedDecodeWorkload:
    """The paged GQA decode benchmark config. Tables and Q are drawn on the CPU generator; the
    caches (gigabytes) are drawn on the device generator with the same seed."""
    kv_lens, kv_indptr, kv_indices, last, num_pages = paged_decode_tables(batch, page_size, lo, hi, seed)
    g = torch.Generator(device="cpu").manual_seed(seed + 1)
    q = torch.randn(batch, hq, d, generator=g).to(dtype)
    dev = torch.device(device)
    if dev.type == "cuda":
        gd = torch.Generator(device=dev).manual_seed(seed + 2)
        k_cache = torch.randn(num_pages, page_size, hkv, d, generator=gd, device=dev, dtype=dtype)
        v_cache = torch.randn(num_pages, page_size, hkv, d, generator=gd, device=dev, dtype=dtype)
    else:
        k_cache = torch.randn(num_pages, page_size, hkv, d, generator=g).to(dtype)
        v_cache = torch.randn(num_pages, page_size, hkv, d, generator=g).to(dtype)
    return PagedDecodeWorkload(q.to(dev), k_cache, v_cache, kv_indptr.to(dev), kv_indices.to(dev),
                               last.to(dev), float(d) ** -0.5, kv_lens)


def sub_workload(w: PagedDecodeWorkload, requests) -> PagedDecodeWorkload:
    """The same requests on a private pool holding only their pages (page ids renumbered),
    on the CPU: what a CPU baseline or one shard of a request-partitioned job sees."""
    ptr = w.kv_indptr.cpu().long()
    idx = w.kv_indices.cpu().long()
    new_ptr, new_idx, pages = [0], [], []
    for b in requests:
        mine = idx[ptr[b]:ptr[b + 1]]
        new_idx.append(torch.arange(len(pages), len(pages) + mine.numel()))
        pages.extend(mine.tolist())
        new_ptr.append(new_ptr[-1] + mine.numel())
    sel = torch.tensor(pages, dtype=torch.long)
    req = torch.tensor(list(requests), dtype=torch.long)
    kc = w.k_cache.index_select(0, sel.to(w.k_cache.device)).cpu()
    vc = w.v_cache.index_select(0, sel.to(w.v_cache.device)).cpu()
    return PagedDecodeWorkload(w.q.cpu()[req], kc, vc, torch.tensor(new_ptr, dtype=torch.int32),
                               torch.cat(new_idx).to(torch.int32) if new_idx else torch.zeros(0, dtype=torch.int32),
                               w.kv_last_page_len.cpu()[req], w.sm_scale, w.kv_lens[req])


def sharded_paged_decode_workload(world, rank, batch_per_gpu=128, hq=32, hkv=8, d=128, page_size=64, lo=512,
                                  hi=32768, seed=0, dtype=torch.float16, device="cuda"):
    """Rank ``rank``'s share of ONE global batch of ``world * batch_per_gpu`` requests, split by request
    with :func:`cleave_b200.sharding.partition_requests` (longest first over KV tile counts) and held in
    a private pool (:func:`cleave_b200.sharding.shard_paged_tables` with the global table's scatter kept).
    Returns ``(workload, requests, tiles_per_rank)``: the rank's workload, the global indices of its
    requests and every rank's KV tile count. Lengths, tables and Q of the global batch are drawn on the
    CPU generator exactly as :func:`paged_decode_workload` draws them (``world = 1`` gives that
    workload's tables and Q); a rank's cache pages are drawn on its own device."""
    from . import sharding

    batch = world * batch_per_gpu
    kv_lens, kv_indptr, kv_indices, last, _ = paged_decode_tables(batch, page_size, lo, hi, seed)
    parts = sharding.partition_requests(kv_lens.tolist(), world, tile=64)
    tiles = [sum(max(1, -(-int(kv_lens[i]) // 64)) for i in p) for p in parts]
    mine = parts[rank]
    lptr, lidx, llast, held = sharding.shard_paged_tables(kv_indptr.tolist(), kv_indices.tolist(), last.tolist(),
                                                          mine, keep_order=True)
    g = torch.Generator(device="cpu").manual_seed(seed + 1)
    q = torch.randn(batch, hq, d, generator=g).to(dtype)[torch.tensor(mine, dtype=torch.long)]
    dev = torch.device(device)
    shape = (len(held), page_size, hkv, d)
    if dev.type == "cuda":
        gd = torch.Generator(device=dev).manual_seed(seed + 2 + rank)
        k_cache = torch.randn(shape, generator=gd, device=dev, dtype=dtype)
        v_cache = torch.randn(shape, generator=gd, device=dev, dtype=dtype)
    else:
        k_cache = torch.randn(shape, generator=g).to(dtype)
        v_cache = torch.randn(shape, generator=g).to(dtype)
    w = PagedDecodeWorkload(q.to(dev), k_cache, v_cache, torch.tensor(lptr, dtype=torch.int32, device=dev),
                            torch.tensor(lidx, dtype=torch.int32, device=dev),
                            torch.tensor(llast, dtype=torch.int32, device=dev), float(d) ** -0.5,
                            kv_lens[torch.tensor(mine, dtype=torch.long)])
    return w, mine, tiles
