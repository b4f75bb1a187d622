"""Paged KV cache with one page pool and one page table per iteration depth.

The reference grows a dense ``(B, n, heads, hd)`` tensor per ``(layer, depth)`` slot with
``torch.cat`` on every step (reference ``tah/model/causal_cache.py:84-95``) and pads the
depth->=1 slots over the whole batch.  Here each depth has a pool of fixed-size pages

    pool[depth]: [layers, pages, 2 (K,V), kv_heads, page_size, head_dim]   bf16

and a row owns only the pages its real entries need; the depth->=1 pools hold hard-token
entries only.  Free pages are handed out on the device (``free_stack``/``free_count``,
popped by the tick kernel), so decode never returns to the host for memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import os

import torch


@dataclass
class CacheGeometry:
    n_layers: int
    n_kv_heads: int
    head_dim: int
    page_size: int = 16


GUARD_PATTERN = 0x5A5A          # int16 view of the bf16 guard pages


class PagedKVCache:
    def __init__(self, geo: CacheGeometry, rows: int, max_tokens_per_row: int, n_depths: int,
                 deep_fraction: float = 0.25, device="cuda", dtype=torch.bfloat16):
        self.geo, self.rows, self.n_depths = geo, rows, n_depths
        self.page_size = geo.page_size
        ppr = (max_tokens_per_row + geo.page_size - 1) // geo.page_size + 1
        self.max_pages = [ppr] * n_depths
        self.n_pages: List[int] = []
        self.pool: List[torch.Tensor] = []
        self.page_table: List[torch.Tensor] = []
        self.len: List[torch.Tensor] = []
        self.free_stack: List[torch.Tensor] = []
        self.free_count: List[torch.Tensor] = []
        # TAH_B200_CANARY=G: G guard pages behind every layer's pool, filled with a bit pattern that no kernel may
        # touch (pages are only ever handed out from the free stack); check_guards() verifies them on the host
        self.guard_pages = int(os.environ.get("TAH_B200_CANARY", "0") or 0)
        for d in range(n_depths):
            pages = rows * ppr if d == 0 else max(rows * 2, int(rows * ppr * deep_fraction))
            self.n_pages.append(pages)
            pool = torch.zeros(geo.n_layers, pages + self.guard_pages, 2, geo.n_kv_heads, geo.page_size, geo.head_dim,
                               dtype=dtype, device=device)
            if self.guard_pages:
                pool[:, pages:].view(torch.int16).fill_(GUARD_PATTERN)
            self.pool.append(pool)
            self.page_table.append(torch.zeros(rows, ppr, dtype=torch.int32, device=device))
            self.len.append(torch.zeros(rows, dtype=torch.int32, device=device))
            self.free_stack.append(torch.arange(pages, dtype=torch.int32, device=device))
            self.free_count.append(torch.full((1,), pages, dtype=torch.int32, device=device))

    def check_guards(self) -> bool:
        """True when every guard page still holds the pattern (always true without ``TAH_B200_CANARY``)."""
        if not self.guard_pages:
            return True
        return all(bool((p[:, n:].view(torch.int16) == GUARD_PATTERN).all()) for p, n in zip(self.pool, self.n_pages))

    def bytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.pool)

    def reset(self) -> None:
        for d in range(self.n_depths):
            self.len[d].zero_()
            self.page_table[d].zero_()
            self.free_stack[d].copy_(torch.arange(self.n_pages[d], dtype=torch.int32, device=self.free_stack[d].device))
            self.free_count[d].fill_(self.n_pages[d])

    def layer_pool(self, depth: int, layer: int) -> torch.Tensor:
        return self.pool[depth][layer]

    def assign_prefill(self, depth: int, counts: torch.Tensor) -> torch.Tensor:
        """Give each row ``ceil(counts[r] / page_size)`` pages from the top of the free stack, set
        ``len`` and the page table (host-side, once per request batch).  Returns for every one of the
        ``sum(counts)`` entries, in row-major order, its slot ``page * page_size + offset``."""
        ps = self.page_size
        dev = self.len[depth].device
        counts = counts.to(device=dev, dtype=torch.int64)
        need = (counts + ps - 1) // ps
        total = int(need.sum())
        free = int(self.free_count[depth])
        if total > free or int(need.max() if need.numel() else 0) > self.max_pages[depth]:
            raise RuntimeError(f"KV pool of depth {depth} too small: need {total} pages, {free} free")
        first = torch.cumsum(need, 0) - need                     # first page rank of each row
        # pages are taken from the top of the stack: rank k -> stack[free - 1 - k]
        row_of_page = torch.repeat_interleave(torch.arange(self.rows, device=dev), need)
        rank = torch.arange(total, device=dev)
        page_ids = self.free_stack[depth][(free - 1 - rank).long()]
        col = rank - first[row_of_page]
        self.page_table[depth][row_of_page, col] = page_ids
        self.free_count[depth].fill_(free - total)
        self.len[depth].copy_(counts.to(torch.int32))
        # slots of the entries
        row_of_entry = torch.repeat_interleave(torch.arange(self.rows, device=dev), counts)
        start = torch.cumsum(counts, 0) - counts
        j = torch.arange(int(counts.sum()), device=dev) - start[row_of_entry]
        pg = self.page_table[depth][row_of_entry, (j // ps)].long()
        return (pg * ps + j % ps).to(torch.int32)

    def assign_rows(self, depth: int, rows: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        """Like :meth:`assign_prefill` for a subset of rows (request admission while other rows keep decoding):
        ``rows [n]`` get ``counts [n]`` entries each; the other rows' lengths and pages are untouched.  The rows
        must be empty at this depth (see :meth:`free_rows`).  Returns the slots of the entries, row-major."""
        ps = self.page_size
        dev = self.len[depth].device
        rows = rows.to(device=dev, dtype=torch.int64)
        counts = counts.to(device=dev, dtype=torch.int64)
        need = (counts + ps - 1) // ps
        total = int(need.sum())
        free = int(self.free_count[depth])
        if total > free or int(need.max() if need.numel() else 0) > self.max_pages[depth]:
            raise RuntimeError(f"KV pool of depth {depth} too small: need {total} pages, {free} free")
        first = torch.cumsum(need, 0) - need
        which = torch.repeat_interleave(torch.arange(rows.numel(), device=dev), need)
        rank = torch.arange(total, device=dev)
        page_ids = self.free_stack[depth][(free - 1 - rank).long()]
        col = rank - first[which]
        self.page_table[depth][rows[which], col] = page_ids
        self.free_count[depth].fill_(free - total)
        self.len[depth][rows] = counts.to(torch.int32)
        which_e = torch.repeat_interleave(torch.arange(rows.numel(), device=dev), counts)
        start = torch.cumsum(counts, 0) - counts
        j = torch.arange(int(counts.sum()), device=dev) - start[which_e]
        pg = self.page_table[depth][rows[which_e], (j // ps)].long()
        return (pg * ps + j % ps).to(torch.int32)

    def free_rows(self, rows: torch.Tensor) -> int:
        """Return every page of ``rows`` (all depths) to the free stacks and clear their lengths.  Call between
        ticks.  Returns the number of pages released."""
        ps = self.page_size
        released = 0
        for d in range(self.n_depths):
            dev = self.len[d].device
            r = rows.to(device=dev, dtype=torch.int64)
            n = (self.len[d][r].to(torch.int64) + ps - 1) // ps
            total = int(n.sum())
            if total:
                which = torch.repeat_interleave(r, n)
                first = torch.cumsum(n, 0) - n
                col = torch.arange(total, device=dev) - torch.repeat_interleave(first, n)
                pages = self.page_table[d][which, col]
                free = int(self.free_count[d])
                self.free_stack[d][free:free + total] = pages
                self.free_count[d].fill_(free + total)
                released += total
            self.len[d][r] = 0
        return released

    def pages_in_use(self, depth: int) -> int:
        return self.n_pages[depth] - int(self.free_count[depth])
