"""Tensor parallelism over one NVLink/NVSwitch node.

One process per GPU (``torch.distributed`` / NCCL for the plumbing and the cold paths).  The
hot path does not call NCCL: activations that cross ranks live in *symmetric memory* (the same
allocation mapped by every rank, plus an NVLS multicast address when the fabric supports it) and
the hand-written kernel in ``csrc/comm.cu`` performs

    all-reduce of the row-parallel partial results + residual add + RMSNorm + broadcast

in a single launch per rank, synchronising with flags it polls itself (bounded waits).

Sharding plan (Megatron style, built in :class:`tah_b200.engine.weights.EngineWeights`):
QKV and gate/up are column-parallel (heads / intermediate channels split), O and down are
row-parallel, the LM head is vocabulary-parallel, KV caches hold the local heads only, and the
residual stream stays sharded by token rows on the rank that owns them.

The reference has no tensor parallelism of its own: its ``tah`` backend ignores ``tp_size``
(reference ``tah/evaluate/backends.py:155``) and only the external sglang backend shards.
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from tah_b200.ops import cuda as K

MAX_GRID = 148          # CTAs of the fused kernel must all be resident: they wait for their peers


class TensorParallel:
    def __init__(self, group, device: torch.device, hidden_size: Optional[int] = None, max_tokens: int = 0,
                 use_multicast: Optional[bool] = None):
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.hidden = hidden_size
        self.max_tokens = 0
        self.partial = self.xout = None
        self._symm = None
        if use_multicast is None:
            use_multicast = os.environ.get("TAH_B200_NVLS", "1") != "0"
        self.use_multicast = use_multicast
        if hidden_size is not None and max_tokens > 0:
            self.allocate(hidden_size, max_tokens)

    # ------------------------------------------------------------------------------------------
    def allocate(self, hidden_size: int, max_tokens: int) -> None:
        """(Re)create the symmetric buffers: partial [T, H], xout [T, H] (bf16) and the flag array."""
        import torch.distributed._symmetric_memory as symm_mem
        if self.partial is not None and self.hidden == hidden_size and self.max_tokens >= max_tokens:
            return
        self.hidden, self.max_tokens = hidden_size, max_tokens
        try:
            symm_mem.enable_symm_mem_for_group(self.group.group_name)
        except Exception:
            pass
        mk = lambda n, dt: symm_mem.empty(n, dtype=dt, device=self.device)
        self._partial_flat = mk(max_tokens * hidden_size, torch.bfloat16)
        self._xout_flat = mk(max_tokens * hidden_size, torch.bfloat16)
        self._flags = mk(MAX_GRID * self.world_size, torch.int32)
        self._flags.zero_()
        self._partial_flat.zero_()
        self._xout_flat.zero_()
        hp = symm_mem.rendezvous(self._partial_flat, self.group)
        hx = symm_mem.rendezvous(self._xout_flat, self.group)
        hf = symm_mem.rendezvous(self._flags, self.group)
        self._handles = (hp, hx, hf)
        self.partial_ptrs = [int(p) for p in hp.buffer_ptrs]
        self.xout_ptrs = [int(p) for p in hx.buffer_ptrs]
        self.flag_ptrs = [int(p) for p in hf.buffer_ptrs]
        mc_p = int(getattr(hp, "multicast_ptr", 0) or 0)
        mc_x = int(getattr(hx, "multicast_ptr", 0) or 0)
        if not self.use_multicast or mc_p == 0 or mc_x == 0:
            mc_p = mc_x = 0
        self.mc_partial, self.mc_xout = mc_p, mc_x
        self.partial = self._partial_flat.view(max_tokens, hidden_size)
        self.xout = self._xout_flat.view(max_tokens, hidden_size)
        self.epoch = torch.zeros(MAX_GRID, dtype=torch.int32, device=self.device)
        # push path (decode ticks): slots [world][rows_per_rank][H] filled by the peers' GEMM epilogues,
        # an arrival counter (word 0) and per-owner landing flags (words 8..8+world) in symmetric memory,
        # and local targets: word 0 = counter target, word 1 = CTA arrivals, words 8.. = flag targets
        self._slot_flat = mk(max_tokens * hidden_size, torch.bfloat16)
        self._pushflags = mk(16, torch.int32)
        self._pushflags.zero_()
        hs = symm_mem.rendezvous(self._slot_flat, self.group)
        hq = symm_mem.rendezvous(self._pushflags, self.group)
        self._handles = self._handles + (hs, hq)
        self.slot_ptrs = [int(p) for p in hs.buffer_ptrs]
        self.cnt_ptrs = [int(p) for p in hq.buffer_ptrs]
        self.xflag_ptrs = [int(p) + 8 * 4 for p in hq.buffer_ptrs]
        self._pstate = torch.zeros(16, dtype=torch.int32, device=self.device)
        self.xflag_local = self._pushflags[8:8 + self.world_size]
        self.xtarget = self._pstate[8:8 + self.world_size]
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    # ------------------------------------------------------------------------------------------
    def rows_of(self, M: int) -> Tuple[int, int]:
        per = (M + self.world_size - 1) // self.world_size
        lo = min(M, self.rank * per)
        return lo, min(M, lo + per)

    def fused_reduce_norm(self, M: int, h: torch.Tensor, ln_w: torch.Tensor, eps: float,
                          add_residual: bool = True) -> torch.Tensor:
        """``self.partial[:M]`` holds this rank's partial result.  Afterwards ``h`` (rows owned by
        this rank) is the updated residual stream and the returned ``xout[:M]`` the RMS-normalised
        rows of all ranks."""
        per = (M + self.world_size - 1) // self.world_size
        grid = max(1, min(MAX_GRID, per))
        K.fused_reduce_residual_norm(self.partial_ptrs, self.xout_ptrs, self.mc_partial, self.mc_xout, h, ln_w,
                                     self.flag_ptrs, self.epoch, M, self.hidden, self.rank, self.world_size, eps,
                                     add_residual, grid)
        return self.xout[:M]

    # ---- push path: GEMM epilogue = reduce-scatter, owner kernel = sum + norm + broadcast ------------
    def push_desc(self, M: int):
        """Arguments that turn a row-parallel GEMM's epilogue into peer stores into the owners'
        slots, or None when ``M`` rows cannot be dealt out in 16-row blocks."""
        if self.hidden % 128 or M % (16 * self.world_size) or M > self.max_tokens:
            return None
        return (self.slot_ptrs, self.cnt_ptrs, self.rank, M // self.world_size)

    @property
    def wait_desc(self):
        """(flags, targets) that consumers of ``xout`` pass as ``tp_wait`` after :meth:`push_reduce_norm`."""
        return (self.xflag_local, self.xtarget)

    def push_reduce_norm(self, M: int, h: torch.Tensor, ln_w: torch.Tensor, eps: float, add_residual: bool = True,
                         final_wait: bool = False, tap=None) -> torch.Tensor:
        """Owner side after a ``tp_push`` GEMM on every rank.  The returned ``xout[:M]`` is complete
        on this rank only once the flags in :attr:`wait_desc` have reached their targets: consumers
        either wait themselves (``tp_wait``) or ask for ``final_wait``.  ``tap = (buffer from alloc_taps, column
        offset in elements)``: that column block also receives the updated residual rows of all ranks, landed
        under the same flags."""
        rpr = M // self.world_size
        grid = max(1, min(MAX_GRID, rpr))
        kw = {}
        if tap is not None:
            tb, col = tap
            kw = dict(tap_ptrs=[p + 2 * col for p in tb.ptrs], mc_tap=tb.mc + 2 * col if tb.mc else 0,
                      tap_ld=tb.tensor.shape[1])
        K.push_reduce_norm_bcast(self._slot_flat, self._pushflags[0:1], self._pstate[0:1], self.xout_ptrs,
                                 self.mc_xout, self.xflag_ptrs, self.xtarget, self._pstate[1:2], h, ln_w, M,
                                 self.hidden, self.rank, self.world_size, rpr, eps, add_residual, final_wait, grid,
                                 **kw)
        return self.xout[:M]

    def alloc_taps(self, rows: int, width: int):
        """Symmetric ``[rows, width]`` bf16 buffer for hidden-state taps that the owner kernels fill on every rank
        (collective: every rank calls it with the same shape; one buffer per shape).  Returns an object with
        ``tensor`` (this rank's view), ``ptrs`` (every rank's address) and ``mc`` (multicast address or 0)."""
        import torch.distributed._symmetric_memory as symm_mem
        from types import SimpleNamespace
        cache = self.__dict__.setdefault("_tap_bufs", {})
        if (rows, width) in cache:
            return cache[(rows, width)]
        flat = symm_mem.empty(rows * width, dtype=torch.bfloat16, device=self.device)
        flat.zero_()
        ht = symm_mem.rendezvous(flat, self.group)
        mc = int(getattr(ht, "multicast_ptr", 0) or 0)
        tb = SimpleNamespace(tensor=flat.view(rows, width), ptrs=[int(p) for p in ht.buffer_ptrs],
                             mc=mc if self.use_multicast and self.mc_xout else 0, handle=ht)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        cache[(rows, width)] = tb
        return tb

    # ---- cold paths: NCCL -----------------------------------------------------------------------
    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.group)
        return t

    def all_gather_cat(self, t: torch.Tensor, dim: int = -1) -> torch.Tensor:
        parts = [torch.empty_like(t) for _ in range(self.world_size)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts, dim=dim)

    def gather_rows(self, h: torch.Tensor, M: int) -> torch.Tensor:
        """Full [M, H] residual stream from the row-sharded ``h`` (owners hold their rows)."""
        per = (M + self.world_size - 1) // self.world_size
        pad = h.new_zeros(per * self.world_size, h.shape[1])
        pad[:M] = h[:M]
        mine = pad[self.rank * per:(self.rank + 1) * per].contiguous()
        out = torch.empty_like(pad)
        dist.all_gather_into_tensor(out, mine, group=self.group)
        return out[:M]

    # ---- vocabulary-parallel arg-max / top-k merge: candidates exchanged by peer stores, merged locally -----
    def _merge_buffers(self, rows: int):
        """Symmetric exchange buffers for :meth:`merge_topk` (values / indices ``[2][world][rows][128]``, one
        arrival word per row and source rank) and the local per-row epoch counters."""
        cache = self.__dict__.setdefault("_merge", {})         # one set of buffers per row count
        st = cache.get(rows)
        if st is not None:
            return st
        import torch.distributed._symmetric_memory as symm_mem
        n = 2 * self.world_size * rows * 128
        xv = symm_mem.empty(n, dtype=torch.float32, device=self.device)
        xi = symm_mem.empty(n, dtype=torch.int32, device=self.device)
        ar = symm_mem.empty(rows * 8, dtype=torch.int32, device=self.device)      # [rows][8 sources]
        ar.zero_()
        hv, hi, ha = (symm_mem.rendezvous(t, self.group) for t in (xv, xi, ar))
        st = dict(rows=rows, keep=(xv, xi, ar, hv, hi, ha), xval=[int(p) for p in hv.buffer_ptrs],
                  xidx=[int(p) for p in hi.buffer_ptrs], arrive=[int(p) for p in ha.buffer_ptrs],
                  epoch=torch.zeros(rows, dtype=torch.int32, device=self.device))
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        cache[rows] = st
        return st

    def prepare_merge(self, rows: int) -> None:
        """Allocate the merge buffers ahead of a CUDA-graph capture (allocation is a collective)."""
        self._merge_buffers(rows)

    def merge_topk(self, vals: torch.Tensor, idx: torch.Tensor, vocab_lo: int, k: int):
        """Sorted global top-k (value desc, index asc) from every rank's sorted per-shard list (``vals`` fp32
        ``[B, k]``, ``idx`` int32 local indices): one kernel per rank that stores the candidates into every peer's
        exchange buffer, waits for theirs and merges (``tp_topk_merge_kernel`` in ``csrc/comm.cu``).  No NCCL."""
        B = vals.shape[0]
        st = self._merge_buffers(B)
        out_v = torch.empty(B, k, dtype=torch.float32, device=vals.device)
        out_i = torch.empty(B, k, dtype=torch.int32, device=vals.device)
        K.tp_topk_merge(st["xval"], st["xidx"], st["arrive"], st["epoch"], vals, idx, out_v, out_i, st["rows"], k,
                        self.rank, self.world_size, vocab_lo)
        return out_v, out_i

    def merge_argmax(self, best_val: torch.Tensor, best_idx: torch.Tensor, vocab_lo: int) -> torch.Tensor:
        """Global arg-max from per-shard (value, local index); the lowest global index wins ties."""
        return self.merge_topk(best_val.view(-1, 1), best_idx.view(-1, 1), vocab_lo, 1)[1].view(-1)

    # NCCL forms of the two merges: the baseline the kernel is tested against
    def merge_argmax_nccl(self, best_val: torch.Tensor, best_idx: torch.Tensor, vocab_lo: int) -> torch.Tensor:
        pack = torch.stack([best_val.float(), (best_idx + vocab_lo).float()], dim=-1)      # [B, 2]
        allp = torch.empty(self.world_size, *pack.shape, dtype=pack.dtype, device=pack.device)
        dist.all_gather_into_tensor(allp, pack.contiguous(), group=self.group)
        vals, idx = allp[..., 0], allp[..., 1]                                            # [ws, B]
        top = vals.max(dim=0, keepdim=True).values
        cand = torch.where(vals == top, idx, torch.full_like(idx, float("inf")))
        return cand.min(dim=0).values.to(torch.int32)

    def merge_topk_nccl(self, vals: torch.Tensor, idx: torch.Tensor, vocab_lo: int, k: int):
        gv = self.all_gather_cat(vals, dim=-1)
        gi = self.all_gather_cat((idx + vocab_lo).to(torch.int32), dim=-1)
        # order by value desc, index asc (the order the single-GPU kernel produces): stable sorts
        o1 = gi.argsort(dim=-1, stable=True)
        gv, gi = gv.gather(1, o1), gi.gather(1, o1)
        o2 = gv.argsort(dim=-1, descending=True, stable=True)[:, :k]
        return gv.gather(1, o2).contiguous(), gi.gather(1, o2).contiguous()
