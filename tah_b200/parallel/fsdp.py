"""Sharded parameters (ZeRO-3 / FSDP style) whose all-gather is consumed by the GEMM itself.

Every rank keeps ``1 / world`` of each weight matrix (a contiguous block of rows).  Ahead of the layer
that needs a matrix, :meth:`ShardedWeightStore.prefetch` launches the push kernel of ``csrc/comm.cu``
(``shard_gather_push_kernel``) on a side stream: each rank stores its shard into the gather buffer of
every rank over NVLink (``multimem.st`` or peer stores) and advances per-source landing flags.
:meth:`ShardedWeightStore.linear` then runs the tcgen05 GEMM whose TMA producer waits on those flags
before its first load, so the parameter all-gather has no kernel of its own on the critical path, no
NCCL call and no host synchronisation; it overlaps the layers before it.  Gather buffers are reused
round-robin; the push kernel exchanges "buffer free" flags with its peers before overwriting.

The reference trains with DeepSpeed ZeRO-2/3 through accelerate (reference
``script/recipes/accelerate_configs/zero2.yaml``, ``zero3.yaml``), i.e. NCCL all-gathers issued by the
framework before each layer.  The trainer of this repository uses :class:`tah_b200.parallel.zero.ZeroAdamW`
(ZeRO-2); this store is the parameter-sharding building block (forward path) for larger models.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from tah_b200.ops import cuda as K

PUSH_GRID = 64          # CTAs of the push kernel: co-resident on every rank, they wait for their peers


class ShardedWeightStore:
    def __init__(self, group, device: torch.device, weights: Sequence[torch.Tensor], n_buffers: int = 2,
                 use_multicast: bool = True):
        import torch.distributed._symmetric_memory as symm_mem
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.shapes = [tuple(w.shape) for w in weights]
        for F, Kd in self.shapes:
            if F % self.world or (F // self.world * Kd * 2) % 16:
                raise ValueError(f"weight {F}x{Kd} does not split into {self.world} 16-byte aligned row blocks")
        self.shards: List[torch.Tensor] = []
        for w in weights:
            per = w.shape[0] // self.world
            self.shards.append(w[self.rank * per:(self.rank + 1) * per].detach().to(device, torch.bfloat16).contiguous())
        self.n_buffers = n_buffers
        cap = max(F * Kd for F, Kd in self.shapes)
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:
            pass
        self._bufs, self._handles, self.buf_ptrs, self.buf_mc = [], [], [], []
        for _ in range(n_buffers):
            t = symm_mem.empty(cap, dtype=torch.bfloat16, device=device)
            t.zero_()
            h = symm_mem.rendezvous(t, group)
            self._bufs.append(t)
            self._handles.append(h)
            self.buf_ptrs.append([int(p) for p in h.buffer_ptrs])
            mc = int(getattr(h, "multicast_ptr", 0) or 0)
            self.buf_mc.append(mc if use_multicast else 0)
        # per buffer: landed flags at words 0..7, ready flags at words 8..15 (symmetric); local targets / state
        self._flags = symm_mem.empty(n_buffers * 16, dtype=torch.int32, device=device)
        self._flags.zero_()
        hf = symm_mem.rendezvous(self._flags, group)
        self._handles.append(hf)
        self.flag_ptrs = [int(p) for p in hf.buffer_ptrs]
        self._target = torch.zeros(n_buffers, 8, dtype=torch.int32, device=device)       # what the consumer waits for
        self._scratch = torch.zeros(n_buffers, 8, dtype=torch.int32, device=device)      # the kernel's own copy
        self._state = torch.zeros(n_buffers, 4, dtype=torch.int32, device=device)
        self._uses = [0] * n_buffers
        self._where = {}
        self._next = 0
        self._reader_done: List[Optional[torch.cuda.Event]] = [None] * n_buffers
        self.side = torch.cuda.Stream(device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)

    # ------------------------------------------------------------------------------------------
    def prefetch(self, i: int) -> None:
        """Start gathering weight ``i`` into the next buffer (asynchronous, side stream)."""
        b = self._next % self.n_buffers                  # buffers are used round-robin in prefetch order
        if any(bb == b for bb, _ in self._where.values()):
            raise RuntimeError(f"gather buffer {b} still holds a weight that has not been consumed "
                               f"(at most {self.n_buffers} prefetches may be outstanding)")
        self._next += 1
        F, Kd = self.shapes[i]
        shard = self.shards[i]
        off = self.rank * shard.numel() * 2
        if self._reader_done[b] is not None:
            self.side.wait_event(self._reader_done[b])
        else:
            self.side.wait_stream(torch.cuda.current_stream(self.device))
        dst = [ptrs + off for ptrs in self.buf_ptrs[b]]
        mc = self.buf_mc[b] + off if self.buf_mc[b] else 0
        landed = [p + b * 64 for p in self.flag_ptrs]
        ready = [p + b * 64 + 32 for p in self.flag_ptrs]
        with torch.cuda.stream(self.side):
            K.shard_gather_push(shard, dst, mc, landed, ready, self._scratch[b], self._state[b], self.rank, self.world,
                                PUSH_GRID)
        self._uses[b] += 1
        self._where[i] = (b, self._uses[b])

    def linear(self, x: torch.Tensor, i: int, **gemm_kwargs) -> torch.Tensor:
        """``x @ W_i^T`` on the gathered weight; the GEMM itself waits for the shards to land."""
        b, use = self._where.pop(i)
        F, Kd = self.shapes[i]
        w_full = self._bufs[b][:F * Kd].view(F, Kd)
        self._target[b, :self.world] = use * PUSH_GRID                      # ordered before the GEMM on this stream
        landed_local = self._flags[b * 16:b * 16 + self.world]
        out = K.gemm(x, w_full, tp_wait=(landed_local, self._target[b, :self.world]), **gemm_kwargs)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._reader_done[b] = ev
        return out
