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

import os
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


# ================================================================================================
# Parameter-sharded training (ZeRO-3 / FSDP)
# ================================================================================================
#
# ``shard_model`` cuts a model into *units* - the token embedding (with the tied LM head) and every decoder
# layer - and leaves on each rank 1/world of every unit's large matrices (bf16 shard + fp32 master weights and
# Adam moments of that shard).  Small tensors (norm gains, decider MLP ...) stay replicated and are handled by
# :class:`~tah_b200.parallel.zero.ZeroAdamW`, like DeepSpeed's parameter-persistence threshold.
#
# A unit's full bf16 parameters exist only inside a *gather buffer* in symmetric memory while the unit is
# in use: two buffers alternate between consecutive layers, the embedding has one of its own.  Hooks on the
# decoder layers drive the schedule
#
#   forward  (every pass): before layer i    gather i (if not prefetched), prefetch i + 1 on the side stream;
#                                            the first tcgen05 GEMM of the layer waits on the landing flags in
#                                            its TMA producer (no separate all-gather step);
#   backward (every pass): before layer i    re-gather i into the SAME buffer (autograd's saved weight views
#                                            point there), prefetch i - 1; an explicit flag-wait kernel gates
#                                            the library GEMMs of the backward;
#   gradients: a parameter's gradient reaches ``p.grad`` once per micro-batch, after the backward of its LAST
#              pass (autograd sums the passes first); ``p.grad`` is a view into one of two rotating unit-sized
#              gradient buffers in symmetric memory; when every parameter of a unit has reported, the
#              reduce-scatter kernel (``csrc/optim.cu``, phase 2: peer loads or ``multimem.ld_reduce``, fp32
#              accumulation into this rank's shard) runs on the side stream under the rest of the backward pass;
#   step:      global gradient norm over the sharded and the replicated part, then AdamW on every fp32 master
#              shard, bf16 written back to the local shard (the next gather distributes it).
#
# Reference behaviour: DeepSpeed ZeRO-3 through accelerate (``script/recipes/accelerate_configs/zero3.yaml``).
# On CPU (gloo) the same schedule runs with ``all_gather`` / ``all_reduce`` in place of the kernels, which is
# what the multi-process CPU test exercises.

import contextlib
import ctypes
import os

from tah_b200.parallel.zero import ZeroAdamW


class _Unit:
    def __init__(self, name: str, params: List[torch.nn.Parameter], world: int, buffer: int):
        self.name, self.params, self.buffer = name, params, buffer
        self.trainable = all(p.requires_grad for p in params)
        if not self.trainable and any(p.requires_grad for p in params):
            raise NotImplementedError(f"unit {name}: a mix of frozen and trainable sharded parameters is not supported")
        self.offsets, off = [], 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + 7) // 8 * 8                 # 16-byte aligned starts
        align = 8 * world
        self.numel = (off + align - 1) // align * align
        self.shard = self.numel // world
        self.pending = 0                                    # gradients still to arrive this micro-batch
        self.prepared = False                               # p.grad points into the unit's gradient buffer
        self.fwd_calls = 0                                  # forward passes of this micro-batch not yet back-propagated
        self.rs_done: Optional[torch.cuda.Event] = None


class FsdpState:
    """Sharded parameters of one model + the gather / reduce-scatter schedule (see the block comment above)."""

    def __init__(self, model, group, device: torch.device, min_shard_numel: int = 1 << 16, use_multicast: bool = True):
        self.model, self.group, self.device = model, group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.cuda = device.type == "cuda"
        base = model.simple_base_model if hasattr(model, "simple_base_model") else model
        layers = list(base.model.layers)
        big = lambda p: p.numel() >= min_shard_numel and p.dim() >= 2
        self.units: List[_Unit] = []
        emb = [p for p in [base.model.embed_tokens.weight] + ([base.lm_head.weight] if base.lm_head is not None else [])
               if big(p)]
        if emb:
            self.units.append(_Unit("embed", emb, self.world, buffer=2))
        self.layer_unit = {}
        for i, layer in enumerate(layers):
            ps = [p for p in layer.parameters() if big(p)]
            if ps:
                self.layer_unit[i] = len(self.units)
                self.units.append(_Unit(f"layer{i}", ps, self.world, buffer=i % 2))
        self.sharded_ids = {id(p) for u in self.units for p in u.params}
        self.dtype = self.units[0].params[0].dtype
        self._alloc(use_multicast)
        # move every unit's parameters into shards; the parameters become views into their gather buffer
        for u in self.units:
            flat = torch.zeros(u.numel, dtype=self.dtype, device=device)
            for p, off in zip(u.params, u.offsets):
                flat[off:off + p.numel()].copy_(p.detach().reshape(-1))
            u.shard_param = flat[self.rank * u.shard:(self.rank + 1) * u.shard].clone()
            if u.trainable:
                u.master = u.shard_param.float()
                u.m = torch.zeros_like(u.master)
                u.v = torch.zeros_like(u.master)
                u.gacc = torch.zeros_like(u.master)
            buf = self.gbuf[u.buffer]
            for p, off in zip(u.params, u.offsets):
                p.data = buf[off:off + p.numel()].view(p.shape)
            del flat
        self.resident = {0: None, 1: None, 2: None}          # buffer -> unit index whose parameters it holds
        self.inflight = {}                                   # unit index -> use number of its pending gather
        # TAH_B200_FSDP_SERIAL=1 puts the gathers and reduce-scatters on the compute stream (nothing overlaps): the
        # reference point for the hidden-communication fraction that the training benchmark reports
        self.serial = os.environ.get("TAH_B200_FSDP_SERIAL", "0") == "1"
        self.side = None if not self.cuda else (torch.cuda.current_stream(device) if self.serial
                                                else torch.cuda.Stream(device=device))
        self._hooks = []
        for i, layer in enumerate(layers):
            if i in self.layer_unit:
                self._hooks.append(layer.register_forward_pre_hook(self._make_fwd_hook(i)))
                self._hooks.append(layer.register_forward_hook(self._after_layer_forward))
                self._hooks.append(layer.register_full_backward_pre_hook(self._make_bwd_hook(i)))
        self._hooks.append(model.register_forward_pre_hook(lambda m, a: self._before_model_forward()))
        for ui, u in enumerate(self.units):
            if u.trainable:
                for p in u.params:
                    self._hooks.append(p.register_post_accumulate_grad_hook(self._make_grad_hook(ui)))
        self.n_layers = len(layers)
        self.stats = {"gathers": 0, "gather_bytes": 0, "reduce_scatters": 0, "prefetched": 0}

    # ---- buffers --------------------------------------------------------------------------------------
    def _alloc(self, use_multicast: bool) -> None:
        cap_layer = max([u.numel for u in self.units if u.buffer < 2] or [8])
        cap_embed = max([u.numel for u in self.units if u.buffer == 2] or [8])
        caps = [cap_layer, cap_layer, cap_embed]
        self.mc, self.gmc = [0, 0, 0], [0, 0, 0]
        self._gradbuf_free = {}
        if self.cuda and self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            try:
                symm_mem.enable_symm_mem_for_group(self.group.group_name)
            except Exception:
                pass
            self._keep = []

            def symm(n, dt):
                t = symm_mem.empty(n, dtype=dt, device=self.device)
                t.zero_()
                h = symm_mem.rendezvous(t, self.group)
                self._keep.append((t, h))
                return t, [int(p) for p in h.buffer_ptrs], int(getattr(h, "multicast_ptr", 0) or 0)

            self.gbuf, self.gbuf_ptrs, self.gradbuf, self.grad_ptrs = [], [], [], []
            for b, cap in enumerate(caps):
                t, ptrs, mc = symm(cap, self.dtype)
                self.gbuf.append(t)
                self.gbuf_ptrs.append(ptrs)
                self.mc[b] = mc if use_multicast else 0
                t, ptrs, mc = symm(cap, self.dtype)
                self.gradbuf.append(t)
                self.grad_ptrs.append(ptrs)
                self.gmc[b] = mc if use_multicast else 0
            # per buffer: landed flags (words 0..7) and ready flags (words 8..15), as shard_gather_push_kernel wants
            self._gflags, self.gflag_ptrs, _ = symm(3 * 16, torch.int32)
            self._rsflags, self.rsflag_ptrs, _ = symm(148 * self.world, torch.int32)
            self._rs_epoch = torch.zeros(148, dtype=torch.int32, device=self.device)
            self._target = torch.zeros(3, 8, dtype=torch.int32, device=self.device)
            self._scratch = torch.zeros(3, 8, dtype=torch.int32, device=self.device)
            self._pstate = torch.zeros(3, 4, dtype=torch.int32, device=self.device)
            self._uses = [0, 0, 0]
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
        else:
            self.gbuf = [torch.zeros(c, dtype=self.dtype, device=self.device) for c in caps]
            self.gradbuf = [torch.zeros(c, dtype=self.dtype, device=self.device) for c in caps]
        if self.cuda:
            # local flags for the one-rank form of the AdamW kernel (it ends with a flag barrier)
            self._lflags = torch.zeros(148, dtype=torch.int32, device=self.device)
            self._lepoch = torch.zeros(148, dtype=torch.int32, device=self.device)
            self._norm = torch.zeros(1, dtype=torch.float32, device=self.device)

    # ---- gather ---------------------------------------------------------------------------------------
    def _issue_gather(self, ui: int) -> None:
        """Start filling unit ``ui``'s buffer on every rank.  On CUDA the push kernel runs on the side stream
        behind everything that is on the current stream NOW: the buffer's last reader (the layer two steps
        back, or the optimizer update of the shard) is already enqueued there, the layer about to run is not,
        so the copy overlaps it.  The kernel itself waits until every peer has released the buffer."""
        u = self.units[ui]
        b = u.buffer
        self.stats["gathers"] += 1
        self.stats["gather_bytes"] += u.numel * 2 * (self.world - 1) // self.world
        if not (self.cuda and self.world > 1):
            if self.world > 1:
                dist.all_gather_into_tensor(self.gbuf[b][:u.numel], u.shard_param, group=self.group)
            else:
                self.gbuf[b][:u.numel].copy_(u.shard_param)
            self.resident[b] = ui
            return
        off = self.rank * u.shard * 2
        self.side.wait_stream(torch.cuda.current_stream(self.device))
        dst = [p + off for p in self.gbuf_ptrs[b]]
        mc = self.mc[b] + off if self.mc[b] else 0
        landed = [p + b * 64 for p in self.gflag_ptrs]
        ready = [p + b * 64 + 32 for p in self.gflag_ptrs]
        with torch.cuda.stream(self.side):
            K.shard_gather_push(u.shard_param, dst, mc, landed, ready, self._scratch[b], self._pstate[b], self.rank,
                                self.world, PUSH_GRID)
        self._uses[b] += 1
        self.inflight[ui] = self._uses[b]
        self.resident[b] = None

    def _require(self, ui: int, fused_wait: bool) -> None:
        """Make unit ``ui``'s parameters usable by the kernels that follow on the current stream."""
        u = self.units[ui]
        b = u.buffer
        if self.resident[b] == ui and ui not in self.inflight:
            return
        if ui in self.inflight:
            self.stats["prefetched"] += 1
        else:
            self._issue_gather(ui)
        if self.cuda and self.world > 1:
            use = self.inflight.pop(ui)
            self._target[b, :self.world] = use * PUSH_GRID
            flags = self._gflags[b * 16:b * 16 + self.world]
            if fused_wait:
                K.set_pending_gemm_wait((flags, self._target[b, :self.world]))   # the next tcgen05 GEMM waits itself
            else:
                K.wait_flags(flags, self._target[b, :self.world])
        self.resident[b] = ui

    def _prefetch(self, ui: Optional[int]) -> None:
        if ui is None or not (self.cuda and self.world > 1):
            return
        u = self.units[ui]
        if self.resident[u.buffer] == ui or ui in self.inflight:
            return
        self._issue_gather(ui)

    def _before_model_forward(self) -> None:
        if self.units and self.units[0].name == "embed":
            self._require(0, fused_wait=False)               # embedding / LM head stay gathered for the whole step

    def _make_fwd_hook(self, i: int):
        ui = self.layer_unit[i]

        def pre(module, args):
            fused = self.cuda and os.environ.get("TAH_B200_FORCE_TORCH", "0") != "1"
            self._require(ui, fused_wait=fused)
            if torch.is_grad_enabled():
                self.units[ui].fwd_calls += 1
            self._prefetch(self.layer_unit.get(i + 1))
        return pre

    def _after_layer_forward(self, module, args, output) -> None:
        if K.clear_pending_gemm_wait():
            raise RuntimeError("parameter-sharded forward: no tcgen05 GEMM of the layer took the gather wait "
                               "(the layer ran on another path); results of this pass are not reliable")

    def _make_bwd_hook(self, i: int):
        ui = self.layer_unit[i]

        def pre(module, grad_output):
            u = self.units[ui]
            self._require(ui, fused_wait=False)              # library GEMMs follow: gate them with the wait kernel
            self._prefetch(self.layer_unit.get(i - 1))
            u.fwd_calls -= 1
            if u.fwd_calls <= 0 and u.trainable:
                self._prepare_grads(ui)                      # the parameter gradients arrive during this backward
        return pre

    # ---- gradients ------------------------------------------------------------------------------------
    def _grad_buffer(self, ui: int) -> torch.Tensor:
        """The unit's (zeroed) gradient buffer, once its previous reduce-scatter has finished reading it."""
        u = self.units[ui]
        prev = self._gradbuf_free.get(u.buffer)
        if prev is not None:
            torch.cuda.current_stream(self.device).wait_event(prev)
        gb = self.gradbuf[u.buffer]
        gb[:u.numel].zero_()
        return gb

    def _prepare_grads(self, ui: int) -> None:
        """Point ``p.grad`` of the unit's parameters into its gradient buffer.  Gradients that arrived earlier
        (parameters used by later passes only, e.g. the adapter) are moved in."""
        u = self.units[ui]
        gb = self._grad_buffer(ui)
        pending = 0
        for p, off in zip(u.params, u.offsets):
            view = gb[off:off + p.numel()].view(p.shape)
            if p.grad is not None:
                view.copy_(p.grad)
            else:
                pending += 1
            p.grad = view
        u.pending = pending
        u.prepared = True
        if pending == 0:
            self._reduce_scatter(ui)

    def _make_grad_hook(self, ui: int):
        def hook(param):
            u = self.units[ui]
            if not getattr(u, "prepared", False):
                if u.name == "embed":                        # no layer hook prepares this unit
                    self._adopt_stray_grads(ui)
                return                                       # early arrival: _prepare_grads moves it in
            u.pending -= 1
            if u.pending == 0:
                self._reduce_scatter(ui)
        return hook

    def _adopt_stray_grads(self, ui: int) -> None:
        u = self.units[ui]
        if any(p.grad is None for p in u.params):
            return
        gb = self._grad_buffer(ui)
        for p, off in zip(u.params, u.offsets):
            gb[off:off + p.numel()].copy_(p.grad.reshape(-1))
        self._reduce_scatter(ui)

    def _reduce_scatter(self, ui: int) -> None:
        """Sum unit ``ui``'s gradient buffer over the ranks and add this rank's shard (x 1/world) to ``gacc``."""
        u = self.units[ui]
        b = u.buffer
        u.prepared = False
        u.pending = 0
        self.stats["reduce_scatters"] += 1
        lo, hi = self.rank * u.shard, (self.rank + 1) * u.shard
        if not (self.cuda and self.world > 1):
            g = self.gradbuf[b][:u.numel].float()
            if self.world > 1:
                dist.all_reduce(g, group=self.group)
            u.gacc.add_(g[lo:hi], alpha=1.0 / self.world)
        else:
            self.side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.side):
                self._zero_step(2, self.grad_ptrs[b], self.grad_ptrs[b], self.gmc[b], 0, u.gacc, u.gacc, u.gacc, u.gacc,
                                self._norm, self.rsflag_ptrs, self._rs_epoch, lo, hi, self.rank, self.world,
                                scale=1.0 / self.world)
                done = torch.cuda.Event()
                done.record(self.side)
            self._gradbuf_free[b] = done
        for p in u.params:
            p.grad = None

    def _zero_step(self, phase, grad_ptrs, param_ptrs, mc_grad, mc_param, gshard, master, m, v, norm_sq, flag_ptrs, epoch,
                   lo, hi, rank, world, scale=1.0, lr=0.0, b1=0.9, b2=0.999, eps=1e-8, wd=0.0, bc1=1.0, bc2=1.0,
                   max_norm=0.0):
        n = len(grad_ptrs)
        arr = lambda ptrs: (ctypes.c_void_p * n)(*ptrs)
        cf, ci, cll, cvp = ctypes.c_float, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
        grid = max(1, min(148, ((hi - lo) // 8 + 255) // 256))
        rc = K.lib().tahb_zero_step(ci(phase), arr(grad_ptrs), arr(param_ptrs), cvp(mc_grad), cvp(mc_param),
                                    cvp(gshard.data_ptr()), cvp(master.data_ptr()), cvp(m.data_ptr()), cvp(v.data_ptr()),
                                    cvp(norm_sq.data_ptr()), arr(flag_ptrs), cvp(epoch.data_ptr()),
                                    cvp(K.status_word(self.device).data_ptr()), cll(lo), cll(hi), ci(rank), ci(world),
                                    cf(scale), cf(lr), cf(b1), cf(b2), cf(eps), cf(wd), cf(bc1), cf(bc2), cf(max_norm),
                                    ci(grid), cvp(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(f"tahb_zero_step phase {phase} failed (code {rc})")

    # ---- whole-model views ----------------------------------------------------------------------------
    @contextlib.contextmanager
    def materialized(self):
        """All ranks: temporarily give every sharded parameter its own full tensor (for saving a checkpoint or
        handing the model to the inference engine)."""
        saved = []
        for ui, u in enumerate(self.units):
            self.inflight.pop(ui, None)
            self.resident[u.buffer] = None
            self._require(ui, fused_wait=False)
            if self.cuda:
                torch.cuda.synchronize(self.device)
            for p, off in zip(u.params, u.offsets):
                saved.append((p, p.data))
                p.data = self.gbuf[u.buffer][off:off + p.numel()].view(p.shape).clone()
        try:
            yield self.model
        finally:
            for p, old in saved:
                p.data = old
            self.resident = {0: None, 1: None, 2: None}

    def sharded_param_bytes(self) -> int:
        return sum(u.numel * u.shard_param.element_size() for u in self.units)


def shard_model(model, group=None, device: Optional[torch.device] = None, min_shard_numel: int = 1 << 16,
                use_multicast: bool = True) -> FsdpState:
    """Shard ``model``'s large matrices over ``group`` (ZeRO-3); returns the state, also kept as ``model._fsdp``."""
    group = group if group is not None else dist.group.WORLD
    device = device if device is not None else next(model.parameters()).device
    state = FsdpState(model, group, device, min_shard_numel, use_multicast)
    model._fsdp = state
    return state


class FsdpAdamW:
    """AdamW over a :func:`shard_model`-ed model: the sharded units update their own fp32 master shards, the small
    replicated parameters go through :class:`ZeroAdamW`; one global gradient norm clips both."""

    def __init__(self, model, lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: float = 0.0, use_multicast: bool = True, no_decay=None):
        self.state: FsdpState = model._fsdp
        st = self.state
        small = [p for p in model.parameters() if p.requires_grad and id(p) not in st.sharded_ids]
        self.small = ZeroAdamW(small, group=st.group if st.world > 1 else None, lr=lr, betas=betas, eps=eps,
                               weight_decay=weight_decay, max_grad_norm=max_grad_norm, use_multicast=use_multicast,
                               no_decay=no_decay) if small else None
        self.lr, self.betas, self.eps, self.weight_decay, self.max_grad_norm = lr, betas, eps, weight_decay, max_grad_norm
        self.step_count = 0
        self.last_grad_norm: Optional[torch.Tensor] = None

    def zero_grad(self, set_to_none: bool = False) -> None:
        if self.small is not None:
            self.small.zero_grad()

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None) -> torch.Tensor:
        st = self.state
        self.step_count += 1
        lr = self.lr if lr is None else lr
        b1, b2 = self.betas
        bc1, bc2 = 1.0 - b1 ** self.step_count, 1.0 - b2 ** self.step_count
        units = [u for u in st.units if u.trainable]
        for ui, u in enumerate(st.units):                     # a unit whose gradients never all arrived (unused branch)
            if u.trainable and u.prepared:
                st._reduce_scatter(ui)
            u.fwd_calls = 0
        if st.cuda and st.world > 1:
            torch.cuda.current_stream(st.device).wait_stream(st.side)        # every reduce-scatter has landed
        # squared norm of the sharded part (this rank's shards), handed to the replicated part's all-reduce
        if st.cuda:
            st._norm.zero_()
            for u in units:
                if grad_scale != 1.0:
                    u.gacc.mul_(grad_scale)
                K.lib().tahb_sumsq_f32(ctypes.c_void_p(u.gacc.data_ptr()), ctypes.c_longlong(u.gacc.numel()),
                                       ctypes.c_void_p(st._norm.data_ptr()),
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            extra = st._norm
        else:
            extra = torch.zeros(1, dtype=torch.float32, device=st.device)
            for u in units:
                if grad_scale != 1.0:
                    u.gacc.mul_(grad_scale)
                extra += (u.gacc * u.gacc).sum()
        if self.small is not None:
            norm = self.small.step(grad_scale=grad_scale, lr=lr, extra_norm_sq=extra)
            total_sq = self.small.norm_sq if st.cuda and self.small.cuda else norm.reshape(1) ** 2
        else:
            total_sq = extra.clone()
            if st.world > 1:
                dist.all_reduce(total_sq, group=st.group)
            norm = total_sq.sqrt()[0]
        for u in units:
            if st.cuda:
                # AdamW kernel in its one-rank form: the "parameter buffer" is the local bf16 shard
                base = u.shard_param.data_ptr() - st.rank * u.shard * 2
                lo, hi = st.rank * u.shard, (st.rank + 1) * u.shard
                st._zero_step(1, [base], [base], 0, 0, u.gacc, u.master, u.m, u.v, total_sq, [st._lflags.data_ptr()],
                              st._lepoch, lo, hi, 0, 1, scale=1.0, lr=lr, b1=b1, b2=b2, eps=self.eps, wd=self.weight_decay,
                              bc1=bc1, bc2=bc2, max_norm=self.max_grad_norm)
            else:
                g = u.gacc
                if self.max_grad_norm > 0:
                    g = g * torch.clamp(self.max_grad_norm / (total_sq.sqrt() + 1e-6), max=1.0)
                u.m.mul_(b1).add_(g, alpha=1 - b1)
                u.v.mul_(b2).addcmul_(g, g, value=1 - b2)
                upd = (u.m / bc1) / ((u.v / bc2).sqrt() + self.eps)
                u.master.mul_(1 - lr * self.weight_decay).add_(upd, alpha=-lr)
                u.shard_param.copy_(u.master.to(u.shard_param.dtype))
            u.gacc.zero_()
        st.resident = {0: None, 1: None, 2: None}              # the shards changed: gather again on next use
        st.inflight.clear()
        self.last_grad_norm = norm
        return norm

    def state_dict(self) -> dict:
        st = self.state
        return {"step": self.step_count, "rank": st.rank, "world": st.world,
                "units": {u.name: {"master": u.master.cpu(), "m": u.m.cpu(), "v": u.v.cpu()} for u in st.units if u.trainable},
                "small": self.small.state_dict() if self.small is not None else None}

    def load_state_dict(self, sd: dict) -> None:
        st = self.state
        if sd["world"] != st.world or sd["rank"] != st.rank:
            raise ValueError("optimizer shard layout differs from the checkpoint (world size changed?)")
        self.step_count = int(sd["step"])
        for u in st.units:
            if u.trainable and u.name in sd["units"]:
                for k in ("master", "m", "v"):
                    getattr(u, k).copy_(sd["units"][u.name][k].to(st.device))
                u.shard_param.copy_(u.master.to(u.shard_param.dtype))
        if self.small is not None and sd.get("small") is not None:
            self.small.load_state_dict(sd["small"])
        st.resident = {0: None, 1: None, 2: None}
