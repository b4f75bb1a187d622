"""Tensor-parallel training of the TaH backbone (Megatron-style sharding of the decoder layers).

``shard_model_tp(model, group)`` cuts every decoder layer over the ranks of ``group``:

* column-parallel projections (fused QKV, fused gate/up): each rank keeps the rows of its attention heads / MLP
  channels (and the matching rows of the LoRA-B factors); their input passes through :class:`_CopyToTP` (identity
  forward, all-reduce of the gradient backward);
* row-parallel projections (O, down): each rank keeps the matching input columns (and the columns of LoRA-A); their
  output passes through :class:`_ReduceFromTP` (all-reduce forward, identity backward);
* attention runs on the rank's own heads (the KV cache of a pass holds those heads only);
* embeddings, norms, LM head, decider and loss stay replicated and are computed by every rank on the full hidden
  state, so the loss and the gradients of those parameters are identical on all ranks of the group.

A few replicated parameters see only their rank's part of the gradient (LoRA-A of the column-parallel projections,
LoRA-B of the row-parallel ones, the per-head q / k norm gains): :meth:`TPTrainState.sync_grads` all-reduces them once
per optimizer step.  :class:`TPOptimizer` wraps the data-parallel optimizer of the rank's DP group, calls
``sync_grads`` and corrects the global gradient norm for the sharded tensors.

The collectives are ``torch.distributed`` all-reduces (NCCL over NVLink on GPUs, gloo on CPU): this is the plain
form of tensor-parallel training, the fused NVLink kernels of ``tp.py`` serve inference.  The reference trains with
data parallelism only (``script/recipes/accelerate_configs/zero2.yaml``); tensor parallelism in training is what
long sequences on the 4B shapes need.
"""
from __future__ import annotations

import contextlib
import copy
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        y = x.contiguous().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


def tp_dp_groups(tp_size: int) -> Tuple[object, object, int, int]:
    """Process groups of a ``world = dp x tp`` layout with the tensor-parallel ranks adjacent (NVLink neighbours):
    returns ``(tp_group, dp_group, tp_rank, dp_rank)``.  Every rank must call it (group creation is collective)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % tp_size:
        raise ValueError(f"world size {world} is not a multiple of the tensor-parallel size {tp_size}")
    tp_group = dp_group = None
    for k in range(world // tp_size):
        ranks = list(range(k * tp_size, (k + 1) * tp_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            tp_group = g
    for j in range(tp_size):
        ranks = list(range(j, world, tp_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            dp_group = g
    return tp_group, dp_group, rank % tp_size, rank // tp_size


def _slice_rows(t: torch.Tensor, splits: List[int], rank: int, world: int) -> torch.Tensor:
    """Rows of a tensor that stacks ``splits`` blocks along dim 0: this rank's 1/world of every block."""
    parts, off = [], 0
    for s in splits:
        per = s // world
        parts.append(t[off + rank * per: off + (rank + 1) * per])
        off += s
    return torch.cat(parts, dim=0).contiguous()


class TPTrainState:
    """What :func:`shard_model_tp` did to a model: the group, the sharded tensors (for the gradient norm and for
    :meth:`materialized`), the replicated parameters whose gradients are partial, and the module hooks."""

    def __init__(self, model, group):
        self.model = model
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.sharded: List[Tuple[torch.nn.Parameter, str, List[int]]] = []     # (param, "rows" | "cols", row splits)
        self.partial_grad: List[torch.nn.Parameter] = []
        self.hooks = []
        self.full_cfg = None
        self.local_cfg = None

    # ---- gradients -------------------------------------------------------------------------------------
    def sync_grads(self) -> None:
        """All-reduce, over the tensor-parallel group, the gradients of the replicated parameters that only saw
        this rank's heads / channels.  Call once per optimizer step, after the last backward."""
        for p in self.partial_grad:
            if p.grad is not None:
                dist.all_reduce(p.grad, group=self.group)

    def extra_norm_sq(self) -> torch.Tensor:
        """Squared gradient norm of the OTHER ranks' shards: what a rank-local norm over this rank's parameters
        misses of the global norm (replicated parameters are counted once, by every rank alike)."""
        dev = self.sharded[0][0].device if self.sharded else torch.device("cpu")
        local = torch.zeros(1, dtype=torch.float32, device=dev)
        for p, _, _ in self.sharded:
            if p.grad is not None:
                local += p.grad.detach().float().pow(2).sum()
        total = local.clone()
        dist.all_reduce(total, group=self.group)
        return total - local

    # ---- full tensors for checkpoints ------------------------------------------------------------------
    def gather_full(self, p: torch.nn.Parameter, how: str, splits: List[int]) -> torch.Tensor:
        parts = [torch.empty_like(p.data) for _ in range(self.world)]
        dist.all_gather(parts, p.data.contiguous(), group=self.group)
        if how == "cols":
            return torch.cat(parts, dim=1)
        out, off = [], 0
        for s in splits:                                   # undo the per-block slicing of _slice_rows
            per = s // self.world
            out.extend(q[off:off + per] for q in parts)
            off += per
        return torch.cat(out, dim=0)

    @contextlib.contextmanager
    def materialized(self):
        """All ranks: temporarily give every sharded parameter its full tensor (and the layers their full head /
        channel counts), e.g. to save a checkpoint in the reference layout.  No training step inside."""
        saved = []
        for p, how, splits in self.sharded:
            saved.append((p, p.data))
            p.data = self.gather_full(p, how, splits)
        mods = _tp_modules(self.model)
        meta = []
        for layer in mods:
            at, mlp = layer.self_attn, layer.mlp
            meta.append((at.cfg, [(m, m.in_features, list(m.out_splits), m.out_features)
                                  for m in (at.qkv_proj, at.o_proj, mlp.gate_up_proj, mlp.down_proj)]))
            at.cfg = self.full_cfg
            w = self.world
            at.qkv_proj.out_splits = [s * w for s in at.qkv_proj.out_splits]
            mlp.gate_up_proj.out_splits = [s * w for s in mlp.gate_up_proj.out_splits]
            at.o_proj.in_features *= w
            mlp.down_proj.in_features *= w
            for m in (at.qkv_proj, mlp.gate_up_proj):
                m.out_features = sum(m.out_splits)
        try:
            yield
        finally:
            for p, data in saved:
                p.data = data
            for layer, (cfg, items) in zip(mods, meta):
                layer.self_attn.cfg = cfg
                for m, inf, outs, outf in items:
                    m.in_features, m.out_splits, m.out_features = inf, outs, outf


def _tp_modules(model):
    base = getattr(model, "simple_base_model", model)
    return list(base.model.layers)


def shard_model_tp(model, group) -> TPTrainState:
    """Shard the decoder layers of ``model`` (a ``TaHForCausalLM`` or the backbone) over ``group`` in place and
    install the communication hooks.  Every rank must hold the same full parameters before the call (they are
    broadcast from the group's first rank to make sure).  Returns the :class:`TPTrainState`, also stored as
    ``model._tp_train``."""
    base = getattr(model, "simple_base_model", model)
    st = TPTrainState(model, group)
    ws, rk = st.world, st.rank
    cfg = base.config
    if cfg.num_attention_heads % ws or cfg.num_key_value_heads % ws or cfg.intermediate_size % ws:
        raise ValueError(f"tensor-parallel size {ws} does not divide the model's heads / MLP channels")
    if getattr(model, "_fsdp", None) is not None:
        raise NotImplementedError("tensor-parallel training does not combine with parameter sharding (zero3)")
    src = dist.get_global_rank(group, 0)
    with torch.no_grad():
        for p in model.parameters():
            dist.broadcast(p.data, src=src, group=group)
    st.full_cfg = cfg
    local = copy.copy(cfg)
    local.num_attention_heads = cfg.num_attention_heads // ws
    local.num_key_value_heads = cfg.num_key_value_heads // ws
    local.intermediate_size = cfg.intermediate_size // ws
    st.local_cfg = local

    def column(lin):
        splits = list(lin.out_splits)
        with torch.no_grad():
            lin.weight.data = _slice_rows(lin.weight.data, splits, rk, ws)
            st.sharded.append((lin.weight, "rows", splits))
            if lin.adapted:
                for j, i in enumerate(lin.adapted):
                    b = lin.lora_B[j]
                    b.data = _slice_rows(b.data, [splits[i]], rk, ws)
                    st.sharded.append((b, "rows", [splits[i]]))
                st.partial_grad.append(lin.lora_A)          # replicated factor, gradient from this rank's rows only
        lin.out_splits = [s // ws for s in splits]
        lin.out_features = sum(lin.out_splits)
        st.hooks.append(lin.register_forward_pre_hook(lambda m, args: (_CopyToTP.apply(args[0], group),) + tuple(args[1:])))

    def row(lin):
        per = lin.in_features // ws
        with torch.no_grad():
            lin.weight.data = lin.weight.data[:, rk * per:(rk + 1) * per].contiguous()
            st.sharded.append((lin.weight, "cols", []))
            if lin.adapted:
                lin.lora_A.data = lin.lora_A.data[:, rk * per:(rk + 1) * per].contiguous()
                st.sharded.append((lin.lora_A, "cols", []))
                st.partial_grad.extend(lin.lora_B)          # replicated factors fed by this rank's partial product
        lin.in_features = per
        st.hooks.append(lin.register_forward_hook(lambda m, args, out: _ReduceFromTP.apply(out, group)))

    for layer in _tp_modules(model):
        at, mlp = layer.self_attn, layer.mlp
        column(at.qkv_proj)
        row(at.o_proj)
        column(mlp.gate_up_proj)
        row(mlp.down_proj)
        at.cfg = local
        st.partial_grad.extend([at.q_norm.weight, at.k_norm.weight])   # applied to this rank's heads only
    st.partial_grad = [p for p in st.partial_grad if p.requires_grad]
    st.sharded = [(p, how, sp) for p, how, sp in st.sharded]
    model._tp_train = st
    return st


class TPOptimizer:
    """The data-parallel optimizer of a rank under tensor parallelism.  ``inner`` is a ``ZeroAdamW`` over the rank's
    DP group (its ``norm_hook`` adds the other tensor-parallel ranks' shards to the clipping norm, exactly: the hook
    sees the rank-averaged gradient shard) or any optimizer with ``step`` / ``zero_grad`` (no norm correction).
    Before the inner step the partial gradients are summed over the tensor-parallel group."""

    def __init__(self, inner, state: TPTrainState):
        self.inner = inner
        self.state = state
        self._ranges = None
        params = getattr(inner, "params", None)
        if params is not None and hasattr(inner, "gshard"):
            where, off = {}, 0
            for p in params:
                where[id(p)] = (off, off + p.numel())
                off += p.numel()
            self._ranges = sorted(where[id(p)] for p, _, _ in state.sharded if id(p) in where)

    def _norm_hook(self, opt) -> torch.Tensor:
        """Share of the squared norm that this rank's optimizer misses: the sharded tensors of the other
        tensor-parallel ranks, restricted to the slice of the flat gradient that this DP rank owns."""
        g = opt.gshard
        mine = torch.zeros(1, dtype=torch.float32, device=g.device)
        for a, b in self._ranges:
            lo, hi = max(a, opt.lo), min(b, opt.hi)
            if lo < hi:
                mine += g[lo - opt.lo:hi - opt.lo].float().pow(2).sum()
        total = mine.clone()
        dist.all_reduce(total, group=self.state.group)
        return total - mine

    def step(self, *a, **k):
        self.state.sync_grads()
        if self._ranges is not None and getattr(self.inner, "max_grad_norm", 0.0):
            k["norm_hook"] = self._norm_hook
        return self.inner.step(*a, **k)

    def zero_grad(self, *a, **k):
        return self.inner.zero_grad(*a, **k)

    def accumulate(self):
        if hasattr(self.inner, "accumulate"):
            self.inner.accumulate()

    def __getattr__(self, name):
        return getattr(self.inner, name)
