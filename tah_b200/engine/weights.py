"""Kernel-ready views of a model's weights for the inference engine.

Base weights are used in place (the backbone already stores ``qkv_proj`` / ``gate_up_proj``
fused).  The LoRA factors are re-laid for the K-extended GEMM: ``a_*`` = the stacked A rows
zero-padded to a multiple of 64 (one GEMM k-block), ``b_*`` = the block-diagonal, pre-scaled B as
``[out_features, R_padded]``.  With tensor parallelism (``tp``) each rank holds its shard:
column-parallel QKV / gate-up (heads and intermediate channels split), row-parallel O / down,
vocabulary-parallel LM head.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import os

import torch

from tah_b200.ops import cuda as K


def _pad64(n: int) -> int:
    return (n + 63) // 64 * 64


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    ln2: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    w_qkv: torch.Tensor
    w_o: torch.Tensor
    w_gu: torch.Tensor
    w_down: torch.Tensor
    a_qkv: Optional[torch.Tensor] = None
    b_qkv: Optional[torch.Tensor] = None
    a_o: Optional[torch.Tensor] = None
    b_o: Optional[torch.Tensor] = None
    a_gu: Optional[torch.Tensor] = None
    b_gu: Optional[torch.Tensor] = None
    a_down: Optional[torch.Tensor] = None
    b_down: Optional[torch.Tensor] = None


def _lora_pair(lin, rows: Optional[torch.Tensor] = None, cols: Optional[torch.Tensor] = None):
    """(A_padded [Rp, K(cols)], B_dense_padded [F(rows), Rp]) or (None, None)."""
    if not lin.adapted:
        return None, None
    A = lin.lora_A.detach()
    Bd = lin.lora_B_dense().detach()
    if cols is not None:
        A = A[:, cols]
    if rows is not None:
        Bd = Bd[rows]
    R = A.shape[0]
    Rp = _pad64(R)
    a = A.new_zeros(Rp, A.shape[1])
    a[:R] = A
    b = Bd.new_zeros(Bd.shape[0], Rp)
    b[:, :R] = Bd
    return a.to(torch.bfloat16).contiguous(), b.to(torch.bfloat16).contiguous()


class EngineWeights:
    def __init__(self, base, tp=None):
        cfg = base.config
        self.cfg = cfg
        self.tp = tp
        ws = 1 if tp is None else tp.world_size
        rk = 0 if tp is None else tp.rank
        # MLP channels per rank: whole 64-wide k-blocks for the down projection; the interleaved gate / up layout then
        # has 2 * 64 rows per pair of k-blocks, i.e. whole 128-row tiles (the stacked layout needs 128 channels)
        chan = 64 if os.environ.get("TAH_B200_SWIGLU", "interleaved") != "dual" else 128
        if ws > 1 and (cfg.num_key_value_heads % ws or cfg.num_attention_heads % ws or cfg.intermediate_size % (ws * chan)):
            raise ValueError(f"tensor-parallel size {ws} does not divide the model's heads/channels")
        self.nq = cfg.num_attention_heads // ws
        self.nkv = cfg.num_key_value_heads // ws
        hd = cfg.head_dim
        self.inter = cfg.intermediate_size // ws
        self.qkv_out = (self.nq + 2 * self.nkv) * hd
        self.r = base.lora.r
        dev = base.device
        bf = lambda t: t.detach().to(torch.bfloat16).contiguous()
        # TAH_B200_SWIGLU=dual keeps the stacked [gate; up] layout and the two-accumulator SwiGLU GEMM
        self.gu_interleaved = os.environ.get("TAH_B200_SWIGLU", "interleaved") != "dual"
        self.embed = bf(base.model.embed_tokens.weight)
        head = base.lm_head_weight
        V = head.shape[0]
        if ws > 1:
            vs = (V + ws - 1) // ws
            vs = (vs + 127) // 128 * 128
            lo, hi = rk * vs, min(V, (rk + 1) * vs)
            self.vocab_shard = (lo, hi, vs)
            shard = head.new_zeros(vs, head.shape[1])
            shard[: hi - lo] = head.detach()[lo:hi]
            self.lm_head = bf(shard)
        else:
            self.vocab_shard = (0, V, V)
            self.lm_head = self.embed if base.lm_head is None else bf(head)
        self.vocab = V
        self.final_norm = bf(base.model.norm.weight)
        self.layers: List[LayerWeights] = []
        I = cfg.intermediate_size
        for layer in base.model.layers:
            at, mlp = layer.self_attn, layer.mlp
            if ws > 1:
                qs, ks = cfg.q_size, cfg.kv_size
                q_rows = torch.arange(rk * self.nq * hd, (rk + 1) * self.nq * hd, device=dev)
                k_rows = qs + torch.arange(rk * self.nkv * hd, (rk + 1) * self.nkv * hd, device=dev)
                v_rows = qs + ks + torch.arange(rk * self.nkv * hd, (rk + 1) * self.nkv * hd, device=dev)
                qkv_rows = torch.cat([q_rows, k_rows, v_rows])
                o_cols = q_rows
                gu_rows = torch.cat([torch.arange(rk * self.inter, (rk + 1) * self.inter, device=dev),
                                     I + torch.arange(rk * self.inter, (rk + 1) * self.inter, device=dev)])
                d_cols = torch.arange(rk * self.inter, (rk + 1) * self.inter, device=dev)
                w_qkv = bf(at.qkv_proj.weight.detach()[qkv_rows])
                w_o = bf(at.o_proj.weight.detach()[:, o_cols])
                w_gu = bf(mlp.gate_up_proj.weight.detach()[gu_rows])
                w_down = bf(mlp.down_proj.weight.detach()[:, d_cols])
            else:
                qkv_rows = o_cols = gu_rows = d_cols = None
                w_qkv, w_o = bf(at.qkv_proj.weight), bf(at.o_proj.weight)
                w_gu, w_down = bf(mlp.gate_up_proj.weight), bf(mlp.down_proj.weight)
            lw = LayerWeights(ln1=bf(layer.input_layernorm.weight), ln2=bf(layer.post_attention_layernorm.weight),
                              q_norm=bf(at.q_norm.weight), k_norm=bf(at.k_norm.weight),
                              w_qkv=w_qkv, w_o=w_o, w_gu=w_gu, w_down=w_down)
            lw.a_qkv, lw.b_qkv = _lora_pair(at.qkv_proj, rows=qkv_rows)
            lw.a_o, lw.b_o = _lora_pair(at.o_proj, cols=o_cols)
            lw.a_gu, lw.b_gu = _lora_pair(mlp.gate_up_proj, rows=gu_rows)
            if self.gu_interleaved:
                # rows gate_0, up_0, gate_1, ...: the GEMM's interleaved SwiGLU epilogue (one accumulator)
                lw.w_gu = K.interleave_gate_up(lw.w_gu)
                if lw.b_gu is not None:
                    lw.b_gu = K.interleave_gate_up(lw.b_gu)
            lw.a_down, lw.b_down = _lora_pair(mlp.down_proj, cols=d_cols)
            self.layers.append(lw)
        l0 = self.layers[0]
        width = lambda a: 0 if a is None else a.shape[0]
        self.r_qkv, self.r_o, self.r_gu, self.r_down = width(l0.a_qkv), width(l0.a_o), width(l0.a_gu), width(l0.a_down)
        if self.r > 0 and min(self.r_qkv, self.r_o, self.r_gu, self.r_down) == 0:
            raise NotImplementedError("the engine expects LoRA on all seven projections (target_modules='all-linear')")
