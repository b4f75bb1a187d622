"""Qwen3 decoder backbone with a fused parameter layout and built-in, gateable LoRA.

The reference delegates the backbone to HuggingFace ``Qwen3ForCausalLM`` wrapped by
PEFT (reference ``tah/model/tah_model.py:378-404``).  This module is a from-scratch
backbone that computes the same function (RMSNorm, per-head QK-norm, rotate-half
RoPE, GQA attention, SwiGLU, tied LM head) but is laid out for the B200 kernels:

* ``qkv_proj`` is one ``[nq*hd + 2*nkv*hd, H]`` weight and ``gate_up_proj`` one
  ``[2*I, H]`` weight, so each is a single GEMM;
* every adapted linear carries its LoRA factors directly (``lora_A`` stacked over
  the fused outputs, one ``lora_B`` block per original projection), and the
  adapter is switched per call (``lora_on``) rather than by walking modules;
* attention receives *positions*, not a materialised mask: the duo-causal rule
  ``kv_pos <= q_pos and kv_depth <= q_depth and kv_valid`` is evaluated by the
  attention op itself.

On disk the weights keep the HuggingFace / PEFT names; :func:`export_hf_state_dict`
and :func:`import_hf_state_dict` translate.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from tah_b200 import ops


@dataclass
class Qwen3Config:
    vocab_size: int = 151936
    hidden_size: int = 2048
    intermediate_size: int = 6144
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = True
    max_position_embeddings: int = 40960
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = 151643
    eos_token_id: Optional[int] = 151645
    pad_token_id: Optional[int] = None
    extra: Dict = field(default_factory=dict)

    # ---- HF config.json round trip -------------------------------------------------
    @classmethod
    def from_hf_dict(cls, d: dict) -> "Qwen3Config":
        d = dict(d)
        rope = d.get("rope_theta")
        if rope is None and isinstance(d.get("rope_parameters"), dict):
            rope = d["rope_parameters"].get("rope_theta")
        known = {f for f in cls.__dataclass_fields__ if f != "extra"}
        kw = {k: d[k] for k in known if k in d and d[k] is not None}
        if rope is not None:
            kw["rope_theta"] = float(rope)
        if "head_dim" not in kw:
            kw["head_dim"] = kw.get("hidden_size", 2048) // kw.get("num_attention_heads", 16)
        dt = d.get("torch_dtype", d.get("dtype"))
        if dt is not None:
            kw["torch_dtype"] = str(dt).replace("torch.", "")
        kw["extra"] = {k: v for k, v in d.items() if k not in known and k not in ("rope_parameters", "dtype")}
        return cls(**kw)

    @classmethod
    def from_pretrained(cls, path: str) -> "Qwen3Config":
        with open(os.path.join(path, "config.json"), encoding="utf-8") as fh:
            return cls.from_hf_dict(json.load(fh))

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        extra = d.pop("extra")
        out = dict(extra)
        out.update(d)
        out.update({
            "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
            "attention_bias": False, "attention_dropout": 0.0, "use_cache": True,
            "rope_scaling": None, "initializer_range": 0.02,
        })
        return out

    def save_pretrained(self, path: str) -> None:
        with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as fh:
            json.dump(self.to_hf_dict(), fh, indent=2)

    @property
    def dtype(self) -> torch.dtype:
        return getattr(torch, self.torch_dtype)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim


PRESETS = {
    # Tiny CPU configuration used by the oracle tests
    "tiny": dict(vocab_size=1024, hidden_size=256, intermediate_size=768, num_hidden_layers=4,
                 num_attention_heads=4, num_key_value_heads=2, head_dim=64, torch_dtype="float32",
                 bos_token_id=None, eos_token_id=None),
    "qwen3-0.6b": dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                       num_attention_heads=16, num_key_value_heads=8),
    "qwen3-1.7b": dict(hidden_size=2048, intermediate_size=6144, num_hidden_layers=28,
                       num_attention_heads=16, num_key_value_heads=8),
    # "TaH" = the base model with one layer pruned; "TaH-plus" keeps all 28
    "tah-1.7b": dict(hidden_size=2048, intermediate_size=6144, num_hidden_layers=27,
                     num_attention_heads=16, num_key_value_heads=8),
    "tah-plus-1.7b": dict(hidden_size=2048, intermediate_size=6144, num_hidden_layers=28,
                          num_attention_heads=16, num_key_value_heads=8),
    "qwen3-4b": dict(hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                     num_attention_heads=32, num_key_value_heads=8),
}


def preset(name: str, **overrides) -> Qwen3Config:
    kw = dict(PRESETS[name])
    kw.update(overrides)
    return Qwen3Config(**kw)


# ------------------------------------------------------------------------------------
# LoRA
# ------------------------------------------------------------------------------------

@dataclass
class LoRASpec:
    r: int = 0
    lora_alpha: float = 1.0
    lora_dropout: float = 0.0
    # names of the original projections that carry an adapter
    targets: Tuple[str, ...] = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")

    @property
    def scaling(self) -> float:
        return self.lora_alpha / self.r if self.r else 0.0

    @classmethod
    def from_adapter_kwargs(cls, kw: Optional[dict]) -> "LoRASpec":
        kw = dict(kw or {})
        tm = kw.get("target_modules", "all-linear")
        all_lin = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
        if isinstance(tm, str):
            targets = all_lin if tm == "all-linear" else (tm,)
        else:
            targets = tuple(tm)
        return cls(r=int(kw.get("r", 0) or 0), lora_alpha=float(kw.get("lora_alpha", kw.get("r", 1) or 1)),
                   lora_dropout=float(kw.get("lora_dropout", 0.0)), targets=targets)


class FusedLoRALinear(nn.Module):
    """``y = x W^T`` for a weight that stacks several projections along the output
    dim, plus (when ``lora_on``) ``scaling * (drop(x) A_i^T) B_i^T`` on each
    projection's output slice ``i``.

    ``lora_A`` is ``[n_adapted * r, in]`` (one r-row block per adapted projection)
    and ``lora_B[i]`` is ``[out_i, r]``: the block structure of PEFT's separate
    per-projection adapters, stored so that ``x A^T`` is one GEMM.
    """

    def __init__(self, in_features: int, out_splits: Sequence[int], names: Sequence[str],
                 lora: LoRASpec, dtype=None, device=None):
        super().__init__()
        self.in_features = in_features
        self.out_splits = list(out_splits)
        self.names = list(names)
        self.out_features = sum(out_splits)
        self.weight = nn.Parameter(torch.empty(self.out_features, in_features, dtype=dtype, device=device))
        self.lora_A = None
        self.lora_B = None
        self.adapted: List[int] = []
        self.lora = lora
        nn.init.normal_(self.weight, std=0.02)
        self.attach_lora(lora)

    def attach_lora(self, lora: LoRASpec) -> None:
        """(Re)create the adapter factors: A ~ kaiming-uniform, B = 0 (the adapter starts as a no-op)."""
        self.lora = lora
        self.adapted = [i for i, n in enumerate(self.names) if lora.r > 0 and n in lora.targets]
        if not self.adapted:
            self.lora_A, self.lora_B = None, None
            return
        kw = dict(dtype=self.weight.dtype, device=self.weight.device)
        self.lora_A = nn.Parameter(torch.empty(len(self.adapted) * lora.r, self.in_features, **kw))
        self.lora_B = nn.ParameterList(
            nn.Parameter(torch.zeros(self.out_splits[i], lora.r, **kw)) for i in self.adapted)
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))

    def lora_B_dense(self) -> torch.Tensor:
        """Block-diagonal ``[out_features, n_adapted*r]`` form of ``lora_B`` (scaled),
        the layout the K-extended GEMM kernel consumes."""
        r = self.lora.r
        out = self.weight.new_zeros(self.out_features, len(self.adapted) * r)
        off = [0]
        for s in self.out_splits:
            off.append(off[-1] + s)
        for j, i in enumerate(self.adapted):
            out[off[i]:off[i + 1], j * r:(j + 1) * r] = self.lora_B[j] * self.lora.scaling
        return out

    def forward(self, x: torch.Tensor, lora_on: bool = False) -> torch.Tensor:
        if not (lora_on and self.adapted):
            return ops.linear(x, self.weight)
        xa = F.dropout(x, self.lora.lora_dropout, self.training) if self.lora.lora_dropout > 0 else x
        return ops.lora_linear(x, self.weight, xa, self.lora_A, list(self.lora_B), self.adapted,
                               self.out_splits, self.lora.r, self.lora.scaling)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps)


def rope_cos_sin(position_ids: torch.Tensor, head_dim: int, theta: float, dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables ``[..., head_dim]`` for rotate-half RoPE, computed in fp32."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=position_ids.device, dtype=torch.float32) / head_dim))
    ang = position_ids.to(torch.float32).unsqueeze(-1) * inv
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x``: [B, T, heads, hd]; cos/sin: [B, T, hd]."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos.unsqueeze(-2) + rot * sin.unsqueeze(-2)


class Attention(nn.Module):
    def __init__(self, cfg: Qwen3Config, lora: LoRASpec, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        kw = dict(dtype=dtype, device=device)
        self.qkv_proj = FusedLoRALinear(cfg.hidden_size, [cfg.q_size, cfg.kv_size, cfg.kv_size],
                                        ["q_proj", "k_proj", "v_proj"], lora, **kw)
        self.o_proj = FusedLoRALinear(cfg.q_size, [cfg.hidden_size], ["o_proj"], lora, **kw)
        self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, **kw)
        self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, **kw)

    def project_qkv(self, x, cos, sin, lora_on: bool, pos=None):
        """Fused QKV projection, per-head QK-norm and RoPE: returns q, k, v as ``[B,T,heads,hd]``.
        With ``pos`` (the integer position ids the tables were built from) a bf16 CUDA pass runs the
        norm + rotation as one kernel forward and one backward."""
        cfg = self.cfg
        B, T, _ = x.shape
        qkv = self.qkv_proj(x, lora_on)
        if pos is not None and ops.fused_qk_norm_rope_ok(qkv, cfg.head_dim):
            return ops.qk_norm_rope(qkv, self.q_norm.weight, self.k_norm.weight, pos, cfg.num_attention_heads,
                                    cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps, cfg.rope_theta)
        q, k, v = qkv.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=-1)
        q = self.q_norm(q.view(B, T, cfg.num_attention_heads, cfg.head_dim))
        k = self.k_norm(k.view(B, T, cfg.num_key_value_heads, cfg.head_dim))
        v = v.view(B, T, cfg.num_key_value_heads, cfg.head_dim)
        return apply_rope(q, cos, sin), apply_rope(k, cos, sin), v.contiguous()

    def forward(self, x, cos, sin, kv, lora_on: bool):
        B, T, _ = x.shape
        q, k, v = self.project_qkv(x, cos, sin, lora_on)
        o = kv.attend(self.layer_idx, q, k, v)
        return self.o_proj(o.reshape(B, T, self.cfg.q_size), lora_on)


class MLP(nn.Module):
    def __init__(self, cfg: Qwen3Config, lora: LoRASpec, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.gate_up_proj = FusedLoRALinear(cfg.hidden_size, [cfg.intermediate_size] * 2,
                                            ["gate_proj", "up_proj"], lora, **kw)
        self.down_proj = FusedLoRALinear(cfg.intermediate_size, [cfg.hidden_size], ["down_proj"], lora, **kw)

    def forward(self, x, lora_on: bool):
        return self.down_proj(ops.swiglu(self.gate_up_proj(x, lora_on)), lora_on)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: Qwen3Config, lora: LoRASpec, layer_idx: int, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.self_attn = Attention(cfg, lora, layer_idx, **kw)
        self.mlp = MLP(cfg, lora, **kw)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **kw)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **kw)

    def _pre_attention(self, h, cos, sin, lora_on: bool, pos=None):
        return self.self_attn.project_qkv(self.input_layernorm(h), cos, sin, lora_on, pos)

    def _post_attention(self, h, o, lora_on: bool):
        h = h + self.self_attn.o_proj(o, lora_on)
        return h + self.mlp(self.post_attention_layernorm(h), lora_on)

    def forward(self, h, cos, sin, kv, lora_on: bool, checkpoint: bool = False, pos=None):
        """With ``checkpoint`` the two dense stages are recomputed in backward while the
        attention itself (and the K/V handed to the cache) stays in the autograd graph,
        so later passes can still back-propagate into this pass's K/V."""
        B, T, _ = h.shape
        if checkpoint:
            from torch.utils.checkpoint import checkpoint as ckpt
            q, k, v = ckpt(self._pre_attention, h, cos, sin, lora_on, pos, use_reentrant=False)
            o = kv.attend(self.self_attn.layer_idx, q, k, v).reshape(B, T, -1)
            return ckpt(self._post_attention, h, o, lora_on, use_reentrant=False)
        q, k, v = self._pre_attention(h, cos, sin, lora_on, pos)
        o = kv.attend(self.self_attn.layer_idx, q, k, v).reshape(B, T, -1)
        return self._post_attention(h, o, lora_on)


class Qwen3Model(nn.Module):
    def __init__(self, cfg: Qwen3Config, lora: LoRASpec, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, **kw)
        self.layers = nn.ModuleList(DecoderLayer(cfg, lora, i, **kw) for i in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **kw)


class PassKV:
    """Attention context of one backbone pass.  ``attend`` stores this pass's K/V
    for a layer and returns the attention output under the duo-causal rule."""

    def attend(self, layer_idx: int, q, k, v):  # pragma: no cover - interface
        raise NotImplementedError


class PlainCausalKV(PassKV):
    """No cache, ordinary causal attention over the tokens of this pass (used by
    utilities that run the backbone as a plain LM, e.g. the labeller and pruner)."""

    def __init__(self, position_ids, valid_mask):
        self.pos, self.valid = position_ids, valid_mask

    def attend(self, layer_idx, q, k, v):
        return ops.duo_attention(q, k, v, self.pos, self.pos, self.valid)


def attach_lora(model: "Qwen3ForCausalLM", spec: LoRASpec) -> None:
    """Give every adapted linear of ``model`` fresh LoRA factors described by ``spec``."""
    model.lora = spec
    for mod in model.modules():
        if isinstance(mod, FusedLoRALinear):
            mod.attach_lora(spec)


class Qwen3ForCausalLM(nn.Module):
    """Backbone + LM head.  ``forward`` runs one pass over ``inputs_embeds``."""

    def __init__(self, cfg: Qwen3Config, lora: Optional[LoRASpec] = None, dtype=None, device=None):
        super().__init__()
        self.config = cfg
        self.lora = lora or LoRASpec()
        dtype = dtype or cfg.dtype
        self.model = Qwen3Model(cfg, self.lora, dtype=dtype, device=device)
        if cfg.tie_word_embeddings:
            self.lm_head = None
        else:
            self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=dtype, device=device)
        self.gradient_checkpointing = False
        nn.init.normal_(self.model.embed_tokens.weight, std=0.02)

    # -- handles ---------------------------------------------------------------------
    @property
    def device(self):
        return self.model.embed_tokens.weight.device

    @property
    def dtype(self):
        return self.model.embed_tokens.weight.dtype

    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.model.embed_tokens.weight if self.lm_head is None else self.lm_head.weight

    def lora_parameters(self):
        for n, p in self.named_parameters():
            if "lora_" in n:
                yield n, p

    def base_parameters(self):
        for n, p in self.named_parameters():
            if "lora_" not in n:
                yield n, p

    # -- compute ---------------------------------------------------------------------
    def backbone(self, inputs_embeds, position_ids, kv: PassKV, lora_on: bool = False,
                 tap_layers: Optional[Sequence[int]] = None):
        """Returns (final-norm hidden states, dict tap_index -> hidden state).

        Tap index ``i < L`` is the input of layer ``i`` (0 = the embeddings), ``L`` the
        output of the final norm: the numbering of HF's ``output_hidden_states``.
        """
        cfg = self.config
        cos, sin = rope_cos_sin(position_ids, cfg.head_dim, cfg.rope_theta, inputs_embeds.dtype)
        taps = {}
        want = set(tap_layers or ())
        h = inputs_embeds
        for i, layer in enumerate(self.model.layers):
            if i in want:
                taps[i] = h
            ck = self.gradient_checkpointing and self.training and torch.is_grad_enabled()
            h = layer(h, cos, sin, kv, lora_on, checkpoint=ck, pos=position_ids)
        h = self.model.norm(h)
        if cfg.num_hidden_layers in want:
            taps[cfg.num_hidden_layers] = h
        return h, taps

    def logits(self, hidden):
        return ops.linear(hidden, self.lm_head_weight)

    def forward(self, input_ids=None, inputs_embeds=None, position_ids=None, attention_mask=None,
                kv: Optional[PassKV] = None, lora_on: bool = False):
        """Plain LM forward (one pass, causal): returns logits ``[B, T, V]``."""
        if inputs_embeds is None:
            inputs_embeds = self.model.embed_tokens(input_ids)
        B, T = inputs_embeds.shape[:2]
        valid = attention_mask if attention_mask is not None else torch.ones(B, T, dtype=torch.long, device=inputs_embeds.device)
        if position_ids is None:
            position_ids = (valid.long().cumsum(-1) - 1).clamp(min=0)
        kv = kv or PlainCausalKV(position_ids, valid)
        h, _ = self.backbone(inputs_embeds, position_ids, kv, lora_on)
        return self.logits(h)


# ------------------------------------------------------------------------------------
# HuggingFace / PEFT name mapping
# ------------------------------------------------------------------------------------

_PEFT_PREFIX = "base_model.model."


def export_hf_state_dict(model: Qwen3ForCausalLM) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor]]:
    """Split the fused parameters back into HF names.  Returns ``(base, lora)``:
    ``base`` uses plain Qwen3 keys, ``lora`` uses PEFT adapter keys
    (``base_model.model.model.layers.{i}.<mod>.<proj>.lora_{A,B}.weight``)."""
    cfg = model.config
    base: Dict[str, torch.Tensor] = {}
    lora: Dict[str, torch.Tensor] = {}
    base["model.embed_tokens.weight"] = model.model.embed_tokens.weight.detach()
    base["model.norm.weight"] = model.model.norm.weight.detach()
    if model.lm_head is not None:
        base["lm_head.weight"] = model.lm_head.weight.detach()
    for i, layer in enumerate(model.model.layers):
        p = f"model.layers.{i}."
        base[p + "input_layernorm.weight"] = layer.input_layernorm.weight.detach()
        base[p + "post_attention_layernorm.weight"] = layer.post_attention_layernorm.weight.detach()
        base[p + "self_attn.q_norm.weight"] = layer.self_attn.q_norm.weight.detach()
        base[p + "self_attn.k_norm.weight"] = layer.self_attn.k_norm.weight.detach()
        for mod_name, lin in (("self_attn", layer.self_attn.qkv_proj), ("self_attn", layer.self_attn.o_proj),
                              ("mlp", layer.mlp.gate_up_proj), ("mlp", layer.mlp.down_proj)):
            chunks = lin.weight.detach().split(lin.out_splits, dim=0)
            for name, w in zip(lin.names, chunks):
                base[f"{p}{mod_name}.{name}.weight"] = w.contiguous()
            r = lin.lora.r
            for j, idx in enumerate(lin.adapted):
                key = f"{_PEFT_PREFIX}{p}{mod_name}.{lin.names[idx]}"
                lora[key + ".lora_A.weight"] = lin.lora_A.detach()[j * r:(j + 1) * r].contiguous()
                lora[key + ".lora_B.weight"] = lin.lora_B[j].detach().contiguous()
    return base, lora


def import_hf_state_dict(model: Qwen3ForCausalLM, base: Optional[Dict[str, torch.Tensor]] = None,
                         lora: Optional[Dict[str, torch.Tensor]] = None, strict: bool = True) -> List[str]:
    """Load HF-named tensors into the fused layout.  Returns the list of keys not consumed."""
    used = set()

    def take(sd, key):
        if sd is None or key not in sd:
            return None
        used.add(key)
        return sd[key]

    def clean(k: str) -> str:
        # tolerate PEFT-wrapped base checkpoints and adapter-name infixes
        k = k.replace(".base_layer", "").replace(".default.weight", ".weight")
        return k

    base = {clean(k): v for k, v in (base or {}).items()}
    lora = {clean(k): v for k, v in (lora or {}).items()}
    missing: List[str] = []

    @torch.no_grad()
    def put(param, value, key):
        if value is None:
            if base:
                missing.append(key)
            return
        param.copy_(value.to(param.dtype))

    if base:
        put(model.model.embed_tokens.weight, take(base, "model.embed_tokens.weight"), "model.embed_tokens.weight")
        put(model.model.norm.weight, take(base, "model.norm.weight"), "model.norm.weight")
        if model.lm_head is not None:
            w = take(base, "lm_head.weight")
            put(model.lm_head.weight, w if w is not None else base.get("model.embed_tokens.weight"), "lm_head.weight")
        else:
            used.add("lm_head.weight")
    for i, layer in enumerate(model.model.layers):
        p = f"model.layers.{i}."
        if base:
            put(layer.input_layernorm.weight, take(base, p + "input_layernorm.weight"), p + "input_layernorm.weight")
            put(layer.post_attention_layernorm.weight, take(base, p + "post_attention_layernorm.weight"), p + "post_attention_layernorm.weight")
            put(layer.self_attn.q_norm.weight, take(base, p + "self_attn.q_norm.weight"), p + "self_attn.q_norm.weight")
            put(layer.self_attn.k_norm.weight, take(base, p + "self_attn.k_norm.weight"), p + "self_attn.k_norm.weight")
        for mod_name, lin in (("self_attn", layer.self_attn.qkv_proj), ("self_attn", layer.self_attn.o_proj),
                              ("mlp", layer.mlp.gate_up_proj), ("mlp", layer.mlp.down_proj)):
            off = 0
            for name, n_out in zip(lin.names, lin.out_splits):
                if base:
                    key = f"{p}{mod_name}.{name}.weight"
                    put(lin.weight[off:off + n_out], take(base, key), key)
                off += n_out
            r = lin.lora.r
            for j, idx in enumerate(lin.adapted):
                key = f"{_PEFT_PREFIX}{p}{mod_name}.{lin.names[idx]}"
                a, b = take(lora, key + ".lora_A.weight"), take(lora, key + ".lora_B.weight")
                if a is not None:
                    with torch.no_grad():
                        lin.lora_A[j * r:(j + 1) * r].copy_(a.to(lin.lora_A.dtype))
                if b is not None:
                    with torch.no_grad():
                        lin.lora_B[j].copy_(b.to(lin.lora_B[j].dtype))
    if strict and missing:
        raise KeyError(f"missing tensors in checkpoint: {missing[:8]}{'...' if len(missing) > 8 else ''}")
    return [k for k in list(base) + list(lora) if k not in used]


def from_hf_model(hf_model, lora: Optional[LoRASpec] = None) -> Qwen3ForCausalLM:
    """Build the fused backbone from an instantiated HuggingFace Qwen3 model."""
    cfg = Qwen3Config.from_hf_dict(hf_model.config.to_dict())
    dtype = next(hf_model.parameters()).dtype
    model = Qwen3ForCausalLM(cfg, lora, dtype=dtype, device=next(hf_model.parameters()).device)
    import_hf_state_dict(model, base=dict(hf_model.state_dict()), strict=True)
    return model
