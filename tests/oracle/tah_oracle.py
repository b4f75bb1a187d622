"""Dense, mask-materialising fp32 statement of the TaH forward pass.

This is the numerical oracle for the framework and the timed CPU baseline.  It is
deliberately naive and shares no code with ``tah_b200``: separate q/k/v/gate/up
matrices, LoRA as explicit extra matmuls, a dict cache grown with ``torch.cat``,
an additive ``finfo.min`` mask built for every pass, dense ``(B, T, V)`` logit
buffers.  The algorithm follows reference ``tah/model/tah_model.py:495-791`` and
``tah/model/causal_cache.py:63-160``; the backbone math follows HuggingFace Qwen3.

Weights are taken from a ``tah_b200`` model through its HF-named state dict, so
both sides compute with identical parameters.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F


class OracleWeights:
    def __init__(self, base_sd: Dict[str, torch.Tensor], lora_sd: Dict[str, torch.Tensor], cfg, r: int, alpha: float):
        self.sd = {k: v.detach().clone().float() for k, v in base_sd.items()}
        self.lora = {k: v.detach().clone().float() for k, v in lora_sd.items()}
        self.cfg, self.r = cfg, r
        self.scaling = alpha / r if r else 0.0
        for t in list(self.sd.values()) + list(self.lora.values()):
            t.requires_grad_(True)

    def lin(self, x, layer: int, mod: str, proj: str, lora_on: bool):
        y = x @ self.sd[f"model.layers.{layer}.{mod}.{proj}.weight"].t()
        key = f"base_model.model.model.layers.{layer}.{mod}.{proj}"
        if lora_on and key + ".lora_A.weight" in self.lora:
            a, b = self.lora[key + ".lora_A.weight"], self.lora[key + ".lora_B.weight"]
            y = y + self.scaling * ((x @ a.t()) @ b.t())
        return y


def _rms(x, w, eps):
    var = x.pow(2).mean(-1, keepdim=True)
    return w * (x * torch.rsqrt(var + eps))


def _rope(x, pos, theta):
    hd = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    ang = pos[..., None].float() * inv
    ang = torch.cat([ang, ang], -1)[:, None]          # (B,1,T,hd)
    x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
    return x * ang.cos() + torch.cat([-x2, x1], -1) * ang.sin()


class OracleCache:
    def __init__(self):
        self.k, self.v, self.pos, self.valid = {}, {}, {}, {}

    def append(self, layer, depth, k, v, pos, valid):
        s = (layer, depth)
        if s in self.k:
            self.k[s] = torch.cat([self.k[s], k], 2)
            self.v[s] = torch.cat([self.v[s], v], 2)
            if layer == 0:
                self.pos[depth] = torch.cat([self.pos[depth], pos], 1)
                self.valid[depth] = torch.cat([self.valid[depth], valid], 1)
        else:
            self.k[s], self.v[s] = k, v
            if layer == 0:
                self.pos[depth], self.valid[depth] = pos, valid

    def upto(self, layer, depth):
        ks = [self.k[(layer, d)] for d in range(depth + 1) if (layer, d) in self.k]
        vs = [self.v[(layer, d)] for d in range(depth + 1) if (layer, d) in self.v]
        return torch.cat(ks, 2), torch.cat(vs, 2)


def backbone_pass(w: OracleWeights, embeds, pos, add_mask, cache: OracleCache, depth: int, valid, want_hidden=False):
    """One full-stack pass on a (B, L, H) block.  ``add_mask`` is (B,1,L,kv_total) additive."""
    cfg = w.cfg
    B, L, _ = embeds.shape
    nq, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    lora_on = depth >= 1
    h = embeds
    hidden = [h]
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        x = _rms(h, w.sd[p + "input_layernorm.weight"], cfg.rms_norm_eps)
        q = w.lin(x, i, "self_attn", "q_proj", lora_on).view(B, L, nq, hd)
        k = w.lin(x, i, "self_attn", "k_proj", lora_on).view(B, L, nkv, hd)
        v = w.lin(x, i, "self_attn", "v_proj", lora_on).view(B, L, nkv, hd)
        q = _rms(q, w.sd[p + "self_attn.q_norm.weight"], cfg.rms_norm_eps).transpose(1, 2)
        k = _rms(k, w.sd[p + "self_attn.k_norm.weight"], cfg.rms_norm_eps).transpose(1, 2)
        v = v.transpose(1, 2)
        q, k = _rope(q, pos, cfg.rope_theta), _rope(k, pos, cfg.rope_theta)
        cache.append(i, depth, k, v, pos, valid)
        K, Vv = cache.upto(i, depth)
        rep = nq // nkv
        K, Vv = K.repeat_interleave(rep, 1), Vv.repeat_interleave(rep, 1)
        scores = (q @ K.transpose(-1, -2)) / math.sqrt(hd) + add_mask
        o = torch.softmax(scores, -1) @ Vv
        o = o.transpose(1, 2).reshape(B, L, nq * hd)
        h = h + w.lin(o, i, "self_attn", "o_proj", lora_on)
        x = _rms(h, w.sd[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        g = w.lin(x, i, "mlp", "gate_proj", lora_on)
        u = w.lin(x, i, "mlp", "up_proj", lora_on)
        h = h + w.lin(F.silu(g) * u, i, "mlp", "down_proj", lora_on)
        hidden.append(h)
    hn = _rms(h, w.sd["model.norm.weight"], cfg.rms_norm_eps)
    hidden[-1] = hn   # HF: the last entry of hidden_states is the final-norm output
    head = w.sd.get("lm_head.weight", w.sd["model.embed_tokens.weight"])
    return hn @ head.t(), (hidden if want_hidden else None)


def duo_additive_mask(q_pos, q_valid, cache: OracleCache, depth: int):
    """(B,1,L,kv_total) additive mask; KV order = [depth-0 slot | depth-1 slot | ... | this pass]."""
    B, L = q_pos.shape
    pos_parts, valid_parts, iter_parts = [], [], []
    for d in range(depth + 1):
        if d in cache.pos:
            pos_parts.append(cache.pos[d])
            valid_parts.append(cache.valid[d])
            iter_parts.append(torch.full((cache.pos[d].shape[1],), d))
    # this pass's tokens are appended to slot `depth`, the last visible slot, so they come last
    kv_pos = torch.cat(pos_parts + [q_pos], 1)
    kv_valid = torch.cat(valid_parts + [q_valid], 1)
    kv_iter = torch.cat(iter_parts + [torch.full((L,), depth)])
    ok = (kv_pos[:, None, :] <= q_pos[:, :, None]) & (kv_iter[None, None, :] <= depth) & (kv_valid[:, None, :] == 1)
    m = torch.full((B, L, kv_pos.shape[1]), torch.finfo(torch.float32).min)
    m[ok] = 0.0
    return m[:, None]


def pack(mask, t, pad=0):
    """Right-padded gather of the True positions of ``mask`` (B,S) from ``t`` (B,S,...)."""
    B, S = mask.shape
    width = int(mask.sum(1).max()) if mask.any() else 0
    out = t.new_full((B, width) + tuple(t.shape[2:]), pad)
    for b in range(B):
        idx = mask[b].nonzero().flatten()
        out[b, : idx.numel()] = t[b, idx]
    return out


def unpack(mask, block, dense, select=None):
    dense = dense.clone()
    for b in range(mask.shape[0]):
        idx = mask[b].nonzero().flatten()
        for j, s in enumerate(idx.tolist()):
            if select is None or bool(select[b, s]):
                dense[b, s] = block[b, j]
    return dense


def tah_forward(w: OracleWeights, input_ids, *, max_iter: int, topk: int, attention_mask=None, labels=None,
                iter_count_labels=None, decider=None, cache: Optional[OracleCache] = None,
                tap_layers=(), num_items_in_batch=None):
    """Returns dict(logits, iter_count, loss, cache).  ``decider(logits_valid, depth, hidden_valid, iter_labels_valid)``
    -> bool (N,) ; default = oracle label decider."""
    cfg = w.cfg
    B, T = input_ids.shape
    V = cfg.vocab_size
    E = w.sd["model.embed_tokens.weight"]
    embeds = E[input_ids]
    cum = torch.zeros(B, T, V)
    final = torch.zeros(B, T, V)
    counts = torch.zeros(B, T, dtype=torch.long)
    cache = cache or OracleCache()
    valid = attention_mask[:, -T:].long() if attention_mask is not None else torch.ones(B, T, dtype=torch.long)
    prior = cache.valid.get(0, torch.zeros(B, 0, dtype=torch.long))
    pos = (torch.cat([prior, valid], 1).cumsum(1)[:, -T:] - 1).clamp(min=0)
    labels_shifted = F.pad(labels, (0, 1), value=-100)[:, 1:] if labels is not None else None

    current = torch.ones(B, T, dtype=torch.bool)
    finished = torch.zeros(B, T, dtype=torch.bool)
    depth = 0
    while depth < max_iter and current.any():
        a_emb, a_cum, a_pos, a_valid = pack(current, embeds), pack(current, cum), pack(current, pos), pack(current, valid)
        a_il = pack(current, iter_count_labels) if iter_count_labels is not None else None
        if a_valid.shape[1] == 0:
            break
        mask = duo_additive_mask(a_pos, a_valid, cache, depth)
        logits, hidden = backbone_pass(w, a_emb, a_pos, mask, cache, depth, a_valid, want_hidden=bool(tap_layers))
        depth += 1
        upd = logits + a_cum
        cum = unpack(current, upd, cum)
        va = a_valid == 1
        hid_valid = None
        if tap_layers:
            hid_valid = torch.cat([hidden[i] for i in tap_layers], -1)[va]
        if decider is None:
            if depth >= max_iter or a_il is None:
                decision = torch.zeros(int(va.sum()), dtype=torch.bool)
            else:
                il = a_il[va]
                decision = (il > depth) & (il != -100)
        else:
            decision = decider(upd[va], depth, hid_valid, None if a_il is None else a_il[va])
        a_fin = torch.ones_like(va)
        a_fin[va] = ~decision
        finished = unpack(current, a_fin, finished)
        counts[current] += 1
        final = unpack(current, upd, final, select=finished)
        nxt = (~finished) & current & (valid == 1)
        if nxt.any():
            a_next = (~a_fin) & va
            kk = min(topk, V)
            tv, ti = torch.topk(upd[a_next], kk, -1)
            soft = (torch.softmax(tv, -1)[..., None] * E[ti]).sum(-2)
            a_emb = a_emb.clone()
            a_emb[a_next] = soft
            embeds = unpack(current, a_emb, torch.zeros_like(embeds), select=nxt)
        current = nxt
    loss = None
    if labels_shifted is not None:
        flat = final.view(-1, V)
        if num_items_in_batch is None:
            loss = F.cross_entropy(flat, labels_shifted.reshape(-1), ignore_index=-100)
        else:
            loss = F.cross_entropy(flat, labels_shifted.reshape(-1), ignore_index=-100, reduction="sum") / num_items_in_batch
    return dict(logits=final, iter_count=counts, loss=loss, cache=cache)


def greedy_decode(w: OracleWeights, input_ids, n_new: int, *, max_iter: int, topk: int, attention_mask=None,
                  hard_mask_fn=None):
    """Greedy token-by-token decode.  ``hard_mask_fn(step, B) -> bool (B,)`` says which rows take a
    second pass for the token processed at that step (step 0 = prefill -> (B,T) mask)."""
    B, T = input_ids.shape
    attn = attention_mask

    def decider_for(step, shape_bt):
        def fn(logits_valid, depth, hid, il):
            if depth >= max_iter or hard_mask_fn is None:
                return torch.zeros(logits_valid.shape[0], dtype=torch.bool)
            m = hard_mask_fn(step, shape_bt)
            v = (attn[:, -shape_bt[1]:] == 1) if attn is not None else torch.ones(shape_bt, dtype=torch.bool)
            return m[v]
        return fn

    with torch.no_grad():
        out = tah_forward(w, input_ids, max_iter=max_iter, topk=topk, attention_mask=attn, decider=decider_for(0, (B, T)))
        cache = out["cache"]
        toks = []
        for step in range(1, n_new + 1):
            nxt = out["logits"][:, -1].argmax(-1)
            toks.append(nxt)
            if attn is not None:
                attn = torch.cat([attn, attn.new_ones(B, 1)], 1)
            out = tah_forward(w, nxt[:, None], max_iter=max_iter, topk=topk, attention_mask=attn, cache=cache,
                              decider=decider_for(step, (B, 1)))
    return torch.stack(toks, 1)
