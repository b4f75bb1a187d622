"""Plain PyTorch statements of every op the framework uses.

They are the CPU path, the autograd path where no hand-written backward exists,
and the fp32 oracles the CUDA kernels are tested against.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F


def linear(x, w):
    return F.linear(x, w)


def lora_linear(x, w, xa, lora_A, lora_B: List[torch.Tensor], adapted: Sequence[int],
                out_splits: Sequence[int], r: int, scaling: float):
    y = F.linear(x, w)
    t = F.linear(xa, lora_A)                     # [..., n_adapted * r]
    offs = [0]
    for s in out_splits:
        offs.append(offs[-1] + s)
    pieces = list(y.split(list(out_splits), dim=-1))
    for j, idx in enumerate(adapted):
        pieces[idx] = pieces[idx] + scaling * F.linear(t[..., j * r:(j + 1) * r], lora_B[j])
    return torch.cat(pieces, dim=-1) if len(pieces) > 1 else pieces[0]


def rms_norm(x, weight, eps: float):
    dt = x.dtype
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return weight * xf.to(dt)


def swiglu(gate_up):
    gate, up = gate_up.chunk(2, dim=-1)
    return F.silu(gate) * up


def duo_mask(q_pos, kv_pos, kv_valid, q_depth: Optional[torch.Tensor] = None, kv_depth: Optional[torch.Tensor] = None):
    """Boolean ``[B, Tq, Tk]``: ``kv_pos <= q_pos & kv_valid`` (& ``kv_depth <= q_depth`` when given)."""
    m = (kv_pos[:, None, :] <= q_pos[:, :, None]) & (kv_valid[:, None, :] == 1)
    if q_depth is not None and kv_depth is not None:
        m = m & (kv_depth[:, None, :] <= q_depth[:, :, None])
    return m


def duo_attention(q, k, v, q_pos, kv_pos, kv_valid, q_depth=None, kv_depth=None):
    """q ``[B,Tq,nq,hd]``, k/v ``[B,Tk,nkv,hd]`` -> ``[B,Tq,nq,hd]``.

    Masked scores take the most negative finite value (not -inf), so a query that
    can see nothing yields a uniform average rather than NaN - the behaviour of an
    additive ``finfo.min`` mask.
    """
    B, Tq, nq, hd = q.shape
    nkv = k.shape[2]
    mask = duo_mask(q_pos, kv_pos, kv_valid, q_depth, kv_depth)
    bias = torch.zeros(mask.shape, dtype=q.dtype, device=q.device).masked_fill(~mask, torch.finfo(q.dtype).min)
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if nq != nkv:
        rep = nq // nkv
        kt = kt.repeat_interleave(rep, dim=1)
        vt = vt.repeat_interleave(rep, dim=1)
    o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=bias[:, None], scale=hd ** -0.5)
    return o.transpose(1, 2)


def topk_softmax_embed(logits, embedding_weight, topk: int):
    """Soft next-pass input: softmax over the top-k logits, weighted sum of embedding rows."""
    k = min(topk, logits.size(-1))
    vals, idx = torch.topk(logits, k=k, dim=-1)
    probs = torch.softmax(vals, dim=-1)
    return (probs.unsqueeze(-1) * embedding_weight[idx]).sum(-2).to(embedding_weight.dtype)


def sample(logits, temperature=1.0, top_p=1.0, top_k=0, min_p=0.0, do_sample=True, generator=None):
    """temperature -> softmax -> min_p -> top_k -> top_p -> draw (greedy when ``do_sample`` is False)."""
    if not do_sample:
        return logits.argmax(-1)
    if temperature != 1.0:
        logits = logits / temperature
    p = torch.softmax(logits, dim=-1)
    if min_p > 0.0:
        p = torch.where(p >= min_p * p.amax(-1, keepdim=True), p, torch.zeros_like(p))
        p = p / p.sum(-1, keepdim=True)
    if top_k > 0:
        kth = torch.topk(p, min(top_k, p.size(-1)), dim=-1).values[..., -1:]
        p = torch.where(p < kth, torch.zeros_like(p), p)
        p = p / p.sum(-1, keepdim=True)
    if top_p < 1.0:
        sp, si = torch.sort(p, descending=True, dim=-1)
        drop = sp.cumsum(-1) > top_p
        drop = torch.cat((torch.zeros_like(drop[..., :1]), drop[..., :-1]), dim=-1)
        p = p.masked_fill(torch.zeros_like(drop).scatter(-1, si, drop), 0.0)
        p = p / p.sum(-1, keepdim=True)
    return torch.multinomial(p, 1, generator=generator).squeeze(-1)
