"""Op entry points used by the model code.

Each function picks the hand-written sm_100a kernel when its inputs live on a
CUDA device (see :mod:`tah_b200.ops.cuda`), and the PyTorch statement in
:mod:`tah_b200.ops.torch_ref` otherwise.  On a CUDA device a missing extension
is an error, never a silent fallback, unless ``TAH_B200_FORCE_TORCH=1`` is set
(used to time the eager baseline).
"""
from __future__ import annotations

import os

import torch

from tah_b200.ops import torch_ref
from tah_b200.ops.torch_ref import duo_mask, sample  # noqa: F401


def _use_cuda(x: torch.Tensor) -> bool:
    return x.is_cuda and os.environ.get("TAH_B200_FORCE_TORCH", "0") != "1"


def linear(x, w):
    if _use_cuda(x):
        from tah_b200.ops import autograd_ops
        return autograd_ops.linear(x, w)
    return torch_ref.linear(x, w)


def lora_linear(x, w, xa, lora_A, lora_B, adapted, out_splits, r, scaling):
    if _use_cuda(x):
        from tah_b200.ops import autograd_ops
        return autograd_ops.lora_linear(x, w, xa, lora_A, lora_B, adapted, out_splits, r, scaling)
    return torch_ref.lora_linear(x, w, xa, lora_A, lora_B, adapted, out_splits, r, scaling)


def rms_norm(x, weight, eps):
    if _use_cuda(x):
        from tah_b200.ops import autograd_ops
        return autograd_ops.rms_norm(x, weight, eps)
    return torch_ref.rms_norm(x, weight, eps)


def swiglu(gate_up):
    if _use_cuda(gate_up):
        from tah_b200.ops import autograd_ops
        return autograd_ops.swiglu(gate_up)
    return torch_ref.swiglu(gate_up)


def fused_qk_norm_rope_ok(qkv, head_dim: int) -> bool:
    if not _use_cuda(qkv):
        return False
    from tah_b200.ops import autograd_ops
    return autograd_ops.qk_norm_rope_ok(qkv, head_dim)


def qk_norm_rope(qkv, q_w, k_w, position_ids, nq, nkv, hd, eps, theta):
    """Per-head RMSNorm of q and k + rotate-half RoPE of a fused qkv projection (CUDA bf16 only; callers
    check :func:`fused_qk_norm_rope_ok` and otherwise use the module-level PyTorch statement)."""
    from tah_b200.ops import autograd_ops
    return autograd_ops.qk_norm_rope(qkv, q_w, k_w, position_ids, nq, nkv, hd, eps, theta)


def topk_softmax_embed(logits, embedding_weight, topk: int):
    if _use_cuda(logits):
        from tah_b200.ops import autograd_ops
        return autograd_ops.topk_softmax_embed(logits, embedding_weight, topk)
    return torch_ref.topk_softmax_embed(logits, embedding_weight, topk)


def duo_attention(q, k, v, q_pos, kv_pos, kv_valid, q_depth=None, kv_depth=None):
    if _use_cuda(q):
        from tah_b200.ops import autograd_ops
        return autograd_ops.duo_attention(q, k, v, q_pos, kv_pos, kv_valid, q_depth, kv_depth)
    return torch_ref.duo_attention(q, k, v, q_pos, kv_pos, kv_valid, q_depth, kv_depth)
