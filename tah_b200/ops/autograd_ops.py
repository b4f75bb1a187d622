"""Differentiable CUDA ops used by the PyTorch model path (training, parity tests on GPU).

Forward passes run the hand-written kernels where the tensor layout allows (bf16, K a multiple
of 64); the backward passes are written out explicitly here.  Inputs the kernels do not cover
(fp32 models, odd shapes) take the PyTorch statement of the op.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.nn.functional as F

from tah_b200.ops import cuda as K
from tah_b200.ops import torch_ref


def _gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 64 == 0
            and w.shape[0] % 8 == 0 and x.numel() > 0)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        out = K.gemm(x2, w if w.is_contiguous() else w.contiguous())
        return out.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        gx = gw = None
        g2 = gy.reshape(-1, gy.shape[-1])
        if ctx.needs_input_grad[0]:
            gx = (g2 @ w).view_as(x)
        if ctx.needs_input_grad[1]:
            gw = g2.t() @ x.reshape(-1, x.shape[-1])
        return gx, gw


def linear(x, w):
    if _gemm_ok(x, w):
        return _Linear.apply(x, w)
    return torch_ref.linear(x, w)


def lora_linear(x, w, xa, lora_A, lora_B: List[torch.Tensor], adapted: Sequence[int], out_splits: Sequence[int],
                r: int, scaling: float):
    y = linear(x, w)
    t = F.linear(xa, lora_A)
    pieces = list(y.split(list(out_splits), dim=-1))
    for j, idx in enumerate(adapted):
        pieces[idx] = pieces[idx] + scaling * F.linear(t[..., j * r:(j + 1) * r], lora_B[j])
    return torch.cat(pieces, dim=-1) if len(pieces) > 1 else pieces[0]


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        ctx.save_for_backward(x, w)
        ctx.eps = eps
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        return K.rms_norm(x2, w, eps).view_as(x)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        xf, gf, wf = x.float(), gy.float(), w.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + ctx.eps)
        xn = xf * rstd
        gw = (gf * xn).reshape(-1, x.shape[-1]).sum(0).to(w.dtype) if ctx.needs_input_grad[1] else None
        gx = None
        if ctx.needs_input_grad[0]:
            gn = gf * wf
            gx = (rstd * (gn - xn * (gn * xn).mean(-1, keepdim=True))).to(x.dtype)
        return gx, gw, None


def rms_norm(x, weight, eps):
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 \
            and x.shape[-1] <= 8192 and x.numel() > 0:
        return _RMSNorm.apply(x, weight, eps)
    return torch_ref.rms_norm(x, weight, eps)


def swiglu(gate_up):
    return torch_ref.swiglu(gate_up)


def duo_attention(q, k, v, q_pos, kv_pos, kv_valid, q_depth=None, kv_depth=None):
    return torch_ref.duo_attention(q, k, v, q_pos, kv_pos, kv_valid, q_depth, kv_depth)
