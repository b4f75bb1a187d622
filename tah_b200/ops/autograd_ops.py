"""Differentiable CUDA ops used by the PyTorch model path (training, parity tests on GPU).

Forward passes run the hand-written kernels where the tensor layout allows (bf16, K a multiple
of 64); the backward passes are written out explicitly here.  Inputs the kernels do not cover
(fp32 models, odd shapes) take the PyTorch statement of the op.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from tah_b200.ops import cuda as K
from tah_b200.ops import torch_ref


def _gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 64 == 0
            and w.shape[0] % 8 == 0 and x.numel() > 0)


def _own_bwd() -> bool:
    return os.environ.get("TAH_B200_BWD_GEMM", "tcgen05") != "cublas"


def _dgrad(g2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``g2 [T, F] @ w [F, K] -> [T, K]`` (data gradient of ``y = x w^T``) on the tcgen05 GEMM: ``w`` is read
    transposed from its row-major storage (MN-major operand), no transposed copy is made."""
    if (_own_bwd() and g2.is_cuda and g2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 128 == 0
            and g2.shape[1] % 64 == 0 and g2.numel() > 0):
        return K.gemm_t(g2 if g2.is_contiguous() else g2.contiguous(), w if w.is_contiguous() else w.contiguous(), w_t=True)
    return g2 @ w


def _wgrad(g2: torch.Tensor, x2: torch.Tensor) -> torch.Tensor:
    """``g2^T [F, T] @ x2 [T, K] -> [F, K]`` (weight gradient): both operands are read transposed from their
    token-major storage, the reduction runs over the tokens.  When ``K`` cannot sit on the 128 tensor-memory lanes
    but ``F`` can, the transposed product is computed and returned as a view."""
    ok = (_own_bwd() and g2.is_cuda and g2.dtype == torch.bfloat16 and x2.dtype == torch.bfloat16 and g2.numel() > 0
          and g2.shape[1] % 8 == 0 and x2.shape[1] % 8 == 0)
    if ok:
        g2 = g2 if g2.is_contiguous() else g2.contiguous()
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        if x2.shape[1] % 128 == 0:
            return K.gemm_t(g2, x2, x_t=True, w_t=True)
        if g2.shape[1] % 128 == 0:
            return K.gemm_t(x2, g2, x_t=True, w_t=True).t()
    return g2.t() @ x2


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
            gx = _dgrad(g2, w).view_as(x)
        if ctx.needs_input_grad[1]:
            gw = _wgrad(g2, x.reshape(-1, x.shape[-1]))
        return gx, gw


def linear(x, w):
    if _gemm_ok(x, w):
        return _Linear.apply(x, w)
    return torch_ref.linear(x, w)


class _LoRALinear(torch.autograd.Function):
    """``x W^T + t Bd^T`` in one tcgen05 GEMM (the adapter is a K-extension of the base GEMM, as in the
    inference engine); ``t = xa A^T`` and the block-diagonal scaled ``Bd`` are built by the caller."""

    @staticmethod
    def forward(ctx, x, w, t, bd):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        t2 = t.reshape(-1, t.shape[-1]).contiguous()
        ctx.save_for_backward(x2, w, t2, bd)
        ctx.shapes = (x.shape, t.shape)
        out = K.gemm(x2, w if w.is_contiguous() else w.contiguous(), x2=t2, w2=bd)
        return out.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w, t2, bd = ctx.saved_tensors
        xs, ts = ctx.shapes
        g2 = gy.reshape(-1, gy.shape[-1])
        gx = _dgrad(g2, w).view(xs) if ctx.needs_input_grad[0] else None
        gw = _wgrad(g2, x2) if ctx.needs_input_grad[1] else None
        gt = None
        if ctx.needs_input_grad[2]:
            # rank-sized output: the K-major form on a transposed copy of the small block-diagonal B
            if _own_bwd() and g2.shape[1] % 64 == 0 and bd.shape[1] % 8 == 0:
                gt = K.gemm(g2 if g2.is_contiguous() else g2.contiguous(), bd.t().contiguous()).view(ts)
            else:
                gt = (g2 @ bd).view(ts)
        gbd = _wgrad(g2, t2) if ctx.needs_input_grad[3] else None
        return gx, gw, gt, gbd


def lora_linear(x, w, xa, lora_A, lora_B: List[torch.Tensor], adapted: Sequence[int], out_splits: Sequence[int],
                r: int, scaling: float):
    R = len(adapted) * r
    if _gemm_ok(x, w) and R % 64 == 0 and lora_A.dtype == torch.bfloat16:
        t = linear(xa, lora_A)
        bd = w.new_zeros(w.shape[0], R)
        off = [0]
        for sz in out_splits:
            off.append(off[-1] + sz)
        for j, idx in enumerate(adapted):
            bd[off[idx]:off[idx + 1], j * r:(j + 1) * r] = lora_B[j] * scaling
        return _LoRALinear.apply(x, w, t, bd)
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
        if x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
            x2 = x.reshape(-1, x.shape[-1]).contiguous()
            g2 = gy.reshape(-1, x.shape[-1]).contiguous()
            gx, gw = K.rms_norm_bwd(x2, w.contiguous(), g2, ctx.eps, want_gw=ctx.needs_input_grad[1])
            return (gx.view_as(x) if ctx.needs_input_grad[0] else None), (gw.to(w.dtype) if gw is not None else None), None
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


class _QKNormRope(torch.autograd.Function):
    """Per-head QK RMSNorm + rotate-half RoPE of a fused ``[B, T, (nq + 2 nkv) * hd]`` projection."""

    @staticmethod
    def forward(ctx, qkv, q_w, k_w, pos, nq, nkv, hd, eps, theta):
        B, T, _ = qkv.shape
        x2 = qkv.reshape(B * T, -1).contiguous()
        p32 = pos.reshape(-1).to(torch.int32).contiguous()
        k = torch.empty(B * T, nkv * hd, dtype=qkv.dtype, device=qkv.device)
        v = torch.empty_like(k)
        q = K.qk_norm_rope_kv(x2, q_w, k_w, p32, nq, nkv, hd, eps, theta, k_dense=k, v_dense=v)
        ctx.save_for_backward(x2, q_w, k_w, p32)
        ctx.dims = (B, T, nq, nkv, hd, eps, theta)
        return q.view(B, T, nq, hd), k.view(B, T, nkv, hd), v.view(B, T, nkv, hd)

    @staticmethod
    def backward(ctx, gq, gk, gv):
        x2, q_w, k_w, p32 = ctx.saved_tensors
        B, T, nq, nkv, hd, eps, theta = ctx.dims
        gqkv, gqw, gkw = K.qk_norm_rope_bwd(x2, q_w, k_w, gq.reshape(B * T, -1).contiguous(),
                                            gk.reshape(B * T, -1).contiguous(), gv.reshape(B * T, -1).contiguous(),
                                            p32, nq, nkv, hd, eps, theta)
        return gqkv.view(B, T, -1), gqw.to(q_w.dtype), gkw.to(k_w.dtype), None, None, None, None, None, None


def qk_norm_rope_ok(qkv: torch.Tensor, hd: int) -> bool:
    return qkv.is_cuda and qkv.dtype == torch.bfloat16 and hd in (64, 128) and qkv.dim() == 3 and qkv.numel() > 0


def qk_norm_rope(qkv, q_w, k_w, position_ids, nq, nkv, hd, eps, theta):
    return _QKNormRope.apply(qkv, q_w, k_w, position_ids, nq, nkv, hd, eps, theta)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        g2 = gate_up.reshape(-1, gate_up.shape[-1]).contiguous()
        ctx.save_for_backward(g2)
        ctx.shape = gate_up.shape
        return K.swiglu(g2).view(*gate_up.shape[:-1], gate_up.shape[-1] // 2)

    @staticmethod
    def backward(ctx, gy):
        (g2,) = ctx.saved_tensors
        return K.swiglu_bwd(g2, gy.reshape(-1, gy.shape[-1]).contiguous()).view(ctx.shape)


class _CrossEntropySum(torch.autograd.Function):
    """Sum over rows of the cross entropy of bf16 logits, one kernel forward (online log-sum-exp in fp32, no fp32
    copy of the logits) and one backward that writes ``(softmax - onehot) * g`` in bf16."""

    @staticmethod
    def forward(ctx, logits, labels):
        loss, lse = K.ce_fwd(logits, labels)
        ctx.save_for_backward(logits, labels, lse)
        return loss.sum()

    @staticmethod
    def backward(ctx, g):
        logits, labels, lse = ctx.saved_tensors
        return K.ce_bwd(logits, labels, lse, g.reshape(1).float().contiguous()), None


def cross_entropy_sum_ok(logits: torch.Tensor) -> bool:
    return (logits.is_cuda and logits.dtype == torch.bfloat16 and logits.dim() == 2 and logits.stride(1) == 1
            and logits.stride(0) % 8 == 0 and logits.data_ptr() % 16 == 0 and logits.numel() > 0
            and os.environ.get("TAH_B200_FORCE_TORCH", "0") != "1")


def cross_entropy_sum(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """``sum_r CE(logits[r], labels[r])`` over rows whose label is not -100 (fp32 scalar)."""
    return _CrossEntropySum.apply(logits, labels.to(torch.int64).contiguous())


class _BceSum(torch.autograd.Function):
    """(weighted BCE-with-logits sum, labelled count, correct decisions) of the decider logits in one launch."""

    @staticmethod
    def forward(ctx, z, labels, depth, pos_weight, thr):
        ctx.save_for_backward(z, labels)
        ctx.args = (depth, pos_weight, thr)
        out = K.bce_logits(z, labels, depth, pos_weight, thr)
        ctx.mark_non_differentiable(out[1:])
        return out[0], out[1], out[2]

    @staticmethod
    def backward(ctx, g, _gn, _gc):
        z, labels = ctx.saved_tensors
        depth, pos_weight, thr = ctx.args
        return K.bce_logits(z, labels, depth, pos_weight, thr, g=g.reshape(1).float().contiguous()), None, None, None, None


def bce_sum(z: torch.Tensor, labels: torch.Tensor, depth: int, pos_weight: float, thr: float):
    return _BceSum.apply(z.float().contiguous(), labels.to(torch.int64).contiguous(), int(depth), float(pos_weight), float(thr))


def swiglu(gate_up):
    if gate_up.dtype == torch.bfloat16 and gate_up.shape[-1] % 16 == 0 and gate_up.numel() > 0:
        return _SwiGLU.apply(gate_up)
    return torch_ref.swiglu(gate_up)


def topk_softmax_embed(logits, embedding_weight, topk: int):
    """Soft next-pass input with the top-k indices from the radix-select kernel; the values are gathered
    from ``logits`` so that gradients flow to the logits and to the embedding rows as in the reference."""
    k = min(topk, logits.size(-1))
    if logits.dtype != torch.bfloat16 or logits.dim() != 2 or k > 128 or logits.numel() == 0:
        return torch_ref.topk_softmax_embed(logits, embedding_weight, topk)
    _, idx = K.topk_rows(logits.detach().contiguous(), k)
    vals = logits.gather(-1, idx.long())
    if embedding_weight.dtype == torch.bfloat16 and embedding_weight.is_contiguous() and embedding_weight.shape[1] % 8 == 0:
        return _SoftEmbedMix.apply(vals.float(), embedding_weight, idx)
    probs = torch.softmax(vals, dim=-1)
    return (probs.unsqueeze(-1) * embedding_weight[idx.long()]).sum(-2).to(embedding_weight.dtype)


class _SoftEmbedMix(torch.autograd.Function):
    """``sum_k softmax(vals)_k E[idx_k]`` with the mix kernel forward and one kernel backward: no ``[rows, k, H]``
    gather exists in either direction; the embedding gradient is scattered with vector reductions into an fp32
    accumulator (reference ``tah/model/tah_model.py:57-75`` and its autograd)."""

    @staticmethod
    def forward(ctx, vals, E, idx):
        ctx.save_for_backward(vals, E, idx)
        return K.soft_embed_rows(vals.contiguous(), idx.contiguous(), E)

    @staticmethod
    def backward(ctx, dout):
        vals, E, idx = ctx.saved_tensors
        dE = torch.zeros(E.shape, dtype=torch.float32, device=E.device)
        dval = K.soft_embed_bwd(dout.contiguous(), vals.contiguous(), idx.contiguous(), E, dE)
        return dval.to(vals.dtype), dE.to(E.dtype) if ctx.needs_input_grad[1] else None, None


def duo_attention(q, k, v, q_pos, kv_pos, kv_valid, q_depth=None, kv_depth=None):
    return torch_ref.duo_attention(q, k, v, q_pos, kv_pos, kv_valid, q_depth, kv_depth)


# ---------------------------------------------------------------------------------------------
# Duo-causal attention over per-depth KV segments on the tensor-core kernels (forward + backward)
# ---------------------------------------------------------------------------------------------
class SegmentMeta:
    """Index arrays that the packed attention kernels take, built once per backbone pass (the
    counterpart of the reference's per-pass mask construction, ``tah/model/tah_model.py:744-791``,
    with the KV order ``[iter-0 slot | iter-1 slot | ...]`` of ``tah/model/causal_cache.py:97-109``).

    Queries are the ``[B, Tq]`` tokens of the pass (row ``b * Tq + i``); segment ``s`` is the
    ``[B, Ts]`` K/V of iteration depth ``s``.  A query sees, in every segment, the valid entries of
    its own sample whose position is ``<=`` its own: with the valid entries of a sample stored
    contiguously in position order that is a prefix, described by ``base`` (row of the sample's
    first valid entry) and ``count`` (prefix length).
    """

    def __init__(self, q_pos: torch.Tensor, seg_pos: Sequence[torch.Tensor], seg_valid: Sequence[torch.Tensor],
                 q_valid: Optional[torch.Tensor] = None):
        B, Tq = q_pos.shape
        dev = q_pos.device
        self.B, self.Tq = B, Tq
        self.tile_q0, self.tile_qn = K.attn_tiles(torch.full((B,), Tq, device=dev))
        self.bases, self.counts, self.bounds, self.items, self.seg_T = [], [], [], [], []
        q_rows = torch.full((B,), Tq, device=dev)
        big = torch.iinfo(torch.int64).max
        for pos, valid in zip(seg_pos, seg_valid):
            Ts = pos.shape[1]
            v = valid.to(torch.bool)
            n_valid = v.sum(-1)
            first = torch.where(n_valid > 0, v.to(torch.int64).argmax(-1), torch.zeros_like(n_valid))
            keyed = torch.where(v, pos.to(torch.int64), torch.full_like(pos, big, dtype=torch.int64))
            keyed, _ = keyed.sort(dim=-1)
            cnt = torch.searchsorted(keyed, q_pos.to(torch.int64).contiguous(), right=True)
            cnt = torch.minimum(cnt, n_valid[:, None])
            if q_valid is not None:              # padding queries see nothing (zero output, zero gradients)
                cnt = cnt * q_valid.to(cnt.dtype)
            # the kernels size a tile's key walk by its last row: give them a non-decreasing bound
            bound = torch.cummax(cnt, dim=-1).values
            base = (torch.arange(B, device=dev) * Ts + first)
            self.bases.append(base[:, None].expand(B, Tq).reshape(-1).to(torch.int32).contiguous())
            self.counts.append(cnt.reshape(-1).to(torch.int32).contiguous())
            self.bounds.append(bound.reshape(-1).to(torch.int32).contiguous())
            self.items.append(K.attn_kv_items(n_valid, base, q_rows))
            self.seg_T.append(Ts)


class _SegmentAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, meta: SegmentMeta, *kv):
        B, Tq, nq, hd = q.shape
        n_seg = len(kv) // 2
        nkv = kv[0].shape[2]
        q2 = q.reshape(B * Tq, nq * hd).contiguous()
        ks = [kv[2 * s].reshape(-1, nkv * hd).contiguous() for s in range(n_seg)]
        vs = [kv[2 * s + 1].reshape(-1, nkv * hd).contiguous() for s in range(n_seg)]
        lse = torch.empty(B * Tq, nq, dtype=torch.float32, device=q.device)
        out = K.prefill_attn(q2, ks, vs, meta.bases, meta.counts, meta.tile_q0, meta.tile_qn, nq, nkv, hd, hd ** -0.5,
                             lse=lse, bounds=meta.bounds)
        ctx.meta, ctx.dims = meta, (B, Tq, nq, nkv, hd, n_seg)
        ctx.save_for_backward(q2, out, lse, *ks, *vs)
        return out.view(B, Tq, nq, hd)

    @staticmethod
    def backward(ctx, dout):
        B, Tq, nq, nkv, hd, n_seg = ctx.dims
        meta = ctx.meta
        q2, out, lse = ctx.saved_tensors[:3]
        ks = list(ctx.saved_tensors[3:3 + n_seg])
        vs = list(ctx.saved_tensors[3 + n_seg:])
        do2 = dout.reshape(B * Tq, nq * hd).contiguous()
        dsum = (do2.float() * out.float()).view(B * Tq, nq, hd).sum(-1).contiguous()
        scale = hd ** -0.5
        dq = K.attn_bwd_dq(q2, do2, ks, vs, meta.bases, meta.counts, meta.tile_q0, meta.tile_qn, nq, nkv, hd, scale,
                           lse, dsum, bounds=meta.bounds)
        grads = []
        for s in range(n_seg):
            dk, dv = K.attn_bwd_dkv(q2, do2, ks[s], vs[s], meta.counts[s], meta.items[s], nq, nkv, hd, scale, lse, dsum,
                                    bound=meta.bounds[s])
            grads += [dk.view(B, meta.seg_T[s], nkv, hd), dv.view(B, meta.seg_T[s], nkv, hd)]
        return (dq.view(B, Tq, nq, hd), None, *grads)


def segment_attention_ok(q: torch.Tensor, n_seg: int) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and 1 <= n_seg <= 3
            and q.shape[1] >= 16)


def segment_attention(q, k_list, v_list, meta: SegmentMeta):
    """Attention of the pass's queries ``[B, Tq, nq, hd]`` over the per-depth K/V segments
    (``[B, Ts, nkv, hd]`` each) on the tcgen05 kernels, differentiable in q and every K/V."""
    kv = []
    for k, v in zip(k_list, v_list):
        kv += [k, v]
    return _SegmentAttention.apply(q, meta, *kv)
