"""Training / evaluation losses for TaH.

A loss object follows a three-call protocol (reference ``tah/model/loss.py:36-54``):
``prepare_loss`` once per forward, ``intra_iter_loss_func`` after every pass when
``_is_intra_iter_loss`` is set, and ``final_loss_func`` at the end.

The model hands the per-pass call *flat* tensors: ``active_index`` holds the
row-major ``b*T+t`` index of every token processed in the pass, in the same
order in which the reference's boolean-mask indexing visits them, so sums and
means are taken over the same sets as in the reference.

* :class:`NextTokenPredLoss` - CE in fp32 on the final logits (reference ``loss.py:57-81``).
* :class:`IterDeciderLoss` - per-pass BCE on the decider logits, spread over the
  contributing tokens and reduced at the end (reference ``loss.py:89-245``),
  including its normalisation: ``sum / num_items_in_batch`` when the trainer
  supplies a count, otherwise a mean over every position that was processed
  and carries a label.
* :class:`CombinedLoss` - CE + weight * BCE, the objective named by the FSDP
  benchmark configuration (no counterpart in the reference).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F


def fixed_cross_entropy(source, target, num_items_in_batch=None, ignore_index: int = -100, **_):
    """CE that sums and divides by ``num_items_in_batch`` when given (reference
    ``tah/train/trainer.py:95-107``), else averages over non-ignored targets."""
    if num_items_in_batch is None:
        return F.cross_entropy(source, target, ignore_index=ignore_index, reduction="mean")
    return F.cross_entropy(source, target, ignore_index=ignore_index, reduction="sum") / num_items_in_batch


class LossFunc:
    _is_intra_iter_loss: bool = False

    def __init__(self, **kwargs):
        self.config = kwargs

    def prepare_loss(self, batch_size, query_len, device, dtype, **kwargs) -> None:
        pass

    def intra_iter_loss_func(self, *args, **kwargs):
        raise NotImplementedError

    def final_loss_func(self, *args, **kwargs) -> torch.Tensor:
        raise NotImplementedError


class NextTokenPredLoss(LossFunc):
    def __init__(self, **kwargs):
        super().__init__()

    def final_loss_func(self, logits, labels_shifted, iter_count=None, training=True, **kwargs):
        flat = logits.reshape(-1, logits.shape[-1])
        labels = labels_shifted.reshape(-1).to(flat.device)
        n_items = kwargs.get("num_items_in_batch")
        if flat.is_cuda and flat.dtype == torch.bfloat16:
            from tah_b200.ops import autograd_ops
            if autograd_ops.cross_entropy_sum_ok(flat):
                # one kernel over the bf16 logits (fp32 math): no fp32 copy of the [B*T, V] tensor
                total = autograd_ops.cross_entropy_sum(flat, labels)
                if n_items is None:
                    return total / (labels != -100).sum().clamp(min=1)
                return total / n_items
        return fixed_cross_entropy(flat.float(), labels, num_items_in_batch=n_items)


class IterDeciderLoss(LossFunc):
    _is_intra_iter_loss = True

    def __init__(self, pos_weight: Optional[float] = None, skip_last_iter: bool = True,
                 max_iter: Optional[int] = None, **kwargs):
        super().__init__()
        self.pos_weight = pos_weight
        self.skip_last_iter = bool(skip_last_iter)
        self.max_iter = None if max_iter is None else int(max_iter)
        if self.skip_last_iter and self.max_iter is None:
            raise ValueError("max_iter must be set when skip_last_iter is True")
        self.iter_decider_loss_per_token: Optional[torch.Tensor] = None
        self._correct = None
        self._total = None

    def prepare_loss(self, batch_size, query_len, device, dtype, **kwargs):
        self.iter_decider_loss_per_token = torch.zeros(batch_size, query_len, device=device, dtype=torch.float32)
        self._correct = torch.zeros((), device=device, dtype=torch.float32)
        self._total = torch.zeros((), device=device, dtype=torch.float32)

    def intra_iter_loss_func(self, *, active_index, active_valid, continue_logits, iter_depth,
                             active_iter_count_labels=None, iter_decider_threshold=0.5, **kwargs):
        """``active_index`` (N,), ``active_valid`` (N,) bool, ``continue_logits`` (N_valid,),
        ``active_iter_count_labels`` (N,) or None.  No host synchronisation."""
        if (active_iter_count_labels is None or continue_logits is None or active_index.numel() == 0
                or (self.skip_last_iter and int(iter_depth) >= int(self.max_iter))):
            return None
        labels = active_iter_count_labels[active_valid]
        has_label = labels != -100
        w = has_label.float()
        n = w.sum()
        z = continue_logits.float()
        thr = iter_decider_threshold
        if z.is_cuda and os.environ.get("TAH_B200_FORCE_TORCH", "0") != "1":
            # BCE terms, labelled count and accuracy counter in one kernel (and one for the backward)
            from tah_b200.ops import autograd_ops
            thr_f = float(thr.detach().float()) if isinstance(thr, torch.Tensor) else float(thr)
            bsum, n, correct = autograd_ops.bce_sum(z, labels, int(iter_depth), 1.0 if self.pos_weight is None
                                                    else float(self.pos_weight), thr_f)
            denom = n.clamp(min=1.0)
            mean_bce = bsum / denom
            with torch.no_grad():
                self._correct += correct
                self._total += n
        else:
            target = (labels > iter_depth).float()
            pw = None if self.pos_weight is None else torch.tensor(self.pos_weight, device=z.device)
            per = F.binary_cross_entropy_with_logits(z, target, pos_weight=pw, reduction="none")
            denom = n.clamp(min=1.0)
            mean_bce = (per * w).sum() / denom                # BCE averaged over contributing tokens
            if isinstance(thr, torch.Tensor):
                thr = thr.detach().float()
            with torch.no_grad():
                pred = (torch.sigmoid(z) > thr).float()
                self._correct += ((pred == target).float() * w).sum()
                self._total += n
        # every contributing token receives mean_bce / n, so that the final
        # sum over tokens reproduces the per-pass mean
        share = (mean_bce / denom) * w
        dense = torch.zeros_like(self.iter_decider_loss_per_token).view(-1)
        dense = dense.index_put((active_index[active_valid],), share, accumulate=True)
        self.iter_decider_loss_per_token = self.iter_decider_loss_per_token + dense.view_as(self.iter_decider_loss_per_token)
        return dense

    def final_loss_func(self, logits, labels_shifted, iter_count, iter_count_labels=None,
                        training=True, **kwargs):
        if self.iter_decider_loss_per_token is None:
            raise RuntimeError("prepare_loss has not been called")
        acc, self.iter_decider_loss_per_token = self.iter_decider_loss_per_token, None
        valid = iter_count > 0
        if iter_count_labels is not None:
            valid = valid & (iter_count_labels != -100)
        callback = kwargs.get("logger_callback")
        num_items = kwargs.get("num_items_in_batch")
        if callback is not None and self._total is not None:
            with torch.no_grad():
                if num_items:
                    inc = self._correct / num_items
                else:
                    inc = self._correct / self._total.clamp(min=1.0)
                callback.iter_decider_accuracy = getattr(callback, "iter_decider_accuracy", 0.0) + float(inc)
        self._correct = self._total = None
        vf = valid.float()
        if num_items is not None:
            return (acc * vf).sum() / num_items
        return (acc * vf).sum() / vf.sum().clamp(min=1.0)


class CombinedLoss(LossFunc):
    """Next-token CE on the selected output plus ``bce_weight`` x decider BCE."""

    _is_intra_iter_loss = True

    def __init__(self, bce_weight: float = 1.0, pos_weight: Optional[float] = None,
                 skip_last_iter: bool = True, max_iter: Optional[int] = None, **kwargs):
        super().__init__()
        self.bce_weight = bce_weight
        self.ce = NextTokenPredLoss()
        self.bce = IterDeciderLoss(pos_weight=pos_weight, skip_last_iter=skip_last_iter, max_iter=max_iter)

    def prepare_loss(self, *a, **kw):
        self.bce.prepare_loss(*a, **kw)

    def intra_iter_loss_func(self, **kw):
        return self.bce.intra_iter_loss_func(**kw)

    def final_loss_func(self, logits, labels_shifted, iter_count, **kw):
        ce = self.ce.final_loss_func(logits, labels_shifted, iter_count, **kw)
        bce = self.bce.final_loss_func(logits, labels_shifted, iter_count, **kw)
        return ce + self.bce_weight * bce


LOSS_BY_NAME = {
    "NextTokenPredLoss": NextTokenPredLoss,
    "IterDeciderLoss": IterDeciderLoss,
    "CombinedLoss": CombinedLoss,
}


def get_loss_func_class(name: str):
    try:
        return LOSS_BY_NAME[name]
    except KeyError:
        raise ValueError(f"Unknown loss {name!r}; have {sorted(LOSS_BY_NAME)}") from None
