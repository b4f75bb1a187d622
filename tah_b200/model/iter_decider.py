"""Per-token "iterate again?" deciders.

Call contract (reference ``tah/model/iter_decider.py:15-21``)::

    decision, decision_logits = decider(logits, iter_depth, all_hidden_states=...,
                                        labels_shifted=..., iter_count_labels=...)

``decision`` is a bool tensor over the leading dims of ``logits`` (True means
"run one more pass"), ``decision_logits`` the pre-sigmoid score used by the BCE
loss.  ``iter_depth`` is the number of passes already done, so a decider
returns all-False once ``iter_depth >= max_iter``.

Classes:

* :class:`IterLabelDecider` - oracle labels decide (reference ``:100-119``).
* :class:`MLPIterDecider` - learned classifier over tapped hidden states and
  the sorted top-k logit values (reference ``:194-301``).  Sub-module names
  match the reference so ``iter_decider.bin`` state dicts are interchangeable.
* :class:`SimpleMLPIterDecider` - the two-layer ``H -> H/4 -> 1`` decider used
  by the synthetic benchmark configurations.
* :class:`BernoulliIterDecider` - a seeded random hard-token mask, used to give
  random-init benchmark models the 6 % hard-token rate of a trained model.

Unlike the reference, no decider reads a tensor back to the host: thresholds
are compared on the device, so a forward pass can be captured in a CUDA graph.
"""
from __future__ import annotations

import inspect
import os
from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn

NEUTRAL_LOGITS = 0.0
MINUS_INFINITY_LOGITS = -10.0


def _remember_init_args(cls):
    """Record constructor arguments on ``self._init_args`` (for persistence)."""
    init = cls.__init__
    names = [n for n in inspect.signature(init).parameters if n != "self"]

    def wrapped(self, *args, **kwargs):
        init(self, *args, **kwargs)
        seen = dict(zip(names, args))
        seen.update(kwargs)
        self._init_args = seen

    wrapped.__wrapped__ = init
    cls.__init__ = wrapped
    return cls


class IterDecider(nn.Module):
    def __init__(self, threshold: float = 0.5, max_iter: int = 3):
        super().__init__()
        self.register_buffer("threshold", torch.tensor(float(threshold), dtype=torch.float32))
        self.max_iter = max_iter
        self._init_args: dict = {}

    def forward(self, logits: torch.Tensor, iter_depth: int, **kwargs):
        raise NotImplementedError

    def _stop_decision(self, logits: torch.Tensor, fill: float) -> Tuple[torch.Tensor, torch.Tensor]:
        lead = logits.shape[:-1]
        return (
            torch.zeros(lead, dtype=torch.bool, device=logits.device),
            torch.full(lead, fill, dtype=logits.dtype, device=logits.device),
        )


@_remember_init_args
class IterLabelDecider(IterDecider):
    """Continue iff the oracle label says the token needs more than ``iter_depth`` passes."""

    def __init__(self, max_iter: int = 3):
        super().__init__(max_iter=max_iter)

    def forward(self, logits, iter_depth, iter_count_labels: Optional[torch.Tensor] = None, **kwargs):
        if iter_depth >= self.max_iter:
            return self._stop_decision(logits, MINUS_INFINITY_LOGITS)
        stop, neutral = self._stop_decision(logits, NEUTRAL_LOGITS)
        if iter_count_labels is None:
            return stop, neutral
        go = (iter_count_labels > iter_depth) & (iter_count_labels != -100)
        return go, neutral


class _ClassifierBlock(nn.Module):
    """Pre-norm residual MLP block; a linear shortcut when the width changes."""

    def __init__(self, input_dim, output_dim, expansion_factor, dropout_rate, dtype=None):
        super().__init__()
        kw = {} if dtype is None else {"dtype": dtype}
        self.layer_norm = nn.LayerNorm(input_dim, **kw)
        # indices 0 and 3 hold the weights: keep this ordering for checkpoint keys
        self.mlp = nn.Sequential(
            nn.Linear(input_dim, input_dim * expansion_factor, **kw),
            nn.GELU(),
            nn.Dropout(dropout_rate),
            nn.Linear(input_dim * expansion_factor, output_dim, **kw),
            nn.Dropout(dropout_rate),
        )
        self.dim_change = nn.Identity() if input_dim == output_dim else nn.Linear(input_dim, output_dim, **kw)

    def forward(self, x):
        return self.dim_change(x) + self.mlp(self.layer_norm(x))


class _ClassifierBackbone(nn.Module):
    def __init__(self, input_dim, hidden_dims, expansion_factor, dropout_rate, output_dim=1, dtype=None):
        super().__init__()
        kw = {} if dtype is None else {"dtype": dtype}
        dims = list(hidden_dims)
        self.input_projection = nn.Linear(input_dim, dims[0], **kw)
        widths = dims + [dims[-1]]
        self.blocks = nn.ModuleList(
            _ClassifierBlock(widths[i], widths[i + 1], expansion_factor, dropout_rate, **kw)
            for i in range(len(widths) - 1)
        )
        self.output_layer = nn.Sequential(nn.LayerNorm(dims[-1], **kw), nn.Linear(dims[-1], output_dim, **kw))
        for mod in self.modules():
            if isinstance(mod, nn.Linear):
                nn.init.kaiming_normal_(mod.weight)
                if mod.bias is not None:
                    nn.init.zeros_(mod.bias)

    def forward(self, x):
        x = self.input_projection(x)
        for blk in self.blocks:
            x = blk(x)
        return self.output_layer(x)


@_remember_init_args
class MLPIterDecider(IterDecider):
    """Learned decider: features = [tapped hidden states || Linear(sorted top-k logits)]."""

    def __init__(
        self,
        topk: int = 100,
        hidden_states_size: int = 1024,
        hidden_states_layer_nums: Sequence[int] = (16, 20, 24, 28),
        hidden_dims: Sequence[int] = (256, 512, 256),
        expansion_factor: int = 4,
        dropout_rate: float = 0.3,
        normalize_input: bool = False,
        threshold: float = 0.5,
        max_iter: int = 3,
        dtype: torch.dtype = torch.bfloat16,
    ):
        super().__init__(max_iter=max_iter)
        self.topk = topk
        self.hidden_states_size = hidden_states_size
        self.hidden_states_layer_nums = list(hidden_states_layer_nums)
        self.normalize_input = normalize_input
        # the threshold is stored as a parameter (state-dict key "threshold") but never
        # receives a gradient: the decision is a hard comparison.
        del self._buffers["threshold"]
        self.threshold = nn.Parameter(torch.tensor(threshold, dtype=dtype))
        taps = max(1, len(self.hidden_states_layer_nums))
        if normalize_input:
            self.layer_norm_hidden_states = nn.LayerNorm(hidden_states_size * taps)
        self.logits_projection = nn.Linear(topk, hidden_states_size, dtype=dtype)
        self.combined_projection = nn.Linear(hidden_states_size * (taps + 1), hidden_dims[0], dtype=dtype)
        self.backbone = _ClassifierBackbone(hidden_dims[0], hidden_dims, expansion_factor, dropout_rate, dtype=dtype)
        self.sigmoid = nn.Sigmoid()

    def select_hidden(self, all_hidden_states, lead_shape, device, dtype):
        """``(..., L, H)`` (or ``(..., H)``) -> ``(..., taps*H)``; zeros when absent."""
        taps = max(1, len(self.hidden_states_layer_nums))
        width = self.hidden_states_size * taps
        if all_hidden_states is None:
            return torch.zeros(*lead_shape, width, device=device, dtype=dtype)
        hs = all_hidden_states
        if hs.dim() == len(lead_shape) + 1:
            hs = hs.unsqueeze(-2)
        n_layers = hs.size(-2)
        wanted = self.hidden_states_layer_nums or [n_layers - 1]
        if min(wanted) < 0 or max(wanted) >= n_layers:
            raise ValueError(f"hidden_states_layer_nums {wanted} out of range for {n_layers} layers")
        idx = torch.as_tensor(wanted, device=hs.device, dtype=torch.long)
        return hs.index_select(-2, idx).reshape(*lead_shape, width)

    def score(self, hidden_concat: torch.Tensor, topk_values: torch.Tensor) -> torch.Tensor:
        """Decision logits from already-selected features (used by the engine,
        which taps hidden states itself and gets sorted top-k values from the LM-head kernel)."""
        if self.normalize_input:
            hidden_concat = self.layer_norm_hidden_states(hidden_concat)
            topk_values = torch.softmax(topk_values, dim=-1)
        feats = torch.cat([hidden_concat, self.logits_projection(topk_values)], dim=-1)
        return self.backbone(self.combined_projection(feats)).squeeze(-1)

    def forward(self, logits, iter_depth, all_hidden_states=None, **kwargs):
        if iter_depth >= self.max_iter:
            return self._stop_decision(logits, MINUS_INFINITY_LOGITS)
        lead = logits.shape[:-1]
        hidden = kwargs.get("tapped_hidden_states")
        if hidden is None:
            hidden = self.select_hidden(all_hidden_states, lead, logits.device, logits.dtype)
        values, _ = torch.topk(logits, k=min(self.topk, logits.size(-1)), dim=-1)
        z = self.score(hidden, values)
        return torch.sigmoid(z) > self.threshold.detach().to(z.dtype), z


@_remember_init_args
class SimpleMLPIterDecider(IterDecider):
    """Two-layer decider ``H -> H/4 -> 1`` on the last tapped hidden state.

    Not part of the reference; it is the decider named by the synthetic
    benchmark configurations (e.g. 2048 -> 512 -> 1 for the 1.7B model).
    """

    def __init__(self, hidden_states_size: int = 1024, inner_size: Optional[int] = None,
                 hidden_states_layer_nums: Sequence[int] = (), threshold: float = 0.5,
                 max_iter: int = 2, dtype: torch.dtype = torch.bfloat16):
        super().__init__(threshold=threshold, max_iter=max_iter)
        inner = inner_size or hidden_states_size // 4
        self.hidden_states_size = hidden_states_size
        self.hidden_states_layer_nums = list(hidden_states_layer_nums)
        self.fc1 = nn.Linear(hidden_states_size, inner, dtype=dtype)
        self.fc2 = nn.Linear(inner, 1, dtype=dtype)

    def score(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.fc2(torch.nn.functional.silu(self.fc1(hidden))).squeeze(-1)

    def forward(self, logits, iter_depth, all_hidden_states=None, **kwargs):
        tapped = kwargs.get("tapped_hidden_states")
        if tapped is not None:
            all_hidden_states = tapped[..., -self.hidden_states_size:]
        if iter_depth >= self.max_iter or all_hidden_states is None:
            return self._stop_decision(logits, MINUS_INFINITY_LOGITS if iter_depth >= self.max_iter else NEUTRAL_LOGITS)
        hs = all_hidden_states
        if hs.dim() == logits.dim() + 1:
            tap = self.hidden_states_layer_nums[-1] if self.hidden_states_layer_nums else hs.size(-2) - 1
            hs = hs.select(-2, tap)
        z = self.score(hs.to(self.fc1.weight.dtype))
        return torch.sigmoid(z.float()) > self.threshold, z


@_remember_init_args
class BernoulliIterDecider(IterDecider):
    """Seeded coin flip per token: continue with probability ``p`` (``p_by_depth[d-1]`` if given).

    Optionally wraps an ``inner`` decider whose logits are still computed (so the
    decider's cost is part of a benchmark) while its decision is overridden.
    """

    def __init__(self, p: float = 0.06, seed: int = 0, max_iter: int = 2,
                 p_by_depth: Optional[Sequence[float]] = None, inner: Optional[nn.Module] = None):
        super().__init__(max_iter=max_iter)
        self.p = p
        self.p_by_depth = list(p_by_depth) if p_by_depth else None
        self.seed = seed
        self.inner = inner
        if inner is not None and hasattr(inner, "hidden_states_layer_nums"):
            self.hidden_states_layer_nums = inner.hidden_states_layer_nums
        self._gens = {}

    def _generator(self, device):
        key = str(device)
        if key not in self._gens:
            g = torch.Generator(device=device)
            g.manual_seed(self.seed)
            self._gens[key] = g
        return self._gens[key]

    def forward(self, logits, iter_depth, **kwargs):
        if iter_depth >= self.max_iter:
            return self._stop_decision(logits, MINUS_INFINITY_LOGITS)
        stop, z = self._stop_decision(logits, NEUTRAL_LOGITS)
        if self.inner is not None:
            _, z = self.inner(logits, iter_depth, **kwargs)
        p = self.p_by_depth[min(iter_depth - 1, len(self.p_by_depth) - 1)] if self.p_by_depth else self.p
        coin = torch.rand(stop.shape, device=logits.device, generator=self._generator(logits.device))
        return coin < p, z


ITER_DECIDER_BY_NAME = {
    "IterLabelDecider": IterLabelDecider,
    "MLPIterDecider": MLPIterDecider,
    "SimpleMLPIterDecider": SimpleMLPIterDecider,
    "BernoulliIterDecider": BernoulliIterDecider,
}


def get_iter_decider_class(name: str):
    try:
        return ITER_DECIDER_BY_NAME[name]
    except KeyError:
        raise ValueError(f"Unknown iter_decider {name!r}; have {sorted(ITER_DECIDER_BY_NAME)}") from None


def save_iter_decider(decider: IterDecider, save_directory: str) -> None:
    """Write ``iter_decider.bin`` = ``{"class", "state_dict" (cpu), "init_args"}``
    (same payload as reference ``iter_decider.py:322-330``)."""
    payload = {
        "class": type(decider).__name__,
        "state_dict": {k: v.detach().cpu() for k, v in decider.state_dict().items()},
        "init_args": {k: v for k, v in getattr(decider, "_init_args", {}).items() if not isinstance(v, nn.Module)},
    }
    torch.save(payload, os.path.join(save_directory, "iter_decider.bin"))


def load_iter_decider(load_directory: str, class_name: Optional[str] = None,
                      init_args: Optional[dict] = None) -> IterDecider:
    """Rebuild a decider.  State-dict entries whose name is also a constructor
    argument (e.g. ``threshold``) are dropped, so the configured value wins."""
    path = os.path.join(load_directory, "iter_decider.bin")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no iter_decider.bin at {path}")
    blob = torch.load(path, map_location="cpu", weights_only=False)
    name = class_name or blob.get("class")
    if not name:
        raise ValueError("iter_decider.bin lacks a class name")
    args = init_args if init_args is not None else blob.get("init_args", {})
    decider = get_iter_decider_class(name)(**args)
    weights = {k: v for k, v in (blob.get("state_dict") or {}).items() if k not in args}
    if weights:
        decider.load_state_dict(weights, strict=False)
    return decider
