"""TaHForCausalLM: selective latent iterations on hard tokens.

Function (reference ``tah/model/tah_model.py:495-740``): pass 0 runs the plain
backbone on every token; a per-token decider marks tokens that continue; for
those the next pass's input is the top-k-softmax mix of embedding rows taken
from the cumulative logits, the backbone is re-run with the LoRA adapter on, at
the same positions, attending under the duo-causal rule, and the new logits are
added to the old ones.  At most ``max_iter`` passes in total.

Implementation differences, all result-preserving:

* an :class:`ActiveSet` computes the compaction indices of a pass once and every
  gather/scatter of the pass reuses them (the reference re-sorts about eight
  times per pass);
* cumulative logits are carried only for the tokens that are still active; no
  dense ``(B, T, V)`` cumulative buffer exists;
* attention gets positions, never a materialised additive mask;
* hidden states are tapped only at the layers the decider reads;
* one host synchronisation per pass (the padded width of the next active block)
  instead of six or more, and none in the deciders or losses.
"""
from __future__ import annotations

import json
import logging
import os
from dataclasses import asdict, dataclass
from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from tah_b200 import ops
from tah_b200.model.causal_cache import TaHCache
from tah_b200.model.iter_decider import (ITER_DECIDER_BY_NAME, IterDecider, load_iter_decider,
                                         save_iter_decider)
from tah_b200.model.loss import LOSS_BY_NAME, LossFunc
from tah_b200.model.tah_config import TaHConfig, resolve_config, save_config
from tah_b200.models import qwen3
from tah_b200.models.qwen3 import LoRASpec, Qwen3Config, Qwen3ForCausalLM

log = logging.getLogger(__name__)


# ------------------------------------------------------------------------------------
# public helpers
# ------------------------------------------------------------------------------------

def topk_softmax_input_update(logits: torch.Tensor, embedding_weight: torch.Tensor, topk: int) -> torch.Tensor:
    """Next-pass input embedding: ``sum_k softmax(top-k logits)_k * E[idx_k]`` (reference ``:57-75``)."""
    return ops.topk_softmax_embed(logits, embedding_weight, topk)


def additive_logits_update(logits: torch.Tensor, prev_logits: Optional[torch.Tensor]) -> torch.Tensor:
    return logits if prev_logits is None else prev_logits + logits


class ActiveSet:
    """Compaction indices of one pass: the True entries of a ``(B, S)`` mask, row-major.

    ``b``/``s`` are the coordinates of the active tokens in the dense layout and
    ``k`` their column in the right-padded ``(B, width)`` block, so
    ``block[b, k] = dense[b, s]`` packs and ``dense[b, s] = block[b, k]`` unpacks.
    """

    def __init__(self, mask: torch.Tensor, min_width: int = 0):
        self.mask = mask
        B, S = mask.shape
        self.counts = mask.sum(1)
        self.b, self.s = mask.nonzero(as_tuple=True)
        self.k = (mask.cumsum(1) - 1)[self.b, self.s]
        self.width = max(int(self.counts.max()) if B > 0 and S > 0 else 0, min_width)   # one host sync
        self.pad_mask = torch.arange(self.width, device=mask.device)[None, :] >= self.counts[:, None]
        self.flat = self.b * S + self.s

    @property
    def n(self) -> int:
        return self.b.numel()

    @property
    def full(self) -> bool:
        """Every slot of the ``(B, width)`` block is active: the block is the active list reshaped."""
        return self.width > 0 and self.n == self.mask.shape[0] * self.width

    def pack(self, dense: Optional[torch.Tensor], pad_value=0):
        if dense is None:
            return None
        if self.full and self.width == dense.shape[1]:
            return dense                      # every token active: the block is the tensor itself
        out = dense.new_full((dense.shape[0], self.width) + tuple(dense.shape[2:]), pad_value)
        out[self.b, self.k] = dense[self.b, self.s]
        return out

    def pack_flat(self, values: torch.Tensor, pad_value=0):
        """``values`` ``(n, ...)`` in active order -> padded ``(B, width, ...)`` block."""
        if self.full:
            return values.view(self.mask.shape[0], self.width, *values.shape[1:])
        out = values.new_full((self.mask.shape[0], self.width) + tuple(values.shape[1:]), pad_value)
        out[self.b, self.k] = values
        return out

    def unpack_into(self, block: torch.Tensor, dense: torch.Tensor, select: Optional[torch.Tensor] = None):
        """In-place ``dense[b, s] = block[b, k]`` (restricted to ``select`` (n,) bool when given)."""
        if select is None:
            dense[self.b, self.s] = block[self.b, self.k]
        else:
            dense[self.b[select], self.s[select]] = block[self.b[select], self.k[select]]
        return dense


def gather_active(current_iter_mask: torch.Tensor, *tensors, pad_value=0):
    """Pack the active positions of each ``(B, S, ...)`` tensor to the left of a
    right-padded ``(B, max_active, ...)`` block.  Returns ``(pad_mask, *packed)``;
    ``None`` inputs pass through (reference ``tah_model.py:96-135``)."""
    act = ActiveSet(current_iter_mask)
    return (act.pad_mask,) + tuple(act.pack(t, pad_value) for t in tensors)


def scatter_back(current_iter_mask: torch.Tensor, src: torch.Tensor, dest: torch.Tensor, *,
                 in_place: bool = False, assignment_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inverse of :func:`gather_active`: write the valid prefix of each row of ``src``
    to the True positions of ``current_iter_mask`` in ``dest``; with
    ``assignment_mask`` only where that is True too (reference ``:138-176``)."""
    act = ActiveSet(current_iter_mask)
    out = dest if in_place else dest.clone()
    sel = None if assignment_mask is None else assignment_mask[act.b, act.s]
    return act.unpack_into(src, out, sel)


@dataclass
class TaHCausalLMOutputWithPast:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    past_key_values: Optional[TaHCache] = None
    hidden_states: Optional[Tuple[torch.Tensor]] = None
    attentions: Optional[Tuple[torch.Tensor]] = None
    iter_count: Optional[torch.Tensor] = None
    iter_count_labels: Optional[torch.Tensor] = None

    def __getitem__(self, key):
        if isinstance(key, str):
            return getattr(self, key)
        return tuple(v for v in asdict(self).values() if v is not None)[key]


def _with_max_iter(kwargs: Optional[dict], max_iter: int) -> dict:
    out = dict(kwargs or {})
    out.setdefault("max_iter", max_iter)
    return out


def _build_loss(name: str, kwargs: dict, max_iter: int) -> LossFunc:
    return LOSS_BY_NAME[name](**_with_max_iter(kwargs, max_iter))


def _build_iter_decider(name: str, kwargs: dict, max_iter: int) -> IterDecider:
    return ITER_DECIDER_BY_NAME[name](**_with_max_iter(kwargs, max_iter))


def _resolve_attr_path(root, dotted: str):
    obj = root
    for seg in dotted.split("."):
        if seg and seg != "self":
            obj = getattr(obj, seg)
    return obj


# ------------------------------------------------------------------------------------
# the model
# ------------------------------------------------------------------------------------

class TaHForCausalLM(nn.Module):
    """``TaHForCausalLM(base_model, config)``; ``base_model`` is a
    :class:`~tah_b200.models.qwen3.Qwen3ForCausalLM` or a HuggingFace Qwen3 causal LM
    (converted on entry).  Public attributes follow the reference: ``tah_config``,
    ``max_iter``, ``input_topk``, ``iter_decider``, ``eval_iter_decider``,
    ``train_loss``, ``eval_loss``, ``simple_base_model``, ``embedding_key``,
    optional ``logger_callback``; properties ``device`` and ``embed_tokens``."""

    def __init__(self, base_model, config: Optional[TaHConfig] = None):
        super().__init__()
        config = config or TaHConfig()
        if config.adapter != "lora":
            raise ValueError(f"adapter must be 'lora', got {config.adapter!r}")
        self.tah_config = config
        spec = LoRASpec.from_adapter_kwargs(config.adapter_kwargs)
        if not isinstance(base_model, Qwen3ForCausalLM):
            base_model = qwen3.from_hf_model(base_model, spec)
        elif base_model.lora.r != spec.r or tuple(base_model.lora.targets) != tuple(spec.targets) \
                or base_model.lora.lora_alpha != spec.lora_alpha or base_model.lora.lora_dropout != spec.lora_dropout:
            qwen3.attach_lora(base_model, spec)
        self.simple_base_model = base_model
        self.config = base_model.config
        try:
            _resolve_attr_path(base_model, config.embedding_key)
        except AttributeError as exc:
            raise ValueError(f"embedding_key {config.embedding_key!r} not found in base model") from exc
        self.embedding_key = config.embedding_key
        self.max_iter = config.max_iter if config.max_iter is not None else 1
        self.input_topk = int(config.input_updater_kwargs.get("topk", 100))
        self.iter_decider = _build_iter_decider(config.iter_decider or "IterLabelDecider",
                                                config.iter_decider_kwargs, self.max_iter)
        self.eval_iter_decider = self._resolve_eval_iter_decider(config)
        self.train_loss = _build_loss(config.train_loss or "NextTokenPredLoss", config.train_loss_kwargs, self.max_iter)
        self.eval_loss = (_build_loss(config.eval_loss, config.eval_loss_kwargs, self.max_iter)
                          if config.eval_loss else self.train_loss)
        self._set_lora_grad_flags(config.adapter_kwargs.get("base_grad", True),
                                  config.adapter_kwargs.get("adapter_grad", True))
        # run every forward for exactly max_iter passes (possibly over empty active sets), so
        # that ranks of a sharded training job issue the same collectives
        self.uniform_passes = False
        self.supports_gradient_checkpointing = True

    # ---- adapters / deciders -----------------------------------------------------------
    def _set_lora_grad_flags(self, base_grad: bool, adapter_grad: bool) -> None:
        for name, p in self.simple_base_model.named_parameters():
            p.requires_grad = adapter_grad if "lora" in name.lower() else base_grad

    def _resolve_eval_iter_decider(self, config: TaHConfig) -> IterDecider:
        name = config.eval_iter_decider
        if not name:
            return self.iter_decider
        if isinstance(name, str) and name.startswith("iter_decider"):
            return _resolve_attr_path(self, name)
        return _build_iter_decider(name, config.eval_iter_decider_kwargs, self.max_iter)

    @property
    def device(self):
        return self.simple_base_model.device

    @property
    def dtype(self):
        return self.simple_base_model.dtype

    @property
    def embed_tokens(self):
        return _resolve_attr_path(self.simple_base_model, self.embedding_key)

    @property
    def _active_iter_decider(self) -> IterDecider:
        return self.iter_decider if self.training else (self.eval_iter_decider or self.iter_decider)

    def gradient_checkpointing_enable(self, *a, **k):
        self.simple_base_model.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.simple_base_model.gradient_checkpointing = False

    @staticmethod
    def _forward_kwargs(kwargs: dict) -> dict:
        return {k: v for k, v in kwargs.items() if k in ("num_items_in_batch",)}

    def _force_one_continuation(self, decision, labels_valid, iter_depth: int):
        """When labels exist and the decider stopped every labelled token, make one
        random labelled token continue (keeps decider gradients alive).  Sync-free."""
        if labels_valid is None or decision is None or decision.numel() == 0 or iter_depth >= self.max_iter:
            return decision
        labelled = labels_valid != -100
        need = labelled.any() & ~(decision & labelled).any()
        pick = (torch.rand(labelled.shape, device=decision.device) + 1.0) * labelled
        forced = torch.zeros_like(decision)
        forced[pick.argmax()] = True
        return decision | (forced & need)

    # ---- forward -----------------------------------------------------------------------
    def forward(self, input_ids: torch.LongTensor, attention_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.LongTensor] = None, past_key_values: Optional[TaHCache] = None,
                labels: Optional[torch.LongTensor] = None, iter_count_labels: Optional[torch.LongTensor] = None,
                use_cache: bool = False, new_sequence: bool = False, **kwargs) -> TaHCausalLMOutputWithPast:
        assert not kwargs.get("output_attentions"), "TaH does not support output_attentions"
        assert not kwargs.get("output_hidden_states"), "TaH does not support output_hidden_states"
        base = self.simple_base_model
        B, T = input_ids.shape
        V = self.config.vocab_size
        device = input_ids.device

        if labels is not None:
            labels_shifted = F.pad(labels, (0, 1), value=-100)[..., 1:].contiguous()
            labels_all_shifted = F.pad(input_ids, (0, 1), value=-100)[..., 1:].contiguous()
        else:
            labels_shifted = labels_all_shifted = None

        embed_w = self.embed_tokens.weight
        input_embeds = F.embedding(input_ids, embed_w)
        dtype = input_embeds.dtype
        cache = past_key_values if past_key_values is not None else TaHCache().to(device=device, dtype=dtype)

        if attention_mask is not None:
            valid_mask = attention_mask[:, -T:].to(torch.long)
            assert valid_mask.shape == (B, T), f"attention_mask shape {tuple(attention_mask.shape)} bad for T={T}"
        else:
            valid_mask = torch.ones(B, T, dtype=torch.long, device=device)
        if position_ids is None:
            prior = cache.get_valid_mask_upto_iter(0, 0, init_batch_size=B).to(device)
            position_ids = (torch.cat((prior, valid_mask), dim=-1).cumsum(-1)[:, -T:] - 1).clamp(min=0)

        loss_func = self.train_loss if self.training else self.eval_loss
        loss_func.prepare_loss(B, T, device, dtype)
        track_labels = iter_count_labels is not None and labels_shifted is not None
        full_iter_labels = torch.zeros(B, T, dtype=torch.long, device=device) if track_labels else None

        final_logits = torch.zeros(B, T, V, device=device, dtype=dtype)
        iter_counts = torch.zeros(B, T, dtype=torch.long, device=device)
        decider = self._active_iter_decider
        taps: Sequence[int] = tuple(getattr(decider, "hidden_states_layer_nums", ()) or ())
        wants_all_layers = bool(getattr(decider, "needs_all_hidden_states", False))

        all_valid = bool(valid_mask.all())            # no padding anywhere: validity gathers are identities
        current = torch.ones(B, T, dtype=torch.bool, device=device)
        act = ActiveSet(current)
        block_embeds = input_embeds                       # (B, width, H) input of the pass
        carried: Optional[torch.Tensor] = None            # (n, V) cumulative logits of the active tokens
        depth = 0
        while depth < self.max_iter and (act.n > 0 or self.uniform_passes):
            if act.width == 0:
                act = ActiveSet(current, min_width=1)
                block_embeds = input_embeds.new_zeros(B, 1, input_embeds.shape[-1])
            a_pos = act.pack(position_ids)
            a_valid = act.pack(valid_mask)
            a_labels = act.pack(labels_shifted, -100)
            a_labels_all = act.pack(labels_all_shifted, -100)
            a_iter_labels = act.pack(iter_count_labels)

            store = True if depth < self.max_iter - 1 else use_cache
            cache.begin_pass(depth, a_pos, a_valid, store=store)
            tap_layers = range(self.config.num_hidden_layers + 1) if wants_all_layers else taps
            hidden, tapped = base.backbone(block_embeds, a_pos, cache, lora_on=depth >= 1, tap_layers=tap_layers)
            pass_logits = base.logits(hidden)              # (B, width, V)
            depth += 1

            # (n, V) in active order; with every slot active this is a view, not a gather of the logits
            flat_logits = pass_logits.reshape(-1, V) if act.full else pass_logits[act.b, act.k]
            updated = additive_logits_update(flat_logits, carried)

            v_act = a_valid[act.b, act.k] == 1             # (n,) validity of the active tokens
            pick = (lambda t: t) if all_valid else (lambda t: t[v_act])
            dec_kwargs = {}
            if wants_all_layers:
                stack = torch.stack([tapped[i] for i in range(self.config.num_hidden_layers + 1)], dim=2)
                dec_kwargs["all_hidden_states"] = pick(stack[act.b, act.k])
            elif taps:
                dec_kwargs["tapped_hidden_states"] = pick(torch.cat([tapped[i] for i in taps], dim=-1)[act.b, act.k])
            decision, continue_logits = decider(
                logits=pick(updated), iter_depth=depth,
                labels_shifted=None if a_labels_all is None else pick(a_labels_all[act.b, act.k]),
                iter_count_labels=None if a_iter_labels is None else pick(a_iter_labels[act.b, act.k]),
                **dec_kwargs)
            if self.training or labels is not None:
                decision = self._force_one_continuation(
                    decision, None if a_labels is None else pick(a_labels[act.b, act.k]), depth)

            # finished = invalid tokens, plus valid ones the decider stopped
            if all_valid:
                go = decision
            else:
                go = torch.zeros(act.n, dtype=torch.bool, device=device)
                go[v_act] = decision
            finished = ~go
            n_go = int(go.sum())                           # one host sync; the next ActiveSet needs one anyway
            iter_counts[act.b, act.s] += 1

            if labels_shifted is not None and loss_func._is_intra_iter_loss:
                loss_func.intra_iter_loss_func(
                    active_index=act.flat, active_valid=v_act, continue_logits=continue_logits,
                    iter_depth=depth,
                    active_iter_count_labels=None if a_iter_labels is None else a_iter_labels[act.b, act.k],
                    iter_decider_threshold=decider.threshold, model=self, **self._forward_kwargs(kwargs))

            if n_go == 0 and act.full and act.width == T:
                final_logits = updated.view(B, T, V)       # every token ends here: no scatter of the logits
            elif n_go == 0:
                final_logits.index_put_((act.b, act.s), updated)
            elif n_go < act.n:
                final_logits.index_put_((act.b[finished], act.s[finished]), updated[finished])

            if track_labels:
                prop = a_iter_labels[act.b, act.k]
                prop = torch.where(prop == -100, torch.zeros_like(prop), prop)
                merged = torch.zeros_like(full_iter_labels)
                merged[act.b, act.s] = prop
                full_iter_labels = torch.maximum(full_iter_labels, merged)

            if depth >= self.max_iter:
                break
            current = torch.zeros_like(current)
            current[act.b[go], act.s[go]] = True
            nxt = ActiveSet(current)
            if nxt.n == 0 and not self.uniform_passes:
                break
            carried = updated if n_go == act.n else updated[go]
            soft = topk_softmax_input_update(carried, embed_w, self.input_topk)
            block_embeds = nxt.pack_flat(soft)
            act = nxt

        loss = None
        if labels_shifted is not None:
            lk = self._forward_kwargs(kwargs)
            lk["iter_count_labels"] = full_iter_labels if full_iter_labels is not None else iter_count_labels
            lk["model"] = self
            if hasattr(self, "logger_callback"):
                lk["logger_callback"] = self.logger_callback
            loss = loss_func.final_loss_func(logits=final_logits, labels_shifted=labels_shifted,
                                             iter_count=iter_counts, training=self.training, **lk)
            if hasattr(self, "logger_callback"):
                n_items = kwargs.get("num_items_in_batch")
                with torch.no_grad():
                    if n_items is not None:
                        s = iter_counts[labels_shifted != -100].float().sum()
                        self.logger_callback.avg_iter_count += float(s / n_items)
                    else:
                        self.logger_callback.avg_iter_count = float(iter_counts.float().mean())

        return TaHCausalLMOutputWithPast(loss=loss, logits=final_logits,
                                         past_key_values=cache if use_cache else None,
                                         iter_count=iter_counts, iter_count_labels=full_iter_labels)

    # ---- persistence -------------------------------------------------------------------
    def save_pretrained(self, save_directory: str, **kwargs) -> None:
        """Write the reference checkpoint layout (reference ``tah_model.py:795-826``)::

            config.json, generation_config.json, model.safetensors   base weights, HF names
            lora/adapter_config.json, lora/adapter_model.safetensors  PEFT adapter names
            iter_decider.bin, tah_config.json
        """
        from tah_b200.utils.checkpoint import save_hf_checkpoint
        os.makedirs(save_directory, exist_ok=True)
        save_hf_checkpoint(self.simple_base_model, save_directory,
                           adapter_kwargs=self.tah_config.adapter_kwargs,
                           max_shard_bytes=kwargs.get("max_shard_bytes", 5 * 1024 ** 3))
        save_iter_decider(self.iter_decider, save_directory)
        save_config(self.tah_config, save_directory)

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str, *args, tah_config: Optional[TaHConfig] = None,
                        **kwargs) -> "TaHForCausalLM":
        """Load a checkpoint directory (or hub id, fetched with ``snapshot_download``).
        Recognised kwargs: ``torch_dtype``/``dtype``, ``device_map``/``device``; others
        that only select a HuggingFace attention backend are accepted and ignored."""
        from tah_b200.utils.checkpoint import load_hf_checkpoint
        path = pretrained_model_name_or_path
        if not os.path.isdir(path):
            from huggingface_hub import snapshot_download
            path = snapshot_download(path)
        cfg = resolve_config(path, tah_config)
        decider_path = None
        if "load_path" in (cfg.iter_decider_kwargs or {}):
            cfg.iter_decider_kwargs = dict(cfg.iter_decider_kwargs)
            decider_path = cfg.iter_decider_kwargs.pop("load_path")

        dtype = kwargs.get("torch_dtype", kwargs.get("dtype"))
        if isinstance(dtype, str):
            dtype = getattr(torch, dtype.replace("torch.", "")) if dtype != "auto" else None
        device = kwargs.get("device")
        dm = kwargs.get("device_map")
        if device is None and dm is not None:
            device = ("cuda" if torch.cuda.is_available() else "cpu") if dm == "auto" else (dm if isinstance(dm, (str, torch.device)) else None)
        spec = LoRASpec.from_adapter_kwargs(cfg.adapter_kwargs)
        base = load_hf_checkpoint(path, spec, dtype=dtype, device=device)
        model = cls(base, config=cfg)
        src = decider_path if decider_path is not None else (path if os.path.isfile(os.path.join(path, "iter_decider.bin")) else None)
        if src is not None:
            model.iter_decider = load_iter_decider(src, class_name=cfg.iter_decider, init_args=cfg.iter_decider_kwargs)
        model.iter_decider = model.iter_decider.to(device=model.device, dtype=model.dtype)
        model.eval_iter_decider = model._resolve_eval_iter_decider(cfg)
        if model.eval_iter_decider is not model.iter_decider:
            model.eval_iter_decider = model.eval_iter_decider.to(device=model.device, dtype=model.dtype)
        return model
