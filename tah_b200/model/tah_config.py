"""TaHConfig: the persistent knobs of a Think-at-Hard model.

Field names and defaults follow the reference dataclass (reference
``tah/model/tah_config.py:20-51``) so that a ``tah_config.json`` written by
either code base loads in the other.  This module also owns the JSON codec for
``torch.dtype`` / ``type`` values (reference ``tah/model/tah_model.py:202-233``)
and the checkpoint-vs-override merge rule (``tah_model.py:263-294``).
"""
from __future__ import annotations

import importlib
import json
import logging
import os
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Dict, Optional

import torch

log = logging.getLogger(__name__)


@dataclass
class TaHConfig:
    embedding_key: str = "model.embed_tokens"
    max_iter: Optional[int] = None
    iter_decider: Optional[str] = None
    iter_decider_kwargs: Dict[str, Any] = field(default_factory=dict)
    eval_iter_decider: Optional[str] = None
    eval_iter_decider_kwargs: Dict[str, Any] = field(default_factory=dict)
    # only "topk" is read
    input_updater_kwargs: Dict[str, Any] = field(default_factory=dict)
    adapter: str = "lora"
    # LoRA settings (r, lora_alpha, lora_dropout, target_modules, ...) plus the
    # two TaH-only switches base_grad / adapter_grad.
    adapter_kwargs: Dict[str, Any] = field(default_factory=dict)
    train_loss: Optional[str] = None
    train_loss_kwargs: Dict[str, Any] = field(default_factory=dict)
    eval_loss: Optional[str] = None
    eval_loss_kwargs: Dict[str, Any] = field(default_factory=dict)


_DTYPES = {str(d): d for d in (torch.float32, torch.float16, torch.bfloat16)}


def encode_config(obj):
    """Make a config tree JSON-safe: dtypes and classes become tagged dicts."""
    if isinstance(obj, dict):
        return {k: encode_config(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [encode_config(v) for v in obj]
    if isinstance(obj, torch.dtype):
        return {"__dtype__": True, "__str__": str(obj)}
    if isinstance(obj, type):
        return {"__type__": True, "__module__": obj.__module__, "__name__": obj.__name__}
    return obj


def decode_config(obj):
    """Inverse of :func:`encode_config`.  Unknown dtype strings become fp32."""
    if isinstance(obj, list):
        return [decode_config(v) for v in obj]
    if not isinstance(obj, dict):
        return obj
    if obj.get("__dtype__") is True:
        return _DTYPES.get(obj.get("__str__"), torch.float32)
    if obj.get("__type__") is True:
        return getattr(importlib.import_module(obj["__module__"]), obj["__name__"])
    return {k: decode_config(v) for k, v in obj.items()}


def load_saved_config(checkpoint_dir: str) -> Optional[TaHConfig]:
    path = os.path.join(checkpoint_dir, "tah_config.json")
    if not os.path.exists(path):
        return None
    with open(path, encoding="utf-8") as fh:
        raw = decode_config(json.load(fh))
    known = {f.name for f in fields(TaHConfig)}
    return TaHConfig(**{k: v for k, v in raw.items() if k in known})


def resolve_config(checkpoint_dir: str, override: Optional[TaHConfig]) -> TaHConfig:
    """Saved JSON first; non-None, non-``{}`` override fields win; else defaults."""
    saved = load_saved_config(checkpoint_dir)
    if saved is not None and override is not None:
        merged = asdict(saved)
        for key, val in asdict(override).items():
            if val is not None and val != {}:
                merged[key] = val
        return TaHConfig(**merged)
    if override is not None:
        return override
    if saved is not None:
        return saved
    log.warning("no tah_config.json under %s and no tah_config passed: using defaults", checkpoint_dir)
    return TaHConfig()


def save_config(cfg: TaHConfig, directory: str) -> None:
    with open(os.path.join(directory, "tah_config.json"), "w", encoding="utf-8") as fh:
        json.dump(encode_config(asdict(cfg)), fh, indent=2, ensure_ascii=False)
