"""Minimal stand-in for the parts of ``peft`` that the reference TaH package imports.

The reference wraps its HuggingFace base model with ``peft.get_peft_model(model, LoraConfig(...))`` and
toggles the adapter per iteration with ``enable_adapter_layers`` / ``disable_adapter_layers``.  ``peft`` is
not installed on this image and cannot be fetched, so the benchmark's reference arm puts this directory on
``sys.path``: it implements exactly that surface with the same arithmetic PEFT's LoRA ``Linear`` performs
(``base(x) + lora_B(lora_A(dropout(x))) * (lora_alpha / r)``, two extra unfused ``nn.Linear`` calls) and the
same module / parameter names (``base_layer``, ``lora_A.default``, ``lora_B.default``).  It is used for
nothing else; the framework itself has its own LoRA.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Any, List, Optional, Union

import torch
from torch import nn

__version__ = "0.0-standin"


@dataclass
class LoraConfig:
    r: int = 8
    lora_alpha: int = 8
    lora_dropout: float = 0.0
    target_modules: Optional[Union[str, List[str]]] = None
    bias: str = "none"
    task_type: Optional[str] = None
    init_lora_weights: Any = True
    peft_type: str = "LORA"
    extra: dict = field(default_factory=dict)


class LoraLinear(nn.Module):
    def __init__(self, base: nn.Linear, cfg: LoraConfig):
        super().__init__()
        self.base_layer = base
        self.r = cfg.r
        self.scaling = cfg.lora_alpha / cfg.r
        self.lora_dropout = nn.ModuleDict({"default": nn.Dropout(cfg.lora_dropout) if cfg.lora_dropout > 0 else nn.Identity()})
        kw = dict(device=base.weight.device, dtype=base.weight.dtype)
        self.lora_A = nn.ModuleDict({"default": nn.Linear(base.in_features, cfg.r, bias=False, **kw)})
        self.lora_B = nn.ModuleDict({"default": nn.Linear(cfg.r, base.out_features, bias=False, **kw)})
        nn.init.kaiming_uniform_(self.lora_A["default"].weight, a=math.sqrt(5))
        nn.init.zeros_(self.lora_B["default"].weight)
        self.disable_adapters = False

    @property
    def weight(self):
        return self.base_layer.weight

    def forward(self, x):
        y = self.base_layer(x)
        if self.disable_adapters:
            return y
        a, b, d = self.lora_A["default"], self.lora_B["default"], self.lora_dropout["default"]
        return y + b(a(d(x.to(a.weight.dtype)))) * self.scaling


class LoraModel(nn.Module):
    """``peft_model.base_model``: owns the wrapped model as ``.model`` and the adapter switches."""

    def __init__(self, model: nn.Module, cfg: LoraConfig):
        super().__init__()
        self.model = model
        targets = cfg.target_modules
        skip = set()
        if targets == "all-linear":      # every nn.Linear except the output layer, as PEFT resolves it
            get_out = getattr(model, "get_output_embeddings", None)
            out = get_out() if get_out is not None else None
            skip = {id(out)} if out is not None else set()
        for name, mod in list(model.named_modules()):
            for child_name, child in list(mod.named_children()):
                if not isinstance(child, nn.Linear) or id(child) in skip:
                    continue
                if targets != "all-linear" and child_name not in (targets or []):
                    continue
                setattr(mod, child_name, LoraLinear(child, cfg))
        for n, p in self.named_parameters():
            p.requires_grad = "lora_" in n

    def forward(self, *a, **k):
        return self.model(*a, **k)

    def _set(self, disabled: bool):
        for m in self.modules():
            if isinstance(m, LoraLinear):
                m.disable_adapters = disabled

    def enable_adapter_layers(self):
        self._set(False)

    def disable_adapter_layers(self):
        self._set(True)


class PeftModel(nn.Module):
    def __init__(self, model: nn.Module, cfg: LoraConfig):
        super().__init__()
        self.peft_config = {"default": cfg}
        self.base_model = LoraModel(model, cfg)
        self.config = getattr(model, "config", None)

    def forward(self, *a, **k):
        return self.base_model(*a, **k)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            if name == "base_model":
                raise
            return getattr(self.base_model.model, name)

    @property
    def device(self):
        return next(self.parameters()).device

    def get_base_model(self):
        return self.base_model.model

    def save_pretrained(self, save_directory: str, **kwargs):
        from safetensors.torch import save_file
        os.makedirs(save_directory, exist_ok=True)
        sd = {"base_model.model." + k.replace(".default", ""): v.detach().cpu().contiguous()
              for k, v in self.base_model.model.state_dict().items() if "lora_" in k}
        save_file(sd, os.path.join(save_directory, "adapter_model.safetensors"))
        cfg = asdict(self.peft_config["default"])
        cfg.pop("extra", None)
        with open(os.path.join(save_directory, "adapter_config.json"), "w") as fh:
            json.dump(cfg, fh, indent=2)

    def load_adapter(self, model_id: str, adapter_name: str = "default", **kwargs):
        from safetensors.torch import load_file
        sd = load_file(os.path.join(model_id, "adapter_model.safetensors"))
        own = self.base_model.model.state_dict()
        for k, v in sd.items():
            k2 = k[len("base_model.model."):] if k.startswith("base_model.model.") else k
            k2 = k2.replace("lora_A.weight", "lora_A.default.weight").replace("lora_B.weight", "lora_B.default.weight")
            own[k2].copy_(v)


def get_peft_model(model: nn.Module, peft_config: LoraConfig, **kwargs) -> PeftModel:
    return PeftModel(model, peft_config)


class PeftMixedModel(PeftModel):
    """Name that ``transformers`` imports when it finds a ``peft`` module; not used by the reference."""
