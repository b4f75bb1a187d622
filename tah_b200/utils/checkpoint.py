"""Checkpoint I/O in the reference's on-disk layout.

::

    <dir>/config.json, generation_config.json      HuggingFace Qwen3 config of the base model
    <dir>/model.safetensors                        base weights under HuggingFace names
          (or model-0000i-of-0000n.safetensors + model.safetensors.index.json when sharded)
    <dir>/lora/adapter_config.json                 PEFT LoRA config
    <dir>/lora/adapter_model.safetensors           base_model.model.model.layers.{i}.<mod>.<proj>.lora_{A,B}.weight

(reference ``tah/model/tah_model.py:795-826``).  In memory the projections are
fused; :mod:`tah_b200.models.qwen3` translates names both ways.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch
from safetensors import safe_open
from safetensors.torch import save_file

from tah_b200.models.qwen3 import (LoRASpec, Qwen3Config, Qwen3ForCausalLM, export_hf_state_dict,
                                   import_hf_state_dict)


def _save_sharded(tensors: Dict[str, torch.Tensor], directory: str, max_shard_bytes: int) -> None:
    tensors = {k: v.detach().to("cpu").contiguous() for k, v in tensors.items()}
    total = sum(t.numel() * t.element_size() for t in tensors.values())
    if total <= max_shard_bytes:
        save_file(tensors, os.path.join(directory, "model.safetensors"), metadata={"format": "pt"})
        return
    shards, cur, cur_bytes = [], {}, 0
    for k, t in tensors.items():
        nb = t.numel() * t.element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = t
        cur_bytes += nb
    shards.append(cur)
    index = {"metadata": {"total_size": total}, "weight_map": {}}
    for i, shard in enumerate(shards, 1):
        name = f"model-{i:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, os.path.join(directory, name), metadata={"format": "pt"})
        for k in shard:
            index["weight_map"][k] = name
    with open(os.path.join(directory, "model.safetensors.index.json"), "w", encoding="utf-8") as fh:
        json.dump(index, fh, indent=2)


def _load_all(directory: str) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    index = os.path.join(directory, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index, encoding="utf-8") as fh:
            files = sorted(set(json.load(fh)["weight_map"].values()))
    elif os.path.exists(os.path.join(directory, "model.safetensors")):
        files = ["model.safetensors"]
    else:
        raise FileNotFoundError(f"no model.safetensors[.index.json] under {directory}")
    for name in files:
        with safe_open(os.path.join(directory, name), framework="pt", device="cpu") as fh:
            for k in fh.keys():
                out[k] = fh.get_tensor(k)
    return out


def adapter_config_dict(adapter_kwargs: Optional[dict], spec: LoRASpec, base_name: str = "") -> dict:
    kw = {k: v for k, v in (adapter_kwargs or {}).items() if k not in ("base_grad", "adapter_grad")}
    cfg = {
        "peft_type": "LORA", "task_type": kw.get("task_type"), "base_model_name_or_path": base_name,
        "r": spec.r, "lora_alpha": spec.lora_alpha, "lora_dropout": spec.lora_dropout,
        "target_modules": sorted(spec.targets), "bias": "none", "fan_in_fan_out": False,
        "inference_mode": False, "init_lora_weights": True, "modules_to_save": None,
        "use_rslora": False, "use_dora": False,
    }
    for k, v in kw.items():
        cfg.setdefault(k, v)
    return cfg


def save_hf_checkpoint(model: Qwen3ForCausalLM, directory: str, adapter_kwargs: Optional[dict] = None,
                       max_shard_bytes: int = 5 * 1024 ** 3) -> None:
    os.makedirs(directory, exist_ok=True)
    base, lora = export_hf_state_dict(model)
    model.config.save_pretrained(directory)
    gen = {k: getattr(model.config, k) for k in ("bos_token_id", "eos_token_id", "pad_token_id")
           if getattr(model.config, k) is not None}
    with open(os.path.join(directory, "generation_config.json"), "w", encoding="utf-8") as fh:
        json.dump(gen, fh, indent=2)
    _save_sharded(base, directory, max_shard_bytes)
    lora_dir = os.path.join(directory, "lora")
    os.makedirs(lora_dir, exist_ok=True)
    with open(os.path.join(lora_dir, "adapter_config.json"), "w", encoding="utf-8") as fh:
        json.dump(adapter_config_dict(adapter_kwargs, model.lora), fh, indent=2)
    save_file({k: v.detach().to("cpu").contiguous() for k, v in lora.items()},
              os.path.join(lora_dir, "adapter_model.safetensors"), metadata={"format": "pt"})


def load_hf_checkpoint(directory: str, lora: Optional[LoRASpec] = None, dtype=None, device=None) -> Qwen3ForCausalLM:
    cfg = Qwen3Config.from_pretrained(directory)
    if dtype is not None:
        cfg.torch_dtype = str(dtype).replace("torch.", "")
    model = Qwen3ForCausalLM(cfg, lora, dtype=cfg.dtype, device=device)
    lora_sd = None
    lora_file = os.path.join(directory, "lora", "adapter_model.safetensors")
    if os.path.exists(lora_file) and model.lora.r > 0:
        lora_sd = {}
        with safe_open(lora_file, framework="pt", device="cpu") as fh:
            for k in fh.keys():
                lora_sd[k] = fh.get_tensor(k)
    import_hf_state_dict(model, base=_load_all(directory), lora=lora_sd, strict=True)
    return model
