#!/usr/bin/env python
"""TaH supervised fine-tuning entry point.

    python script/train/SFT_TaH.py --config script/recipes/qwen3_1.7_1gpu/sft_tah_step1.yaml
    torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 script/train/SFT_TaH.py --config <recipe>

YAML sections ``model`` / ``data`` / ``training`` as in the upstream recipes (reference
``script/train/SFT_TaH.py:175-243``): ``model`` keys that are ``TaHConfig`` fields configure the
wrapper, the rest (``name``, ``tah_model_path``, ``eos_token``, ``pad_token``, ``torch_dtype``...)
are consumed here; ``training`` feeds :class:`TaHTrainingArguments` plus ``freeze_component``,
``resume_from_ckpt`` and the wandb keys.  ``--synthetic N`` replaces tokenizer and data by random
tokens of a tiny model, for smoke runs without any downloaded asset.
"""
from __future__ import annotations

import argparse
import datetime
import os
import sys
from dataclasses import fields
from typing import Dict

import torch
import torch.distributed as dist
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from tah_b200 import TaHConfig, TaHForCausalLM  # noqa: E402
from tah_b200.model.iter_decider import load_iter_decider  # noqa: E402
from tah_b200.model.utils import compute_trainable_param_size_gb, freeze_components, set_all_seeds  # noqa: E402
from tah_b200.train import CustomTaHDataCollator, CustomTaHTrainer, LoggerCallback, TaHTrainingArguments  # noqa: E402
from tah_b200.utils.data_prepare import preprocess_dataset  # noqa: E402

set_all_seeds(420, verbose=False)
_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


class _Launcher:
    """Rank-aware print and the "main process first" ordering the data code expects."""

    def __init__(self):
        self.on = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank() if self.on else 0

    def print(self, *a, **k):
        if self.rank == 0:
            print(*a, **k, flush=True)

    def main_process_first(self):
        from contextlib import contextmanager

        @contextmanager
        def ctx():
            if self.on and self.rank != 0:
                dist.barrier()
            yield
            if self.on and self.rank == 0:
                dist.barrier()
        return ctx()


def _single_token_id(tokenizer, name: str, token: str) -> int:
    ids = tokenizer.encode(token, add_special_tokens=False)
    if len(ids) != 1 or tokenizer.convert_ids_to_tokens(ids[0]) != token:
        raise ValueError(f"{name} must be an existing single token: {token!r} -> {ids}")
    return ids[0]


def _configure_special_tokens(model, tokenizer, model_config: Dict) -> None:
    eos = model_config.get("eos_token") or tokenizer.eos_token
    pad = model_config.get("pad_token") or tokenizer.pad_token or eos
    eos_id, pad_id = _single_token_id(tokenizer, "eos_token", eos), _single_token_id(tokenizer, "pad_token", pad)
    tokenizer.eos_token, tokenizer.pad_token = eos, pad
    model.config.eos_token_id, model.config.pad_token_id = eos_id, pad_id     # saved into config.json


def _build_model_and_tokenizer(mc: Dict, launcher, device):
    from transformers import AutoTokenizer
    dtype = _DTYPES.get(str(mc.get("torch_dtype", "bfloat16")), torch.bfloat16)
    tokenizer = AutoTokenizer.from_pretrained(mc.get("name", mc.get("tah_model_path")),
                                              trust_remote_code=mc.get("trust_remote_code", True), padding_side="right")
    valid = {f.name for f in fields(TaHConfig)}
    cfg = TaHConfig(**{k: v for k, v in mc.items() if k in valid})
    if "tah_model_path" in mc:
        launcher.print(f"Resuming from TaH checkpoint: {mc['tah_model_path']}")
        model = TaHForCausalLM.from_pretrained(mc["tah_model_path"], tah_config=cfg, torch_dtype=dtype, device=device)
    else:
        from tah_b200.utils.checkpoint import load_hf_checkpoint
        from tah_b200.models.qwen3 import LoRASpec
        path = mc["name"]
        if not os.path.isdir(path):
            from huggingface_hub import snapshot_download
            path = snapshot_download(path)
        decider_path = None
        if "load_path" in (cfg.iter_decider_kwargs or {}):
            cfg.iter_decider_kwargs = dict(cfg.iter_decider_kwargs)
            decider_path = cfg.iter_decider_kwargs.pop("load_path")
        base = load_hf_checkpoint(path, LoRASpec.from_adapter_kwargs(cfg.adapter_kwargs), dtype=dtype, device=device)
        model = TaHForCausalLM(base, cfg)
        if decider_path:
            model.iter_decider = load_iter_decider(decider_path)
    model.iter_decider.to(device=device, dtype=dtype)
    _configure_special_tokens(model, tokenizer, mc)
    launcher.print(f"EOS: {tokenizer.eos_token!r} ({tokenizer.eos_token_id}); PAD: {tokenizer.pad_token!r} ({tokenizer.pad_token_id})")
    return model, tokenizer


def _synthetic(n: int, device, max_iter: int):
    """Tiny random model + random labelled data, for smoke runs."""
    from tah_b200.models import Qwen3ForCausalLM, preset
    cfg = preset("tiny", torch_dtype="bfloat16" if device.type == "cuda" else "float32")
    base = Qwen3ForCausalLM(cfg, device=device)
    tc = TaHConfig(max_iter=max_iter, iter_decider="IterLabelDecider", train_loss="NextTokenPredLoss",
                   adapter_kwargs=dict(r=8, lora_alpha=16, lora_dropout=0.0, target_modules="all-linear"),
                   input_updater_kwargs={"topk": 100})
    model = TaHForCausalLM(base, tc)
    g = torch.Generator().manual_seed(0)
    rows = []
    for _ in range(n):
        T = int(torch.randint(32, 96, (1,), generator=g))
        ids = torch.randint(0, cfg.vocab_size, (T,), generator=g).tolist()
        hard = (torch.rand(T, generator=g) < 0.06).long() + 1
        hard[5] = 2
        rows.append({"input_ids": ids, "attention_mask": [1] * T, "labels": [-100] * 4 + ids[4:],
                     "iter_count_labels": hard.tolist()})
    return model, rows


def _parallel_config(path):
    """Launch-topology file (``script/recipes/parallel_configs/zero{2,3}.yaml``; the reference's accelerate /
    DeepSpeed files, ``script/recipes/accelerate_configs/zero2.yaml:3-16``, play this role there).  Keys read:
    ``strategy`` (zero2 | zero3), ``tp_size`` (tensor-parallel group size, layers sharded over adjacent ranks),
    ``nvls`` (use NVLS multimem in the fused collectives)."""
    if not path:
        return {}
    with open(path, encoding="utf-8") as fh:
        pc = yaml.safe_load(fh) or {}
    if pc.get("nvls") is False:
        os.environ["TAH_B200_NVLS"] = "0"
    return pc


def main(config_path: str, synthetic: int = 0, max_steps: int = -1, parallel_config: str = None):
    if "RANK" in os.environ and not dist.is_initialized():
        local = int(os.environ.get("LOCAL_RANK", 0))
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
    launcher = _Launcher()
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    with open(config_path, encoding="utf-8") as fh:
        cfg = yaml.safe_load(fh)
    mc, dc, tc = cfg.get("model", {}), cfg.get("data", {}), dict(cfg.get("training", {}))
    # one timestamp for all ranks
    stamp = [datetime.datetime.now().strftime("%Y%m%d_%H%M%S")]
    if launcher.on:
        dist.broadcast_object_list(stamp, src=0)
    out_dir = os.path.join(dc.get("output_dir", "output"), f"{os.path.splitext(os.path.basename(config_path))[0]}_{stamp[0]}")
    if synthetic:
        model, train_rows = _synthetic(synthetic, device, int(mc.get("max_iter", 2) or 2))
        tokenizer, train_ds, eval_ds = None, train_rows, train_rows[: max(1, synthetic // 8)]
    else:
        model, tokenizer = _build_model_and_tokenizer(mc, launcher, device)
        train_ds, eval_ds = preprocess_dataset(tc, dc, mc, launcher)
    freeze_components(model, tc.pop("freeze_component", None) or [], launcher)
    launcher.print(f"Trainable parameters: {compute_trainable_param_size_gb(model):.3f} GB")
    resume = tc.pop("resume_from_ckpt", None)
    for k in ("wandb_project", "wandb_name", "wandb_entity"):
        v = tc.pop(k, None)
        if v and tc.get("report_to") == "wandb":
            os.environ[{"wandb_project": "WANDB_PROJECT", "wandb_name": "WANDB_NAME", "wandb_entity": "WANDB_ENTITY"}[k]] = str(v)
    pc = _parallel_config(parallel_config or tc.pop("parallel_config", None))
    if pc.get("strategy") and "strategy" not in tc:
        tc["strategy"] = pc["strategy"]
    if pc.get("tp_size") and "tp_size" not in tc:
        tc["tp_size"] = int(pc["tp_size"])
    args = TaHTrainingArguments.from_dict(dict(tc, output_dir=out_dir))
    if max_steps > 0:
        args.max_steps = max_steps
    if launcher.rank == 0:
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, "training_config.yaml"), "w") as fh:
            yaml.safe_dump(cfg, fh, sort_keys=False)
    collator = CustomTaHDataCollator(tokenizer, padding=True, pad_token_id=None if tokenizer else 0, padding_side="right")
    trainer = CustomTaHTrainer(model, args, train_ds, eval_ds, processing_class=tokenizer, data_collator=collator)
    model.logger_callback = LoggerCallback()
    trainer.insert_callback(0, model.logger_callback)
    trainer.train(resume_from_checkpoint=mc.get("tah_model_path") if resume else None)
    final = os.path.join(out_dir, "final_model")
    trainer.save_model(final)
    launcher.print(f"Saved final model to {final}")
    return trainer


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--synthetic", type=int, default=0, help="train a tiny random model on N random sequences")
    ap.add_argument("--max_steps", type=int, default=-1)
    ap.add_argument("--parallel_config", default=None,
                    help="launch topology YAML (script/recipes/parallel_configs/zero2.yaml or zero3.yaml)")
    a = ap.parse_args()
    main(a.config, a.synthetic, a.max_steps, a.parallel_config)
