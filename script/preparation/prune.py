#!/usr/bin/env python
"""Layer pruning: drop the decoder layers whose removal hurts perplexity least.

"TaH" (as opposed to "TaH-plus") starts from a base model with one layer removed so that the total
parameter count including the LoRA adapter matches the un-iterated baseline.  For each layer the
loss on a few calibration texts is measured with that layer skipped; the ``num_prune`` layers with
the smallest increase are removed and the model is saved in HuggingFace layout
(procedure and flags of reference ``script/preparation/prune.py:65-85,87-231``: ``--model --dataset --text_field
--output --num_prune --batch_size --max_samples --max_length --device --dtype``).
"""
import argparse
import math
import os
import sys
from typing import List

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


@torch.no_grad()
def lm_loss(model, batches) -> float:
    tot, cnt = 0.0, 0
    for ids, mask in batches:
        logits = model(input_ids=ids, attention_mask=mask).float()
        tgt = ids[:, 1:].clone()
        tgt[mask[:, 1:] == 0] = -100
        loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]), tgt.reshape(-1),
                                                 ignore_index=-100, reduction="sum")
        tot += float(loss)
        cnt += int((tgt != -100).sum())
    return tot / max(cnt, 1)


def loss_without_layer(model, idx: int, batches) -> float:
    layers = model.model.layers
    kept = torch.nn.ModuleList([l for i, l in enumerate(layers) if i != idx])
    model.model.layers = kept
    try:
        return lm_loss(model, batches)
    finally:
        model.model.layers = layers


def prune_layers_inplace(model, drop: List[int]) -> None:
    keep = [l for i, l in enumerate(model.model.layers) if i not in set(drop)]
    for new_idx, layer in enumerate(keep):
        layer.self_attn.layer_idx = new_idx
    model.model.layers = torch.nn.ModuleList(keep)
    model.config.num_hidden_layers = len(keep)


def choose_layers(model, batches, num_prune: int):
    ref = lm_loss(model, batches)
    deltas = [(loss_without_layer(model, i, batches) - ref, i) for i in range(len(model.model.layers))]
    deltas.sort()
    return ref, deltas, sorted(i for _, i in deltas[:num_prune])


def read_calibration_texts(dataset: str, text_field: str = "real_text", max_samples: int = 16) -> List[str]:
    """Up to ``max_samples`` non-empty strings of column ``text_field``.  ``dataset`` is a dataset directory
    written by ``Dataset.save_to_disk`` (e.g. the labeller's output, whose ``real_text`` column is the default
    field), a hub dataset id, or a plain ``.txt`` file with one calibration text per line."""
    if os.path.isfile(dataset) and dataset.endswith(".txt"):
        with open(dataset, encoding="utf-8") as fh:
            texts = [l.strip() for l in fh if l.strip()][:max_samples]
    else:
        import datasets as hfds
        ds = hfds.load_from_disk(dataset) if os.path.isdir(dataset) else hfds.load_dataset(dataset)
        if isinstance(ds, hfds.DatasetDict):
            ds = ds[next(iter(ds))]
        if text_field not in ds.column_names:
            raise KeyError(f"column {text_field!r} not found; available: {ds.column_names}")
        texts = []
        for value in ds[text_field]:
            if isinstance(value, str) and value.strip():
                texts.append(value.strip())
                if len(texts) >= max_samples:
                    break
    if not texts:
        raise RuntimeError(f"no usable calibration text in {dataset!r} (field {text_field!r})")
    return texts


def _finite(x: float) -> float:
    return x if math.isfinite(x) else float("inf")


def main(argv=None):
    ap = argparse.ArgumentParser(description="Drop the decoder layers whose removal raises perplexity least")
    ap.add_argument("--model", default="Qwen/Qwen3-4B-Base", help="model directory (HF Qwen3 layout) or hub id")
    ap.add_argument("--dataset", "--calibration", dest="dataset", default=None,
                    help="calibration data: a saved HuggingFace dataset directory, a hub dataset id, or a .txt file")
    ap.add_argument("--text_field", default="real_text")
    ap.add_argument("--output", default="model/qwen3_4_base_pruned")
    ap.add_argument("--num_prune", type=int, default=1)
    ap.add_argument("--batch_size", type=int, default=4)
    ap.add_argument("--max_samples", type=int, default=16)
    ap.add_argument("--max_length", type=int, default=4096)
    ap.add_argument("--device", default="", help="e.g. cuda:0 or cpu (default: cuda:0 when available)")
    ap.add_argument("--dtype", default="auto", choices=["auto", "fp16", "bf16", "fp32"])
    a = ap.parse_args(argv)
    from transformers import AutoTokenizer
    from tah_b200.utils.checkpoint import load_hf_checkpoint, save_hf_checkpoint
    dev = torch.device(a.device) if a.device else torch.device("cuda:0" if torch.cuda.is_available() else "cpu")
    dtype = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}.get(
        a.dtype, torch.bfloat16 if dev.type == "cuda" else torch.float32)
    tok = AutoTokenizer.from_pretrained(a.model, use_fast=True)
    if tok.pad_token is None:
        tok.pad_token = tok.eos_token
    model = load_hf_checkpoint(a.model, dtype=dtype, device=dev).eval()
    if a.dataset:
        texts = read_calibration_texts(a.dataset, a.text_field, a.max_samples)
    else:
        texts = ["The quick brown fox jumps over the lazy dog. " * 20, "Let x be a real number such that x^2 = 2. " * 20]
    batches = []
    for i in range(0, len(texts), max(1, a.batch_size)):
        enc = tok(texts[i:i + a.batch_size], return_tensors="pt", padding=True, truncation=True, max_length=a.max_length).to(dev)
        batches.append((enc["input_ids"], enc["attention_mask"]))
    ref, deltas, drop = choose_layers(model, batches, min(a.num_prune, len(model.model.layers) - 1))
    ref_ppl = math.exp(ref)
    print(f"baseline loss {ref:.4f}, PPL {ref_ppl:.4f}")
    for d, i in sorted(deltas, key=lambda t: t[1]):
        ppl = _finite(math.exp(ref + d))
        print(f"layer {i} -> PPL {ppl:.4f}, dPPL {_finite(ppl - ref_ppl):.4f}")
    print(f"pruning layer indices (smallest dPPL first): {drop}")
    prune_layers_inplace(model, drop)
    after = lm_loss(model, batches)
    print(f"PPL after pruning: {math.exp(after):.4f} (d = {math.exp(after) - ref_ppl:.4f})")
    os.makedirs(a.output, exist_ok=True)
    save_hf_checkpoint(model, a.output)
    tok.save_pretrained(a.output)


if __name__ == "__main__":
    main()
