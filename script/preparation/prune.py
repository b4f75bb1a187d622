#!/usr/bin/env python
"""Layer pruning: drop the decoder layers whose removal hurts perplexity least.

"TaH" (as opposed to "TaH-plus") starts from a base model with one layer removed so that the total
parameter count including the LoRA adapter matches the un-iterated baseline.  For each layer the
loss on a few calibration texts is measured with that layer skipped; the ``num_prune`` layers with
the smallest increase are removed and the model is saved in HuggingFace layout
(procedure of reference ``script/preparation/prune.py:87-143``).
"""
import argparse
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


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--num_prune", type=int, default=1)
    ap.add_argument("--calibration", default=None, help=".txt file, one calibration text per line (at most 16 used)")
    ap.add_argument("--max_length", type=int, default=1024)
    a = ap.parse_args(argv)
    from transformers import AutoTokenizer
    from tah_b200.utils.checkpoint import load_hf_checkpoint, save_hf_checkpoint
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    tok = AutoTokenizer.from_pretrained(a.model)
    model = load_hf_checkpoint(a.model, dtype=torch.bfloat16 if dev == "cuda" else torch.float32, device=dev).eval()
    if a.calibration:
        with open(a.calibration, encoding="utf-8") as fh:
            texts = [l.strip() for l in fh if l.strip()][:16]
    else:
        texts = ["The quick brown fox jumps over the lazy dog. " * 20, "Let x be a real number such that x^2 = 2. " * 20]
    enc = tok(texts, return_tensors="pt", padding=True, truncation=True, max_length=a.max_length).to(dev)
    batches = [(enc["input_ids"][i:i + 4], enc["attention_mask"][i:i + 4]) for i in range(0, len(texts), 4)]
    ref, deltas, drop = choose_layers(model, batches, a.num_prune)
    print(f"reference loss {ref:.4f}; least harmful layers: {[(i, round(d, 4)) for d, i in deltas[:5]]}; dropping {drop}")
    prune_layers_inplace(model, drop)
    save_hf_checkpoint(model, a.output)
    tok.save_pretrained(a.output)


if __name__ == "__main__":
    main()
