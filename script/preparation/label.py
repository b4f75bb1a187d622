#!/usr/bin/env python
"""Hard-token labeller.

A small reference LM is run (prefill only) over every chat-formatted training sample; position
``i`` is *hard* (``mismatch[i] = 1``) iff the model's next-token prediction at ``i`` differs from
the real token ``i + 1``.  ``mask`` is 1 from the ``<think>`` token on (the supervised span).  The
dataset is split contiguously over the GPUs, one worker process per GPU; each worker writes its
shard to disk, and the parent merges the shards into one HuggingFace ``Dataset`` with the columns
``data_id, real_text, real_token, mask, mismatch`` (+ ``entropy``, ``cross_entropy`` on request)
(pipeline of reference ``script/preparation/label.py:228-483``).  Workers are terminated, then
killed, on SIGINT/SIGTERM or when they exceed the join timeout.

The labelling model is any checkpoint :func:`tah_b200.utils.checkpoint.load_hf_checkpoint` can read
(HuggingFace Qwen3 layout); it runs through this framework's backbone, not through transformers.
"""
import argparse
import json
import multiprocessing as mp
import os
import signal
import sys
from typing import List, Optional, Tuple

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

QWEN3_THINK_TOKEN_ID = 151667
JOIN_TIMEOUT_S = 24 * 3600
_children: List[mp.Process] = []


def _split_reasoning(conversations):
    user = asst = None
    for c in conversations:
        if c.get("from") in ("human", "user"):
            user = c["value"]
        elif c.get("from") in ("gpt", "assistant"):
            asst = c["value"]
    if not user or not asst or "<think>" not in asst or "</think>" not in asst:
        return None, None, None
    a, b = asst.find("<think>") + len("<think>"), asst.find("</think>")
    return user, asst[a:b].strip(), asst[b + len("</think>"):].strip()


def _format_prompt(sample: dict, tokenizer) -> Optional[str]:
    """Accepts ``{"conversations": [...], "system"?}`` or ``{"problem"|"question", "output"|"solution"|
    "generation"|"answer"}`` records."""
    if "conversations" in sample:
        user, reasoning, response = _split_reasoning(sample["conversations"])
        if not user or response is None:
            return None
        content = f"{reasoning}\n</think>\n\n{response}" if reasoning else response
        msgs = ([{"role": "system", "content": sample["system"]}] if sample.get("system") else [])
        msgs += [{"role": "user", "content": user}, {"role": "assistant", "content": content}]
        return tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=False, enable_thinking=True)
    q = sample.get("problem") or sample.get("question") or ""
    a = sample.get("output") or sample.get("solution") or sample.get("generation") or sample.get("answer") or ""
    if not q or not a:
        return None
    return tokenizer.apply_chat_template([{"role": "user", "content": q}, {"role": "assistant", "content": a}],
                                         tokenize=False, add_generation_prompt=False, enable_thinking=False)


def _categorize_masks(ids: List[int], think_id: int = QWEN3_THINK_TOKEN_ID) -> List[int]:
    out, on = [], 0
    for t in ids:
        if t == think_id:
            on = 1
        out.append(on)
    return out


def _calculate_mismatch(predictions: torch.Tensor, real_tokens: torch.Tensor) -> torch.Tensor:
    """Per sample: ``mismatch[i] = pred[i] != real[i + 1]``; the last position has no target and stays 0."""
    mm = torch.zeros_like(real_tokens, dtype=torch.int32)
    if real_tokens.numel() > 1:
        mm[:-1] = (predictions[:-1] != real_tokens[1:]).int()
    return mm


def label_batch(model, input_ids: torch.Tensor, attention_mask: torch.Tensor, temperature: float = 0.0,
                with_stats: bool = False):
    """Prefill ``model`` (a plain LM: ``model(input_ids=..., attention_mask=...) -> logits``) and return
    per-sample (predictions, entropy?, cross-entropy?) lists over the valid positions."""
    from tah_b200.model.utils import sample_next_token
    with torch.no_grad():
        logits = model(input_ids=input_ids, attention_mask=attention_mask).float()
    outs = []
    for b in range(input_ids.shape[0]):
        n = int(attention_mask[b].sum())
        lg = logits[b, :n]
        pred = sample_next_token(lg, temperature=max(temperature, 1e-6), do_sample=temperature > 0)
        rec = {"pred": pred.cpu()}
        if with_stats:
            lp = torch.log_softmax(lg, -1)
            rec["entropy"] = (-(lp.exp() * lp).sum(-1)).cpu()
            tgt = input_ids[b, 1:n]
            ce = torch.zeros(n)
            ce[:-1] = -lp[:-1].gather(1, tgt[:, None]).squeeze(1).cpu()
            rec["cross_entropy"] = ce
        outs.append(rec)
    return outs


def _process_single_gpu(args, device_id: int, lo: int, hi: int) -> None:
    from datasets import Dataset
    from transformers import AutoTokenizer
    from tah_b200.utils.checkpoint import load_hf_checkpoint
    dev = torch.device("cuda", device_id) if torch.cuda.is_available() else torch.device("cpu")
    tok = AutoTokenizer.from_pretrained(args.model, padding_side="right")
    try:
        model = load_hf_checkpoint(args.model, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, device=dev).eval()
    except Exception as exc:
        print(f"[gpu {device_id}] cannot load {args.model}: {exc}")
        return
    with open(args.input, encoding="utf-8") as fh:
        samples = [json.loads(l) for i, l in enumerate(fh) if lo <= i < hi]
    rows = []
    for s in range(0, len(samples), args.batch_size):
        chunk = samples[s:s + args.batch_size]
        texts = [(lo + s + j, _format_prompt(x, tok)) for j, x in enumerate(chunk)]
        texts = [(i, t) for i, t in texts if t]
        if not texts:
            continue
        enc = tok([t for _, t in texts], return_tensors="pt", padding=True, truncation=True,
                  max_length=args.max_input_length).to(dev)
        res = label_batch(model, enc["input_ids"], enc["attention_mask"], args.temperature, args.stats)
        for (data_id, text), r, ids, am in zip(texts, res, enc["input_ids"], enc["attention_mask"]):
            n = int(am.sum())
            real = ids[:n].cpu()
            row = {"data_id": data_id, "real_text": text, "real_token": real.tolist(),
                   "mask": _categorize_masks(real.tolist()), "mismatch": _calculate_mismatch(r["pred"], real).tolist()}
            if args.stats:
                row["entropy"], row["cross_entropy"] = r["entropy"].tolist(), r["cross_entropy"].tolist()
            rows.append(row)
    Dataset.from_list(rows).save_to_disk(os.path.join(args.output, f"_shard_gpu{device_id}"))


def _merge_gpu_results(output: str, n: int):
    from datasets import concatenate_datasets, load_from_disk
    parts = [load_from_disk(os.path.join(output, f"_shard_gpu{i}")) for i in range(n)
             if os.path.isdir(os.path.join(output, f"_shard_gpu{i}"))]
    if not parts:
        raise RuntimeError("no labelled shard was produced")
    ds = concatenate_datasets(parts).sort("data_id")
    hard = sum(sum(m and h for m, h in zip(r["mask"], r["mismatch"])) for r in ds)
    sup = sum(sum(r["mask"]) for r in ds)
    print(f"{len(ds)} samples, {sup} supervised tokens, {hard} hard ({100.0 * hard / max(1, sup):.2f} %)")
    ds.save_to_disk(os.path.join(output, "labelled"))
    return ds


def _terminate_children(*_):
    for p in _children:
        if p.is_alive():
            p.terminate()
    for p in _children:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
    sys.exit(1)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True, help=".jsonl of chat samples")
    ap.add_argument("--output", required=True)
    ap.add_argument("--model", required=True, help="labelling model (HF Qwen3 checkpoint dir)")
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--max_input_length", type=int, default=10000)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--num_gpus", type=int, default=max(1, torch.cuda.device_count()))
    ap.add_argument("--stats", action="store_true", help="also record entropy and cross-entropy")
    args = ap.parse_args(argv)
    os.makedirs(args.output, exist_ok=True)
    with open(args.input, encoding="utf-8") as fh:
        total = sum(1 for _ in fh)
    per = (total + args.num_gpus - 1) // args.num_gpus
    signal.signal(signal.SIGINT, _terminate_children)
    signal.signal(signal.SIGTERM, _terminate_children)
    ctx = mp.get_context("spawn")
    for g in range(args.num_gpus):
        p = ctx.Process(target=_process_single_gpu, args=(args, g, g * per, min(total, (g + 1) * per)))
        p.start()
        _children.append(p)
    for p in _children:
        p.join(timeout=JOIN_TIMEOUT_S)
        if p.is_alive():
            p.terminate()
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    _merge_gpu_results(args.output, args.num_gpus)


if __name__ == "__main__":
    main()
