#!/usr/bin/env python
"""Hard-token labeller.

A small reference LM is run (prefill only) over every chat-formatted training sample; position
``i`` is *hard* (``mismatch[i] = 1``) iff the model's next-token prediction at ``i`` differs from
the real token ``i + 1``.  ``mask`` is 1 from the ``<think>`` token on (the supervised span).

Pipeline and flags follow reference ``script/preparation/label.py:497-529``:

* ``--dataset_path`` (``.jsonl`` or ``.json``), ``--index_range START END``, ``--random_num N`` (seed 42) select
  the samples; they are split into ``--num_gpu`` near-equal contiguous ranges, one worker process per GPU;
* ``--test_model_list`` names one or more labelling models; each is processed in turn;
* a worker drops samples longer than ``--max_input_length`` tokens (or truncates them with ``--is_cutoff
  True``), predicts with ``--temperature / --top_k / --top_p`` (arg-max at temperature 0), and writes a
  token-level table ``results_gpu_{g}_{model}`` with the columns ``predictions, small_token, data_id, mask,
  real_token, mismatch`` (+ ``entropy`` with ``--save_entropy``, ``cross_entropy`` with ``--save_ce``);
* the parent concatenates the tables, groups them by ``data_id`` into one row per sample (``data_id, real_text,
  real_token, mask, mismatch`` + the optional columns), prints the label statistics, saves the HuggingFace
  ``Dataset`` at ``--output_path``, removes the per-GPU tables and writes ``args.json``.

Workers are terminated, then killed, on SIGINT/SIGTERM or when they exceed the 24 h join timeout.

The labelling model is any checkpoint :func:`tah_b200.utils.checkpoint.load_hf_checkpoint` can read
(HuggingFace Qwen3 layout); it runs through this framework's backbone, not through transformers.
"""
import argparse
import json
import multiprocessing as mp
import os
import random
import shutil
import signal
import sys
from typing import Dict, List, Optional, Sequence, Tuple

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

QWEN3_THINK_TOKEN_ID = 151667
JOIN_TIMEOUT_S = 24 * 3600
_children: List[mp.Process] = []


# ---------------------------------------------------------------------------------------------
# sample selection
# ---------------------------------------------------------------------------------------------
def load_samples(path: str, index_range: Optional[Sequence[int]] = None, random_num: Optional[int] = None) -> List[dict]:
    """Records of a ``.jsonl`` (one object per line) or ``.json`` (list or single object) file, sliced to
    ``index_range = [start, end)`` and then sub-sampled to ``random_num`` records with seed 42."""
    with open(path, encoding="utf-8") as fh:
        if path.lower().endswith(".json"):
            blob = json.load(fh)
            data = blob if isinstance(blob, list) else [blob]
        else:
            data = [json.loads(line) for line in fh if line.strip()]
    if index_range:
        data = data[int(index_range[0]):int(index_range[1])]
    if random_num and 0 < random_num < len(data):
        data = random.Random(42).sample(data, random_num)
    return data


def gpu_ranges(n: int, k: int) -> List[Tuple[int, int]]:
    """``[0, n)`` cut into ``k`` contiguous ranges whose sizes differ by at most one."""
    base, extra = divmod(n, k)
    out, lo = [], 0
    for i in range(k):
        hi = lo + base + (1 if i < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


# ---------------------------------------------------------------------------------------------
# prompt formatting and per-token labels
# ---------------------------------------------------------------------------------------------
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
                with_stats: bool = False, top_k: int = 0, top_p: float = 1.0):
    """Prefill ``model`` (a plain LM: ``model(input_ids=..., attention_mask=...) -> logits``) and return
    per-sample (predictions, entropy?, cross-entropy?) lists over the valid positions."""
    from tah_b200.model.utils import sample_next_token
    with torch.no_grad():
        logits = model(input_ids=input_ids, attention_mask=attention_mask).float()
    outs = []
    for b in range(input_ids.shape[0]):
        n = int(attention_mask[b].sum())
        lg = logits[b, :n]
        pred = sample_next_token(lg, temperature=max(temperature, 1e-6), top_p=top_p, top_k=max(top_k, 0),
                                 do_sample=temperature > 0)
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


def token_table(rows: List[dict], save_entropy: bool, save_ce: bool) -> Dict[str, list]:
    """Per-sample results -> the token-level table a worker stores: one entry per token, ``small_token`` = the
    token's index inside its sample, ``data_id`` = the sample's index in the selected dataset."""
    cols: Dict[str, list] = {k: [] for k in ("predictions", "small_token", "data_id", "mask", "real_token", "mismatch")}
    if save_entropy:
        cols["entropy"] = []
    if save_ce:
        cols["cross_entropy"] = []
    for r in rows:
        n = len(r["real_token"])
        cols["predictions"] += r["predictions"]
        cols["small_token"] += list(range(n))
        cols["data_id"] += [r["data_id"]] * n
        cols["mask"] += r["mask"]
        cols["real_token"] += r["real_token"]
        cols["mismatch"] += r["mismatch"]
        if save_entropy:
            cols["entropy"] += r["entropy"]
        if save_ce:
            cols["cross_entropy"] += r["cross_entropy"]
    return cols


def samples_from_token_table(table, decode) -> List[dict]:
    """Group a token-level table (mapping of equal-length columns) by ``data_id`` into one record per
    sample, tokens in ``small_token`` order; ``decode(list[int]) -> str`` rebuilds ``real_text``."""
    order = sorted(range(len(table["data_id"])), key=lambda i: (table["data_id"][i], table["small_token"][i]))
    optional = [c for c in ("entropy", "cross_entropy") if c in table]
    out, cur = [], None
    for i in order:
        did = table["data_id"][i]
        if cur is None or cur["data_id"] != did:
            cur = {"data_id": did, "real_text": "", "real_token": [], "mask": [], "mismatch": []}
            for c in optional:
                cur[c] = []
            out.append(cur)
        cur["real_token"].append(table["real_token"][i])
        cur["mask"].append(table["mask"][i])
        cur["mismatch"].append(table["mismatch"][i])
        for c in optional:
            cur[c].append(table[c][i])
    for rec in out:
        rec["real_text"] = decode(rec["real_token"])
    return out


def label_statistics(samples: List[dict]) -> dict:
    tokens = sum(len(s["real_token"]) for s in samples)
    mism = sum(sum(s["mismatch"]) for s in samples)
    asst = sum(sum(s["mask"]) for s in samples)
    asst_m = sum(sum(1 for m, h in zip(s["mask"], s["mismatch"]) if m and h) for s in samples)
    return {"samples": len(samples), "tokens": tokens, "mismatch": mism, "assistant_tokens": asst,
            "assistant_mismatch": asst_m}


# ---------------------------------------------------------------------------------------------
# workers
# ---------------------------------------------------------------------------------------------
def _shard_dir(output_path: str, gpu: int, model_name: str) -> str:
    return os.path.join(output_path, f"results_gpu_{gpu}_{model_name.rstrip('/').split('/')[-1]}")


def _process_single_gpu(args, device_id: int, data_range: Tuple[int, int], model_name: str) -> None:
    from datasets import Dataset
    from transformers import AutoTokenizer
    from tah_b200.utils.checkpoint import load_hf_checkpoint
    lo, hi = data_range
    dev = torch.device("cuda", device_id) if torch.cuda.is_available() else torch.device("cpu")
    tok = AutoTokenizer.from_pretrained(model_name, padding_side="right")
    if tok.pad_token_id is None:
        tok.pad_token = tok.eos_token
    try:
        model = load_hf_checkpoint(model_name, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32,
                                   device=dev).eval()
    except Exception as exc:
        print(f"[gpu {device_id}] cannot load {model_name}: {exc}")
        return
    samples = load_samples(args.dataset_path, args.index_range, args.random_num)[lo:hi]
    stats = bool(args.save_entropy or args.save_ce)
    rows = []
    bs = max(1, int(args.batch_size))
    for s in range(0, len(samples), bs):
        batch = []
        for j, x in enumerate(samples[s:s + bs]):
            text = _format_prompt(x, tok)
            if not text:
                continue
            ids = tok(text, return_tensors="pt").input_ids[0]
            if ids.numel() > args.max_input_length:
                if not args.is_cutoff:
                    continue
                ids = ids[:args.max_input_length]
            batch.append((lo + s + j, ids))
        if not batch:
            continue
        width = max(ids.numel() for _, ids in batch)
        input_ids = torch.full((len(batch), width), tok.pad_token_id, dtype=torch.long)
        attn = torch.zeros(len(batch), width, dtype=torch.long)
        for b, (_, ids) in enumerate(batch):
            input_ids[b, :ids.numel()] = ids
            attn[b, :ids.numel()] = 1
        res = label_batch(model, input_ids.to(dev), attn.to(dev), args.temperature, stats, args.top_k, args.top_p)
        for (data_id, ids), r in zip(batch, res):
            real = ids.cpu()
            row = {"data_id": data_id, "real_token": real.tolist(), "predictions": r["pred"].tolist(),
                   "mask": _categorize_masks(real.tolist()), "mismatch": _calculate_mismatch(r["pred"], real).tolist()}
            if args.save_entropy:
                row["entropy"] = r["entropy"].tolist()
            if args.save_ce:
                row["cross_entropy"] = r["cross_entropy"].tolist()
            rows.append(row)
    if not rows:
        print(f"[gpu {device_id}] no valid samples")
        return
    Dataset.from_dict(token_table(rows, args.save_entropy, args.save_ce)).save_to_disk(
        _shard_dir(args.output_path, device_id, model_name))


def _merge_gpu_results(args, model_name: str):
    from datasets import Dataset, concatenate_datasets, load_from_disk
    from transformers import AutoTokenizer
    dirs = [d for d in (_shard_dir(args.output_path, g, model_name) for g in range(args.num_gpu)) if os.path.isdir(d)]
    if not dirs:
        print(f"no labelled shard was produced for {model_name}")
        return None
    merged = concatenate_datasets([load_from_disk(d) for d in dirs])
    tok = AutoTokenizer.from_pretrained(model_name)
    samples = samples_from_token_table({c: merged[c] for c in merged.column_names}, tok.decode)
    st = label_statistics(samples)
    print("=== Label statistics ===")
    print(f"  samples: {st['samples']:,}")
    print(f"  tokens: {st['tokens']:,}  (mismatch {st['mismatch']:,}, {100.0 * st['mismatch'] / max(1, st['tokens']):.2f}%)")
    print(f"  assistant tokens: {st['assistant_tokens']:,}  (mismatch {st['assistant_mismatch']:,}, "
          f"{100.0 * st['assistant_mismatch'] / max(1, st['assistant_tokens']):.2f}%)")
    ds = Dataset.from_list(samples)
    ds.save_to_disk(args.output_path)
    for d in dirs:
        shutil.rmtree(d, ignore_errors=True)
    return ds


def _stop(p: mp.Process, soft: int = 30, hard: int = 60) -> None:
    if not p.is_alive():
        return
    p.terminate()
    p.join(timeout=soft)
    if p.is_alive():
        p.kill()
        p.join(timeout=hard)


def _terminate_children(*_):
    for p in _children:
        _stop(p, soft=10, hard=10)
    sys.exit(1)


def _process_dataset_multi_gpu(args) -> None:
    os.makedirs(args.output_path, exist_ok=True)
    total = len(load_samples(args.dataset_path, args.index_range, args.random_num))
    ranges = gpu_ranges(total, args.num_gpu)
    print(f"{total} samples; per-GPU ranges {ranges}")
    ctx = mp.get_context("spawn")
    for model_name in args.test_model_list:
        _children.clear()
        for g in range(args.num_gpu):
            p = ctx.Process(target=_process_single_gpu, args=(args, g, ranges[g], model_name))
            p.start()
            _children.append(p)
        for g, p in enumerate(_children):
            p.join(timeout=JOIN_TIMEOUT_S)
            if p.is_alive():
                print(f"[gpu {g}] timed out, terminating")
                _stop(p)
            elif p.exitcode != 0:
                print(f"[gpu {g}] exited with code {p.exitcode}")
        _children.clear()
        _merge_gpu_results(args, model_name)


def _bool(v) -> bool:
    return str(v).lower() in ("1", "true", "yes", "y")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Multi-GPU prefill of a small LM -> hard-token (mismatch) labels")
    ap.add_argument("--dataset_path", "--input", dest="dataset_path", required=True, help=".jsonl or .json of chat samples")
    ap.add_argument("--num_gpu", "--num_gpus", dest="num_gpu", type=int, default=4)
    ap.add_argument("--test_model_list", "--model", dest="test_model_list", nargs="+", required=True,
                    help="labelling model(s): HF Qwen3 checkpoint directories or hub ids")
    ap.add_argument("--output_path", "--output", dest="output_path", required=True)
    ap.add_argument("--max_input_length", type=int, default=32768)
    ap.add_argument("--is_cutoff", type=_bool, default=False, help="True: truncate over-long samples; False: drop them")
    ap.add_argument("--index_range", nargs=2, type=int, default=None, help="[start, end) slice of the dataset")
    ap.add_argument("--random_num", type=int, default=None, help="sub-sample N records (seed 42)")
    ap.add_argument("--top_k", type=int, default=-1)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top_p", type=float, default=1.0)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--save_entropy", action="store_true", help="store the per-token softmax entropy")
    ap.add_argument("--save_ce", action="store_true", help="store the per-token cross-entropy of the next real token")
    ap.add_argument("--stats", action="store_true", help="shorthand for --save_entropy --save_ce")
    return ap


def main(argv=None):
    args = build_parser().parse_args(argv)
    if args.stats:
        args.save_entropy = args.save_ce = True
    signal.signal(signal.SIGINT, _terminate_children)
    signal.signal(signal.SIGTERM, _terminate_children)
    try:
        _process_dataset_multi_gpu(args)
        with open(os.path.join(args.output_path, "args.json"), "w", encoding="utf-8") as fh:
            json.dump(vars(args), fh, indent=2)
        print("All processing complete.")
    except Exception:
        for p in _children:
            _stop(p)
        raise
    finally:
        _children.clear()


if __name__ == "__main__":
    main()
