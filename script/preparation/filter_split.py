#!/usr/bin/env python
"""OpenR1-Math parquet -> train/eval ``.jsonl`` of ``{"question", "generation", "num_tokens"}``.

Per problem the shortest *verified* generation is kept (``correctness_math_verify`` flags, falling
back to ``correctness_llama``), samples of ``MAX_OUTPUT_TOKENS`` or more tokens are dropped, and the
result is split 99 / 1 with seed 42 (behaviour of reference ``script/preparation/filter_split.py``).
"""
import argparse
import glob
import json
import os
import random
from multiprocessing import Pool

MAX_OUTPUT_TOKENS = 8192
TRAIN_FRACTION = 0.99
SEED = 42
_TOKENIZER = None


def _init(tokenizer_name):
    global _TOKENIZER
    if tokenizer_name:
        from transformers import AutoTokenizer
        _TOKENIZER = AutoTokenizer.from_pretrained(tokenizer_name)


def _n_tokens(text: str) -> int:
    return len(_TOKENIZER.encode(text)) if _TOKENIZER is not None else len(text.split())


def process_row(row: dict):
    gens = row.get("generations") or []
    flags = row.get("correctness_math_verify")
    if flags is None or not any(flags):
        flags = row.get("correctness_llama")
    if flags is None:
        return None
    good = [g for g, ok in zip(gens, flags) if ok and g]
    if not good:
        return None
    best = min(good, key=len)
    n = _n_tokens(best)
    if n >= MAX_OUTPUT_TOKENS:
        return None
    return {"question": row.get("problem", ""), "generation": best, "num_tokens": n}


def process_data(input_glob: str, out_dir: str, tokenizer_name=None, workers: int = 8):
    import pandas as pd
    rows = []
    for path in sorted(glob.glob(input_glob, recursive=True)):
        rows.extend(pd.read_parquet(path).to_dict("records"))
    with Pool(workers, initializer=_init, initargs=(tokenizer_name,)) as pool:
        kept = [r for r in pool.imap(process_row, rows, chunksize=256) if r is not None]
    random.Random(SEED).shuffle(kept)
    cut = int(len(kept) * TRAIN_FRACTION)
    os.makedirs(out_dir, exist_ok=True)
    for name, part in (("train", kept[:cut]), ("eval", kept[cut:])):
        with open(os.path.join(out_dir, f"{name}.jsonl"), "w", encoding="utf-8") as fh:
            for r in part:
                fh.write(json.dumps(r, ensure_ascii=False) + "\n")
    print(f"kept {len(kept)} of {len(rows)} rows: {cut} train / {len(kept) - cut} eval")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", default="data/raw/openr1_math/**/*.parquet")
    ap.add_argument("--out", default="data/initial_data/openr1_math")
    ap.add_argument("--tokenizer", default="Qwen/Qwen3-1.7B-Base")
    ap.add_argument("--workers", type=int, default=8)
    a = ap.parse_args()
    process_data(a.input, a.out, a.tokenizer, a.workers)
