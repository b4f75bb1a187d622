"""SFT preprocessing: labeller output -> training examples.

Input rows (written by the hard-token labeller) carry ``real_token`` (token ids), ``mask`` (1 from
the start of the supervised span) and ``mismatch`` (1 where the small reference model mispredicted
the next token).  Output rows carry ``input_ids``, ``attention_mask`` (all ones), ``labels`` (-100
on unsupervised positions) and ``iter_count_labels``: 1 for easy supervised tokens, a random count
in ``[2, max_iter]`` for hard supervised tokens (or ``mismatch + 1`` when the labeller already wrote
counts), ``query_iter_count`` on prompt positions.  Rows without any supervised hard token are
dropped, so every training step runs the extra pass.  (Behaviour of reference
``tah/utils/data_prepare.py:36-202``.)
"""
from __future__ import annotations

from functools import partial
from typing import Dict, List, Optional

import numpy as np

_LABELLER_COLUMNS = ("data_id", "real_text", "real_token", "mask", "mismatch", "divergent", "entropy",
                     "cross_entropy", "ds_divergence", "problem_idx")


def _build_sft_example(input_ids: list, prompt_mask: list, mismatch_mask: Optional[list], max_iter: int,
                       max_length: Optional[int], truncate: bool, query_iter_count: int,
                       rng: Optional[np.random.Generator] = None) -> Optional[Dict]:
    if not any(prompt_mask):
        return None
    if max_length is not None and len(input_ids) > max_length:
        if not truncate:
            return None
        input_ids, prompt_mask = input_ids[:max_length], prompt_mask[:max_length]
        mismatch_mask = None if mismatch_mask is None else mismatch_mask[:max_length]
    sup = np.asarray(prompt_mask) != 0
    labels = np.asarray(input_ids, dtype=np.int64).copy()
    labels[~sup] = -100
    counts = np.ones(len(input_ids), dtype=np.int32)
    if max_iter > 1 and mismatch_mask is not None:
        mm = np.asarray(mismatch_mask)
        if (mm > 1).any():
            counts = (mm + 1).astype(np.int32)
        else:
            hard = np.nonzero((mm != 0) & sup)[0]
            if hard.size:
                draw = (rng.integers(2, max_iter + 1, hard.size) if rng is not None
                        else np.random.randint(2, max_iter + 1, hard.size))
                counts[hard] = draw
        counts[~sup] = query_iter_count
    return {"input_ids": list(input_ids), "attention_mask": [1] * len(input_ids), "labels": labels.tolist(),
            "iter_count_labels": counts.tolist()}


def _preprocess_for_sft_batch(examples: Dict, *, max_iter: int, max_length: Optional[int], truncate: bool,
                              query_iter_count: int) -> Dict:
    out: Dict[str, List] = {"input_ids": [], "attention_mask": [], "labels": []}
    if max_iter > 1:
        out["iter_count_labels"] = []
    mism = examples.get("mismatch")
    for i in range(len(examples["real_token"])):
        ex = _build_sft_example(examples["real_token"][i], examples["mask"][i], None if mism is None else mism[i],
                                max_iter, max_length, truncate, query_iter_count)
        if ex is None:
            continue
        for k in out:
            out[k].append(ex[k])
    return out


def _filter_keep(examples: Dict, *, max_length: Optional[int], truncate: bool) -> List[bool]:
    masks, tokens, mism = examples["mask"], examples["real_token"], examples.get("mismatch")
    keep = []
    for i in range(len(tokens)):
        end = max_length if (max_length and truncate) else len(tokens[i])
        m = masks[i][:end]
        ok = any(m)
        if ok and mism is not None:
            mm = mism[i][:end]
            ok = any(a == 1 and b == 1 for a, b in zip(m, mm))
        if max_length and not truncate:
            ok = ok and len(tokens[i]) <= max_length
        keep.append(bool(ok))
    return keep


class _SoloAccelerator:
    """Stand-in exposing the two members preprocessing needs when no launcher object is passed."""

    def print(self, *a, **k):
        print(*a, **k)

    def main_process_first(self):
        from contextlib import nullcontext
        return nullcontext()


def preprocess_dataset(training_config: Dict, data_config: Dict, model_config: Dict, accelerator=None,
                       num_proc: Optional[int] = None):
    """Load the labelled dataset(s) from disk, filter, map to SFT examples, split off an eval set."""
    from datasets import load_from_disk
    acc = accelerator or _SoloAccelerator()
    max_iter = model_config.get("max_iter", 1) or 1
    max_length = data_config.get("max_length")
    truncate = (data_config.get("max_length_action", "cutoff") or "cutoff").lower() != "filter"
    qic = int(data_config.get("query_iter_count", 1))
    train_ratio = data_config.get("train_data_ratio", 1.0)
    eval_ratio = data_config.get("eval_data_ratio", 0.05)
    with acc.main_process_first():
        train = load_from_disk(data_config["train_data_path"])
    if train_ratio != 1.0:
        train = train.select(range(int(len(train) * train_ratio)))
    evald = None
    if data_config.get("eval_data_path"):
        try:
            with acc.main_process_first():
                evald = load_from_disk(data_config["eval_data_path"])
        except Exception as exc:  # a missing eval set falls back to a split of train
            acc.print(f"Warning: could not load eval dataset {data_config['eval_data_path']}: {exc}")
    filt = partial(_filter_keep, max_length=max_length, truncate=truncate)
    prep = partial(_preprocess_for_sft_batch, max_iter=max_iter, max_length=max_length, truncate=truncate,
                   query_iter_count=qic)
    drop = lambda ds: [c for c in _LABELLER_COLUMNS if c in ds.column_names]
    with acc.main_process_first():
        train = train.filter(filt, batched=True, batch_size=1000, num_proc=num_proc)
        train = train.map(prep, batched=True, batch_size=2000, num_proc=num_proc, remove_columns=drop(train))
        if evald is not None:
            evald = evald.filter(filt, batched=True, batch_size=1000, num_proc=num_proc)
            evald = evald.map(prep, batched=True, batch_size=2000, num_proc=num_proc, remove_columns=drop(evald))
    if evald is None and eval_ratio and eval_ratio > 0 and len(train) > 1:
        split = train.train_test_split(test_size=eval_ratio, seed=42)
        train, evald = split["train"], split["test"]
    acc.print(f"Train dataset size: {len(train)}" + (f"; eval dataset size: {len(evald)}" if evald is not None else ""))
    return train, evald
