"""Benchmark loading for the evaluation driver.

A registry (``eval_configs/dataset_configs.json``) maps a benchmark name to where it lives (a
HuggingFace hub id or a local ``.jsonl``) and to its field names.  Every row is standardised to
``{id: "<dataset>_<original id>", _original_id, question, answer, _source_dataset, entry_point?,
_original_*}`` so that several benchmarks can be evaluated in one run (schema of reference
``tah/evaluate/datasets.py:91-104``).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Tuple

_CFG = os.path.join(os.path.dirname(os.path.abspath(__file__)), "eval_configs", "dataset_configs.json")


def load_registry(path: str = _CFG) -> Dict[str, dict]:
    with open(path, encoding="utf-8") as fh:
        return json.load(fh)


def _rows_from_source(cfg: dict) -> List[dict]:
    path = cfg["path"]
    if path.endswith(".jsonl") or path.endswith(".json"):
        if not os.path.exists(path):
            raise FileNotFoundError(f"local benchmark file not found: {path}")
        with open(path, encoding="utf-8") as fh:
            if path.endswith(".jsonl"):
                return [json.loads(line) for line in fh if line.strip()]
            return list(json.load(fh))
    from datasets import load_dataset
    kw = {}
    if cfg.get("version_tag"):
        kw["version_tag"] = cfg["version_tag"]
        kw["trust_remote_code"] = True
    ds = load_dataset(path, cfg.get("subset"), **kw) if cfg.get("subset") else load_dataset(path, **kw)
    split = cfg.get("split_name") or ("test" if "test" in ds else list(ds.keys())[0])
    return [dict(r) for r in ds[split]]


def _standardise(name: str, cfg: dict, rows: List[dict]) -> List[dict]:
    out = []
    flt = cfg.get("filter") or {}
    for i, row in enumerate(rows):
        if any(row.get(k) != v for k, v in flt.items()):
            continue
        orig = row.get(cfg["id_field"], i)
        q = row.get(cfg["question_field"], "")
        tmpl = cfg.get("prompt_template") or "{question}"
        item = {
            "id": f"{name}_{orig}",
            "_original_id": orig,
            "question": tmpl.format(question=q) if "{question}" in tmpl else str(q),
            "answer": row.get(cfg["answer_field"], ""),
            "_source_dataset": name,
        }
        ep_field = cfg.get("entry_point")
        if ep_field and ep_field in row:
            item["entry_point"] = row[ep_field]
        for k, v in row.items():
            item.setdefault(f"_original_{k}", v)
        out.append(item)
    return out


def load_combined_dataset(dataset_names, registry: Dict[str, dict] = None) -> Tuple[List[dict], dict]:
    """Load one or several registered benchmarks.  Returns ``(rows, field_mapping)`` where
    ``field_mapping`` names the standardised fields and carries ``answer_type``."""
    registry = registry or load_registry()
    if isinstance(dataset_names, str):
        dataset_names = [n.strip() for n in dataset_names.split(",") if n.strip()]
    rows: List[dict] = []
    answer_types = set()
    for name in dataset_names:
        if name not in registry:
            raise KeyError(f"unknown dataset {name!r}; registered: {sorted(registry)}")
        cfg = registry[name]
        rows.extend(_standardise(name, cfg, _rows_from_source(cfg)))
        answer_types.add(cfg.get("answer_type", "boxed"))
    if len(answer_types) > 1:
        raise ValueError(f"cannot mix answer types in one run: {sorted(answer_types)}")
    mapping = {"id_field": "id", "question_field": "question", "answer_field": "answer",
               "answer_type": answer_types.pop() if answer_types else "boxed"}
    return rows, mapping
