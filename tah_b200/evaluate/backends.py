"""Inference backends for the evaluation driver.

Contract (reference ``tah/evaluate/backends.py:24``): ``setup_backend(name, config, model_path,
tokenizer, tp_size) -> (model, infer)`` with ``infer(list[str]) -> list[(text, seconds)]``; the
per-sample time is the batch time divided by the batch size.

* ``tah`` - this framework's paged-KV engine (left-padded prompts, ``do_sample = temperature > 0``).
  Unlike the reference, ``tp_size > 1`` is honoured: one tensor-parallel engine over ``tp_size`` GPUs, either the
  ranks of a ``torchrun`` job or follower processes spawned by the job (:mod:`tah_b200.evaluate.tp_group`).
* ``hf`` - a plain HuggingFace ``generate`` on the base model (needs the checkpoint's HF weights).
* ``sglang`` - only if the optional package is importable.
"""
from __future__ import annotations

import gc
import os
import time
from typing import Callable, Dict, List, Tuple

import torch

InferFn = Callable[[List[str]], List[Tuple[str, float]]]


def time_inference(fn, *args, **kwargs):
    """Run ``fn`` and return ``(result, seconds)``; CUDA events when a GPU is present, wall clock otherwise."""
    if torch.cuda.is_available():
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        out = fn(*args, **kwargs)
        end.record()
        torch.cuda.synchronize()
        return out, start.elapsed_time(end) / 1e3
    t0 = time.perf_counter()
    out = fn(*args, **kwargs)
    return out, time.perf_counter() - t0


def warmup(infer: InferFn, n: int = 1) -> None:
    for _ in range(n):
        infer(["Hello"])


def cleanup(model, backend: str) -> None:
    if backend == "sglang" and hasattr(model, "shutdown"):
        model.shutdown()
    group = getattr(model, "_tp_group", None)
    if group is not None:
        group.close()                             # stop the follower ranks of a tensor-parallel engine
    del model
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def _dtype(config: Dict):
    name = str(config.get("dtype", "bfloat16")).replace("torch.", "")
    return getattr(torch, name)


def _setup_tah_tp(config: Dict, model_path: str, tokenizer, tp_size: int):
    from tah_b200.evaluate.tp_group import TPEngineGroup
    group = TPEngineGroup(model_path, config, tp_size)
    model = group.model
    model._tp_group = group                       # cleanup() closes the group
    tokenizer.padding_side = "left"
    temperature = float(config.get("temperature", 0.0))
    gen_kw = dict(max_new_tokens=int(config.get("max_new_tokens", 1024)), do_sample=temperature > 0,
                  temperature=temperature if temperature > 0 else 1.0, top_p=float(config.get("top_p", 1.0)),
                  top_k=int(config.get("top_k", 0)), min_p=float(config.get("min_p", 0.0)),
                  eos_token_id=getattr(tokenizer, "eos_token_id", None))

    def infer(prompts: List[str]) -> List[Tuple[str, float]]:
        enc = tokenizer(prompts, return_tensors="pt", padding=True)
        res, secs = time_inference(group.generate, enc["input_ids"], enc.get("attention_mask"), **gen_kw)
        texts = [tokenizer.decode(t) if t else "" for t in res.tokens]
        return [(t, secs / max(1, len(prompts))) for t in texts]

    return model, infer


def setup_tah(config: Dict, model_path: str, tokenizer, tp_size: int = 1):
    if tp_size and tp_size > 1:
        return _setup_tah_tp(config, model_path, tokenizer, tp_size)
    from tah_b200 import TaHConfig, TaHForCausalLM
    from tah_b200.model.utils import TaHForCasualLM_generate
    fields = TaHConfig.__dataclass_fields__
    override = TaHConfig(**{k: v for k, v in config.items() if k in fields})
    model = TaHForCausalLM.from_pretrained(model_path, tah_config=override, torch_dtype=_dtype(config),
                                           device_map="auto")
    model.eval()
    tokenizer.padding_side = "left"
    temperature = float(config.get("temperature", 0.0))
    gen_kw = dict(max_new_tokens=int(config.get("max_new_tokens", 1024)), do_sample=temperature > 0,
                  temperature=temperature if temperature > 0 else 1.0, top_p=float(config.get("top_p", 1.0)),
                  top_k=int(config.get("top_k", 0)), min_p=float(config.get("min_p", 0.0)), verbose=False)

    def infer(prompts: List[str]) -> List[Tuple[str, float]]:
        enc = tokenizer(prompts, return_tensors="pt", padding=True)
        inputs = {k: v.to(model.device) for k, v in enc.items() if k in ("input_ids", "attention_mask")}
        (_, texts), secs = time_inference(TaHForCasualLM_generate, model, tokenizer, inputs, **gen_kw)
        return [(t, secs / max(1, len(prompts))) for t in texts]

    def serve_all(prompts: List[str], rows: int) -> List[Tuple[str, float]]:
        """All prompts of a job through the engine's continuous batching: ``rows`` requests decode at a time and a
        request that finishes hands its row (and KV pages) to the next queued one, instead of whole batches waiting
        for their longest answer (reasoning benchmarks have answers of 100 to 4096 tokens).  CUDA only."""
        from tah_b200.engine import get_engine
        eng = get_engine(model, max_rows=max(int(rows), 1))
        ids = [torch.tensor(tokenizer.encode(p), dtype=torch.long) for p in prompts]
        kw = {k: gen_kw[k] for k in ("max_new_tokens", "do_sample", "temperature", "top_p", "top_k", "min_p")}
        (tokens, stats), secs = time_inference(eng.serve, ids, rows=int(rows),
                                               eos_token_id=getattr(tokenizer, "eos_token_id", None), **kw)
        per = secs / max(1, len(prompts))
        return [(tokenizer.decode(t) if t else "", per) for t in tokens]

    if model.device.type == "cuda" and os.environ.get("TAH_B200_FORCE_TORCH", "0") != "1" \
            and bool(config.get("continuous_batching", True)):
        infer.serve_all = serve_all
    return model, infer


def setup_hf(config: Dict, model_path: str, tokenizer, tp_size: int = 1):
    from transformers import AutoModelForCausalLM
    model = AutoModelForCausalLM.from_pretrained(model_path, torch_dtype=_dtype(config), device_map="auto")
    model.eval()
    tokenizer.padding_side = "left"
    temperature = float(config.get("temperature", 0.0))

    def infer(prompts):
        enc = tokenizer(prompts, return_tensors="pt", padding=True).to(model.device)
        kw = dict(max_new_tokens=int(config.get("max_new_tokens", 1024)), do_sample=temperature > 0)
        if temperature > 0:
            kw.update(temperature=temperature, top_p=float(config.get("top_p", 1.0)), top_k=int(config.get("top_k", 0)) or None)
        out, secs = time_inference(model.generate, **enc, **kw)
        texts = tokenizer.batch_decode(out[:, enc["input_ids"].shape[1]:], skip_special_tokens=True)
        return [(t, secs / max(1, len(prompts))) for t in texts]

    return model, infer


def setup_sglang(config: Dict, model_path: str, tokenizer, tp_size: int = 1):
    try:
        import sglang as sgl
    except ImportError as exc:
        raise RuntimeError("the sglang backend needs the optional 'sglang' package") from exc
    engine = sgl.Engine(model_path=model_path, tp_size=tp_size, dtype=str(config.get("dtype", "bfloat16")),
                        mem_fraction_static=float(config.get("mem_fraction_static", 0.8)))
    params = {"temperature": float(config.get("temperature", 0.0)), "top_p": float(config.get("top_p", 1.0)),
              "top_k": int(config.get("top_k", -1)) or -1, "min_p": float(config.get("min_p", 0.0)),
              "max_new_tokens": int(config.get("max_new_tokens", 1024))}

    def infer(prompts):
        outs, secs = time_inference(engine.generate, prompts, params)
        return [(o["text"], secs / max(1, len(prompts))) for o in outs]

    return engine, infer


_SETUP_BY_NAME = {"tah": setup_tah, "hf": setup_hf, "sglang": setup_sglang}


def setup_backend(backend: str, config: Dict, model_path: str, tokenizer, tp_size: int = 1):
    if backend not in _SETUP_BY_NAME:
        raise ValueError(f"unknown backend {backend!r}; have {sorted(_SETUP_BY_NAME)}")
    return _SETUP_BY_NAME[backend](config, model_path, tokenizer, tp_size=tp_size)
