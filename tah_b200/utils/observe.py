"""Tracing and metrics: NVTX ranges, CUDA-event timers, a JSONL metrics sink.

The reference's only timing primitive is a CUDA-event pair around one ``generate`` call
(reference ``tah/evaluate/backends.py:27-41``).  Here every pass/layer/kernel family can be wrapped
in an NVTX range (visible to Nsight tools when they are available), device time is taken with
events on the launching stream, and counters go to a JSONL file (and to wandb when configured).
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from typing import Dict, Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available() and os.environ.get("TAH_B200_NVTX", "0") == "1"
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class DeviceTimer:
    """CUDA-event timer on the current stream: ``with DeviceTimer() as t: ...`` then ``t.ms``."""

    def __enter__(self):
        self.cuda = torch.cuda.is_available()
        if self.cuda:
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            self.e0.record()
        else:
            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            self.e1.record()
            torch.cuda.synchronize()
            self.ms = self.e0.elapsed_time(self.e1)
        else:
            self.ms = (time.perf_counter() - self.t0) * 1e3
        return False


class MetricsSink:
    """Append-only JSONL sink for counters such as hard-token rate, ticks per token, KV page
    occupancy per iteration cache, achieved GB/s of a collective."""

    def __init__(self, path: Optional[str] = None, wandb_run=None):
        self.path, self.wandb = path, wandb_run
        self._fh = open(path, "a") if path else None

    def log(self, record: Dict, step: Optional[int] = None) -> None:
        rec = dict(record, time=time.time())
        if step is not None:
            rec["step"] = step
        if self._fh:
            self._fh.write(json.dumps(rec) + "\n")
            self._fh.flush()
        if self.wandb is not None:
            self.wandb.log(record, step=step)

    def close(self):
        if self._fh:
            self._fh.close()


def engine_counters(engine, result) -> Dict:
    """Counters of one ``TaHEngine.generate`` call."""
    kv = engine.kv
    occ = {}
    if kv is not None:
        for d in range(kv.n_depths):
            free = int(kv.free_count[d])
            occ[f"kv_pages_used_depth{d}"] = kv.n_pages[d] - free
            occ[f"kv_pages_total_depth{d}"] = kv.n_pages[d]
    toks = max(1, result.tokens_emitted)
    return dict(occ, ticks=result.ticks, tokens=result.tokens_emitted,
                ticks_per_token=result.ticks * len(result.tokens) / toks,
                mean_passes_per_token=sum(result.iter_counts) / max(1, len(result.iter_counts)),
                prefill_ms=result.prefill_ms, decode_ms=result.decode_ms,
                launches_per_tick=engine.kernel_launches_per_tick)
