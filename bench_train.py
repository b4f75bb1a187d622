"""Training throughput benchmark: TaH-plus-1.7B supervised fine-tuning step, tokens/s.

    python bench_train.py --steps 3 --warmup 1                       # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        bench_train.py --steps 3 --warmup 1                          # data parallel, sharded optimizer

Configuration (the reference's SFT recipe shape, reference ``script/recipes/qwen3_1.7/sft_tah_step2.yaml``,
on synthetic data): full 28-layer Qwen3-1.7B shapes, LoRA rank 64 on every linear for iteration 2, packed
sequences of ``--seq`` uniform-random token ids, one sequence per micro-batch and ``--accum``
micro-batches per optimizer step on every rank, per-token hard labels Bernoulli(``--hard-rate``) (1.0 =
every token takes the second iteration, the oracle-iteration mode) followed by the label decider,
next-token cross entropy on the iteration-selected logits (plus the decider BCE with ``--decider mlp``),
bf16 parameters with fp32 master weights in the sharded AdamW (lr 2e-5, weight decay 0.01); ``--checkpoint``
turns on gradient checkpointing per decoder stage (the 1.7B model at 8192 tokens fits without it).  One step = forward + backward of ``accum`` micro-batches + the
optimizer step (gradient reduce-scatter, AdamW, parameter broadcast).  Time is CUDA-event time of
``--steps`` steps after ``--warmup``, maximum over ranks; prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--accum", type=int, default=1)
    ap.add_argument("--hard-rate", type=float, default=1.0)
    ap.add_argument("--model", default="tah-plus-1.7b")
    ap.add_argument("--decider", default="label", choices=["label", "mlp"])
    ap.add_argument("--lora-rank", type=int, default=64)
    ap.add_argument("--checkpoint", action="store_true",
                    help="recompute the dense stages of every layer in backward (needed for longer sequences / larger models)")
    a = ap.parse_args()

    import torch
    import torch.distributed as dist
    from tah_b200.model.tah_config import TaHConfig
    from tah_b200.model.tah_model import TaHForCausalLM
    from tah_b200.models.qwen3 import Qwen3ForCausalLM, preset
    from tah_b200.parallel.zero import ZeroAdamW

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    cfg = preset(a.model, torch_dtype="bfloat16")
    with torch.device(dev):
        base = Qwen3ForCausalLM(cfg, dtype=torch.bfloat16)
    if a.decider == "label":
        tcfg = TaHConfig(max_iter=2, iter_decider="IterLabelDecider", iter_decider_kwargs={},
                         adapter_kwargs=dict(r=a.lora_rank, lora_alpha=2 * a.lora_rank, lora_dropout=0.0,
                                             target_modules="all-linear"),
                         input_updater_kwargs={"topk": 100}, train_loss="NextTokenPredLoss")
    else:
        tcfg = TaHConfig(max_iter=2, iter_decider="SimpleMLPIterDecider",
                         iter_decider_kwargs=dict(hidden_states_size=cfg.hidden_size, inner_size=cfg.hidden_size // 4,
                                                  threshold=0.5),
                         adapter_kwargs=dict(r=a.lora_rank, lora_alpha=2 * a.lora_rank, lora_dropout=0.0,
                                             target_modules="all-linear"),
                         input_updater_kwargs={"topk": 100}, train_loss="CombinedLoss")
    model = TaHForCausalLM(base, tcfg).to(dev)
    model.iter_decider.to(device=dev, dtype=torch.bfloat16)
    model.train()
    if a.checkpoint:
        model.gradient_checkpointing_enable()
    opt = ZeroAdamW(model.parameters(), lr=2e-5, weight_decay=0.01, max_grad_norm=1.0)

    g = torch.Generator().manual_seed(100 + rank)
    V = cfg.vocab_size

    def batch():
        ids = torch.randint(0, V, (1, a.seq), generator=g).pin_memory()
        hard = (torch.rand(1, a.seq, generator=g) < a.hard_rate).long() + 1
        return ids.to(dev, non_blocking=True), hard.pin_memory().to(dev, non_blocking=True)

    def step():
        total = 0.0
        for _ in range(a.accum):
            ids, hard = batch()
            out = model(ids, labels=ids, iter_count_labels=hard)
            (out.loss / a.accum).backward()
            total += float(out.loss.detach())
        opt.step()
        opt.zero_grad()
        return total / a.accum

    for _ in range(a.warmup):
        loss = step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    toks = a.steps * a.accum * a.seq * world
    if rank == 0:
        print(json.dumps({
            "metric": "TaH-plus-1.7B SFT training tokens/s", "value": round(toks / (ms / 1e3), 1), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms / a.steps, 1),
            "wall_s": round(wall, 2), "loss": round(loss, 4), "dtype": "bf16 (fp32 master weights)",
            "data": "synthetic", "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
            "config": {"model": a.model, "seq_len": a.seq, "micro_batches_per_step": a.accum, "global_batch": a.accum * world,
                       "hard_rate": a.hard_rate, "decider": a.decider, "lora_rank": a.lora_rank, "max_iter": 2,
                       "parallelism": f"dp{world} + sharded AdamW", "grad_checkpointing": bool(a.checkpoint)}}))
    if world > 1:
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
