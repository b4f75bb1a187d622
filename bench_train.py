"""Training throughput benchmark: TaH-plus-1.7B supervised fine-tuning step, tokens/s.

    python bench_train.py --steps 3 --warmup 1                       # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        bench_train.py --steps 3 --warmup 1 [--strategy zero3]       # N GPUs

Configuration (the reference's SFT recipe shape, reference ``script/recipes/qwen3_1.7/sft_tah_step2.yaml``,
on synthetic data): full 28-layer Qwen3-1.7B shapes, LoRA rank 64 on every linear for iteration 2, packed
sequences of ``--seq`` uniform-random token ids, one sequence per micro-batch and ``--accum``
micro-batches per optimizer step on every rank, bf16 parameters with fp32 master weights in the sharded
AdamW (lr 2e-5, weight decay 0.01).  ``--decider`` picks the objective:

* ``oracle-mlp`` (default; the FSDP training configuration as named): every token takes the second iteration
  (oracle-iteration mode), per-token hard labels are Bernoulli(``--hard-rate``, default 0.06) and supervise the
  two-layer decider MLP through BCE, which is added to the next-token CE on the iteration-selected output;
* ``label``: the label decider with next-token CE only (``--hard-rate 1.0`` = every token iterates);
* ``mlp``: the decider MLP decides by itself (threshold 0.5), CE + BCE.

``--strategy``: ``zero2`` (replicated bf16 parameters; sharded fp32 state; fused gradient reduce-scatter + AdamW +
broadcast) or ``zero3`` (parameters sharded as well: every layer's weights are gathered by the push kernel ahead
of their first use in the forward and the backward pass, its gradients are reduce-scattered when its backward
ends; see ``tah_b200/parallel/fsdp.py``).  ``--checkpoint`` turns on gradient checkpointing per decoder stage.
One step = forward + backward of ``accum`` micro-batches + the optimizer step.  Time is CUDA-event time of
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


def add_args(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--accum", type=int, default=1)
    ap.add_argument("--hard-rate", type=float, default=None)
    ap.add_argument("--train-model", default="tah-plus-1.7b")
    ap.add_argument("--decider", default="oracle-mlp", choices=["oracle-mlp", "label", "mlp"])
    ap.add_argument("--lora-rank", type=int, default=64)
    ap.add_argument("--strategy", default="zero2", choices=["zero2", "zero3"])
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (layers sharded over groups of adjacent ranks)")
    ap.add_argument("--kernel-table", default=None,
                    help="after the timed steps, run one more step under the PyTorch profiler and write the kernels' "
                         "device-time table to this file (rank 0)")
    ap.add_argument("--checkpoint", action="store_true",
                    help="recompute the dense stages of every layer in backward (needed for longer sequences / larger models)")


def build_train_model(a, dev):
    import torch
    from tah_b200.model.iter_decider import BernoulliIterDecider
    from tah_b200.model.tah_config import TaHConfig
    from tah_b200.model.tah_model import TaHForCausalLM
    from tah_b200.models.qwen3 import Qwen3ForCausalLM, preset
    torch.manual_seed(0)
    cfg = preset(a.train_model, torch_dtype="bfloat16")
    with torch.device(dev):
        base = Qwen3ForCausalLM(cfg, dtype=torch.bfloat16)
    adapter = dict(r=a.lora_rank, lora_alpha=2 * a.lora_rank, lora_dropout=0.0, target_modules="all-linear")
    if a.decider == "label":
        tcfg = TaHConfig(max_iter=2, iter_decider="IterLabelDecider", iter_decider_kwargs={}, adapter_kwargs=adapter,
                         input_updater_kwargs={"topk": 100}, train_loss="NextTokenPredLoss")
    else:
        tcfg = TaHConfig(max_iter=2, iter_decider="SimpleMLPIterDecider",
                         iter_decider_kwargs=dict(hidden_states_size=cfg.hidden_size, inner_size=cfg.hidden_size // 4,
                                                  hidden_states_layer_nums=[cfg.num_hidden_layers], threshold=0.5),
                         adapter_kwargs=adapter, input_updater_kwargs={"topk": 100}, train_loss="CombinedLoss")
    model = TaHForCausalLM(base, tcfg).to(dev)
    model.iter_decider.to(device=dev, dtype=torch.bfloat16)
    if a.decider == "oracle-mlp":
        # every token continues (p = 1); the MLP's logits are still computed and trained by the BCE term
        model.iter_decider = BernoulliIterDecider(p=1.0, seed=0, max_iter=2, inner=model.iter_decider)
        model.eval_iter_decider = model.iter_decider
    model.train()
    if a.checkpoint:
        model.gradient_checkpointing_enable()
    return model, cfg


def run(a, steps: int, warmup: int) -> dict:
    """Build the model and optimizer, run ``warmup`` + ``steps`` optimizer steps, return the result record
    (the same on every rank; times are the maximum over ranks).  ``torch.distributed`` must already be
    initialised when WORLD_SIZE > 1."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    hard_rate = a.hard_rate if a.hard_rate is not None else (1.0 if a.decider == "label" else 0.06)
    model, cfg = build_train_model(a, dev)
    tp_size = int(getattr(a, "tp", 1) or 1)
    dp_world, dp_rank = world, rank
    if tp_size > 1:
        from tah_b200.parallel.tp_train import TPOptimizer, shard_model_tp, tp_dp_groups
        from tah_b200.parallel.zero import ZeroAdamW
        tp_group, dp_group, _, dp_rank = tp_dp_groups(tp_size)
        dp_world = world // tp_size
        st = shard_model_tp(model, tp_group)
        opt = TPOptimizer(ZeroAdamW(model.parameters(), group=dp_group, lr=2e-5, weight_decay=0.01, max_grad_norm=1.0), st)
    elif a.strategy == "zero3" and world > 1:
        from tah_b200.parallel.fsdp import FsdpAdamW, shard_model
        shard_model(model, dist.group.WORLD, dev)
        opt = FsdpAdamW(model, lr=2e-5, weight_decay=0.01, max_grad_norm=1.0)
    else:
        from tah_b200.parallel.zero import ZeroAdamW
        opt = ZeroAdamW(model.parameters(), lr=2e-5, weight_decay=0.01, max_grad_norm=1.0)

    g = torch.Generator().manual_seed(100 + dp_rank)          # ranks of one tensor-parallel group see the same batch
    V = cfg.vocab_size
    h2d = 0

    def batch():
        nonlocal h2d
        ids = torch.randint(0, V, (1, a.seq), generator=g).pin_memory()
        hard = ((torch.rand(1, a.seq, generator=g) < hard_rate).long() + 1).pin_memory()
        h2d = ids.numel() * ids.element_size() + hard.numel() * hard.element_size()
        return ids.to(dev, non_blocking=True), hard.to(dev, non_blocking=True)

    def step():
        total = 0.0
        for _ in range(a.accum):
            ids, hard = batch()
            out = model(ids, labels=ids, iter_count_labels=hard)
            (out.loss / a.accum).backward()
            total += float(out.loss.detach())          # device -> host read of the step's result
        opt.step()
        opt.zero_grad()
        return total / a.accum

    loss = float("nan")
    for _ in range(warmup):
        loss = step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.reset_peak_memory_stats()
    from bench_clocks import ClockSampler
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    if getattr(a, "kernel_table", None):
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        if rank == 0:
            with open(a.kernel_table, "w") as fh:
                fh.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=60, max_name_column_width=90))
    ms = torch.tensor([e0.elapsed_time(e1), wall * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms, wall_ms = float(ms[0]), float(ms[1])
    toks = steps * a.accum * a.seq * dp_world
    rec = {
        "metric": ("TaH-plus-1.7B" if a.train_model == "tah-plus-1.7b" else a.train_model) + " SFT training tokens/s", "value": round(toks / (ms / 1e3), 1), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms / max(1, steps), 1),
        "e2e": {"value": round(toks / (wall_ms / 1e3), 1), "unit": "tokens/s",
                "includes": "pinned-host batch H2D every micro-batch, forward, backward, optimizer, loss D2H",
                "h2d_bytes_per_step": h2d * a.accum, "d2h_bytes_per_step": 4 * a.accum},
        "loss": round(loss, 4), "dtype": "bf16 (fp32 master weights)", "clocks": clocks,
        "data": "synthetic", "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
        "config": {"model": a.train_model, "seq_len": a.seq, "micro_batches_per_step": a.accum,
                   "global_batch": a.accum * dp_world, "hard_rate": hard_rate, "decider": a.decider,
                   "loss": "CE" if a.decider == "label" else "CE + decider BCE",
                   "second_iteration_on": "labelled tokens" if a.decider == "label" else
                                          ("every token" if a.decider == "oracle-mlp" else "tokens the decider picks"),
                   "lora_rank": a.lora_rank, "max_iter": 2,
                   "parallelism": (f"tp{tp_size} x dp{dp_world} (layers sharded over the tensor-parallel group, zero2 over the data-parallel group)"
                                   if tp_size > 1 else f"fsdp{world} (zero3: sharded parameters, gradients, optimizer state)"
                                   if a.strategy == "zero3" and world > 1 else f"dp{world} + sharded AdamW (zero2)"),
                   "grad_checkpointing": bool(a.checkpoint)}}
    del opt, model
    torch.cuda.empty_cache()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--model", dest="train_model_alias", default=None)
    add_args(ap)
    a = ap.parse_args()
    if a.train_model_alias:
        a.train_model = a.train_model_alias

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rec = run(a, a.steps, a.warmup)
    if rank == 0:
        print(json.dumps(rec))
    if world > 1:
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
