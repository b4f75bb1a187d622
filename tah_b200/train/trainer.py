"""Training loop for TaH SFT.

The reference subclasses HuggingFace ``Trainer`` and leaves distribution to accelerate/DeepSpeed
(reference ``tah/train/trainer.py:34-129``, ``script/train/SFT_TaH.py:134-243``).  This trainer is
self-contained: it shards data over ``torch.distributed`` ranks, accumulates gradients, and
steps the framework's own ZeRO optimizer (:class:`tah_b200.parallel.zero.ZeroAdamW`).  It accepts the
reference's ``training:`` YAML keys (unknown ones are ignored) and reproduces its conventions:

* the training dataloader always shuffles;
* ``num_items_in_batch`` = supervised label tokens over the whole accumulation window on the rank;
  every micro-batch loss is ``sum / num_items_in_batch`` and is NOT divided again by the number of
  accumulation steps; gradients are then averaged over ranks;
* ``avg_iter_count`` and ``iter_decider_accuracy`` are accumulated by the model on its
  ``logger_callback`` and flushed into every log record;
* ``_save`` writes the TaH checkpoint layout plus the tokenizer.
"""
from __future__ import annotations

import json
import math
import os
import shutil
import time
from dataclasses import dataclass, field, fields
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from tah_b200.model.loss import fixed_cross_entropy  # noqa: F401  (re-exported like the reference module)
from tah_b200.parallel.zero import ZeroAdamW
from tah_b200.train.schedule import lr_factor
from tah_b200.utils.failure import RankFailure, RankHeartbeat, StepTimeout, StepWatchdog
from tah_b200.utils.observe import MetricsSink, nvtx_range


@dataclass
class TaHTrainingArguments:
    output_dir: str = "output"
    per_device_train_batch_size: int = 1
    per_device_eval_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    learning_rate: float = 5e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    num_train_epochs: float = 1.0
    max_steps: int = -1
    lr_scheduler_type: str = "linear"
    lr_scheduler_kwargs: Dict[str, Any] = field(default_factory=dict)
    warmup_ratio: float = 0.0
    warmup_steps: int = 0
    logging_steps: int = 10
    eval_strategy: str = "no"
    eval_steps: Optional[int] = None
    eval_on_start: bool = False
    save_strategy: str = "epoch"
    save_steps: Optional[int] = None
    save_total_limit: Optional[int] = None
    save_only_model: bool = False
    bf16: bool = True
    seed: int = 42
    report_to: Any = "none"
    run_name: Optional[str] = None
    gradient_checkpointing: bool = False
    dataloader_num_workers: int = 0
    dataloader_drop_last: bool = False
    ddp_find_unused_parameters: bool = False
    remove_unused_columns: bool = False
    # parallel strategy: "zero2" (replicated bf16 parameters, sharded fp32 state) or "zero3" (parameters sharded too)
    strategy: str = "zero2"
    # tensor-parallel size: the decoder layers are sharded over groups of tp_size adjacent ranks
    # (tah_b200.parallel.tp_train), the remaining world / tp_size ranks are data parallel (zero2 over that group)
    tp_size: int = 1
    # failure detection (multi-rank jobs): every rank bumps a heartbeat counter in the rendezvous store; before each
    # optimizer step the peers' counters are checked and a rank whose counter stood still for heartbeat_timeout_s is
    # reported as a RankFailure; a step that runs longer than step_timeout_s (> 0) raises StepTimeout
    heartbeat_interval_s: float = 1.0
    heartbeat_timeout_s: float = 60.0
    step_timeout_s: float = 0.0
    metrics_file: Optional[str] = None          # JSONL sink for per-step counters (default <output_dir>/metrics.jsonl)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TaHTrainingArguments":
        known = {f.name for f in fields(cls)}
        d = dict(d)
        if "evaluation_strategy" in d and "eval_strategy" not in d:
            d["eval_strategy"] = d.pop("evaluation_strategy")
        return cls(**{k: v for k, v in d.items() if k in known and v is not None})


@dataclass
class TrainerState:
    global_step: int = 0
    epoch: float = 0.0
    max_steps: int = 0
    log_history: List[Dict[str, Any]] = field(default_factory=list)


class TrainerCallback:
    def on_log(self, args, state, control, **kwargs):
        pass

    def on_step_end(self, args, state, control, **kwargs):
        pass


class LoggerCallback(TrainerCallback):
    """Forwards the model's iteration counters into the log stream and resets them
    (reference ``tah/train/trainer.py:110-129``)."""

    def __init__(self):
        self.avg_iter_count = 0.0
        self.iter_decider_accuracy = 0.0

    def on_log(self, args, state, control, **kwargs):
        logs = kwargs["logs"]
        logs["avg_iter_count"] = self.avg_iter_count
        if self.iter_decider_accuracy > 0.0:
            logs["iter_decider_accuracy"] = self.iter_decider_accuracy
        self.avg_iter_count = 0.0
        self.iter_decider_accuracy = 0.0


class CustomTaHTrainer:
    def __init__(self, model, args: TaHTrainingArguments, train_dataset=None, eval_dataset=None,
                 processing_class=None, tokenizer=None, data_collator: Optional[Callable] = None,
                 callbacks: Optional[List[TrainerCallback]] = None):
        self.model, self.args = model, args
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self.tokenizer = processing_class if processing_class is not None else tokenizer
        self.data_collator = data_collator
        self.callbacks: List[TrainerCallback] = list(callbacks or [])
        self.state = TrainerState()
        self.dist_on = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank() if self.dist_on else 0
        self.world = dist.get_world_size() if self.dist_on else 1
        self.dp_rank, self.dp_world = self.rank, self.world      # data-parallel coordinates (differ under TP)
        self.optimizer: Optional[ZeroAdamW] = None
        self._log_file = None
        self._wandb = None
        self.heartbeat: Optional[RankHeartbeat] = None
        self.metrics: Optional[MetricsSink] = None

    # ---- callbacks ------------------------------------------------------------------------------
    def add_callback(self, cb):
        self.callbacks.append(cb)

    def insert_callback(self, index: int, cb):
        self.callbacks.insert(index, cb)

    def _emit_log(self, logs: Dict[str, Any]):
        for cb in self.callbacks:
            cb.on_log(self.args, self.state, None, logs=logs)
        logs["step"] = self.state.global_step
        logs["epoch"] = round(self.state.epoch, 4)
        self.state.log_history.append(dict(logs))
        if self.rank == 0:
            if self._log_file is None:
                os.makedirs(self.args.output_dir, exist_ok=True)
                self._log_file = open(os.path.join(self.args.output_dir, "trainer_log.jsonl"), "a")
            self._log_file.write(json.dumps(logs) + "\n")
            self._log_file.flush()
            print(logs, flush=True)
            if self._wandb is not None:
                self._wandb.log(logs, step=self.state.global_step)

    # ---- data -----------------------------------------------------------------------------------
    def _loader(self, dataset, batch_size: int, shuffle: bool, epoch: int = 0):
        """Index batches of this rank.  Training always shuffles (seeded per epoch)."""
        n = len(dataset)
        if shuffle:
            g = torch.Generator().manual_seed(self.args.seed + epoch)
            order = torch.randperm(n, generator=g).tolist()
        else:
            order = list(range(n))
        dw = self.dp_world
        per_rank = math.ceil(n / dw) if not self.args.dataloader_drop_last else n // dw
        order = (order + order[: per_rank * dw - n])[: per_rank * dw] if per_rank * dw > n else order
        mine = order[self.dp_rank::dw]
        for i in range(0, len(mine), batch_size):
            idx = mine[i:i + batch_size]
            if len(idx) < batch_size and self.args.dataloader_drop_last:
                break
            feats = [dict(dataset[j]) for j in idx]
            yield self.data_collator(feats) if self.data_collator else feats

    def _to_device(self, batch):
        dev = self.model.device
        return {k: (v.to(dev, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}

    def steps_per_epoch(self) -> int:
        per_rank = math.ceil(len(self.train_dataset) / self.dp_world)
        micro = math.ceil(per_rank / self.args.per_device_train_batch_size)
        return max(1, micro // self.args.gradient_accumulation_steps)

    # ---- optimizer ------------------------------------------------------------------------------
    def create_optimizer(self):
        """``strategy: zero2`` - replicated bf16 parameters, sharded fp32 state (:class:`ZeroAdamW`);
        ``strategy: zero3`` - parameters sharded as well: the model is cut into units whose weights are gathered
        layer by layer (:mod:`tah_b200.parallel.fsdp`).  One process falls back to the first form.
        ``tp_size > 1``: the layers are sharded over tensor-parallel groups first (:mod:`tah_b200.parallel.tp_train`)
        and the optimizer runs zero2 over the data-parallel group of the rank."""
        a = self.args
        kw = dict(lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                  weight_decay=a.weight_decay, max_grad_norm=a.max_grad_norm or 0.0)
        no_decay = [p for n, p in self.model.named_parameters()
                    if p.dim() < 2 or n.endswith("bias") or "norm" in n.lower() or n.endswith("threshold")]
        if int(getattr(a, "tp_size", 1) or 1) > 1:
            if not self.dist_on or self.world % int(a.tp_size):
                raise ValueError(f"tp_size {a.tp_size} needs a world size that is a multiple of it")
            if str(a.strategy).lower() in ("zero3", "fsdp"):
                raise NotImplementedError("tp_size > 1 runs with strategy zero2 (parameter sharding is not combined)")
            from tah_b200.parallel.tp_train import TPOptimizer, shard_model_tp, tp_dp_groups
            tp_group, dp_group, _, self.dp_rank = tp_dp_groups(int(a.tp_size))
            self.dp_world = self.world // int(a.tp_size)
            st = getattr(self.model, "_tp_train", None) or shard_model_tp(self.model, tp_group)
            no_decay = [p for n, p in self.model.named_parameters()
                        if p.dim() < 2 or n.endswith("bias") or "norm" in n.lower() or n.endswith("threshold")]
            self.optimizer = TPOptimizer(ZeroAdamW(self.model.parameters(), group=dp_group, no_decay=no_decay, **kw), st)
        elif str(a.strategy).lower() in ("zero3", "fsdp") and self.dist_on and self.world > 1:
            from tah_b200.parallel.fsdp import FsdpAdamW, shard_model
            if getattr(self.model, "_fsdp", None) is None:
                shard_model(self.model, dist.group.WORLD, self.model.device)
            self.optimizer = FsdpAdamW(self.model, no_decay=no_decay, **kw)
        else:
            self.optimizer = ZeroAdamW(self.model.parameters(), group=None, no_decay=no_decay, **kw)
        return self.optimizer

    def _lr_at(self, step: int) -> float:
        a = self.args
        warm = a.warmup_steps or int(a.warmup_ratio * self.state.max_steps)
        kw = a.lr_scheduler_kwargs or {}
        return a.learning_rate * lr_factor(step, self.state.max_steps, warm, a.lr_scheduler_type,
                                           float(kw.get("min_lr_rate", 0.0)), float(kw.get("num_cycles", 0.5)))

    # ---- train ----------------------------------------------------------------------------------
    def train(self, resume_from_checkpoint: Optional[str] = None):
        a = self.args
        if a.gradient_checkpointing and hasattr(self.model, "gradient_checkpointing_enable"):
            self.model.gradient_checkpointing_enable()
        if self.optimizer is None:
            self.create_optimizer()
        torch.manual_seed(a.seed + self.dp_rank)        # ranks of one tensor-parallel group draw the same dropout masks
        self._resume_rng = None
        spe = self.steps_per_epoch()
        self.state.max_steps = a.max_steps if a.max_steps and a.max_steps > 0 else int(math.ceil(spe * a.num_train_epochs))
        if resume_from_checkpoint:
            self._load_training_state(resume_from_checkpoint)
            if self._resume_rng is not None:
                torch.set_rng_state(self._resume_rng["cpu"])
                if self._resume_rng.get("cuda") is not None and self.model.device.type == "cuda":
                    torch.cuda.set_rng_state(self._resume_rng["cuda"], self.model.device)
        if a.report_to in ("wandb", ["wandb"]) and self.rank == 0:
            try:
                import wandb
                self._wandb = wandb
                wandb.init(project=os.environ.get("WANDB_PROJECT"), name=a.run_name, config=vars(a))
            except Exception:
                self._wandb = None
        if a.eval_on_start and self.eval_dataset is not None:
            self._emit_log(self.evaluate())
        self.model.train()
        accum = a.gradient_accumulation_steps
        loss_window, t0 = [], time.time()
        start_epoch = self.state.global_step // spe
        self._start_failure_detection()
        if self.rank == 0 and self.metrics is None:
            os.makedirs(a.output_dir, exist_ok=True)
            self.metrics = MetricsSink(a.metrics_file or os.path.join(a.output_dir, "metrics.jsonl"), self._wandb)
        try:
            return self._train_loop(a, spe, accum, loss_window, t0, start_epoch)
        except (RankFailure, StepTimeout) as exc:
            # a peer is gone or a collective stalled: say so in the log and stop cleanly; the job is restarted from
            # the last checkpoint with resume_from_checkpoint
            self._emit_log({"event": type(exc).__name__, "detail": str(exc)})
            raise
        finally:
            if self.heartbeat is not None:
                self.heartbeat.stop()
            if self.metrics is not None:
                self.metrics.close()
                self.metrics = None

    def _start_failure_detection(self):
        a = self.args
        if not self.dist_on or self.world < 2 or a.heartbeat_interval_s <= 0 or self.heartbeat is not None:
            return
        try:
            store = dist.distributed_c10d._get_default_store()
        except Exception:
            return
        self.heartbeat = RankHeartbeat(dist.PrefixStore("tah_b200_hb", store), self.rank, self.world,
                                       interval_s=a.heartbeat_interval_s).start()

    def _check_device_status(self):
        """Raise KernelTimeout if a kernel of this step gave up on a bounded wait (reads the status word)."""
        dev = self.model.device
        if dev.type == "cuda":
            from tah_b200.ops import cuda as K
            K.check_status(dev)

    def _train_loop(self, a, spe, accum, loss_window, t0, start_epoch):
        for epoch in range(start_epoch, int(math.ceil(a.num_train_epochs)) if a.max_steps <= 0 else 10 ** 9):
            micro = list(self._loader(self.train_dataset, a.per_device_train_batch_size, True, epoch))
            if not micro:
                raise RuntimeError("the training set is empty on this rank")
            # an epoch with fewer micro-batches than the accumulation window is one (shorter) window, so that every
            # epoch makes at least the one step that steps_per_epoch() promises
            accum = min(accum, len(micro))
            skip = (self.state.global_step - epoch * spe) * accum if epoch == start_epoch else 0
            for w in range(skip, len(micro) - accum + 1, accum):
                window = micro[w:w + accum]
                n_items = sum(int((b["labels"][..., 1:] != -100).sum()) for b in window if "labels" in b)
                n_items = max(n_items, 1)
                step_loss = 0.0
                if self.heartbeat is not None:
                    self.heartbeat.check_peers(a.heartbeat_timeout_s)      # before launching kernels that wait on peers
                t_step = time.perf_counter()
                n_tok = 0
                with StepWatchdog(a.step_timeout_s if a.step_timeout_s > 0 else 10 ** 9), \
                        nvtx_range(f"train/step{self.state.global_step}"):
                    for b in window:
                        b = self._to_device(b)
                        n_tok += int(b["input_ids"].numel()) if "input_ids" in b else 0
                        with nvtx_range("train/forward"):
                            out = self.model(**b, num_items_in_batch=n_items)
                        with nvtx_range("train/backward"):
                            out.loss.backward()
                        if accum > 1 and hasattr(self.optimizer, "accumulate"):
                            self.optimizer.accumulate()          # fp32 sum over the window, one rounding at the step
                        step_loss += float(out.loss.detach())
                    lr = self._lr_at(self.state.global_step)
                    with nvtx_range("train/optimizer"):
                        gnorm = self.optimizer.step(grad_scale=1.0, lr=lr)
                    self.optimizer.zero_grad()
                    self._check_device_status()
                if self.metrics is not None:
                    dt = time.perf_counter() - t_step
                    rec = {"step_s": round(dt, 4), "tokens": n_tok, "tokens_per_s": round(n_tok * self.dp_world / max(dt, 1e-9), 1),
                           "loss": step_loss}
                    if self.model.device.type == "cuda":
                        rec["peak_mem_gb"] = round(torch.cuda.max_memory_allocated(self.model.device) / 2 ** 30, 2)
                    self.metrics.log(rec, step=self.state.global_step)
                self.state.global_step += 1
                self.state.epoch = self.state.global_step / spe
                loss_window.append(step_loss)
                if self.state.global_step % a.logging_steps == 0 or self.state.global_step == self.state.max_steps:
                    mean_loss = sum(loss_window) / len(loss_window)
                    if self.dist_on:
                        t = torch.tensor([mean_loss], device=self.model.device)
                        dist.all_reduce(t)
                        mean_loss = float(t) / self.world
                    self._emit_log({"loss": round(mean_loss, 6), "learning_rate": lr, "grad_norm": float(gnorm),
                                    "steps_per_s": round(len(loss_window) / max(1e-9, time.time() - t0), 4)})
                    loss_window, t0 = [], time.time()
                if a.eval_strategy == "steps" and a.eval_steps and self.state.global_step % a.eval_steps == 0 \
                        and self.eval_dataset is not None:
                    self._emit_log(self.evaluate())
                    self.model.train()
                if a.save_strategy == "steps" and a.save_steps and self.state.global_step % a.save_steps == 0:
                    self.save_checkpoint()
                if self.state.global_step >= self.state.max_steps:
                    break
            if a.eval_strategy == "epoch" and self.eval_dataset is not None:
                self._emit_log(self.evaluate())
                self.model.train()
            if a.save_strategy == "epoch":
                self.save_checkpoint()
            if self.state.global_step >= self.state.max_steps:
                break
        return self.state

    # ---- eval -----------------------------------------------------------------------------------
    @torch.no_grad()
    def evaluate(self) -> Dict[str, float]:
        self.model.eval()
        tot, cnt = 0.0, 0
        for b in self._loader(self.eval_dataset, self.args.per_device_eval_batch_size, False):
            b = self._to_device(b)
            out = self.model(**b)
            if out.loss is not None:
                tot += float(out.loss)
                cnt += 1
        if self.dist_on:
            t = torch.tensor([tot, cnt], dtype=torch.float64, device=self.model.device)
            dist.all_reduce(t)
            tot, cnt = float(t[0]), int(t[1])
        return {"eval_loss": tot / max(cnt, 1)}

    # ---- save / resume --------------------------------------------------------------------------
    def _save(self, output_dir: Optional[str] = None, state_dict=None):
        output_dir = output_dir or self.args.output_dir
        os.makedirs(output_dir, exist_ok=True)
        fsdp = getattr(self.model, "_fsdp", None) or getattr(self.model, "_tp_train", None)
        if fsdp is not None:
            # parameter-sharded model: every rank takes part in gathering the full 16-bit weights, rank 0 writes
            with fsdp.materialized():
                if self.rank == 0:
                    print(f"Saving TaH model to: {output_dir}")
                    self.model.save_pretrained(output_dir)
        elif self.rank == 0:
            print(f"Saving TaH model to: {output_dir}")
            self.model.save_pretrained(output_dir)
        if self.rank == 0 and self.tokenizer is not None and hasattr(self.tokenizer, "save_pretrained"):
            self.tokenizer.save_pretrained(output_dir)

    def save_model(self, output_dir: Optional[str] = None):
        self._save(output_dir)

    def save_checkpoint(self):
        a = self.args
        ckpt = os.path.join(a.output_dir, f"checkpoint-{self.state.global_step}")
        self._save(ckpt)
        if not a.save_only_model and self.optimizer is not None:
            os.makedirs(os.path.join(ckpt, "optim"), exist_ok=True)
            sd = self.optimizer.state_dict()
            # random-number state of this rank (dropout masks, forced continuations): an exact resume continues it
            sd["rng"] = {"cpu": torch.get_rng_state(),
                         "cuda": torch.cuda.get_rng_state(self.model.device) if self.model.device.type == "cuda" else None}
            torch.save(sd, os.path.join(ckpt, "optim", f"rank{self.rank}.pt"))
        if self.rank == 0:
            with open(os.path.join(ckpt, "trainer_state.json"), "w") as fh:
                json.dump({"global_step": self.state.global_step, "epoch": self.state.epoch,
                           "max_steps": self.state.max_steps, "log_history": self.state.log_history}, fh, indent=1)
            if a.save_total_limit:
                kept = sorted((d for d in os.listdir(a.output_dir) if d.startswith("checkpoint-")),
                              key=lambda d: int(d.split("-")[1]))
                for old in kept[:-a.save_total_limit]:
                    shutil.rmtree(os.path.join(a.output_dir, old), ignore_errors=True)
        if self.dist_on:
            dist.barrier()

    def _load_training_state(self, ckpt: str):
        st = os.path.join(ckpt, "trainer_state.json")
        if os.path.exists(st):
            with open(st) as fh:
                d = json.load(fh)
            self.state.global_step, self.state.epoch = int(d["global_step"]), float(d["epoch"])
        opt = os.path.join(ckpt, "optim", f"rank{self.rank}.pt")
        if os.path.exists(opt) and self.optimizer is not None:
            sd = torch.load(opt, map_location="cpu", weights_only=False)
            rng = sd.pop("rng", None)
            self.optimizer.load_state_dict(sd)
            if rng is not None:
                self._resume_rng = rng                       # applied after train() has seeded the generators
