"""A tensor-parallel engine group for the evaluation backend.

The reference's ``tah`` backend ignores ``tp_size`` (reference ``tah/evaluate/backends.py:154-156``) and its job
runner only uses it to size the GPU group of a job (``tah/evaluate/jobs.py:399-423``).  Here ``tp_size > 1`` runs
one :class:`~tah_b200.engine.TaHEngine` over ``tp_size`` GPUs with the fused NVLink kernels of
:mod:`tah_b200.parallel.tp`:

* under ``torchrun`` (``torch.distributed`` already initialised with ``tp_size`` ranks) every rank builds its
  shard and calls ``generate`` with the same arguments;
* inside a plain job process, which sees ``tp_size`` GPUs, :class:`TPEngineGroup` spawns ``tp_size - 1`` follower
  processes (one per extra GPU).  The leader broadcasts every ``generate`` call (token ids, sampling
  parameters, seed) with ``broadcast_object_list``; followers run the same call on their shard and drop the
  result.  ``close()`` sends the stop message and joins them.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import socket
from typing import Dict, Optional

import torch
import torch.distributed as dist


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dtype(config: Dict):
    return getattr(torch, str(config.get("dtype", "bfloat16")).replace("torch.", ""))


def build_engine(model_path: str, config: Dict, device: torch.device, tp):
    """Load the checkpoint on ``device`` and wrap it in an engine over the tensor-parallel group ``tp``."""
    from tah_b200 import TaHConfig, TaHForCausalLM
    from tah_b200.engine import TaHEngine
    fields = TaHConfig.__dataclass_fields__
    override = TaHConfig(**{k: v for k, v in config.items() if k in fields})
    model = TaHForCausalLM.from_pretrained(model_path, tah_config=override, torch_dtype=_dtype(config), device=device)
    model.eval()
    rows = int(config.get("batch_size", 16))
    seq = int(config.get("max_prompt_tokens", 4096)) + int(config.get("max_new_tokens", 1024)) + 8
    return model, TaHEngine(model, max_rows=rows, max_seq_len=seq, tp=tp)


def _follower(rank: int, world: int, port: int, model_path: str, config: Dict) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from tah_b200.parallel.tp import TensorParallel
    _, eng = build_engine(model_path, config, dev, TensorParallel(dist.group.WORLD, dev))
    while True:
        box = [None]
        dist.broadcast_object_list(box, src=0)
        call = box[0]
        if call is None:
            break
        eng.generate(call["input_ids"], call["attention_mask"], **call["kwargs"])
    dist.barrier()
    os._exit(0)          # symmetric-memory mappings make process-group teardown block


class TPEngineGroup:
    """Leader side: owns rank 0's engine and the follower processes."""

    def __init__(self, model_path: str, config: Dict, tp_size: int):
        self.world = tp_size
        self.procs = []
        self.spawned = False
        if dist.is_available() and dist.is_initialized():
            if dist.get_world_size() != tp_size:
                raise ValueError(f"tp_size {tp_size} != torch.distributed world size {dist.get_world_size()}")
            self.rank = dist.get_rank()
            local = int(os.environ.get("LOCAL_RANK", self.rank))
        else:
            if torch.cuda.device_count() < tp_size:
                raise RuntimeError(f"tp_size {tp_size} needs {tp_size} visible GPUs, found {torch.cuda.device_count()}")
            port = _free_port()
            ctx = mp.get_context("spawn")
            for r in range(1, tp_size):
                p = ctx.Process(target=_follower, args=(r, tp_size, port, model_path, config), daemon=True)
                p.start()
                self.procs.append(p)
            os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK="0", WORLD_SIZE=str(tp_size),
                              LOCAL_RANK="0")
            self.rank, local, self.spawned = 0, 0, True
            torch.cuda.set_device(0)
            dist.init_process_group("nccl", device_id=torch.device("cuda", 0))
        dev = torch.device("cuda", local)
        from tah_b200.parallel.tp import TensorParallel
        self.model, self.engine = build_engine(model_path, config, dev, TensorParallel(dist.group.WORLD, dev))

    def generate(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor], **kwargs):
        """Same call on every rank of the group.  The sampling seed is fixed here so that all ranks draw the
        same tokens."""
        if kwargs.get("do_sample") and kwargs.get("seed") is None:
            kwargs["seed"] = int(torch.randint(0, 2 ** 62, (1,)).item())
        if self.spawned:
            dist.broadcast_object_list([{"input_ids": input_ids.cpu(), "attention_mask": None if attention_mask is None
                                         else attention_mask.cpu(), "kwargs": kwargs}], src=0)
        elif kwargs.get("seed") is not None:
            box = [kwargs["seed"]]
            dist.broadcast_object_list(box, src=0)                        # torchrun: agree on rank 0's seed
            kwargs["seed"] = box[0]
        return self.engine.generate(input_ids, attention_mask, **kwargs)

    def close(self) -> None:
        if self.spawned and self.procs:
            dist.broadcast_object_list([None], src=0)
            dist.barrier()
            for p in self.procs:
                p.join(timeout=30)
                if p.is_alive():
                    p.terminate()
            self.procs = []
