"""Worker for the multi-GPU parameter-sharding test (launched by torchrun from test_fsdp_gpu.py).

On ``WORLD_SIZE`` GPUs: the same tiny TaH model is trained for a few steps (two micro-batches per step, two
passes per micro-batch) once with the ZeRO-2 optimizer (replicated parameters) and once parameter-sharded
(``shard_model`` + ``FsdpAdamW``: layer-wise gather by the push kernel, the layer's first tcgen05 GEMM waiting
on the landing flags, re-gather in backward, per-unit reduce-scatter on the side stream).  Losses and final
parameters must agree to bf16 rounding, and the sharded run must hold 1/world of the large matrices.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from tah_b200.ops import cuda as K
    from tah_b200.parallel.fsdp import FsdpAdamW, shard_model
    from tah_b200.parallel.zero import ZeroAdamW
    from tests.helpers import tiny_tah

    g = torch.Generator().manual_seed(3)
    batches = []
    for _ in range(3):
        ids = torch.randint(0, 1024, (world, 2, 64), generator=g)
        hard = (torch.rand(world, 2, 64, generator=g) < 0.3).long() + 1
        batches.append((ids.to(dev), hard.to(dev)))
    ok = True
    # (multimem stores?, gradient checkpointing?): the checkpointed layers recompute their forward inside the backward
    # pass, after the backward hook has made the unit resident again
    for use_mc, ckpt in ((False, False), (True, False), (True, True)):
        losses, params, mem = {}, {}, {}
        for mode in ("zero2", "zero3"):
            torch.cuda.synchronize()
            model = tiny_tah(seed=0, dtype=torch.bfloat16).to(dev)
            model.train()
            if ckpt:
                model.gradient_checkpointing_enable()
            if mode == "zero3":
                st = shard_model(model, dist.group.WORLD, dev, min_shard_numel=1 << 12, use_multicast=use_mc)
                opt = FsdpAdamW(model, lr=1e-3, weight_decay=0.01, max_grad_norm=1.0, use_multicast=use_mc)
                mem[mode] = sum(u.shard_param.numel() * 2 for u in st.units)
                full = st.sharded_param_bytes()
            else:
                opt = ZeroAdamW(model.parameters(), lr=1e-3, weight_decay=0.01, max_grad_norm=1.0, use_multicast=use_mc)
            ls = []
            for ids, hard in batches:
                for micro in range(2):
                    o = model(ids[rank, micro:micro + 1], labels=ids[rank, micro:micro + 1],
                              iter_count_labels=hard[rank, micro:micro + 1])
                    (o.loss / 2).backward()
                    ls.append(float(o.loss))
                opt.step()
                opt.zero_grad()
                torch.cuda.synchronize()
                K.check_status(dev)
            losses[mode] = ls
            if mode == "zero3":
                with model._fsdp.materialized():
                    params[mode] = {n: p.detach().float().clone() for n, p in model.named_parameters()}
                stats = dict(model._fsdp.stats)
            else:
                params[mode] = {n: p.detach().float().clone() for n, p in model.named_parameters()}
            del model, opt
        perr = max(float((params["zero2"][n] - params["zero3"][n]).abs().max()) for n in params["zero2"])
        lerr = max(abs(a - b) for a, b in zip(losses["zero2"], losses["zero3"]))
        good = perr < 2e-2 and lerr < 5e-2 and mem["zero3"] * world == full and stats["prefetched"] > 0
        ok = ok and good
        if rank == 0:
            print(f"fsdp world={world} multicast={use_mc} checkpointing={ckpt}: param err {perr:.2e}, loss err {lerr:.2e}, local shard "
                  f"{mem['zero3']} of {full} bytes, stats {stats} {'ok' if good else 'BAD'}")
        dist.barrier()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    passed = int(flag.item()) == 1
    dist.barrier()
    if rank == 0:
        print("FSDP_WORKER_PASS" if passed else "FSDP_WORKER_FAIL")
    sys.stdout.flush()
    os._exit(0 if passed else 1)


if __name__ == "__main__":
    main()
