"""Worker for the multi-GPU tensor-parallel training test (launched by torchrun from test_fsdp_gpu.py).

On ``WORLD_SIZE`` GPUs (TP pairs x data-parallel replicas): the same tiny TaH model is trained for a few steps
unsharded (ZeRO-2 over the data-parallel group) and with its layers sharded over the tensor-parallel group
(``shard_model_tp`` + ``TPOptimizer``), through the CUDA kernel path in bf16.  Losses, clipped gradient norms and
final (gathered) parameters must agree to bf16 rounding.
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
    from tah_b200.parallel.tp_train import TPOptimizer, shard_model_tp, tp_dp_groups
    from tah_b200.parallel.zero import ZeroAdamW
    from tests.helpers import tiny_tah

    tp_group, dp_group, tp_rank, dp_rank = tp_dp_groups(2)
    dp = world // 2
    g = torch.Generator().manual_seed(3)
    batches = []
    for _ in range(3):
        ids = torch.randint(0, 1024, (dp, 2, 64), generator=g)
        hard = (torch.rand(dp, 2, 64, generator=g) < 0.3).long() + 1
        batches.append((ids.to(dev), hard.to(dev)))
    ok = True
    for ckpt in (False, True):
        losses, params, norms = {}, {}, {}
        for mode in ("full", "tp"):
            model = tiny_tah(seed=0, dtype=torch.bfloat16).to(dev)
            model.train()
            if ckpt:
                model.gradient_checkpointing_enable()
            if mode == "tp":
                st = shard_model_tp(model, tp_group)
                opt = TPOptimizer(ZeroAdamW(model.parameters(), group=dp_group, lr=1e-3, weight_decay=0.01, max_grad_norm=0.3), st)
            else:
                opt = ZeroAdamW(model.parameters(), group=dp_group, lr=1e-3, weight_decay=0.01, max_grad_norm=0.3)
            ls, ns = [], []
            for ids, hard in batches:
                for micro in range(2):
                    o = model(ids[dp_rank, micro:micro + 1], labels=ids[dp_rank, micro:micro + 1],
                              iter_count_labels=hard[dp_rank, micro:micro + 1])
                    (o.loss / 2).backward()
                    ls.append(float(o.loss))
                ns.append(float(opt.step()))
                opt.zero_grad()
                torch.cuda.synchronize()
                K.check_status(dev)
            losses[mode], norms[mode] = ls, ns
            if mode == "tp":
                with st.materialized():
                    params[mode] = {n: p.detach().float().clone() for n, p in model.named_parameters()}
            else:
                params[mode] = {n: p.detach().float().clone() for n, p in model.named_parameters()}
            del model, opt
        perr = max(float((params["full"][n] - params["tp"][n]).abs().max()) for n in params["full"])
        lerr = max(abs(a - b) for a, b in zip(losses["full"], losses["tp"]))
        nerr = max(abs(a - b) / max(a, 1e-6) for a, b in zip(norms["full"], norms["tp"]))
        good = perr < 2e-2 and lerr < 5e-2 and nerr < 3e-2
        ok = ok and good
        if rank == 0:
            print(f"tp-train world={world} (tp 2 x dp {dp}) checkpointing={ckpt}: param err {perr:.2e}, loss err {lerr:.2e}, "
                  f"grad-norm rel err {nerr:.2e} {'ok' if good else 'BAD'}")
        dist.barrier()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    passed = int(flag.item()) == 1
    dist.barrier()
    if rank == 0:
        print("TP_TRAIN_WORKER_PASS" if passed else "TP_TRAIN_WORKER_FAIL")
    sys.stdout.flush()
    os._exit(0 if passed else 1)


if __name__ == "__main__":
    main()
