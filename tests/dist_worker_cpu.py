"""CPU (gloo) worker for the multi-process tests: ``python dist_worker_cpu.py <case> <out.json>`` under torchrun."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def case_zero(out):
    """N-rank ZeroAdamW on each rank's micro-batch == single-process AdamW on the global batch."""
    from tah_b200.parallel.zero import ZeroAdamW
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    lin = torch.nn.Sequential(torch.nn.Linear(7, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
    ref = torch.nn.Sequential(torch.nn.Linear(7, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
    ref.load_state_dict(lin.state_dict())
    opt = ZeroAdamW(lin.parameters(), lr=1e-2, weight_decay=0.01, max_grad_norm=0.5)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    g = torch.Generator().manual_seed(1)
    for step in range(4):
        x, y = torch.randn(world, 6, 7, generator=g), torch.randn(world, 6, 3, generator=g)
        loss = ((lin(x[rank]) - y[rank]) ** 2).mean()
        loss.backward()
        gn = opt.step()
        opt.zero_grad()
        rl = sum(((ref(x[r]) - y[r]) ** 2).mean() for r in range(world)) / world
        rl.backward()
        rgn = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        ropt.step()
        ropt.zero_grad()
        assert abs(float(gn) - float(rgn)) < 1e-5, (float(gn), float(rgn))
    err = max(float((a - b).abs().max()) for a, b in zip(lin.parameters(), ref.parameters()))
    sd = opt.state_dict()
    opt.load_state_dict(sd)
    out.update(err=err, shard=opt.hi - opt.lo, numel=opt.numel)
    assert err < 1e-5, err


def case_trainer(out):
    """The trainer on N ranks follows the same loss curve as on one (same global data, ZeRO optimizer)."""
    from tah_b200.train import CustomTaHDataCollator, CustomTaHTrainer, TaHTrainingArguments
    from tests.helpers import tiny_tah
    rank, world = dist.get_rank(), dist.get_world_size()
    model = tiny_tah(seed=0)
    g = torch.Generator().manual_seed(3)
    rows = []
    for _ in range(8):
        ids = torch.randint(0, 1024, (24,), generator=g).tolist()
        hard = [1] * 24
        hard[7] = 2
        rows.append(dict(input_ids=ids, attention_mask=[1] * 24, labels=[-100] * 3 + ids[3:], iter_count_labels=hard))
    tp = int(os.environ.get("TAH_TEST_TP", "1"))          # tensor-parallel size: world / tp data-parallel replicas
    dp = world // tp
    args = TaHTrainingArguments(output_dir=os.environ["TAH_TEST_OUT"], per_device_train_batch_size=1,
                                gradient_accumulation_steps=4 // dp if dp <= 4 else 1, learning_rate=1e-3,
                                max_grad_norm=1.0, num_train_epochs=1, logging_steps=1, save_strategy="no", seed=0,
                                tp_size=tp)
    tr = CustomTaHTrainer(model, args, rows, None, data_collator=CustomTaHDataCollator(None, pad_token_id=0))
    tr.train()
    out.update(losses=[h["loss"] for h in tr.state.log_history if "loss" in h], steps=tr.state.global_step)
    if tp > 1:
        # saving gathers the shards: the written checkpoint has the full shapes again
        tr.save_model(os.path.join(os.environ["TAH_TEST_OUT"], "final"))
        dist.barrier()
        if rank == 0:
            from safetensors import safe_open
            with safe_open(os.path.join(os.environ["TAH_TEST_OUT"], "final", "model.safetensors"), "pt") as fh:
                out.update(saved_q_rows=int(fh.get_tensor("model.layers.0.self_attn.q_proj.weight").shape[0]),
                           saved_down_cols=int(fh.get_tensor("model.layers.0.mlp.down_proj.weight").shape[1]))


def case_fsdp(out):
    """Parameter-sharded training step (ZeRO-3 schedule on gloo) == ZeroAdamW step on the same data, and the
    per-rank parameter storage is 1/world of the large matrices."""
    from tah_b200.parallel.fsdp import FsdpAdamW, shard_model
    from tah_b200.parallel.zero import ZeroAdamW
    from tests.helpers import tiny_tah
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(3)
    batches = []
    for _ in range(3):
        ids = torch.randint(0, 1024, (world, 2, 24), generator=g)
        hard = (torch.rand(world, 2, 24, generator=g) < 0.3).long() + 1
        batches.append((ids, hard))
    losses = {}
    params = {}
    for mode in ("zero2", "zero3"):
        model = tiny_tah(seed=0)
        model.train()
        if mode == "zero3":
            st = shard_model(model, dist.group.WORLD, torch.device("cpu"), min_shard_numel=1 << 12)
            opt = FsdpAdamW(model, lr=1e-3, weight_decay=0.01, max_grad_norm=1.0)
            out.update(units=len(st.units), sharded_bytes=st.sharded_param_bytes(),
                       local_shard_bytes=sum(u.shard_param.numel() * u.shard_param.element_size() for u in st.units))
        else:
            opt = ZeroAdamW(model.parameters(), lr=1e-3, weight_decay=0.01, max_grad_norm=1.0)
        ls = []
        for ids, hard in batches:
            for micro in range(2):                      # two micro-batches per step: gradient accumulation
                o = model(ids[rank, micro:micro + 1], labels=ids[rank, micro:micro + 1], iter_count_labels=hard[rank, micro:micro + 1])
                (o.loss / 2).backward()
                ls.append(float(o.loss))
            opt.step()
            opt.zero_grad()
        losses[mode] = ls
        if mode == "zero3":
            with model._fsdp.materialized():
                params[mode] = {n: p.detach().clone() for n, p in model.named_parameters()}
            out.update(stats=model._fsdp.stats)
        else:
            params[mode] = {n: p.detach().clone() for n, p in model.named_parameters()}
    err = max(float((params["zero2"][n] - params["zero3"][n]).abs().max()) for n in params["zero2"])
    dl = max(abs(a - b) for a, b in zip(losses["zero2"], losses["zero3"]))
    out.update(param_err=err, loss_err=dl, losses=losses["zero3"])
    assert err < 2e-5 and dl < 1e-4, (err, dl)


def case_tp_train(out):
    """Tensor-parallel training (heads / MLP channels of every layer sharded over the group) == the same steps on
    the full model: losses, clipped gradient norm and final (gathered) parameters.  World 2: pure TP; world 4: two
    data-parallel replicas of a TP pair, the same global batch as two unsharded ranks."""
    from tah_b200.parallel.tp_train import TPOptimizer, shard_model_tp, tp_dp_groups
    from tah_b200.parallel.zero import ZeroAdamW
    from tests.helpers import tiny_tah
    rank, world = dist.get_rank(), dist.get_world_size()
    tp_group, dp_group, tp_rank, dp_rank = tp_dp_groups(2)
    dp = world // 2
    g = torch.Generator().manual_seed(5)
    batches = []
    for _ in range(3):
        ids = torch.randint(0, 1024, (dp, 2, 24), generator=g)
        hard = (torch.rand(dp, 2, 24, generator=g) < 0.3).long() + 1
        batches.append((ids, hard))
    losses, params, norms = {}, {}, {}
    for mode in ("full", "tp"):
        model = tiny_tah(seed=0, max_iter=2)
        model.train()
        if mode == "tp":
            st = shard_model_tp(model, tp_group)
            opt = TPOptimizer(ZeroAdamW(model.parameters(), group=dp_group, lr=1e-3, weight_decay=0.01, max_grad_norm=0.3), st)
            out.update(sharded=len(st.sharded), partial=len(st.partial_grad),
                       local_fraction=sum(p.numel() for p, _, _ in st.sharded) / max(1, sum(
                           st.gather_full(p, how, sp).numel() for p, how, sp in st.sharded)))
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
        losses[mode], norms[mode] = ls, ns
        if mode == "tp":
            with st.materialized():
                params[mode] = {n: p.detach().clone() for n, p in model.named_parameters()}
                # the gathered model is a valid full model again: one forward must run
                model.eval()
                with torch.no_grad():
                    for h in st.hooks:
                        h.remove()
                    full_loss = float(model(batches[0][0][0, :1], labels=batches[0][0][0, :1]).loss)
            out.update(full_loss_after=full_loss)
        else:
            params[mode] = {n: p.detach().clone() for n, p in model.named_parameters()}
    err = max(float((params["full"][n] - params["tp"][n]).abs().max()) for n in params["full"])
    dl = max(abs(a - b) for a, b in zip(losses["full"], losses["tp"]))
    dn = max(abs(a - b) / max(a, 1e-6) for a, b in zip(norms["full"], norms["tp"]))
    out.update(param_err=err, loss_err=dl, norm_err=dn, norms=norms["tp"], losses=losses["tp"])
    assert err < 5e-5 and dl < 1e-4 and dn < 1e-4, (err, dl, dn)


def case_heartbeat(out):
    """Rank 1 leaves between steps; rank 0 learns of it from the store before its next collective."""
    from tah_b200.utils.failure import RankFailure, RankHeartbeat
    rank, world = dist.get_rank(), dist.get_world_size()
    store = dist.distributed_c10d._get_default_store()
    hb = RankHeartbeat(store, rank, world, interval_s=0.1).start()
    t = torch.ones(1)
    dist.all_reduce(t)                       # step 1: everyone is here
    if rank == 1:
        hb.stop()
        out.update(left=True)
        return "leave"
    detected, t0 = None, time.time()
    while time.time() - t0 < 10:
        try:
            hb.check_peers(timeout_s=0.6)
        except RankFailure as exc:
            detected = exc.dead
            break
        time.sleep(0.1)
    hb.stop()
    out.update(detected=detected, seconds=time.time() - t0)
    assert detected == [1]
    return "leave"


def case_collective_timeout(out):
    """A rank that never joins turns the others' next collective into an error after the group timeout."""
    rank = dist.get_rank()
    if rank == 1:
        time.sleep(6)
        return "leave"
    t0 = time.time()
    try:
        dist.all_reduce(torch.ones(1))
        out.update(raised=False)
    except Exception as exc:
        out.update(raised=True, seconds=time.time() - t0, kind=type(exc).__name__)
    return "leave"


if __name__ == "__main__":
    import datetime
    case, path = sys.argv[1], sys.argv[2]
    timeout = datetime.timedelta(seconds=3 if case == "collective_timeout" else 120)
    dist.init_process_group("gloo", timeout=timeout)
    result = {}
    how = globals()[f"case_{case}"](result)
    with open(f"{path}.rank{dist.get_rank()}", "w") as fh:
        json.dump(result, fh)
    if how == "leave":
        os._exit(0)
    dist.barrier()
    dist.destroy_process_group()
