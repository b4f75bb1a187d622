"""CPU unit tests of the model layer: config, compaction, mask, deciders, losses, sampler, data glue."""
import json
import os

import pytest
import torch

from tah_b200 import TaHConfig, TaHForCausalLM
from tah_b200.model.iter_decider import (IterLabelDecider, MLPIterDecider, load_iter_decider, save_iter_decider)
from tah_b200.model.loss import IterDeciderLoss, NextTokenPredLoss, fixed_cross_entropy
from tah_b200.model.tah_config import decode_config, encode_config, resolve_config, save_config
from tah_b200.model.tah_model import ActiveSet, gather_active, scatter_back, topk_softmax_input_update
from tah_b200.ops import torch_ref
from tests.helpers import tiny_tah


# ---- config -----------------------------------------------------------------------------------------
def test_config_json_sentinels_round_trip():
    cfg = {"iter_decider_kwargs": {"dtype": torch.bfloat16, "cls": torch.nn.Linear, "dims": [1, 2]}, "max_iter": 2}
    enc = encode_config(cfg)
    assert enc["iter_decider_kwargs"]["dtype"] == {"__dtype__": True, "__str__": "torch.bfloat16"}
    assert enc["iter_decider_kwargs"]["cls"]["__type__"] is True
    dec = decode_config(json.loads(json.dumps(enc)))
    assert dec["iter_decider_kwargs"]["dtype"] is torch.bfloat16
    assert dec["iter_decider_kwargs"]["cls"] is torch.nn.Linear


def test_config_merge_precedence(tmp_path):
    saved = TaHConfig(max_iter=2, iter_decider="MLPIterDecider", iter_decider_kwargs={"threshold": 0.8},
                      adapter_kwargs={"r": 32})
    save_config(saved, str(tmp_path))
    # unknown keys in an old file are ignored
    raw = json.load(open(tmp_path / "tah_config.json"))
    raw["iter_attention_mode"] = "duo"
    json.dump(raw, open(tmp_path / "tah_config.json", "w"))
    over = TaHConfig(iter_decider_kwargs={"threshold": 0.9}, max_iter=None, adapter_kwargs={})
    got = resolve_config(str(tmp_path), over)
    assert got.max_iter == 2 and got.iter_decider == "MLPIterDecider"
    assert got.iter_decider_kwargs == {"threshold": 0.9}          # non-empty override wins
    assert got.adapter_kwargs == {"r": 32}                         # {} means "use saved"
    assert resolve_config(str(tmp_path), None).iter_decider_kwargs == {"threshold": 0.8}


# ---- compaction -------------------------------------------------------------------------------------
def test_gather_scatter_round_trip():
    g = torch.Generator().manual_seed(0)
    for _ in range(20):
        B, S = int(torch.randint(1, 5, (1,), generator=g)), int(torch.randint(1, 12, (1,), generator=g))
        mask = torch.rand(B, S, generator=g) < 0.4
        x = torch.randn(B, S, 3, generator=g)
        ids = torch.randint(0, 50, (B, S), generator=g)
        pad, gx, gi, none = gather_active(mask, x, ids, None, pad_value=0)
        assert none is None and gx.shape[1] == int(mask.sum(1).max()) and pad.shape == gx.shape[:2]
        for b in range(B):
            n = int(mask[b].sum())
            assert torch.equal(gx[b, :n], x[b][mask[b]]) and torch.equal(gi[b, :n], ids[b][mask[b]])
            assert (gx[b, n:] == 0).all() and pad[b, n:].all() and not pad[b, :n].any()
        back = scatter_back(mask, gx, torch.full_like(x, -7.0))
        assert torch.equal(back[mask], x[mask]) and (back[~mask] == -7).all()
        sel = torch.rand(B, S, generator=g) < 0.5
        part = scatter_back(mask, gx, torch.zeros_like(x), assignment_mask=sel)
        assert torch.equal(part[mask & sel], x[mask & sel]) and (part[~(mask & sel)] == 0).all()


def test_active_set_empty():
    act = ActiveSet(torch.zeros(2, 5, dtype=torch.bool))
    assert act.n == 0 and act.width == 0


# ---- duo-causal predicate --------------------------------------------------------------------------
def test_duo_mask_matches_brute_force():
    g = torch.Generator().manual_seed(1)
    B, Tq, Tk = 2, 5, 9
    qp, kp = torch.randint(0, 6, (B, Tq), generator=g), torch.randint(0, 6, (B, Tk), generator=g)
    kvalid = (torch.rand(B, Tk, generator=g) < 0.8).long()
    qd, kd = torch.randint(0, 3, (B, Tq), generator=g), torch.randint(0, 3, (B, Tk), generator=g)
    m = torch_ref.duo_mask(qp, kp, kvalid, qd, kd)
    for b in range(B):
        for i in range(Tq):
            for j in range(Tk):
                want = bool(kp[b, j] <= qp[b, i] and kd[b, j] <= qd[b, i] and kvalid[b, j] == 1)
                assert bool(m[b, i, j]) == want


def test_depth0_queries_never_see_deeper_kv():
    model = tiny_tah().eval()
    ids = torch.randint(0, 1024, (1, 10))
    labels_hard = torch.ones(1, 10, dtype=torch.long)
    labels_hard[0, 3] = 2
    with torch.no_grad():
        # no `labels`: with labels the model forces one continuation when the decider stops everything
        a = model(ids, iter_count_labels=labels_hard)
        b = model(ids, iter_count_labels=torch.ones(1, 10, dtype=torch.long))
    # only the hard token's own logits change: depth-0 passes of later tokens ignore its depth-1 K/V
    same = torch.ones(10, dtype=torch.bool)
    same[3] = False
    torch.testing.assert_close(a.logits[0, same], b.logits[0, same])
    assert not torch.allclose(a.logits[0, 3], b.logits[0, 3])
    assert a.iter_count.tolist() == [[1, 1, 1, 2, 1, 1, 1, 1, 1, 1]]


# ---- soft embedding / deciders ----------------------------------------------------------------------
def test_topk_softmax_input_update():
    E = torch.randn(50, 8)
    logits = torch.randn(3, 50)
    out = topk_softmax_input_update(logits, E, 5)
    v, i = logits.topk(5, -1)
    ref = (torch.softmax(v, -1)[..., None] * E[i]).sum(-2)
    torch.testing.assert_close(out, ref)
    assert topk_softmax_input_update(logits, E, 500).shape == (3, 8)     # k is clipped to the vocabulary


def test_label_decider_rules():
    d = IterLabelDecider(max_iter=3)
    logits = torch.zeros(4, 7)
    labels = torch.tensor([1, 2, 3, -100])
    dec, z = d(logits, 1, iter_count_labels=labels)
    assert dec.tolist() == [False, True, True, False] and (z == 0).all()
    dec, z = d(logits, 3, iter_count_labels=labels)
    assert not dec.any() and (z == -10).all()
    dec, _ = d(logits, 1)
    assert not dec.any()


def test_mlp_decider_features_keys_and_persistence(tmp_path):
    torch.manual_seed(0)
    d = MLPIterDecider(topk=4, hidden_states_size=8, hidden_states_layer_nums=[0, 2], hidden_dims=[6, 6],
                       dropout_rate=0.0, threshold=0.8, max_iter=2, dtype=torch.float32).eval()
    keys = set(d.state_dict())
    assert {"threshold", "logits_projection.weight", "combined_projection.bias", "backbone.input_projection.weight",
            "backbone.blocks.0.layer_norm.weight", "backbone.blocks.0.mlp.0.weight", "backbone.blocks.0.mlp.3.bias",
            "backbone.output_layer.0.weight", "backbone.output_layer.1.weight"} <= keys
    logits, hs = torch.randn(5, 20), torch.randn(5, 3, 8)
    dec, z = d(logits, 1, all_hidden_states=hs)
    feats = torch.cat([hs[:, 0], hs[:, 2], d.logits_projection(logits.topk(4, -1).values)], -1)   # taps first, then logits
    torch.testing.assert_close(z, d.backbone(d.combined_projection(feats)).squeeze(-1))
    assert torch.equal(dec, torch.sigmoid(z) > 0.8)
    dec2, z2 = d(logits, 1, tapped_hidden_states=torch.cat([hs[:, 0], hs[:, 2]], -1))
    torch.testing.assert_close(z2, z)
    assert not d(logits, 2, all_hidden_states=hs)[0].any()
    with pytest.raises(ValueError):
        d(logits, 1, all_hidden_states=torch.randn(5, 2, 8))
    save_iter_decider(d, str(tmp_path))
    blob = torch.load(tmp_path / "iter_decider.bin", weights_only=False)
    assert blob["class"] == "MLPIterDecider" and blob["init_args"]["threshold"] == 0.8
    args = dict(blob["init_args"], threshold=0.9)
    d2 = load_iter_decider(str(tmp_path), class_name="MLPIterDecider", init_args=args).eval()
    assert abs(float(d2.threshold) - 0.9) < 1e-6                     # configured value beats the stored one
    torch.testing.assert_close(d2(logits, 1, all_hidden_states=hs)[1], z)


# ---- losses -----------------------------------------------------------------------------------------
def test_fixed_cross_entropy_normalisation():
    x, t = torch.randn(6, 9), torch.tensor([1, 2, -100, 4, -100, 0])
    ref_sum = torch.nn.functional.cross_entropy(x, t, ignore_index=-100, reduction="sum")
    torch.testing.assert_close(fixed_cross_entropy(x, t, num_items_in_batch=10), ref_sum / 10)
    torch.testing.assert_close(fixed_cross_entropy(x, t), ref_sum / 4)


def test_iter_decider_loss_scale_and_accuracy():
    loss = IterDeciderLoss(pos_weight=2.0, skip_last_iter=True, max_iter=2)
    B, T = 2, 4
    loss.prepare_loss(B, T, torch.device("cpu"), torch.float32)
    active_index = torch.arange(B * T)
    valid = torch.tensor([1, 1, 1, 0, 1, 1, 1, 1], dtype=torch.bool)
    labels = torch.tensor([1, 2, -100, 1, 2, 1, 1, 1])
    z = torch.tensor([-1.0, 2.0, 0.3, 0.5, -0.2, 0.1, -3.0])        # one per valid token
    loss.intra_iter_loss_func(active_index=active_index, active_valid=valid, continue_logits=z, iter_depth=1,
                              active_iter_count_labels=labels, iter_decider_threshold=0.5)
    lab_v = labels[valid]
    use = lab_v != -100
    bce = torch.nn.functional.binary_cross_entropy_with_logits(z[use], (lab_v[use] > 1).float(),
                                                               pos_weight=torch.tensor(2.0))
    iter_count = torch.ones(B, T, dtype=torch.long)
    full_labels = torch.tensor([[1, 2, 0, 1], [2, 1, 1, 1]])          # max-merged dense view: zeros, not -100
    out = loss.final_loss_func(torch.zeros(B, T, 3), None, iter_count, iter_count_labels=full_labels)
    # every processed position counts in the mean (the reference's scale quirk): the sum of the spread
    # per-token shares equals the mean BCE, divided by all B*T positions
    torch.testing.assert_close(out, bce / (B * T))
    loss.prepare_loss(B, T, torch.device("cpu"), torch.float32)
    loss.intra_iter_loss_func(active_index=active_index, active_valid=valid, continue_logits=z, iter_depth=2,
                              active_iter_count_labels=labels)
    assert float(loss.final_loss_func(torch.zeros(B, T, 3), None, iter_count, iter_count_labels=full_labels)) == 0.0
    with pytest.raises(ValueError):
        IterDeciderLoss(skip_last_iter=True)


def test_next_token_loss_matches_shifted_ce():
    model = tiny_tah(max_iter=1).eval()
    ids = torch.randint(0, 1024, (2, 12))
    labels = ids.clone()
    labels[:, :4] = -100
    with torch.no_grad():
        out = model(ids, labels=labels)
    ref = torch.nn.functional.cross_entropy(out.logits[:, :-1].reshape(-1, 1024).float(), labels[:, 1:].reshape(-1),
                                            ignore_index=-100)
    torch.testing.assert_close(out.loss, ref)
    assert isinstance(model.train_loss, NextTokenPredLoss)


# ---- sampler ----------------------------------------------------------------------------------------
def test_sampler_filters_in_order():
    logits = torch.log(torch.tensor([[0.5, 0.25, 0.15, 0.06, 0.04]]))
    g = torch.Generator().manual_seed(0)
    assert int(torch_ref.sample(logits, do_sample=False)) == 0
    draws = torch.stack([torch_ref.sample(logits, top_k=2, generator=g) for _ in range(200)])
    assert set(draws.flatten().tolist()) <= {0, 1}
    draws = torch.stack([torch_ref.sample(logits, top_p=0.7, generator=g) for _ in range(200)])
    assert set(draws.flatten().tolist()) <= {0, 1}                    # the token crossing top_p stays
    draws = torch.stack([torch_ref.sample(logits, min_p=0.4, generator=g) for _ in range(200)])
    assert set(draws.flatten().tolist()) <= {0, 1}
    draws = torch.stack([torch_ref.sample(logits, temperature=0.05, generator=g) for _ in range(50)])
    assert (draws == 0).all()


# ---- forward bookkeeping ----------------------------------------------------------------------------
def test_force_one_continuation_and_uniform_passes():
    model = tiny_tah(decider="MLPIterDecider",
                     decider_kwargs=dict(topk=10, hidden_states_size=256, hidden_states_layer_nums=[1, 4],
                                         hidden_dims=[32, 32], dropout_rate=0.0, threshold=0.999999, dtype=torch.float32),
                     train_loss="IterDeciderLoss", train_loss_kwargs=dict(pos_weight=5.4, skip_last_iter=True))
    model.train()
    ids = torch.randint(0, 1024, (2, 16))
    hard = torch.ones(2, 16, dtype=torch.long)
    out = model(ids, labels=ids, iter_count_labels=hard)
    assert int((out.iter_count == 2).sum()) == 1                      # exactly one forced continuation
    out.loss.backward()
    assert model.iter_decider.combined_projection.weight.grad.abs().sum() > 0
    model.eval()
    with torch.no_grad():
        out = model(ids)
    assert int(out.iter_count.max()) == 1
    model.uniform_passes = True
    with torch.no_grad():
        out2 = model(ids)
    torch.testing.assert_close(out2.logits, out.logits)


def test_padding_positions_count_one_pass():
    model = tiny_tah().eval()
    ids = torch.randint(0, 1024, (2, 8))
    attn = torch.ones(2, 8, dtype=torch.long)
    attn[0, :3] = 0
    hard = torch.full((2, 8), 2)
    with torch.no_grad():
        out = model(ids, attention_mask=attn, labels=ids, iter_count_labels=hard)
    assert out.iter_count[0, :3].tolist() == [1, 1, 1] and (out.iter_count[attn.bool()] == 2).all()


def test_segment_meta_matches_duo_mask_cpu():
    """The (base, count) prefixes handed to the tensor-core attention kernels describe exactly the keys
    that the duo-causal mask allows, for left-padded and right-padded batches and a sparse deeper pass."""
    import torch
    from tah_b200.ops.autograd_ops import SegmentMeta
    from tah_b200.ops.torch_ref import duo_mask
    B, T = 3, 11
    for pad_left in (True, False):
        lens = torch.tensor([11, 7, 3])
        valid0 = torch.zeros(B, T, dtype=torch.long)
        for b, n in enumerate(lens.tolist()):
            if pad_left:
                valid0[b, T - n:] = 1
            else:
                valid0[b, :n] = 1
        pos0 = (valid0.cumsum(-1) - 1).clamp(min=0)
        # deeper pass: a subset of the valid tokens, packed to the left of a narrower block
        g = torch.Generator().manual_seed(3)
        act = (torch.rand(B, T, generator=g) < 0.5) & valid0.bool()
        act[:, -1] |= valid0[:, -1].bool()
        width = int(act.sum(1).max())
        pos1 = torch.zeros(B, width, dtype=torch.long)
        valid1 = torch.zeros(B, width, dtype=torch.long)
        for b in range(B):
            idx = act[b].nonzero().flatten()
            pos1[b, :idx.numel()] = pos0[b, idx]
            valid1[b, :idx.numel()] = 1
        # queries of the deeper pass see depth-0 keys and depth-1 keys
        meta = SegmentMeta(pos1, [pos0, pos1], [valid0, valid1], q_valid=valid1)
        for s, (kp, kv, Ts) in enumerate(((pos0, valid0, T), (pos1, valid1, width))):
            mask = duo_mask(pos1, kp, kv)                               # [B, width, Ts]
            base = meta.bases[s].view(B, width)
            cnt = meta.counts[s].view(B, width)
            for b in range(B):
                for i in range(width):
                    if not valid1[b, i]:
                        continue
                    want = mask[b, i].nonzero().flatten() + b * Ts
                    got = torch.arange(int(base[b, i]), int(base[b, i]) + int(cnt[b, i]))
                    assert torch.equal(want, got), (pad_left, s, b, i)
            # padding queries see nothing; the tiling bound never decreases along a sample's rows and
            # is never below the count
            assert (cnt[valid1 == 0] == 0).all()
            bound = meta.bounds[s].view(B, width)
            assert (bound[:, 1:] >= bound[:, :-1]).all() and (bound >= cnt).all()
        row0, nkeys, kidx0, qa, qb = meta.items[0]
        assert int(nkeys.sum()) == int(valid0.sum()) and torch.equal(qb - qa, torch.full_like(qa, width))


def test_attention_tiling_helpers_cpu():
    """Query tiles and key-block work items of the packed attention kernels (pure index arithmetic)."""
    import torch
    from tah_b200.ops.cuda import attn_kv_items, attn_tiles
    q0, qn = attn_tiles(torch.tensor([300, 0, 128, 5]))
    assert q0.tolist() == [0, 128, 256, 300, 428] and qn.tolist() == [128, 128, 44, 128, 5]
    row0, nkeys, kidx0, qa, qb = attn_kv_items(torch.tensor([260, 3]), torch.tensor([10, 500]), torch.tensor([7, 9]))
    assert row0.tolist() == [10, 138, 266, 500] and nkeys.tolist() == [128, 128, 4, 3]
    assert kidx0.tolist() == [0, 128, 256, 0]
    assert qa.tolist() == [0, 0, 0, 7] and qb.tolist() == [7, 7, 7, 16]


def test_gemm_planner_choices_cpu():
    """The split-K / tile planner (pure host arithmetic): legal plans, split-K for small-M long-K shapes,
    none for shapes that already fill the GPU."""
    from tah_b200.ops.cuda import _fits, plan_gemm
    for (M, F, Kd, R, dual) in [(256, 4096, 2048, 192, False), (256, 2048, 6144, 64, False), (64, 2048, 2048, 0, False),
                                (256, 6144, 2048, 128, True), (8192, 4096, 2048, 0, False), (1, 128, 128, 0, False)]:
        bn, s = plan_gemm(M, F, Kd, R, dual)
        assert bn in (16, 32, 64, 128, 256) and s in (1, 2, 4)
        assert s == 1 or (bn % s == 0 and (bn // s) % 16 == 0 and _fits(bn, s, 2 if dual else 1))
    assert plan_gemm(256, 2048, 6144)[1] > 1            # few feature tiles, long K: split
    assert plan_gemm(8192, 4096, 2048)[1] == 1          # 1024 CTAs already
    assert plan_gemm(256, 151936, 2048)[1] == 1         # LM head


def test_reference_import_names_resolve_to_this_package():
    """``import tah`` (the reference's package name) serves the same module objects as ``tah_b200``."""
    import importlib
    import tah
    import tah_b200
    assert tah.TaHForCausalLM is tah_b200.TaHForCausalLM
    for sub in ("model", "model.tah_model", "model.iter_decider", "model.loss", "model.utils", "model.causal_cache",
                "model.tah_config", "train", "utils", "evaluate", "evaluate.backends", "evaluate.jobs",
                "evaluate.datasets", "evaluate.matheval", "evaluate.codeeval"):
        assert importlib.import_module("tah." + sub) is importlib.import_module("tah_b200." + sub)
    from tah.model.tah_model import additive_logits_update, gather_active, scatter_back, topk_softmax_input_update  # noqa: F401
    from tah.model.utils import TaHForCasualLM_generate, sample_next_token, set_all_seeds  # noqa: F401
    from tah.train import CustomTaHDataCollator, CustomTaHTrainer, LoggerCallback, fixed_cross_entropy  # noqa: F401
    from tah.utils import preprocess_dataset  # noqa: F401
    from tah.evaluate.backends import cleanup, setup_backend, setup_hf, setup_sglang, setup_tah, time_inference, warmup  # noqa: F401


def test_zero_adamw_no_decay_group_matches_torch_param_groups():
    """Parameters named as no-decay (norm gains, biases) take no weight decay, like the two parameter groups of the
    HuggingFace trainer the reference builds on."""
    from tah_b200.parallel.zero import ZeroAdamW
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.LayerNorm(5), torch.nn.Linear(5, 3))
    ref = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.LayerNorm(5), torch.nn.Linear(5, 3))
    ref.load_state_dict(net.state_dict())
    nd = [p for n, p in net.named_parameters() if p.dim() < 2]
    opt = ZeroAdamW(net.parameters(), lr=1e-2, weight_decay=0.1, no_decay=nd)
    rnd = {id(p) for n, p in ref.named_parameters() if p.dim() < 2}
    ropt = torch.optim.AdamW([{"params": [p for p in ref.parameters() if id(p) not in rnd], "weight_decay": 0.1},
                              {"params": [p for p in ref.parameters() if id(p) in rnd], "weight_decay": 0.0}], lr=1e-2)
    for step in range(3):
        x = torch.randn(4, 6, generator=torch.Generator().manual_seed(step))
        net(x).pow(2).mean().backward()
        ref(x).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
        ropt.step()
        ropt.zero_grad()
    for (n, a), b in zip(net.named_parameters(), ref.parameters()):
        torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5, msg=n)


def test_zero_adamw_accumulates_micro_batch_gradients_in_fp32():
    """``accumulate()`` after every backward: the window's gradient is summed in fp32 and rounded to bf16 once, so
    sixteen micro-batches whose gradients differ by orders of magnitude keep their small terms."""
    from tah_b200.parallel.zero import ZeroAdamW
    torch.manual_seed(0)
    n = 4096
    grads = [torch.randn(n) * (1.0 if i == 0 else 2e-3) for i in range(16)]
    exact = torch.stack(grads).sum(0)

    def run(use_acc):
        p = torch.nn.Parameter(torch.zeros(n, dtype=torch.bfloat16))
        opt = ZeroAdamW([p], lr=1e-3, weight_decay=0.0, max_grad_norm=0.0)
        for g in grads:
            p.grad.add_(g.to(torch.bfloat16))            # what autograd does: accumulate into the 16-bit buffer
            if use_acc:
                opt.accumulate()
        opt._collect_stray_grads()
        opt._flush_accumulator()
        return opt.flat_grad[:n].float().clone()

    err_plain = (run(False) - exact).abs().mean()
    err_acc = (run(True) - exact).abs().mean()
    assert err_acc < 0.5 * err_plain                      # one rounding instead of sixteen
    assert err_acc < 2.5e-3                                # bf16 rounding of values of order one


def test_kv_cache_guard_pages(monkeypatch):
    from tah_b200.engine.kv_cache import CacheGeometry, PagedKVCache
    monkeypatch.setenv("TAH_B200_CANARY", "2")
    kv = PagedKVCache(CacheGeometry(2, 2, 64, 16), 3, 40, 2, device="cpu")
    assert kv.pool[0].shape[1] == kv.n_pages[0] + 2 and kv.check_guards()
    slots = kv.assign_prefill(0, torch.tensor([5, 17, 33]))
    assert int(slots.max()) < kv.n_pages[0] * 16            # slots never reach into the guard pages
    kv.pool[1][0, kv.n_pages[1], 0, 0, 0, 0] = 1.0
    assert not kv.check_guards()
    monkeypatch.delenv("TAH_B200_CANARY")
    assert PagedKVCache(CacheGeometry(2, 2, 64, 16), 3, 40, 2, device="cpu").check_guards()
