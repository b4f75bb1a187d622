"""Framework model vs the dense fp32 oracle (tiny TaH: 4 layers, H 256, 4q/2kv heads, hd 64,
I 768, V 1024, LoRA r 8, max_iter 2, batch 2 x seq 128, hard labels Bernoulli(0.06))."""
import torch

from tests.helpers import oracle_weights, tiny_tah
from tests.oracle import tah_oracle as orc


def _data(seed=0, B=2, T=128, p=0.06):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 1024, (B, T), generator=g)
    hard = (torch.rand(B, T, generator=g) < p).long() + 1
    return ids, hard


def test_forward_matches_oracle():
    model = tiny_tah()
    model.eval()
    ids, hard = _data()
    w = oracle_weights(model)
    with torch.no_grad():
        out = model(ids, labels=ids, iter_count_labels=hard)
        ref = orc.tah_forward(w, ids, max_iter=2, topk=100, labels=ids, iter_count_labels=hard)
    assert torch.equal(out.iter_count, ref["iter_count"])
    assert (out.iter_count == 2).sum() > 0
    torch.testing.assert_close(out.logits, ref["logits"], atol=2e-4, rtol=1e-4)
    torch.testing.assert_close(out.loss, ref["loss"], atol=1e-5, rtol=1e-5)


def test_left_padding_and_attention_mask():
    model = tiny_tah()
    model.eval()
    ids, hard = _data(seed=1, T=48)
    attn = torch.ones_like(ids)
    attn[0, :7] = 0
    attn[1, :19] = 0
    w = oracle_weights(model)
    with torch.no_grad():
        out = model(ids, attention_mask=attn, labels=ids, iter_count_labels=hard)
        ref = orc.tah_forward(w, ids, max_iter=2, topk=100, attention_mask=attn, labels=ids, iter_count_labels=hard)
    assert torch.equal(out.iter_count, ref["iter_count"])
    keep = attn.bool()
    torch.testing.assert_close(out.logits[keep], ref["logits"][keep], atol=2e-4, rtol=1e-4)


def test_backward_and_adamw_step_match_oracle():
    model = tiny_tah()
    model.train()
    ids, hard = _data(seed=2)
    w = oracle_weights(model)
    out = model(ids, labels=ids, iter_count_labels=hard)
    out.loss.backward()
    ref = orc.tah_forward(w, ids, max_iter=2, topk=100, labels=ids, iter_count_labels=hard)
    ref["loss"].backward()
    torch.testing.assert_close(out.loss.detach(), ref["loss"].detach(), atol=1e-5, rtol=1e-5)
    base = model.simple_base_model
    # embedding gradient collects three uses: lookup, tied LM head, soft-embedding mix
    torch.testing.assert_close(base.model.embed_tokens.weight.grad, w.sd["model.embed_tokens.weight"].grad,
                               atol=1e-5, rtol=1e-3)
    l0 = base.model.layers[0]
    gq = w.sd["model.layers.0.self_attn.q_proj.weight"].grad
    gk = w.sd["model.layers.0.self_attn.k_proj.weight"].grad
    gv = w.sd["model.layers.0.self_attn.v_proj.weight"].grad
    torch.testing.assert_close(l0.self_attn.qkv_proj.weight.grad, torch.cat([gq, gk, gv]), atol=1e-5, rtol=1e-3)
    # pass-1 attention back-propagates into pass-0 K/V: the LoRA factors of layer 0's k_proj only see pass 1,
    # while the base k_proj sees both
    ga = w.lora["base_model.model.model.layers.0.self_attn.k_proj.lora_A.weight"].grad
    r = base.lora.r
    torch.testing.assert_close(l0.self_attn.qkv_proj.lora_A.grad[r:2 * r], ga, atol=1e-5, rtol=1e-3)
    gd = w.lora["base_model.model.model.layers.3.mlp.down_proj.lora_B.weight"].grad
    torch.testing.assert_close(base.model.layers[3].mlp.down_proj.lora_B[0].grad, gd, atol=1e-5, rtol=1e-3)
    # one AdamW step (lr 1e-4) on both sides, then the forward must still agree
    opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=1e-4)
    opt.step()
    oopt = torch.optim.AdamW(list(w.sd.values()) + list(w.lora.values()), lr=1e-4)
    oopt.step()
    model.eval()
    with torch.no_grad():
        o2 = model(ids, labels=ids, iter_count_labels=hard)
        r2 = orc.tah_forward(w, ids, max_iter=2, topk=100, labels=ids, iter_count_labels=hard)
    torch.testing.assert_close(o2.loss, r2["loss"], atol=1e-4, rtol=1e-4)


def test_greedy_decode_matches_oracle():
    from tah_b200.model.utils import generate_loop
    model = tiny_tah(decider="BernoulliIterDecider", decider_kwargs=dict(p=0.06, seed=0))
    model.eval()
    ids, _ = _data(seed=3, T=24)
    B, T = ids.shape
    n_new = 32
    # fix the hard mask per step so that both sides see the same one
    g = torch.Generator().manual_seed(11)
    masks = {0: torch.rand(B, T, generator=g) < 0.06}
    for s in range(1, n_new + 1):
        masks[s] = torch.rand(B, 1, generator=g) < 0.3

    class Scripted(torch.nn.Module):
        threshold = torch.tensor(0.5)
        max_iter = 2

        def __init__(self):
            super().__init__()
            self.step = 0

        def forward(self, logits, iter_depth, **kw):
            n = logits.shape[0]
            if iter_depth >= 2:
                return torch.zeros(n, dtype=torch.bool), torch.zeros(n)
            m = masks[self.step].reshape(-1)
            self.step += 1
            return m, torch.zeros(n)

    model.iter_decider = model.eval_iter_decider = Scripted()
    toks, _ = generate_loop(model, None, {"input_ids": ids}, max_new_tokens=n_new, do_sample=False, verbose=False)
    w = oracle_weights(model)
    ref = orc.greedy_decode(w, ids, n_new, max_iter=2, topk=100, hard_mask_fn=lambda step, shape: masks[step])
    assert torch.equal(torch.tensor(toks), ref)
