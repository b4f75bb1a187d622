"""This framework against the reference package itself (installed under ``baseline/_ref``), on CPU in fp32.

The reference imports ``peft``, which this image lacks; ``baseline/peft_standin`` supplies the three names it
uses.  The tests skip when the reference install is absent.  They check (a) that a checkpoint written by the
reference's ``save_pretrained`` loads here (and one written here loads there), and (b) that forward logits,
iteration counts, the loss and a greedy decode with a seeded hard-token decider agree.
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _purge_tah_modules():
    for name in [n for n in sys.modules if n == "tah" or n.startswith("tah.")]:
        del sys.modules[name]


@pytest.fixture
def reference():
    """Imports the reference's ``tah`` (not this repository's alias package of the same name) for one test and
    removes it again afterwards."""
    if not os.path.isdir(os.path.join(REF, "tah")):
        pytest.skip("reference package not installed under baseline/_ref")
    added = []
    try:
        import peft  # noqa: F401
    except ImportError:
        added.append(os.path.join(ROOT, "baseline", "peft_standin"))
    added.append(REF)
    _purge_tah_modules()
    for p in added:
        sys.path.insert(0, p)
    try:
        try:
            import tah
            from transformers import AutoModelForCausalLM, Qwen3Config
        except Exception as exc:  # pragma: no cover - environment dependent
            pytest.skip(f"reference does not import here: {type(exc).__name__}: {exc}")
        assert os.path.realpath(tah.__file__).startswith(os.path.realpath(REF))
        yield tah, AutoModelForCausalLM, Qwen3Config
    finally:
        for p in added:
            if p in sys.path:
                sys.path.remove(p)
        _purge_tah_modules()
        for name in [n for n in sys.modules if n == "peft" or n.startswith("peft.")]:
            if "peft_standin" in (getattr(sys.modules[name], "__file__", "") or ""):
                del sys.modules[name]


def _ref_model(tah, AutoModelForCausalLM, Qwen3Config, max_iter=2):
    cfg = Qwen3Config(vocab_size=1024, hidden_size=256, intermediate_size=768, num_hidden_layers=4,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6,
                      tie_word_embeddings=True, max_position_embeddings=4096)
    torch.manual_seed(0)
    base = AutoModelForCausalLM.from_config(cfg, attn_implementation="sdpa").float()
    tc = tah.TaHConfig(max_iter=max_iter, iter_decider="IterLabelDecider",
                       adapter_kwargs=dict(r=8, lora_alpha=16, lora_dropout=0.0, target_modules="all-linear"),
                       input_updater_kwargs={"topk": 100}, train_loss="NextTokenPredLoss")
    model = tah.TaHForCausalLM(base, tc)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "lora_B" in n:
                p.normal_(std=0.05)
    return model.eval()


def _coin(base_cls, p, seed):
    class Coin(base_cls):
        """Seeded Bernoulli hard-token decider written against the decider call contract."""

        def __init__(self):
            super().__init__(max_iter=2)
            self.g = torch.Generator().manual_seed(seed)

        def forward(self, logits, iter_depth, **kw):
            if iter_depth >= 2:
                return self._stop_decision(logits, -10.0)
            return torch.rand(logits.shape[0], generator=self.g) < p, torch.zeros(logits.shape[0])

    return Coin()


def test_checkpoint_from_reference_loads_here_and_forward_matches(tmp_path, reference):
    tah, AM, QC = reference
    from tah_b200 import TaHForCausalLM
    ref = _ref_model(tah, AM, QC)
    ref.save_pretrained(str(tmp_path / "ck"))
    mine = TaHForCausalLM.from_pretrained(str(tmp_path / "ck"), torch_dtype=torch.float32).eval()
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 1024, (2, 48), generator=g)
    hard = (torch.rand(2, 48, generator=g) < 0.2).long() + 1
    attn = torch.ones_like(ids)
    with torch.no_grad():
        a = ref(input_ids=ids, attention_mask=attn, labels=ids, iter_count_labels=hard)
        b = mine(ids, attention_mask=attn, labels=ids, iter_count_labels=hard)
    assert torch.equal(a.iter_count, b.iter_count)
    assert (b.iter_count == 2).sum() > 0
    torch.testing.assert_close(b.logits, a.logits, atol=3e-4, rtol=1e-4)
    torch.testing.assert_close(b.loss, a.loss, atol=1e-5, rtol=1e-5)


def test_checkpoint_written_here_loads_in_reference(tmp_path, reference):
    tah, AM, QC = reference
    from tests.helpers import tiny_tah
    mine = tiny_tah().eval()
    mine.save_pretrained(str(tmp_path / "ck"))
    ref = tah.TaHForCausalLM.from_pretrained(str(tmp_path / "ck"), torch_dtype=torch.float32).eval()
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, 1024, (2, 32), generator=g)
    hard = (torch.rand(2, 32, generator=g) < 0.2).long() + 1
    with torch.no_grad():
        a = ref(input_ids=ids, attention_mask=torch.ones_like(ids), labels=ids, iter_count_labels=hard)
        b = mine(ids, labels=ids, iter_count_labels=hard)
    assert torch.equal(a.iter_count, b.iter_count)
    torch.testing.assert_close(b.logits, a.logits, atol=3e-4, rtol=1e-4)


def test_greedy_decode_with_seeded_hard_tokens_matches_reference(tmp_path, reference):
    tah, AM, QC = reference
    from tah.model.iter_decider import IterDecider as RefDecider
    from tah.model.utils import TaHForCasualLM_generate as ref_generate
    from tah_b200 import TaHForCausalLM
    from tah_b200.model.iter_decider import IterDecider
    from tah_b200.model.utils import TaHForCasualLM_generate
    ref = _ref_model(tah, AM, QC)
    ref.save_pretrained(str(tmp_path / "ck"))
    mine = TaHForCausalLM.from_pretrained(str(tmp_path / "ck"), torch_dtype=torch.float32).eval()
    ref.iter_decider = ref.eval_iter_decider = _coin(RefDecider, 0.2, 11)
    mine.iter_decider = mine.eval_iter_decider = _coin(IterDecider, 0.2, 11)

    class Tok:
        eos_token_id = None

        def decode(self, ids, **kw):
            return ""

    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 1024, (2, 24), generator=g)
    inputs = {"input_ids": ids, "attention_mask": torch.ones_like(ids)}
    a, _ = ref_generate(ref, Tok(), dict(inputs), max_new_tokens=12, do_sample=False, verbose=False)
    b, _ = TaHForCasualLM_generate(mine, Tok(), dict(inputs), max_new_tokens=12, do_sample=False, verbose=False)
    assert a == b
