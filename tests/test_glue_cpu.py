"""CPU tests of the glue around the model: checkpoints, collator, preprocessing, eval driver, scripts."""
import csv
import json
import os
import socket
import sys

import pytest
import torch

from tah_b200 import TaHConfig, TaHForCausalLM
from tah_b200.evaluate import codeeval
from tah_b200.evaluate.jobs import _free_port, combine_job_results, parse_data_range, run_single_job
from tah_b200.train import CustomTaHDataCollator
from tah_b200.train.schedule import lr_factor
from tah_b200.utils.data_prepare import _build_sft_example, _filter_keep
from tests.helpers import tiny_tah


def test_checkpoint_layout_and_round_trip(tmp_path):
    from safetensors import safe_open
    model = tiny_tah(decider="MLPIterDecider",
                     decider_kwargs=dict(topk=10, hidden_states_size=256, hidden_states_layer_nums=[1, 4],
                                         hidden_dims=[32, 32], dropout_rate=0.0, threshold=0.8, dtype=torch.float32)).eval()
    model.save_pretrained(str(tmp_path))
    names = set(os.listdir(tmp_path))
    assert {"config.json", "generation_config.json", "model.safetensors", "lora", "iter_decider.bin", "tah_config.json"} <= names
    assert set(os.listdir(tmp_path / "lora")) == {"adapter_config.json", "adapter_model.safetensors"}
    with safe_open(str(tmp_path / "model.safetensors"), "pt") as fh:
        keys = set(fh.keys())
    assert "model.layers.0.self_attn.q_proj.weight" in keys and "model.layers.3.mlp.up_proj.weight" in keys
    assert "model.embed_tokens.weight" in keys and "lm_head.weight" not in keys        # tied head is not duplicated
    assert not any("lora" in k or "base_layer" in k or "qkv_proj" in k for k in keys)
    with safe_open(str(tmp_path / "lora" / "adapter_model.safetensors"), "pt") as fh:
        lkeys = set(fh.keys())
    assert "base_model.model.model.layers.2.mlp.down_proj.lora_B.weight" in lkeys
    assert "base_model.model.model.layers.0.self_attn.k_proj.lora_A.weight" in lkeys
    acfg = json.load(open(tmp_path / "lora" / "adapter_config.json"))
    assert acfg["r"] == 8 and acfg["peft_type"] == "LORA" and "base_grad" not in acfg
    hf = json.load(open(tmp_path / "config.json"))
    assert hf["model_type"] == "qwen3" and hf["num_hidden_layers"] == 4 and hf["tie_word_embeddings"] is True
    loaded = TaHForCausalLM.from_pretrained(str(tmp_path)).eval()
    ids = torch.randint(0, 1024, (2, 12))
    hard = torch.ones(2, 12, dtype=torch.long)
    hard[:, 5] = 2
    with torch.no_grad():
        a, b = model(ids), loaded(ids)
    torch.testing.assert_close(a.logits, b.logits)
    assert torch.equal(a.iter_count, b.iter_count)
    # an override of the eval threshold wins over the stored decider state
    over = TaHConfig(iter_decider_kwargs=dict(model.tah_config.iter_decider_kwargs, threshold=0.3))
    l2 = TaHForCausalLM.from_pretrained(str(tmp_path), tah_config=over)
    assert abs(float(l2.iter_decider.threshold.detach()) - 0.3) < 1e-6


def test_sharded_safetensors_round_trip(tmp_path):
    model = tiny_tah().eval()
    model.save_pretrained(str(tmp_path), max_shard_bytes=2_000_000)
    assert os.path.exists(tmp_path / "model.safetensors.index.json")
    loaded = TaHForCausalLM.from_pretrained(str(tmp_path)).eval()
    ids = torch.randint(0, 1024, (1, 9))
    with torch.no_grad():
        torch.testing.assert_close(model(ids).logits, loaded(ids).logits)


def test_hf_backbone_parity():
    """The fused backbone computes what HuggingFace's Qwen3 computes with the same weights."""
    transformers = pytest.importorskip("transformers")
    from tah_b200.models import from_hf_model
    cfg = transformers.Qwen3Config(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6,
                                   tie_word_embeddings=True, rope_parameters={"rope_theta": 1e6, "rope_type": "default"})
    torch.manual_seed(0)
    hf = transformers.Qwen3ForCausalLM(cfg).float().eval()
    mine = from_hf_model(hf).eval()
    ids = torch.randint(0, 512, (2, 17))
    with torch.no_grad():
        ref = hf(input_ids=ids).logits
        out = mine(input_ids=ids)
    torch.testing.assert_close(out, ref, atol=2e-4, rtol=1e-4)


def test_collator_pads_on_tokenizer_side():
    class Tok:
        pad_token_id, padding_side = 9, "left"
    feats = [dict(input_ids=[1, 2, 3], attention_mask=[1, 1, 1], labels=[-100, 2, 3], iter_count_labels=[1, 1, 2]),
             dict(input_ids=[4], attention_mask=[1], labels=[4], iter_count_labels=[1])]
    b = CustomTaHDataCollator(Tok())(feats)
    assert b["input_ids"].tolist() == [[1, 2, 3], [9, 9, 4]]
    assert b["attention_mask"].tolist() == [[1, 1, 1], [0, 0, 1]]
    assert b["labels"].tolist() == [[-100, 2, 3], [-100, -100, 4]]
    assert b["iter_count_labels"].tolist() == [[1, 1, 2], [-100, -100, 1]]
    Tok.padding_side = "right"
    b = CustomTaHDataCollator(Tok(), pad_to_multiple_of=4)(feats)
    assert b["input_ids"].tolist()[1] == [4, 9, 9, 9] and b["iter_count_labels"].tolist()[1] == [1, -100, -100, -100]


def test_build_sft_example_and_filter():
    ex = _build_sft_example([5, 6, 7, 8, 9], [0, 0, 1, 1, 1], [1, 0, 1, 0, 0], max_iter=2, max_length=None,
                            truncate=True, query_iter_count=1)
    assert ex["labels"] == [-100, -100, 7, 8, 9] and ex["iter_count_labels"] == [1, 1, 2, 1, 1]
    assert ex["attention_mask"] == [1] * 5
    ex = _build_sft_example([5, 6, 7], [0, 1, 1], [0, 2, 0], 3, None, True, 1)
    assert ex["iter_count_labels"] == [1, 3, 1]                      # counts written by the labeller: mismatch + 1
    assert _build_sft_example([1, 2], [0, 0], [0, 0], 2, None, True, 1) is None
    assert _build_sft_example([1, 2, 3], [1, 1, 1], None, 2, 2, False, 1) is None
    assert len(_build_sft_example([1, 2, 3], [1, 1, 1], None, 2, 2, True, 1)["input_ids"]) == 2
    batch = {"real_token": [[1, 2, 3], [1, 2, 3], [1, 2, 3, 4]], "mask": [[0, 1, 1], [0, 0, 0], [0, 1, 1, 1]],
             "mismatch": [[0, 1, 0], [0, 0, 0], [0, 0, 0, 1]]}
    assert _filter_keep(batch, max_length=3, truncate=True) == [True, False, False]
    assert _filter_keep(batch, max_length=3, truncate=False) == [True, False, False]
    assert _filter_keep(batch, max_length=None, truncate=True) == [True, False, True]


def test_lr_schedule_cosine_with_min_lr():
    assert lr_factor(0, 100, 10) == 0.0 and abs(lr_factor(5, 100, 10) - 0.5) < 1e-9
    assert abs(lr_factor(10, 100, 10, "cosine_with_min_lr", 0.1) - 1.0) < 1e-9
    assert abs(lr_factor(100, 100, 10, "cosine_with_min_lr", 0.1) - 0.1) < 1e-9
    assert abs(lr_factor(55, 100, 10, "cosine_with_min_lr", 0.1) - 0.55) < 1e-9
    assert lr_factor(100, 100, 0, "linear") == 0.0


def test_parse_data_range_and_free_port():
    assert parse_data_range([5], 100) == (0, 5) and parse_data_range([2, 9], 6) == (2, 6)
    assert parse_data_range(None, 7) == (0, 7)
    with pytest.raises(ValueError):
        parse_data_range([5, 5], 10)
    with pytest.raises(ValueError):
        parse_data_range([1, 2, 3])
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        busy = s.getsockname()[1]
        s.listen(1)
        got = _free_port(busy)
        assert got != busy and busy < got < busy + 100


class _FakeTok:
    chat_template = None
    pad_token = eos_token = "<e>"

    def encode(self, text):
        return text.split()


def test_run_single_job_and_combine(tmp_path, monkeypatch):
    from tah_b200.evaluate import jobs, matheval

    class Grader:
        def rule_judge(self, out, gold):
            ans = out.strip().split()[-1] if out.strip() else ""
            return (ans == gold, ans or "No extracted answer")
    monkeypatch.setitem(matheval.evaluator_map, "toy", Grader())

    def factory(backend, config, model_path, tokenizer, tp_size=1):
        def infer(prompts):
            return [(f"the answer is {len(p.split())}", 0.5) for p in prompts]
        return object(), infer

    mapping = {"id_field": "id", "question_field": "question", "answer_field": "answer", "answer_type": "boxed"}
    for job_id, probs in enumerate([[{"id": "toy_0", "question": "a b c", "answer": "3"}],
                                    [{"id": "toy_1", "question": "a b", "answer": "5"}]]):
        run_single_job(config={"batch_size": 2, "repeat_size": 2}, combined_dataset_name="toy", output_dir=str(tmp_path),
                       timestamp="ts", model_path="", job_id=job_id, job_nums=2, start_idx=0, end_idx=1, tp_size=1,
                       backend="tah", data_range=None, problems_data=probs, field_mapping=mapping,
                       unified_code_solutions_file=None, tokenizer=_FakeTok(), backend_factory=factory)
    base = tmp_path / "toy_tah" / "ts"
    assert (base / "job_0" / "details" / "toy_0" / "sample_1.json").exists()
    summary = combine_job_results(base, 2)
    assert summary == {"total": 4, "correct": 2, "accuracy": 0.5}
    rows = list(csv.DictReader(open(base / "detailed_results.csv")))
    assert len(rows) == 4 and rows[0]["processing_time"] == "0.5" and set(rows[0]) == set(jobs._CSV_FIELDS)
    assert sum(1 for _ in open(base / "samples.jsonl")) == 4
    assert "Total Accuracy" in open(base / "evaluation_stats.csv").read()


def test_run_single_job_hands_the_whole_job_to_a_continuous_batching_backend(tmp_path, monkeypatch):
    """A backend whose ``infer`` carries ``serve_all`` gets all prompts of the job in one call (rows = batch_size);
    results land on their problems and repeats in order."""
    import csv
    from tah_b200.evaluate import jobs, matheval
    from tah_b200.evaluate.jobs import run_single_job

    class Grader:
        def rule_judge(self, out, gold):
            ans = out.strip().split()[-1] if out.strip() else ""
            return (ans == gold, ans or "No extracted answer")
    monkeypatch.setitem(matheval.evaluator_map, "toy", Grader())
    calls = []

    def factory(backend, config, model_path, tokenizer, tp_size=1):
        def infer(prompts):
            raise AssertionError("static batches must not be used when serve_all exists and the job is larger than a batch")

        def serve_all(prompts, rows):
            calls.append((len(prompts), rows))
            return [(f"the answer is {len(p.split())}", 0.25) for p in prompts]
        infer.serve_all = serve_all
        return object(), infer

    mapping = {"id_field": "id", "question_field": "question", "answer_field": "answer", "answer_type": "boxed"}
    probs = [{"id": f"toy_{i}", "question": " ".join("w" * (i + 1)), "answer": str(i + 1)} for i in range(5)]
    monkeypatch.setattr(jobs, "_make_prompt", lambda text, tok, is_code: text)
    run_single_job(config={"batch_size": 2, "repeat_size": 2}, combined_dataset_name="toy", output_dir=str(tmp_path),
                   timestamp="ts", model_path="", job_id=0, job_nums=1, start_idx=0, end_idx=5, tp_size=1,
                   backend="tah", data_range=None, problems_data=probs, field_mapping=mapping,
                   unified_code_solutions_file=None, tokenizer=_FakeTok(), backend_factory=factory)
    assert calls == [(10, 2)]
    rows = list(csv.DictReader(open(tmp_path / "toy_tah" / "ts" / "job_0" / "detailed_results.csv")))
    assert len(rows) == 10 and all(r["is_correct"] == "True" for r in rows)
    assert [r["problem_id"] for r in rows[:4]] == ["toy_0", "toy_0", "toy_1", "toy_1"]


def test_code_sanitize_and_evaluate(tmp_path):
    text = "Here you go:\n```python\nimport math\n\ndef helper(x):\n    return x + 1\n\ndef unused():\n    return 0\n\ndef add1(x):\n    return helper(x)\n```\nthanks"
    code = codeeval.sanitize(text, "add1")
    assert "def add1" in code and "def helper" in code and "import math" in code
    problems = tmp_path / "p.jsonl"
    problems.write_text(json.dumps({"task_id": "t/0", "entry_point": "add1",
                                    "test": "def check(f):\n    assert f(1) == 2\n"}) + "\n")
    samples = tmp_path / "s.jsonl"
    samples.write_text(json.dumps({"task_id": "t/0", "solution": code}) + "\n" +
                       json.dumps({"task_id": "t/0", "solution": "def add1(x):\n    return x"}) + "\n")
    res = codeeval.evaluate("toy", str(samples), problems_path=str(problems), parallel=2, ks=(1, 2))
    assert abs(res["pass_at_k"]["base"]["pass@1"] - 0.5) < 1e-9 and res["pass_at_k"]["base"]["pass@2"] == 1.0
    # a second call loads the stored result file instead of re-running
    again = codeeval.evaluate("toy", str(samples), problems_path=str(problems), parallel=2, ks=(1, 2))
    assert again["pass_at_k"] == res["pass_at_k"]


def test_code_evaluate_against_canonical_ground_truth(tmp_path, monkeypatch):
    """Problems in the base/plus-input shape: expected outputs come from the canonical solution (cached on
    disk); a solution that is right on the base inputs only passes 'base' but not 'plus'."""
    monkeypatch.setattr(codeeval, "CACHE_DIR", str(tmp_path / "cache"))
    pb = {"task_id": "t/0", "entry_point": "absdiff", "prompt": "def absdiff(a, b):\n",
          "canonical_solution": "    return abs(a - b)\n", "base_input": [[3, 1], [5, 2]], "plus_input": [[1, 4], [2.0, 2.5]],
          "atol": 1e-6}
    problems = tmp_path / "p.jsonl"
    problems.write_text(json.dumps(pb) + "\n")
    samples = tmp_path / "s.jsonl"
    samples.write_text(json.dumps({"task_id": "t/0", "solution": "def absdiff(a, b):\n    return abs(a - b)"}) + "\n" +
                       json.dumps({"task_id": "t/0", "completion": "    return a - b\n"}) + "\n")
    res = codeeval.evaluate("toy", str(samples), problems_path=str(problems), parallel=2, ks=(1,))
    assert res["pass_at_k"]["base"]["pass@1"] == 1.0
    assert abs(res["pass_at_k"]["plus"]["pass@1"] - 0.5) < 1e-9
    assert res["eval"]["t/0"][1]["plus_status"] == "fail" and res["eval"]["t/0"][1]["plus_fail_tests"]
    assert len(os.listdir(tmp_path / "cache")) == 1


def test_download_retries_with_backoff(monkeypatch):
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "script", "preparation"))
    import download
    calls, sleeps = [], []
    monkeypatch.setattr(download.time, "sleep", lambda s: sleeps.append(s))

    def flaky(**kw):
        calls.append(kw)
        if len(calls) < 4:
            raise ConnectionError("boom")
        return "/tmp/x"
    assert download.download_with_retry("a/b", "/tmp/x", downloader=flaky) == "/tmp/x"
    assert len(calls) == 4 and sleeps == [1.0, 2.0, 4.0]


def test_labeller_helpers():
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "script", "preparation"))
    import label
    assert label._categorize_masks([1, 2, 151667, 3, 4]) == [0, 0, 1, 1, 1]
    mm = label._calculate_mismatch(torch.tensor([5, 6, 7, 8]), torch.tensor([1, 5, 9, 7]))
    assert mm.tolist() == [0, 1, 0, 0]                                # pred[i] vs real[i+1]; last stays 0


def test_label_selection_token_table_and_grouping(tmp_path):
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "script", "preparation"))
    import label
    path = tmp_path / "d.jsonl"
    path.write_text("".join(json.dumps({"question": f"q{i}", "answer": f"a{i}"}) + "\n" for i in range(10)))
    assert [s["question"] for s in label.load_samples(str(path), (2, 7))] == ["q2", "q3", "q4", "q5", "q6"]
    sub = label.load_samples(str(path), None, 4)
    assert len(sub) == 4 and sub == label.load_samples(str(path), None, 4)          # seeded sub-sample
    (tmp_path / "d.json").write_text(json.dumps([{"question": "x", "answer": "y"}]))
    assert len(label.load_samples(str(tmp_path / "d.json"))) == 1
    assert label.gpu_ranges(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    rows = [{"data_id": 7, "real_token": [1, 2, 3], "predictions": [2, 9, 9], "mask": [0, 1, 1], "mismatch": [0, 1, 0],
             "entropy": [0.1, 0.2, 0.3]},
            {"data_id": 3, "real_token": [4, 5], "predictions": [5, 5], "mask": [1, 1], "mismatch": [0, 0],
             "entropy": [0.4, 0.5]}]
    table = label.token_table(rows, save_entropy=True, save_ce=False)
    assert set(table) == {"predictions", "small_token", "data_id", "mask", "real_token", "mismatch", "entropy"}
    assert table["small_token"] == [0, 1, 2, 0, 1] and table["data_id"] == [7, 7, 7, 3, 3]
    samples = label.samples_from_token_table(table, lambda ids: " ".join(map(str, ids)))
    assert [s["data_id"] for s in samples] == [3, 7]
    assert samples[1] == {"data_id": 7, "real_text": "1 2 3", "real_token": [1, 2, 3], "mask": [0, 1, 1],
                          "mismatch": [0, 1, 0], "entropy": [0.1, 0.2, 0.3]}
    assert label.label_statistics(samples) == {"samples": 2, "tokens": 5, "mismatch": 1, "assistant_tokens": 4,
                                               "assistant_mismatch": 1}
    args = label.build_parser().parse_args(["--dataset_path", "d", "--test_model_list", "a", "b", "--output_path", "o",
                                            "--index_range", "0", "5", "--is_cutoff", "True", "--save_ce"])
    assert args.test_model_list == ["a", "b"] and args.is_cutoff is True and args.index_range == [0, 5] and args.top_k == -1


def test_prune_reads_calibration_from_a_saved_dataset(tmp_path):
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "script", "preparation"))
    import prune
    from datasets import Dataset
    Dataset.from_dict({"real_text": ["alpha", "", "beta", "gamma"], "n": [1, 2, 3, 4]}).save_to_disk(str(tmp_path / "ds"))
    assert prune.read_calibration_texts(str(tmp_path / "ds"), "real_text", 2) == ["alpha", "beta"]
    with pytest.raises(KeyError):
        prune.read_calibration_texts(str(tmp_path / "ds"), "text", 2)
    (tmp_path / "c.txt").write_text("one\n\ntwo\n")
    assert prune.read_calibration_texts(str(tmp_path / "c.txt")) == ["one", "two"]


def test_trainer_resume_is_exact_with_optimizer_and_rng_state(tmp_path):
    """Train four steps with a checkpoint after two; a second trainer resumed from that checkpoint reaches the same
    parameters: model weights, sharded optimizer state, data position and the random-number state (LoRA dropout is
    on, so the masks of steps 3 and 4 must continue the first run's stream)."""
    from tah_b200 import TaHForCausalLM
    from tah_b200.train import CustomTaHDataCollator, CustomTaHTrainer, TaHTrainingArguments
    from tests.helpers import tiny_tah

    def rows():
        g = torch.Generator().manual_seed(11)
        out = []
        for _ in range(8):
            ids = torch.randint(0, 1024, (20,), generator=g).tolist()
            hard = [1] * 20
            hard[5] = 2
            out.append(dict(input_ids=ids, attention_mask=[1] * 20, labels=[-100] * 2 + ids[2:], iter_count_labels=hard))
        return out

    def args(out_dir, **kw):
        return TaHTrainingArguments(output_dir=str(out_dir), per_device_train_batch_size=1, gradient_accumulation_steps=2,
                                    learning_rate=1e-3, max_grad_norm=1.0, num_train_epochs=1, logging_steps=1, seed=0,
                                    save_strategy="steps", save_steps=2, save_only_model=False, **kw)

    def build():
        m = tiny_tah(seed=0)
        for mod in m.modules():
            if hasattr(mod, "lora") and getattr(mod.lora, "r", 0) > 0:
                mod.lora.lora_dropout = 0.25
        return m

    m1 = build()
    t1 = CustomTaHTrainer(m1, args(tmp_path / "a"), rows(), None, data_collator=CustomTaHDataCollator(None, pad_token_id=0))
    t1.train()
    assert t1.state.global_step == 4 and (tmp_path / "a" / "checkpoint-2" / "optim" / "rank0.pt").exists()
    final = {n: p.detach().clone() for n, p in m1.named_parameters()}

    m2 = TaHForCausalLM.from_pretrained(str(tmp_path / "a" / "checkpoint-2"))
    for mod in m2.modules():
        if hasattr(mod, "lora") and getattr(mod.lora, "r", 0) > 0:
            mod.lora.lora_dropout = 0.25
    t2 = CustomTaHTrainer(m2, args(tmp_path / "b"), rows(), None, data_collator=CustomTaHDataCollator(None, pad_token_id=0))
    t2.train(resume_from_checkpoint=str(tmp_path / "a" / "checkpoint-2"))
    assert t2.state.global_step == 4
    err = max(float((final[n] - p.detach()).abs().max()) for n, p in m2.named_parameters())
    assert err < 1e-6, err


def test_trainer_with_fewer_micro_batches_than_the_accumulation_window_still_steps(tmp_path):
    """Three rows against ``gradient_accumulation_steps=8`` and ``max_steps=2``: each epoch is one shorter window (the
    loop used to spin over epochs without ever taking a step)."""
    from tah_b200.train import CustomTaHDataCollator, CustomTaHTrainer, TaHTrainingArguments
    from tests.helpers import tiny_tah
    g = torch.Generator().manual_seed(2)
    rows = []
    for _ in range(3):
        ids = torch.randint(0, 1024, (16,), generator=g).tolist()
        rows.append(dict(input_ids=ids, attention_mask=[1] * 16, labels=ids, iter_count_labels=[1] * 15 + [2]))
    args = TaHTrainingArguments(output_dir=str(tmp_path), per_device_train_batch_size=1, gradient_accumulation_steps=8,
                                learning_rate=1e-3, max_steps=2, logging_steps=1, save_strategy="no", seed=0)
    tr = CustomTaHTrainer(tiny_tah(seed=0), args, rows, None, data_collator=CustomTaHDataCollator(None, pad_token_id=0))
    tr.train()
    assert tr.state.global_step == 2


def test_sft_script_runs_a_shipped_recipe_on_synthetic_data(tmp_path):
    """``script/train/SFT_TaH.py --synthetic`` with the shipped step-1 recipe (16 accumulation steps, more than the
    eight synthetic rows): two optimizer steps, evaluation, final checkpoint in the reference layout."""
    import subprocess
    import sys
    import yaml
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = yaml.safe_load(open(os.path.join(root, "script", "recipes", "qwen3_1.7", "sft_tah_step1.yaml")))
    cfg["data"]["output_dir"] = str(tmp_path / "run")
    cfg["training"]["save_strategy"] = "no"
    cfg["training"]["report_to"] = "none"
    path = tmp_path / "cfg.yaml"
    yaml.safe_dump(cfg, open(path, "w"))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    res = subprocess.run([sys.executable, os.path.join(root, "script", "train", "SFT_TaH.py"), "--config", str(path),
                          "--synthetic", "8", "--max_steps", "2"], capture_output=True, text=True, timeout=400, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "Saved final model" in res.stdout
    finals = [os.path.join(dp, "final_model") for dp, dn, _ in os.walk(tmp_path / "run") if "final_model" in dn]
    assert finals and {"model.safetensors", "tah_config.json", "iter_decider.bin"} <= set(os.listdir(finals[0]))
