"""Evaluation job runner: split a benchmark over worker processes, generate, grade, merge.

Flow (reference ``tah/evaluate/jobs.py:480-543``): the parent loads the benchmark(s), selects
problems (``--data_ids`` or ``--data_range``), deals them round-robin to ``job_nums`` jobs
(job *j* takes ``selected[j::job_nums]``), pins each job to its GPUs through
``CUDA_VISIBLE_DEVICES`` *before* the child starts, and spawns one process per job.  A child
dies with its parent (``PR_SET_PDEATHSIG``), picks a free rendezvous port, runs its batches and
reports ``(job_id, ok, message)`` on a queue; the parent polls liveness, counts failures, still
merges partial results, and finally runs code grading when the benchmark is a code benchmark.

Artefacts per job: ``details/<problem>/sample_<k>.json``, ``detailed_results.csv``,
``evaluation_stats.csv``; merged: ``samples.jsonl``, ``detailed_results.csv``, ``evaluation_stats.csv``.
"""
from __future__ import annotations

import csv
import ctypes
import fcntl
import json
import logging
import math
import multiprocessing as mp
import os
import shutil
import signal
import socket
import time
import traceback
from pathlib import Path
from typing import Dict, List, Optional, Tuple

from tah_b200.evaluate import codeeval, matheval
from tah_b200.evaluate.backends import cleanup, setup_backend
from tah_b200.evaluate.datasets import load_combined_dataset

# worker processes must not inherit CUDA state from the parent
try:
    mp.set_start_method("spawn", force=True)
except RuntimeError:
    pass

_CSV_FIELDS = ["problem_id", "sample_idx", "correct_answer", "predicted_answer", "has_answer", "is_correct",
               "input_tokens", "output_tokens", "processing_time"]
_CODE_ANSWER_TYPES = {"humaneval", "mbpp", "livecodebench"}
log = logging.getLogger(__name__)


# ---------------------------------------------------------------------------------------------
# small helpers
# ---------------------------------------------------------------------------------------------
def parse_data_range(data_range_list, total_problems: Optional[int] = None) -> Tuple[int, int]:
    """``[end]`` or ``[start, end]`` (end exclusive, clipped to the benchmark size)."""
    if not data_range_list:
        return 0, total_problems if total_problems is not None else 0
    if len(data_range_list) == 1:
        start, end = 0, data_range_list[0]
    elif len(data_range_list) == 2:
        start, end = data_range_list
    else:
        raise ValueError(f"data_range expects 1 or 2 values, got {len(data_range_list)}")
    if total_problems is not None:
        end = min(end, total_problems)
    if start < 0 or end <= start:
        raise ValueError(f"invalid data_range: start={start}, end={end}")
    return start, end


def _free_port(start: int = 29555, max_tries: int = 100) -> int:
    for i in range(max_tries):
        port = start + i
        if port > 65535:
            port = 30514 + (i % 100)
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            try:
                s.bind(("127.0.0.1", port))
                return port
            except OSError:
                continue
    raise RuntimeError(f"no free port after {max_tries} tries from {start}")


def _install_pdeathsig() -> None:
    """Ask the kernel to SIGTERM this process when its parent dies (Linux only)."""
    try:
        ctypes.CDLL("libc.so.6", use_errno=True).prctl(1, signal.SIGTERM)   # PR_SET_PDEATHSIG = 1
    except Exception:
        pass


def _job_dir(output_dir: str, dataset: str, backend: str, timestamp: str, job_id: int, data_range) -> Path:
    out = Path(output_dir) / f"{dataset}_{backend}" / timestamp
    if data_range:
        a, b = parse_data_range(data_range)
        out = out / f"TASK_{a}_{b}"
    return out / f"job_{job_id}"


def _make_prompt(text: str, tokenizer, is_code: bool) -> str:
    if is_code:
        return codeeval.make_raw_chat_prompt_for_code_evaluation(text, reasoning=False, tokenizer=tokenizer)
    if getattr(tokenizer, "chat_template", None) is None:
        return text
    return tokenizer.apply_chat_template([{"role": "user", "content": text}], tokenize=False,
                                         add_generation_prompt=True)


def _score(output: str, gold: str, dataset: str, is_code: bool):
    if is_code:
        return "pending_code_eval", False, False
    ok, pred = matheval.evaluator_map[dataset].rule_judge(output, gold)
    if pred == "No extracted answer":
        return "", False, bool(ok)
    return pred, True, bool(ok)


def _append_locked(path: Path, record: dict) -> None:
    with open(path, "a", encoding="utf-8") as fh:
        fcntl.flock(fh.fileno(), fcntl.LOCK_EX)
        try:
            fh.write(json.dumps(record, ensure_ascii=False) + "\n")
        finally:
            fcntl.flock(fh.fileno(), fcntl.LOCK_UN)


def _write_stats(out: Path, rows: List[dict]) -> None:
    per: Dict[str, List[dict]] = {}
    for r in rows:
        per.setdefault(r["problem_id"], []).append(r)
    with open(out / "evaluation_stats.csv", "w", newline="", encoding="utf-8") as fh:
        w = csv.writer(fh)
        w.writerow(["problem_id", "accuracy", "correct_count", "total_samples", "avg_output_length"])
        for pid, rs in per.items():
            c = sum(1 for r in rs if str(r["is_correct"]) == "True" or r["is_correct"] is True)
            w.writerow([pid, f"{c / len(rs):.3f}", c, len(rs), f"{sum(float(r['output_tokens']) for r in rs) / len(rs):.2f}"])
        n = len(rows)
        c = sum(1 for r in rows if str(r["is_correct"]) == "True" or r["is_correct"] is True)
        w.writerow([])
        w.writerow(["Total Accuracy", f"{(c / n if n else 0):.3f}", c, n,
                    f"{(sum(float(r['output_tokens']) for r in rows) / n if n else 0):.2f}"])


# ---------------------------------------------------------------------------------------------
# one job
# ---------------------------------------------------------------------------------------------
def run_single_job(*, config: Dict, combined_dataset_name: str, output_dir: str, timestamp: str, model_path: str,
                   job_id: int, job_nums: int, start_idx: int, end_idx: int, tp_size: int, backend: str, data_range,
                   problems_data, field_mapping: Dict, unified_code_solutions_file: Optional[Path],
                   tokenizer=None, backend_factory=None) -> List[dict]:
    """Generate and grade the problems of one job.  ``tokenizer`` / ``backend_factory`` can be injected
    (tests use a fake backend); by default the tokenizer is loaded from ``model_path``."""
    out = _job_dir(output_dir, combined_dataset_name, backend, timestamp, job_id, data_range)
    details = out / "details"
    details.mkdir(parents=True, exist_ok=True)
    if tokenizer is None:
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(model_path)
    if getattr(tokenizer, "pad_token", None) is None:
        tokenizer.pad_token = tokenizer.eos_token
    model, infer = (backend_factory or setup_backend)(backend, config, model_path, tokenizer, tp_size=tp_size)
    is_code = field_mapping.get("answer_type", "boxed") in _CODE_ANSWER_TYPES
    problems = []
    for i, item in enumerate(problems_data):
        pid = str(item.get(field_mapping["id_field"]) or f"problem_{item.get('_original_index', start_idx + i)}")
        pdir = details / pid
        pdir.mkdir(parents=True, exist_ok=True)
        problems.append({"problem_id": pid, "original_problem_id": item.get("_original_id", pid),
                         "text": str(item.get(field_mapping["question_field"], "")).strip(),
                         "answer": str(item.get(field_mapping["answer_field"], "")).strip(),
                         "dir": pdir, "entry_point": item.get("entry_point")})
    repeat, bs = int(config.get("repeat_size", 1)), int(config.get("batch_size", 1))
    prompts, owner = [], []
    for pi, p in enumerate(problems):
        rendered = _make_prompt(p["text"], tokenizer, is_code)
        for k in range(repeat):
            prompts.append(rendered)
            owner.append((pi, k))
    results_file = out / "detailed_results.csv"
    with open(results_file, "w", newline="", encoding="utf-8") as fh:
        csv.DictWriter(fh, fieldnames=_CSV_FIELDS).writeheader()
    rows: List[dict] = []
    # a backend with continuous batching takes the whole job at once (batch_size = rows decoding at a time)
    serve_all = getattr(infer, "serve_all", None)
    all_outputs = serve_all(prompts, bs) if serve_all is not None and len(prompts) > bs else None
    for b in range(math.ceil(len(prompts) / bs)):
        lo, hi = b * bs, min(len(prompts), (b + 1) * bs)
        outputs = all_outputs[lo:hi] if all_outputs is not None else infer(prompts[lo:hi])
        with open(results_file, "a", newline="", encoding="utf-8") as fh:
            writer = csv.DictWriter(fh, fieldnames=_CSV_FIELDS)
            for j, (text, secs) in enumerate(outputs):
                pi, k = owner[lo + j]
                p = problems[pi]
                pred, has, ok = _score(text, p["answer"], combined_dataset_name, is_code)
                detail = {"problem": p["text"], "output": text, "correct_answer": p["answer"],
                          "predicted_answer": pred, "is_correct": ok}
                if is_code:
                    code = codeeval.sanitize(text, p["entry_point"])
                    detail.update(extracted_code=code, entry_point=p["entry_point"])
                    if unified_code_solutions_file is not None:
                        _append_locked(Path(unified_code_solutions_file),
                                       {"task_id": p["original_problem_id"], "solution": str(code)})
                with open(p["dir"] / f"sample_{k}.json", "w", encoding="utf-8") as fd:
                    json.dump(detail, fd, ensure_ascii=False, indent=2)
                row = {"problem_id": p["problem_id"], "sample_idx": k, "correct_answer": p["answer"],
                       "predicted_answer": pred, "has_answer": has, "is_correct": ok,
                       "input_tokens": len(tokenizer.encode(p["text"])), "output_tokens": len(tokenizer.encode(text)),
                       "processing_time": secs}
                writer.writerow(row)
                rows.append(row)
    _write_stats(out, rows)
    acc = sum(1 for r in rows if r["is_correct"]) / len(rows) if rows else 0.0
    print(f"Job {job_id} done; accuracy={acc:.4f}")
    cleanup(model, backend)
    return rows


def _run_job_process(job_id, config, dataset, output_dir, timestamp, model_path, job_nums, start_idx, end_idx,
                     tp_size, backend, data_range, gpus, problems, field_mapping, code_file, queue):
    _install_pdeathsig()
    try:
        port = _free_port(29555 + 100 * job_id)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), SGLANG_NCCL_PORT=str(port + 1))
        logging.basicConfig(level=str(config.get("_logger_level", "INFO")).upper())
        from tah_b200.model.utils import set_all_seeds
        set_all_seeds(int(config.get("_random_seed", 420)), verbose=False)
        import torch
        if torch.cuda.is_available():
            torch.cuda.init()
        run_single_job(config=config, combined_dataset_name=dataset, output_dir=output_dir, timestamp=timestamp,
                       model_path=model_path, job_id=job_id, job_nums=job_nums, start_idx=start_idx,
                       end_idx=end_idx, tp_size=tp_size, backend=backend, data_range=data_range,
                       problems_data=problems, field_mapping=field_mapping, unified_code_solutions_file=code_file)
        queue.put((job_id, True, "ok"))
    except Exception:
        queue.put((job_id, False, traceback.format_exc()))


# ---------------------------------------------------------------------------------------------
# orchestration
# ---------------------------------------------------------------------------------------------
def _select_problems(args, dataset: List[dict]) -> List:
    if getattr(args, "data_ids", None):
        valid = {str(it.get("id")) for it in dataset}
        out, seen = [], set()
        for pid in (s.strip() for s in str(args.data_ids).split(",")):
            if pid and pid in valid and pid not in seen:
                seen.add(pid)
                out.append(pid)
        if not out:
            raise ValueError("--data_ids matched no problem IDs (use <dataset>_<original_id>)")
        return out
    a, b = parse_data_range(args.data_range, len(dataset))
    return list(range(a, b))


def _build_job_args(args, dataset, selected, config, name, timestamp, gpus, gpus_per_job, mapping, code_file):
    by_id = {str(it.get("id")): it for it in dataset} if getattr(args, "data_ids", None) else None
    jobs = []
    for j in range(args.job_nums):
        mine = selected[j::args.job_nums]
        if not mine:
            continue
        if by_id is not None:
            probs = [by_id[str(p)] for p in mine if str(p) in by_id]
        else:
            probs = [dict(dataset[i], _original_index=i) for i in mine]
        jobs.append((j, config, name, args.output_dir, timestamp, args.model_path, args.job_nums, 0, len(mine),
                     gpus_per_job, args.backend, args.data_range, gpus[j * gpus_per_job:(j + 1) * gpus_per_job],
                     probs, mapping, code_file))
    return jobs


def _run_jobs(jobs, target=_run_job_process, poll_s: float = 1.0) -> Tuple[int, int]:
    queue = mp.Queue()
    procs = {}
    saved = os.environ.get("CUDA_VISIBLE_DEVICES")
    for job in jobs:
        gpus = job[12]
        # the device mask must be in the environment before the child initialises CUDA
        if gpus:
            os.environ["CUDA_VISIBLE_DEVICES"] = ",".join(str(g) for g in gpus)
        p = mp.Process(target=target, args=(*job, queue))
        p.start()
        procs[job[0]] = p
    if saved is None:
        os.environ.pop("CUDA_VISIBLE_DEVICES", None)
    else:
        os.environ["CUDA_VISIBLE_DEVICES"] = saved
    done, ok, failed = set(), 0, 0
    while len(done) < len(procs):
        try:
            job_id, good, msg = queue.get(timeout=poll_s)
            done.add(job_id)
            ok, failed = ok + bool(good), failed + (not good)
            if not good:
                print(f"Job {job_id} failed:\n{msg}")
        except Exception:
            for job_id, p in procs.items():
                if job_id not in done and not p.is_alive():      # died without reporting
                    done.add(job_id)
                    failed += 1
                    print(f"Job {job_id} exited with code {p.exitcode} without a result")
    for p in procs.values():
        p.join(timeout=30)
    return ok, failed


def combine_job_results(base_dir, job_nums: int, del_job_dir: bool = False) -> Optional[dict]:
    """Merge the per-job CSV/JSON artefacts under ``base_dir`` (works with partial results)."""
    base = Path(base_dir)
    rows: List[dict] = []
    samples_path = base / "samples.jsonl"
    with open(samples_path, "w", encoding="utf-8") as sj:
        for j in range(job_nums):
            jd = base / f"job_{j}"
            res = jd / "detailed_results.csv"
            if not res.exists():
                continue
            with open(res, newline="", encoding="utf-8") as fh:
                rows.extend(csv.DictReader(fh))
            for sample in sorted((jd / "details").glob("*/sample_*.json")):
                with open(sample, encoding="utf-8") as fd:
                    rec = json.load(fd)
                rec["problem_id"], rec["sample"] = sample.parent.name, sample.stem
                sj.write(json.dumps(rec, ensure_ascii=False) + "\n")
    if not rows:
        print("Warning: no job produced results")
        return None
    with open(base / "detailed_results.csv", "w", newline="", encoding="utf-8") as fh:
        w = csv.DictWriter(fh, fieldnames=_CSV_FIELDS)
        w.writeheader()
        w.writerows(rows)
    _write_stats(base, rows)
    n = len(rows)
    c = sum(1 for r in rows if str(r["is_correct"]) == "True")
    summary = {"total": n, "correct": c, "accuracy": c / n}
    print(f"Combined {n} samples: accuracy {summary['accuracy']:.4f}")
    if del_job_dir:
        for j in range(job_nums):
            shutil.rmtree(base / f"job_{j}", ignore_errors=True)
    return summary


def allocate_gpus_and_run_jobs(args) -> Optional[dict]:
    import yaml
    gpus = [int(g) for g in os.environ.get("CUDA_VISIBLE_DEVICES", "0,1,2,3,4,5,6,7").split(",") if g.strip() != ""]
    dataset, mapping = load_combined_dataset(args.dataset_name)
    name = args.dataset_name if isinstance(args.dataset_name, str) else "_".join(args.dataset_name)
    selected = _select_problems(args, dataset)
    with open(args.eval_config, encoding="utf-8") as fh:
        config = yaml.safe_load(fh) or {}
    config["_logger_level"] = getattr(args, "logger_level", "INFO")
    config["_random_seed"] = getattr(args, "random_seed", 420)
    timestamp = time.strftime("%Y%m%d_%H%M%S")
    base = _job_dir(args.output_dir, name, args.backend, timestamp, 0, args.data_range).parent
    base.mkdir(parents=True, exist_ok=True)
    shutil.copy(args.eval_config, base / Path(args.eval_config).name)
    tp = int(getattr(args, "tp_size_per_job", 1))
    if args.job_nums * tp > len(gpus):
        raise ValueError(f"{args.job_nums} jobs x {tp} GPUs need {args.job_nums * tp} GPUs, {len(gpus)} visible")
    is_code = mapping.get("answer_type") in _CODE_ANSWER_TYPES
    code_file = base / "code_solutions.jsonl" if is_code else None
    jobs = _build_job_args(args, dataset, selected, config, name, timestamp, gpus, tp, mapping, code_file)
    ok, failed = _run_jobs(jobs)
    if failed:
        print(f"Warning: {failed} of {ok + failed} jobs failed; combining partial results")
    summary = combine_job_results(base, args.job_nums, bool(getattr(args, "del_job_dir", False)))
    if is_code and code_file is not None and code_file.exists():
        codeeval.evaluate(name, str(code_file))
    return summary
