"""Code-generation grading (HumanEval / MBPP style benchmarks).

* :func:`make_raw_chat_prompt_for_code_evaluation` - chat-template priming so that the model
  continues inside a ```python block (same contract as reference ``tah/evaluate/codeeval.py:71-91``).
* :func:`sanitize` - pull the code block out of a completion and keep the entry-point function with
  the imports and helper definitions it needs.
* :func:`evaluate` - run every ``{task_id, solution}`` of a solutions ``.jsonl`` against the
  benchmark's tests in isolated worker processes with time limits, report pass@k.

When ``evalplus`` is installed its ground-truth machinery (base + plus inputs, oracle outputs) is
used; otherwise the tests shipped in the benchmark rows (``test`` + ``entry_point``) are executed
directly, which needs nothing beyond the standard library.  A watchdog thread warns when no sample
has finished for a long time (reference ``codeeval.py:238-244``).
"""
from __future__ import annotations

import ast
import json
import multiprocessing as mp
import os
import re
import threading
import time
from collections import defaultdict
from concurrent.futures import ProcessPoolExecutor, as_completed
from typing import Dict, List, Optional

_PROMPT_INSTRUCTION = "Please provide a self-contained Python script that solves the following problem in a markdown code block:"
_RESPONSE_PREFIX = "Below is a Python script with a self-contained function that solves the problem and passes corresponding tests:"
_SPLIT = "<<<tah-b200-code-split>>>"


def make_raw_chat_prompt_for_code_evaluation(task_prompt: str, reasoning: bool, tokenizer) -> str:
    if getattr(tokenizer, "chat_template", None) is None:
        return task_prompt
    user = f"{_PROMPT_INSTRUCTION}\n```\n{task_prompt.strip()}\n```\n"
    if reasoning:
        return tokenizer.apply_chat_template([{"role": "user", "content": user}], tokenize=False)
    primed = f"\n{_RESPONSE_PREFIX}\n```python\n{_SPLIT}\n```\n"
    text = tokenizer.apply_chat_template([{"role": "user", "content": user}, {"role": "assistant", "content": primed}],
                                         tokenize=False)
    return text.split(_SPLIT)[0]


_FENCE = re.compile(r"```(?:python|py)?\s*\n(.*?)```", re.S)


def _longest_parsable(code: str) -> str:
    lines = code.split("\n")
    for end in range(len(lines), 0, -1):
        chunk = "\n".join(lines[:end])
        try:
            ast.parse(chunk)
            return chunk
        except SyntaxError:
            continue
    return ""


def sanitize(text: str, entry_point: Optional[str] = None) -> str:
    """Extract runnable code from a model completion."""
    try:
        from evalplus.sanitize import sanitize as ep_sanitize
        return ep_sanitize(text, entry_point)
    except Exception:
        pass
    blocks = _FENCE.findall(text)
    code = max(blocks, key=len) if blocks else text
    if "```" in code:                      # unterminated fence: keep what precedes it
        code = code.split("```")[0]
    code = _longest_parsable(code)
    if not code or not entry_point:
        return code
    try:
        tree = ast.parse(code)
    except SyntaxError:
        return code
    defs = {n.name: n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef))}
    if entry_point not in defs:
        return code
    # keep imports, top-level assignments, and every definition reachable from the entry point
    wanted, stack = set(), [entry_point]
    while stack:
        name = stack.pop()
        if name in wanted or name not in defs:
            continue
        wanted.add(name)
        stack.extend(n.id for n in ast.walk(defs[name]) if isinstance(n, ast.Name))
    keep = [n for n in tree.body
            if isinstance(n, (ast.Import, ast.ImportFrom, ast.Assign, ast.AnnAssign))
            or (isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)) and n.name in wanted)]
    return "\n\n".join(ast.unparse(n) for n in keep)


def _run_one(task_id: str, completion_id: int, program: str, timeout: float) -> dict:
    """Execute ``program`` (solution + tests) in a fresh interpreter process."""
    import subprocess
    import sys
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "prog.py")
        with open(path, "w", encoding="utf-8") as fh:
            fh.write(program)
        try:
            res = subprocess.run([sys.executable, "-I", path], capture_output=True, text=True, timeout=timeout,
                                 cwd=tmp, env={"PATH": os.environ.get("PATH", ""), "PYTHONHASHSEED": "0"})
            ok = res.returncode == 0
            detail = "" if ok else (res.stderr or res.stdout)[-500:]
        except subprocess.TimeoutExpired:
            ok, detail = False, "timeout"
    return {"task_id": task_id, "completion_id": completion_id, "passed": ok, "detail": detail}


def _program_for(problem: dict, solution: str) -> str:
    test = problem.get("test") or ""
    entry = problem.get("entry_point") or ""
    tail = f"\ncheck({entry})\n" if "def check(" in test and entry else "\n"
    return f"{solution}\n\n{test}\n{tail}"


def estimate_pass_at_k(n: int, c: int, k: int) -> float:
    if n - c < k:
        return 1.0
    p = 1.0
    for i in range(n - c + 1, n + 1):
        p *= 1.0 - k / i
    return 1.0 - p


def _load_problems(dataset: str, problems_path: Optional[str]) -> Dict[str, dict]:
    if problems_path and os.path.exists(problems_path):
        with open(problems_path, encoding="utf-8") as fh:
            rows = [json.loads(line) for line in fh if line.strip()]
        return {str(r["task_id"]): r for r in rows}
    try:
        if dataset == "humaneval":
            from evalplus.data import get_human_eval_plus
            return dict(get_human_eval_plus())
        if dataset == "mbpp":
            from evalplus.data import get_mbpp_plus
            return dict(get_mbpp_plus())
    except ImportError as exc:
        raise RuntimeError("code evaluation needs either a local benchmark .jsonl (with 'test' and 'entry_point') "
                           "or the evalplus package") from exc
    raise ValueError(f"unknown code dataset {dataset!r}")


# ---------------------------------------------------------------------------------------------
# input/output grading against ground truth computed from the canonical solutions (the shape of the
# HumanEval+/MBPP+ data: ``prompt, canonical_solution, entry_point, base_input, plus_input, atol``)
# ---------------------------------------------------------------------------------------------
PASS, FAIL, TIMEOUT = "pass", "fail", "timeout"
DEFAULT_MIN_TIME_LIMIT = 4.0
DEFAULT_GT_TIME_LIMIT_FACTOR = 4.0
CACHE_DIR = os.environ.get("TAH_CODEEVAL_CACHE", os.path.join(os.path.expanduser("~"), ".cache", "tah_b200", "codeeval"))

_IO_RUNNER = '''
import copy, pickle, sys, time
src, entry, inputs = pickle.load(open(sys.argv[1], "rb"))
ns = {"__name__": "__solution__"}
outs, times = [], []
try:
    exec(src, ns)
    fn = ns[entry]
    for inp in inputs:
        t0 = time.time()
        try:
            outs.append(("ok", fn(*copy.deepcopy(inp))))
        except BaseException as exc:
            outs.append(("exc", type(exc).__name__))
        times.append(time.time() - t0)
        pickle.dump((outs, times), open(sys.argv[2], "wb"))
except BaseException as exc:
    pickle.dump(([("exc", type(exc).__name__)] * len(inputs), [0.0] * len(inputs)), open(sys.argv[2], "wb"))
'''


def _exec_on_inputs(source: str, entry_point: str, inputs: list, time_limit: float):
    """Run ``entry_point`` of ``source`` on every input in a fresh isolated interpreter.  Returns
    ``(outputs, seconds)``; outputs are ``("ok", value)`` / ``("exc", name)``, and fewer than ``len(inputs)``
    entries mean the time limit ran out."""
    import pickle
    import subprocess
    import sys
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        fin, fout, prog = (os.path.join(tmp, n) for n in ("in.pkl", "out.pkl", "run.py"))
        with open(fin, "wb") as fh:
            pickle.dump((source, entry_point, inputs), fh)
        with open(prog, "w", encoding="utf-8") as fh:
            fh.write(_IO_RUNNER)
        try:
            subprocess.run([sys.executable, "-I", prog, fin, fout], capture_output=True, timeout=time_limit, cwd=tmp,
                           env={"PATH": os.environ.get("PATH", ""), "PYTHONHASHSEED": "0"})
        except subprocess.TimeoutExpired:
            pass
        if not os.path.exists(fout):
            return [], []
        try:
            with open(fout, "rb") as fh:
                return pickle.load(fh)
        except Exception:
            return [], []


def _same(a, b, atol: float) -> bool:
    if atol and isinstance(a, (int, float)) and isinstance(b, (int, float)) and not isinstance(a, bool):
        return abs(a - b) <= atol
    if atol and isinstance(a, (list, tuple)) and isinstance(b, (list, tuple)) and len(a) == len(b):
        return all(_same(x, y, atol) for x, y in zip(a, b))
    return a == b


def get_groundtruth(problems: Dict[str, dict], hashcode: str) -> Dict[str, dict]:
    """Expected outputs (and their run time) of every problem's canonical solution on its ``base_input`` and
    ``plus_input``; cached on disk under ``CACHE_DIR/<hashcode>.pkl`` (reference ``codeeval.py:94-125``)."""
    import pickle
    cache = os.path.join(CACHE_DIR, f"{hashcode}.pkl")
    if os.path.exists(cache):
        with open(cache, "rb") as fh:
            return pickle.load(fh)
    expected = {}
    for task_id, pb in problems.items():
        src = pb["prompt"] + pb["canonical_solution"]
        rec = {}
        for which in ("base", "plus"):
            inputs = pb.get(f"{which}_input") or []
            outs, times = _exec_on_inputs(src, pb["entry_point"], inputs, 600.0)
            rec[which] = [o[1] if o[0] == "ok" else None for o in outs]
            rec[f"{which}_time"] = times
        expected[task_id] = rec
    os.makedirs(CACHE_DIR, exist_ok=True)
    with open(cache, "wb") as fh:
        pickle.dump(expected, fh)
    return expected


def _check_io(task_id: str, completion_id: int, problem: dict, solution: str, expected: dict, base_only: bool,
              min_time_limit: float, gt_time_limit_factor: float) -> dict:
    out = {"task_id": task_id, "completion_id": completion_id, "solution": solution}
    for which in (("base",) if base_only else ("base", "plus")):
        inputs = problem.get(f"{which}_input") or []
        want = expected[which]
        limit = sum(max(min_time_limit, gt_time_limit_factor * t) for t in expected[f"{which}_time"]) + 2.0
        got, _ = _exec_on_inputs(solution, problem["entry_point"], inputs, limit)
        details = [g[0] == "ok" and _same(g[1], w, problem.get("atol", 0) or 0) for g, w in zip(got, want)]
        if len(got) < len(inputs):
            stat = TIMEOUT
        else:
            stat = PASS if all(details) else FAIL
        out[which] = (stat, details)
    return out


def _dataset_hash(problems: Dict[str, dict]) -> str:
    import hashlib
    h = hashlib.md5()
    for t in sorted(problems):
        h.update(repr((t, problems[t].get("prompt"), problems[t].get("canonical_solution"),
                       problems[t].get("base_input"), problems[t].get("plus_input"))).encode())
    return h.hexdigest()


def _pass_at_k(totals: List[int], corrects: List[int], ks) -> Dict[str, float]:
    return {f"pass@{k}": sum(estimate_pass_at_k(n, c, k) for n, c in zip(totals, corrects)) / len(totals)
            for k in ks if totals and min(totals) >= k}


def _result_path(samples: str, output_file: Optional[str]) -> str:
    if output_file:
        return output_file
    if os.path.isdir(samples):
        return os.path.join(samples, "eval_results.json")
    legacy = samples.replace(".jsonl", "_eval_results.json")
    return legacy if os.path.exists(legacy) else samples.replace(".jsonl", ".eval_results.json")


def _load_solutions(samples: str) -> List[dict]:
    files = [samples]
    if os.path.isdir(samples):
        files = sorted(os.path.join(samples, f) for f in os.listdir(samples) if f.endswith(".jsonl"))
    rows = []
    for f in files:
        with open(f, encoding="utf-8") as fh:
            rows += [json.loads(line) for line in fh if line.strip()]
    return rows


def evaluate(dataset: str, samples: str, problems_path: Optional[str] = None, parallel: Optional[int] = None,
             timeout: float = 20.0, ks=(1, 10, 100), stall_warning_s: float = 100.0, *, base_only: bool = False,
             test_details: bool = False, min_time_limit: float = DEFAULT_MIN_TIME_LIMIT,
             gt_time_limit_factor: float = DEFAULT_GT_TIME_LIMIT_FACTOR, output_file: Optional[str] = None) -> dict:
    """Grade a solutions file (one ``{"task_id", "solution" | "completion"}`` JSON object per line, or a
    directory of such files) and write ``pass@k`` (reference ``codeeval.py:161-305``).

    Problems that carry ``base_input`` / ``plus_input`` (the HumanEval+/MBPP+ shape) are graded by comparing the
    solution's outputs with those of the canonical solution (cached ground truth), on the base inputs and,
    unless ``base_only``, on the extra "plus" inputs: ``pass_at_k = {"base": ..., "plus": ...}``.  Problems that
    only ship a ``test`` program are graded by running it (``pass_at_k = {"base": ...}``).  An existing result
    file is loaded instead of re-running."""
    result_path = _result_path(samples, output_file)
    if os.path.isfile(result_path):
        with open(result_path, encoding="utf-8") as fh:
            out = json.load(fh)
        print(f"Loaded previous results from {result_path}: {out.get('pass_at_k')}")
        return out
    problems = _load_problems(dataset, problems_path)
    io_mode = bool(problems) and all("base_input" in p and "canonical_solution" in p for p in problems.values())
    rows = _load_solutions(samples)
    per_task: Dict[str, List[str]] = defaultdict(list)
    for r in rows:
        tid = str(r["task_id"])
        if tid not in problems:
            print(f"Warning: task {tid} in samples but not in dataset")
            continue
        per_task[tid].append(r.get("solution") or (problems[tid].get("prompt", "") + r.get("completion", "")))
    missing = [t for t in problems if t not in per_task]
    if missing:
        print(f"Warning: {len(missing)} tasks have no sample (e.g. {missing[:3]})")
    expected = get_groundtruth(problems, _dataset_hash(problems)) if io_mode else None
    results: Dict[str, List[dict]] = defaultdict(list)
    last_done = [time.time()]
    stop = threading.Event()

    def watchdog():
        while not stop.wait(10.0):
            if time.time() - last_done[0] > stall_warning_s:
                print(f"Warning: no code sample finished in the last {stall_warning_s:.0f} s")
                last_done[0] = time.time()

    threading.Thread(target=watchdog, daemon=True).start()
    n_workers = parallel or max(1, (os.cpu_count() or 2) // 2)
    ctx = mp.get_context("spawn")
    with ProcessPoolExecutor(max_workers=n_workers, mp_context=ctx) as pool:
        futs = []
        for task_id, sols in per_task.items():
            for cid, sol in enumerate(sols):
                if io_mode:
                    futs.append(pool.submit(_check_io, task_id, cid, problems[task_id], sol, expected[task_id], base_only,
                                            min_time_limit, gt_time_limit_factor))
                else:
                    futs.append(pool.submit(_run_one, task_id, cid, _program_for(problems[task_id], sol), timeout))
        for f in as_completed(futs):
            r = f.result()
            results[r["task_id"]].append(r)
            last_done[0] = time.time()
    stop.set()
    ev: Dict[str, List[dict]] = {}
    for t, v in results.items():
        v.sort(key=lambda r: r["completion_id"])
        if io_mode:
            ev[t] = []
            for r in v:
                rec = {"task_id": t, "solution": r["solution"], "base_status": r["base"][0],
                       "plus_status": None if base_only else r["plus"][0]}
                for which in (("base",) if base_only else ("base", "plus")):
                    stat, details = r[which]
                    inputs = problems[t].get(f"{which}_input") or []
                    bad = [i for i, ok in enumerate(details) if not ok]
                    rec[f"{which}_fail_tests"] = ([inputs[i] for i in bad] if test_details else [inputs[i] for i in bad[-1:]]) \
                        if stat != PASS else []
                ev[t].append(rec)
        else:
            ev[t] = [{"task_id": t, "completion_id": r["completion_id"], "base_status": PASS if r["passed"] else FAIL,
                      "plus_status": None, "passed": r["passed"], "detail": r["detail"]} for r in v]
    totals = [len(v) for v in ev.values()]
    base_ok = [sum(1 for r in v if r["base_status"] == PASS) for v in ev.values()]
    pass_at_k = {"base": _pass_at_k(totals, base_ok, ks)}
    if io_mode and not base_only:
        both = [sum(1 for r in v if r["base_status"] == PASS and r["plus_status"] == PASS) for v in ev.values()]
        pass_at_k["plus"] = _pass_at_k(totals, both, ks)
    out = {"date": time.strftime("%Y-%m-%d %H:%M"), "dataset": dataset, "n_tasks": len(ev), "pass_at_k": pass_at_k,
           "eval": ev}
    with open(result_path, "w", encoding="utf-8") as fh:
        json.dump(out, fh, indent=1, default=repr)
    for name, v in pass_at_k.items():
        print(f"{dataset} ({name} tests): {v}")
    return out
