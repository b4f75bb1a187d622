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


def evaluate(dataset: str, samples: str, problems_path: Optional[str] = None, parallel: Optional[int] = None,
             timeout: float = 20.0, ks=(1, 10, 100), stall_warning_s: float = 100.0) -> dict:
    """Grade a solutions file (one ``{"task_id", "solution"}`` JSON object per line)."""
    problems = _load_problems(dataset, problems_path)
    with open(samples, encoding="utf-8") as fh:
        rows = [json.loads(line) for line in fh if line.strip()]
    per_task: Dict[str, List[str]] = defaultdict(list)
    for r in rows:
        per_task[str(r["task_id"])].append(r["solution"])
    missing = [t for t in problems if t not in per_task]
    if missing:
        print(f"Warning: {len(missing)} tasks have no sample (e.g. {missing[:3]})")
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
            if task_id not in problems:
                continue
            for cid, sol in enumerate(sols):
                futs.append(pool.submit(_run_one, task_id, cid, _program_for(problems[task_id], sol), timeout))
        for f in as_completed(futs):
            r = f.result()
            results[r["task_id"]].append(r)
            last_done[0] = time.time()
    stop.set()
    totals = [len(v) for v in results.values()]
    corrects = [sum(1 for r in v if r["passed"]) for v in results.values()]
    pass_at_k = {}
    for k in ks:
        if totals and min(totals) >= k:
            pass_at_k[f"pass@{k}"] = sum(estimate_pass_at_k(n, c, k) for n, c in zip(totals, corrects)) / len(totals)
    out = {"dataset": dataset, "n_tasks": len(results), "pass_at_k": pass_at_k,
           "eval": {t: sorted(v, key=lambda r: r["completion_id"]) for t, v in results.items()}}
    with open(samples.replace(".jsonl", "_eval_results.json"), "w", encoding="utf-8") as fh:
        json.dump(out, fh, indent=1)
    print(f"{dataset}: {pass_at_k}")
    return out
