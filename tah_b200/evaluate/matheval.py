"""Rule-based math graders over ``math_verify``.

Three ground-truth shapes: a bare expression (AIME, GSM8K), LaTeX (MATH-500, AMC, OlympiadBench,
Minerva) and a string / multiple-choice letter (GPQA, MMLU, ARC).  ``evaluator_map`` assigns a
grader to each registered benchmark (mapping of reference ``tah/evaluate/matheval.py:99-117``).
``math_verify`` is imported lazily so that the rest of the package works without it.
"""
from __future__ import annotations

from typing import Tuple


class MathEvaluator:
    def __init__(self, mode: str):
        if mode not in ("expr", "latex", "string"):
            raise ValueError(f"unsupported grader mode {mode!r}")
        self.mode = mode

    @staticmethod
    def _output_configs():
        from latex2sympy2_extended import NormalizationConfig
        from math_verify import ExprExtractionConfig, LatexExtractionConfig
        norm = NormalizationConfig(nits=False, malformed_operators=False, basic_latex=True, boxed="all", units=True)
        return [LatexExtractionConfig(normalization_config=norm, boxed_match_priority=0,
                                      try_extract_without_anchor=False), ExprExtractionConfig()]

    def rule_judge(self, solution: str, ground_truth: str) -> Tuple[bool, str]:
        """``(is_correct, extracted answer | "No extracted answer")``."""
        from math_verify import (ExprExtractionConfig, LatexExtractionConfig, StringExtractionConfig, parse,
                                 verify)
        if self.mode == "string":
            gold = parse(ground_truth, extraction_config=[StringExtractionConfig()])
            answer = parse(solution, extraction_config=[StringExtractionConfig()])
        else:
            if self.mode == "latex":
                if not ground_truth.startswith("$"):
                    ground_truth = f"${ground_truth}$"
                gold = parse(ground_truth, extraction_config=[LatexExtractionConfig()])
            else:
                gold = parse(ground_truth, extraction_config=[ExprExtractionConfig()])
            # math answers: the first match in the output decides
            answer = parse(solution, extraction_config=self._output_configs(), extraction_mode="first_match")
        if not answer:
            return False, "No extracted answer"
        return bool(verify(gold, answer)), str(answer)


_EXPR, _LATEX, _STRING = MathEvaluator("expr"), MathEvaluator("latex"), MathEvaluator("string")

evaluator_map = {
    "aime24": _EXPR, "aime25": _EXPR, "brumo25": _EXPR, "gsm8k": _EXPR,
    "math500": _LATEX, "amc23": _LATEX, "chmath": _LATEX, "olympiadbench": _LATEX, "minerva": _LATEX,
    "gpqa": _STRING, "mmlu_stem": _STRING, "mmlu_redux": _STRING, "arc_e": _STRING, "arc_c": _STRING,
}
