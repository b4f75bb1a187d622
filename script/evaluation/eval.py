#!/usr/bin/env python
"""Evaluation CLI: fan a benchmark out over GPU jobs, generate, grade, merge.

    python script/evaluation/eval.py --eval_config script/recipes/qwen3_1.7/eval_tah.yaml \
        --model_path <ckpt> --backend tah --dataset_name gsm8k --job_nums 8 --tp_size_per_job 1
"""
import argparse
import logging
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description="TaH evaluation")
    ap.add_argument("--eval_config", required=True)
    ap.add_argument("--model_path", required=True)
    ap.add_argument("--backend", default="tah", choices=["sglang", "hf", "tah"])
    ap.add_argument("--dataset_name", required=True, help="registered benchmark name(s), comma separated")
    ap.add_argument("--job_nums", type=int, default=8)
    ap.add_argument("--tp_size_per_job", type=int, default=1)
    ap.add_argument("--output_dir", default="output/eval")
    ap.add_argument("--data_range", type=int, nargs="*", default=None, help="[end] or [start end), end exclusive")
    ap.add_argument("--data_ids", default=None, help="comma separated <dataset>_<original_id>")
    ap.add_argument("--del_job_dir", type=bool, default=False)
    ap.add_argument("--logger_level", default="INFO")
    ap.add_argument("--random_seed", type=int, default=42)
    return ap.parse_args(argv)


def main(argv=None):
    args = parse_args(argv)
    logging.basicConfig(level=args.logger_level.upper())
    from tah_b200.evaluate import allocate_gpus_and_run_jobs
    return allocate_gpus_and_run_jobs(args)


if __name__ == "__main__":
    main()
