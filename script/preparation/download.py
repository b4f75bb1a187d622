#!/usr/bin/env python
"""Fetch the OpenR1-Math-220k dataset snapshot with exponential-backoff retries.

    python script/preparation/download.py [--repo open-r1/OpenR1-Math-220k] [--out data/raw/openr1]

``HF_MIRROR=<url>`` selects a hub mirror (sets ``HF_ENDPOINT``).
"""
import argparse
import os
import time


def download_with_retry(repo_id: str, local_dir: str, repo_type: str = "dataset", max_attempts: int = 100,
                        base_delay: float = 1.0, max_delay: float = 300.0, downloader=None) -> str:
    if downloader is None:
        from huggingface_hub import snapshot_download as downloader
    delay = base_delay
    for attempt in range(1, max_attempts + 1):
        try:
            return downloader(repo_id=repo_id, repo_type=repo_type, local_dir=local_dir)
        except Exception as exc:  # network errors of any kind: wait and retry
            if attempt == max_attempts:
                raise
            print(f"attempt {attempt} failed ({type(exc).__name__}: {exc}); retrying in {delay:.0f} s")
            time.sleep(delay)
            delay = min(max_delay, delay * 2)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo", default="open-r1/OpenR1-Math-220k")
    ap.add_argument("--out", default="data/raw/openr1_math")
    a = ap.parse_args()
    if os.environ.get("HF_MIRROR"):
        os.environ["HF_ENDPOINT"] = os.environ["HF_MIRROR"]
    print(download_with_retry(a.repo, a.out))
