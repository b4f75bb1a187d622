#!/usr/bin/env python
"""Load a TaH checkpoint and generate with per-token iteration counts shown in colour.

    python script/playground/inference_example.py --model nics-efc/TaH-plus-1.7B --max_new_tokens 512

With ``--random_init`` a tiny random model is used (no download), which is enough to see the
engine and the colouring at work.
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from tah_b200 import TaHForCausalLM  # noqa: E402
from tah_b200.model.utils import IterCountColors, TaHForCasualLM_generate  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="nics-efc/TaH-plus-1.7B")
    ap.add_argument("--prompt", default="What is the sum of the first 20 positive odd integers?")
    ap.add_argument("--max_new_tokens", type=int, default=512)
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--top_p", type=float, default=0.95)
    ap.add_argument("--top_k", type=int, default=20)
    ap.add_argument("--random_init", action="store_true")
    a = ap.parse_args()
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    if a.random_init:
        from tests.helpers import tiny_tah
        model = tiny_tah(dtype=torch.bfloat16 if dev == "cuda" else torch.float32).to(dev)

        class Tok:
            eos_token_id = None
            def decode(self, ids):
                return " ".join(f"<{i}>" for i in ids)
        tok = Tok()
        inputs = {"input_ids": torch.randint(0, 1024, (1, 16), device=dev)}
    else:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.model)
        model = TaHForCausalLM.from_pretrained(a.model, torch_dtype=torch.bfloat16, device_map="auto")
        text = tok.apply_chat_template([{"role": "user", "content": a.prompt}], tokenize=False, add_generation_prompt=True)
        inputs = {k: v.to(model.device) for k, v in tok(text, return_tensors="pt").items()}
    print(IterCountColors.get_legend())
    TaHForCasualLM_generate(model, tok, inputs, max_new_tokens=a.max_new_tokens, do_sample=a.temperature > 0,
                            temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, verbose=True, engine="loop")


if __name__ == "__main__":
    main()
