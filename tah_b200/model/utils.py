"""Generation loop, sampler front-end and small training utilities.

Same call surface as the reference helper module (reference ``tah/model/utils.py``):
``set_all_seeds``, ``freeze_components``, ``compute_trainable_param_size_gb``,
``sample_next_token``, ``IterCountColors``, ``TaHForCasualLM_generate`` (the
spelling is the reference's).  On a CUDA device ``TaHForCasualLM_generate`` runs
on the paged-KV inference engine (:mod:`tah_b200.engine`), which produces the same
token streams as the token-by-token loop below; the loop is the CPU path and the
parity oracle for the engine.
"""
from __future__ import annotations

import os
import random
from typing import List, Optional

import numpy as np
import torch

from tah_b200 import ops


def set_all_seeds(seed: int = 42, verbose: bool = True) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    os.environ["PYTHONHASHSEED"] = str(seed)
    if verbose:
        print(f"All random seeds set to {seed}")


def _get_attr_by_path(root, path: str):
    obj = root
    for name in path.split("."):
        if not hasattr(obj, name):
            return None
        obj = getattr(obj, name)
    return obj


def freeze_components(model, component_paths, accelerator=None) -> None:
    """Freeze sub-modules named by dotted paths (a leading ``model.`` is dropped).
    Missing paths are reported, not raised (reference ``utils.py:50-71``)."""
    say = accelerator.print if accelerator is not None and hasattr(accelerator, "print") else print
    for raw in component_paths or ():
        path = raw[len("model."):] if raw.startswith("model.") else raw
        target = _get_attr_by_path(model, path)
        if target is None:
            say(f"Warning: freeze_component {raw!r} not found on model.")
            continue
        params = list(target.parameters()) if hasattr(target, "parameters") else []
        if not params:
            say(f"Warning: freeze_component {raw!r} has no parameters to freeze.")
            continue
        for p in params:
            p.requires_grad = False
        say(f"Froze component {raw!r} ({sum(p.numel() for p in params):,} params).")


def compute_trainable_param_size_gb(model) -> float:
    return sum(p.numel() * p.element_size() for p in model.parameters() if p.requires_grad) / 1024 ** 3


def sample_next_token(logits: torch.Tensor, temperature: float = 1.0, top_p: float = 1.0, top_k: int = 0,
                      min_p: float = 0.0, do_sample: bool = True, generator=None) -> torch.Tensor:
    """One token per row of ``(B, V)`` logits: temperature -> softmax -> min_p -> top_k -> top_p -> draw."""
    return ops.sample(logits, temperature, top_p, top_k, min_p, do_sample, generator)


class IterCountColors:
    """ANSI colour per iteration count, for the playground printer."""

    _COLORS = {1: "\033[0m", 2: "\033[92m", 3: "\033[94m", 4: "\033[91m", 5: "\033[95m", 6: "\033[93m"}
    _OVERFLOW = "\033[96m"

    @classmethod
    def get_color(cls, n: int) -> str:
        return cls._COLORS.get(n, cls._OVERFLOW)

    @classmethod
    def print_token(cls, token_text: str, n: int) -> None:
        print(f"{cls.get_color(n)}{token_text}\033[0m", end="", flush=True)

    @classmethod
    def get_legend(cls) -> str:
        return "Color legend: " + ", ".join(f"{cls.get_color(n)}={n} iter\033[0m" for n in range(1, 8))


def _print_counts(tokenizer, ids, counts, attention_mask):
    counts = counts[0]
    row = ids[0]
    if attention_mask is not None:
        keep = attention_mask[0, -counts.shape[0]:] == 1
        row, counts = row[keep], counts[keep]
    for tok, c in zip(row.tolist(), counts.tolist()):
        IterCountColors.print_token(tokenizer.decode([tok]), int(c))


def generate_loop(tah_model, tokenizer, model_inputs: dict, *, max_new_tokens: int = 1024, do_sample: bool = True,
                  temperature: float = 1.0, top_p: float = 1.0, top_k: int = 0, min_p: float = 0.0,
                  verbose: bool = True, eos_token_id: Optional[int] = None, generator=None, **kwargs):
    """Token-by-token loop over ``TaHForCausalLM.forward`` with a dense ``TaHCache``."""
    ids = model_inputs["input_ids"]
    device, B = ids.device, ids.shape[0]
    tah_model.eval()
    eos = eos_token_id if eos_token_id is not None else getattr(tokenizer, "eos_token_id", None)
    out_tokens: List[List[int]] = [[] for _ in range(B)]
    iter_counts: List[List[int]] = [[] for _ in range(B)]
    finished = torch.zeros(B, dtype=torch.bool, device=device)
    attn = model_inputs.get("attention_mask")
    if verbose:
        print("Input tokens with iteration counts:")
    with torch.no_grad():
        out = tah_model(input_ids=ids, attention_mask=attn, use_cache=True, new_sequence=True, **kwargs)
        if verbose:
            _print_counts(tokenizer, ids, out.iter_count, attn)
            print("\n\nGenerating new tokens:")
        cache = out.past_key_values
        for _ in range(max_new_tokens):
            nxt = sample_next_token(out.logits[:, -1, :], temperature, top_p, top_k, min_p, do_sample, generator)
            if eos is not None:
                finished = finished | (nxt == eos)
            alive = (~finished).tolist()
            for i, tok in enumerate(nxt.tolist()):
                if alive[i]:
                    out_tokens[i].append(int(tok))
            if bool(finished.all()):
                break
            if attn is not None:
                attn = torch.cat([attn, attn.new_ones(B, 1)], dim=1)
            out = tah_model(input_ids=nxt.unsqueeze(1), attention_mask=attn, past_key_values=cache,
                            use_cache=True, new_sequence=False, **kwargs)
            cache = out.past_key_values
            for i, c in enumerate(out.iter_count[:, -1].tolist()):
                if alive[i]:
                    iter_counts[i].append(int(c))
            if verbose:
                _print_counts(tokenizer, nxt.unsqueeze(1), out.iter_count, None)
    if verbose:
        print("\033[0m")
    texts = [tokenizer.decode(t) if (t and tokenizer is not None) else "" for t in out_tokens]
    return out_tokens, texts


def TaHForCasualLM_generate(tah_model, tokenizer, model_inputs: dict, *, max_new_tokens: int = 1024,
                            do_sample: bool = True, temperature: float = 1.0, top_p: float = 1.0, top_k: int = 0,
                            min_p: float = 0.0, verbose: bool = True, **kwargs):
    """Batched generation; returns ``(token id lists, decoded strings)`` (reference ``utils.py:196-264``).

    The EOS token is not appended; a finished row keeps being stepped until every
    row has finished or ``max_new_tokens`` is reached.  Extra keyword ``engine``:
    ``"auto"`` (default: the paged-KV engine on CUDA, the loop elsewhere), ``"loop"``, ``"paged"``.
    """
    engine = kwargs.pop("engine", "auto")
    ids = model_inputs["input_ids"]
    use_engine = engine == "paged" or (engine == "auto" and ids.is_cuda and not verbose
                                       and os.environ.get("TAH_B200_FORCE_TORCH", "0") != "1")
    if use_engine:
        from tah_b200.engine import get_engine
        eng = get_engine(tah_model)
        res = eng.generate(ids, model_inputs.get("attention_mask"), max_new_tokens=max_new_tokens,
                           do_sample=do_sample, temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p,
                           eos_token_id=kwargs.pop("eos_token_id", getattr(tokenizer, "eos_token_id", None)))
        texts = [tokenizer.decode(t) if (t and tokenizer is not None) else "" for t in res.tokens]
        return res.tokens, texts
    return generate_loop(tah_model, tokenizer, model_inputs, max_new_tokens=max_new_tokens, do_sample=do_sample,
                         temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p, verbose=verbose, **kwargs)
