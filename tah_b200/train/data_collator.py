"""Batch collation for TaH SFT.

Pads ``input_ids`` (pad token), ``attention_mask`` (0), ``labels`` (-100) and the TaH-specific
``iter_count_labels`` (-100) to the longest example, on the tokenizer's padding side
(behaviour of reference ``tah/train/data_collator.py:25-81``, without the HuggingFace base collator).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


class CustomTaHDataCollator:
    def __init__(self, tokenizer=None, padding=True, max_length: Optional[int] = None,
                 pad_to_multiple_of: Optional[int] = None, label_pad_token_id: int = -100,
                 return_tensors: str = "pt", pad_token_id: Optional[int] = None, padding_side: Optional[str] = None):
        self.tokenizer = tokenizer
        self.padding = padding
        self.max_length = max_length
        self.pad_to_multiple_of = pad_to_multiple_of
        self.label_pad_token_id = label_pad_token_id
        self.return_tensors = return_tensors
        pid = pad_token_id if pad_token_id is not None else getattr(tokenizer, "pad_token_id", None)
        self.pad_token_id = 0 if pid is None else pid
        self.padding_side = padding_side or getattr(tokenizer, "padding_side", "right")

    def _pad(self, rows: List[List[int]], value: int, width: int) -> torch.Tensor:
        out = torch.full((len(rows), width), value, dtype=torch.long)
        for i, r in enumerate(rows):
            r = list(r)[:width]
            if self.padding_side == "right":
                out[i, :len(r)] = torch.as_tensor(r, dtype=torch.long)
            else:
                out[i, width - len(r):] = torch.as_tensor(r, dtype=torch.long)
        return out

    def __call__(self, features: List[Dict], return_tensors=None) -> Dict[str, torch.Tensor]:
        width = max(len(f["input_ids"]) for f in features)
        if self.max_length is not None and self.padding == "max_length":
            width = self.max_length
        if self.pad_to_multiple_of:
            m = self.pad_to_multiple_of
            width = (width + m - 1) // m * m
        batch = {"input_ids": self._pad([f["input_ids"] for f in features], self.pad_token_id, width)}
        batch["attention_mask"] = self._pad([f.get("attention_mask", [1] * len(f["input_ids"])) for f in features], 0, width)
        if "labels" in features[0]:
            batch["labels"] = self._pad([f["labels"] for f in features], self.label_pad_token_id, width)
        if "iter_count_labels" in features[0]:
            batch["iter_count_labels"] = self._pad([f["iter_count_labels"] for f in features],
                                                   self.label_pad_token_id, width)
        return batch
