"""TaHCache: K/V, positions and validity per ``(layer, iteration depth)`` slot.

Keeps the accessor names of the reference cache (reference
``tah/model/causal_cache.py:30-239``) so analysis code written against it keeps
working, but it is a plain class (no HuggingFace ``DynamicCache`` base) and it
doubles as the attention context of a backbone pass: the model calls
:meth:`begin_pass` and every layer calls :meth:`attend`, which stores the pass's
K/V in slot ``(layer, depth)`` and attends over slots ``0..depth`` under the
duo-causal rule.  Because only slots of depth ``<= current`` are visible, a
depth-0 query never sees depth->=1 entries, in prefill or decode.

K/V are stored ``[B, T, n_kv_heads, head_dim]`` and are *not* detached: in training
a later pass back-propagates into an earlier pass's K/V projections.

This dense cache serves the PyTorch path (training, CPU, parity tests).  The
inference engine uses the paged cache in :mod:`tah_b200.engine.kv_cache`.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from tah_b200 import ops
from tah_b200.models.qwen3 import PassKV

_Slot = Tuple[int, int]


class TaHCache(PassKV):
    def __init__(self):
        self._k: Dict[_Slot, torch.Tensor] = {}
        self._v: Dict[_Slot, torch.Tensor] = {}
        self._pos: Dict[_Slot, torch.Tensor] = {}
        self._valid: Dict[_Slot, torch.Tensor] = {}
        self.current_iter_depth: int = 0
        self.position_ids_to_cache: Optional[torch.Tensor] = None
        self.valid_mask_to_cache: Optional[torch.Tensor] = None
        self.batch_size: Optional[int] = None
        self._store_pass: bool = True
        self._seg_meta = None
        self._appended = False         # a slot has been extended by a later forward (decode with this cache)
        self._device = torch.device("cpu")
        self._dtype = torch.bfloat16

    # ---- pass protocol ---------------------------------------------------------------
    def begin_pass(self, iter_depth: int, position_ids: torch.Tensor, valid_mask: torch.Tensor, store: bool = True):
        self.current_iter_depth = iter_depth
        self.position_ids_to_cache = position_ids
        self.valid_mask_to_cache = valid_mask
        self._store_pass = store
        self._seg_meta = None          # index arrays of the tensor-core attention path, built once per pass

    def _segments(self, layer_idx: int, k, v):
        """Per-depth K/V, positions and validity visible to this pass (this pass's own last)."""
        d = self.current_iter_depth
        ks, vs, ps, ms = [], [], [], []
        for i in range(d + 1):
            if (layer_idx, i) in self._k and not (i == d and self._store_pass):
                ks.append(self._k[(layer_idx, i)]); vs.append(self._v[(layer_idx, i)])
                ps.append(self._pos[(layer_idx, i)]); ms.append(self._valid[(layer_idx, i)])
        own_new = self._store_pass and (layer_idx, d) in self._k
        if own_new or (not self._store_pass and ks and (layer_idx, d) in self._k):
            return None                  # slot d already holds earlier tokens: not a from-scratch pass
        ks.append(k); vs.append(v)
        ps.append(self.position_ids_to_cache); ms.append(self.valid_mask_to_cache)
        return ks, vs, ps, ms

    def _attend_segments(self, layer_idx: int, q, k, v):
        """Tensor-core path (CUDA, bf16, from-scratch forward: every slot holds one pass's tokens, whose
        valid entries are contiguous and in position order).  Returns None when it does not apply."""
        import os
        from tah_b200.ops import autograd_ops
        if not q.is_cuda or os.environ.get("TAH_B200_FORCE_TORCH", "0") == "1" or self._appended:
            return None
        seg = self._segments(layer_idx, k, v)
        if seg is None or not autograd_ops.segment_attention_ok(q, len(seg[0])):
            return None
        ks, vs, ps, ms = seg
        if self._seg_meta is None:
            self._seg_meta = autograd_ops.SegmentMeta(self.position_ids_to_cache, ps, ms,
                                                      q_valid=self.valid_mask_to_cache)
        out = autograd_ops.segment_attention(q, ks, vs, self._seg_meta)
        if self._store_pass:
            self.update(k, v, layer_idx)
        return out

    def attend(self, layer_idx: int, q, k, v):
        d = self.current_iter_depth
        pos_new, valid_new = self.position_ids_to_cache, self.valid_mask_to_cache
        fast = self._attend_segments(layer_idx, q, k, v)
        if fast is not None:
            return fast
        if self._store_pass:
            ks, vs = self.update(k, v, layer_idx)
            kv_pos = self.get_position_id_upto_iter(layer_idx, d, init_batch_size=q.shape[0])
            kv_valid = self.get_valid_mask_upto_iter(layer_idx, d, init_batch_size=q.shape[0])
        else:
            # last pass of a forward that keeps no cache: attend over the stored slots
            # (slot (layer, d) may hold earlier tokens of this depth) plus this pass's K/V
            pk, pv = self.get_cache_upto_iter(layer_idx, d)
            ks = k if pk is None else torch.cat([pk, k], dim=1)
            vs = v if pv is None else torch.cat([pv, v], dim=1)
            kv_pos = torch.cat([self.get_position_id_upto_iter(layer_idx, d, q.shape[0]).to(pos_new.device), pos_new], dim=-1)
            kv_valid = torch.cat([self.get_valid_mask_upto_iter(layer_idx, d, q.shape[0]).to(valid_new.device), valid_new], dim=-1)
        return ops.duo_attention(q, ks, vs, pos_new, kv_pos, kv_valid)

    # ---- write -----------------------------------------------------------------------
    def has_layer(self, layer_idx: int = 0) -> bool:
        return any(l == layer_idx for (l, _) in self._k)

    def update(self, key_states, value_states, layer_idx: int, cache_kwargs=None):
        """Append to slot ``(layer_idx, current_iter_depth)``; return K/V over depths ``0..current``."""
        if self.batch_size is None:
            self.batch_size = key_states.shape[0]
        elif key_states.shape[0] != self.batch_size:
            raise AssertionError(f"batch size mismatch: cached {self.batch_size}, got {key_states.shape[0]}")
        self._device, self._dtype = key_states.device, key_states.dtype
        slot = (layer_idx, self.current_iter_depth)
        if slot in self._k:
            self._appended = True
            self._k[slot] = torch.cat([self._k[slot], key_states], dim=1)
            self._v[slot] = torch.cat([self._v[slot], value_states], dim=1)
            self._pos[slot] = torch.cat([self._pos[slot], self.position_ids_to_cache], dim=-1)
            self._valid[slot] = torch.cat([self._valid[slot], self.valid_mask_to_cache], dim=-1)
        else:
            self._k[slot], self._v[slot] = key_states, value_states
            self._pos[slot], self._valid[slot] = self.position_ids_to_cache, self.valid_mask_to_cache
        return self.get_cache_upto_iter(layer_idx, self.current_iter_depth)

    # ---- read views ------------------------------------------------------------------
    def get_cache_upto_iter(self, layer_idx: int, upto_iter_idx: int):
        ks = [self._k[(layer_idx, i)] for i in range(upto_iter_idx + 1) if (layer_idx, i) in self._k]
        if not ks:
            return None, None
        vs = [self._v[(layer_idx, i)] for i in range(upto_iter_idx + 1) if (layer_idx, i) in self._v]
        if len(ks) == 1:
            return ks[0], vs[0]
        return torch.cat(ks, dim=1), torch.cat(vs, dim=1)

    def _meta(self, store, layer_idx, upto, batch):
        parts = []
        for i in range(upto + 1):
            t = store.get((layer_idx, i))
            if t is None:
                parts.append(torch.empty((batch, 0), device=self.device, dtype=torch.long))
            else:
                batch = t.shape[0]
                parts.append(t)
        return torch.cat(parts, dim=-1)

    def get_position_id_upto_iter(self, layer_idx: int, upto_iter_idx: int, init_batch_size: int = 1):
        return self._meta(self._pos, layer_idx, upto_iter_idx, init_batch_size)

    def get_valid_mask_upto_iter(self, layer_idx: int, upto_iter_idx: int, init_batch_size: int = 1):
        return self._meta(self._valid, layer_idx, upto_iter_idx, init_batch_size)

    def get_cache_iter_index_upto_iter(self, layer_idx: int, upto_iter_idx: int) -> torch.Tensor:
        """Depth of every visible KV entry, in storage order (``[depth-0 ... | depth-1 ... | ...]``)."""
        lens = [self.get_cache_length(layer_idx, i) for i in range(upto_iter_idx + 1)]
        pieces = [torch.full((n,), i, device=self.device, dtype=torch.long) for i, n in enumerate(lens) if n > 0]
        return torch.cat(pieces) if pieces else torch.empty((0,), device=self.device, dtype=torch.long)

    # ---- lengths ---------------------------------------------------------------------
    def get_cache_length(self, layer_idx: Optional[int] = 0, iter_idx: Optional[int] = None) -> int:
        if iter_idx is not None:
            t = self._k.get((layer_idx, iter_idx))
            return 0 if t is None else t.shape[1]
        return sum(t.shape[1] for (l, _), t in self._k.items() if l == layer_idx)

    def get_kv_length_upto_iter(self, layer_idx: int = 0, upto_iter_idx: int = 0) -> int:
        return sum(self.get_cache_length(layer_idx, i) for i in range(upto_iter_idx + 1))

    def get_seq_length(self, layer_idx: Optional[int] = 0, iter_idx: Optional[int] = 0) -> int:
        return self.get_cache_length(layer_idx, iter_idx)

    def get_usable_length(self, new_seq_length: int, layer_idx: Optional[int] = 0) -> int:
        return self.get_cache_length(layer_idx)

    def get_max_length(self):
        return None

    def get_max_cache_shape(self):
        return None

    def get_mask_sizes(self, cache_position, layer_idx: int):
        return cache_position.shape[0] + self.get_cache_length(layer_idx), 0

    def reorder_cache(self, beam_idx: torch.LongTensor) -> None:
        for store in (self._k, self._v, self._pos, self._valid):
            for slot, t in store.items():
                store[slot] = t.index_select(0, beam_idx.to(t.device))

    def __len__(self):
        return len({l for (l, _) in self._k})

    # ---- device / dtype --------------------------------------------------------------
    @property
    def device(self):
        for t in self._k.values():
            return t.device
        return self._device

    @property
    def dtype(self):
        for t in self._k.values():
            return t.dtype
        return self._dtype

    def to(self, *args, **kwargs) -> "TaHCache":
        device, dtype = kwargs.get("device"), kwargs.get("dtype")
        for a in args:
            if isinstance(a, torch.dtype):
                dtype = a
            elif isinstance(a, (str, torch.device)):
                device = a
        if device is not None:
            self._device = torch.device(device)
        if dtype is not None:
            self._dtype = dtype
        for store in (self._k, self._v):
            for slot, t in store.items():
                store[slot] = t.to(device=device, dtype=dtype)
        if device is not None:
            for store in (self._pos, self._valid):
                for slot, t in store.items():
                    store[slot] = t.to(device)
        return self
