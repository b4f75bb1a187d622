"""TaHEngine: KV-cached inference on the hand-written kernels.

Two phases:

* **prefill** - the prompts are packed (no padding) into one token stream; pass 0 runs the
  backbone on all prompt tokens, the decider picks the hard ones, passes 1.. run on the packed
  hard subset with the LoRA K-extension on, attending under the duo-causal rule over the dense
  K/V of the earlier passes; every pass also writes its K/V into that depth's paged cache.
* **decode** - *iteration-level continuous batching*: one "tick" processes exactly one token
  per row, at whatever depth that row is at.  An easy row emits a token every tick; a hard row
  spends ``1 + extra`` ticks on its token (soft embedding in, LoRA gated on for that row, K/V
  into the deeper cache, logits accumulated).  Rows are independent, so every row's token
  stream equals the reference schedule (two full-batch passes whenever any row is hard,
  reference ``tah/model/utils.py:233-260`` + ``tah_model.py:580``), while the weights are read
  once per tick for all rows.  A tick has static shapes and no host synchronisation: it is
  captured once in a CUDA graph and replayed.

The per-tick state (token, depth, position, KV lengths, page tables, free-page stacks, output
buffers) lives on the device; see ``csrc/sampling.cu``.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from tah_b200.engine.kv_cache import CacheGeometry, PagedKVCache
from tah_b200.engine.weights import EngineWeights
from tah_b200.model.iter_decider import (BernoulliIterDecider, IterLabelDecider, MLPIterDecider,
                                         SimpleMLPIterDecider)
from tah_b200.ops import cuda as K
from tah_b200.utils.observe import MetricsSink, engine_counters, nvtx_range


@dataclass
class GenerationResult:
    tokens: List[List[int]]
    iter_counts: List[float]            # mean passes per emitted token, per row
    ticks: int = 0
    tokens_emitted: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    extra: dict = field(default_factory=dict)


def _fusions(default: str):
    """Kernel fusions selected by ``TAH_B200_FUSE``: "1" = all, "0" = none, or a comma list of "qkv" (QK-norm, RoPE
    and the K/V write in the QKV GEMM's epilogue) and "lora" (LoRA-A of the gated rows inside the RMSNorm launch);
    unset = ``default`` (nothing: the chains of separate launches measured faster in decode and in prefill)."""
    v = os.environ.get("TAH_B200_FUSE", default)
    if v == "1":
        return {"qkv", "lora"}
    return {t for t in v.split(",") if t in ("qkv", "lora")}


class TaHEngine:
    def __init__(self, model, max_rows: int = 64, max_seq_len: int = 2048, page_size: int = 16,
                 deep_fraction: float = 0.25, use_cuda_graph: bool = True, tp=None):
        self.model = model
        base = model.simple_base_model
        self.cfg = base.config
        self.device = base.device
        if self.device.type != "cuda":
            raise RuntimeError("TaHEngine needs the model on a CUDA device")
        self.max_iter = int(model.max_iter)
        if self.max_iter > 4:
            raise ValueError("the engine supports max_iter <= 4")
        self.topk = int(model.input_topk)
        self.tp = tp
        self.w = EngineWeights(base, tp=tp)
        self.max_rows, self.max_seq_len, self.page_size = max_rows, max_seq_len, page_size
        self.deep_fraction = deep_fraction
        self.use_cuda_graph = use_cuda_graph and os.environ.get("TAH_B200_NO_GRAPH", "0") != "1"
        self.kv: Optional[PagedKVCache] = None
        self._states = {}          # (rows, max_new, sampling, eos, override) -> tick state with its captured graph
        self._calls = 0
        self.graph_captures = 0
        self.graph_reuses = 0
        self.hard_override: Optional[torch.Tensor] = None     # [rows, max_seq_len] int8: extra passes per position
        inner = self._decider()[1]
        thr = getattr(inner, "threshold", None)
        self._thr = float(thr.detach().float().cpu()) if isinstance(thr, torch.Tensor) else 0.5
        self.kernel_launches_per_tick = 0
        # counters of the last generate() call (KV page occupancy per depth, ticks per token, passes per token,
        # graph reuse ...); appended to the JSONL file named by TAH_B200_METRICS when that variable is set
        self.last_counters: dict = {}
        path = os.environ.get("TAH_B200_METRICS")
        self.metrics = MetricsSink(path) if path else None

    # ------------------------------------------------------------------------------------------
    # decider plumbing
    # ------------------------------------------------------------------------------------------
    def _decider(self):
        d = self.model.eval_iter_decider or self.model.iter_decider
        inner = d.inner if isinstance(d, BernoulliIterDecider) else d
        return d, inner

    def _tap_layers(self) -> Sequence[int]:
        _, inner = self._decider()
        if isinstance(inner, MLPIterDecider):
            return list(inner.hidden_states_layer_nums)
        if isinstance(inner, SimpleMLPIterDecider):
            return list(inner.hidden_states_layer_nums[-1:]) or [self.cfg.num_hidden_layers]
        return []

    def _score(self, taps: Optional[torch.Tensor], topk_vals: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Decider logits ``z`` (fp32 ``[n]``) from tapped hidden states / sorted top-k values."""
        _, inner = self._decider()
        if isinstance(inner, MLPIterDecider):
            return self._score_mlp(inner, taps, topk_vals)
        if isinstance(inner, SimpleMLPIterDecider):
            return self._score_simple_mlp(inner, taps)
        return None

    def _mlp_decider_plan(self, dec: MLPIterDecider, device):
        """Kernel-ready weights of the learned decider (reference ``tah/model/iter_decider.py:194-301``), or None
        when a shape or option is outside what the kernel chain covers (then the module runs)."""
        plan = getattr(self, "_mlp_plan", None)
        if plan is not None and plan["dec"] is dec:
            return plan["w"]
        H, k = dec.hidden_states_size, dec.topk
        lin = [dec.logits_projection, dec.combined_projection, dec.backbone.input_projection, dec.backbone.output_layer[1]]
        ok = (not dec.normalize_input and k <= 128 and H % 64 == 0 and all(m.weight.dtype == torch.bfloat16 for m in lin)
              and all(isinstance(b.dim_change, torch.nn.Identity) for b in dec.backbone.blocks)
              and all(m.weight.shape[1] % 64 == 0 and m.weight.shape[0] % 8 == 0 for m in lin[1:3])
              and dec.backbone.output_layer[1].weight.shape[0] == 1
              and all(b.mlp[0].weight.shape[0] % 64 == 0 and b.mlp[0].weight.shape[1] % 64 == 0 for b in dec.backbone.blocks))
        w = None
        if ok:
            bf = lambda t: t.detach().to(device=device, dtype=torch.bfloat16).contiguous()

            def bias_ext(m):              # the bias enters the fp32 accumulation as a K-extension: ones column x bias
                e = torch.zeros(m.weight.shape[0], 64, dtype=torch.bfloat16, device=device)
                if m.bias is not None:
                    e[:, 0] = m.bias.detach()
                return e

            lp = torch.zeros(H, 128, dtype=torch.bfloat16, device=device)
            lp[:, :k] = dec.logits_projection.weight.detach()
            ones = torch.zeros(max(self.max_rows, 4096), 64, dtype=torch.bfloat16, device=device)
            ones[:, 0] = 1
            out_ln, out_lin = dec.backbone.output_layer[0], dec.backbone.output_layer[1]
            w = dict(k=k, H=H, ones=ones, lp=lp, lp_b=bias_ext(dec.logits_projection),
                     cp=bf(dec.combined_projection.weight), cp_b=bias_ext(dec.combined_projection),
                     ip=bf(dec.backbone.input_projection.weight), ip_b=bias_ext(dec.backbone.input_projection),
                     blocks=[dict(ln_w=bf(b.layer_norm.weight), ln_b=bf(b.layer_norm.bias), eps=b.layer_norm.eps,
                                  w1=bf(b.mlp[0].weight), b1=bias_ext(b.mlp[0]), w2=bf(b.mlp[3].weight), b2=bias_ext(b.mlp[3]))
                             for b in dec.backbone.blocks],
                     oln_w=bf(out_ln.weight), oln_b=bf(out_ln.bias), oeps=out_ln.eps,
                     ow=bf(out_lin.weight[0]), ob=bf(out_lin.bias) if out_lin.bias is not None else None)
        self._mlp_plan = {"dec": dec, "w": w}
        return w

    def _score_mlp(self, dec: MLPIterDecider, taps: torch.Tensor, topk_vals: torch.Tensor) -> torch.Tensor:
        """The learned decider as a kernel chain: ``Linear(topk -> H)`` on the sorted top-k values written next to
        the tapped hidden states, the combined and input projections, the residual blocks ``x + W2 gelu(W1 LN(x))``
        (LayerNorm kernel; tcgen05 GEMMs with the bias as a K-extension, GELU / residual epilogues) and the output
        layer ``LayerNorm -> Linear(d, 1)`` as one reduction kernel.  ``taps``: ``[M, n_taps*H]`` or, with room for
        the projection, ``[M, (n_taps+1)*H]``."""
        w = self._mlp_decider_plan(dec, taps.device) if taps.is_cuda and taps.dtype == torch.bfloat16 else None
        n_taps = max(1, len(dec.hidden_states_layer_nums))
        if w is None or taps.shape[0] > w["ones"].shape[0]:
            hid = taps[:, :n_taps * dec.hidden_states_size]
            return dec.score(hid, topk_vals[:, :dec.topk].to(hid.dtype)).float()
        M, H, k = taps.shape[0], w["H"], w["k"]
        feats = taps
        if taps.shape[1] == n_taps * H:
            feats = torch.empty(M, (n_taps + 1) * H, dtype=torch.bfloat16, device=taps.device)
            feats[:, :n_taps * H].copy_(taps)
        tv = getattr(self, "_mlp_tv", None)
        if tv is None or tv.shape[0] < M:
            tv = self._mlp_tv = torch.zeros(max(M, self.max_rows), 128, dtype=torch.bfloat16, device=taps.device)
        tv[:M, :k].copy_(topk_vals[:, :k])
        ones = w["ones"][:M]
        K.gemm(tv[:M], w["lp"], x2=ones, w2=w["lp_b"], out=feats[:, n_taps * H:])
        x = K.gemm(feats, w["cp"], x2=ones, w2=w["cp_b"])
        x = K.gemm(x, w["ip"], x2=ones, w2=w["ip_b"])
        for b in w["blocks"]:
            n = K.layer_norm(x, b["ln_w"], b["ln_b"], b["eps"])
            u = K.gemm(n, b["w1"], x2=ones, w2=b["b1"], gelu=True)
            x = K.gemm(u, b["w2"], x2=ones, w2=b["b2"], residual=x, out=x)
        return K.layer_norm_dot(x, w["oln_w"], w["oln_b"], w["ow"], w["ob"], w["oeps"])

    def _score_simple_mlp(self, dec: SimpleMLPIterDecider, taps: torch.Tensor) -> torch.Tensor:
        """The two-layer decider as kernels: tcgen05 GEMM for the first layer (its bias enters the fp32
        accumulation as a K-extension: a column of ones times the bias), then SiLU + dot + bias per row."""
        w1 = dec.fc1.weight
        if (taps.dtype != torch.bfloat16 or w1.dtype != torch.bfloat16 or not taps.is_cuda or taps.shape[-1] % 64
                or w1.shape[0] % 8):
            return dec.score(taps).float()
        M = taps.shape[0]
        cache = getattr(self, "_dec_cache", None)
        if cache is None or cache[0] is not w1 or cache[1].shape[0] < M:
            ones = torch.zeros(max(M, self.max_rows), 64, dtype=torch.bfloat16, device=taps.device)
            ones[:, 0] = 1
            bias_ext = torch.zeros(w1.shape[0], 64, dtype=torch.bfloat16, device=taps.device)
            if dec.fc1.bias is not None:
                bias_ext[:, 0] = dec.fc1.bias.detach()
            cache = self._dec_cache = (w1, ones, bias_ext)
        _, ones, bias_ext = cache
        x = taps if taps.is_contiguous() else taps.contiguous()
        h1 = K.gemm(x, w1.detach(), x2=ones[:M], w2=bias_ext)
        return K.decider_head(h1, dec.fc2.weight.detach()[0].contiguous(), dec.fc2.bias.detach() if dec.fc2.bias is not None else None)

    def _needs_topk_for_decider(self) -> bool:
        return isinstance(self._decider()[1], MLPIterDecider)

    def make_bernoulli_override(self, rows: int, p: Sequence[float], seed: int = 0) -> torch.Tensor:
        """Seeded hard-token mask: ``override[r, pos]`` = number of extra passes of the token at
        ``pos`` (depth d continues with probability ``p[d]`` given it reached d)."""
        g = torch.Generator().manual_seed(seed)
        extra = torch.zeros(rows, self.max_seq_len, dtype=torch.int8)
        alive = torch.ones(rows, self.max_seq_len, dtype=torch.bool)
        for d in range(self.max_iter - 1):
            pd = p[min(d, len(p) - 1)]
            alive = alive & (torch.rand(rows, self.max_seq_len, generator=g) < pd)
            extra += alive.to(torch.int8)
        return extra.to(self.device)

    # ------------------------------------------------------------------------------------------
    # one backbone pass over packed tokens (prefill)
    # ------------------------------------------------------------------------------------------
    def _packed_pass(self, x, pos, depth: int, slots, seg_k, seg_v, seg_base, seg_count, seq_counts, taps_out=None):
        """x ``[n, H]`` packed tokens at iteration ``depth``.  seg_k/seg_v: per layer lists of the
        dense K/V of shallower passes; this pass's K/V are appended as the last segment.
        ``seq_counts [B]``: how many of the packed tokens each sequence owns (query tiling).  Returns
        (final-norm hidden, list of this pass's dense (k, v) per layer)."""
        cfg, w, tp = self.cfg, self.w, self.tp
        n = x.shape[0]
        nq, nkv, hd = w.nq, w.nkv, cfg.head_dim
        lora = depth >= 1 and w.r > 0
        scale = hd ** -0.5
        own = []
        nL = len(w.layers)
        bf = lambda *shape: torch.empty(*shape, dtype=torch.bfloat16, device=x.device)
        h = x.clone()                                   # residual stream (row-sharded under TP)
        xn_buf = bf(n, cfg.hidden_size)
        t_o = bf(n, w.r_o) if lora else None
        t_down = bf(n, w.r_down) if lora else None
        tap_layers = self._tap_layers()
        tensor_core_attn = hd in (64, 128) and os.environ.get("TAH_B200_NAIVE_PREFILL", "0") != "1"
        # off by default here as well: at thousands of tokens per tile column the epilogue's QK-norm / RoPE arithmetic
        # on four warps costs as much as the tile's main loop (prefill 272 ms fused, 254 ms with the separate kernel)
        fuse_qkv = hd == 128 and "qkv" in _fusions("")
        if tensor_core_attn:
            tile_q0, tile_qn = K.attn_tiles(seq_counts)
        rope_cs = K.rope_table(pos, hd, cfg.rope_theta) if fuse_qkv else None     # once per pass, shared by the layers
        # tensor parallel: token counts that deal out in 16-row blocks take the push path (reduce-scatter in the
        # GEMM epilogue, consumers wait on landing flags), the others the pull kernel
        push = (tp is not None and os.environ.get("TAH_B200_TP_PULL", "0") != "1" and tp.push_desc(n) is not None)
        self._xn_wait = None
        xn = K.rms_norm(h, w.layers[0].ln1, cfg.rms_norm_eps, out=xn_buf)
        for li, L in enumerate(w.layers):
            if taps_out is not None and li in tap_layers:
                taps_out[li] = h.clone() if tp is None else tp.gather_rows(h, n)
            kw = dict(x2=K.gemm(xn, L.a_qkv, tp_wait=self._xn_wait), w2=L.b_qkv) if lora else {}
            kd, vd = bf(n, nkv * hd), bf(n, nkv * hd)
            if fuse_qkv:
                q = K.gemm_qkv(xn, L.w_qkv, L.q_norm, L.k_norm, pos, nq, nkv, cfg.rms_norm_eps, cfg.rope_theta,
                               k_dense=kd, v_dense=vd, caches=[self.kv.layer_pool(depth, li)], slot=slots,
                               page_size=self.page_size, rope_cs=rope_cs, tp_wait=self._xn_wait, **kw)
            else:
                qkv = K.gemm(xn, L.w_qkv, tp_wait=self._xn_wait, **kw)
                q = K.qk_norm_rope_kv(qkv, L.q_norm, L.k_norm, pos, nq, nkv, hd, cfg.rms_norm_eps, cfg.rope_theta,
                                      k_dense=kd, v_dense=vd, caches=[self.kv.layer_pool(depth, li)], slot=slots,
                                      page_size=self.page_size)
            own.append((kd, vd))
            ks = [sk[li] for sk in seg_k] + [kd]
            vs = [sv[li] for sv in seg_v] + [vd]
            if tensor_core_attn:
                o = K.prefill_attn(q, ks, vs, seg_base, seg_count, tile_q0, tile_qn, nq, nkv, hd, scale)
            else:
                o = K.varlen_attn_naive(q, ks, vs, seg_base, seg_count, nq, nkv, hd, scale)
            xn = self._row_parallel(o, L.w_o, L.a_o if lora else None, L.b_o, t_o, None, h, L.ln2, xn_buf, n, push=push)
            sw = dict(swiglu_interleaved=True) if w.gu_interleaved else dict(swiglu=True)
            if lora:
                t = K.gemm(xn, L.a_gu, tp_wait=self._xn_wait)
                act = K.gemm(xn, L.w_gu, x2=t, w2=L.b_gu, tp_wait=self._xn_wait, **sw)
            else:
                act = K.gemm(xn, L.w_gu, tp_wait=self._xn_wait, **sw)
            next_ln = w.layers[li + 1].ln1 if li + 1 < nL else w.final_norm
            xn = self._row_parallel(act, L.w_down, L.a_down if lora else None, L.b_down, t_down, None, h, next_ln,
                                    xn_buf, n, push=push, final=li + 1 == nL)
        hn = xn.clone()
        if taps_out is not None and cfg.num_hidden_layers in tap_layers:
            taps_out[cfg.num_hidden_layers] = hn
        return hn, own

    # ------------------------------------------------------------------------------------------
    # prefill
    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor], max_new_tokens: int,
                row_ids: Optional[torch.Tensor] = None):
        """Prefill a batch of prompts.  ``row_ids`` (optional ``[B]``): admit these prompts into those rows of the
        existing cache (their pages must have been released with ``kv.free_rows``) while the other rows keep their
        state; without it the cache is (re)built for exactly this batch."""
        cfg, w, dev = self.cfg, self.w, self.device
        B, T = input_ids.shape
        valid = attention_mask[:, -T:].bool() if attention_mask is not None else torch.ones(B, T, dtype=torch.bool, device=dev)
        lens = valid.sum(1)
        max_total = int(lens.max()) + max_new_tokens + 1
        if row_ids is not None:
            if self.kv is None or self.kv.max_pages[0] * self.page_size < max_total:
                raise RuntimeError("admission needs an existing KV cache whose rows can hold prompt + new tokens")
            row_ids = row_ids.to(dev)
        elif self.kv is None or self.kv.rows != B or self.kv.max_pages[0] * self.page_size < max_total:
            geo = CacheGeometry(cfg.num_hidden_layers, w.nkv, cfg.head_dim, self.page_size)
            self.kv = None
            torch.cuda.empty_cache()
            self.kv = PagedKVCache(geo, B, max(max_total, 1), self.max_iter, self.deep_fraction, dev)
            self._states.clear()          # captured ticks point into the old pools
        if row_ids is None:
            self.kv.reset()
        assign = (lambda d, c: self.kv.assign_prefill(d, c)) if row_ids is None else \
                 (lambda d, c: self.kv.assign_rows(d, row_ids, c))
        self._prefill_rows = row_ids
        if self.tp is not None:
            self.tp.allocate(cfg.hidden_size, max(int(valid.sum()), B))
        rows_idx, cols_idx = valid.nonzero(as_tuple=True)
        ids = input_ids[rows_idx, cols_idx].to(torch.int32).contiguous()
        n0 = ids.numel()
        seq_start = (torch.cumsum(lens, 0) - lens).to(torch.int32)
        pos = (torch.arange(n0, device=dev, dtype=torch.int32) - seq_start[rows_idx]).contiguous()
        seq = rows_idx.to(torch.int32)

        # ---- pass 0 -------------------------------------------------------------------------
        slots0 = assign(0, lens)
        x = K.embed_gather(w.embed, ids)
        taps = {}
        base0 = seq_start[rows_idx].contiguous()
        count0 = (pos + 1).contiguous()
        with nvtx_range("prefill/pass0"):
            hn, kv0 = self._packed_pass(x, pos, 0, slots0, [], [], [base0], [count0], lens, taps_out=taps)
        seg_k, seg_v = [[k for k, _ in kv0]], [[v for _, v in kv0]]

        # ---- continue decision for every prompt token ----------------------------------------
        last_idx = (seq_start.long() + lens - 1)
        is_last = torch.zeros(n0, dtype=torch.bool, device=dev)
        is_last[last_idx] = True
        extra = self._prompt_extra_passes(hn, taps, seq, pos)                 # [n0] int: extra passes wanted
        cur_idx = torch.arange(n0, device=dev)                                # packed indices of the current set
        cur_cum = None                                                        # cumulative logits of current set
        final_last_logits = torch.empty(B, w.vocab_shard[1] - w.vocab_shard[0], dtype=torch.bfloat16, device=dev)
        # tokens needing logits after pass 0: last tokens + hard tokens
        need0 = is_last | (extra > 0)
        sel = need0.nonzero().flatten()
        logits_sel = self._lm_head(hn[sel])
        done_last = is_last[sel] & (extra[sel] == 0)
        final_last_logits[seq[sel][done_last].long()] = logits_sel[done_last]
        go = extra[sel] > 0
        cur_idx = sel[go]
        cur_cum = logits_sel[go]
        prev_bases = [base0]
        prev_counts = [count0]
        depth = 1
        iter_extra_prompt = extra.clone()
        while depth < self.max_iter and cur_idx.numel() > 0:
            n1 = cur_idx.numel()
            rows1 = seq[cur_idx].long()
            cnt1 = torch.bincount(rows1, minlength=B)
            slots1 = assign(depth, cnt1)
            val = torch.zeros(n1, self.topk, dtype=torch.float32, device=dev)
            idx = torch.zeros(n1, self.topk, dtype=torch.int32, device=dev)
            self._topk(cur_cum, self.topk, None, val, idx)
            x1 = K.soft_embed_rows(val, idx, w.embed)
            pos1 = pos[cur_idx].contiguous()
            start1 = (torch.cumsum(cnt1, 0) - cnt1).to(torch.int32)
            rank1 = (torch.arange(n1, device=dev, dtype=torch.int32) - start1[rows1])
            bases = [b[cur_idx].contiguous() for b in prev_bases] + [start1[rows1].contiguous()]
            counts = [c[cur_idx].contiguous() for c in prev_counts] + [(rank1 + 1).contiguous()]
            # shallower segments (1..depth-1) index into the packed arrays of those passes: their
            # (base, count) were computed against those arrays when the passes ran
            learned = self.hard_override is None and isinstance(self._decider()[1], (MLPIterDecider, SimpleMLPIterDecider))
            taps1 = {} if learned and depth + 1 < self.max_iter else None
            with nvtx_range(f"prefill/pass{depth}"):
                hn1, kv1 = self._packed_pass(x1, pos1, depth, slots1, seg_k, seg_v, bases, counts, cnt1, taps_out=taps1)
            logits1 = self._lm_head(hn1)
            cum1 = cur_cum + logits1
            if taps1 is not None:
                # a learned decider is asked again after every pass, on this pass's hidden states and the cumulative
                # logits, as the model's forward and the decode tick do (reference tah_model.py:625-645)
                inner = self._decider()[1]
                tl = self._tap_layers()
                tcat = torch.cat([taps1[i] for i in tl], dim=-1) if tl else None
                tv = None
                if isinstance(inner, MLPIterDecider):
                    tv = torch.zeros(n1, inner.topk, dtype=torch.float32, device=dev)
                    self._topk(cum1, inner.topk, None, tv, torch.zeros(n1, inner.topk, dtype=torch.int32, device=dev))
                z1 = self._score(tcat, tv)
                want_more = torch.sigmoid(z1) > self._thr
            else:
                want_more = (extra[cur_idx] > depth) & (depth + 1 < self.max_iter)
            fin = ~want_more
            lastfin = fin & is_last[cur_idx]
            final_last_logits[rows1[lastfin]] = cum1[lastfin]
            # next pass: subset of this one; its view of this pass's segment
            seg_k.append([k for k, _ in kv1])
            seg_v.append([v for _, v in kv1])
            full_b = torch.zeros(n0, dtype=torch.int32, device=dev)
            full_c = torch.zeros(n0, dtype=torch.int32, device=dev)
            full_b[cur_idx] = bases[-1]
            full_c[cur_idx] = counts[-1]
            prev_bases.append(full_b)
            prev_counts.append(full_c)
            cur_idx = cur_idx[want_more]
            cur_cum = cum1[want_more]
            depth += 1
        del seg_k, seg_v
        return final_last_logits, lens, iter_extra_prompt

    def _prompt_extra_passes(self, hn, taps, seq, pos) -> torch.Tensor:
        """How many extra passes each prompt token takes (0 = easy)."""
        n0 = hn.shape[0]
        dev = hn.device
        if self.max_iter <= 1:
            return torch.zeros(n0, dtype=torch.int32, device=dev)
        decider, inner = self._decider()
        z = None
        tl = self._tap_layers()
        if isinstance(inner, (MLPIterDecider, SimpleMLPIterDecider)):
            # scored in chunks: the MLP decider needs sorted top-k logits of every token
            zs = []
            step = 4096
            for s in range(0, n0, step):
                sl = slice(s, min(n0, s + step))
                tcat = torch.cat([taps[i][sl] for i in tl], dim=-1) if tl else None
                tv = None
                if isinstance(inner, MLPIterDecider):
                    lg = self._lm_head(hn[sl])
                    tv = torch.zeros(lg.shape[0], inner.topk, dtype=torch.float32, device=dev)
                    self._topk(lg, inner.topk, None, tv, torch.zeros(lg.shape[0], inner.topk, dtype=torch.int32, device=dev))
                zs.append(self._score(tcat, tv))
            z = torch.cat(zs)
        if self.hard_override is not None:
            rows = seq.long() if getattr(self, "_prefill_rows", None) is None else self._prefill_rows[seq.long()]
            return self.hard_override[rows, pos.long()].to(torch.int32)
        if isinstance(decider, BernoulliIterDecider):
            raise RuntimeError("BernoulliIterDecider needs engine.hard_override (see make_bernoulli_override)")
        if z is None:
            return torch.zeros(n0, dtype=torch.int32, device=dev)
        return (torch.sigmoid(z) > self._thr).to(torch.int32)

    def _lm_head(self, hn: torch.Tensor) -> torch.Tensor:
        """Logits of this rank's vocabulary shard (the whole vocabulary on one GPU)."""
        lo, hi, _ = self.w.vocab_shard
        return K.gemm(hn.contiguous(), self.w.lm_head)[:, :hi - lo]

    def _argmax(self, logits: torch.Tensor) -> torch.Tensor:
        val, idx = logits.float().max(dim=-1)
        if self.tp is None:
            return idx.to(torch.int32)
        return self.tp.merge_argmax(val, idx.to(torch.int32), self.w.vocab_shard[0])

    # ------------------------------------------------------------------------------------------
    # decode tick
    # ------------------------------------------------------------------------------------------
    def _alloc_tick_buffers(self, B: int, max_new: int):
        cfg, w, dev = self.cfg, self.w, self.device
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
        H = cfg.hidden_size
        s = type("S", (), {})()
        s.tok, s.depth, s.pos, s.finished, s.n_out = i32(B), i32(B), i32(B), i32(B), i32(B)
        s.out_tokens, s.iter_sum, s.cur_iters, s.slot, s.gate = i32(B, max_new), i32(B), i32(B), i32(B), i32(B)
        s.tokens_done = torch.zeros(1, dtype=torch.int64, device=dev)
        s.need_soft, s.best, s.sampled = i32(B), i32(B), i32(B)
        s.best_val = torch.zeros(B, dtype=torch.float32, device=dev)
        # split the KV walk of a row when (rows x local KV heads) CTAs would leave SM slots empty
        # (small batches, wide tensor-parallel groups); the partial results meet in a merge kernel
        s.attn_split = max(1, min(4, (148 * 4) // max(1, B * w.nkv)))
        s.attn_ws = None
        if s.attn_split > 1:
            n_ws = int(K.lib().tahb_decode_attn_ws_floats(B, w.nq, cfg.head_dim, s.attn_split))
            s.attn_ws = torch.empty(n_ws, dtype=torch.float32, device=dev)
        s.samp_v = torch.zeros(B, 128, dtype=torch.float32, device=dev)
        s.samp_i = i32(B, 128)
        s.seed_dev = torch.zeros(1, dtype=torch.int64, device=dev)     # per-call sampling seed, read on the device
        s.rope_cs = bf(B, cfg.head_dim)                                # RoPE cos | sin row of the tick's positions
        s.graph = None
        s.x_in, s.soft, s.h, s.xn = bf(B, H), bf(B, H), bf(B, H), bf(B, H)
        s.qkv = bf(B, w.qkv_out)
        s.q, s.o = bf(B, w.nq * cfg.head_dim), bf(B, w.nq * cfg.head_dim)
        s.act = bf(B, w.inter)
        s.t_qkv, s.t_o, s.t_gu, s.t_down = bf(B, w.r_qkv), bf(B, w.r_o), bf(B, w.r_gu), bf(B, w.r_down)
        s.logits, s.cum = bf(B, w.vocab_shard[2]), bf(B, w.vocab_shard[2])
        s.topv = torch.zeros(B, self.topk, dtype=torch.float32, device=dev)
        s.topi = i32(B, self.topk)
        tl = self._tap_layers()
        # the learned decider's Linear(topk -> H) output is written behind the tapped hidden states
        tap_w = (max(1, len(tl)) + (1 if self._needs_topk_for_decider() else 0)) * H
        s.tap_buf = None
        if self.tp is not None and any(0 < li < cfg.num_hidden_layers for li in tl) and B % (16 * self.tp.world_size) == 0:
            # tensor parallel: the owner kernels of the push path store the tapped residual rows into this
            # symmetric buffer on every rank (no collective call inside the tick)
            s.tap_buf = self.tp.alloc_taps(B, tap_w)
            s.taps = s.tap_buf.tensor
        else:
            s.taps = bf(B, tap_w)
        s.z = torch.zeros(B, dtype=torch.float32, device=dev)
        kv = self.kv
        pad = lambda lst: list(lst) + [lst[0]] * (4 - len(lst))
        tensors = [s.tok, s.depth, s.pos, s.finished, s.n_out, s.out_tokens, s.iter_sum, s.cur_iters, s.slot, s.gate]
        tensors += pad(kv.len) + pad(kv.page_table) + pad(kv.free_stack) + pad(kv.free_count)
        tensors += [K.status_word(dev), s.tokens_done]
        ints = pad(kv.max_pages) + [kv.n_depths, self.page_size, B, max_new, -1, self.max_iter]
        s.ints = ints
        s.tensors = tensors
        return s

    def _row_parallel(self, x, w_, a_, b_, t_buf, gate, h, ln_w, xn_out, M, push=False, final=False, next_lora=None,
                      tap=None):
        """Row-parallel projection + residual + the RMSNorm that follows it.

        One GPU: the GEMM epilogue adds the residual in place and a norm kernel follows.  Tensor
        parallel: the GEMM writes this rank's partial result into symmetric memory and the fused
        NVLink kernel does all-reduce + residual + norm + broadcast; ``h`` stays row-sharded.
        ``next_lora = (A, t_buf)`` (one GPU, decode): fuse the LoRA-A product of the consumer of ``xn`` into the
        norm launch.  ``tap = (tap buffer, column)`` (push path): the owner kernel also broadcasts the updated
        residual rows into that column of every rank's tap buffer."""
        cfg, tp = self.cfg, self.tp
        lora = a_ is not None and t_buf is not None
        if lora:
            if gate is not None:
                K.lora_a_rows(x, a_, gate, out=t_buf)
            else:
                K.gemm(x, a_, out=t_buf)
        kw = dict(x2=t_buf, w2=b_) if lora else {}
        if tp is None:
            K.gemm(x, w_, residual=h, out=h, **kw)
            if next_lora is not None:
                # the norm kernel also forms t = gate * xn A^T for the projection that consumes xn
                return K.rms_norm_lora(h, ln_w, cfg.rms_norm_eps, gate, next_lora[0], out=xn_out, t_out=next_lora[1])[0]
            return K.rms_norm(h, ln_w, cfg.rms_norm_eps, out=xn_out)
        desc = tp.push_desc(M) if push else None
        if desc is not None:
            # reduce-scatter inside the GEMM epilogue (peer stores), then sum + norm + broadcast on
            # the owners; the consumers of xn wait for the broadcast rows themselves (self._xn_wait)
            K.gemm(x, w_, tp_push=desc, **kw)
            self._xn_wait = None if final else tp.wait_desc
            return tp.push_reduce_norm(M, h, ln_w, cfg.rms_norm_eps, add_residual=True, final_wait=final, tap=tap)
        self._xn_wait = None
        K.gemm(x, w_, out=tp.partial[:M], **kw)
        return tp.fused_reduce_norm(M, h, ln_w, cfg.rms_norm_eps, add_residual=True)

    def _tick(self, s, sampling):
        """Enqueue one decode tick on the current stream (graph-capturable)."""
        cfg, w, kv, tp = self.cfg, self.w, self.kv, self.tp
        B = s.tok.shape[0]
        nq, nkv, hd = w.nq, w.nkv, cfg.head_dim
        scale = hd ** -0.5
        lora = w.r > 0 and self.max_iter > 1
        tl = self._tap_layers()
        H = cfg.hidden_size
        nL = len(w.layers)
        # Optional fusions of the decode chain.  Off by default: at 256 rows the chain of separate launches measured
        # 1.7 % faster per tick than the fused kernels (whose extra work runs on four epilogue warps per CTA).
        fuse = _fusions("")
        fuse_norm_lora = "lora" in fuse and lora and tp is None  # RMSNorm + LoRA-A of the gated rows in one launch
        fuse_qkv = "qkv" in fuse and hd == 128                   # QK-norm + RoPE + KV write in the QKV GEMM epilogue
        rope = dict(rope_cs=s.rope_cs, hd=hd, theta=cfg.rope_theta) if fuse_qkv else {}
        if tp is None:
            s.binding.tick_begin(w.embed, s.soft, s.h, **rope)   # the input embedding is the residual stream
        else:
            s.binding.tick_begin(w.embed, s.soft, s.x_in, **rope)
            s.h.copy_(s.x_in)
        pools = [[kv.layer_pool(d, li) for d in range(kv.n_depths)] for li in range(nL)]
        if fuse_norm_lora:
            xn = K.rms_norm_lora(s.h, w.layers[0].ln1, cfg.rms_norm_eps, s.gate, w.layers[0].a_qkv, out=s.xn,
                                 t_out=s.t_qkv)[0]
        else:
            xn = K.rms_norm(s.h, w.layers[0].ln1, cfg.rms_norm_eps, out=s.xn)
        self._xn_wait = None       # set by _row_parallel when xn is a tensor-parallel broadcast in flight
        push = tp is not None and os.environ.get("TAH_B200_TP_PULL", "0") != "1"
        kernel_taps = (push and s.tap_buf is not None and tp.push_desc(B) is not None
                       and os.environ.get("TAH_B200_TP_TAPS", "kernel") != "nccl")   # "nccl": all-gather form (baseline)
        for li, L in enumerate(w.layers):
            if li in tl and not (kernel_taps and li > 0):
                j = tl.index(li)
                if tp is None:
                    s.taps[:, j * H:(j + 1) * H].copy_(s.h)
                elif li == 0:
                    s.taps[:, j * H:(j + 1) * H].copy_(s.x_in)      # the embeddings: every rank has all rows
                else:
                    s.taps[:, j * H:(j + 1) * H].copy_(tp.gather_rows(s.h, B))
            if lora and not fuse_norm_lora:
                K.lora_a_rows(xn, L.a_qkv, s.gate, out=s.t_qkv, tp_wait=self._xn_wait)
            kw = dict(x2=s.t_qkv, w2=L.b_qkv) if lora else {}
            if fuse_qkv:
                K.gemm_qkv(xn, L.w_qkv, L.q_norm, L.k_norm, s.pos, nq, nkv, cfg.rms_norm_eps, cfg.rope_theta, q_out=s.q,
                           caches=pools[li], cache_sel=s.depth, slot=s.slot, page_size=self.page_size,
                           tp_wait=self._xn_wait, rope_cs=s.rope_cs, **kw)
            else:
                K.gemm(xn, L.w_qkv, out=s.qkv, tp_wait=self._xn_wait, **kw)
                K.qk_norm_rope_kv(s.qkv, L.q_norm, L.k_norm, s.pos, nq, nkv, hd, cfg.rms_norm_eps, cfg.rope_theta,
                                  q_out=s.q, caches=pools[li], cache_sel=s.depth, slot=s.slot, page_size=self.page_size)
            K.decode_attn(s.q, pools[li], kv.page_table, kv.len, s.depth, nq, nkv, hd, self.page_size, scale, out=s.o,
                          n_split=s.attn_split, ws=s.attn_ws)
            xn = self._row_parallel(s.o, L.w_o, L.a_o if lora else None, L.b_o, s.t_o, s.gate, s.h, L.ln2, s.xn, B,
                                    push=push, next_lora=(L.a_gu, s.t_gu) if fuse_norm_lora else None)
            if lora and not fuse_norm_lora:
                K.lora_a_rows(xn, L.a_gu, s.gate, out=s.t_gu, tp_wait=self._xn_wait)
            sw = dict(swiglu_interleaved=True) if w.gu_interleaved else dict(swiglu=True)
            if lora:
                K.gemm(xn, L.w_gu, x2=s.t_gu, w2=L.b_gu, out=s.act, tp_wait=self._xn_wait, **sw)
            else:
                K.gemm(xn, L.w_gu, out=s.act, tp_wait=self._xn_wait, **sw)
            next_ln = w.layers[li + 1].ln1 if li + 1 < nL else w.final_norm
            nxt_lora = (w.layers[li + 1].a_qkv, s.t_qkv) if fuse_norm_lora and li + 1 < nL else None
            # a tap of the next layer's input is this projection's updated residual stream
            tap = (s.tap_buf, tl.index(li + 1) * H) if kernel_taps and li + 1 < nL and (li + 1) in tl else None
            xn = self._row_parallel(s.act, L.w_down, L.a_down if lora else None, L.b_down, s.t_down, s.gate, s.h,
                                    next_ln, s.xn, B, push=push, final=li + 1 == nL, next_lora=nxt_lora, tap=tap)
        # xn is now the final-norm output of every row
        if cfg.num_hidden_layers in tl:
            j = tl.index(cfg.num_hidden_layers)
            s.taps[:, j * H:(j + 1) * H].copy_(xn)
        K.gemm(xn, w.lm_head, out=s.logits)
        lo, hi, _ = w.vocab_shard
        logits, cum = s.logits[:, :hi - lo], s.cum[:, :hi - lo]
        K.logits_post(logits, cum, s.depth, s.best, s.best_val)
        if tp is not None:
            s.best.copy_(tp.merge_argmax(s.best_val, s.best, lo))
        # decision
        z = None
        if self.max_iter > 1:
            topk_done = False
            if self._needs_topk_for_decider():
                self._topk(cum, self.topk, None, s.topv, s.topi)
                topk_done = True
            zz = self._score(s.taps, s.topv)
            if zz is not None:
                s.z.copy_(zz)
                z = s.z
            K.decide(z, self._thr, self.hard_override, s.pos, s.depth, self.max_iter, s.need_soft)
            if not topk_done:
                self._topk(cum, self.topk, s.need_soft, s.topv, s.topi)
            K.soft_embed_rows(s.topv, s.topi, w.embed, flag=s.need_soft, out=s.soft)
        nxt = s.best
        if sampling is not None:
            kk = sampling["top_k"]
            if 0 < kk <= 128:
                self._topk(cum, kk, None, s.samp_v, s.samp_i)
                K.sample_topk(s.samp_v, s.samp_i, sampling["temperature"], sampling["top_p"], sampling["min_p"],
                              0, step=s.pos, out=s.sampled, seed_dev=s.seed_dev)
            else:
                # no top-k filter (the reference's default top_k=0) or a set wider than the sorted route holds
                K.sample_full(cum, sampling["temperature"], kk, sampling["top_p"], sampling["min_p"], 0, step=s.pos,
                              out=s.sampled, seed_dev=s.seed_dev)
            nxt = s.sampled
        s.binding.tick_end(s.need_soft, nxt)

    def _topk(self, x, k, flag, out_val, out_idx):
        """Sorted top-k of (this rank's vocabulary shard of) ``x``; merged across shards under TP."""
        K.topk_rows(x, k, flag=flag, out_val=out_val, out_idx=out_idx)
        if self.tp is not None:
            v, i = self.tp.merge_topk(out_val, out_idx, self.w.vocab_shard[0], k)
            out_val.copy_(v)
            out_idx.copy_(i)

    # ------------------------------------------------------------------------------------------
    # generate
    # ------------------------------------------------------------------------------------------
    BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024)

    def bucket_rows(self, n: int) -> int:
        """Row count of the batch bucket that serves ``n`` requests (the engine keeps one set of tick buffers and
        one captured graph per bucket); exact under tensor parallelism or when bucketing is switched off."""
        if self.tp is not None or os.environ.get("TAH_B200_NO_BUCKETS", "0") == "1" or self.hard_override is not None:
            return n
        for b in self.BUCKETS:
            if b >= n:
                return b
        return n

    def _tick_state(self, B: int, max_new: int, sampling: Optional[dict], eos_token_id: Optional[int]):
        """Tick buffers + captured graph for this (rows, max_new, sampling, eos, hard mask) shape.  A repeat call
        with the same shape clears the scheduler state and replays the graph captured by the first one."""
        samp_key = None if sampling is None else (sampling["temperature"], sampling["top_p"], sampling["min_p"],
                                                  sampling["top_k"])
        ov = self.hard_override
        key = (B, max_new, samp_key, eos_token_id, None if ov is None else (ov.data_ptr(), tuple(ov.shape)))
        s = self._states.get(key)
        if s is None:
            if len(self._states) >= 4:                      # keep a handful of shapes (batch buckets)
                self._states.pop(next(iter(self._states)))
            s = self._alloc_tick_buffers(B, max_new)
            if sampling is not None and 0 < sampling["top_k"] <= 128:
                s.samp_v = torch.zeros(B, sampling["top_k"], dtype=torch.float32, device=self.device)
                s.samp_i = torch.zeros(B, sampling["top_k"], dtype=torch.int32, device=self.device)
            s.ints[8] = -1 if eos_token_id is None else int(eos_token_id)
            s.binding = K.TickStateBinding(s.tensors, s.ints)
            self._states[key] = s
        else:
            for t in (s.tok, s.depth, s.pos, s.finished, s.n_out, s.out_tokens, s.iter_sum, s.cur_iters, s.slot,
                      s.gate, s.tokens_done, s.need_soft, s.best, s.sampled):
                t.zero_()
        return s

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None, *,
                 max_new_tokens: int = 128, do_sample: bool = False, temperature: float = 1.0, top_p: float = 1.0,
                 top_k: int = 0, min_p: float = 0.0, eos_token_id: Optional[int] = None, seed: Optional[int] = None,
                 max_ticks: Optional[int] = None, sync_every: int = 64, on_tick=None) -> GenerationResult:
        """Prefill + decode.  ``seed=None`` draws the sampling seed from torch's global generator, so
        ``set_all_seeds`` / ``torch.manual_seed`` govern it and successive calls differ (the reference's loop
        samples with ``torch.multinomial`` on the global generator, ``tah/model/utils.py:84-125``)."""
        dev = self.device
        input_ids = input_ids.to(dev)
        if attention_mask is not None:
            attention_mask = attention_mask.to(dev)
        B_user = input_ids.shape[0]
        B = self.bucket_rows(B_user)
        if B != B_user:
            # batch bucket: pad with copies of the first prompt (their output is dropped), so that batch sizes of one
            # bucket share tick buffers and the captured graph
            pad = B - B_user
            input_ids = torch.cat([input_ids, input_ids[:1].expand(pad, -1)], 0)
            if attention_mask is not None:
                attention_mask = torch.cat([attention_mask, attention_mask[:1].expand(pad, -1)], 0)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        with nvtx_range("engine/prefill"):
            last_logits, lens, _ = self.prefill(input_ids, attention_mask, max_new_tokens)
        sampling = None
        if do_sample:
            if temperature <= 0:
                raise ValueError("sampling needs temperature > 0")
            if not (0 < top_k <= 128) and self.tp is not None:
                raise NotImplementedError("tensor-parallel engine sampling needs 0 < top_k <= 128 "
                                          "(the full-vocabulary sampler runs on one GPU)")
            sampling = dict(temperature=float(temperature), top_p=float(top_p), min_p=float(min_p), top_k=int(top_k))
            if seed is None:
                seed = int(torch.randint(0, 2 ** 62, (1,)).item())
        self._calls += 1
        s = self._tick_state(B, max_new_tokens, sampling, eos_token_id)
        if sampling is not None:
            s.seed_dev.fill_(int(seed) & (2 ** 62 - 1))
        # first token from the prefill logits
        if sampling is None:
            first = self._argmax(last_logits)
        elif 0 < top_k <= 128:
            val = torch.zeros(B, top_k, dtype=torch.float32, device=dev)
            idx = torch.zeros(B, top_k, dtype=torch.int32, device=dev)
            self._topk(last_logits, top_k, None, val, idx)
            first = K.sample_topk(val, idx, temperature, top_p, min_p, 0, step=lens.to(torch.int32) - 1,
                                  seed_dev=s.seed_dev)
        else:
            ll = last_logits if last_logits.stride(0) % 8 == 0 else torch.nn.functional.pad(
                last_logits, (0, -last_logits.shape[1] % 8))[:, :last_logits.shape[1]]
            first = K.sample_full(ll, temperature, top_k, top_p, min_p, 0, step=lens.to(torch.int32) - 1,
                                  seed_dev=s.seed_dev)
        s.pos.copy_(lens.to(torch.int32) - 1)
        s.need_soft.zero_()
        s.binding.tick_end(s.need_soft, first)          # emits token 1, pos = len, depth = 0
        s.cur_iters.zero_()
        ev[1].record()
        ticks = 0
        limit = max_ticks if max_ticks is not None else max_new_tokens * self.max_iter + 1
        if self.use_cuda_graph and limit > 0 and s.graph is None:
            self._tick(s, sampling)            # eager tick: lazy one-time kernel setup happens outside capture
            ticks = 1
            if on_tick is not None:
                on_tick(ticks, s)
        run = self._tick_runner(s, sampling)
        with nvtx_range("engine/decode"):
            while ticks < limit:
                run()
                ticks += 1
                if on_tick is not None:
                    on_tick(ticks, s)
                if ticks % sync_every == 0 or ticks == limit:
                    done = bool(((s.finished != 0) | (s.n_out >= max_new_tokens))[:B_user].all())
                    if done:
                        break
        ev[2].record()
        torch.cuda.synchronize()
        K.check_status(dev)
        n_out = s.n_out.tolist()
        out = s.out_tokens.tolist()
        iters = (s.iter_sum.float() / s.n_out.clamp(min=1).float()).tolist()
        out, n_out, iters = out[:B_user], n_out[:B_user], iters[:B_user]
        res = GenerationResult(tokens=[row[:n] for row, n in zip(out, n_out)], iter_counts=iters, ticks=ticks,
                               tokens_emitted=int(s.tokens_done.item()) if B == B_user else int(sum(n_out)),
                               prefill_ms=ev[0].elapsed_time(ev[1]),
                               decode_ms=ev[1].elapsed_time(ev[2]),
                               extra={"graph_captures": self.graph_captures, "graph_reuses": self.graph_reuses})
        self.last_counters = dict(engine_counters(self, res), graph_captures=self.graph_captures,
                                  graph_reuses=self.graph_reuses, rows=B)
        if self.metrics is not None:
            self.metrics.log(self.last_counters, step=self._calls)
        return res

    # ------------------------------------------------------------------------------------------
    # serving: request admission into free rows, pages returned on completion
    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def serve(self, prompts: Sequence[torch.Tensor], *, max_new_tokens: int = 128, rows: Optional[int] = None,
              eos_token_id: Optional[int] = None, do_sample: bool = False, temperature: float = 1.0, top_p: float = 1.0,
              top_k: int = 0, min_p: float = 0.0, seed: Optional[int] = None, check_every: int = 16):
        """Continuous batching over a queue of requests (1-D token id tensors of any lengths).

        ``rows`` batch rows decode in lock step (one captured tick graph for that row count).  Every
        ``check_every`` ticks the host looks at the rows: a row whose request finished (EOS or ``max_new_tokens``)
        hands back its tokens, its KV pages of every depth return to the device free stacks, and the next queued
        request is admitted into the row - its prompt is prefilled into freshly assigned pages while the other rows
        keep their state - so the batch stays full while requests of different lengths come and go.  Returns the
        generated token lists in request order and a statistics dict (ticks, admissions, peak pages in use)."""
        dev = self.device
        if self.tp is not None:
            raise NotImplementedError("serve() runs on one GPU; use generate() under tensor parallelism")
        n_req = len(prompts)
        B = min(rows or self.max_rows, n_req, self.max_rows)
        longest = max(int(p.numel()) for p in prompts)
        sampling = None
        if do_sample:
            sampling = dict(temperature=float(temperature), top_p=float(top_p), min_p=float(min_p), top_k=int(top_k))
            if seed is None:
                seed = int(torch.randint(0, 2 ** 62, (1,)).item())

        def pad_batch(ps):
            T = max(int(p.numel()) for p in ps)
            ids = torch.zeros(len(ps), T, dtype=torch.long, device=dev)
            mask = torch.zeros(len(ps), T, dtype=torch.long, device=dev)
            for i, p in enumerate(ps):
                ids[i, T - p.numel():] = p.to(dev)
                mask[i, T - p.numel():] = 1
            return ids, mask

        def first_tokens(logits, lens):
            if sampling is None:
                return self._argmax(logits)
            k = sampling["top_k"]
            if 0 < k <= 128:
                val = torch.zeros(logits.shape[0], k, dtype=torch.float32, device=dev)
                idx = torch.zeros(logits.shape[0], k, dtype=torch.int32, device=dev)
                self._topk(logits, k, None, val, idx)
                return K.sample_topk(val, idx, temperature, top_p, min_p, int(seed), step=lens.to(torch.int32) - 1)
            return K.sample_full(logits.contiguous(), temperature, k, top_p, min_p, int(seed), step=lens.to(torch.int32) - 1)

        # the cache is sized for the longest request in every row
        ids, mask = pad_batch(prompts[:B])
        if self.kv is not None and (self.kv.rows != B or self.kv.max_pages[0] * self.page_size < longest + max_new_tokens + 1):
            self.kv = None
        if self.kv is None:
            geo = CacheGeometry(self.cfg.num_hidden_layers, self.w.nkv, self.cfg.head_dim, self.page_size)
            torch.cuda.empty_cache()
            self.kv = PagedKVCache(geo, B, longest + max_new_tokens + 1, self.max_iter, self.deep_fraction, dev)
            self._states.clear()
        logits, lens, _ = self.prefill(ids, mask, max_new_tokens)
        self._calls += 1
        s = self._tick_state(B, max_new_tokens, sampling, eos_token_id)
        if sampling is not None:
            s.seed_dev.fill_(int(seed) & (2 ** 62 - 1))
        s.pos.copy_(lens.to(torch.int32) - 1)
        s.need_soft.zero_()
        s.binding.tick_end(s.need_soft, first_tokens(logits, lens))
        s.cur_iters.zero_()
        owner = list(range(B))                       # request index held by each row (-1 = idle)
        next_req = B
        results: List[Optional[List[int]]] = [None] * n_req
        stats = {"ticks": 0, "admitted": B, "rows": B, "peak_pages": [0] * self.kv.n_depths, "pages_released": 0}
        if self.use_cuda_graph and s.graph is None:
            self._tick(s, sampling)                  # lazy one-time kernel setup outside capture
            stats["ticks"] += 1
        run = self._tick_runner(s, sampling)
        budget = (n_req // B + 2) * (max_new_tokens * self.max_iter + check_every + 1)
        while any(o >= 0 for o in owner) and stats["ticks"] < budget:
            for _ in range(check_every):
                run()
            stats["ticks"] += check_every
            done = ((s.finished != 0) | (s.n_out >= max_new_tokens)).tolist()
            for d in range(self.kv.n_depths):
                stats["peak_pages"][d] = max(stats["peak_pages"][d], self.kv.pages_in_use(d))
            fin = [r for r in range(B) if done[r] and owner[r] >= 0]
            if not fin:
                continue
            n_out = s.n_out.tolist()
            toks = s.out_tokens[fin].tolist()
            for r, row_toks in zip(fin, toks):
                results[owner[r]] = row_toks[:n_out[r]]
                owner[r] = -1
            rows_t = torch.tensor(fin, device=dev)
            stats["pages_released"] += self.kv.free_rows(rows_t)
            take = min(len(fin), n_req - next_req)
            if take:
                rows_new = rows_t[:take]
                ids, mask = pad_batch(prompts[next_req:next_req + take])
                logits, lens, _ = self.prefill(ids, mask, max_new_tokens, row_ids=rows_new)
                first = first_tokens(logits, lens).to(torch.int32)
                # what tick_end does for a row that emits its first token
                hit_eos = (first == eos_token_id) if eos_token_id is not None else torch.zeros_like(first, dtype=torch.bool)
                s.out_tokens[rows_new] = 0
                s.out_tokens[rows_new, 0] = torch.where(hit_eos, torch.zeros_like(first), first)
                s.n_out[rows_new] = (~hit_eos).to(torch.int32)
                s.finished[rows_new] = hit_eos.to(torch.int32)
                s.tokens_done += int((~hit_eos).sum())
                s.tok[rows_new], s.depth[rows_new] = first, 0
                s.pos[rows_new] = lens.to(torch.int32)
                s.cur_iters[rows_new], s.iter_sum[rows_new], s.need_soft[rows_new] = 0, 0, 0
                for j in range(take):
                    owner[fin[j]] = next_req + j
                next_req += take
                stats["admitted"] += take
        torch.cuda.synchronize()
        K.check_status(dev)
        if any(r is None for r in results):
            raise RuntimeError("serve(): tick budget exhausted before every request finished")
        stats["tokens"] = sum(len(r) for r in results)
        return results, stats

    def _tick_runner(self, s, sampling):
        if not self.use_cuda_graph:
            def run_eager():
                before = K.launch_count
                self._tick(s, sampling)
                self.kernel_launches_per_tick = K.launch_count - before
            return run_eager
        if s.graph is not None:
            self.graph_reuses += 1
            return s.graph.replay
        # Capture records the launches of one tick without running them.  Everything a tick touches
        # was allocated beforehand, so replays reuse the same addresses.
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        before = K.launch_count
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                self._tick(s, sampling)
        self.kernel_launches_per_tick = K.launch_count - before      # own kernels recorded in the graph
        torch.cuda.current_stream().wait_stream(side)
        s.graph = graph
        self.graph_captures += 1
        return graph.replay

    # ------------------------------------------------------------------------------------------
    # synthetic context (benchmarks)
    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def fast_forward(self, s, context: int) -> None:
        """Benchmark aid: make every row look as if it had already processed ``context`` tokens, so that ticks
        can be timed at a chosen decode depth without generating up to it.  The page tables of every depth
        get the pages a row of that length owns (taken from the free stacks exactly as a tick would), the
        lengths and positions are advanced, and the skipped tokens are counted as emitted.  The K/V content of
        the skipped positions is whatever the pools hold (zeros after allocation): the kernels' work per tick
        depends on the lengths only.  Call between ticks, with no tick in flight."""
        kv, ps, dev = self.kv, self.page_size, self.device
        B = s.pos.shape[0]
        torch.cuda.synchronize()
        pos_new = torch.full_like(s.pos, int(context))
        delta = (pos_new - s.pos).clamp(min=0)
        targets = [pos_new + (s.depth > 0).to(torch.int32)]
        for d in range(1, kv.n_depths):
            if self.hard_override is not None:
                cnt = (self.hard_override[:B, :context] >= d).sum(1).to(torch.int32)
            else:
                cnt = kv.len[d].clone()
            targets.append(cnt + (s.depth > d).to(torch.int32))
        rows = torch.arange(B, device=dev)
        for d, tgt in enumerate(targets):
            tgt = torch.maximum(tgt, kv.len[d]).to(torch.int64)
            have = (kv.len[d].to(torch.int64) + ps - 1) // ps
            need = (tgt + ps - 1) // ps - have
            total, free = int(need.sum()), int(kv.free_count[d])
            if total > free or int(((tgt + ps - 1) // ps).max()) > kv.max_pages[d]:
                raise RuntimeError(f"KV pool of depth {d} too small for a context of {context} tokens")
            if total > 0:
                first = torch.cumsum(need, 0) - need
                row_of_page = torch.repeat_interleave(rows, need)
                rank = torch.arange(total, device=dev)
                page_ids = kv.free_stack[d][(free - 1 - rank)]
                col = have[row_of_page] + rank - first[row_of_page]
                kv.page_table[d][row_of_page, col] = page_ids
                kv.free_count[d].fill_(free - total)
            kv.len[d].copy_(tgt.to(torch.int32))
        s.n_out += delta
        s.tokens_done += int(delta.sum())
        s.pos.copy_(torch.maximum(pos_new, s.pos))
        torch.cuda.synchronize()


_ENGINES = {}


def _lora_versions(model) -> tuple:
    """Version counters of the weights the engine copied or re-laid at construction (LoRA factors always,
    base weights when they are not already contiguous bf16)."""
    return tuple(p._version for p in model.simple_base_model.parameters())


def get_engine(model, **kw) -> TaHEngine:
    """One cached engine per model instance.  The engine keeps pre-scaled, re-laid copies of the LoRA factors,
    so it is rebuilt when those parameters were modified in place since it was made (e.g. by an optimizer step)."""
    key = id(model)
    ver = _lora_versions(model)
    hit = _ENGINES.get(key)
    if hit is not None and hit[1] == ver and hit[0].model is model:
        return hit[0]
    eng = TaHEngine(model, **kw)
    _ENGINES[key] = (eng, ver)
    return eng
