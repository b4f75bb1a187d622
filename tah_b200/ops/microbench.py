"""Per-kernel micro-benchmarks with roofline fractions.

``python -m tah_b200.ops.microbench --op gemm --m 256 --f 4096 --k 2048``

Each case rotates through enough distinct operand copies that a timed launch never finds its
inputs in L2 (the working set is larger than the 126 MB L2), is warmed up, and is timed with CUDA
events on the launching stream.  Fractions are against the measured copy bandwidth / cuBLAS bf16
throughput in ``MEASURED_PEAKS.json`` at the repository root when present (else 6.65 TB/s,
1.59 PFLOP/s).  ``--iters 1 --warmup 0 --copies 1`` gives the minimal run used under a profiler.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from tah_b200.ops import cuda as K

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
L2_BYTES = 126 << 20


def peaks():
    path = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


USE_GRAPH = False


def _time(fn, iters, warmup):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if USE_GRAPH:
        # the launches of one timed batch replayed as a CUDA graph: no host launch cost in the number
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(iters):
                fn(warmup + i)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
    else:
        e0.record()
        for i in range(iters):
            fn(warmup + i)
        e1.record()
    torch.cuda.synchronize()
    K.check_status()
    return e0.elapsed_time(e1) * 1e-3 / max(iters, 1)


def _copies(bytes_per_copy, want):
    return want if want > 0 else max(2, min(64, (2 * L2_BYTES) // max(bytes_per_copy, 1) + 1))


def bench_gemm(a):
    M, F, Kd, R = a.m, a.f, a.k, a.r
    wrows = 2 * F if a.swiglu else F
    n = _copies(wrows * Kd * 2 + M * Kd * 2, a.copies)
    ws = [_rand(wrows, Kd, scale=Kd ** -0.5) for _ in range(n)]
    xs = [_rand(M, Kd) for _ in range(n)]
    w2 = _rand(wrows, R, scale=0.05) if R else None
    x2 = _rand(M, R) if R else None
    out = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    plan = dict(bn=a.bn, splits=a.splits) if a.bn else {}
    fn = lambda i: K.gemm(xs[i % n], ws[i % n], out=out, x2=x2, w2=w2, swiglu=a.swiglu, **plan)
    t = _time(fn, a.iters, a.warmup)
    flops = 2.0 * M * wrows * (Kd + R)
    byts = (wrows * (Kd + R) + M * (Kd + R) + M * F) * 2
    res = {"op": "gemm", "M": M, "F": F, "K": Kd, "R": R, "swiglu": a.swiglu, "plan_bn_splits": [a.bn, a.splits] if a.bn else K.plan_gemm(M, F, Kd, R, a.swiglu)}
    if a.cublas:
        ref = lambda i: torch.matmul(xs[i % n], ws[i % n].t())
        res["cublas_us"] = round(_time(ref, a.iters, a.warmup) * 1e6, 2)
    return res, t, flops, byts


def bench_decode_attn(a):
    nq, nkv, hd, page = a.nq, a.nkv, a.hd, 16
    rows, ctx = a.rows, a.ctx
    ppr = (ctx + page - 1) // page + 1
    per_copy = rows * ppr * 2 * nkv * page * hd * 2
    n = _copies(per_copy, a.copies)
    pools = [_rand(rows * ppr, 2, nkv, page, hd) for _ in range(n)]
    pt = torch.randperm(rows * ppr, device="cuda").view(rows, ppr).int()
    ln = torch.full((rows,), ctx, dtype=torch.int32, device="cuda")
    pool1 = _rand(rows * 4, 2, nkv, page, hd)
    pt1 = torch.arange(rows * 4, device="cuda").view(rows, 4).int()
    ln1 = torch.full((rows,), 20, dtype=torch.int32, device="cuda")
    depth = (torch.rand(rows, device="cuda") < 0.06).int()
    q = _rand(rows, nq * hd)
    out = torch.empty_like(q)
    ws = None
    if a.nsplit > 1:
        ws = torch.empty(int(K.lib().tahb_decode_attn_ws_floats(rows, nq, hd, a.nsplit)), dtype=torch.float32, device="cuda")
    fn = lambda i: K.decode_attn(q, [pools[i % n], pool1], [pt, pt1], [ln, ln1], depth, nq, nkv, hd, page, hd ** -0.5, out=out,
                                 n_split=a.nsplit, ws=ws)
    t = _time(fn, a.iters, a.warmup)
    byts = rows * ctx * 2 * nkv * hd * 2
    return {"op": "decode_attn", "rows": rows, "ctx": ctx, "nq": nq, "nkv": nkv, "hd": hd, "n_split": a.nsplit}, t, 4.0 * rows * nq * hd * ctx, byts


def bench_prefill_attn(a):
    nq, nkv, hd = a.nq, a.nkv, a.hd
    B, L = a.rows, a.ctx
    ntok = B * L
    per_copy = ntok * (nq + 2 * nkv) * hd * 2
    n = _copies(per_copy, a.copies)
    qs = [_rand(ntok, nq * hd) for _ in range(n)]
    ks = [_rand(ntok, nkv * hd) for _ in range(n)]
    vs = [_rand(ntok, nkv * hd) for _ in range(n)]
    lens = torch.full((B,), L, device="cuda")
    base = (torch.arange(B, device="cuda") * L).repeat_interleave(L).to(torch.int32)
    cnt = (torch.arange(L, device="cuda") + 1).repeat(B).to(torch.int32)
    tq0, tqn = K.attn_tiles(lens)
    out = torch.empty_like(qs[0])
    fn = lambda i: K.prefill_attn(qs[i % n], [ks[i % n]], [vs[i % n]], [base], [cnt], tq0, tqn, nq, nkv, hd, hd ** -0.5, out=out)
    t = _time(fn, a.iters, a.warmup)
    flops = 4.0 * B * nq * hd * L * (L + 1) / 2
    byts = per_copy + ntok * nq * hd * 2
    return {"op": "prefill_attn", "seqs": B, "len": L, "nq": nq, "nkv": nkv, "hd": hd, "flops_counted": "causal half"}, t, flops, byts


def bench_attn_bwd(a):
    """Backward of the packed causal attention: dQ kernel + dK/dV kernel (the forward supplies lse)."""
    nq, nkv, hd = a.nq, a.nkv, a.hd
    B, L = a.rows, a.ctx
    ntok = B * L
    q, k, v, do = _rand(ntok, nq * hd), _rand(ntok, nkv * hd), _rand(ntok, nkv * hd), _rand(ntok, nq * hd)
    lens = torch.full((B,), L, device="cuda")
    base = (torch.arange(B, device="cuda") * L).repeat_interleave(L).to(torch.int32)
    cnt = (torch.arange(L, device="cuda") + 1).repeat(B).to(torch.int32)
    tq0, tqn = K.attn_tiles(lens)
    items = K.attn_kv_items(lens, torch.arange(B, device="cuda") * L, lens)
    lse = torch.empty(ntok, nq, dtype=torch.float32, device="cuda")
    out = K.prefill_attn(q, [k], [v], [base], [cnt], tq0, tqn, nq, nkv, hd, hd ** -0.5, lse=lse)
    dsum = (do.float() * out.float()).view(ntok, nq, hd).sum(-1).contiguous()
    dq = torch.empty_like(q)
    dk, dv = torch.zeros_like(k), torch.zeros_like(v)
    f_dq = lambda i: K.attn_bwd_dq(q, do, [k], [v], [base], [cnt], tq0, tqn, nq, nkv, hd, hd ** -0.5, lse, dsum, out=dq)
    f_kv = lambda i: K.attn_bwd_dkv(q, do, k, v, cnt, items, nq, nkv, hd, hd ** -0.5, lse, dsum, dk=dk, dv=dv)
    t_dq = _time(f_dq, a.iters, a.warmup)
    t_kv = _time(f_kv, a.iters, a.warmup)
    fwd = 4.0 * B * nq * hd * L * (L + 1) / 2
    res = {"op": "attn_bwd", "seqs": B, "len": L, "nq": nq, "nkv": nkv, "hd": hd, "dq_us": round(t_dq * 1e6, 1),
           "dkv_us": round(t_kv * 1e6, 1), "flops_counted": "2.5 x causal forward"}
    return res, t_dq + t_kv, 2.5 * fwd, ntok * (2 * nq + 2 * nkv) * hd * 2 * 2


def bench_topk(a):
    rows, V, k = a.rows, a.v, a.topk
    n = _copies(rows * V * 2, a.copies)
    xs = [_rand(rows, V, scale=3.0) for _ in range(n)]
    val = torch.zeros(rows, k, dtype=torch.float32, device="cuda")
    idx = torch.zeros(rows, k, dtype=torch.int32, device="cuda")
    fn = lambda i: K.topk_rows(xs[i % n], k, out_val=val, out_idx=idx)
    t = _time(fn, a.iters, a.warmup)
    return {"op": "topk_rows", "rows": rows, "V": V, "k": k}, t, 0.0, rows * V * 2


def bench_rmsnorm(a):
    M, H = a.m, a.k
    n = _copies(M * H * 2, a.copies)
    xs = [_rand(M, H) for _ in range(n)]
    w = _rand(H)
    out = torch.empty_like(xs[0])
    fn = lambda i: K.rms_norm(xs[i % n], w, 1e-6, out=out)
    t = _time(fn, a.iters, a.warmup)
    return {"op": "rms_norm", "M": M, "H": H}, t, 0.0, 2 * M * H * 2


OPS = {"attn_bwd": bench_attn_bwd, "gemm": bench_gemm, "decode_attn": bench_decode_attn, "prefill_attn": bench_prefill_attn, "topk": bench_topk,
       "rmsnorm": bench_rmsnorm}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--op", choices=sorted(OPS), required=True)
    ap.add_argument("--m", type=int, default=256)
    ap.add_argument("--f", type=int, default=4096)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--r", type=int, default=0, help="LoRA K-extension width")
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--bn", type=int, default=0, help="force the token-tile width (with --splits) instead of the planner")
    ap.add_argument("--splits", type=int, default=1, help="split-K cluster size used with --bn")
    ap.add_argument("--cublas", action="store_true", help="also time torch.matmul on the same operands")
    ap.add_argument("--rows", type=int, default=256, help="decode rows / prefill sequences / top-k rows")
    ap.add_argument("--ctx", type=int, default=1024, help="context (decode) or sequence length (prefill)")
    ap.add_argument("--nsplit", type=int, default=1, help="decode attention: split each row's KV walk over this many CTAs")
    ap.add_argument("--nq", type=int, default=16)
    ap.add_argument("--nkv", type=int, default=8)
    ap.add_argument("--hd", type=int, default=128)
    ap.add_argument("--v", type=int, default=151936)
    ap.add_argument("--topk", type=int, default=100)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--copies", type=int, default=0, help="operand copies to rotate through (0 = enough to exceed L2)")
    ap.add_argument("--graph", action="store_true", help="replay the timed launches as one CUDA graph (small kernels)")
    a = ap.parse_args(argv)
    global USE_GRAPH
    USE_GRAPH = a.graph
    torch.manual_seed(0)
    res, t, flops, byts = OPS[a.op](a)
    bw, fl, src = peaks()
    res.update({"graph": a.graph, "us": round(t * 1e6, 2), "GBps": round(byts / t / 1e9, 1), "TFLOPs": round(flops / t / 1e12, 1),
                "frac_hbm": round(byts / t / bw, 3), "frac_bf16": round(flops / t / fl, 3), "peaks": src})
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
