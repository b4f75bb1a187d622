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
    il = a.swiglu_interleaved
    wrows = 2 * F if (a.swiglu or il) else F
    n = _copies(wrows * Kd * 2 + M * Kd * 2, a.copies)
    ws = [_rand(wrows, Kd, scale=Kd ** -0.5) for _ in range(n)]
    xs = [_rand(M, Kd) for _ in range(n)]
    w2 = _rand(wrows, R, scale=0.05) if R else None
    x2 = _rand(M, R) if R else None
    out = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    plan = dict(bn=a.bn, splits=a.splits) if a.bn else {}
    if a.pair is not None:
        plan["pair"] = bool(a.pair)
    if a.transposed == "dgrad":          # dx[M, F] = dy[M, Kd] w[Kd, F]: the weight is read transposed in place
        fn = lambda i: K.gemm_t(xs[i % n], ws[i % n].view(Kd, wrows), w_t=True, out=out, **plan)
    elif a.transposed == "wgrad":        # dw[M, F] = dy[Kd, M]^T x[Kd, F]: both operands transposed (reduction over Kd tokens)
        gy = [_rand(Kd, M) for _ in range(n)]
        fn = lambda i: K.gemm_t(gy[i % n], ws[i % n].view(Kd, wrows), x_t=True, w_t=True, out=out, **plan)
    else:
        fn = lambda i: K.gemm(xs[i % n], ws[i % n], out=out, x2=x2, w2=w2, swiglu=a.swiglu, swiglu_interleaved=il, **plan)
    t = _time(fn, a.iters, a.warmup)
    flops = 2.0 * M * wrows * (Kd + R)
    byts = (wrows * (Kd + R) + M * (Kd + R) + M * F) * 2
    auto_pair = K.PAIR_AUTO and M >= K.PAIR_MIN_TOKENS and not a.bn and wrows % 256 == 0 and not a.swiglu
    res = {"op": "gemm", "M": M, "F": F, "K": Kd, "R": R, "swiglu": a.swiglu, "swiglu_interleaved": il,
           "transposed": a.transposed, "pair": bool(a.pair) if a.pair is not None else auto_pair,
           "plan_bn_splits": [a.bn, a.splits] if a.bn else K.plan_gemm(M, F, Kd, R, a.swiglu)}
    if a.cublas:
        ref = lambda i: torch.matmul(xs[i % n], ws[i % n].t())
        res["cublas_us"] = round(_time(ref, a.iters, a.warmup) * 1e6, 2)
    return res, t, flops, byts


def bench_gemm_qkv(a):
    """QKV projection of a decode tick (``--m`` rows, 16 q / 8 KV heads of 128, LoRA extension ``--r``): the plain
    GEMM followed by the QK-norm + RoPE + paged-KV-write kernel, against the GEMM with that work in its epilogue."""
    M, H, nq, nkv, hd, R = a.m, a.k, a.nq, a.nkv, 128, a.r
    F = (nq + 2 * nkv) * hd
    n = _copies(F * H * 2, a.copies)
    ws = [_rand(F, H, scale=H ** -0.5) for _ in range(n)]
    b = _rand(F, R, scale=0.05) if R else None
    x, t = _rand(M, H), (_rand(M, R) if R else None)
    qw, kw = torch.ones(hd, device="cuda", dtype=torch.bfloat16), torch.ones(hd, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 2000, (M,), device="cuda", dtype=torch.int32)
    pages = (M + 15) // 16 + 4
    caches = [torch.zeros(pages, 2, nkv, 16, hd, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    slot = torch.randperm(pages * 16, device="cuda")[:M].to(torch.int32)
    sel = torch.zeros(M, dtype=torch.int32, device="cuda")
    q = torch.empty(M, nq * hd, dtype=torch.bfloat16, device="cuda")
    qkv = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    table = K.rope_table(pos, hd, 1e6)
    ext = dict(x2=t, w2=b) if R else {}

    def separate(i):
        K.gemm(x, ws[i % n], out=qkv, **ext)
        K.qk_norm_rope_kv(qkv, qw, kw, pos, nq, nkv, hd, 1e-6, 1e6, q_out=q, caches=caches, cache_sel=sel, slot=slot,
                          page_size=16)

    def fused(i):
        K.gemm_qkv(x, ws[i % n], qw, kw, pos, nq, nkv, 1e-6, 1e6, q_out=q, caches=caches, cache_sel=sel, slot=slot,
                   page_size=16, rope_cs=table, **ext)

    t_sep = _time(separate, a.iters, a.warmup)
    t_fused = _time(fused, a.iters, a.warmup)
    res = {"op": "gemm_qkv", "M": M, "F": F, "K": H, "R": R, "separate_us": round(t_sep * 1e6, 2),
           "fused_us": round(t_fused * 1e6, 2)}
    return res, t_fused, 2.0 * M * F * (H + R), (F * (H + R) + M * (H + R) + M * F) * 2


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


# ---------------------------------------------------------------------------------------------
# multi-GPU cases: launch with  python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1
#                               -m tah_b200.ops.microbench --op tp_chain | shard_gather
# Device-timed with CUDA events, the launches of a batch replayed as one CUDA graph per rank where the
# sequence is capturable, maximum over ranks; rank 0 prints one JSON line.
# ---------------------------------------------------------------------------------------------
def _dist_init():
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    return dist, dev, dist.get_rank(), dist.get_world_size()


def _time_ranks(dist, dev, fn, iters, graph=True):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0.record()
        g.replay()
        e1.record()
    else:
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return round(float(t), 2)


def bench_tp_chain(a):
    """Row-parallel projection -> reduce + residual + RMSNorm -> column-parallel projection of a decode tick
    (``--m`` rows, hidden ``--k``), as the push chain (GEMM epilogue stores into the owners' slots, owner kernel
    broadcasts, the next GEMM's producer waits on landing flags), the pull chain (one fused all-reduce kernel
    between two plain GEMMs) and NCCL's all-reduce alone; plus the vocabulary-parallel top-k merge kernel against
    its all-gather + sort form.  Microseconds per iteration."""
    from tah_b200.parallel.tp import TensorParallel
    dist, dev, rank, world = _dist_init()
    M, H, Fq = a.m, a.k, a.f
    iters = a.iters if a.iters > 20 else 100
    tp = TensorParallel(dist.group.WORLD, dev, H, M, use_multicast=not a.no_multicast)
    h, ln = _rand(M, H).to(dev), torch.ones(H, device=dev, dtype=torch.bfloat16)
    x, w = _rand(M, H // world).to(dev), _rand(H, H // world, scale=0.02).to(dev)
    wq = _rand(Fq // world, H, scale=0.02).to(dev)
    qkv = torch.empty(M, Fq // world, device=dev, dtype=torch.bfloat16)
    desc = tp.push_desc(M)
    tp.partial.normal_()
    buf = _rand(M, H).to(dev)

    def chain_push():
        K.gemm(x, w, tp_push=desc)
        xn = tp.push_reduce_norm(M, h, ln, 1e-6)
        K.gemm(xn, wq, out=qkv, tp_wait=tp.wait_desc)

    def chain_pull():
        K.gemm(x, w, out=tp.partial[:M])
        xn = tp.fused_reduce_norm(M, h, ln, 1e-6)
        K.gemm(xn, wq, out=qkv)

    res = {"op": "tp_chain", "world": world, "rows": M, "hidden": H, "multicast": bool(tp.mc_partial),
           "us": {"chain_push": _time_ranks(dist, dev, chain_push, iters),
                  "chain_pull": _time_ranks(dist, dev, chain_pull, iters),
                  "fused_reduce_norm_alone": _time_ranks(dist, dev, lambda: tp.fused_reduce_norm(M, h, ln, 1e-6), iters),
                  "row_gemm_alone": _time_ranks(dist, dev, lambda: K.gemm(x, w, out=tp.partial[:M]), iters),
                  "col_gemm_alone": _time_ranks(dist, dev, lambda: K.gemm(tp.xout[:M], wq, out=qkv), iters),
                  "nccl_all_reduce_alone": _time_ranks(dist, dev, lambda: dist.all_reduce(buf), iters)}}
    k = a.topk
    val = torch.sort(torch.randn(M, k, device=dev), dim=-1, descending=True).values.contiguous()
    idx = torch.sort(torch.randint(0, 1 << 14, (M, k), device=dev, dtype=torch.int32), dim=-1).values.contiguous()
    tp.prepare_merge(M)
    lo = rank << 14
    res["us"]["topk_merge_kernel"] = _time_ranks(dist, dev, lambda: tp.merge_topk(val, idx, lo, k), 20)
    res["us"]["topk_merge_nccl_sort"] = _time_ranks(dist, dev, lambda: tp.merge_topk_nccl(val, idx, lo, k), 20)
    # bytes that must cross NVLink per rank and chain: partial rows out to the owners + normalised rows out to the peers
    byts = 2 * M * H * 2 * (world - 1) / world
    res["nvlink_bytes_per_rank"] = int(byts)
    res["nvlink_floor_us_at_770GBps"] = round(byts / 770e9 * 1e6, 2)
    K.check_status()
    return res, rank


def bench_shard_gather(a):
    """Parameter-sharded linears: the 4 x 7 matrices of seven 1.7B-model layers, every rank holding 1/world of each,
    gathered by the push kernel one matrix ahead on a side stream while the tcgen05 GEMM of the previous matrix
    (whose producer waits on the landing flags) runs.  Milliseconds for the 28 GEMMs at ``--m`` tokens."""
    from tah_b200.parallel.fsdp import ShardedWeightStore
    dist, dev, rank, world = _dist_init()
    M = a.m if a.m > 256 else 8192
    shapes = [(4096, 2048), (2048, 2048), (12288, 2048), (2048, 6144)] * 7
    full = [_rand(F, Kd, scale=0.02).to(dev) for F, Kd in shapes]
    xs = {Kd: _rand(M, Kd).to(dev) for Kd in (2048, 6144)}
    us = lambda f: round(_time_ranks(dist, dev, f, 3, graph=False) / 1e3, 3)

    def plain():
        for w in full:
            K.gemm(xs[w.shape[1]], w)

    store = ShardedWeightStore(dist.group.WORLD, dev, full, n_buffers=2, use_multicast=not a.no_multicast)

    def sharded():
        store.prefetch(0)
        for i in range(len(full)):
            if i + 1 < len(full):
                store.prefetch(i + 1)
            store.linear(xs[shapes[i][1]], i)

    def gather_only():
        for i in range(len(full)):
            store.prefetch(i)
            store._where.pop(i)
        torch.cuda.current_stream().wait_stream(store.side)

    byts = sum(F * Kd * 2 for F, Kd in shapes)
    t_plain, t_sh, t_g = us(plain), us(sharded), us(gather_only)
    recv = byts * (world - 1) / world
    res = {"op": "shard_gather", "world": world, "tokens": M, "multicast": bool(store.buf_mc[0]),
           "ms": {"gemms_on_full_weights": t_plain, "gemms_on_sharded_weights_prefetch_one_ahead": t_sh, "gathers_alone": t_g},
           "gathered_GB": round(byts / 1e9, 3), "received_GBps_per_rank": round(recv / (t_g * 1e-3) / 1e9, 1),
           "hidden_fraction_of_gather": round(max(0.0, 1.0 - (t_sh - t_plain) / t_g), 3),
           "nvlink_floor_ms_at_770GBps": round(recv / 770e9 * 1e3, 3)}
    K.check_status()
    return res, rank


DIST_OPS = {"tp_chain": bench_tp_chain, "shard_gather": bench_shard_gather}

OPS = {"gemm_qkv": bench_gemm_qkv, "attn_bwd": bench_attn_bwd, "gemm": bench_gemm, "decode_attn": bench_decode_attn, "prefill_attn": bench_prefill_attn, "topk": bench_topk,
       "rmsnorm": bench_rmsnorm}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--op", choices=sorted(list(OPS) + list(DIST_OPS)), required=True)
    ap.add_argument("--no-multicast", action="store_true", help="multi-GPU cases: plain peer stores instead of multimem")
    ap.add_argument("--m", type=int, default=256)
    ap.add_argument("--f", type=int, default=4096)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--r", type=int, default=0, help="LoRA K-extension width")
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--swiglu-interleaved", action="store_true", help="SwiGLU on interleaved gate / up rows (one accumulator)")
    ap.add_argument("--pair", type=int, default=None, help="1 / 0: force the two-tile (pair) form on / off (default: automatic)")
    ap.add_argument("--transposed", default="", choices=["", "dgrad", "wgrad"],
                    help="time the transposed-operand forms used by the backward pass (reduction length = --k)")
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
    if a.op in DIST_OPS:
        res, rank = DIST_OPS[a.op](a)
        if rank == 0:
            print(json.dumps(res), flush=True)
        import torch.distributed as dist
        dist.barrier()
        os._exit(0)                       # symmetric-memory mappings are alive: skip the process-group teardown
    res, t, flops, byts = OPS[a.op](a)
    bw, fl, src = peaks()
    res.update({"graph": a.graph, "us": round(t * 1e6, 2), "GBps": round(byts / t / 1e9, 1), "TFLOPs": round(flops / t / 1e12, 1),
                "frac_hbm": round(byts / t / bw, 3), "frac_bf16": round(flops / t / fl, 3), "peaks": src})
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
