"""ctypes bindings for the hand-written sm_100a kernels in ``csrc/`` (``libtahb200.so``).

Every wrapper takes torch CUDA tensors, launches on the current torch stream and
returns torch tensors.  The library is built in-tree by :mod:`tah_b200.ops.build`; if it
is missing on a machine with a CUDA device, loading raises (no silent fallback).

Kernels that wait on hardware barriers give up after a bounded time and set a status
word; :func:`check_status` reads it (a host sync) and raises :class:`KernelTimeout`.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence

import torch

_LIB = None
# TAH_B200_LIB: load another build of the library (A/B timing of kernel changes)
_LIB_PATH = os.environ.get("TAH_B200_LIB") or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                                           "lib", "libtahb200.so")

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


class KernelTimeout(RuntimeError):
    pass


STATUS_NAMES = {1: "timeout waiting for a TMA load", 2: "timeout waiting for a free pipeline stage",
                3: "timeout waiting for the accumulator", 4: "timeout waiting for a peer flag",
                5: "index out of range / KV pages exhausted"}


def lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(_LIB_PATH):
            from tah_b200.ops.build import build
            build()
        _LIB = ctypes.CDLL(_LIB_PATH)
        _LIB.tahb_decode_attn_ws_floats.restype = c_ll
    return _LIB


def available() -> bool:
    return torch.cuda.is_available()


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_status = {}


def status_word(device=None) -> torch.Tensor:
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    if dev.type != "cuda":
        dev = torch.device("cuda", torch.cuda.current_device())
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _status[key]


def check_status(device=None) -> None:
    """Read the status word (synchronises) and raise if a kernel reported a failure."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise KernelTimeout(f"tah_b200 kernel status {code}: {STATUS_NAMES.get(code, 'unknown')}")


launch_count = 0      # number of library entry points called (each launches at least one kernel)


def _rc(rc: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed on the host side (code {rc})")


def _check_bf16_2d(t: torch.Tensor, name: str):
    if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1 or not t.is_cuda:
        raise ValueError(f"{name}: need a 2-D bf16 CUDA tensor with unit inner stride, got {t.dtype} {tuple(t.shape)} {t.stride()}")


# -------------------------------------------------------------------------------------------
# GEMM
# -------------------------------------------------------------------------------------------
SM_COUNT = 148


def _fits(bn: int, s: int, nacc: int) -> bool:
    stage = 16384 * nacc + bn * 128
    ns = min(8, (196 * 1024) // stage)
    if s == 1:
        return True
    per = bn // s
    if bn % s or per % 16:
        return False
    red = ((s - 1) * 128 * nacc * per * 4 + 1023) // 1024 * 1024
    return red + per * 256 <= ns * stage


def plan_gemm(M: int, F: int, K: int, R: int = 0, dual: bool = False):
    """Pick the token-tile width and the split-K cluster size with a small cost model.

    Measured on B200: a k-block (64 of K) costs about 0.3 us of load latency per CTA unless the
    tensor-core time of the tile is larger, the epilogue about 0.5 us + 8 ns per token column,
    and clusters larger than 4 CTAs (one ~200 KB CTA per SM) no longer fit in one wave.
    """
    nacc = 2 if dual else 1
    kb = K // 64 + R // 64
    base = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
    cands = [base] + ([128, 64] if base == 256 else [64] if base == 128 else [])
    best = None
    for bn in cands:
        for s in (1, 2, 4):
            if s > 1 and (kb // s < 2 or not _fits(bn, s, nacc)):
                continue
            ctas = ((F + 127) // 128) * ((M + bn - 1) // bn) * s
            waves = (ctas + SM_COUNT - 1) // SM_COUNT
            t_kb = max(0.30, 128 * bn * 64 * 2 * nacc / 8192 / 1900.0)
            per = bn // s
            t_cta = (kb / s) * t_kb + 0.5 + 0.009 * per
            if s > 1:
                pushed_kb = (s - 1) * per * nacc * 0.5            # KiB sent to the peers through DSMEM
                t_cta += 1.0 + pushed_kb / 19.0 + (0.07 * per if dual else 0.0)
            t = waves * t_cta
            if best is None or t < best[0] - 1e-9:
                best = (t, bn, s)
    return best[1], best[2]


# token count from which the two-tile ("pair") GEMM is the default; TAH_B200_GEMM_PAIR=0 turns it off
PAIR_AUTO = os.environ.get("TAH_B200_GEMM_PAIR", "1") != "0"
PAIR_MIN_TOKENS = 1024


def interleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    """``[2I, K]`` gate rows then up rows -> ``[2I, K]`` with rows ``gate_0, up_0, gate_1, up_1, ...`` (the layout
    :func:`gemm` wants for ``swiglu_interleaved``; apply it to the LoRA-B extension of the projection as well)."""
    half = w.shape[0] // 2
    return torch.stack((w[:half], w[half:]), dim=1).reshape(w.shape).contiguous()


def pick_splits(M: int, F: int, K: int, R: int = 0, dual: bool = False) -> int:
    return plan_gemm(M, F, K, R, dual)[1]


_pending_gemm_wait = None


def set_pending_gemm_wait(desc) -> None:
    """The next :func:`gemm` / :func:`gemm_qkv` call without a ``tp_wait`` of its own takes ``desc = (flags,
    targets)``: its TMA producer waits for those landing flags before the first load.  Used by parameter-sharded
    training, where the first GEMM of a layer consumes the all-gather of the layer's weights."""
    global _pending_gemm_wait
    _pending_gemm_wait = desc


def clear_pending_gemm_wait() -> bool:
    """Drop a pending wait; returns True if one was still pending (nobody consumed it)."""
    global _pending_gemm_wait
    had = _pending_gemm_wait is not None
    _pending_gemm_wait = None
    return had


def _take_pending_wait(tp_wait):
    global _pending_gemm_wait
    if tp_wait is None and _pending_gemm_wait is not None:
        tp_wait, _pending_gemm_wait = _pending_gemm_wait, None
    return tp_wait


def wait_flags(flags: torch.Tensor, targets: torch.Tensor) -> None:
    """Stream-ordered bounded wait (one tiny kernel) until ``flags[q] >= targets[q]`` for every q: gates kernels
    that cannot wait themselves, e.g. library GEMMs reading a gather buffer that peers fill."""
    _rc(lib().tahb_wait_flags(_p(flags), _p(targets), c_int(flags.numel()), _p(status_word(flags.device)), _stream()),
        "tahb_wait_flags")


def gemm(x: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, x2: Optional[torch.Tensor] = None,
         w2: Optional[torch.Tensor] = None, swiglu: bool = False, splits: Optional[int] = None,
         bn: int = 0, tp_push=None, tp_wait=None, gelu: bool = False, swiglu_interleaved: bool = False,
         pair: Optional[bool] = None) -> torch.Tensor:
    """``out[M,F] = x[M,K] @ w[F,K]^T (+ x2[M,R] @ w2[F,R]^T) (+ residual)``; with ``swiglu`` the
    weight is ``[2F, K]`` (gate rows then up rows) and ``out = silu(gate) * up``.

    ``gelu``: the epilogue applies the erf GELU to the bf16-rounded output (not together with ``residual``).

    ``pair``: every CTA computes two 128-feature output tiles (features ``f`` and ``F/2 + f``) from one 256-token
    activation tile, unsplit.  It halves the activation bytes a CTA pulls per unit of work, which is what bounds
    the kernel at large token counts (1350-1400 vs 915-1100 TFLOP/s at 8192+ tokens); default: on from
    ``PAIR_MIN_TOKENS`` tokens when the shape allows it (also with ``swiglu_interleaved``).

    ``swiglu_interleaved``: the rows of ``w`` (and ``w2``) alternate ``gate_i, up_i`` (see :func:`interleave_gate_up`)
    and ``out[M, F/2] = silu(gate) * up``: one accumulator and one wide MMA per k step, the faster SwiGLU form.

    Tensor parallel (see :class:`tah_b200.parallel.tp.TensorParallel`): ``tp_push =
    (slot_ptrs, cnt_ptrs, rank, rows_per_rank)`` replaces the output by peer stores of the tile
    rows into their owners' slot buffers (reduce-scatter by push, ``out`` is not written);
    ``tp_wait = (flags, targets)`` makes the kernel wait for the broadcast rows of ``x``."""
    _check_bf16_2d(x, "x")
    _check_bf16_2d(w, "w")
    tp_wait = _take_pending_wait(tp_wait)
    M, K = x.shape
    F = w.shape[0] // 2 if swiglu else w.shape[0]
    F_out = F // 2 if swiglu_interleaved else F
    if swiglu_interleaved and (swiglu or gelu or residual is not None or tp_push is not None or F % 2):
        raise ValueError("swiglu_interleaved excludes swiglu / gelu / residual / tp_push")
    if w.shape[1] != K:
        raise ValueError(f"K mismatch: x {tuple(x.shape)} w {tuple(w.shape)}")
    R = 0
    if x2 is not None:
        _check_bf16_2d(x2, "x2")
        _check_bf16_2d(w2, "w2")
        R = x2.shape[1]
        if w2.shape[1] != R or w2.shape[0] != w.shape[0] or x2.shape[0] != M:
            raise ValueError("K-extension operands do not match")
    if tp_push is not None:
        out = x.new_empty(0, F) if out is None else out
    elif out is None:
        out = torch.empty(M, F_out, dtype=torch.bfloat16, device=x.device)
    else:
        _check_bf16_2d(out, "out")
    if residual is not None:
        _check_bf16_2d(residual, "residual")
    if pair is None:
        pair = (PAIR_AUTO and M >= PAIR_MIN_TOKENS and bn == 0 and splits is None and not swiglu and not gelu
                and w.shape[0] % 256 == 0)
    pair = bool(pair) and not swiglu and not gelu and w.shape[0] % 256 == 0
    if pair:
        bn, splits = 256, 1
    elif swiglu_interleaved:
        splits = 1                       # the interleaved epilogue exists for unsplit tiles
        if bn == 0:
            bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
    elif splits is None and bn == 0:
        bn, splits = plan_gemm(M, F, K, R, swiglu)
    elif splits is None:
        splits = 1
    args = (_p(w), _p(x), _p(out), _p(residual), _p(w2), _p(x2), c_int(M), c_int(F), c_int(K), c_int(R),
            c_ll(w.stride(0)), c_ll(x.stride(0)), c_ll(out.stride(0)),
            c_ll(residual.stride(0) if residual is not None else 0),
            c_ll(w2.stride(0) if w2 is not None else 0), c_ll(x2.stride(0) if x2 is not None else 0),
            c_int(1 if swiglu else 3 if gelu else (6 if pair else 4) if swiglu_interleaved else 2 if pair else 0), c_int(F if swiglu else 0), c_int(splits), c_int(bn),
            _p(status_word(x.device)), _stream())
    if tp_push is None and tp_wait is None:
        rc = lib().tahb_gemm(*args)
    else:
        if tp_push is not None:
            slot_ptrs, cnt_ptrs, rank, rpr = tp_push
            n = len(slot_ptrs)
            push = ((c_void_p * n)(*slot_ptrs), (c_void_p * n)(*cnt_ptrs), c_int(n), c_int(rank), c_int(rpr))
        else:
            push = (None, None, c_int(0), c_int(0), c_int(0))
        if tp_wait is not None:
            flags, targets = tp_wait
            wait = (_p(flags), _p(targets), c_int(flags.numel()))
        else:
            wait = (None, None, c_int(0))
        rc = lib().tahb_gemm_tp(*args, *push, *wait)
    _rc(rc, "tahb_gemm")
    return out


def gemm_t(x: torch.Tensor, w: torch.Tensor, *, x_t: bool = False, w_t: bool = False, out: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None, splits: Optional[int] = None, bn: int = 0,
           pair: Optional[bool] = None) -> torch.Tensor:
    """GEMM with operands read transposed straight from their row-major storage (the backward GEMMs):

    * ``w_t``: ``w`` is ``[K, F]`` (instead of ``[F, K]``); * ``x_t``: ``x`` is ``[K, M]`` (instead of ``[M, K]``);

    ``out[M, F] = op(x) @ op(w)^T (+ residual)``.  Data gradient of ``y = x W^T``: ``gemm_t(dy, W, w_t=True)``; weight
    gradient: ``gemm_t(dy, x, x_t=True, w_t=True, residual=grad, out=grad)`` (reduction over the tokens, any count).
    Same tcgen05 kernel as :func:`gemm`; the transposed tiles are described to the tensor core as MN-major."""
    _check_bf16_2d(x, "x")
    _check_bf16_2d(w, "w")
    if x_t:
        Kx, M = x.shape
    else:
        M, Kx = x.shape
    if w_t:
        Kw, F = w.shape
    else:
        F, Kw = w.shape
    if Kx != Kw:
        raise ValueError(f"reduction mismatch: x {tuple(x.shape)} (x_t={x_t}) w {tuple(w.shape)} (w_t={w_t})")
    if not (x_t or w_t):
        return gemm(x, w, out=out, residual=residual, splits=splits, bn=bn, pair=pair)
    if out is None:
        out = torch.empty(M, F, dtype=torch.bfloat16, device=x.device)
    if residual is not None:
        _check_bf16_2d(residual, "residual")
    if pair is None:
        pair = PAIR_AUTO and M >= PAIR_MIN_TOKENS and bn == 0 and splits is None
    pair = bool(pair) and F % 256 == 0 and (not x_t or M % 64 == 0)
    if pair:
        bn, splits = 256, 1
    elif splits is None and bn == 0:
        bn, splits = plan_gemm(M, F, (Kx + 63) // 64 * 64, 0, False)
        if x_t:
            bn = max(bn, 64)
    elif splits is None:
        splits = 1
    _rc(lib().tahb_gemm_t(_p(w), _p(x), _p(out), _p(residual), c_int(M), c_int(F), c_int(Kx), c_ll(w.stride(0)),
                          c_ll(x.stride(0)), c_ll(out.stride(0)), c_ll(residual.stride(0) if residual is not None else 0),
                          c_int(1 if w_t else 0), c_int(1 if x_t else 0), c_int(splits), c_int(bn),
                          _p(status_word(x.device)), _stream(), c_int(1 if pair else 0)), "tahb_gemm_t")
    return out


# -------------------------------------------------------------------------------------------
# elementwise / norm / rope
# -------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _check_bf16_2d(x, "x")
    if out is None:
        out = torch.empty_like(x)
    _rc(lib().tahb_rmsnorm(_p(x), _p(w), _p(out), c_int(x.shape[0]), c_int(x.shape[1]), c_ll(x.stride(0)),
                           c_ll(out.stride(0)), c_float(eps), _stream()), "tahb_rmsnorm")
    return out


def rms_norm_lora(x: torch.Tensor, w: torch.Tensor, eps: float, gate: torch.Tensor, A: torch.Tensor,
                  out: Optional[torch.Tensor] = None, t_out: Optional[torch.Tensor] = None):
    """RMSNorm of every row and, in the same launch, ``t[r] = gate[r] ? y[r] @ A^T : 0`` (the LoRA-A product of the
    rows at depth >= 1 of a decode tick).  Returns ``(y, t)``."""
    _check_bf16_2d(x, "x")
    M, H = x.shape
    R = A.shape[0]
    if out is None:
        out = torch.empty_like(x)
    if t_out is None:
        t_out = torch.empty(M, R, dtype=torch.bfloat16, device=x.device)
    if A.shape[1] != H or not A.is_contiguous():
        raise ValueError("rms_norm_lora: A must be a contiguous [R, H] matrix")
    _rc(lib().tahb_rmsnorm_lora(_p(x), _p(w), _p(out), c_int(M), c_int(H), c_ll(x.stride(0)), c_ll(out.stride(0)),
                                c_float(eps), _p(gate), _p(A), _p(t_out), c_int(R), c_ll(t_out.stride(0)), _stream()),
        "tahb_rmsnorm_lora")
    return out, t_out


def layer_norm(x, w, b, eps: float = 1e-5, out=None):
    """LayerNorm over the last dimension of bf16 ``x [M, D]`` (fp32 statistics)."""
    _check_bf16_2d(x, "x")
    M, D = x.shape
    if out is None:
        out = torch.empty(M, D, dtype=torch.bfloat16, device=x.device)
    _rc(lib().tahb_layernorm(_p(x), _p(w), _p(b), _p(out), None, None, None, c_int(M), c_int(D), c_ll(x.stride(0)),
                             c_ll(out.stride(0)), c_float(eps), _stream()), "tahb_layernorm")
    return out


def layer_norm_dot(x, w, b, dot_w, dot_b, eps: float = 1e-5, out=None):
    """``z[r] = bf16(LayerNorm(x[r]) . dot_w + dot_b)`` as fp32: LayerNorm followed by ``Linear(D, 1)``."""
    _check_bf16_2d(x, "x")
    M, D = x.shape
    if out is None:
        out = torch.empty(M, dtype=torch.float32, device=x.device)
    _rc(lib().tahb_layernorm(_p(x), _p(w), _p(b), None, _p(dot_w), _p(dot_b), _p(out), c_int(M), c_int(D),
                             c_ll(x.stride(0)), c_ll(0), c_float(eps), _stream()), "tahb_layernorm")
    return out


def rope_table(pos: torch.Tensor, hd: int, theta: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[M, hd]`` bf16 RoPE table of a pass: ``cos`` of the ``hd/2`` frequencies at ``pos[t]``, then ``sin``."""
    M = pos.shape[0]
    if out is None:
        out = torch.empty(M, hd, dtype=torch.bfloat16, device=pos.device)
    _rc(lib().tahb_rope_table(_p(pos), _p(out), c_int(M), c_int(hd), c_float(theta), _stream()), "tahb_rope_table")
    return out


def set_peer_wait_limit_ns(ns: int) -> int:
    """How long kernels wait for a flag that a peer GPU advances before they give up (status 4); 0 = default
    (2 s).  Returns the previous limit."""
    fn = lib().tahb_set_peer_wait_limit_ns
    fn.restype = ctypes.c_ulonglong
    return int(fn(ctypes.c_ulonglong(int(ns))))


class _QkvEpilogue(ctypes.Structure):
    _fields_ = [("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("q_out", c_void_p), ("k_dense", c_void_p),
                ("v_dense", c_void_p), ("kv_cache", c_void_p * 4), ("cache_sel", c_void_p), ("slot", c_void_p),
                ("pos", c_void_p), ("rope_cs", c_void_p), ("n_caches", c_int), ("nq", c_int), ("nkv", c_int), ("page_size", c_int),
                ("eps", c_float), ("theta", c_float)]


def gemm_qkv(x: torch.Tensor, w: torch.Tensor, q_w, k_w, pos, nq: int, nkv: int, eps: float, theta: float, *,
             x2: Optional[torch.Tensor] = None, w2: Optional[torch.Tensor] = None, q_out=None, k_dense=None,
             v_dense=None, caches: Sequence[torch.Tensor] = (), cache_sel=None, slot=None, page_size: int = 16,
             tp_wait=None, splits: Optional[int] = None, bn: int = 0, rope_cs: Optional[torch.Tensor] = None):
    """QKV projection (``x @ w^T`` + LoRA K-extension) whose epilogue applies the per-head QK RMSNorm and RoPE and
    writes q to ``q_out`` and K / V into the paged cache slots (and / or ``k_dense`` / ``v_dense``): the fused form
    of :func:`gemm` followed by :func:`qk_norm_rope_kv`, for head_dim 128 (one 128-feature tile = one head)."""
    _check_bf16_2d(x, "x")
    _check_bf16_2d(w, "w")
    M, K = x.shape
    F = w.shape[0]
    if F != (nq + 2 * nkv) * 128:
        raise ValueError("gemm_qkv needs head_dim 128 and w of (nq + 2 nkv) * 128 rows")
    R = 0
    if x2 is not None:
        _check_bf16_2d(x2, "x2")
        _check_bf16_2d(w2, "w2")
        R = x2.shape[1]
    if q_out is None:
        q_out = torch.empty(M, nq * 128, dtype=torch.bfloat16, device=x.device)
    if splits is None and bn == 0:
        bn, splits = plan_gemm(M, F, K, R, False)
    elif splits is None:
        splits = 1
    e = _QkvEpilogue()
    e.q_norm_w, e.k_norm_w, e.q_out = q_w.data_ptr(), k_w.data_ptr(), q_out.data_ptr()
    e.k_dense = 0 if k_dense is None else k_dense.data_ptr()
    e.v_dense = 0 if v_dense is None else v_dense.data_ptr()
    for i in range(4):
        e.kv_cache[i] = caches[i].data_ptr() if i < len(caches) else 0
    e.cache_sel = 0 if cache_sel is None else cache_sel.data_ptr()
    e.slot = 0 if slot is None else slot.data_ptr()
    e.pos = pos.data_ptr()
    e.rope_cs = 0 if rope_cs is None else rope_cs.data_ptr()     # [M, 128] table from rope_table(), else computed in place
    e.n_caches, e.nq, e.nkv, e.page_size, e.eps, e.theta = len(caches), nq, nkv, page_size, eps, theta
    if tp_wait is not None:
        flags, targets = tp_wait
        wait = (_p(flags), _p(targets), c_int(flags.numel()))
    else:
        wait = (None, None, c_int(0))
    _rc(lib().tahb_gemm_qkv(_p(w), _p(x), _p(w2), _p(x2), c_int(M), c_int(F), c_int(K), c_int(R), c_ll(w.stride(0)),
                            c_ll(x.stride(0)), c_ll(w2.stride(0) if w2 is not None else 0),
                            c_ll(x2.stride(0) if x2 is not None else 0), c_int(splits), c_int(bn),
                            _p(status_word(x.device)), _stream(), *wait, ctypes.byref(e)), "tahb_gemm_qkv")
    return q_out


def _ptr_array(tensors: Sequence[Optional[torch.Tensor]]):
    arr = (c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = 0 if t is None else t.data_ptr()
    return arr


def qk_norm_rope_kv(qkv, q_w, k_w, pos, nq: int, nkv: int, hd: int, eps: float, theta: float, *,
                    q_out=None, k_dense=None, v_dense=None, caches: Sequence[torch.Tensor] = (),
                    cache_sel=None, slot=None, page_size: int = 16):
    """Per-head QK RMSNorm + RoPE on a fused ``[M, (nq+2nkv)*hd]`` projection; writes normed/rotated
    q to ``q_out``, K/V to ``k_dense``/``v_dense`` and/or into the paged cache(s) at ``slot``."""
    _check_bf16_2d(qkv, "qkv")
    M = qkv.shape[0]
    if q_out is None:
        q_out = torch.empty(M, nq * hd, dtype=torch.bfloat16, device=qkv.device)
    arr = _ptr_array(list(caches)) if caches else (c_void_p * 1)()
    _rc(lib().tahb_qk_norm_rope_kv(_p(qkv), _p(q_w), _p(k_w), _p(q_out), _p(k_dense), _p(v_dense), arr,
                                   c_int(len(caches)), _p(cache_sel), _p(slot), _p(pos), c_int(M), c_int(nq),
                                   c_int(nkv), c_int(hd), c_int(page_size), c_ll(qkv.stride(0)), c_float(eps),
                                   c_float(theta), _stream()), "tahb_qk_norm_rope_kv")
    return q_out


def rms_norm_bwd(x: torch.Tensor, w: torch.Tensor, gy: torch.Tensor, eps: float, want_gw: bool = True):
    """Backward of :func:`rms_norm` on contiguous ``[M, H]`` bf16 tensors: returns ``(gx, gw_fp32 or None)``."""
    M, H = x.shape
    gx = torch.empty_like(x)
    gw = torch.zeros(H, dtype=torch.float32, device=x.device) if want_gw else None
    _rc(lib().tahb_rmsnorm_bwd(_p(x), _p(w), _p(gy), _p(gx), _p(gw), c_int(M), c_int(H), c_float(eps), _stream()),
        "tahb_rmsnorm_bwd")
    return gx, gw


def swiglu_bwd(gate_up: torch.Tensor, gy: torch.Tensor) -> torch.Tensor:
    """Backward of :func:`swiglu`: ``gate_up`` ``[M, 2I]``, ``gy`` ``[M, I]`` (contiguous bf16) -> ``[M, 2I]``."""
    M, I2 = gate_up.shape
    out = torch.empty_like(gate_up)
    _rc(lib().tahb_swiglu_bwd(_p(gate_up), _p(gy), _p(out), c_ll(M), c_int(I2 // 2), _stream()), "tahb_swiglu_bwd")
    return out


def qk_norm_rope_bwd(qkv, q_w, k_w, gq, gk, gv, pos, nq: int, nkv: int, hd: int, eps: float, theta: float):
    """Backward of :func:`qk_norm_rope_kv` (dense outputs): returns ``(gqkv, gq_w_fp32, gk_w_fp32)``."""
    M = qkv.shape[0]
    gqkv = torch.empty_like(qkv)
    gqw = torch.zeros(hd, dtype=torch.float32, device=qkv.device)
    gkw = torch.zeros(hd, dtype=torch.float32, device=qkv.device)
    _rc(lib().tahb_qk_norm_rope_bwd(_p(qkv), _p(q_w), _p(k_w), _p(gq), _p(gk), _p(gv), _p(gqkv), _p(gqw), _p(gkw),
                                    _p(pos), c_int(M), c_int(nq), c_int(nkv), c_int(hd), c_float(eps), c_float(theta),
                                    _stream()), "tahb_qk_norm_rope_bwd")
    return gqkv, gqw, gkw


def embed_gather(E, tok, out=None):
    M, H = tok.shape[0], E.shape[1]
    if out is None:
        out = torch.empty(M, H, dtype=E.dtype, device=E.device)
    _rc(lib().tahb_embed_gather(_p(E), _p(tok), _p(out), c_int(M), c_int(H), c_ll(out.stride(0)), _stream()),
        "tahb_embed_gather")
    return out


def lora_a_rows(x, A, gate=None, out=None, tp_wait=None):
    """``out[r] = gate[r] ? x[r] @ A^T : 0`` for the few gated rows of a decode tick.  ``tp_wait =
    (flags, targets)``: gated rows first wait for the tensor-parallel broadcast of ``x``."""
    _check_bf16_2d(x, "x")
    M, K = x.shape
    R = A.shape[0]
    if out is None:
        out = torch.empty(M, R, dtype=torch.bfloat16, device=x.device)
    if tp_wait is None:
        _rc(lib().tahb_lora_a_rows(_p(x), _p(A), _p(out), _p(gate), c_int(M), c_int(K), c_int(R), c_ll(x.stride(0)),
                                   c_ll(out.stride(0)), _stream()), "tahb_lora_a_rows")
    else:
        flags, targets = tp_wait
        _rc(lib().tahb_lora_a_rows_tp(_p(x), _p(A), _p(out), _p(gate), c_int(M), c_int(K), c_int(R),
                                      c_ll(x.stride(0)), c_ll(out.stride(0)), _p(flags), _p(targets),
                                      c_int(flags.numel()), _p(status_word(x.device)), _stream()), "tahb_lora_a_rows_tp")
    return out


def swiglu(gate_up, out=None):
    _check_bf16_2d(gate_up, "gate_up")
    M, I2 = gate_up.shape
    if out is None:
        out = torch.empty(M, I2 // 2, dtype=torch.bfloat16, device=gate_up.device)
    _rc(lib().tahb_swiglu(_p(gate_up), _p(out), c_int(M), c_int(I2 // 2), c_ll(gate_up.stride(0)),
                          c_ll(out.stride(0)), _stream()), "tahb_swiglu")
    return out


def logits_post(logits, cum, depth, best, best_val=None):
    _rc(lib().tahb_logits_post(_p(logits), _p(cum), _p(depth), _p(best), _p(best_val), c_int(logits.shape[0]),
                               c_int(logits.shape[1]), c_ll(logits.stride(0)), c_ll(cum.stride(0)), _stream()),
        "tahb_logits_post")
    return best


# -------------------------------------------------------------------------------------------
# attention
# -------------------------------------------------------------------------------------------
def decode_attn(q, caches: Sequence[torch.Tensor], page_tables: Sequence[torch.Tensor], lens: Sequence[torch.Tensor],
                depth, nq: int, nkv: int, hd: int, page_size: int, scale: float, out=None, n_split: int = 1,
                ws: Optional[torch.Tensor] = None):
    rows = q.shape[0]
    if out is None:
        out = torch.empty_like(q)
    n = len(caches)
    mp = (c_int * n)(*[pt.shape[1] for pt in page_tables])
    if n_split > 1 and ws is None:
        ws = torch.empty(int(lib().tahb_decode_attn_ws_floats(rows, nq, hd, n_split)), dtype=torch.float32, device=q.device)
    _rc(lib().tahb_decode_attn(_p(q), _p(out), _ptr_array(caches), _ptr_array(page_tables), _ptr_array(lens), mp,
                               c_int(n), _p(depth), c_int(rows), c_int(nq), c_int(nkv), c_int(hd), c_int(page_size),
                               c_float(scale), c_int(n_split), _p(ws), _p(status_word(q.device)), _stream()), "tahb_decode_attn")
    return out


def varlen_attn_naive(q, ks, vs, bases, counts, nq, nkv, hd, scale, out=None):
    """Packed duo-causal attention: query i attends rows ``bases[s][i] + j, j < counts[s][i]`` of the
    packed ``ks[s]``/``vs[s]`` for each of up to three segments ``s``."""
    if out is None:
        out = torch.empty_like(q)
    n = len(ks)
    _rc(lib().tahb_varlen_attn_naive(_p(q), _p(out), _ptr_array(ks), _ptr_array(vs), _ptr_array(bases),
                                     _ptr_array(counts), c_int(n), c_int(q.shape[0]), c_int(nq), c_int(nkv),
                                     c_int(hd), c_float(scale), _stream()), "tahb_varlen_attn_naive")
    return out


def attn_tiles(seq_counts: torch.Tensor, tile: int = 128):
    """Query tiles for :func:`prefill_attn`: every sequence's packed tokens (``seq_counts[b]`` of
    them, sequences laid out back to back) are cut into runs of at most ``tile`` tokens.  Returns
    int32 ``(tile_q0, tile_qn)``."""
    cnt = seq_counts.to(torch.int64)
    per = (cnt + tile - 1) // tile
    n_tiles = int(per.sum())
    dev = cnt.device
    seq_of = torch.repeat_interleave(torch.arange(cnt.numel(), device=dev), per, output_size=n_tiles)
    rank = torch.arange(n_tiles, device=dev) - (torch.cumsum(per, 0) - per)[seq_of]
    q0 = (torch.cumsum(cnt, 0) - cnt)[seq_of] + tile * rank
    qn = torch.clamp(cnt[seq_of] - tile * rank, max=tile)
    return q0.to(torch.int32).contiguous(), qn.to(torch.int32).contiguous()


def prefill_attn(q, ks, vs, bases, counts, tile_q0, tile_qn, nq, nkv, hd, scale, out=None, lse=None, bounds=None):
    """Packed duo-causal attention on the tensor cores (``csrc/attn_prefill.cu``).  The reference builds a
    dense additive mask ``(kv_pos <= q_pos) & (kv_iter <= q_iter) & kv_valid`` per pass (reference
    ``tah/model/tah_model.py:744-791``) and hands it to SDPA; here the same rule is the per-query prefix
    ``bases[s] .. bases[s] + counts[s]`` of every depth's K/V and no mask tensor exists.  Same contract as
    :func:`varlen_attn_naive` plus the query tiling of :func:`attn_tiles`: the tokens of a tile belong
    to one sequence and share ``bases[s]``.  ``counts[s]`` must be non-decreasing along a sequence's rows, or
    ``bounds[s]`` must give such a non-decreasing upper bound (rows whose count was zeroed, e.g. padding).  ``lse`` (optional fp32
    ``[n_q, nq]``) receives the base-2 log-sum-exp of the scaled scores, which the backward kernels take."""
    if out is None:
        out = torch.empty_like(q)
    n = len(ks)
    for t in (q, out, *ks, *vs):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError("prefill_attn wants contiguous bf16 tensors")
    n_kv = (c_ll * n)(*[k.shape[0] for k in ks])
    _rc(lib().tahb_prefill_attn(_p(q), _p(out), _ptr_array(ks), _ptr_array(vs), n_kv, _ptr_array(bases),
                                _ptr_array(counts), _ptr_array(bounds if bounds is not None else counts), c_int(n), _p(tile_q0), _p(tile_qn), c_int(tile_q0.numel()),
                                c_ll(q.shape[0]), c_int(nq), c_int(nkv), c_int(hd), c_float(scale), _p(lse),
                                _p(status_word(q.device)), _stream()), "tahb_prefill_attn")
    return out


def attn_kv_items(seq_kv_counts: torch.Tensor, seq_kv_base: torch.Tensor, seq_q_counts: torch.Tensor, block: int = 128):
    """Work items of :func:`attn_bwd_dkv` for one KV segment: every sequence's ``seq_kv_counts[b]`` keys
    (stored from row ``seq_kv_base[b]`` of the segment's K/V matrices) are cut into blocks of ``block``.
    Returns int32 ``(row0, nkeys, kidx0, qa, qb)``; ``qa:qb`` are the sequence's packed query rows
    (sequences laid out back to back, ``seq_q_counts[b]`` rows each)."""
    cnt = seq_kv_counts.to(torch.int64)
    per = (cnt + block - 1) // block
    n = int(per.sum())
    dev = cnt.device
    seq_of = torch.repeat_interleave(torch.arange(cnt.numel(), device=dev), per, output_size=n)
    rank = torch.arange(n, device=dev) - (torch.cumsum(per, 0) - per)[seq_of]
    kidx0 = block * rank
    row0 = seq_kv_base.to(torch.int64)[seq_of] + kidx0
    nkeys = torch.clamp(cnt[seq_of] - kidx0, max=block)
    qc = seq_q_counts.to(torch.int64)
    qstart = torch.cumsum(qc, 0) - qc
    qa = qstart[seq_of]
    qb = qa + qc[seq_of]
    i32 = lambda t: t.to(torch.int32).contiguous()
    return i32(row0), i32(nkeys), i32(kidx0), i32(qa), i32(qb)


def attn_bwd_dq(q, dout, ks, vs, bases, counts, tile_q0, tile_qn, nq, nkv, hd, scale, lse, dsum, out=None,
                bounds=None):
    """dQ of :func:`prefill_attn` (``csrc/attn_prefill_bwd.cu``); ``dsum = rowsum(dO * O)`` per (query, head)."""
    if out is None:
        out = torch.empty_like(q)
    n = len(ks)
    n_kv = (c_ll * n)(*[k.shape[0] for k in ks])
    _rc(lib().tahb_attn_bwd_dq(_p(q), _p(dout), _p(out), _ptr_array(ks), _ptr_array(vs), n_kv, _ptr_array(bases),
                               _ptr_array(counts), _ptr_array(bounds if bounds is not None else counts), c_int(n), _p(tile_q0), _p(tile_qn), c_int(tile_q0.numel()),
                               c_ll(q.shape[0]), c_int(nq), c_int(nkv), c_int(hd), c_float(scale), _p(lse), _p(dsum),
                               _p(status_word(q.device)), _stream()), "tahb_attn_bwd_dq")
    return out


def attn_bwd_dkv(q, dout, k, v, count, items, nq, nkv, hd, scale, lse, dsum, dk=None, dv=None, bound=None):
    """dK, dV of one KV segment of :func:`prefill_attn`; ``items`` from :func:`attn_kv_items`, ``count`` the
    segment's visible-key counts per packed query.  Keys outside every item keep a zero gradient."""
    if dk is None:
        dk = torch.zeros_like(k)
    if dv is None:
        dv = torch.zeros_like(v)
    row0, nkeys, kidx0, qa, qb = items
    _rc(lib().tahb_attn_bwd_dkv(_p(q), _p(dout), _p(k), _p(v), _p(dk), _p(dv), c_ll(k.shape[0]), _p(count),
                                _p(bound if bound is not None else count), _p(row0),
                                _p(nkeys), _p(kidx0), _p(qa), _p(qb), c_int(row0.numel()), c_ll(q.shape[0]),
                                c_int(nq), c_int(nkv), c_int(hd), c_float(scale), _p(lse), _p(dsum),
                                _p(status_word(q.device)), _stream()), "tahb_attn_bwd_dkv")
    return dk, dv


# -------------------------------------------------------------------------------------------
# losses
# -------------------------------------------------------------------------------------------
def ce_fwd(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
    """Per-row cross entropy of bf16 ``logits [rows, V]`` in fp32 without an fp32 copy: returns ``(loss, lse)``."""
    _check_bf16_2d(logits, "logits")
    rows, V = logits.shape
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    _rc(lib().tahb_ce_fwd(_p(logits), _p(labels), _p(loss), _p(lse), c_int(rows), c_int(V), c_ll(logits.stride(0)),
                          c_int(ignore_index), _stream()), "tahb_ce_fwd")
    return loss, lse


def ce_bwd(logits: torch.Tensor, labels: torch.Tensor, lse: torch.Tensor, gscale: torch.Tensor, ignore_index: int = -100):
    """``dlogits = (softmax(logits) - onehot(labels)) * gscale[0]`` in bf16 (zero rows where the label is ignored)."""
    rows, V = logits.shape
    d = torch.empty(rows, V, dtype=torch.bfloat16, device=logits.device)
    _rc(lib().tahb_ce_bwd(_p(logits), _p(labels), _p(lse), _p(gscale), _p(d), c_int(rows), c_int(V),
                          c_ll(logits.stride(0)), c_ll(d.stride(0)), c_int(ignore_index), _stream()), "tahb_ce_bwd")
    return d


def soft_embed_bwd(dout: torch.Tensor, val: torch.Tensor, idx: torch.Tensor, E: torch.Tensor, dE: torch.Tensor):
    """Backward of :func:`soft_embed_rows`: returns ``dval [rows, K]`` (fp32) and adds ``p_k * dout`` into the fp32
    accumulator ``dE [V, H]`` at the rows ``idx``."""
    rows, Kk = val.shape
    dval = torch.empty(rows, Kk, dtype=torch.float32, device=val.device)
    _rc(lib().tahb_soft_embed_bwd(_p(dout), _p(val), _p(idx), _p(E), _p(dval), _p(dE), c_int(rows), c_int(Kk),
                                  c_int(E.shape[1]), c_ll(dout.stride(0)), _stream()), "tahb_soft_embed_bwd")
    return dval


def bce_logits(z: torch.Tensor, labels: torch.Tensor, depth: int, pos_weight: float, thr: float, g=None):
    """Forward (``g`` None): fp32 ``[3]`` = (sum of BCE terms over labelled tokens, their count, correct threshold
    decisions).  Backward (``g`` = upstream gradient scalar tensor): ``dz``."""
    n = z.shape[0]
    if g is None:
        out = torch.zeros(3, dtype=torch.float32, device=z.device)
        _rc(lib().tahb_bce_logits(_p(z), _p(labels), c_int(depth), c_float(pos_weight), c_float(thr), c_int(n), _p(out),
                                  None, None, _stream()), "tahb_bce_logits")
        return out
    dz = torch.empty(n, dtype=torch.float32, device=z.device)
    _rc(lib().tahb_bce_logits(_p(z), _p(labels), c_int(depth), c_float(pos_weight), c_float(thr), c_int(n), None, _p(g),
                              _p(dz), _stream()), "tahb_bce_logits")
    return dz


# -------------------------------------------------------------------------------------------
# sampling / control
# -------------------------------------------------------------------------------------------
def topk_rows(x, k: int, flag=None, out_val=None, out_idx=None, ordered: bool = False):
    """Sorted top-``k`` (value desc, index asc) of every flagged bf16 row.  ``ordered=True`` forces
    the kernel's slower index-ordered path (its fallback for rows with > 1024 near-threshold ties)."""
    rows, V = x.shape
    if out_val is None:
        out_val = torch.zeros(rows, k, dtype=torch.float32, device=x.device)
    if out_idx is None:
        out_idx = torch.zeros(rows, k, dtype=torch.int32, device=x.device)
    fn = lib().tahb_topk_rows_ordered if ordered else lib().tahb_topk_rows
    _rc(fn(_p(x), _p(flag), _p(out_val), _p(out_idx), c_int(rows), c_int(V), c_int(k), c_ll(x.stride(0)), _stream()),
        "tahb_topk_rows")
    return out_val, out_idx


def soft_embed_rows(val, idx, E, flag=None, out=None):
    rows, K = val.shape
    H = E.shape[1]
    if out is None:
        out = torch.zeros(rows, H, dtype=E.dtype, device=E.device)
    _rc(lib().tahb_soft_embed_rows(_p(val), _p(idx), _p(flag), _p(E), _p(out), c_int(rows), c_int(K), c_int(H),
                                   c_ll(out.stride(0)), _stream()), "tahb_soft_embed_rows")
    return out


def sample_topk(val, idx, temperature: float, top_p: float, min_p: float, seed: int, step=None, out=None,
                seed_dev: Optional[torch.Tensor] = None):
    """Draw one token per row from a sorted top-k set.  ``seed_dev`` (optional int64 device scalar) is mixed
    into the seed on the device, so a captured launch can be replayed with a fresh seed."""
    rows, K = val.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=val.device)
    _rc(lib().tahb_sample_topk(_p(val), _p(idx), _p(out), c_int(rows), c_int(K), c_float(temperature), c_float(top_p),
                               c_float(min_p), ctypes.c_ulonglong(seed & (2 ** 64 - 1)), _p(seed_dev), _p(step),
                               _stream()),
        "tahb_sample_topk")
    return out


def sample_full(x, temperature: float, top_k: int, top_p: float, min_p: float, seed: int, step=None, out=None,
                seed_dev: Optional[torch.Tensor] = None):
    """Draw one token per row of bf16 logits ``x [rows, V]`` over the whole vocabulary (temperature ->
    softmax -> min_p -> top_k -> top_p -> draw, reference ``tah/model/utils.py:84-125``); ``top_k <= 0``
    means no top-k filter.  Used where the sorted top-k route (``top_k <= 128``) does not apply."""
    _check_bf16_2d(x, "x")
    rows, V = x.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=x.device)
    _rc(lib().tahb_sample_full(_p(x), _p(out), c_int(rows), c_int(V), c_ll(x.stride(0)), c_float(temperature),
                               c_int(top_k), c_float(top_p), c_float(min_p), ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
                               _p(seed_dev), _p(step), _stream()), "tahb_sample_full")
    return out


def decider_head(h, w2, b2, out=None):
    """``z[r] = bf16(sum_j bf16(silu(h[r, j])) * w2[j] + b2)`` as fp32: the output layer of the two-layer
    decider MLP on the first layer's bf16 activations ``h`` (``[rows, inner]``)."""
    rows, inner = h.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.float32, device=h.device)
    _rc(lib().tahb_decider_head(_p(h), _p(w2), _p(b2), _p(out), c_int(rows), c_int(inner), c_ll(h.stride(0)),
                                _stream()), "tahb_decider_head")
    return out


def decide(z, threshold: float, override, pos, depth, max_iter: int, need_soft):
    rows = need_soft.shape[0]
    _rc(lib().tahb_decide(_p(z), c_float(threshold), _p(override), c_int(override.shape[1] if override is not None else 0),
                          _p(pos), _p(depth), c_int(max_iter), _p(need_soft), c_int(rows), _stream()), "tahb_decide")
    return need_soft


def fused_reduce_residual_norm(partial_ptrs, xout_ptrs, mc_partial: int, mc_xout: int, h, ln_w, flag_ptrs, epoch,
                               M: int, H: int, rank: int, world: int, eps: float, add_residual: bool, grid: int):
    """Row-parallel epilogue over NVLink: all-reduce of the ranks' partial [M, H] results + residual
    add + RMSNorm + broadcast of the normalised rows, one launch per rank (see csrc/comm.cu)."""
    n = len(partial_ptrs)
    arr = lambda ptrs: (c_void_p * n)(*ptrs)
    _rc(lib().tahb_fused_reduce_residual_norm(arr(partial_ptrs), arr(xout_ptrs), c_void_p(mc_partial),
                                              c_void_p(mc_xout), _p(h), _p(ln_w), arr(flag_ptrs), _p(epoch),
                                              _p(status_word(h.device)), c_int(M), c_int(H), c_int(rank),
                                              c_int(world), c_float(eps), c_int(1 if add_residual else 0),
                                              c_int(grid), _stream()), "tahb_fused_reduce_residual_norm")


def push_reduce_norm_bcast(slot, cnt, cnt_target, xout_ptrs, mc_xout: int, xflag_ptrs, xtarget, arrive, h, ln_w,
                           M: int, H: int, rank: int, world: int, rpr: int, eps: float, add_residual: bool,
                           final_wait: bool, grid: int, tap_ptrs=None, mc_tap: int = 0, tap_ld: int = 0):
    """Owner side of the push-based row-parallel epilogue: sum the slots that the peers' GEMMs
    filled, residual add, RMSNorm, broadcast, flag (see ``push_reduce_norm_bcast_kernel``).  ``tap_ptrs``:
    every rank's address of the tap column that also receives the updated residual rows (row pitch ``tap_ld``)."""
    n = len(xout_ptrs)
    arr = lambda ptrs: (c_void_p * n)(*ptrs)
    _rc(lib().tahb_push_reduce_norm_bcast(_p(slot), _p(cnt), _p(cnt_target), arr(xout_ptrs), c_void_p(mc_xout),
                                          arr(xflag_ptrs), _p(xtarget), _p(arrive), _p(h), _p(ln_w),
                                          _p(status_word(h.device)), c_int(M), c_int(H), c_int(rank), c_int(world),
                                          c_int(rpr), c_float(eps), c_int(1 if add_residual else 0),
                                          c_int(1 if final_wait else 0), c_int(grid), _stream(),
                                          arr(tap_ptrs) if tap_ptrs else None, c_void_p(mc_tap if tap_ptrs else 0),
                                          c_ll(tap_ld if tap_ptrs else 0)),
        "tahb_push_reduce_norm_bcast")


def tp_topk_merge(xval_ptrs, xidx_ptrs, arrive_ptrs, epoch, vals, idx, out_val, out_idx, buf_rows: int, k: int, rank: int,
                  world: int, vocab_lo: int):
    """Exchange sorted per-shard top-``k`` candidates with the peers of a tensor-parallel group through
    symmetric memory and merge them (``tp_topk_merge_kernel``).  ``buf_rows``: the row capacity the exchange
    buffers were laid out for."""
    n = len(xval_ptrs)
    arr = lambda ptrs: (c_void_p * n)(*ptrs)
    rows = vals.shape[0]
    if rows != buf_rows:
        raise ValueError("tp_topk_merge: the exchange buffers are laid out for a fixed number of rows")
    _rc(lib().tahb_tp_topk_merge(arr(xval_ptrs), arr(xidx_ptrs), arr(arrive_ptrs), _p(epoch), _p(vals), _p(idx),
                                 _p(out_val), _p(out_idx), _p(status_word(vals.device)), c_int(rows), c_int(k),
                                 c_int(vals.stride(0)), c_int(out_idx.stride(0)), c_int(rank), c_int(world),
                                 c_int(vocab_lo), _stream()), "tahb_tp_topk_merge")


def shard_gather_push(shard, dst_ptrs, mc_dst: int, landed_ptrs, ready_ptrs, target, state, rank: int, world: int,
                      grid: int):
    """Store this rank's parameter shard into every rank's gather buffer and advance the landing flags
    (``shard_gather_push_kernel`` in ``csrc/comm.cu``); the consumer is :func:`gemm` with ``tp_wait``."""
    n = len(dst_ptrs)
    arr = lambda ptrs: (c_void_p * n)(*ptrs)
    _rc(lib().tahb_shard_gather_push(_p(shard), arr(dst_ptrs), c_void_p(mc_dst), arr(landed_ptrs), arr(ready_ptrs),
                                     _p(target), _p(state), c_ll(shard.numel() * shard.element_size()), c_int(rank),
                                     c_int(world), c_int(grid), _p(status_word(shard.device)), _stream()),
        "tahb_shard_gather_push")


class TickStateBinding:
    """Packs the scheduler state tensors into the pointer/int arrays the tick kernels take."""

    def __init__(self, tensors: List[Optional[torch.Tensor]], ints: List[int]):
        assert len(tensors) == 28 and len(ints) == 10
        self._keep = tensors
        self.ptrs = _ptr_array(tensors)
        self.ints = (c_int * len(ints))(*ints)

    def tick_begin(self, E, soft, x_in, rope_cs=None, hd: int = 0, theta: float = 0.0):
        """``rope_cs`` (optional ``[rows, hd]`` bf16): also write the RoPE cos | sin row of every row's position."""
        _rc(lib().tahb_tick_begin(self.ptrs, self.ints, _p(E), _p(soft), _p(x_in), c_int(E.shape[1]), _p(rope_cs),
                                  c_int(hd), c_float(theta), _stream()), "tahb_tick_begin")

    def tick_end(self, need_soft, next_tok):
        _rc(lib().tahb_tick_end(self.ptrs, self.ints, _p(need_soft), _p(next_tok), _stream()), "tahb_tick_end")
