"""Numerics of the hand-written sm_100a kernels against plain PyTorch fp32 statements of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cuda():
    from tah_b200.ops import cuda as K
    return K


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _close(out, ref, atol, rtol):
    torch.testing.assert_close(out.float(), ref.float(), atol=atol, rtol=rtol)


GEMM_SHAPES = [(64, 256, 256), (16, 128, 64), (1, 128, 128), (100, 384, 512), (256, 4096, 2048), (300, 2048, 6144),
               (64, 192, 2048), (130, 256, 320)]


@pytest.mark.parametrize("M,F,K,R", [(256, 4096, 2048, 192), (64, 2048, 6144, 64), (100, 512, 256, 0), (256, 2048, 1024, 64)])
@pytest.mark.parametrize("bn,splits", [(0, None), (128, 1), (128, 2), (64, 4)])
@pytest.mark.parametrize("residual", [False, True])
def test_gemm_forced_plans(M, F, K, R, bn, splits, residual):
    """Forced token-tile widths and split-K cluster sizes with LoRA K-extension and residual against fp32."""
    Kc = _cuda()
    x, w = _rand(M, K, seed=1), _rand(F, K, scale=K ** -0.5, seed=2)
    x2 = _rand(M, R, seed=3) if R else None
    w2 = _rand(F, R, scale=0.05, seed=4) if R else None
    res = _rand(M, F, seed=5) if residual else None
    kw = dict(bn=bn, splits=splits) if bn else {}
    out = Kc.gemm(x, w, x2=x2, w2=w2, residual=res, **kw)
    Kc.check_status()
    ref = x.float() @ w.float().t()
    if R:
        ref = ref + x2.float() @ w2.float().t()
    if residual:
        ref = ref.to(torch.bfloat16).float() + res.float()
    _close(out, ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("M,F,K", GEMM_SHAPES)
@pytest.mark.parametrize("splits", [1, None])
def test_gemm_plain(M, F, K, splits):
    Kc = _cuda()
    x, w = _rand(M, K, seed=1), _rand(F, K, scale=K ** -0.5, seed=2)
    out = Kc.gemm(x, w, splits=splits)
    Kc.check_status()
    _close(out, x.float() @ w.float().t(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M,F,K,R", [(64, 256, 256, 64), (48, 4096, 2048, 192), (256, 2048, 6144, 64), (7, 128, 64, 128), (256, 4096, 2048, 192), (128, 2048, 2048, 64)])
@pytest.mark.parametrize("splits", [1, None])
def test_gemm_lora_extension_and_residual(M, F, K, R, splits):
    Kc = _cuda()
    x, w = _rand(M, K, seed=1), _rand(F, K, scale=K ** -0.5, seed=2)
    t, b = _rand(M, R, seed=3), _rand(F, R, scale=R ** -0.5, seed=4)
    res = _rand(M, F, seed=5)
    out = Kc.gemm(x, w, x2=t, w2=b, residual=res, splits=splits)
    Kc.check_status()
    acc = x.float() @ w.float().t() + t.float() @ b.float().t()
    ref = res.float() + acc.to(torch.bfloat16).float()
    _close(out, ref, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("M,I,K", [(64, 768, 256), (16, 6144, 2048), (200, 1536, 512), (256, 6144, 2048), (130, 768, 2048)])
@pytest.mark.parametrize("splits", [1, None])
def test_gemm_swiglu(M, I, K, splits):
    Kc = _cuda()
    x, w = _rand(M, K, seed=1), _rand(2 * I, K, scale=K ** -0.5, seed=2)
    out = Kc.gemm(x, w, swiglu=True, splits=splits)
    Kc.check_status()
    gu = (x.float() @ w.float().t()).to(torch.bfloat16).float()
    ref = torch.nn.functional.silu(gu[:, :I]).to(torch.bfloat16).float() * gu[:, I:]
    _close(out, ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("M,I,K,R", [(64, 768, 256, 0), (16, 6144, 2048, 64), (200, 1536, 512, 64), (256, 6144, 2048, 64),
                                     (130, 1216, 2048, 0), (700, 768, 512, 64), (1, 128, 128, 0)])
def test_gemm_swiglu_interleaved(M, I, K, R):
    """SwiGLU on interleaved gate / up rows (one accumulator, partner value in the neighbouring TMEM lane) equals the
    stacked-layout reference, with and without the LoRA K-extension, for token counts on and off the tile sizes."""
    Kc = _cuda()
    x, w = _rand(M, K, seed=1), _rand(2 * I, K, scale=K ** -0.5, seed=2)
    x2 = _rand(M, R, seed=3) if R else None
    w2 = _rand(2 * I, R, scale=0.05, seed=4) if R else None
    out = Kc.gemm(x, Kc.interleave_gate_up(w), x2=x2, w2=None if w2 is None else Kc.interleave_gate_up(w2),
                  swiglu_interleaved=True)
    Kc.check_status()
    assert out.shape == (M, I)
    acc = x.float() @ w.float().t()
    if R:
        acc = acc + x2.float() @ w2.float().t()
    gu = acc.to(torch.bfloat16).float()
    ref = torch.nn.functional.silu(gu[:, :I]).to(torch.bfloat16).float() * gu[:, I:]
    _close(out, ref, atol=3e-2, rtol=3e-2)
    # same values as the two-accumulator form (unsplit: the same summation order over K)
    dual = Kc.gemm(x, w, x2=x2, w2=w2, swiglu=True, splits=1)
    assert torch.equal(out, dual)


@pytest.mark.parametrize("M,F,K,R", [(256, 4096, 2048, 64), (1000, 512, 256, 0), (2048, 2048, 1024, 64), (77, 256, 128, 0)])
@pytest.mark.parametrize("residual", [False, True])
def test_gemm_pair_mode(M, F, K, R, residual):
    """Two output tiles per CTA sharing a 256-token activation tile (the large-token-count form), with the LoRA
    K-extension and a residual, against fp32; bitwise equal to the one-tile form (same summation order)."""
    Kc = _cuda()
    x, w = _rand(M, K, seed=1), _rand(F, K, scale=K ** -0.5, seed=2)
    x2 = _rand(M, R, seed=3) if R else None
    w2 = _rand(F, R, scale=0.05, seed=4) if R else None
    res = _rand(M, F, seed=5) if residual else None
    out = Kc.gemm(x, w, x2=x2, w2=w2, residual=res, pair=True)
    Kc.check_status()
    ref = x.float() @ w.float().t()
    if R:
        ref = ref + x2.float() @ w2.float().t()
    if residual:
        ref = ref.to(torch.bfloat16).float() + res.float()
    _close(out, ref, atol=3e-2, rtol=3e-2)
    assert torch.equal(out, Kc.gemm(x, w, x2=x2, w2=w2, residual=res, pair=False, bn=256, splits=1))


@pytest.mark.parametrize("M,I,K,R", [(2048, 1536, 512, 64), (300, 768, 256, 0)])
def test_gemm_pair_mode_with_interleaved_swiglu(M, I, K, R):
    Kc = _cuda()
    x, w = _rand(M, K, seed=1), Kc.interleave_gate_up(_rand(2 * I, K, scale=K ** -0.5, seed=2))
    x2 = _rand(M, R, seed=3) if R else None
    w2 = Kc.interleave_gate_up(_rand(2 * I, R, scale=0.05, seed=4)) if R else None
    a = Kc.gemm(x, w, x2=x2, w2=w2, swiglu_interleaved=True, pair=True)
    b = Kc.gemm(x, w, x2=x2, w2=w2, swiglu_interleaved=True, pair=False)
    Kc.check_status()
    assert a.shape == (M, I) and torch.equal(a, b)


@pytest.mark.parametrize("T,F,K", [(2048, 1024, 512), (4096, 2048, 2048)])
def test_backward_gemms_pair_mode_equals_one_tile_form(T, F, K):
    """The transposed-operand GEMMs (data and weight gradient) in pair mode give the same bits as the one-tile form."""
    Kc = _cuda()
    x, w = _rand(T, K, seed=1), _rand(F, K, scale=K ** -0.5, seed=2)
    gy = _rand(T, F, seed=3, scale=F ** -0.5)
    assert torch.equal(Kc.gemm_t(gy, w, w_t=True, pair=True), Kc.gemm_t(gy, w, w_t=True, pair=False, bn=256, splits=1))
    assert torch.equal(Kc.gemm_t(gy, x, x_t=True, w_t=True, pair=True),
                       Kc.gemm_t(gy, x, x_t=True, w_t=True, pair=False, bn=256, splits=1))
    Kc.check_status()


def test_gemm_strided_views():
    Kc = _cuda()
    big = _rand(64, 1024, seed=7)
    x = big[:, 256:512]                     # row stride 1024, 512-byte offset (16-byte aligned)
    w = _rand(256, 256, scale=1 / 16, seed=8)
    out = Kc.gemm(x, w)
    Kc.check_status()
    _close(out, x.float() @ w.float().t(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M,H", [(5, 256), (64, 2048), (33, 2560), (3, 6144)])
def test_rmsnorm(M, H):
    Kc = _cuda()
    from tah_b200.ops import torch_ref
    x, w = _rand(M, H, seed=1), (_rand(H, seed=2).float() * 0.1 + 1).to(torch.bfloat16)
    _close(Kc.rms_norm(x, w, 1e-6), torch_ref.rms_norm(x, w, 1e-6), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("hd,nq,nkv", [(128, 16, 8), (64, 4, 2), (128, 32, 8)])
def test_qk_norm_rope_and_paged_write(hd, nq, nkv):
    Kc = _cuda()
    from tah_b200.models.qwen3 import apply_rope, rope_cos_sin
    from tah_b200.ops import torch_ref
    M, page = 37, 16
    qkv = _rand(M, (nq + 2 * nkv) * hd, seed=1)
    qw, kw = (_rand(hd, seed=2).float() * 0.1 + 1).bfloat16(), (_rand(hd, seed=3).float() * 0.1 + 1).bfloat16()
    pos = torch.randint(0, 5000, (M,), device="cuda", dtype=torch.int32)
    n_pages = 8
    cache = torch.zeros(n_pages, 2, nkv, page, hd, dtype=torch.bfloat16, device="cuda")
    slot = torch.randperm(n_pages * page, device="cuda")[:M].to(torch.int32)
    kd = torch.empty(M, nkv * hd, dtype=torch.bfloat16, device="cuda")
    vd = torch.empty_like(kd)
    q = Kc.qk_norm_rope_kv(qkv, qw, kw, pos, nq, nkv, hd, 1e-6, 1e6, k_dense=kd, v_dense=vd, caches=[cache],
                           slot=slot, page_size=page)
    qr, kr, vr = qkv.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
    cos, sin = rope_cos_sin(pos[None].long(), hd, 1e6, torch.bfloat16)
    q_ref = apply_rope(torch_ref.rms_norm(qr.view(1, M, nq, hd), qw, 1e-6), cos, sin)[0]
    k_ref = apply_rope(torch_ref.rms_norm(kr.view(1, M, nkv, hd), kw, 1e-6), cos, sin)[0]
    _close(q.view(M, nq, hd), q_ref, atol=3e-2, rtol=2e-2)
    _close(kd.view(M, nkv, hd), k_ref, atol=3e-2, rtol=2e-2)
    assert torch.equal(vd, vr.contiguous())
    pg, off = (slot // page).long(), (slot % page).long()
    assert torch.equal(cache[pg, 0, :, off], kd.view(M, nkv, hd))
    assert torch.equal(cache[pg, 1, :, off], vd.view(M, nkv, hd))


@pytest.mark.parametrize("M,nq,nkv,R,bn,splits", [(37, 16, 8, 0, 0, None), (256, 16, 8, 192, 0, None), (300, 4, 2, 64, 128, 2),
                                                   (256, 2, 1, 64, 128, 1), (200, 16, 8, 0, 256, 4), (16, 4, 4, 64, 16, 1)])
def test_gemm_qkv_fused_epilogue_equals_gemm_then_qk_norm_rope(M, nq, nkv, R, bn, splits):
    """QKV GEMM with the QK-norm / RoPE / KV-write epilogue == plain GEMM followed by the separate kernel
    (bit for bit: both round the projection to bf16 first), and both match the fp32 statement."""
    Kc = _cuda()
    from tah_b200.models.qwen3 import apply_rope, rope_cos_sin
    from tah_b200.ops import torch_ref
    hd, K, page = 128, 512, 16
    F = (nq + 2 * nkv) * hd
    x, w = _rand(M, K, seed=1), _rand(F, K, scale=K ** -0.5, seed=2)
    x2 = _rand(M, R, seed=3) if R else None
    w2 = _rand(F, R, scale=0.05, seed=4) if R else None
    qw, kw = (_rand(hd, seed=5).float() * 0.1 + 1).bfloat16(), (_rand(hd, seed=6).float() * 0.1 + 1).bfloat16()
    pos = torch.randint(0, 5000, (M,), device="cuda", dtype=torch.int32)
    n_pages = (M + page - 1) // page + 2
    slot = torch.randperm(n_pages * page, device="cuda")[:M].to(torch.int32)
    slot[M // 2] = -1                                                   # a row that must not touch the cache
    sel = (torch.arange(M, device="cuda") % 2).to(torch.int32)
    outs = []
    for fused in (False, True, "table"):
        caches = [torch.zeros(n_pages, 2, nkv, page, hd, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        kd = torch.zeros(M, nkv * hd, dtype=torch.bfloat16, device="cuda")
        vd = torch.zeros_like(kd)
        if fused:
            table = Kc.rope_table(pos, hd, 1e6) if fused == "table" else None      # cos | sin computed once per pass
            q = Kc.gemm_qkv(x, w, qw, kw, pos, nq, nkv, 1e-6, 1e6, x2=x2, w2=w2, k_dense=kd, v_dense=vd, caches=caches,
                            cache_sel=sel, slot=slot, page_size=page, bn=bn, splits=splits, rope_cs=table)
        else:
            qkv = Kc.gemm(x, w, x2=x2, w2=w2, bn=bn, splits=splits)
            q = Kc.qk_norm_rope_kv(qkv, qw, kw, pos, nq, nkv, hd, 1e-6, 1e6, k_dense=kd, v_dense=vd, caches=caches,
                                   cache_sel=sel, slot=slot, page_size=page)
        Kc.check_status()
        outs.append((q, kd, vd, caches))
    (q0, k0, v0, c0), (q1, k1, v1, c1), (q2, k2, v2, c2) = outs
    assert torch.equal(q0, q1) and torch.equal(k0, k1) and torch.equal(v0, v1)
    assert torch.equal(c0[0], c1[0]) and torch.equal(c0[1], c1[1])
    assert torch.equal(q0, q2) and torch.equal(k0, k2) and torch.equal(c0[0], c2[0]) and torch.equal(c0[1], c2[1])
    assert float(c1[0].abs().sum()) > 0 and float(c1[1].abs().sum()) > 0
    ref = x.float() @ w.float().t() + (x2.float() @ w2.float().t() if R else 0)
    qr, kr, vr = ref.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
    cos, sin = rope_cos_sin(pos[None].long(), hd, 1e6, torch.float32)
    q_ref = apply_rope(torch_ref.rms_norm(qr.view(1, M, nq, hd), qw.float(), 1e-6), cos, sin)[0]
    _close(q1.view(M, nq, hd), q_ref, atol=6e-2, rtol=3e-2)
    _close(v1, vr, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("M,H,R", [(9, 2048, 192), (256, 2048, 128), (33, 1024, 72), (5, 2560, 64)])
def test_rmsnorm_lora_fused(M, H, R):
    """RMSNorm + gated LoRA-A in one launch against the two separate kernels and the fp32 statement."""
    Kc = _cuda()
    from tah_b200.ops import torch_ref
    x, w = _rand(M, H, seed=1), (_rand(H, seed=2).float() * 0.1 + 1).to(torch.bfloat16)
    A = _rand(R, H, scale=H ** -0.5, seed=3)
    gate = (torch.rand(M, device="cuda") < 0.3).to(torch.int32)
    gate[0] = 1
    t = torch.full((M, R + 8), 5.0, dtype=torch.bfloat16, device="cuda")
    y, _ = Kc.rms_norm_lora(x, w, 1e-6, gate, A, t_out=t[:, :R])
    y_ref = torch_ref.rms_norm(x, w, 1e-6)
    _close(y, y_ref, atol=1e-2, rtol=1e-2)
    assert torch.equal(Kc.lora_a_rows(y, A, gate), t[:, :R].contiguous())        # same bits as the separate kernel
    _close(t[:, :R], (y.float() @ A.float().t()) * gate[:, None], atol=2e-2, rtol=2e-2)
    assert (t[:, R:] == 5.0).all() and (t[gate == 0][:, :R] == 0).all()


@pytest.mark.parametrize("M,D", [(5, 512), (256, 512), (33, 256), (7, 2048)])
def test_layernorm_and_layernorm_dot(M, D):
    Kc = _cuda()
    x = _rand(M, D, seed=1, scale=2.0)
    w, b = (_rand(D, seed=2).float() * 0.2 + 1).bfloat16(), (_rand(D, seed=3).float() * 0.2).bfloat16()
    y = Kc.layer_norm(x, w, b, 1e-5)
    ref = torch.nn.functional.layer_norm(x.float(), (D,), w.float(), b.float(), 1e-5)
    _close(y, ref, atol=2e-2, rtol=2e-2)
    dw, db = _rand(D, seed=4, scale=D ** -0.5), _rand(1, seed=5)
    z = Kc.layer_norm_dot(x, w, b, dw, db, 1e-5)
    zref = ref.to(torch.bfloat16).float() @ dw.float() + db.float()
    _close(z, zref, atol=3e-2, rtol=3e-2)


def test_gemm_gelu_epilogue_and_bias_extension():
    """``gelu(x W^T + b)`` and ``res + (u W^T + b)``: the two GEMMs of a decider block."""
    Kc = _cuda()
    M, K, F = 200, 512, 2048
    x, w = _rand(M, K, seed=1), _rand(F, K, scale=K ** -0.5, seed=2)
    bias = _rand(F, seed=3, scale=0.3)
    ones = torch.zeros(M, 64, dtype=torch.bfloat16, device="cuda")
    ones[:, 0] = 1
    bext = torch.zeros(F, 64, dtype=torch.bfloat16, device="cuda")
    bext[:, 0] = bias
    y = Kc.gemm(x, w, x2=ones, w2=bext, gelu=True)
    ref = torch.nn.functional.gelu((x.float() @ w.float().t() + bias.float()).to(torch.bfloat16).float())
    _close(y, ref, atol=2e-2, rtol=2e-2)
    w2 = _rand(K, F, scale=F ** -0.5, seed=4)
    res = _rand(M, K, seed=5)
    out = res.clone()
    Kc.gemm(y, w2, residual=out, out=out)
    _close(out, res.float() + (y.float() @ w2.float().t()).to(torch.bfloat16).float(), atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("T,F,K", [(300, 512, 256), (8192, 2048, 2048), (1000, 4096, 2048), (77, 192, 2048), (130, 2048, 64)])
def test_backward_gemms_with_transposed_operands(T, F, K):
    """Data and weight gradients of ``y = x w^T`` on the tcgen05 GEMM reading its operands transposed in place
    (MN-major tiles), against fp32 matmuls; the weight gradient also in accumulate-into-grad form."""
    Kc = _cuda()
    from tah_b200.ops import autograd_ops as ao
    x, w = _rand(T, K, seed=1), _rand(F, K, scale=K ** -0.5, seed=2)
    gy = _rand(T, F, seed=3, scale=F ** -0.5)
    if K % 128 == 0:
        gx = Kc.gemm_t(gy, w, w_t=True)
        _close(gx, gy.float() @ w.float(), atol=3e-2, rtol=3e-2)
    gw = ao._wgrad(gy, x)
    ref = gy.float().t() @ x.float()
    assert gw.shape == (F, K)
    _close(gw, ref, atol=max(3e-2, 2e-2 * float(ref.abs().max())), rtol=3e-2)
    if K % 128 == 0:
        acc0 = _rand(F, K, seed=4, scale=0.1)
        acc = acc0.clone()
        Kc.gemm_t(gy, x, x_t=True, w_t=True, residual=acc, out=acc)
        _close(acc, acc0.float() + ref.to(torch.bfloat16).float(), atol=max(4e-2, 2e-2 * float(ref.abs().max())), rtol=3e-2)
    Kc.check_status()


def _paged_setup(rows, lens, nkv, hd, page, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    max_pages = (max(lens) + page - 1) // page + 1
    n_pages = rows * max_pages + 3
    cache = (torch.randn(n_pages, 2, nkv, page, hd, generator=g, device="cuda")).to(torch.bfloat16)
    perm = torch.randperm(n_pages, device="cuda", generator=g)[: rows * max_pages].view(rows, max_pages).to(torch.int32)
    return cache, perm, torch.tensor(lens, dtype=torch.int32, device="cuda")


def _gather_paged(cache, pt, n, page):
    ks, vs = [], []
    for i in range(n):
        pg = int(pt[i // page])
        ks.append(cache[pg, 0, :, i % page])
        vs.append(cache[pg, 1, :, i % page])
    return torch.stack(ks), torch.stack(vs)     # [n, nkv, hd]


@pytest.mark.parametrize("hd,nq,nkv", [(128, 16, 8), (64, 4, 2), (128, 32, 8)])
@pytest.mark.parametrize("n_split", [1, 3])
def test_decode_attention_two_caches(hd, nq, nkv, n_split):
    Kc = _cuda()
    rows, page = 5, 16
    lens0, lens1 = [1, 17, 130, 64, 333], [0, 3, 0, 20, 1]
    c0, pt0, l0 = _paged_setup(rows, lens0, nkv, hd, page, 1)
    c1, pt1, l1 = _paged_setup(rows, lens1, nkv, hd, page, 2)
    depth = torch.tensor([0, 1, 0, 1, 0], dtype=torch.int32, device="cuda")
    q = _rand(rows, nq * hd, seed=3)
    scale = hd ** -0.5
    out = Kc.decode_attn(q, [c0, c1], [pt0, pt1], [l0, l1], depth, nq, nkv, hd, page, scale, n_split=n_split)
    G = nq // nkv
    for r in range(rows):
        k, v = _gather_paged(c0, pt0[r], lens0[r], page)
        if int(depth[r]) >= 1 and lens1[r] > 0:
            k1, v1 = _gather_paged(c1, pt1[r], lens1[r], page)
            k, v = torch.cat([k, k1]), torch.cat([v, v1])
        qr = q[r].view(nq, hd).float()
        kf = k.float().repeat_interleave(G, dim=1)
        vf = v.float().repeat_interleave(G, dim=1)
        s = torch.einsum("hd,nhd->hn", qr, kf) * scale
        ref = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), vf)
        _close(out[r].view(nq, hd), ref, atol=2e-2, rtol=2e-2)


def test_varlen_attention_duo_segments():
    Kc = _cuda()
    nq, nkv, hd = 4, 2, 64
    seqlens = [9, 30, 1]
    n0 = sum(seqlens)
    starts = [0, 9, 39]
    k0, v0 = _rand(n0, nkv * hd, seed=1), _rand(n0, nkv * hd, seed=2)
    # depth-1 tokens: a subset of positions per sequence
    hard = [[2, 7], [0, 5, 29], []]
    q_list, b0, c0, b1, c1 = [], [], [], [], []
    n1 = sum(len(h) for h in hard)
    k1, v1 = _rand(n1, nkv * hd, seed=3), _rand(n1, nkv * hd, seed=4)
    off1 = 0
    for s, hs in enumerate(hard):
        for j, p in enumerate(hs):
            b0.append(starts[s]); c0.append(p + 1); b1.append(off1); c1.append(j + 1)
        off1 += len(hs)
    q = _rand(n1, nq * hd, seed=5)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    out = Kc.varlen_attn_naive(q, [k0, k1], [v0, v1], [i32(b0), i32(b1)], [i32(c0), i32(c1)], nq, nkv, hd, hd ** -0.5)
    G = nq // nkv
    for i in range(n1):
        k = torch.cat([k0[b0[i]:b0[i] + c0[i]], k1[b1[i]:b1[i] + c1[i]]]).view(-1, nkv, hd).float().repeat_interleave(G, 1)
        v = torch.cat([v0[b0[i]:b0[i] + c0[i]], v1[b1[i]:b1[i] + c1[i]]]).view(-1, nkv, hd).float().repeat_interleave(G, 1)
        s = torch.einsum("hd,nhd->hn", q[i].view(nq, hd).float(), k) * hd ** -0.5
        ref = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), v)
        _close(out[i].view(nq, hd), ref, atol=2e-2, rtol=2e-2)


def _ref_duo_attention(q, ks, vs, bases, counts, nq, nkv, hd):
    G = nq // nkv
    out = torch.zeros(q.shape[0], nq, hd, dtype=torch.float32, device=q.device)
    for i in range(q.shape[0]):
        kk = torch.cat([k[b[i]:b[i] + c[i]] for k, b, c in zip(ks, bases, counts)])
        vv = torch.cat([v[b[i]:b[i] + c[i]] for v, b, c in zip(vs, bases, counts)])
        kk = kk.view(-1, nkv, hd).float().repeat_interleave(G, 1)
        vv = vv.view(-1, nkv, hd).float().repeat_interleave(G, 1)
        s = torch.einsum("hd,nhd->hn", q[i].view(nq, hd).float(), kk) * hd ** -0.5
        out[i] = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), vv)
    return out


@pytest.mark.parametrize("hd,seqlens", [(64, [9, 30, 1]), (128, [200, 5, 131, 128]), (128, [300])])
def test_prefill_attention_tcgen05_causal(hd, seqlens):
    """Pass-0 packed causal attention on the tensor cores against an fp32 softmax reference."""
    Kc = _cuda()
    nq, nkv = 4, 2
    n0 = sum(seqlens)
    starts = [sum(seqlens[:i]) for i in range(len(seqlens))]
    q = _rand(n0, nq * hd, seed=11)
    k0, v0 = _rand(n0, nkv * hd, seed=12), _rand(n0, nkv * hd, seed=13)
    b0 = [starts[s] for s, L in enumerate(seqlens) for _ in range(L)]
    c0 = [j + 1 for L in seqlens for j in range(L)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    tq0, tqn = Kc.attn_tiles(torch.tensor(seqlens, device="cuda"))
    out = Kc.prefill_attn(q, [k0], [v0], [i32(b0)], [i32(c0)], tq0, tqn, nq, nkv, hd, hd ** -0.5)
    Kc.check_status()
    ref = _ref_duo_attention(q, [k0], [v0], [b0], [c0], nq, nkv, hd)
    _close(out.view(n0, nq, hd), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("hd", [64, 128])
def test_prefill_attention_tcgen05_duo_segments(hd):
    """Deeper pass: hard tokens attend all depth-0 keys up to their position plus the depth-1 keys
    of earlier hard tokens of the same sequence (two segments, several key blocks)."""
    Kc = _cuda()
    nq, nkv = 4, 2
    seqlens = [260, 40, 3]
    starts = [0, 260, 300]
    n0 = sum(seqlens)
    g = torch.Generator().manual_seed(5)
    hard = [sorted(torch.randperm(L, generator=g)[: max(1, (L * 3) // 5)].tolist()) for L in seqlens]
    k0, v0 = _rand(n0, nkv * hd, seed=1), _rand(n0, nkv * hd, seed=2)
    n1 = sum(len(h) for h in hard)
    k1, v1 = _rand(n1, nkv * hd, seed=3), _rand(n1, nkv * hd, seed=4)
    b0, c0, b1, c1 = [], [], [], []
    off1 = 0
    for s, hs in enumerate(hard):
        for j, p in enumerate(hs):
            b0.append(starts[s]); c0.append(p + 1); b1.append(off1); c1.append(j + 1)
        off1 += len(hs)
    q = _rand(n1, nq * hd, seed=5)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    tq0, tqn = Kc.attn_tiles(torch.tensor([len(h) for h in hard], device="cuda"))
    out = Kc.prefill_attn(q, [k0, k1], [v0, v1], [i32(b0), i32(b1)], [i32(c0), i32(c1)], tq0, tqn, nq, nkv, hd,
                          hd ** -0.5)
    Kc.check_status()
    ref = _ref_duo_attention(q, [k0, k1], [v0, v1], [b0, b1], [c0, c1], nq, nkv, hd)
    _close(out.view(n1, nq, hd), ref, atol=2e-2, rtol=2e-2)
    naive = Kc.varlen_attn_naive(q, [k0, k1], [v0, v1], [i32(b0), i32(b1)], [i32(c0), i32(c1)], nq, nkv, hd, hd ** -0.5)
    _close(out, naive.float(), atol=2e-2, rtol=2e-2)


def _ref_attention_autograd(q, ks, vs, bases, counts, nq, nkv, hd, dout):
    """fp32 masked-softmax attention with autograd: returns out, dq, [dk], [dv]."""
    G = nq // nkv
    qf = q.float().view(-1, nq, hd).requires_grad_(True)
    kf = [k.float().view(-1, nkv, hd).requires_grad_(True) for k in ks]
    vf = [v.float().view(-1, nkv, hd).requires_grad_(True) for v in vs]
    n = qf.shape[0]
    kk = torch.cat(kf).repeat_interleave(G, 1)
    vv = torch.cat(vf).repeat_interleave(G, 1)
    offs = [0]
    for k in kf:
        offs.append(offs[-1] + k.shape[0])
    mask = torch.zeros(n, kk.shape[0], dtype=torch.bool, device=q.device)
    for s, (b, c) in enumerate(zip(bases, counts)):
        idx = torch.arange(kf[s].shape[0], device=q.device)[None]
        b_t = torch.tensor(b, device=q.device)[:, None]
        c_t = torch.tensor(c, device=q.device)[:, None]
        mask[:, offs[s]:offs[s + 1]] = (idx >= b_t) & (idx < b_t + c_t)
    sc = torch.einsum("qhd,khd->hqk", qf, kk) * hd ** -0.5
    sc = sc.masked_fill(~mask[None], float("-inf"))
    out = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), vv)
    out.backward(dout.float().view(n, nq, hd))
    return out.detach(), qf.grad, [k.grad for k in kf], [v.grad for v in vf]


@pytest.mark.parametrize("hd", [64, 128])
def test_prefill_attention_backward_tcgen05(hd):
    """dQ / dK / dV kernels (two segments, several key blocks and query tiles, GQA) against fp32 autograd."""
    Kc = _cuda()
    nq, nkv = 4, 2
    seqlens = [300, 70, 5]
    starts = [0, 300, 370]
    n0 = sum(seqlens)
    g = torch.Generator().manual_seed(7)
    hard = [sorted(torch.randperm(L, generator=g)[: max(1, (L * 3) // 5)].tolist()) for L in seqlens]
    n1s = [len(h) for h in hard]
    n1 = sum(n1s)
    k0, v0 = _rand(n0, nkv * hd, seed=1), _rand(n0, nkv * hd, seed=2)
    k1, v1 = _rand(n1, nkv * hd, seed=3), _rand(n1, nkv * hd, seed=4)
    b0, c0, b1, c1 = [], [], [], []
    off1 = 0
    for s, hs in enumerate(hard):
        for j, p in enumerate(hs):
            b0.append(starts[s]); c0.append(p + 1); b1.append(off1); c1.append(j + 1)
        off1 += len(hs)
    q = _rand(n1, nq * hd, seed=5)
    dout = _rand(n1, nq * hd, seed=6)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    qcnt = torch.tensor(n1s, device="cuda")
    tq0, tqn = Kc.attn_tiles(qcnt)
    bases, counts = [i32(b0), i32(b1)], [i32(c0), i32(c1)]
    lse = torch.empty(n1, nq, dtype=torch.float32, device="cuda")
    out = Kc.prefill_attn(q, [k0, k1], [v0, v1], bases, counts, tq0, tqn, nq, nkv, hd, hd ** -0.5, lse=lse)
    ref_out, ref_dq, ref_dk, ref_dv = _ref_attention_autograd(q, [k0, k1], [v0, v1], [b0, b1], [c0, c1], nq, nkv, hd, dout)
    _close(out.view(n1, nq, hd), ref_out, atol=2e-2, rtol=2e-2)
    dsum = (dout.float() * out.float()).view(n1, nq, hd).sum(-1).contiguous()
    dq = Kc.attn_bwd_dq(q, dout, [k0, k1], [v0, v1], bases, counts, tq0, tqn, nq, nkv, hd, hd ** -0.5, lse, dsum)
    Kc.check_status()
    _close(dq.view(n1, nq, hd), ref_dq, atol=3e-2, rtol=3e-2)
    # segment 0: every sequence's depth-0 keys; segment 1: its depth-1 keys
    items0 = Kc.attn_kv_items(torch.tensor(seqlens, device="cuda"), torch.tensor(starts, device="cuda"), qcnt)
    start1 = [sum(n1s[:i]) for i in range(len(n1s))]
    items1 = Kc.attn_kv_items(qcnt, torch.tensor(start1, device="cuda"), qcnt)
    dk0, dv0 = Kc.attn_bwd_dkv(q, dout, k0, v0, counts[0], items0, nq, nkv, hd, hd ** -0.5, lse, dsum)
    dk1, dv1 = Kc.attn_bwd_dkv(q, dout, k1, v1, counts[1], items1, nq, nkv, hd, hd ** -0.5, lse, dsum)
    Kc.check_status()
    for got, ref in ((dk0, ref_dk[0]), (dv0, ref_dv[0]), (dk1, ref_dk[1]), (dv1, ref_dv[1])):
        _close(got.view(-1, nkv, hd), ref, atol=4e-2, rtol=4e-2)


@pytest.mark.parametrize("V,K", [(1024, 100), (151936, 100), (151936, 20), (5000, 1)])
def test_topk_rows_sorted(V, K):
    Kc = _cuda()
    x = _rand(6, V, scale=3.0, seed=V)
    flag = torch.tensor([1, 1, 0, 1, 1, 1], dtype=torch.int32, device="cuda")
    val, idx = Kc.topk_rows(x, K, flag=flag)
    ref_v, _ = torch.topk(x.float(), K, dim=-1)
    keep = flag.bool()
    assert torch.equal(val[keep], ref_v[keep])
    assert torch.equal(torch.gather(x.float(), 1, idx.long())[keep], ref_v[keep])
    assert (val[~keep] == 0).all()
    # ties at equal value are ordered by index
    same = val[keep][:, 1:] == val[keep][:, :-1]
    assert (idx[keep][:, 1:][same] > idx[keep][:, :-1][same]).all()
    # the index-ordered fallback path gives the identical result
    val2, idx2 = Kc.topk_rows(x, K, flag=flag, ordered=True)
    assert torch.equal(val2[keep], val[keep]) and torch.equal(idx2[keep], idx[keep])


def test_topk_rows_many_ties_takes_fallback():
    """A row with far more ties at the threshold than the candidate buffer holds: the kernel falls
    back to the index-ordered path and returns the lowest indices."""
    Kc = _cuda()
    V, K = 20000, 50
    x = torch.zeros(3, V, dtype=torch.bfloat16, device="cuda")
    x[1, 777] = 2.0
    x[2, ::2] = -1.0
    val, idx = Kc.topk_rows(x, K)
    assert torch.equal(idx[0].cpu(), torch.arange(K, dtype=torch.int32))
    assert idx[1, 0].item() == 777 and val[1, 0].item() == 2.0
    assert torch.equal(idx[1, 1:].cpu(), torch.arange(K - 1, dtype=torch.int32))
    assert torch.equal(idx[2].cpu(), torch.arange(1, 2 * K, 2, dtype=torch.int32))
    assert (val[2] == 0).all()


def test_soft_embed_and_logits_post():
    Kc = _cuda()
    from tah_b200.ops import torch_ref
    V, H, K, rows = 4096, 512, 100, 4
    E = _rand(V, H, seed=1)
    logits = _rand(rows, V, scale=4.0, seed=2)
    val, idx = Kc.topk_rows(logits, K)
    out = Kc.soft_embed_rows(val, idx, E)
    ref = torch_ref.topk_softmax_embed(logits, E, K)
    _close(out, ref, atol=2e-2, rtol=2e-2)
    cum = _rand(rows, V, seed=3)
    cum0 = cum.clone()
    depth = torch.tensor([0, 1, 0, 2], dtype=torch.int32, device="cuda")
    best = torch.zeros(rows, dtype=torch.int32, device="cuda")
    Kc.logits_post(logits, cum, depth, best)
    ref_cum = torch.where(depth[:, None] > 0, cum0 + logits, logits)
    assert torch.equal(cum, ref_cum)
    assert torch.equal(best.long(), ref_cum.float().argmax(-1))


def test_lora_a_rows_and_swiglu():
    Kc = _cuda()
    x, A = _rand(9, 2048, seed=1), _rand(192, 2048, scale=2048 ** -0.5, seed=2)
    gate = torch.tensor([0, 1, 0, 0, 1, 1, 0, 0, 1], dtype=torch.int32, device="cuda")
    t = Kc.lora_a_rows(x, A, gate)
    ref = (x.float() @ A.float().t()) * gate[:, None]
    _close(t, ref, atol=2e-2, rtol=2e-2)
    # more gated rows than compaction slots, a row count that is not a multiple of 4, dirty output
    x2 = _rand(203, 1024, seed=4)
    A2 = _rand(72, 1024, scale=1024 ** -0.5, seed=5)
    gate2 = (torch.rand(203, device="cuda") < 0.4).to(torch.int32)
    out2 = torch.full((203, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    Kc.lora_a_rows(x2, A2, gate2, out=out2[:, :72])
    _close(out2[:, :72], (x2.float() @ A2.float().t()) * gate2[:, None], atol=2e-2, rtol=2e-2)
    assert (out2[:, 72:] == 7.0).all()
    # no gate: every row (dense kernel)
    _close(Kc.lora_a_rows(x2, A2), x2.float() @ A2.float().t(), atol=2e-2, rtol=2e-2)
    gu = _rand(11, 2 * 768, seed=3)
    from tah_b200.ops import torch_ref
    _close(Kc.swiglu(gu), torch_ref.swiglu(gu), atol=1e-2, rtol=1e-2)


def test_rmsnorm_and_swiglu_backward_kernels():
    Kc = _cuda()
    M, H = 77, 2048
    x = _rand(M, H, seed=1).requires_grad_(True)
    w = (_rand(H, seed=2) * 0.1 + 1).to(torch.bfloat16).requires_grad_(True)
    gy = _rand(M, H, seed=3)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yf = wf * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6))
    yf.backward(gy.float())
    gx, gw = Kc.rms_norm_bwd(x.detach(), w.detach(), gy, 1e-6)
    _close(gx, xf.grad, atol=2e-2, rtol=2e-2)
    _close(gw, wf.grad, atol=5e-2, rtol=2e-2)
    gu = _rand(33, 2 * 768, seed=4)
    gy2 = _rand(33, 768, seed=5)
    guf = gu.float().requires_grad_(True)
    g, u = guf.chunk(2, -1)
    (torch.nn.functional.silu(g) * u).backward(gy2.float())
    _close(Kc.swiglu_bwd(gu, gy2), guf.grad, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("hd", [64, 128])
def test_qk_norm_rope_forward_backward(hd):
    """Fused QK-norm + RoPE autograd function against the module-level PyTorch statement in fp32."""
    from tah_b200.ops import autograd_ops
    from tah_b200.models.qwen3 import apply_rope, rope_cos_sin
    B, T, nq, nkv = 2, 37, 4, 2
    qkv = _rand(B, T, (nq + 2 * nkv) * hd, seed=1).requires_grad_(True)
    qw = (_rand(hd, seed=2) * 0.1 + 1).to(torch.bfloat16).requires_grad_(True)
    kw = (_rand(hd, seed=3) * 0.1 + 1).to(torch.bfloat16).requires_grad_(True)
    pos = torch.arange(T, device="cuda")[None].repeat(B, 1) + torch.tensor([[0], [5]], device="cuda")
    q, k, v = autograd_ops.qk_norm_rope(qkv, qw, kw, pos, nq, nkv, hd, 1e-6, 1e6)
    gq, gk, gv = _rand(B, T, nq, hd, seed=4), _rand(B, T, nkv, hd, seed=5), _rand(B, T, nkv, hd, seed=6)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    x = qkv.detach().float().requires_grad_(True)
    qwf, kwf = qw.detach().float().requires_grad_(True), kw.detach().float().requires_grad_(True)
    cos, sin = rope_cos_sin(pos, hd, 1e6, torch.float32)
    xq, xk, xv = x.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
    norm = lambda t, w: w * (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6))
    rq = apply_rope(norm(xq.view(B, T, nq, hd), qwf), cos, sin)
    rk = apply_rope(norm(xk.view(B, T, nkv, hd), kwf), cos, sin)
    rv = xv.reshape(B, T, nkv, hd)
    torch.autograd.backward([rq, rk, rv], [gq.float(), gk.float(), gv.float()])
    _close(q, rq, atol=3e-2, rtol=3e-2)
    _close(k, rk, atol=3e-2, rtol=3e-2)
    _close(qkv.grad, x.grad, atol=4e-2, rtol=4e-2)
    _close(qw.grad, qwf.grad, atol=0.3, rtol=5e-2)
    _close(kw.grad, kwf.grad, atol=0.3, rtol=5e-2)


def test_sampler_topk_distribution():
    Kc = _cuda()
    rows, K = 4096, 8
    val = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -2.0, -3.0, -9.0], device="cuda").repeat(rows, 1)
    idx = torch.arange(K, dtype=torch.int32, device="cuda").repeat(rows, 1) + 10
    step = torch.arange(rows, dtype=torch.int32, device="cuda")
    out = Kc.sample_topk(val, idx, temperature=0.7, top_p=0.9, min_p=0.0, seed=123, step=step)
    p = torch.softmax(val[0] / 0.7, -1)
    c = p.cumsum(0)
    n = int((c < 0.9).sum()) + 1
    expect = p[:n] / p[:n].sum()
    freq = torch.bincount(out.long() - 10, minlength=K).float() / rows
    assert (freq[n:] == 0).all()
    assert torch.allclose(freq[:n], expect, atol=0.03)


@pytest.mark.parametrize("top_k,top_p,min_p", [(0, 1.0, 0.0), (0, 0.9, 0.0), (5, 1.0, 0.0), (200, 0.8, 0.02), (0, 1.0, 0.05)])
def test_sampler_full_vocabulary_distribution(top_k, top_p, min_p):
    """Full-vocabulary sampler against the filtered distribution of the PyTorch statement of the same
    order (temperature -> softmax -> min_p -> top_k -> top_p)."""
    Kc = _cuda()
    rows, V, T = 8192, 1000, 0.8
    g = torch.Generator().manual_seed(1)
    base = (torch.randn(V, generator=g) * 2.0).to(torch.bfloat16)
    x = base.cuda().repeat(rows, 1).contiguous()
    step = torch.arange(rows, dtype=torch.int32, device="cuda")
    out = Kc.sample_full(x, T, top_k, top_p, min_p, seed=99, step=step)
    p = torch.softmax(base.float() / T, -1)
    if min_p > 0:
        p = torch.where(p >= min_p * p.max(), p, torch.zeros_like(p))
        p = p / p.sum()
    if top_k > 0:
        kth = torch.topk(p, min(top_k, V)).values[-1]
        p = torch.where(p < kth, torch.zeros_like(p), p)
        p = p / p.sum()
    if top_p < 1.0:
        sp, si = torch.sort(p, descending=True)
        drop = sp.cumsum(0) > top_p
        drop = torch.cat((torch.zeros(1, dtype=torch.bool), drop[:-1]))
        p[si[drop]] = 0
        p = p / p.sum()
    freq = torch.bincount(out.long().cpu(), minlength=V).float() / rows
    assert int(out.min()) >= 0 and int(out.max()) < V
    # nothing outside the kept set (ties at a threshold are kept by both statements)
    assert float(freq[p == 0].sum()) <= 1e-3
    assert float((freq - p).abs().max()) < 0.02
    # same seed and step -> same draw; another seed -> another sample
    again = Kc.sample_full(x, T, top_k, top_p, min_p, seed=99, step=step)
    other = Kc.sample_full(x, T, top_k, top_p, min_p, seed=100, step=step)
    assert torch.equal(out, again) and not torch.equal(out, other)


def test_sampler_device_seed_word_changes_the_draw():
    Kc = _cuda()
    rows, K = 512, 8
    val = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -2.0, -3.0, -9.0], device="cuda").repeat(rows, 1)
    idx = torch.arange(K, dtype=torch.int32, device="cuda").repeat(rows, 1)
    step = torch.arange(rows, dtype=torch.int32, device="cuda")
    word = torch.zeros(1, dtype=torch.int64, device="cuda")
    a = Kc.sample_topk(val, idx, 1.0, 1.0, 0.0, 0, step=step, seed_dev=word).clone()
    b = Kc.sample_topk(val, idx, 1.0, 1.0, 0.0, 0, step=step, seed_dev=word).clone()
    word.fill_(12345)
    c = Kc.sample_topk(val, idx, 1.0, 1.0, 0.0, 0, step=step, seed_dev=word)
    assert torch.equal(a, b) and not torch.equal(a, c)


def test_zero_adamw_cuda_single_gpu_matches_fp32_adamw():
    """Fused reduce + AdamW + broadcast kernels (world size 1) against torch.optim.AdamW on fp32 masters."""
    from tah_b200.parallel.zero import ZeroAdamW
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.Tanh(), torch.nn.Linear(96, 40)).cuda().bfloat16()
    ref = [p.detach().float().clone().requires_grad_(True) for p in net.parameters()]
    opt = ZeroAdamW(net.parameters(), lr=1e-2, weight_decay=0.01, max_grad_norm=0.7)
    ropt = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.01)
    K = _cuda()
    for step in range(3):
        x = _rand(32, 64, seed=step)
        loss = (net(x).float() ** 2).mean()
        loss.backward()
        grads = [p.grad.detach().float().clone() for p in net.parameters()]
        gn = opt.step()
        opt.zero_grad()
        K.check_status()
        for r, g in zip(ref, grads):
            r.grad = g
        rgn = torch.nn.utils.clip_grad_norm_(ref, 0.7)
        ropt.step()
        assert abs(float(gn) - float(rgn)) / float(rgn) < 1e-3
        # the bf16 parameters are the rounded fp32 masters; feed them back so both sides see the same forward
        off = 0
        for p, r in zip(net.parameters(), ref):
            k = p.numel()
            torch.testing.assert_close(opt.master[off:off + k].view_as(r), r.detach(), atol=2e-5, rtol=1e-4)
            torch.testing.assert_close(p.detach().float(), r.detach().to(torch.bfloat16).float(), atol=1e-2, rtol=1e-2)
            off += k


@pytest.mark.parametrize("pad", [False, True])
def test_training_step_on_gpu_matches_cpu_reference(pad):
    """bf16 model on the GPU (kernel forward, explicit backward) vs the same model in fp32 on the CPU;
    with ``pad`` the second sample is left-padded (padding queries and keys, ragged deeper pass)."""
    import copy
    from tests.helpers import tiny_tah
    model = tiny_tah(dtype=torch.bfloat16)
    ref = copy.deepcopy(model).float()
    model = model.cuda().train()
    ref.train()
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 1024, (2, 48), generator=g)
    hard = (torch.rand(2, 48, generator=g) < 0.1).long() + 1
    mask = torch.ones(2, 48, dtype=torch.long)
    labels = ids.clone()
    if pad:
        mask[1, :13] = 0
        labels[1, :13] = -100
    out = model(ids.cuda(), attention_mask=mask.cuda(), labels=labels.cuda(), iter_count_labels=hard.cuda())
    out.loss.backward()
    rout = ref(ids, attention_mask=mask, labels=labels, iter_count_labels=hard)
    rout.loss.backward()
    assert abs(float(out.loss.detach()) - float(rout.loss.detach())) < 0.05
    ga = model.simple_base_model.model.layers[0].self_attn.qkv_proj.weight.grad.float().cpu()
    gb = ref.simple_base_model.model.layers[0].self_attn.qkv_proj.weight.grad
    cos = torch.nn.functional.cosine_similarity(ga.flatten(), gb.flatten(), dim=0)
    assert float(cos) > 0.98


def test_training_step_kernel_path_matches_torch_path_multi_tile(monkeypatch):
    """Same bf16 model, same batch (300 tokens, one left-padded sample, ~30 % hard tokens): loss and
    gradients of the kernel path against the all-PyTorch path of this repository, both on the GPU."""
    import copy
    from tests.helpers import tiny_tah
    model = tiny_tah(dtype=torch.bfloat16).cuda().train()
    twin = copy.deepcopy(model)
    g = torch.Generator().manual_seed(0)
    B, T = 2, 300
    ids = torch.randint(0, 1024, (B, T), generator=g).cuda()
    hard = ((torch.rand(B, T, generator=g) < 0.3).long() + 1).cuda()
    mask = torch.ones(B, T, dtype=torch.long, device="cuda")
    labels = ids.clone()
    mask[1, :77] = 0
    labels[1, :77] = -100
    out = model(ids, attention_mask=mask, labels=labels, iter_count_labels=hard)
    out.loss.backward()
    monkeypatch.setenv("TAH_B200_FORCE_TORCH", "1")
    ref = twin(ids, attention_mask=mask, labels=labels, iter_count_labels=hard)
    ref.loss.backward()
    monkeypatch.delenv("TAH_B200_FORCE_TORCH")
    assert abs(float(out.loss.detach()) - float(ref.loss.detach())) < 0.03
    for name in ("layers.0.self_attn.qkv_proj.weight", "layers.3.mlp.down_proj.weight", "layers.1.self_attn.q_norm.weight"):
        ga = dict(model.simple_base_model.model.named_parameters())[name].grad.float().flatten()
        gb = dict(twin.simple_base_model.model.named_parameters())[name].grad.float().flatten()
        cos = torch.nn.functional.cosine_similarity(ga, gb, dim=0)
        assert float(cos) > 0.97, (name, float(cos))


def test_peer_flag_wait_runs_out_and_reports_a_timeout():
    """A consumer GEMM that waits for rows a peer would broadcast: nothing advances the landing flags, the wait
    limit is 5 ms, so the kernel gives up, records the timeout code and returns; the host reads the status word
    and raises.  Nothing traps or hangs, and the context stays usable."""
    import time
    Kc = _cuda()
    x, w = _rand(64, 256, seed=1), _rand(256, 256, scale=256 ** -0.5, seed=2)
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    targets = torch.ones(2, dtype=torch.int32, device="cuda")
    prev = Kc.set_peer_wait_limit_ns(5_000_000)
    try:
        torch.cuda.synchronize()
        t0 = time.time()
        Kc.gemm(x, w, tp_wait=(flags, targets))
        Kc.wait_flags(flags, targets)
        torch.cuda.synchronize()
        assert time.time() - t0 < 1.0                                   # two 5 ms limits, not the 2 s default
        with pytest.raises(Kc.KernelTimeout, match="peer flag"):
            Kc.check_status()
    finally:
        Kc.set_peer_wait_limit_ns(prev)
    Kc.check_status()                                                   # the status word was cleared
    flags.fill_(1)                                                      # the flags arrive: same launch succeeds
    y = Kc.gemm(x, w, tp_wait=(flags, targets))
    Kc.check_status()
    _close(y, x.float() @ w.float().t(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("rows,V", [(37, 151936), (300, 1024), (5, 1000)])
def test_fused_cross_entropy_forward_backward(rows, V):
    """CE kernel on bf16 logits (fp32 math, no fp32 copy) against ``F.cross_entropy`` on the upcast logits."""
    from tah_b200.ops import autograd_ops as ao
    g = torch.Generator(device="cuda").manual_seed(1)
    logits = (torch.randn(rows, V, generator=g, device="cuda") * 3).to(torch.bfloat16).requires_grad_(True)
    labels = torch.randint(0, V, (rows,), generator=g, device="cuda")
    labels[::5] = -100
    assert ao.cross_entropy_sum_ok(logits)
    loss = ao.cross_entropy_sum(logits, labels) / 7.0
    loss.backward()
    ref_in = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in, labels, ignore_index=-100, reduction="sum") / 7.0
    ref.backward()
    torch.testing.assert_close(loss.float(), ref, atol=1e-3, rtol=1e-4)
    _close(logits.grad, ref_in.grad, atol=2e-3, rtol=2e-2)
    assert float(logits.grad[::5].abs().max()) == 0.0


def test_fused_bce_with_logits_forward_backward():
    from tah_b200.ops import autograd_ops as ao
    g = torch.Generator(device="cuda").manual_seed(2)
    n = 5000
    z = (torch.randn(n, generator=g, device="cuda") * 2).requires_grad_(True)
    labels = torch.randint(1, 4, (n,), generator=g, device="cuda")
    labels[::7] = -100
    depth, pw, thr = 1, 5.4, 0.8
    s, cnt, correct = ao.bce_sum(z, labels, depth, pw, thr)
    (s / cnt).backward()
    zr = z.detach().clone().requires_grad_(True)
    w = (labels != -100).float()
    y = (labels > depth).float()
    per = torch.nn.functional.binary_cross_entropy_with_logits(zr, y, pos_weight=torch.tensor(pw, device="cuda"), reduction="none")
    ref = (per * w).sum() / w.sum()
    ref.backward()
    torch.testing.assert_close(s / cnt, ref, atol=1e-4, rtol=1e-4)
    assert float(cnt) == float(w.sum())
    assert float(correct) == float((((torch.sigmoid(zr) > thr).float() == y).float() * w).sum())
    torch.testing.assert_close(z.grad, zr.grad, atol=1e-6, rtol=1e-4)


def test_soft_embedding_mix_forward_backward_kernels():
    """Top-k soft input (values -> softmax -> mix of embedding rows) through the kernel pair against the fp32
    PyTorch statement, gradients to the logits and to the embedding rows included."""
    from tah_b200.ops import autograd_ops as ao
    g = torch.Generator(device="cuda").manual_seed(5)
    n, V, H, k = 50, 4096, 512, 100
    logits = (torch.randn(n, V, generator=g, device="cuda") * 2).to(torch.bfloat16).requires_grad_(True)
    E = (torch.randn(V, H, generator=g, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    gout = torch.randn(n, H, generator=g, device="cuda").to(torch.bfloat16)
    out = ao.topk_softmax_embed(logits, E, k)
    out.backward(gout)
    lf, Ef = logits.detach().float().requires_grad_(True), E.detach().float().requires_grad_(True)
    vals, idx = torch.topk(lf, k, dim=-1)
    ref = (torch.softmax(vals, -1).unsqueeze(-1) * Ef[idx]).sum(-2)
    ref.backward(gout.float())
    _close(out, ref, atol=3e-2, rtol=3e-2)
    _close(logits.grad, lf.grad, atol=3e-2, rtol=5e-2)
    _close(E.grad, Ef.grad, atol=3e-2, rtol=5e-2)
