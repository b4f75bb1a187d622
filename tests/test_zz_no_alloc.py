"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need attention results: a
serving loop that lives inside another framework's fixed memory budget, a plug-in whose host
forbids cudaMalloc after start-up, or latency-critical code that cannot afford the device
synchronisation a cudaMalloc/cudaFree implies.  For them ``tahb_decode_attn_noalloc`` keeps the
split-KV scratch in a static device array inside the library.  This test checks that it returns
what the regular entry point (caller-allocated scratch) returns, on two calls in a row that share
the scratch, and that an oversized request is refused.  The file name makes pytest collect it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, rows, lens0, lens1, nq, nkv, hd, page=16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    def pool(lens):
        mp = (max(lens) + page - 1) // page + 1
        n_pages = rows * mp + 2
        cache = torch.randn(n_pages, 2, nkv, page, hd, generator=g, device="cuda").to(torch.bfloat16)
        pt = torch.randperm(n_pages, device="cuda", generator=g)[: rows * mp].view(rows, mp).to(torch.int32)
        return cache, pt, torch.tensor(lens, dtype=torch.int32, device="cuda")
    c0, p0, l0 = pool(lens0)
    c1, p1, l1 = pool(lens1)
    depth = (torch.rand(rows, generator=g, device="cuda") < 0.5).to(torch.int32)
    q = torch.randn(rows, nq * hd, generator=g, device="cuda").to(torch.bfloat16)
    return q, [c0, c1], [p0, p1], [l0, l1], depth


def _call_noalloc(lib, q, caches, pts, lens, depth, nq, nkv, hd, n_split, status):
    n = len(caches)
    arr = lambda ts: (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
    mp = (ctypes.c_int * n)(*[p.shape[1] for p in pts])
    out = torch.empty_like(q)
    fn = lib.tahb_decode_attn_noalloc            # the exported C symbol
    fn.restype = ctypes.c_int
    rc = fn(ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(out.data_ptr()), arr(caches), arr(pts), arr(lens), mp,
            ctypes.c_int(n), ctypes.c_void_p(depth.data_ptr()), ctypes.c_int(q.shape[0]), ctypes.c_int(nq),
            ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(16), ctypes.c_float(hd ** -0.5), ctypes.c_int(n_split),
            ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    from tah_b200.ops import cuda as K
    lib = K.lib()
    lib.tahb_decode_attn_noalloc_capacity.restype = ctypes.c_longlong
    cap = lib.tahb_decode_attn_noalloc_capacity()
    assert cap == 1 << 20
    status = K.status_word()
    nq, nkv, hd, n_split = 16, 8, 128, 3
    cases = [_case(1, 5, [1, 17, 130, 64, 333], [0, 3, 0, 20, 1], nq, nkv, hd),
             _case(2, 7, [40, 5, 260, 16, 33, 90, 2], [7, 0, 31, 0, 0, 16, 1], nq, nkv, hd)]
    for q, caches, pts, lens, depth in cases:          # second call reuses the scratch the first one dirtied
        ref = K.decode_attn(q, caches, pts, lens, depth, nq, nkv, hd, 16, hd ** -0.5, n_split=n_split)
        rc, out = _call_noalloc(lib, q, caches, pts, lens, depth, nq, nkv, hd, n_split, status)
        assert rc == 0
        torch.cuda.synchronize()
        K.check_status()
        torch.testing.assert_close(out.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_noalloc_rejects_requests_beyond_its_scratch():
    from tah_b200.ops import cuda as K
    lib = K.lib()
    status = K.status_word()
    nq, nkv, hd = 16, 8, 128
    rows = 4096                                         # 4096 * 16 * 2 * 130 floats > 2^20
    q, caches, pts, lens, depth = _case(3, 4, [4, 4, 4, 4], [0, 0, 0, 0], nq, nkv, hd)
    big_q = torch.zeros(rows, nq * hd, dtype=torch.bfloat16, device="cuda")
    fn = lib.tahb_decode_attn_noalloc
    fn.restype = ctypes.c_int
    n = 2
    arr = lambda ts: (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
    rc = fn(ctypes.c_void_p(big_q.data_ptr()), ctypes.c_void_p(big_q.data_ptr()), arr(caches), arr(pts), arr(lens),
            (ctypes.c_int * n)(*[p.shape[1] for p in pts]), ctypes.c_int(n), ctypes.c_void_p(0), ctypes.c_int(rows),
            ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(16), ctypes.c_float(hd ** -0.5),
            ctypes.c_int(2), ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(0))
    assert rc == -7                                     # refused before anything is launched
