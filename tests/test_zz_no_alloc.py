"""The allocation-free split-K GEMM entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need a GEMM (the KV pool already owns the
whole GPU, or they are a bare C host without an allocator); ``cb_wq_gemm_splitk_noalloc`` keeps the split-K
scratch inside the library image for them.  The test drives the raw symbol with ctypes -- no Python wrapper in
between -- and checks it against the regular entry point, twice in a row because both calls share one scratch
array whose counters must come back to zero.  This file sorts last so that a failure here cannot hide others.
"""
import ctypes

import pytest
import torch

from cubic_serve_b200.ops import native, wq_pack
from cubic_serve_b200.quantization import cubic

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _symbol():
    lib = ctypes.CDLL(str(native.build()))       # a handle of our own: the symbol is reached exactly as a C caller would
    fn = lib.cb_wq_gemm_splitk_noalloc
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [i, vp, i, vp, vp, vp, i, vp, f, i, i, i, i, i, vp]
    fn.restype = i
    st = lib.cb_wq_gemm_splitk_noalloc_status
    st.argtypes = [ctypes.POINTER(ctypes.c_uint)]
    st.restype = i
    return fn, st


@pytest.mark.parametrize("m,n,k,splits", [(48, 512, 2048, 4), (48, 512, 2048, 16), (200, 1000, 1024, 3)])
def test_noalloc_entry_matches_regular_entry_twice(m, n, k, splits):
    """The entry point always reduces its K splits through the built-in scratch array (partial sums + arrival
    counters), so every case here reads and writes that array; the regular entry point, left at its default,
    reduces the same splits inside a thread-block cluster -- two different reduction paths that must agree with
    each other and with the fp32 product.  ``n = 1000`` leaves a partly filled last weight tile."""
    from cubic_serve_b200.ops import kernels as K
    fn, status = _symbol()
    g = torch.Generator().manual_seed(0)
    w = torch.randn(n, k, generator=g) * 0.02
    scheme = cubic.CubicScheme(4, 128)
    p = cubic.quantize(w, scheme)
    pw = wq_pack.pack_cubic4(cubic.unpack_codes(p["weight_packed"], 4, k), p["weight_scale"], p["weight_a"],
                             p["weight_b"], 128).to("cuda")
    dense = wq_pack.unpack_to_dense(pw)[:n]
    for rep in range(2):
        x = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).cuda()
        res = torch.randn(m, n, generator=g).to(torch.bfloat16).cuda()
        expect = K.wq_gemm(x, pw, residual=res, splits=min(splits, 8))
        y = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
        rc = fn(pw.fmt, x.data_ptr(), x.stride(0), pw.codes.data_ptr(), pw.meta.data_ptr(), y.data_ptr(), y.stride(0),
                res.data_ptr(), 1.0, m, n, k, pw.group_k, splits, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        word = ctypes.c_uint(7)
        assert status(ctypes.byref(word)) == 0 and word.value == 0
        assert _rel(y, expect) < 1e-2
        assert _rel(y, x.float() @ dense.t() + res.float()) < 1e-2


def test_noalloc_entry_rejects_oversized_requests():
    fn, _ = _symbol()
    # 256 rows x 152 k columns x 16 splits needs far more than the 8 MiB of built-in partial-sum space
    assert fn(0, None, 4096, None, None, None, 151936, None, 1.0, 256, 151936, 4096, 128, 16, None) == -40
    assert fn(0, None, 4096, None, None, None, 4096, None, 1.0, 300, 4096, 4096, 128, 2, None) == -40
