"""The allocation-free norm backward (``mrk_norm_bwd_noalloc``) must agree with the regular entry
point.

Some users of the kernel library cannot allocate device memory when they need this gradient (they
run under an allocator lock, inside a pre-partitioned memory budget, or are simply forbidden to
call cudaMalloc), so the library offers a variant whose partial-sum workspace is a fixed array
inside the shared object.  The test drives it the way such a caller would: through the exported C
symbol, with caller-owned input and output buffers only, twice in a row with different shapes so
that the second call reuses the array the first one accumulated into and cleared.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "merak_b200", "_mrk_kernels.so")


def _lib():
    lib = ctypes.CDLL(LIB)
    P, LL, I, F = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    lib.mrk_norm_bwd_noalloc.restype = I
    lib.mrk_norm_bwd_noalloc.argtypes = [P] * 10 + [LL, I, I, I, P]
    lib.mrk_norm_bwd.restype = I
    lib.mrk_norm_bwd.argtypes = [P] * 12 + [ctypes.c_ulonglong, F, LL, I, I, I, P]
    lib.mrk_norm_bwd_workspace_rows.restype = I
    lib.mrk_last_error.restype = ctypes.c_char_p
    return lib


def _case(M, H, rms, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    z = r(M, H).bfloat16()
    dy = r(M, H).bfloat16()
    extra = r(M, H).bfloat16()
    gamma = (1 + 0.1 * r(H)).bfloat16()
    zf = z.float()
    if rms:
        mean = None
        rstd = torch.rsqrt(zf.pow(2).mean(-1) + 1e-5)
    else:
        mean = zf.mean(-1)
        rstd = torch.rsqrt(zf.var(-1, unbiased=False) + 1e-5)
    return dy, z, extra, gamma, mean, rstd


def _ptr(t):
    return 0 if t is None else t.data_ptr()


@pytest.mark.parametrize("rms", [False, True])
def test_noalloc_matches_regular_entry_point_twice(rms):
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second one reuses the scratch the first one used (and cleared),
    # with a different row count and hidden size
    for M, H, seed in ((3000, 1024, 1), (333, 1600, 2)):
        dy, z, extra, gamma, mean, rstd = _case(M, H, rms, seed)
        outs = []
        for which in ("regular", "noalloc"):
            dres = torch.empty_like(dy)
            dgamma = torch.full((H,), float("nan"), device="cuda")
            dbeta = None if rms else torch.full((H,), float("nan"), device="cuda")
            if which == "regular":
                ws = torch.zeros((lib.mrk_norm_bwd_workspace_rows(), 2, H), device="cuda")   # must start at zero
                rc = lib.mrk_norm_bwd(dy.data_ptr(), z.data_ptr(), extra.data_ptr(), gamma.data_ptr(), _ptr(mean),
                                      rstd.data_ptr(), dres.data_ptr(), dres.data_ptr(), dgamma.data_ptr(),
                                      _ptr(dbeta), ws.data_ptr(), 0, 0, 0.0, M, H, int(rms), 0, stream)
            else:
                rc = lib.mrk_norm_bwd_noalloc(dy.data_ptr(), z.data_ptr(), extra.data_ptr(), gamma.data_ptr(),
                                              _ptr(mean), rstd.data_ptr(), dres.data_ptr(), dres.data_ptr(),
                                              dgamma.data_ptr(), _ptr(dbeta), M, H, int(rms), 0, stream)
            assert rc == 0, lib.mrk_last_error()
            torch.cuda.synchronize()
            outs.append((dres, dgamma, dbeta))
        (r_dres, r_dg, r_db), (n_dres, n_dg, n_db) = outs
        assert torch.equal(r_dres, n_dres)                      # row-local math: identical
        scale = r_dg.abs().max().item() + 1e-6
        assert (r_dg - n_dg).abs().max().item() / scale < 2e-2   # summation order differs
        if not rms:
            assert (r_db - n_db).abs().max().item() / (r_db.abs().max().item() + 1e-6) < 2e-2


def test_noalloc_rejects_sizes_beyond_its_scratch():
    lib = _lib()
    M, H = 16, 4096
    dy, z, extra, gamma, mean, rstd = _case(M, H, False, 3)
    dres = torch.empty_like(dy)
    dgamma = torch.zeros(H, device="cuda")
    rc = lib.mrk_norm_bwd_noalloc(dy.data_ptr(), z.data_ptr(), 0, gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                  dres.data_ptr(), dres.data_ptr(), dgamma.data_ptr(), 0, M, H, 0, 0,
                                  torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    assert b"exceeds the built-in scratch" in lib.mrk_last_error()
