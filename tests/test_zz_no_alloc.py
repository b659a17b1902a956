"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some embedders of the library may not allocate GPU memory at run time (their process has
already committed all of it to a pool of its own), so ``hpb_rmsnorm_bwd_noalloc`` keeps its
scratch inside the library.  It must give the same result as ``hpb_rmsnorm_bwd`` with
caller-provided scratch -- on two consecutive calls, because both share one scratch array.
This file sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _fns():
    from hyper_parallel_b200.ops import native
    lib = native.lib()
    vp, ci, c64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    noalloc = lib.hpb_rmsnorm_bwd_noalloc
    noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, c64, ci, vp]
    noalloc.restype = ci
    strerror = lib.hpb_noalloc_strerror
    strerror.argtypes = [ci]
    strerror.restype = ctypes.c_char_p
    return lib, noalloc, strerror


def _case(T, H, seed, with_dres):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    x, dy = mk(T, H), mk(T, H)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    dres = mk(T, H) if with_dres else None
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    return x, dy, w, dres, rstd


def test_noalloc_matches_existing_entry_point_twice_in_a_row():
    from hyper_parallel_b200.ops import native
    lib, noalloc, strerror = _fns()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (T, H, with_dres) in enumerate([(300, 4096, False), (513, 7168, True)]):
        x, dy, w, dres, rstd = _case(T, H, 100 + call, with_dres)
        # existing entry point: scratch allocated by the caller
        P = min(T, native.sm_count("cuda") * 2)
        part = torch.empty(P, H, dtype=torch.float32, device="cuda")
        dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
        rc = lib.hpb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                 native.ptr(dres), dx_ref.data_ptr(), part.data_ptr(), P,
                                 dw_ref.data_ptr(), 0, 0, T, H, stream)
        assert rc == 0
        # new entry point: no scratch argument at all
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        rc = noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), native.ptr(dres),
                     dx.data_ptr(), dw.data_ptr(), 0, 0, T, H, stream)
        assert rc == 0, strerror(rc)
        torch.cuda.synchronize()
        # dx is computed row by row, independent of the number of partial rows: identical
        assert torch.equal(dx, dx_ref)
        # dw sums a different number of partial rows: same tolerance as the kernel tests
        err = (dw.float() - dw_ref.float()).norm() / dw_ref.float().norm()
        assert err < 1e-2, err.item()
        # and both agree with the fp32 formula
        xf, gf = x.float(), dy.float()
        dw_true = (gf * xf * rstd[:, None]).sum(0)
        assert (dw.float() - dw_true).norm() / dw_true.norm() < 1e-2


def test_noalloc_rejects_oversize_and_bad_shapes():
    lib, noalloc, strerror = _fns()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.hpb_noalloc_max_h() == 8192
    rc = noalloc(None, None, None, None, None, None, None, 0, 0, 16, 8192 + 8, stream)
    assert rc == -100 and b"exceeds" in strerror(rc)
    rc = noalloc(None, None, None, None, None, None, None, 0, 0, 16, 100, stream)
    assert rc == -101
