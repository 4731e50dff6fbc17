"""The allocation-free RMSNorm backward (`b200_rmsnorm_bwd_static`, scratch in a fixed device
array) against the regular entry point with caller-provided scratch. Collected last on purpose:
it must pass both alone and after every other GPU test has used the library."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_TOO_SMALL = -120


def _lib_and_stream():
    from areal_b200.ops import _lib

    lib = _lib.kernels()
    lib.b200_ensure_device(ctypes.c_int(torch.cuda.current_device()))
    for f in (lib.b200_rmsnorm_bwd_static, lib.b200_rmsnorm_bwd, lib.b200_rmsnorm_bwd_blocks):
        f.restype = ctypes.c_int
    return _lib, lib


def _inputs(T, H, seed, with_res):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).bfloat16()
    x, dy, w = mk(T, H), mk(T, H), mk(H)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    return dy, x, w, rstd, (mk(T, H) if with_res else None)


def _regular(_lib, lib, dy, x, w, rstd, dres, dw, acc):
    T, H = x.shape
    partial = torch.empty((lib.b200_rmsnorm_bwd_blocks(ctypes.c_int(T)), H), dtype=torch.float32, device="cuda")
    dx = torch.empty_like(x)
    rc = lib.b200_rmsnorm_bwd(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres), _lib.ptr(dx),
                              _lib.ptr(partial), _lib.ptr(dw), ctypes.c_int(acc), ctypes.c_int(T), ctypes.c_int(H),
                              _lib.stream_ptr())
    assert rc == 0
    return dx


def _static(_lib, lib, dy, x, w, rstd, dres, dw, acc):
    T, H = x.shape
    dx = torch.empty_like(x)
    rc = lib.b200_rmsnorm_bwd_static(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres),
                                     _lib.ptr(dx), _lib.ptr(dw), ctypes.c_int(acc), ctypes.c_int(T),
                                     ctypes.c_int(H), _lib.stream_ptr())
    assert rc == 0
    return dx


def test_static_scratch_matches_regular_entry_point_twice_in_a_row():
    _lib, lib = _lib_and_stream()
    # two calls back to back on one stream, different shapes: the second reuses (and fully
    # overwrites) the scratch rows the first one left behind
    cases = [(4099, 2048, 1, True, 0), (517, 4096, 2, False, 1)]
    got, want = [], []
    for T, H, seed, with_res, acc in cases:
        dy, x, w, rstd, dres = _inputs(T, H, seed, with_res)
        dw = torch.full((H,), 0.5, dtype=torch.float32, device="cuda")
        got.append((_static(_lib, lib, dy, x, w, rstd, dres, dw, acc), dw))
    for T, H, seed, with_res, acc in cases:
        dy, x, w, rstd, dres = _inputs(T, H, seed, with_res)
        dw = torch.full((H,), 0.5, dtype=torch.float32, device="cuda")
        want.append((_regular(_lib, lib, dy, x, w, rstd, dres, dw, acc), dw))
    torch.cuda.synchronize()
    for (dx_s, dw_s), (dx_r, dw_r) in zip(got, want):
        assert torch.equal(dx_s, dx_r)
        assert torch.equal(dw_s, dw_r)
    # and against plain PyTorch fp32 for the first case
    T, H, seed, with_res, _ = cases[0]
    dy, x, w, rstd, dres = _inputs(T, H, seed, with_res)
    xf = x.float().requires_grad_()
    wf = w.float().requires_grad_()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    y.backward(dy.float())
    torch.testing.assert_close(got[0][0].float(), xf.grad + dres.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got[0][1], wf.grad, rtol=2e-2, atol=0.5)


def test_static_scratch_at_the_documented_width_limit():
    """H = 8192 is the widest row the built-in scratch takes (128 KB of dynamic shared memory per block, which
    needs the opt-in attribute): same bits as the regular entry point, overwrite and accumulate."""
    _lib, lib = _lib_and_stream()
    T, H = 301, 8192
    for seed, with_res, acc in ((5, True, 0), (6, False, 1)):
        dy, x, w, rstd, dres = _inputs(T, H, seed, with_res)
        dw_s = torch.full((H,), 0.25, dtype=torch.float32, device="cuda")
        dw_r = dw_s.clone()
        dx_s = _static(_lib, lib, dy, x, w, rstd, dres, dw_s, acc)
        dx_r = _regular(_lib, lib, dy, x, w, rstd, dres, dw_r, acc)
        torch.cuda.synchronize()
        assert torch.equal(dx_s, dx_r) and torch.equal(dw_s, dw_r)


def test_static_scratch_rejects_sizes_beyond_its_limit():
    _lib, lib = _lib_and_stream()
    dummy = torch.zeros(8, device="cuda")
    rc = lib.b200_rmsnorm_bwd_static(_lib.ptr(dummy), _lib.ptr(dummy), _lib.ptr(dummy), _lib.ptr(dummy), None,
                                     _lib.ptr(dummy), _lib.ptr(dummy), ctypes.c_int(0), ctypes.c_int(4),
                                     ctypes.c_int(8200), _lib.stream_ptr())
    assert rc == ERR_TOO_SMALL  # nothing was launched
    torch.cuda.synchronize()
