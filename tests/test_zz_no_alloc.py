"""The allocation-free LayerNorm backward, called through its exported C symbol.

Some callers of this library may not allocate device memory while they run (a real-time loop, a process
whose memory pool owns the whole device, code that is handed its buffers).  For them ``rb_ln_bwd_noalloc``
keeps the kernel's scratch in a fixed array inside the library.  This test checks that it gives the same
results as the regular entry point, twice in a row (the array is shared between calls and keeps the last
call's contents), and that it refuses sizes it cannot serve.  It is collected last on purpose."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _close(a, b, tol=2e-2):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err / scale < tol, f"rel err {err / scale:.4g}"


def test_ln_bwd_noalloc_matches_regular_entry_point():
    from rannc_b200.ops import kernels as K

    so = os.path.join(ROOT, "rannc_b200", "_kernels.so")
    lib = ctypes.CDLL(so)
    lib.rb_ln_bwd_noalloc.restype = ctypes.c_int
    lib.rb_ln_bwd_noalloc_strerror.restype = ctypes.c_char_p
    vp = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())  # noqa: E731
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    torch.manual_seed(0)
    for call, (rows, H, p) in enumerate([(1000, 1024, 0.1), (517, 2048, 0.0)]):
        x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
        res = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
        g = (torch.randn(H, device="cuda") * 0.1 + 1).to(torch.bfloat16)
        b = torch.zeros(H, device="cuda", dtype=torch.bfloat16)
        y, z, mean, rstd = K.ln_fwd(x, res, g, b, 1e-5, p, 3, 9)
        dy = torch.randn_like(x)
        ref_dz, ref_dx, ref_dg, ref_db = K.ln_bwd(dy, z, g, mean, rstd, p, 3, 9)
        dz = torch.empty_like(z)
        dx = torch.empty_like(z) if p > 0 else None
        dg = torch.empty(H, device="cuda", dtype=torch.float32)
        db = torch.empty(H, device="cuda", dtype=torch.float32)
        rc = lib.rb_ln_bwd_noalloc(vp(dy), vp(z), vp(g), vp(mean), vp(rstd), vp(dz), vp(dx), vp(dg), vp(db),
                                   ctypes.c_int(rows), ctypes.c_int(H), ctypes.c_float(p), ctypes.c_uint64(3),
                                   ctypes.c_uint64(9), ctypes.c_int(0), ctypes.c_int(1), stream)
        assert rc == 0, lib.rb_ln_bwd_noalloc_strerror(rc)
        torch.cuda.synchronize()
        _close(dz, ref_dz)
        _close(dg, ref_dg)
        _close(db, ref_db)
        if p > 0:
            _close(dx, ref_dx)
    # a width the kernel does not support and a size beyond the built-in scratch are refused, nothing launched
    rc = lib.rb_ln_bwd_noalloc(vp(dy), vp(z), vp(g), vp(mean), vp(rstd), vp(dz), vp(dx), vp(dg), vp(db),
                               ctypes.c_int(8), ctypes.c_int(8192), ctypes.c_float(0.0), ctypes.c_uint64(0),
                               ctypes.c_uint64(0), ctypes.c_int(0), ctypes.c_int(1), stream)
    assert rc == -2 and b"unsupported" in lib.rb_ln_bwd_noalloc_strerror(rc)
    rc = lib.rb_ln_bwd_noalloc(vp(dy), vp(z), vp(g), vp(mean), vp(rstd), vp(dz), vp(dx), vp(dg), vp(db),
                               ctypes.c_int(1000), ctypes.c_int(4096), ctypes.c_float(0.0), ctypes.c_uint64(0),
                               ctypes.c_uint64(0), ctypes.c_int(0), ctypes.c_int(1), stream)
    assert rc == -7 and b"scratch" in lib.rb_ln_bwd_noalloc_strerror(rc)
    # the limit itself: at H = 3072 the built-in scratch serves 394 rows and refuses 395
    H = 3072
    x = torch.randn(395, H, device="cuda", dtype=torch.bfloat16)
    g = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(H, device="cuda", dtype=torch.bfloat16)
    y, z, mean, rstd = K.ln_fwd(x, None, g, b, 1e-5, 0.0, 0, 0)
    dy = torch.randn_like(x)
    dz = torch.empty_like(z)
    dg = torch.empty(H, device="cuda", dtype=torch.float32)
    db = torch.empty(H, device="cuda", dtype=torch.float32)
    for rows, want in ((394, 0), (395, -7)):
        rc = lib.rb_ln_bwd_noalloc(vp(dy), vp(z), vp(g), vp(mean), vp(rstd), vp(dz), vp(None), vp(dg), vp(db),
                                   ctypes.c_int(rows), ctypes.c_int(H), ctypes.c_float(0.0), ctypes.c_uint64(0),
                                   ctypes.c_uint64(0), ctypes.c_int(0), ctypes.c_int(1), stream)
        assert rc == want, (rows, rc, lib.rb_ln_bwd_noalloc_strerror(rc))
    torch.cuda.synchronize()
    ref_dz, _, ref_dg, _ = K.ln_bwd(dy[:394], z[:394], g, mean[:394], rstd[:394])
    _close(dz[:394], ref_dz)
    _close(dg, ref_dg)
