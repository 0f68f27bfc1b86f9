"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the point where they call it (a
host application that reserved the whole device pool, a callback that runs while a stream is being
captured, a real-time loop that must not trigger cudaFree's device synchronisation).  For them
``b2_rmsnorm_bwd_noalloc`` keeps its temporary partial sums in a static device array inside the
library.  The test compares it against the regular entry point (which receives its scratch buffer
from the caller) twice in a row, so that the second call runs on a scratch area the first one left
dirty.  This file sorts last on purpose: if it fails under ``-x`` every other test has already run.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _c(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _run(lib, name, dy, x, w, rstd, with_scratch):
    M, H = x.shape
    dx = torch.empty_like(x)
    dw = torch.empty(H, device=x.device, dtype=torch.float32)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    fn = getattr(lib, name)
    fn.restype = ctypes.c_int
    if with_scratch:
        ctas = lib.b2_rmsnorm_bwd_ctas()
        scratch = torch.full((ctas * H,), float("nan"), device=x.device)     # caller-provided scratch
        rc = fn(_c(dy), _c(x), _c(w), _c(rstd), _c(dx), _c(dw), _c(scratch), M, H, 0, 0, 1, stream)
    else:
        rc = fn(_c(dy), _c(x), _c(w), _c(rstd), _c(dx), _c(dw), M, H, 0, 0, 1, stream)
    assert rc == 0, lib.b2_last_error().decode()
    torch.cuda.synchronize()
    return dx, dw


@pytest.mark.parametrize("M,H", [(4096, 1024), (300, 2048), (17, 256)])
def test_noalloc_entry_matches_regular_entry_twice(M, H):
    from b200fw import _native as nv
    lib = nv.lib()
    torch.manual_seed(M + H)
    for attempt in range(2):       # the second pass reuses the scratch array the first one wrote
        x = torch.randn(M, H, device="cuda", dtype=torch.bfloat16) * (1 + attempt)
        dy = torch.randn(M, H, device="cuda", dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        dx_a, dw_a = _run(lib, "b2_rmsnorm_bwd", dy, x, w, rstd, with_scratch=True)
        dx_b, dw_b = _run(lib, "b2_rmsnorm_bwd_noalloc", dy, x, w, rstd, with_scratch=False)
        assert torch.equal(dx_a, dx_b)
        scale = dw_a.abs().max().item() + 1e-6
        assert (dw_a - dw_b).abs().max().item() / scale < 1.5e-2      # tolerance of the other kernel tests
        # and both agree with the fp32 formula
        xh = x.float() * rstd[:, None]
        want_dw = (dy.float() * xh).sum(0)
        assert (dw_b - want_dw).abs().max().item() / (want_dw.abs().max().item() + 1e-6) < 1.5e-2
    assert nv.read_status() == 0


def test_noalloc_entry_rejects_sizes_beyond_its_scratch():
    from b200fw import _native as nv
    lib = nv.lib()
    lib.b2_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    x = torch.zeros(8, 4096, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(4096, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(8, device="cuda")
    dw = torch.zeros(4096, device="cuda")
    rc = lib.b2_rmsnorm_bwd_noalloc(_c(x), _c(x), _c(w), _c(rstd), _c(x.clone()), _c(dw), 8, 4096, 0, 0, 1,
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and b"outside the built-in scratch" in lib.b2_last_error()


def test_noalloc_entry_rejects_null_pointers_and_checks_h_before_the_empty_case():
    from b200fw import _native as nv
    lib = nv.lib()
    lib.b2_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    x = torch.zeros(8, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(8, device="cuda")
    dw = torch.zeros(1024, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.b2_rmsnorm_bwd_noalloc(_c(x), _c(x), _c(w), ctypes.c_void_p(0), _c(x.clone()), _c(dw), 8, 1024, 0, 0, 1, stream)
    assert rc == 10 and b"null pointer" in lib.b2_last_error()
    # an out-of-range H is an error even when there are no rows to process
    rc = lib.b2_rmsnorm_bwd_noalloc(_c(x), _c(x), _c(w), _c(rstd), _c(x.clone()), _c(dw), 0, 4096, 0, 0, 1, stream)
    assert rc == 10
    rc = lib.b2_rmsnorm_bwd_noalloc(_c(x), _c(x), _c(w), _c(rstd), _c(x.clone()), _c(dw), 0, 1024, 0, 0, 1, stream)
    assert rc == 0
    assert nv.read_status() == 0
