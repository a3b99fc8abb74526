"""The allocation-free RMSNorm backward (``ceo_rmsnorm_bwd_noalloc``), called through its
exported C symbol the way an embedder that may not allocate would call it, must give the
same dx and dw as the regular entry point that takes a caller-provided scratch buffer.
Collected last on purpose: a failure here cannot hide the result of any other test."""
import ctypes

import pytest
import torch

from ceo_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _fn():
    cdll = ctypes.CDLL(str(_lib.LIB_PATH))
    fn = cdll.ceo_rmsnorm_bwd_noalloc
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, vp]
    fn.restype = ci
    return fn


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("rows,D", [(777, 2048), (64, 256), (130, 1000)])
def test_noalloc_matches_regular_entry_point_twice(rows, D):
    dev = torch.device("cuda", 0)
    fn = _fn()
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):  # second call reuses the library's scratch with stale contents
        g = torch.Generator(device=dev).manual_seed(100 + call)
        x = torch.randn(rows, D, device=dev, generator=g).bfloat16()
        dy = torch.randn(rows, D, device=dev, generator=g).bfloat16()
        dres = torch.randn(rows, D, device=dev, generator=g).bfloat16()
        w = (1 + 0.1 * torch.randn(D, device=dev, generator=g)).bfloat16()
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        # outputs and the regular path's scratch are allocated before the call under test
        dx_a, dx_b = torch.empty_like(x), torch.empty_like(x)
        dw_a = torch.full((D,), 0.5, device=dev)
        dw_b = dw_a.clone()
        scratch = torch.empty(L.ceo_norm_bwd_blocks(rows) * D, device=dev)
        rc = L.ceo_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                               dres.data_ptr(), dx_a.data_ptr(), dw_a.data_ptr(), 1,
                               scratch.data_ptr(), rows, D, stream)
        assert rc == 0
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(),
                dx_b.data_ptr(), dw_b.data_ptr(), 1, rows, D, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(dx_a, dx_b)
        assert _rel(dw_b, dw_a) < 1e-6
        # and both agree with the fp32 formula within the tolerance of the other GPU tests
        xf, gf = x.float(), dy.float() * w.float()
        rs = rstd[:, None]
        want = rs * gf - xf * rs.pow(3) * (gf * xf).mean(-1, keepdim=True) + dres.float()
        assert _rel(dx_b, want) < 8e-3
        assert _rel(dw_b - 0.5, (dy.float() * xf * rs).sum(0)) < 8e-3


def test_noalloc_rejects_oversize():
    fn = _fn()
    t = torch.zeros(8, device="cuda")
    p = t.data_ptr()
    assert fn(p, p, p, p, None, p, p, 0, 4, 4096, None) == -6
