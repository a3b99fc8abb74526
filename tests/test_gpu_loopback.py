"""The fused compute + collective kernels on ONE GPU, with every "peer" pointer aimed at local
memory (``ceo_b200.parallel.loopback``): numerics of the fused optimizer step, of the FSDP
weight all-gather inside the GEMM and of the GEMM reduce-scatter, and the time-out path of the
bounded peer waits (a flag that nothing sets; nothing here faults, traps or hangs the GPU)."""
import ctypes

import pytest
import torch

from ceo_b200.ops import _lib, reference as ref
from ceo_b200.ops.matmul import gemm
from ceo_b200.parallel.loopback import LoopbackPeers, table
from ceo_b200.runtime.fault import KernelWatch, describe_status
from ceo_b200.utils import errors

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _ranges(rows):
    return torch.tensor(rows, dtype=torch.int64, device=DEV)


def _zero_step(peers, grads, params, master, m, v, ranges, total, decay_end, *, kind=0,
               do_reduce=1, lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, step=1, gscale=0.5,
               max_norm=1.0, acc=None, norm=None, clip=None):
    L = _lib.lib()
    acc = acc if acc is not None else torch.zeros(2, device=DEV)
    norm = norm if norm is not None else torch.zeros(1, device=DEV)
    clip = clip if clip is not None else torch.ones(1, device=DEV)
    _lib.check(L.ceo_zero_step(table(grads), table(params), peers.flags(), peers.slots(),
                               master.data_ptr(), m.data_ptr(), _lib.ptr(v), acc.data_ptr(),
                               norm.data_ptr(), clip.data_ptr(), peers.status().data_ptr(),
                               ranges.data_ptr(), ranges.shape[0], total, decay_end, 0,
                               peers.world, peers.next_epoch(), kind, do_reduce, lr, b1, b2, eps,
                               wd, step, gscale, max_norm, 0, _lib.stream()), "ceo_zero_step")
    torch.cuda.synchronize()
    return norm, clip


@pytest.mark.parametrize("kind", [0, 1])
def test_zero_step_loopback_matches_reference(kind):
    """Rank 0 of a pretend world of 2: two ownership ranges, one gathered, one kept local."""
    torch.manual_seed(0)
    total, la, lb = 4096, 1024, 512          # range A: [0, 2048), range B: [2048, 3072)
    ranges = _ranges([[0, la, 0, 1], [2048, lb, la, 0]])
    peers = LoopbackPeers(2)
    peers.status().zero_()
    g = [torch.randn(total, device=DEV) * 0.02 for _ in range(2)]
    p = [torch.randn(total, device=DEV).bfloat16() for _ in range(2)]
    p[1].copy_(p[0])
    owned = torch.cat([torch.arange(0, la), torch.arange(2048, 2048 + lb)]).to(DEV)
    master = p[0].float()[owned].clone()
    m = torch.zeros_like(master)
    v = torch.zeros_like(master)
    gsum = (g[0] + g[1])
    # the pretend peer owns the second half of each range; its partial squared norm goes
    # into rank 0's slot block as the peer kernel would have written it
    peer_owned = torch.cat([torch.arange(la, 2 * la), torch.arange(2048 + lb, 2048 + 2 * lb)]).to(DEV)
    peers.signal(0)
    peers.ctrl[0][128:136].view(torch.float32)[1] = gsum[peer_owned].pow(2).sum()
    g0_before, p1_before = g[0].clone(), p[1].clone()
    norm, clip = _zero_step(peers, g, p, master, m, v if kind == 0 else None, ranges, total,
                            decay_end=2048, kind=kind, step=2)
    assert _lib.read_status() == 0
    full = torch.cat([gsum[owned], gsum[peer_owned]])
    nrm = full.norm().item() * 0.5
    assert abs(float(norm) - nrm) < 1e-4 * nrm
    sc = ref.clip_scale(nrm, 1.0)
    assert abs(float(clip) - sc) < 1e-5
    gg = gsum[owned] * 0.5 * sc
    wd = torch.where(owned < 2048, 0.1, 0.0)
    m0 = torch.zeros_like(gg)
    p0 = p1_before.float()[owned]
    if kind == 0:
        mm = 0.1 * gg
        vv = 0.05 * gg * gg
        upd = (mm / (1 - 0.9 ** 2)) / ((vv / (1 - 0.95 ** 2)).sqrt() + 1e-8)
        assert _rel(v, vv) < 1e-5
    else:
        upd = torch.sign(0.9 * m0 + 0.1 * gg)
        mm = 0.05 * gg
    want = p0 * (1 - 1e-2 * wd) - 1e-2 * upd
    assert _rel(master, want) < 1e-6 and _rel(m, mm) < 1e-5
    # gathered range: stored into both parameter buffers; the other only into rank 0's
    assert torch.equal(p[0][:la], want[:la].bfloat16()) and torch.equal(p[1][:la], want[:la].bfloat16())
    assert torch.equal(p[0][2048:2048 + lb], want[la:].bfloat16())
    assert torch.equal(p[1][2048:2048 + lb], p1_before[2048:2048 + lb])
    # this rank's gradient buffer is zero over both ranges (its own slices and the peer's)
    assert float(g[0][:2 * la].abs().max()) == 0.0 and float(g[0][2048:2048 + 2 * lb].abs().max()) == 0.0
    assert torch.equal(g[0][3072:], g0_before[3072:])


def test_zero_step_skips_non_finite_gradients():
    total, ln = 2048, 1024
    ranges = _ranges([[0, ln, 0, 1]])
    peers = LoopbackPeers(2)
    peers.status().zero_()
    peers.signal(0)
    g = [torch.randn(total, device=DEV) * 0.02 for _ in range(2)]
    g[1][5] = float("inf")
    p = [torch.randn(total, device=DEV).bfloat16() for _ in range(2)]
    master = p[0].float()[:ln].clone()
    m = torch.full_like(master, 0.25)
    v = torch.full_like(master, 0.5)
    keep = [t.clone() for t in (master, m, v, p[0], p[1])]
    norm, clip = _zero_step(peers, g, p, master, m, v, ranges, total, decay_end=total)
    assert float(clip) == 0.0 and not torch.isfinite(norm).item()
    for a, b in zip((master, m, v, p[0], p[1]), keep):
        assert torch.equal(a, b)
    assert float(g[0][:total].abs().max()) == 0.0  # the bad gradients are dropped


def test_bounded_peer_waits_run_out_and_leave_state_alone():
    L = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    st = _lib.status_word(dev)
    st.zero_()
    _lib.check(L.ceo_set_wait_limit(3000), "ceo_set_wait_limit")
    try:
        peers = LoopbackPeers(2)  # nobody ever signals for pretend rank 1
        _lib.check(L.ceo_symm_barrier(peers.flags(), 0, 2, 3, peers.next_epoch(), st.data_ptr(),
                                      _lib.stream()), "ceo_symm_barrier")
        torch.cuda.synchronize()
        assert _lib.read_status() == 100 + 3 * 10 + 1
        assert "rank 1" in describe_status(131)
        with pytest.raises(errors.KernelWaitTimeout, match="rank 1"):
            KernelWatch().check()
        assert _lib.read_status() == 0  # the watch resets the word

        out = torch.zeros(4, device=DEV)
        _lib.check(L.ceo_symm_allreduce(peers.staging(), peers.flags(), out.data_ptr(), 4, 0, 2,
                                        peers.next_epoch(), st.data_ptr(), _lib.stream()),
                   "ceo_symm_allreduce")
        torch.cuda.synchronize()
        assert _lib.read_status() == 131
        st.zero_()

        total, ln = 2048, 1024
        g = [torch.randn(total, device=DEV) for _ in range(2)]
        p = [torch.randn(total, device=DEV).bfloat16() for _ in range(2)]
        master = p[0].float()[:ln].clone()
        m = torch.full_like(master, 0.25)
        v = torch.full_like(master, 0.5)
        keep = [t.clone() for t in (master, m, v, p[0], p[1], g[0])]
        _zero_step(peers, g, p, master, m, v, _ranges([[0, ln, 0, 1]]), total, decay_end=total)
        assert _lib.read_status() == 100 + 0 * 10 + 1
        for a, b in zip((master, m, v, p[0], p[1], g[0]), keep):
            assert torch.equal(a, b)
        st.zero_()

        # a bucket reduction whose barrier ran out reduces nothing
        acc = torch.zeros(2, device=DEV)
        g0 = g[0].clone()
        _lib.check(L.ceo_zero_bucket_reduce(table(g), peers.flags(), _ranges([[0, ln, 0, 1]]).data_ptr(),
                                            0, 1, 0, 2, peers.next_epoch(), acc.data_ptr(),
                                            st.data_ptr(), 8, _lib.stream()), "bucket")
        torch.cuda.synchronize()
        assert _lib.read_status() == 100 + 4 * 10 + 1
        assert torch.equal(g[0], g0) and float(acc[0]) == 0.0
    finally:
        _lib.check(L.ceo_set_wait_limit(0), "ceo_set_wait_limit")
        st.zero_()
    # the context is intact: an ordinary GEMM right after is correct
    a = torch.randn(256, 128, device=DEV).bfloat16()
    b = torch.randn(512, 128, device=DEV).bfloat16()
    assert _rel(gemm(a, b), a.float() @ b.float().t()) < 5e-3
    assert _lib.read_status() == 0


def test_bucket_reduce_then_step_without_reduce():
    """Stage 2 order of events on one GPU: the bucket kernel reduces, the step kernel only
    exchanges norms and updates."""
    L = _lib.lib()
    total, ln = 4096, 2048
    ranges = _ranges([[0, ln // 2, 0, 1], [2048, ln // 2, ln // 2, 1]])
    peers = LoopbackPeers(2)
    peers.status().zero_()
    peers.signal(0)
    g = [torch.randn(total, device=DEV) * 0.01 for _ in range(2)]
    gsum = g[0] + g[1]
    p = [torch.zeros(total, device=DEV).bfloat16() for _ in range(2)]
    master = torch.zeros(ln, device=DEV)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    acc = torch.zeros(2, device=DEV)
    for r0 in (0, 1):
        _lib.check(L.ceo_zero_bucket_reduce(table(g), peers.flags(), ranges.data_ptr(), r0, r0 + 1,
                                            0, 2, peers.next_epoch(), acc.data_ptr(),
                                            peers.status().data_ptr(), 8, _lib.stream()), "bucket")
    torch.cuda.synchronize()
    own = torch.cat([gsum[:1024], gsum[2048:3072]])
    assert abs(float(acc[0]) - own.pow(2).sum().item()) < 1e-4 * own.pow(2).sum().item()
    assert torch.allclose(g[0][:1024], gsum[:1024]) and torch.allclose(g[0][2048:3072], gsum[2048:3072])
    norm, _ = _zero_step(peers, g, p, master, m, v, ranges, total, decay_end=total, do_reduce=0,
                         max_norm=0.0, gscale=1.0, wd=0.0, acc=acc)
    assert abs(float(norm) - own.norm().item()) < 1e-4 * own.norm().item()
    mm = 0.1 * own
    assert _rel(m, mm) < 1e-5 and float(acc[0]) == 0.0 and _lib.read_status() == 0


@pytest.mark.parametrize("N,K,M", [(776 * 2, 512, 384), (2048, 256, 200)])
def test_fsdp_weight_gather_inside_gemm(N, K, M):
    """ceo_ag_gemm_bf16(operand = 2): rank 0 of a pretend world of 2 holds rows [0, N/2) of W
    and of a second tensor; the kernel pulls the other halves from the 'peer' buffers while it
    multiplies."""
    import math
    L = _lib.lib()
    torch.manual_seed(1)
    st = _lib.status_word(torch.device("cuda", torch.cuda.current_device()))
    st.zero_()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    e = torch.randn(64, 256, device=DEV).bfloat16()           # the extra tensor, 2 shards of 32 rows
    x = torch.randn(M, K, device=DEV).bfloat16()
    res = torch.randn(M, N, device=DEV).bfloat16()
    mine_w, peer_w = torch.full_like(w, 7.0), torch.full_like(w, -7.0)
    mine_w[:N // 2] = w[:N // 2]
    peer_w[N // 2:] = w[N // 2:]
    mine_e, peer_e = torch.zeros_like(e), torch.zeros_like(e)
    mine_e[:32] = e[:32]
    peer_e[32:] = e[32:]
    blk = math.gcd(N // 2, 64)
    flags = torch.zeros(N // blk, dtype=torch.int32, device=DEV)
    for call in (1, 2):  # the flags count calls: a second gather waits for fresh copies
        if call == 2:
            mine_w[N // 2:] = 3.0
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        _lib.check(L.ceo_ag_gemm_bf16(table([mine_w, peer_w]), 2, x.data_ptr(), out.data_ptr(), M,
                                      N, K, K, N, 0, 0, 0, 1.0, res.data_ptr(), N,
                                      flags.data_ptr(), call, 0, 2, 4, blk, table([mine_e, peer_e]),
                                      e.numel() * 2 // 2, st.data_ptr(), _lib.stream()),
                   "ceo_ag_gemm_bf16")
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        assert torch.equal(mine_w, w) and torch.equal(mine_e, e)
        assert _rel(out, x.float() @ w.float().t() + res.float()) < 5e-3


def test_gemm_reduce_scatter_loopback():
    """ceo_gemm_rs_bf16 as rank 0 of a pretend world of 2: the peer's partial tiles for rank
    0's rows are placed in the staging area and its counters are pre-set, as if it had sent."""
    L = _lib.lib()
    torch.manual_seed(2)
    st = _lib.status_word(torch.device("cuda", torch.cuda.current_device()))
    st.zero_()
    M, N, K = 512, 768, 256
    rows = M // 2
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    res = torch.randn(rows, N, device=DEV).bfloat16()
    peer_part = torch.randn(rows, N, device=DEV).bfloat16()
    stage = [torch.zeros(2, rows, N, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    cnt = [torch.zeros(2, rows // 128, dtype=torch.int32, device=DEV) for _ in range(2)]
    target = 4 * ((N + 255) // 256)
    stage[0][1] = peer_part
    cnt[0][1] = target
    out = torch.empty(rows, N, dtype=torch.bfloat16, device=DEV)
    _lib.check(L.ceo_gemm_rs_bf16(a.data_ptr(), w.data_ptr(), M, N, K, K, K, 0, 0, 1.0,
                                  table(stage), table(cnt), target, out.data_ptr(), res.data_ptr(),
                                  N, 0, 2, 4, st.data_ptr(), _lib.stream()), "ceo_gemm_rs_bf16")
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    full = a.float() @ w.float().t()
    want = full[:rows].bfloat16().float() + peer_part.float() + res.float()
    assert _rel(out, want) < 6e-3
    # the partial tiles for the peer's rows went to the peer's staging area, slot of rank 0
    assert _rel(stage[1][0], full[rows:]) < 6e-3
    assert int(cnt[1][0].min()) == target


def test_fold_affine_matches_fp32_matmul():
    from ceo_b200.parallel.cp import fold_affine
    torch.manual_seed(3)
    for d in (64, 128):
        P = torch.randn(3, 2, d, d, device=DEV)
        s = torch.randn(3, 2, d, d, device=DEV)
        R = torch.randn(3, 2, d, d, device=DEV)
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            want = torch.matmul(P, s) + R
            want_t = torch.matmul(P.transpose(-1, -2), s) + R
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
        assert _rel(fold_affine(P, s, R), want) < 1e-5
        assert _rel(fold_affine(P, s, R, transpose=True), want_t) < 1e-5
