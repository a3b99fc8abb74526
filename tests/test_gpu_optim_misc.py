"""Single-GPU numerics of the optimizer, utility, FP8 and ShortConv kernels."""
import ctypes

import pytest
import torch

from ceo_b200.models.prism import ShortConv
from ceo_b200.ops import _lib, conv, reference as ref
from ceo_b200.optim.flat import FlatParams
from ceo_b200.optim.optimizers import ShardedOptimizer

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _model():
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(256, 512, bias=False), torch.nn.Linear(512, 128, bias=False))
    return m.to(DEV).to(torch.bfloat16)


@pytest.mark.parametrize("kind", ["adamw", "lion"])
def test_flat_optimizers_match_fp32_reference(kind):
    model = _model()
    flat = FlatParams(model)
    opt = ShardedOptimizer(flat, kind, weight_decay=0.1, max_grad_norm=1.0, betas=(0.9, 0.95),
                           lion_betas=(0.9, 0.99))
    master = flat.master.clone()
    m = torch.zeros_like(master)
    v = torch.zeros_like(master)
    n = flat.numel()
    for step in range(1, 4):
        g = torch.randn(flat.total, device=DEV) * 0.01
        g[n:] = 0
        flat.grads.copy_(g)
        gn = opt.step(1e-2, grad_scale=0.5)
        gg = g * 0.5
        nrm = gg.norm().item()
        gg = gg * ref.clip_scale(nrm, 1.0)
        assert abs(float(gn) - nrm) < 1e-3 * nrm
        wd = torch.where(torch.arange(flat.total, device=DEV) < flat.decay_end, 0.1, 0.0)
        if kind == "adamw":
            m.mul_(0.9).add_(gg, alpha=0.1)
            v.mul_(0.95).addcmul_(gg, gg, value=0.05)
            upd = (m / (1 - 0.9 ** step)) / ((v / (1 - 0.95 ** step)).sqrt() + 1e-8)
        else:
            upd = torch.sign(0.9 * m + 0.1 * gg)
            m.mul_(0.99).add_(gg, alpha=0.01)
        master = master * (1 - 1e-2 * wd) - 1e-2 * upd
        assert _rel(flat.master[:n], master[:n]) < 1e-5
        assert torch.equal(flat.params[:n], flat.master[:n].bfloat16())
        assert float(flat.grads.abs().max()) == 0.0


def test_muon_newton_schulz_on_gemm_kernel():
    model = _model()
    flat = FlatParams(model)
    opt = ShardedOptimizer(flat, "lion_muon", max_grad_norm=0.0, muon_iterations=12)
    g = torch.randn(512, 256, device=DEV).bfloat16()
    y = (g.float() / g.float().norm()).bfloat16()
    out = opt._newton_schulz(y).float()
    want = ref.newton_schulz_cubic(g.float(), 12)
    assert _rel(out, want) < 5e-2
    gram = out.t() @ out
    assert _rel(gram, torch.eye(256, device=DEV)) < 0.1
    p0 = flat.params.clone()
    flat.grads.normal_(0, 0.01)
    opt.step(1e-3)
    assert not torch.equal(flat.params, p0) and torch.isfinite(flat.params.float()).all()


def test_fill_cast_copy_reduce_fp8():
    L = _lib.lib()
    st = _lib.stream()
    n = 100003 * 8
    x = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    assert L.ceo_fill(x.data_ptr(), 2, n, 1.5, st) == 0
    assert float(x.float().min()) == 1.5 == float(x.float().max())
    src = torch.randn(n, device=DEV)
    h = torch.empty(n, device=DEV, dtype=torch.float16)
    assert L.ceo_cast(src.data_ptr(), 0, h.data_ptr(), 1, n, st) == 0
    assert torch.equal(h, src.half())
    b = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    assert L.ceo_cast(h.data_ptr(), 1, b.data_ptr(), 2, n, st) == 0
    assert torch.equal(b, h.bfloat16())
    dst = torch.empty_like(src)
    assert L.ceo_copy(src.data_ptr(), dst.data_ptr(), n * 4, st) == 0
    assert torch.equal(dst, src)
    out = torch.empty(1, device=DEV)
    scratch = torch.empty(L.ceo_reduce_blocks(n), device=DEV)
    for mode, want in ((0, src.double().sum()), (1, src.double().pow(2).sum()),
                       (2, src.double().norm())):
        assert L.ceo_reduce(src.data_ptr(), 0, n, mode, out.data_ptr(), scratch.data_ptr(), st) == 0
        assert abs(out.item() - want.item()) < 1e-3 * abs(want.item()) + 1e-2
    # fp8 with delayed scaling
    xb = (torch.randn(n, device=DEV) * 3).bfloat16()
    scale = torch.tensor([448.0 / 16.0], device=DEV)
    amax = torch.zeros(1, device=DEV)
    q = torch.empty(n, device=DEV, dtype=torch.uint8)
    assert L.ceo_fp8_quantize(xb.data_ptr(), q.data_ptr(), n, scale.data_ptr(), amax.data_ptr(), 0,
                              st) == 0
    want_q = (xb.float() * scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert torch.equal(q.view(torch.float8_e4m3fn).float(), want_q.float())
    assert abs(amax.item() - xb.float().abs().max().item()) < 1e-6
    back = torch.empty_like(xb)
    assert L.ceo_fp8_dequantize(q.data_ptr(), back.data_ptr(), n, scale.data_ptr(), 0, st) == 0
    assert _rel(back, xb) < 0.05
    hist = torch.zeros(16, device=DEV)
    cur = torch.zeros(1, device=DEV, dtype=torch.int32)
    assert L.ceo_fp8_update_scale(hist.data_ptr(), 16, cur.data_ptr(), amax.data_ptr(),
                                  scale.data_ptr(), 448.0, 1.0, st) == 0
    assert abs(scale.item() - 448.0 / xb.float().abs().max().item()) < 1e-3 and amax.item() == 0
    assert L.ceo_fill(x.data_ptr(), 7, n, 0.0, st) == -5


@pytest.mark.parametrize("window", [4, 16, 64])
def test_shortconv(window):
    torch.manual_seed(1)
    B, T, D = 2, 200, 512
    x = torch.randn(B, T, D, device=DEV).bfloat16().requires_grad_()
    w = (torch.randn(D, window, device=DEV) * 0.2).bfloat16().requires_grad_()
    y = conv.shortconv(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.shortconv(xr, wr)
    yr.backward(dy.float())
    assert _rel(y, yr) < 6e-3 and _rel(x.grad, xr.grad) < 8e-3 and _rel(w.grad, wr.grad) < 1e-2
    # literal definition on one element
    t, d = 150, 7
    lit = sum(float(xr[0, t - j, d]) * float(wr[d, j]) for j in range(window))
    assert abs(float(yr[0, t, d]) - lit) < 1e-4


def test_model_with_prism_branch_trains_on_gpu():
    from ceo_b200.runtime.engine import TrainEngine
    from ceo_b200.utils.config import Config
    import os
    cfg = Config.parse_from_file(os.path.join(os.path.dirname(os.path.dirname(__file__)),
                                              "configs", "smoke.yaml"))
    cfg.training.optimizer = "adamw"
    eng = TrainEngine(cfg, torch.device(DEV))
    tok = torch.randint(0, cfg.model.vocab_size, (2, 129), device=DEV)
    losses = [float(eng.train_step([(tok[:, :-1].contiguous()[:, :128], tok[:, 1:].contiguous()[:, :128])],
                                   lr=2e-3)[0]) for _ in range(4)]
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    assert _lib.read_status() == 0


@pytest.mark.parametrize("rows,n", [(300, 777), (3, 200_000), (1, 1_000_003)])
@pytest.mark.parametrize("exclusive,reverse", [(False, False), (True, False), (False, True),
                                               (True, True)])
def test_cumsum_matches_fp64(rows, n, exclusive, reverse):
    from ceo_b200.ops import tensor_ops as T
    x = torch.randn(rows, n, device="cuda")
    y = T.cumsum(x, exclusive, reverse)
    xd = x.double().flip(-1) if reverse else x.double()
    r = xd.cumsum(-1)
    if exclusive:
        r = r - xd
    r = r.flip(-1) if reverse else r
    assert (y.double() - r).abs().max().item() < 2e-3 * (n ** 0.5)


def test_gather_scatter_copy_transpose_memset():
    from ceo_b200.ops import tensor_ops as T
    g = torch.Generator(device="cuda").manual_seed(3)
    src = torch.randn(1000, 72, device="cuda", generator=g).bfloat16()
    idx = torch.randint(-2, 1002, (5000,), device="cuda", generator=g)
    out = T.gather_rows(src, idx)
    ok = (idx >= 0) & (idx < 1000)
    exp = torch.where(ok[:, None], src[idx.clamp(0, 999)], torch.zeros_like(out))
    assert torch.equal(out, exp)
    perm = torch.randperm(1000, device="cuda")
    dst = torch.zeros_like(src)
    T.scatter_rows(dst, perm, src)
    assert torch.equal(dst[perm], src)
    acc = torch.zeros(50, 64, device="cuda")
    vals = torch.randn(4000, 64, device="cuda", generator=g)
    where = torch.randint(0, 50, (4000,), device="cuda", generator=g)
    T.scatter_add_rows(acc, where, vals)
    exp = torch.zeros(50, 64, device="cuda", dtype=torch.float64).index_add_(0, where, vals.double())
    assert (acc.double() - exp).abs().max().item() < 1e-3
    big = torch.randn(333, 512, device="cuda", generator=g)
    view = big[:, 128:384]
    d2 = torch.empty(333, 256, device="cuda")
    T.copy2d(d2, view)
    assert torch.equal(d2, view)
    m = torch.randn(301, 190, device="cuda", generator=g).bfloat16()
    assert torch.equal(T.transpose2d(m), m.t().contiguous())
    z = torch.empty(100_003, dtype=torch.int32, device="cuda")
    T.memset32(z, 0xDEADBEEF)
    assert (z.view(torch.int32) == (0xDEADBEEF - 2 ** 32)).all()


def test_bounds_checked_build_is_clean_and_its_recorder_works():
    """The debug build of the library (checked indexing) runs tile-edge shapes without a
    recorded violation, and its recorder reports indices past an extent (which it redirects,
    so nothing outside the buffer is touched)."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = os.path.join(root, "ceo_b200", "lib", "libceo_b200_chk.so")
    if not os.path.exists(lib):
        from ceo_b200 import build as b
        b.build(bounds_check=True)
    env = dict(os.environ, CEO_B200_BOUNDS_CHECK="1")
    r = subprocess.run([sys.executable, os.path.join(root, "tests", "bounds_worker.py")], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("BOUNDS ")][-1]
    out = json.loads(line[len("BOUNDS "):])
    assert out["clean"] == [0, 0, 0, 0]
    n, site, idx, extent = out["selftest"]
    assert n == 5 and site == 199 and 100 <= idx < 105 and extent == 100
    assert out["after_reset"] == [0, 0, 0, 0]
    assert out["sum"] == 100.0 + 5.0             # the five redirected reads saw element 0


@pytest.mark.parametrize("kind", ["adamw", "lion", "lion_muon"])
def test_non_finite_gradient_skips_the_step(kind):
    """One inf in the gradients: parameters, master weights and moments stay bit-identical,
    the gradients are dropped, and the next (finite) step works."""
    model = _model()
    flat = FlatParams(model)
    opt = ShardedOptimizer(flat, kind, weight_decay=0.1, max_grad_norm=1.0)
    flat.grads.copy_(torch.randn(flat.total, device=DEV) * 0.01)
    opt.step(1e-2)  # a normal step first, so that the moments are not all zero
    snap = {k: v.clone() for k, v in flat.optimizer_state().items()}
    muon = {n: {k: v.clone() for k, v in st.items()} for n, st in opt._muon_state.items()}
    params = flat.params.clone()
    flat.grads.copy_(torch.randn(flat.total, device=DEV) * 0.01)
    flat.grads[17] = float("inf")
    gn = opt.step(1e-2)
    assert not torch.isfinite(gn).item()
    assert torch.equal(flat.params, params)
    for k, v in flat.optimizer_state().items():
        assert torch.equal(v, snap[k]), k
    for n, st in opt._muon_state.items():
        for k, v in st.items():
            assert torch.equal(v, muon[n][k]), (n, k)
    assert float(flat.grads.abs().max()) == 0.0
    flat.grads.copy_(torch.randn(flat.total, device=DEV) * 0.01)
    opt.step(1e-2)
    assert not torch.equal(flat.params, params) and torch.isfinite(flat.master).all()
