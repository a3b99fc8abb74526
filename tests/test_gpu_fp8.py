"""FP8 on the GPU: the tcgen05 kind::f8f6f4 GEMM against an fp32 product of the same codes,
the vectorised quantiser against torch's casts, the Linear and a training run."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _codes(shape, kind, scale=1.0):
    from ceo_b200.ops import fp8 as F8
    x = torch.randn(*shape, device=DEV) * scale
    return x.to(F8._TORCH[kind]).view(torch.uint8)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 520, 400), (1000, 72, 48),
                                   (4096, 6144, 2048)])
@pytest.mark.parametrize("ka,kb", [(0, 0), (1, 0)])
def test_gemm_fp8_matches_fp32_product_of_the_codes(M, N, K, ka, kb):
    from ceo_b200.ops import _lib
    from ceo_b200.ops import fp8 as F8
    torch.manual_seed(M + K + ka)
    aq, bq = _codes((M, K), ka), _codes((N, K), kb, 0.5)
    ref = aq.view(F8._TORCH[ka]).float() @ bq.view(F8._TORCH[kb]).float().t()
    out = F8.gemm_fp8(aq, bq, kind_a=ka, kind_b=kb, out_dtype=torch.float32)
    assert (out - ref).norm() / ref.norm() < 1e-5
    assert (out - ref).abs().max() < 1e-3 * ref.abs().max()
    outb = F8.gemm_fp8(aq, bq, kind_a=ka, kind_b=kb)
    assert outb.dtype == torch.bfloat16
    assert (outb.float() - ref).norm() / ref.norm() < 4e-3
    assert _lib.read_status() == 0


def test_gemm_fp8_scales_residual_bias_accumulate():
    from ceo_b200.ops import fp8 as F8
    torch.manual_seed(3)
    M, N, K = 512, 384, 640
    x = torch.randn(M, K, device=DEV).bfloat16() * 3
    w = (torch.randn(N, K, device=DEV) * 0.02).bfloat16()
    mx, mw = F8.Fp8Meta(DEV), F8.Fp8Meta(DEV)
    xq, wq = F8.quantize(x, mx), F8.quantize(w, mw)
    assert abs(mx.scale.item() - 448.0 / x.float().abs().max().item()) < 1e-3 * mx.scale.item()
    deq = lambda q, m: q.view(torch.float8_e4m3fn).float() / m.scale  # noqa: E731
    prod = deq(xq, mx) @ deq(wq, mw).t()
    res = torch.randn(M, N, device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV)
    out = F8.gemm_fp8(xq, wq, mx, mw, out_dtype=torch.float32, alpha=0.5, bias=bias, residual=res)
    want = 0.5 * prod + bias + res.float()
    assert (out - want).norm() / want.norm() < 1e-5
    acc = torch.ones(M, N, device=DEV)
    F8.gemm_fp8(xq, wq, mx, mw, out=acc, accumulate=True)
    assert (acc - (prod + 1)).norm() / (prod + 1).norm() < 1e-5
    # against the unquantised product the error is the quantisation noise
    true = x.float() @ w.float().t()
    assert (prod - true).norm() / true.norm() < 0.05


@pytest.mark.parametrize("n,off", [(1 << 20, 0), (100003, 0), (4099, 1)])
@pytest.mark.parametrize("kind", [0, 1])
def test_quantiser_matches_torch_cast(n, off, kind):
    from ceo_b200.ops import fp8 as F8
    torch.manual_seed(n)
    x = (torch.randn(n + off, device=DEV) * 4).bfloat16()[off:]
    meta = F8.Fp8Meta(DEV, kind)
    meta.calibrated = True
    meta.scale.fill_(2.5)
    q = F8._quantize_raw(x, meta)
    lim = F8._FMAX[kind]
    want = (x.float() * 2.5).clamp(-lim, lim).to(F8._TORCH[kind])
    assert torch.equal(q.view(F8._TORCH[kind]).float(), want.float())
    assert abs(meta.amax.item() - x.float().abs().max().item()) < 1e-6


def test_fp8_linear_forward_and_backward():
    from ceo_b200.ops import fp8 as F8
    torch.manual_seed(5)
    x = torch.randn(4, 256, 512, device=DEV).bfloat16().requires_grad_()
    w = (torch.randn(768, 512, device=DEV) * 0.03).bfloat16().requires_grad_()
    res = torch.randn(4, 256, 768, device=DEV).bfloat16().requires_grad_()
    st = F8.Fp8Recipe().new_state(DEV)
    y = F8.fp8_linear(x, w, st, res)
    ref = x.float() @ w.float().t() + res.float()
    assert (y.float() - ref).norm() / ref.norm() < 0.05
    dy = torch.randn_like(y)
    gx, gw, gr = torch.autograd.grad(y, (x, w, res), dy)
    rx = dy.float() @ w.float()
    rw = dy.float().reshape(-1, 768).t() @ x.float().reshape(-1, 512)
    assert (gx.float() - rx).norm() / rx.norm() < 1e-2
    assert (gw.float() - rw).norm() / rw.norm() < 1e-2
    assert torch.equal(gr, dy)


def test_fp8_data_gradient_option_on_gpu():
    from ceo_b200.ops import fp8 as F8
    torch.manual_seed(6)
    x = torch.randn(1024, 512, device=DEV).bfloat16().requires_grad_()
    w = (torch.randn(784, 512, device=DEV) * 0.03).bfloat16().requires_grad_()
    st = F8.Fp8Recipe(dgrad=True).new_state(DEV)
    y = F8.fp8_linear(x, w, st)
    dy = (torch.randn_like(y.float()) * 1e-3).bfloat16()
    gx, gw = torch.autograd.grad(y, (x, w), dy)
    rx = dy.float() @ w.float()
    rw = dy.float().t() @ x.float()
    err = (gx.float() - rx).norm() / rx.norm()
    assert 0 < err < 0.08
    assert (gw.float() - rw).norm() / rw.norm() < 1e-2
    # same codes through an fp32 product: the kernel itself is exact
    dyq = F8._quantize_raw(dy, st.g_meta)
    want = (dyq.view(torch.float8_e5m2).float() @ st.wtq.view(torch.float8_e4m3fn).float().t()) \
        / (st.g_meta.scale * st.w_meta.scale)
    assert (gx.float() - want).norm() / want.norm() < 4e-3


@pytest.mark.parametrize("rows,cols,kind", [(64, 64, 0), (4096, 2048, 0), (1008, 784, 1),
                                            (16, 6208, 1)])
def test_transposing_quantiser(rows, cols, kind):
    from ceo_b200.ops import fp8 as F8
    torch.manual_seed(rows + cols)
    x = (torch.randn(rows, cols, device=DEV) * 3).bfloat16()
    meta = F8.Fp8Meta(DEV, kind)
    meta.calibrated = True
    meta.scale.fill_(1.7)
    q, qt = F8.quantize_t(x, meta)
    lim = F8._FMAX[kind]
    want = (x.float() * 1.7).clamp(-lim, lim).to(F8._TORCH[kind]).view(torch.uint8)
    assert torch.equal(q, want) and torch.equal(qt, want.t().contiguous())
    assert abs(meta.amax.item() - x.float().abs().max().item()) < 1e-6
    q2, qt2 = F8.quantize_t(x, meta, want_q=False)
    assert q2 is None and torch.equal(qt2, qt)


def test_fp8_weight_gradient_option_on_gpu():
    from ceo_b200.ops import _lib
    from ceo_b200.ops import fp8 as F8
    torch.manual_seed(8)
    x = torch.randn(2048, 512, device=DEV).bfloat16().requires_grad_()
    w = (torch.randn(784 + 16, 512, device=DEV) * 0.03).bfloat16().requires_grad_()
    w.main_grad = torch.ones(800, 512, device=DEV)
    st = F8.Fp8Recipe(dgrad=True, wgrad=True).new_state(DEV)
    y = F8.fp8_linear(x, w, st)
    dy = (torch.randn_like(y.float()) * 1e-3).bfloat16()
    y.backward(dy)
    rw = dy.float().t() @ x.float()
    got = w.main_grad - 1
    assert 0 < (got - rw).norm() / rw.norm() < 0.08
    rx = dy.float() @ w.float()
    assert (x.grad.float() - rx).norm() / rx.norm() < 0.08
    # the same codes through an fp32 product
    dyq, dyqt = F8.quantize_t(dy, st.g_meta)
    xq, xqt = F8.quantize_t(x.detach(), st.x_meta)
    want = (dyqt.view(torch.float8_e5m2).float() @ xqt.view(torch.float8_e4m3fn).float().t()) \
        / (st.g_meta.scale * st.x_meta.scale)
    assert (got - want).norm() / want.norm() < 1e-4
    assert _lib.read_status() == 0


def test_engine_trains_with_fp8_forward_on_gpu():
    from ceo_b200.ops import _lib
    from ceo_b200.runtime.engine import TrainEngine
    from ceo_b200.utils.config import Config
    cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "smoke.yaml"))
    cfg.training.optimizer = "adamw"
    cfg.training.fp8_training = True
    cfg.model.prism.enabled = False
    eng = TrainEngine(cfg, torch.device(DEV))
    eng.fp8.dgrad = eng.fp8.wgrad = True
    ref_cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "smoke.yaml"))
    ref_cfg.training.optimizer = "adamw"
    ref_cfg.model.prism.enabled = False
    ref = TrainEngine(ref_cfg, torch.device(DEV))
    tok = torch.randint(0, cfg.model.vocab_size, (2, 129), device=DEV)
    batch = [(tok[:, :128].contiguous(), tok[:, 1:129].contiguous())]
    a = [float(eng.train_step(batch, lr=2e-3)[0]) for _ in range(4)]
    b = [float(ref.train_step(batch, lr=2e-3)[0]) for _ in range(4)]
    assert all(l == l for l in a) and a[-1] < a[0]
    assert abs(a[0] - b[0]) < 0.02 * b[0]      # same weights: fp8 forward ~ bf16 forward
    assert _lib.read_status() == 0


def test_fp8_convergence_tool_runs_both_arms(capsys):
    # the bf16 / FP8 comparison a user runs before switching fp8_training on
    from ceo_b200.utils import fp8_convergence
    cfg = os.path.join(ROOT, "configs", "smoke.yaml")
    assert fp8_convergence.main(["--config", cfg, "--steps", "6", "--global-batch", "2",
                                 "--seq-len", "128", "--every", "0"]) == 0
    import json
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["steps"] == 6 and abs(rec["loss_first"][0] - rec["loss_first"][1]) < 0.2
    assert abs(rec["rel_gap"]) < 0.05
