"""FP8 recipe on CPU: the quantiser against the bit-exact host codec, delayed scaling against
the host ``ScaleFactor`` (dtype.zig:85-128), the Linear against fp32, and a training run."""
import os

import numpy as np
import torch

from ceo_b200.ops import fp8 as F8
from ceo_b200.utils import dtypes as DT

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_quantize_matches_host_codec_and_tracks_amax():
    torch.manual_seed(0)
    x = torch.randn(4096) * 5
    for kind, dt in ((F8.E4M3, DT.DType.fp8_e4m3), (F8.E5M2, DT.DType.fp8_e5m2)):
        meta = F8.Fp8Meta("cpu", kind)
        meta.calibrated = True
        meta.scale[0] = 3.0
        q = F8.quantize(x, meta)
        lim = 448.0 if kind == F8.E4M3 else 57344.0
        want = DT.encode(np.clip(x.numpy() * 3.0, -lim, lim), dt)
        assert np.array_equal(q.numpy(), np.asarray(want, dtype=np.uint8))
        assert abs(float(meta.amax) - float(x.abs().max())) < 1e-6


def test_delayed_scaling_matches_scale_factor():
    meta = F8.Fp8Meta("cpu", F8.E4M3, history=4, margin=1)
    ref = DT.ScaleFactor(DT.DType.fp8_e4m3, history=4, margin=1)
    for amax in (2.0, 7.5, 0.3, 0.1, 0.2, 0.05, 0.01):
        meta.amax[0] = amax
        meta.update()
        ref.update(amax)
        assert abs(float(meta.scale) - ref.scale) < 1e-4 * ref.scale
        assert float(meta.amax) == 0.0


def test_first_use_calibrates_the_scale():
    x = torch.randn(64, 32) * 0.02
    meta = F8.Fp8Meta("cpu")
    q = F8.quantize(x, meta)
    assert meta.calibrated
    assert abs(float(meta.scale) - 448.0 / float(x.abs().max())) < 1e-2 * float(meta.scale)
    back = q.view(torch.float8_e4m3fn).float() / meta.scale
    assert (back - x).abs().max() < 0.07 * x.abs().max()


def test_fp8_linear_forward_close_and_backward_is_the_plain_linear():
    torch.manual_seed(1)
    x = torch.randn(48, 64, requires_grad=True)
    w = (torch.randn(32, 64) * 0.05).requires_grad_()
    res = torch.randn(48, 32, requires_grad=True)
    rec = F8.Fp8Recipe()
    st = rec.new_state("cpu")
    y = F8.fp8_linear(x, w, st, res)
    ref = x @ w.t() + res
    assert (y - ref).norm() / ref.norm() < 0.05
    dy = torch.randn_like(y)
    gx, gw, gr = torch.autograd.grad(y, (x, w, res), dy)
    rx, rw, rr = torch.autograd.grad(ref, (x, w, res), dy)
    assert torch.allclose(gx, rx, atol=1e-5) and torch.allclose(gw, rw, atol=1e-4)
    assert torch.equal(gr, rr)
    # the quantised weight is reused until the recipe steps
    wq = st.wq
    F8.fp8_linear(x, w, st)
    assert st.wq is wq
    rec.step()
    F8.fp8_linear(x, w, st)
    assert st.wq is not wq


def test_fp8_data_gradient_option():
    torch.manual_seed(2)
    x = torch.randn(40, 64, requires_grad=True)
    w = (torch.randn(48, 64) * 0.05).requires_grad_()
    rec = F8.Fp8Recipe(dgrad=True)
    st = rec.new_state("cpu")
    y = F8.fp8_linear(x, w, st)
    dy = torch.randn_like(y) * 1e-3
    gx, gw = torch.autograd.grad(y, (x, w), dy)
    rx, rw = dy @ w, dy.t() @ x
    assert (gx - rx).norm() / rx.norm() < 0.08      # e5m2 dy x e4m3 W^T
    assert (gx - rx).norm() > 0                     # and it did go through the 8-bit path
    assert torch.allclose(gw, rw, atol=1e-6)        # the weight gradient stays exact
    assert st.g_meta.calibrated and st.wtq.shape == (64, 48)


def test_fp8_weight_gradient_option():
    torch.manual_seed(4)
    x = torch.randn(64, 48, requires_grad=True)
    w = (torch.randn(32, 48) * 0.05).requires_grad_()
    w.main_grad = torch.ones(32, 48)
    rec = F8.Fp8Recipe(dgrad=True, wgrad=True)
    st = rec.new_state("cpu")
    y = F8.fp8_linear(x, w, st)
    assert y.grad_fn.saved_tensors[0].dtype == torch.uint8      # q(x)^T, not the activation
    assert y.grad_fn.saved_tensors[0].shape == (48, 64)
    dy = torch.randn_like(y) * 1e-2
    y.backward(dy)
    gx = x.grad
    rw = (dy.t() @ x).detach()
    got = w.main_grad - 1
    assert 0 < (got - rw).norm() / rw.norm() < 0.08
    assert (gx - (dy @ w).detach()).norm() / (dy @ w).norm() < 0.08
    q, qt = F8.quantize_t(torch.randn(32, 16), F8.Fp8Meta("cpu"))
    assert torch.equal(q.t(), qt)


def test_engine_trains_with_fp8_forward():
    from ceo_b200.runtime.engine import TrainEngine
    from ceo_b200.utils.config import Config
    cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "smoke_cpu.yaml"))
    cfg.training.fp8_training = True
    cfg.training.optimizer = "adamw"
    eng = TrainEngine(cfg, "cpu", seed=0)
    assert eng.fp8 is not None and len(eng.fp8.states) == 4 * cfg.model.num_layers
    torch.manual_seed(0)
    tok = torch.randint(0, cfg.model.vocab_size, (2, 65))
    batch = [(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())]
    losses = [float(eng.train_step(batch, lr=3e-3)[0]) for _ in range(5)]
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    assert eng.fp8.step_id == 5 and not eng.fp8.wgrad
    cfg.training.fp8_gradients = True
    eng2 = TrainEngine(cfg, "cpu", seed=0)
    assert eng2.fp8.dgrad and eng2.fp8.wgrad
    l2 = [float(eng2.train_step(batch, lr=3e-3)[0]) for _ in range(5)]
    assert all(l == l for l in l2) and l2[-1] < l2[0]


def test_recipe_state_roundtrip():
    torch.manual_seed(9)
    rec = F8.Fp8Recipe(dgrad=True)
    st = rec.new_state("cpu")
    x = torch.randn(32, 32, requires_grad=True)
    w = (torch.randn(16, 32) * 0.1).requires_grad_()
    for _ in range(3):
        F8.fp8_linear(x * (1 + _), w, st).sum().backward()
        rec.step()
    d = rec.state_dict()
    import json
    d = json.loads(json.dumps(d))
    rec2 = F8.Fp8Recipe(dgrad=True)
    st2 = rec2.new_state("cpu")
    rec2.load_state_dict(d)
    for a, b in ((st.x_meta, st2.x_meta), (st.w_meta, st2.w_meta), (st.g_meta, st2.g_meta)):
        assert float(a.scale) == float(b.scale) and torch.equal(a.history, b.history)
        assert int(a.cursor) == int(b.cursor) and a.calibrated == b.calibrated
    y1 = F8.fp8_linear(x, w, st)
    y2 = F8.fp8_linear(x, w, st2)
    assert torch.equal(y1, y2)
