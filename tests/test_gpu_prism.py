"""Single-GPU numerics of the PRISM kernels, dropout and softmax(dim) against fp32 PyTorch."""
import os

import pytest
import torch

from ceo_b200.models.model import EflaLM
from ceo_b200.ops import nn as K
from ceo_b200.ops import prism as P
from ceo_b200.utils.config import Config

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_prism_gate_forward_backward():
    torch.manual_seed(0)
    rp, p, bt = ((torch.randn(512, 128, device=DEV)).bfloat16().requires_grad_() for _ in range(3))
    bd = P.gate(rp, p, bt)
    want = P.gate_reference(rp, p, bt)
    assert _rel(bd, want) < 5e-3
    g = torch.randn_like(bd)
    bd.backward(g)
    ref = [t.detach().float().requires_grad_() for t in (rp, p, bt)]
    P.gate_reference(*ref).backward(g.float())
    for a, b in zip((rp, p, bt), ref):
        assert _rel(a.grad, b.grad) < 8e-3


def test_prism_update_and_state():
    torch.manual_seed(1)
    c, r, out = (torch.randn(64, 256, device=DEV).bfloat16().requires_grad_() for _ in range(3))
    r2, o2 = P.update(c, r, out, 0.5)
    assert _rel(r2, r.float() - c.float()) < 5e-3 and _rel(o2, out.float() + 0.5 * c.float()) < 5e-3
    (r2.float().sum() * 2 + o2.float().sum()).backward()
    assert torch.allclose(c.grad.float(), torch.full_like(c, 0.5 - 2.0).float())
    assert torch.allclose(r.grad.float(), torch.full_like(r, 2.0).float())
    for hd in (32, 64, 128):
        L, B, T = 3, 2, 96
        bd = torch.randn(L, B, T, hd, device=DEV).bfloat16()
        k = (torch.randn(L, B, T, hd, device=DEV) * 0.2).bfloat16()
        bt1 = torch.randn(B, T, hd, device=DEV).bfloat16()
        s0 = torch.randn(B, hd, hd, device=DEV)
        got = P.state(bd, k, bt1, s0, 0.95)
        want = P.state_reference(bd.cpu(), k.cpu(), bt1.cpu(), s0.cpu(), 0.95)
        assert _rel(got.cpu(), want) < 1e-4, hd
        assert _rel(P.state(bd, k, bt1, None, 0.95).cpu(),
                    P.state_reference(bd.cpu(), k.cpu(), bt1.cpu(), None, 0.95)) < 1e-4


def test_model_with_prism_trains_and_decodes():
    cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "efla_340m.yaml"))
    m = cfg.model
    m.num_layers, m.vocab_size, m.hidden_dim, m.num_heads, m.intermediate_dim = 2, 1024, 256, 4, 512
    m.prism.enabled, m.prism.num_iterations, m.prism.shortconv_window = True, 2, 8
    model = EflaLM(m, DEV, seed=0)
    tok = torch.randint(0, m.vocab_size, (2, 128), device=DEV)
    loss = model(tok, tok)
    loss.backward()
    assert torch.isfinite(loss) and all(p.grad is not None for n, p in model.named_parameters()
                                        if "prism" in n)
    model.eval()
    with torch.no_grad():
        logits = model(tok[:, :64])
        states = model.new_states(2)
        step = torch.stack([model.decode_step(tok[:, t], states) for t in range(64)], dim=1)
    assert _rel(step, logits) < 3e-2
    assert states.prism[0]["state"].abs().sum() > 0


def test_dropout_kernel_matches_hash_mask_and_backward():
    x = torch.randn(1001, 77, device=DEV).bfloat16().requires_grad_()   # odd size: tail path
    y = K.dropout(x, 0.2, seed=123)
    keep = K.dropout_keep_mask(x.numel(), 0.2, 123, DEV).view(x.shape)
    want = torch.where(keep, x.float() / 0.8, torch.zeros_like(x, dtype=torch.float32))
    assert _rel(y, want) < 4e-3 and torch.equal(y == 0, ~keep | (x == 0))
    y.backward(torch.ones_like(y))
    assert _rel(x.grad, keep.float() / 0.8) < 4e-3
    assert abs(keep.float().mean().item() - 0.8) < 0.01


def test_softmax_over_any_dimension():
    z = torch.randn(6, 33, 20, device=DEV)
    for dim in (0, 1, 2):
        assert torch.allclose(K.softmax(z, dim), torch.softmax(z, dim), atol=1e-5)


def test_embedding_and_decode_accept_strided_ids():
    """A column of a (B, T) id tensor is a strided view: the kernels must not read it as if it
    were dense (decode_step receives exactly such views)."""
    table = torch.randn(500, 128, device=DEV).bfloat16()
    ids = torch.randint(0, 500, (4, 32), device=DEV)
    assert torch.equal(K.embedding(ids[:, 7], table), table[ids[:, 7]])
    cfg = Config.parse_from_file(os.path.join(ROOT, "configs", "efla_340m.yaml"))
    m = cfg.model
    m.num_layers, m.vocab_size, m.hidden_dim, m.num_heads, m.intermediate_dim = 2, 1024, 256, 4, 512
    model = EflaLM(m, DEV, seed=0).eval()
    tok = torch.randint(0, m.vocab_size, (3, 64), device=DEV)
    with torch.no_grad():
        logits = model(tok)
        states = model.new_states(3)
        step = torch.stack([model.decode_step(tok[:, t], states) for t in range(64)], dim=1)
    for b in range(3):
        assert _rel(step[b], logits[b]) < 3e-2, b
