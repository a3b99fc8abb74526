"""Chunked EFLA CUDA kernels against the token-sequential fp32 oracle."""
import pytest
import torch

from ceo_b200.ops import _lib, efla, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _inputs(B, T, H, d, seed=0, fused=False):
    g = torch.Generator(device=DEV).manual_seed(seed)
    if fused:  # q,k,v as column slices of one (B,T,3*H*d) buffer, like a fused QKV GEMM output
        qkv = torch.randn(B, T, 3, H, d, device=DEV, generator=g)
        qkv = qkv / qkv.norm(dim=-1, keepdim=True)
        qkv[:, :, 2] = torch.randn(B, T, H, d, device=DEV, generator=g)
        qkv = qkv.to(torch.bfloat16)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    else:
        q = torch.randn(B, T, H, d, device=DEV, generator=g)
        k = torch.randn(B, T, H, d, device=DEV, generator=g)
        q = (q / q.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
        k = (k / k.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
        v = torch.randn(B, T, H, d, device=DEV, generator=g).to(torch.bfloat16)
    beta = torch.sigmoid(torch.randn(B, T, H, device=DEV, generator=g))
    alpha = ref.efla_coefficient(beta, k.float().pow(2).sum(-1))
    return q, k, v, alpha


@pytest.mark.parametrize("B,T,H,d", [(1, 64, 1, 64), (2, 256, 3, 64), (1, 128, 2, 128),
                                     (2, 512, 4, 128)])
@pytest.mark.parametrize("fused", [False, True])
def test_efla_forward(B, T, H, d, fused):
    q, k, v, alpha = _inputs(B, T, H, d, fused=fused)
    o, s = efla.delta_rule(q, k, v, alpha)
    torch.cuda.synchronize()
    o_ref, s_ref = ref.delta_rule_sequential(q, k, v, alpha)
    assert _rel(o, o_ref) < 1.5e-2
    assert _rel(s, s_ref) < 1.5e-2
    assert _lib.read_status() == 0


@pytest.mark.parametrize("B,T,H,d", [(1, 64, 1, 64), (2, 256, 2, 64), (1, 192, 2, 128),
                                     (2, 256, 3, 128)])
@pytest.mark.parametrize("with_state", [False, True])
def test_efla_backward(B, T, H, d, with_state):
    q, k, v, alpha = _inputs(B, T, H, d, seed=1)
    g = torch.Generator(device=DEV).manual_seed(2)
    do = torch.randn(B, T, H, d, device=DEV, generator=g).to(torch.bfloat16)
    s0 = 0.1 * torch.randn(B, H, d, d, device=DEV, generator=g) if with_state else None
    dsf = 0.05 * torch.randn(B, H, d, d, device=DEV, generator=g) if with_state else None

    leaves = [t.detach().clone().requires_grad_() for t in (q, k, v, alpha)]
    s0k = s0.clone().requires_grad_() if with_state else None
    o, s = efla.delta_rule(*leaves, s0k)
    loss = (o.float() * do.float()).sum()
    if with_state:
        loss = loss + (s * dsf).sum()
    loss.backward()

    rl = [t.detach().float().requires_grad_() for t in (q, k, v, alpha)]
    s0r = s0.clone().requires_grad_() if with_state else None
    o_r, s_r = ref.delta_rule_chunked(*rl, s0r)
    loss_r = (o_r * do.float()).sum()
    if with_state:
        loss_r = loss_r + (s_r * dsf).sum()
    loss_r.backward()
    names = ["dq", "dk", "dv", "dalpha"]
    for nme, a, b in zip(names, leaves, rl):
        assert _rel(a.grad, b.grad) < 3e-2, (nme, _rel(a.grad, b.grad))
    if with_state:
        assert _rel(s0k.grad, s0r.grad) < 3e-2
    assert _lib.read_status() == 0


def test_efla_attention_reference_form():
    # the reference's special case: q = k, one scalar beta, coefficient from ||k||^2
    B, T, H, d = 1, 128, 2, 64
    g = torch.Generator(device=DEV).manual_seed(5)
    k = (0.3 * torch.randn(B, T, H, d, device=DEV, generator=g)).to(torch.bfloat16)
    v = torch.randn(B, T, H, d, device=DEV, generator=g).to(torch.bfloat16)
    o, s = efla.efla_attention(k, k, v, torch.tensor(1.0, device=DEV), normalize_qk=False)
    o_ref, s_ref = ref.efla_reference_form(k, v, 1.0)
    assert _rel(o, o_ref) < 1.5e-2 and _rel(s, s_ref) < 1.5e-2


@pytest.mark.parametrize("P,normalize,scalar_beta", [(3, True, False), (2, False, True),
                                                     (3, False, False), (2, True, False)])
def test_efla_qkv_fused(P, normalize, scalar_beta):
    B, T, H, d = 2, 128, 2, 128
    g = torch.Generator(device=DEV).manual_seed(7)
    qkv = (0.5 * torch.randn(B, T, P, H, d, device=DEV, generator=g)).to(torch.bfloat16)
    if not normalize:
        qkv[:, :, :P - 1] *= 0.15
    beta0 = torch.tensor([0.8], device=DEV) if scalar_beta else \
        torch.sigmoid(torch.randn(B, T, H, device=DEV, generator=g))
    do = torch.randn(B, T, H, d, device=DEV, generator=g).to(torch.bfloat16)

    a = qkv.clone().requires_grad_()
    ba = beta0.clone().requires_grad_()
    o, _ = efla.efla_qkv(a, ba, normalize)
    (o.float() * do.float()).sum().backward()

    b = qkv.float().requires_grad_()
    bb = beta0.clone().requires_grad_()
    q = b[:, :, 0]
    k = b[:, :, 1] if P == 3 else b[:, :, 0]
    if normalize:
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6)
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        alpha = -torch.expm1(-bb.expand(B, T, H))
    else:
        alpha = ref.efla_coefficient(bb.expand(B, T, H), k.pow(2).sum(-1))
    o_r, _ = ref.delta_rule_chunked(q, k, b[:, :, P - 1], alpha)
    (o_r * do.float()).sum().backward()
    assert _rel(o, o_r) < 2e-2
    assert _rel(a.grad, b.grad) < 4e-2, _rel(a.grad, b.grad)
    assert _rel(ba.grad, bb.grad) < 4e-2, _rel(ba.grad, bb.grad)


@pytest.mark.parametrize("P,normalize", [(3, True), (2, False)])
def test_efla_proj_with_beta_logits_in_projection(P, normalize):
    B, T, H, d = 2, 128, 4, 64
    g = torch.Generator(device=DEV).manual_seed(11)
    N = P * H * d + 8
    proj = (0.4 * torch.randn(B, T, N, device=DEV, generator=g)).to(torch.bfloat16)
    if not normalize:
        proj[..., :(P - 1) * H * d] *= 0.2
    do = torch.randn(B, T, H, d, device=DEV, generator=g).to(torch.bfloat16)
    a = proj.clone().requires_grad_()
    o, _ = efla.efla_proj(a, P, H, d, normalize)
    (o.float() * do.float()).sum().backward()
    b = proj.float().requires_grad_()
    o_r, _ = efla.efla_proj(b.cpu().to(DEV) if False else b, P, H, d, normalize) \
        if False else (None, None)
    hd = H * d
    qkv = b[..., :P * hd].reshape(B, T, P, H, d)
    beta = torch.sigmoid(b[..., P * hd:P * hd + H])
    q = qkv[:, :, 0]
    k = qkv[:, :, 1] if P == 3 else qkv[:, :, 0]
    if normalize:
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6)
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        alpha = -torch.expm1(-beta)
    else:
        alpha = ref.efla_coefficient(beta, k.pow(2).sum(-1))
    o_r, _ = ref.delta_rule_chunked(q, k, qkv[:, :, P - 1], alpha)
    (o_r * do.float()).sum().backward()
    assert _rel(o, o_r) < 2e-2
    assert _rel(a.grad[..., :P * hd], b.grad[..., :P * hd]) < 4e-2
    assert _rel(a.grad[..., P * hd:P * hd + H], b.grad[..., P * hd:P * hd + H]) < 5e-2
    assert float(a.grad[..., P * hd + H:].abs().max()) == 0.0


@pytest.mark.parametrize("B,T,H,d", [(2, 256, 2, 64), (2, 320, 2, 128)])
def test_efla_document_resets_forward_and_backward(B, T, H, d):
    """Chunk-aligned state resets (packed documents): kernels against the chunked oracle."""
    q, k, v, alpha = _inputs(B, T, H, d, seed=3)
    n = T // 64
    g = torch.Generator(device=DEV).manual_seed(4)
    do = torch.randn(B, T, H, d, device=DEV, generator=g).to(torch.bfloat16)
    resets = torch.zeros(B, n, dtype=torch.bool, device=DEV)
    resets[0, 0] = resets[0, 2] = resets[1, 1] = resets[1, n - 1] = True
    s0 = 0.1 * torch.randn(B, H, d, d, device=DEV, generator=g)
    dsf = 0.05 * torch.randn(B, H, d, d, device=DEV, generator=g)

    leaves = [t.detach().clone().requires_grad_() for t in (q, k, v, alpha)]
    s0k = s0.clone().requires_grad_()
    o, s = efla.delta_rule(*leaves, s0k, resets=resets)
    ((o.float() * do.float()).sum() + (s * dsf).sum()).backward()

    rl = [t.detach().float().requires_grad_() for t in (q, k, v, alpha)]
    s0r = s0.clone().requires_grad_()
    o_r, s_r = ref.delta_rule_chunked(*rl, s0r, 64, resets)
    ((o_r * do.float()).sum() + (s_r * dsf).sum()).backward()
    assert _rel(o, o_r) < 2e-2 and _rel(s, s_r) < 2e-2
    for nme, a, b in zip(["dq", "dk", "dv", "dalpha"], leaves, rl):
        assert _rel(a.grad, b.grad) < 3e-2, (nme, _rel(a.grad, b.grad))
    # row 0 resets at chunk 0: its initial state has no effect, so no gradient either
    assert s0k.grad[0].abs().max().item() == 0.0
    assert _rel(s0k.grad[1], s0r.grad[1]) < 3e-2
    assert _lib.read_status() == 0


@pytest.mark.parametrize("B,T,H", [(1, 128, 2), (2, 512, 4)])
def test_efla_output_kernel_on_tcgen05_matches_oracle(B, T, H):
    """The tcgen05 variant of the output kernel (off by default) against the fp32 oracle."""
    q, k, v, alpha = _inputs(B, T, H, 128, seed=5)
    L = _lib.lib()
    L.ceo_efla_set_tcgen05(1)
    try:
        o, s = efla.delta_rule(q, k, v, alpha)
        torch.cuda.synchronize()
    finally:
        L.ceo_efla_set_tcgen05(0)
    o_r, s_r = ref.delta_rule_sequential(q, k, v, alpha)
    assert _rel(o, o_r) < 2e-2 and _rel(s, s_r) < 2e-2
    assert _lib.read_status() == 0
