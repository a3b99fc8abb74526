"""Single-GPU numerics: each CUDA kernel against the fp32 PyTorch oracle of the same op."""
import pytest
import torch

from ceo_b200.ops import _lib, matmul as gemm_mod, nn as nn_ops, reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    torch.cuda.synchronize()
    assert _lib.read_status() == 0, "a kernel's bounded wait ran out"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 128), (300, 520, 200),
                                   (1024, 768, 2048), (4096, 6144, 2048)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    if a_mn and M % 8:
        M = (M + 7) // 8 * 8
    a = _rand(K, M) if a_mn else _rand(M, K)
    b = _rand(K, N) if b_mn else _rand(N, K)
    out = gemm_mod.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    want = af @ bf
    assert _rel(out, want) < 2e-5
    out16 = gemm_mod.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    assert out16.dtype == torch.bfloat16 and _rel(out16, want) < 5e-3


def test_gemm_epilogues():
    torch.manual_seed(1)
    M, N, K = 512, 1024, 256
    a, b = _rand(M, K), _rand(N, K)
    res = _rand(M, N)
    bias = torch.randn(N, device=DEV)
    want = 0.5 * (a.float() @ b.float().t()) + bias + res.float()
    out = gemm_mod.gemm(a, b, alpha=0.5, bias=bias, residual=res, out_dtype=torch.float32)
    assert _rel(out, want) < 2e-5
    acc = torch.randn(M, N, device=DEV)
    acc0 = acc.clone()
    gemm_mod.gemm(a, b, out=acc, accumulate=True)
    assert _rel(acc, acc0 + a.float() @ b.float().t()) < 2e-5
    acc16 = _rand(M, N)
    acc16_0 = acc16.clone()
    gemm_mod.gemm(a, b, out=acc16, accumulate=True)
    assert _rel(acc16, acc16_0.float() + a.float() @ b.float().t()) < 5e-3


def test_gemm_batched_and_strided():
    torch.manual_seed(2)
    nb, M, N, K = 5, 192, 320, 128
    a, b = _rand(nb, M, K), _rand(nb, N, K)
    out = gemm_mod.gemm(a, b, out_dtype=torch.float32)
    assert _rel(out, a.float() @ b.float().transpose(1, 2)) < 2e-5
    # strided views: columns of a wider matrix
    wide = _rand(M, 3 * K)
    out2 = gemm_mod.gemm(wide[:, K:2 * K], b[0], out_dtype=torch.float32)
    assert _rel(out2, wide[:, K:2 * K].float() @ b[0].float().t()) < 2e-5


def test_linear_autograd():
    torch.manual_seed(3)
    x = _rand(4, 96, 256).requires_grad_()
    w = _rand(384, 256, scale=0.05).requires_grad_()
    y = gemm_mod.linear(x, w)
    dy = _rand(4, 96, 384)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    (xr @ wr.t()).backward(dy.float())
    assert _rel(y, xr @ wr.t()) < 5e-3
    assert _rel(x.grad, xr.grad) < 5e-3 and _rel(w.grad, wr.grad) < 5e-3
    # fp32 main_grad accumulation fused in the wgrad epilogue
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.zeros(384, 256, device=DEV)
    for _ in range(2):
        gemm_mod.linear(x.detach(), w2).backward(dy)
    assert w2.grad is None and _rel(w2.main_grad, 2 * wr.grad) < 1e-4


@pytest.mark.parametrize("rows,D", [(64, 256), (1000, 2048), (33, 4096), (7, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(rows, D, with_res):
    torch.manual_seed(4)
    x = _rand(rows, D).requires_grad_()
    r = _rand(rows, D).requires_grad_() if with_res else None
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    y, h = nn_ops.rmsnorm(x, w, 1e-6, r)
    dy, dh = _rand(rows, D), _rand(rows, D)
    (y.float() * dy.float()).sum().backward() if not with_res else \
        ((y.float() * dy.float()).sum() + (h.float() * dh.float()).sum()).backward()
    xr = x.detach().float().requires_grad_()
    rr = r.detach().float().requires_grad_() if with_res else None
    wr = w.detach().float().requires_grad_()
    hr = xr + rr if with_res else xr
    if with_res:
        hr = hr + (hr.to(torch.bfloat16).float() - hr).detach()  # stored h is bf16
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    loss = (yr * dy.float()).sum() + ((hr * dh.float()).sum() if with_res else 0)
    loss.backward()
    assert _rel(y, yr) < 6e-3
    assert _rel(x.grad, xr.grad) < 8e-3
    assert _rel(w.grad, wr.grad) < 8e-3
    if with_res:
        assert _rel(r.grad, rr.grad) < 8e-3


def test_layernorm():
    torch.manual_seed(5)
    rows, D = 300, 1024
    x = _rand(rows, D).requires_grad_()
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    b = (0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    y = nn_ops.layernorm(x, w, b)
    dy = _rand(rows, D)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (D,), wr, br, 1e-5)
    yr.backward(dy.float())
    assert _rel(y, yr) < 6e-3 and _rel(x.grad, xr.grad) < 8e-3
    assert _rel(w.grad, wr.grad) < 8e-3 and _rel(b.grad, br.grad) < 8e-3


def test_swiglu_and_activations():
    torch.manual_seed(6)
    gu = _rand(130, 2 * 352).requires_grad_()
    out = nn_ops.swiglu(gu)
    d = _rand(130, 352)
    out.backward(d)
    gr = gu.detach().float().requires_grad_()
    g, u = gr.chunk(2, -1)
    want = torch.nn.functional.silu(g) * u
    want.backward(d.float())
    assert _rel(out, want) < 6e-3 and _rel(gu.grad, gr.grad) < 8e-3
    # interleaved layout (column 2j = gate_j, 2j+1 = up_j)
    gi = _rand(130, 2 * 352).requires_grad_()
    oi = nn_ops.swiglu(gi, interleaved=True)
    oi.backward(d)
    gr2 = gi.detach().float().requires_grad_()
    want2 = torch.nn.functional.silu(gr2[:, 0::2]) * gr2[:, 1::2]
    want2.backward(d.float())
    assert _rel(oi, want2) < 6e-3 and _rel(gi.grad, gr2.grad) < 8e-3
    for kind in ("gelu", "gelu_erf", "silu", "relu"):
        x = _rand(64, 512).requires_grad_()
        y = nn_ops.activation(x, kind)
        y.backward(d.new_ones(64, 512))
        xr = x.detach().float().requires_grad_()
        yr = ref.activation(xr, kind)
        yr.sum().backward()
        assert _rel(y, yr) < 6e-3 and _rel(x.grad, xr.grad) < 8e-3, kind
    z = torch.randn(37, 1000, device=DEV) * 4 - 3
    assert _rel(nn_ops.softmax(z), torch.softmax(z, -1)) < 1e-5


@pytest.mark.parametrize("ls", [0.0, 0.1])
def test_linear_cross_entropy(ls):
    torch.manual_seed(7)
    rows, D, V = 700, 256, 1000
    x = _rand(rows, D).requires_grad_()
    w = _rand(V, D, scale=0.05).requires_grad_()
    t = torch.randint(0, V, (rows,), device=DEV)
    t[::13] = -100
    loss = nn_ops.linear_cross_entropy(x, w, t, ls, -100, chunk_rows=256)
    loss.backward()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = ref.linear_cross_entropy(xr, wr, t, ls, -100)
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-3 * abs(lr.item())
    assert _rel(x.grad, xr.grad) < 1.5e-2 and _rel(w.grad, wr.grad) < 1.5e-2
    rows_l = nn_ops.cross_entropy_rows((xr @ wr.t()).detach(), t, ls)
    assert _rel(rows_l, ref.cross_entropy_rows(xr @ wr.t(), t, ls)) < 1e-5


def test_embedding():
    torch.manual_seed(8)
    V, D = 500, 256
    table = _rand(V, D).requires_grad_()
    ids = torch.randint(0, V, (4, 77), device=DEV)
    ids[0, :10] = 3  # repeated rows exercise the atomic accumulation
    out = nn_ops.embedding(ids, table)
    dy = _rand(4, 77, D)
    out.backward(dy)
    tr = table.detach().float().requires_grad_()
    torch.nn.functional.embedding(ids, tr).backward(dy.float())
    assert torch.equal(out, table.detach()[ids])
    assert _rel(table.grad, tr.grad) < 8e-3


@pytest.mark.parametrize("M,D,F", [(300, 256, 352), (256, 512, 1024), (64, 128, 96)])
def test_swiglu_mlp_fused_epilogues_match_fp32(M, D, F):
    """The MLP with SiLU(gate) * up in the gate/up GEMM's epilogue and the SwiGLU backward in
    the down projection's data-gradient epilogue, against the same math in fp32."""
    from ceo_b200.ops.matmul import swiglu_mlp
    torch.manual_seed(9)
    x = _rand(M, D).requires_grad_()
    w_up = (_rand(2 * F, D) * 0.2).requires_grad_()     # interleaved rows
    w_down = (_rand(D, F) * 0.2).requires_grad_()
    res = _rand(M, D).requires_grad_()
    y = swiglu_mlp(x, w_up, w_down, res)
    dy = _rand(M, D)
    y.backward(dy)
    xr, wur, wdr, rr = (t.detach().float().requires_grad_() for t in (x, w_up, w_down, res))
    gu = xr @ wur.t()
    act = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]
    yr = act @ wdr.t() + rr
    yr.backward(dy.float())
    assert _rel(y, yr) < 8e-3
    for a, b, name in ((x, xr, "dx"), (w_up, wur, "dw_up"), (w_down, wdr, "dw_down"),
                       (res, rr, "dres")):
        assert _rel(a.grad, b.grad) < 1.5e-2, name
    # the unfused path (three ops) gives the same function
    from ceo_b200.ops.matmul import linear
    y2 = linear(nn_ops.swiglu(linear(x.detach(), w_up.detach()), interleaved=True),
                w_down.detach(), res.detach())
    assert _rel(y2, y) < 8e-3
    assert _lib.read_status() == 0
