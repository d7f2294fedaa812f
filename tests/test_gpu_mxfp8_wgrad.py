"""MXFP8 weight-gradient GEMM (both operands MN-major, quantised along the token axis) and the whole MXFP8 MLP against
the rounding-exact PyTorch emulation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("tokens,n_out,n_in", [(512, 256, 256), (4096, 1280, 5120), (2048, 3840, 1280)])
def test_weight_gradient_gemm_matches_emulation(tokens, n_out, n_in):
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ops import mxfp8 as MX
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(3)
    dy = torch.randn(tokens, n_out, device="cuda").bfloat16()
    x = torch.randn(tokens, n_in, device="cuda").bfloat16()
    _, _, dyq, dysf = MX.quant2(dy, row=False, col=True, group_c=128)
    _, _, xq, xsf = MX.quant2(x, row=False, col=True, group_c=MX.BN_WGRAD)
    w = torch.empty(n_out, n_in, device="cuda", dtype=torch.bfloat16)
    w.main_grad = torch.full((n_out, n_in), 1.0, device="cuda")
    MX.wgrad2(dyq, dysf, xq, xsf, w)
    torch.cuda.synchronize()
    L.check_error_word()
    ref = RF.mx_qdq(dy.float(), 0).T @ RF.mx_qdq(x.float(), 0) + 1.0
    assert _rel(w.main_grad, ref) < 1e-4, _rel(w.main_grad, ref)


def test_mx_mlp_forward_backward():
    from them_bones_b200 import ops
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ops import mxfp8 as MX
    torch.manual_seed(2)
    m, c, f = 512, 256, 1024
    x = torch.randn(m, c, device="cuda").bfloat16().requires_grad_(True)
    w_fc = (torch.randn(f, c, device="cuda") * 0.06).bfloat16().requires_grad_(True)
    w_proj = (torch.randn(c, f, device="cuda") * 0.03).bfloat16().requires_grad_(True)
    res = torch.randn(m, c, device="cuda").bfloat16()
    g = torch.randn(m, c, device="cuda").bfloat16()
    y = MX.mlp(x, w_fc, w_proj, res)
    y.backward(g)
    got = (y.detach(), x.grad.clone(), w_fc.grad.clone(), w_proj.grad.clone())
    for t in (x, w_fc, w_proj):
        t.grad = None
    yr = ops._MxMlpRef.apply(x, w_fc, w_proj) + res
    yr.backward(g)
    torch.cuda.synchronize()
    L.check_error_word()
    assert _rel(got[0], yr) < 2e-2
    assert _rel(got[1], x.grad) < 6e-2 and _rel(got[2], w_fc.grad) < 6e-2 and _rel(got[3], w_proj.grad) < 6e-2
    # and the whole thing approximates the bf16 MLP
    yb = torch.relu(x.float() @ w_fc.float().T).square() @ w_proj.float().T + res.float()
    assert _rel(got[0], yb) < 6e-2


def test_mx_linear_qkv_forward_backward_into_slab():
    """The block-scaled projection for three row-adjacent weights with gradient slabs (the optimizer's layout): output,
    input gradient and the fp32 slab against the rounding-exact statement."""
    from them_bones_b200 import ops
    from them_bones_b200.ops import _lib as L
    torch.manual_seed(4)
    m, c, a = 640, 256, 256
    x = torch.randn(m, c, device="cuda").bfloat16().requires_grad_(True)
    slab = (torch.randn(3 * a, c, device="cuda") * 0.08).bfloat16()
    gslab = torch.zeros(3 * a, c, device="cuda")
    ws = []
    for j in range(3):
        w = slab[j * a:(j + 1) * a].requires_grad_(True)
        w.main_grad = gslab[j * a:(j + 1) * a]
        ws.append(w)
    g = torch.randn(m, 3 * a, device="cuda").bfloat16()
    y = ops.linear_qkv(x, *ws, precision="mxfp8")
    y.backward(g)
    torch.cuda.synchronize()
    L.check_error_word()
    assert all(w.grad is None for w in ws)                      # the gradient went into the slab
    xr = x.detach().clone().requires_grad_(True)
    wr = slab.detach().clone().requires_grad_(True)
    yr = ops._MxLinearRef.apply(xr, wr)
    yr.backward(g)
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(gslab, wr.grad) < 1e-2, _rel(gslab, wr.grad)
    # with a fused residual, and weights that are not adjacent (the gradient comes back through autograd)
    w1 = (torch.randn(c, c, device="cuda") * 0.08).bfloat16().requires_grad_(True)
    res = torch.randn(m, c, device="cuda").bfloat16()
    y1 = ops.linear(x.detach(), w1, residual=res, precision="mxfp8")
    y1.backward(torch.ones_like(y1))
    ref = ops._MxLinearRef.apply(x.detach(), w1.detach()) + res
    assert _rel(y1, ref) < 1e-2 and w1.grad is not None


def test_mx_experts_batched_forward_backward():
    """Grouped experts on the batched block-scaled GEMMs against the per-expert rounding-exact statement."""
    from them_bones_b200 import ops
    from them_bones_b200.ops import _lib as L
    torch.manual_seed(5)
    e, rows, d, f = 2, 384, 256, 512
    xs = torch.randn(e * rows, d, device="cuda").bfloat16().requires_grad_(True)
    w_fc = (torch.randn(e, f, d, device="cuda") * 0.06).bfloat16().requires_grad_(True)
    w_proj = (torch.randn(e, d, f, device="cuda") * 0.04).bfloat16().requires_grad_(True)
    g = torch.randn(e * rows, d, device="cuda").bfloat16()
    y = ops.moe_experts(xs, w_fc, w_proj, "mxfp8")
    y.backward(g)
    torch.cuda.synchronize()
    L.check_error_word()
    assert ops.COUNTS["moe_experts_mxfp8"] > 0
    got = (y.detach(), xs.grad.clone(), w_fc.grad.clone(), w_proj.grad.clone())
    for t in (xs, w_fc, w_proj):
        t.grad = None
    ops.set_reference_path(True)
    try:
        yr = ops.moe_experts(xs, w_fc, w_proj, "mxfp8")
        yr.backward(g)
    finally:
        ops.set_reference_path(False)
    assert _rel(got[0], yr) < 2e-2
    assert _rel(got[1], xs.grad) < 6e-2 and _rel(got[2], w_fc.grad) < 6e-2 and _rel(got[3], w_proj.grad) < 6e-2
