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
