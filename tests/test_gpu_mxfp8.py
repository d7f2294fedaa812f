"""MXFP8 quantiser and block-scaled tcgen05 GEMM against the rounding-exact PyTorch emulation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def _unpack_sf(sf, rows, k):
    """Scale chunks -> [rows, k/32] biased exponents."""
    kb = k // 128
    groups = (rows + 127) // 128
    t = sf.view(groups, kb, 32, 4, 4)                 # [g, kb, r%32, (r%128)/32, ksub]
    t = t.permute(0, 3, 2, 1, 4).reshape(groups * 128, kb * 4)
    return t[:rows]


def test_quantiser_matches_emulation():
    from them_bones_b200.ops import mxfp8 as MX
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(0)
    x = (torch.randn(300, 512, device="cuda") * torch.logspace(-4, 2, 300, device="cuda")[:, None]).bfloat16()
    x[5, 64:96] = 0
    q, sf = MX.quantize(x)
    qr, er = RF.mx_quantize(x.float(), -1)
    torch.cuda.synchronize()
    assert torch.equal(_unpack_sf(sf, 300, 512), er)
    assert torch.equal(q.view(torch.float8_e4m3fn).float(), qr.float())


@pytest.mark.parametrize("m,n,k", [(128, 160, 128), (256, 320, 512), (384, 1280, 1280), (1000, 5120, 1280)])
def test_mx_gemm_matches_emulation(m, n, k):
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ops import mxfp8 as MX
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(1)
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    y = MX.linear(x, w)
    torch.cuda.synchronize()
    L.check_error_word()
    ref = RF.mx_qdq(x.float(), -1) @ RF.mx_qdq(w.float(), -1).T
    assert _rel(y, ref) < 5e-3, _rel(y, ref)                    # bf16 output rounding only
    assert _rel(y, x.float() @ w.float().T) < 6e-2             # and close to the unquantised product


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
