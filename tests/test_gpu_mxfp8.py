"""MXFP8 quantiser and block-scaled tcgen05 GEMM against the rounding-exact PyTorch emulation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def _unpack_sf2(sf, rows, k, group):
    """Scale chunks of an operand with ``group`` rows per tile -> [rows, ceil(k/32)] biased exponents."""
    kb = -(-k // 128)
    groups = -(-rows // group)
    chunks = -(-group // 128)
    t = sf.view(groups, kb, chunks, 32, 4, 4)          # [g, kb, chunk, r%32, (r%128)/32, ksub]
    t = t.permute(0, 2, 4, 3, 1, 5).reshape(groups, chunks * 128, kb * 4)[:, :group]
    return t.reshape(groups * group, kb * 4)[:rows, :-(-k // 32)]


def _deq(q, e, axis):
    from them_bones_b200.ref import functional as RF
    return RF.mx_dequantize(q.view(torch.float8_e4m3fn), e, axis)


@pytest.mark.parametrize("r,c", [(320, 512), (1000, 1280), (4096 + 17, 384)])
@pytest.mark.parametrize("group_r,group_c", [(128, 128), (224, 256)])
def test_dual_quantiser_matches_emulation(group_r, group_c, r, c):
    """Whole and ragged row counts (a last block of fewer than 32 rows is quantised as a block of its own)."""
    from them_bones_b200.ops import mxfp8 as MX
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(0)
    x = (torch.randn(r, c, device="cuda") * torch.logspace(-4, 2, r, device="cuda")[:, None]).bfloat16()
    x[5, 64:96] = 0
    x[32:64, 7] = 0
    qr, sfr, qc, sfc = MX.quant2(x, col=True, group_r=group_r, group_c=group_c)
    rr, er = RF.mx_quantize(x.float(), -1)
    xp = torch.nn.functional.pad(x.float(), (0, 0, 0, -r % 32))
    rc, ec = RF.mx_quantize(xp, 0)                              # scales [c, ceil(r/32)]
    rc = rc[:r]
    torch.cuda.synchronize()
    assert torch.equal(_unpack_sf2(sfr, r, c, group_r), er)
    assert torch.equal(qr.view(torch.float8_e4m3fn).float(), rr.float())
    assert torch.equal(_unpack_sf2(sfc, c, r, group_c), ec)
    assert torch.equal(qc.view(torch.float8_e4m3fn).float(), rc.float())


@pytest.mark.parametrize("bn", [160, 224, 256])
@pytest.mark.parametrize("m,n,k", [(256, 320, 512), (384, 1280, 1280), (1000, 5120, 1280), (8192, 1280, 5120)])
def test_pair_gemm_matches_emulation(m, n, k, bn):
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ops import mxfp8 as MX
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(1)
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    xq, xsf, _, _ = MX.quant2(x)
    wq, wsf, _, _ = MX.quant2(w, group_r=bn)
    y = MX.gemm2(xq, xsf, wq, wsf, m, n, k, bn=bn)[0]
    torch.cuda.synchronize()
    L.check_error_word()
    ref = RF.mx_qdq(x.float(), -1) @ RF.mx_qdq(w.float(), -1).T
    assert _rel(y, ref) < 5e-3, _rel(y, ref)                    # bf16 output rounding only


@pytest.mark.parametrize("epi", ["relu2", "res", "mul2sqrt"])
def test_pair_gemm_quantising_epilogues(epi):
    """The epilogue's bf16 result and its two MXFP8 copies (along N and along M) against the emulation applied to the
    stored bf16 tensor."""
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ops import mxfp8 as MX
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(2)
    m, n, k = 640, 1280, 256
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.1).bfloat16()
    r = torch.rand(m, n, device="cuda").bfloat16()
    xq, xsf, _, _ = MX.quant2(x)
    wq, wsf, _, _ = MX.quant2(w, group_r=MX.BN_FWD)
    code = {"relu2": MX.GE_RELU2, "res": MX.GE_BF16_RES, "mul2sqrt": MX.GE_MUL_2SQRT}[epi]
    d, dq, dsf, dt, dtsf = MX.gemm2(xq, xsf, wq, wsf, m, n, k, epi=code, r=None if epi == "relu2" else r, beta=0.5,
                                    want_q=True, want_t=True, dq_group=128, dt_group=256)
    torch.cuda.synchronize()
    L.check_error_word()
    acc = RF.mx_qdq(x.float(), -1) @ RF.mx_qdq(w.float(), -1).T
    ref = {"relu2": torch.relu(acc).square(), "res": acc + 0.5 * r.float(), "mul2sqrt": acc * 2 * r.float().sqrt()}[epi]
    assert _rel(d, ref) < 6e-3, _rel(d, ref)
    # the quantised copies are rounded from the same fp32 values as the bf16 copy: against the emulation applied to the
    # stored bf16 tensor nearly every scale agrees (a block maximum that sits on a power-of-two boundary may differ by
    # the bf16 rounding) and the dequantised values carry only E4M3 rounding noise
    qr, er = RF.mx_quantize(d.float(), -1)
    got_e = _unpack_sf2(dsf, m, n, 128)
    assert float((got_e.int() - er.int()).abs().max()) <= 1 and float((got_e != er).float().mean()) < 0.01
    assert _rel(_deq(dq, got_e, -1), d) < 0.04
    assert _rel(_deq(dq, got_e, -1), RF.mx_dequantize(qr, er, -1)) < 0.02
    qc, ec = RF.mx_quantize(d.float(), 0)
    got_t = _unpack_sf2(dtsf, n, m, 256)
    assert float((got_t.int() - ec.int()).abs().max()) <= 1 and float((got_t != ec).float().mean()) < 0.01
    assert _rel(_deq(dt, got_t, 0), d) < 0.04
