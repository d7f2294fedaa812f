"""tcgen05 flash attention (RoPE + QK-norm + causal + document reset + band) against the fp32 PyTorch statement."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def _inputs(b, t, h, d, seed=0, docs=True):
    from them_bones_b200.ref import functional as RF
    torch.manual_seed(seed)
    qkv = torch.randn(b, t, 3 * h * d, device="cuda", dtype=torch.bfloat16)
    cos, sin = RF.rotary_tables(t, d, 10000.0, device="cuda")
    cos, sin = cos.bfloat16().float(), sin.bfloat16().float()
    ds = None
    if docs:
        idx = torch.randint(1, 100, (b, t), device="cuda")
        idx[:, 0] = 0
        idx[0, t // 3] = 0
        idx[-1, t - 5] = 0
        idx[-1, 130] = 0
        ds = RF.doc_start_positions(idx, 0)
    return qkv, cos, sin, ds


@pytest.mark.parametrize("b,t,h,window,docs", [(1, 128, 1, 0, False), (2, 512, 2, 0, True), (1, 1024, 3, 256, True),
                                               (2, 2048, 2, 0, True)])
def test_attention_forward(b, t, h, window, docs):
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ops import attention_native as AN
    from them_bones_b200.ref import functional as RF
    d = 128
    qkv, cos, sin, ds = _inputs(b, t, h, d, docs=docs)
    scale = 1.0 / math.sqrt(d)
    with torch.no_grad():
        y = AN.attention(qkv, cos, sin, h, d, scale, ds, window)
        ref = RF.attention(qkv.float(), cos, sin, h, d, scale, ds, window)
    torch.cuda.synchronize()
    L.check_error_word()
    assert torch.isfinite(y).all()
    assert _rel(y, ref) < 2e-2, _rel(y, ref)


@pytest.mark.parametrize("b,t,h,window,docs", [(2, 512, 2, 256, True), (1, 2048, 2, 0, True), (1, 2048, 1, 512, True),
                                               (2, 1024, 1, 0, False)])
def test_attention_backward(b, t, h, window, docs):
    """Full-causal and banded, at the training length, with a document start inside the last 128-token tile
    (``_inputs`` puts one at ``t - 5``) and without documents."""
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ops import attention_native as AN
    from them_bones_b200.ref import functional as RF
    d = 128
    qkv, cos, sin, ds = _inputs(b, t, h, d, seed=3, docs=docs)
    scale = 0.11
    g = torch.randn(b, t, h * d, device="cuda", dtype=torch.bfloat16)
    x = qkv.clone().requires_grad_(True)
    y = AN.attention(x, cos, sin, h, d, scale, ds, window)
    y.backward(g)
    xr = qkv.float().requires_grad_(True)
    yr = RF.attention(xr, cos, sin, h, d, scale, ds, window)
    yr.backward(g.float())
    torch.cuda.synchronize()
    L.check_error_word()
    assert _rel(y, yr) < 2e-2
    assert _rel(x.grad, xr.grad) < 4e-2, _rel(x.grad, xr.grad)


def test_attention_backward_repeated_calls_stay_finite_and_equal():
    """The backward kernels pipeline two key tiles per CTA, so a hand-off that lets a fast warp run ahead of a slow one
    shows only now and then (it once left a few non-finite rows in dq every few hundred calls at this geometry).  Three
    hundred calls on the same inputs, with other memory traffic in between, must all give the first call's gradient."""
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ops import attention_native as AN
    b, t, h, d = 16, 2048, 10, 128
    qkv, cos, sin, ds = _inputs(b, t, h, d, seed=11, docs=True)
    g = torch.randn(b, t, h * d, device="cuda", dtype=torch.bfloat16)
    noise = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    first, bad = None, 0
    for it in range(300):
        x = qkv.clone().requires_grad_(True)
        AN.attention(x, cos, sin, h, d, 1.0 / math.sqrt(d), ds, 0).backward(g)
        if it % 3 == 0:
            noise.zero_()
        if first is None:
            first = x.grad.clone()
            assert torch.isfinite(first).all()
        else:
            bad += int(not torch.equal(x.grad, first))
    torch.cuda.synchronize()
    L.check_error_word()
    assert bad == 0, f"{bad} of 299 repeated calls differ from the first"


@pytest.mark.parametrize("b,t,h,window,docs", [(2, 512, 3, 0, True), (1, 1024, 2, 256, True)])
def test_attention_head_dim_64(b, t, h, window, docs):
    """head_dim 64 runs on the 128-wide kernels with zero-padded heads: forward and gradients against the fp32
    statement, through the operator layer."""
    from them_bones_b200 import ops
    from them_bones_b200.ops import _lib as L
    from them_bones_b200.ref import functional as RF
    d = 64
    qkv, cos, sin, ds = _inputs(b, t, h, d, seed=11, docs=docs)
    scale = 1.0 / math.sqrt(d)
    g = torch.randn(b, t, h * d, device="cuda", dtype=torch.bfloat16)
    x = qkv.clone().requires_grad_(True)
    y = ops.attention(x, cos, sin, h, d, scale, ds, window)
    y.backward(g)
    xr = qkv.float().requires_grad_(True)
    yr = RF.attention(xr, cos, sin, h, d, scale, ds, window)
    yr.backward(g.float())
    torch.cuda.synchronize()
    L.check_error_word()
    assert y.shape == (b, t, h * d)
    assert _rel(y, yr) < 2e-2, _rel(y, yr)
    assert _rel(x.grad, xr.grad) < 4e-2, _rel(x.grad, xr.grad)


def test_attention_ragged_length_is_padded_and_unsupported_shapes_raise():
    """The operator layer pads a length that is not a multiple of 128 (scoring, cache-free decoding) and raises --
    rather than taking a library path -- for what the kernels do not cover."""
    from them_bones_b200 import ops
    from them_bones_b200.ref import functional as RF
    b, t, h, d = 2, 200, 2, 128
    qkv, cos, sin, ds = _inputs(b, t, h, d, seed=5)
    with torch.no_grad():
        y = ops.attention(qkv, cos, sin, h, d, 0.11, ds, 0)
        ref = RF.attention(qkv.float(), cos, sin, h, d, 0.11, ds, 0)
    assert y.shape == (b, t, h * d) and _rel(y, ref) < 2e-2
    with pytest.raises(ValueError):
        ops.attention(qkv.float(), cos, sin, h, d, 0.11, ds, 0)


def test_library_ops_match_the_eager_wrappers():
    """The torch.library custom ops run the same kernels: identical outputs and gradients, and they pass opcheck's
    schema / fake-tensor / autograd-registration checks."""
    from them_bones_b200.ops import attention_native as AN
    from them_bones_b200.ops import registry as R
    b, t, h, d = 2, 512, 2, 128
    qkv, cos, sin, ds = _inputs(b, t, h, d, seed=7)
    g = torch.randn(b, t, h * d, device="cuda", dtype=torch.bfloat16)
    x1 = qkv.clone().requires_grad_(True)
    AN.attention(x1, cos, sin, h, d, 0.11, ds, 256).backward(g)
    x2 = qkv.clone().requires_grad_(True)
    y2 = R.attention(x2, cos, sin, h, d, 0.11, ds, 256)
    y2.backward(g)
    torch.cuda.synchronize()
    assert torch.equal(x1.grad, x2.grad)
    z = torch.randn(64, 1280, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    from them_bones_b200.ref import functional as RF
    assert _rel(R.rms_norm(z), RF.rms_norm(z.float())) < 1e-2
    torch.library.opcheck(torch.ops.bones.rmsnorm_fwd.default, (z.detach(),), test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(torch.ops.bones.attention_fwd.default, (qkv, cos, sin, ds.to(torch.int32), h, d, 0.11, 256),
                          test_utils=("test_schema", "test_faketensor"))
