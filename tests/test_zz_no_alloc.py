"""The allocation-free attention backward, called through its exported C symbol.

Some users of the native library cannot allocate device memory at the point where they need the attention backward
(no PyTorch allocator in the process, or a phase in which cudaMalloc is forbidden), so ``bones_attn_bwd_noalloc`` keeps
its scratch inside the library.  This test drives that symbol with ctypes, twice in a row on different data (the second
call meets the scratch left by the first), and checks both results against the regular entry points
``bones_attn_delta`` + ``bones_attn_bwd`` on the same inputs and, after the RoPE / QK-norm backward pass, against the
gradient of the plain fp32 PyTorch statement of the same attention.  It also reads the entry point's own status word
(an expired bounded wait would show there and nowhere else) and checks that an oversized problem is refused.
The file name sorts last so a run that stops at the first failure has already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

_I, _L, _F = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _case(lib, seed, b, t, h, window):
    from them_bones_b200.ops import attention_native as AN
    from them_bones_b200.ref import functional as RF
    d = 128
    torch.manual_seed(seed)
    qkv = torch.randn(b * t, 3 * h * d, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(b * t, h * d, device="cuda", dtype=torch.bfloat16)
    cos, sin = RF.rotary_tables(t, d, 10000.0, device="cuda")
    cos, sin = cos.bfloat16().float().contiguous(), sin.bfloat16().float().contiguous()
    idx = torch.randint(1, 50, (b, t), device="cuda")
    idx[:, 0] = 0
    idx[0, t // 2 + 3] = 0
    ds = RF.doc_start_positions(idx, 0).contiguous()
    scale = 1.0 / math.sqrt(d)
    qk = AN.rope_qknorm(qkv, cos, sin, t, h, d)
    y, lse = AN.attn_forward(qk, qkv, ds, b, t, h, scale, window)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # regular entry points (scratch from the caller)
    delta = torch.empty(b, h, t, device="cuda")
    dqk_ref = torch.empty(b * t, 2 * h * d, device="cuda")
    dv_ref = torch.empty(b * t, h * d, device="cuda", dtype=torch.bfloat16)
    assert lib.bones_attn_delta(_p(dy), _p(y), _p(delta), _L(b * t), _I(t), _I(h), stream) == 0
    assert lib.bones_attn_bwd(_p(qk), _p(qkv), _p(dy), _p(lse), _p(delta), _p(dqk_ref), _p(dv_ref), _p(ds), _I(b), _I(t),
                              _I(h), _F(scale), _I(window // 128), stream) == 0
    # allocation-free entry point (scratch inside the library)
    dqk = torch.full_like(dqk_ref, float("nan"))
    dv = torch.zeros_like(dv_ref)
    rc = lib.bones_attn_bwd_noalloc(_p(qk), _p(qkv), _p(dy), _p(y), _p(lse), _p(dqk), _p(dv), _p(ds), _I(b), _I(t), _I(h),
                                    _F(scale), _I(window // 128), stream)
    assert rc == 0, lib.bones_attn_bwd_noalloc_strerror(rc)
    torch.cuda.synchronize()
    rel = lambda a, r: float((a.float() - r.float()).norm() / r.float().norm().clamp_min(1e-12))  # noqa: E731
    assert torch.isfinite(dqk).all()
    assert rel(dqk, dqk_ref) < 1e-3 and rel(dv, dv_ref) < 1e-3, (rel(dqk, dqk_ref), rel(dv, dv_ref))
    assert lib.bones_attn_bwd_noalloc_error_read_clear(stream) == 0
    # oracle: the fp32 PyTorch statement of the whole op, differentiated by autograd
    dqkv = torch.empty(b * t, 3 * h * d, device="cuda", dtype=torch.bfloat16)
    assert lib.bones_rope_qknorm_bwd(_p(qkv), _p(cos), _p(sin), _p(dqk), _p(dv), _p(dqkv), _L(b * t), _I(t), _I(h), _I(d),
                                     stream) == 0
    x = qkv.float().view(b, t, -1).requires_grad_(True)
    RF.attention(x, cos, sin, h, d, scale, ds, window).backward(dy.float().view(b, t, -1))
    torch.cuda.synchronize()
    assert rel(dqkv.view(b, t, -1), x.grad) < 4e-2, rel(dqkv.view(b, t, -1), x.grad)


def test_noalloc_attention_backward_twice_and_limit():
    from them_bones_b200.ops import _lib as L
    lib = ctypes.CDLL(L.lib_path())
    lib.bones_attn_bwd_noalloc_strerror.restype = ctypes.c_char_p
    _case(lib, seed=0, b=2, t=512, h=2, window=0)
    _case(lib, seed=1, b=1, t=256, h=3, window=128)        # smaller problem: meets the first call's leftovers
    L.check_error_word()
    # beyond the built-in scratch: refused before anything is launched
    rc = lib.bones_attn_bwd_noalloc(None, None, None, None, None, None, None, None, _I(64), _I(2048), _I(16), _F(0.1), _I(0),
                                    None)
    assert rc == -10 and b"exceeds" in lib.bones_attn_bwd_noalloc_strerror(rc)
