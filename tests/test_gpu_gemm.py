"""tcgen05 bf16 GEMM against an fp32 PyTorch reference of the same contraction, for every operand layout and epilogue."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from them_bones_b200.ops import _lib as L
    return L


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (384, 1280, 1280), (1000, 264, 200), (128, 128, 4096)])
def test_gemm_nt(m, n, k):
    L = _lib()
    torch.manual_seed(0)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    L.gemm(x, w, out, m=m, n=n, k=k, lda=k, ldb=k, ldd=n)
    torch.cuda.synchronize()
    L.check_error_word()
    ref = x.float() @ w.float().T
    assert _rel(out, ref) < 6e-3


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_nn_and_tn(bn):
    L = _lib()
    torch.manual_seed(1)
    m, n, k = 512, 384, 640
    dy = torch.randn(m, n, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    dx = torch.empty(m, k, device="cuda", dtype=torch.bfloat16)
    L.gemm(dy, w, dx, m=m, n=k, k=n, lda=n, ldb=k, ldd=k, b_major=1, force_bn=bn)
    g = torch.full((n, k), 0.5, device="cuda", dtype=torch.float32)
    L.gemm(dy, x, g, m=n, n=k, k=m, lda=n, ldb=k, ldd=k, a_major=1, b_major=1, epi=L.EPI_ACC_F32, force_bn=bn)
    torch.cuda.synchronize()
    L.check_error_word()
    assert _rel(dx, dy.float() @ w.float()) < 6e-3
    assert _rel(g, 0.5 + dy.float().T @ x.float()) < 2e-3


def test_gemm_epilogues_and_batch():
    L = _lib()
    torch.manual_seed(2)
    m, n, k, b = 256, 512, 320, 3
    x = torch.randn(b, m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(b, n, k, device="cuda", dtype=torch.bfloat16) * 0.1
    r = torch.randn(b, m, n, device="cuda", dtype=torch.bfloat16)
    kw = dict(m=m, n=n, k=k, lda=k, ldb=k, ldd=n, batch=b, stride_a=m * k, stride_b=n * k, stride_d=m * n)
    acc = torch.einsum("bmk,bnk->bmn", x.float(), w.float())
    o = torch.empty(b, m, n, device="cuda", dtype=torch.bfloat16)
    L.gemm(x, w, o, epi=L.EPI_BF16_RES, r=r, ldr=n, stride_r=m * n, alpha=0.5, beta=2.0, **kw)
    torch.cuda.synchronize()
    assert _rel(o, 0.5 * acc + 2.0 * r.float()) < 6e-3
    L.gemm(x, w, o, epi=L.EPI_RELU2, **kw)
    torch.cuda.synchronize()
    assert _rel(o, torch.relu(acc).square()) < 8e-3
    h = torch.rand(b, m, n, device="cuda", dtype=torch.bfloat16)
    L.gemm(x, w, o, epi=L.EPI_MUL_2SQRT, r=h, ldr=n, stride_r=m * n, **kw)
    torch.cuda.synchronize()
    assert _rel(o, acc * 2 * h.float().sqrt()) < 8e-3
    of = torch.empty(b, m, n, device="cuda", dtype=torch.float32)
    L.gemm(x, w, of, epi=L.EPI_F32, **kw)
    torch.cuda.synchronize()
    L.check_error_word()
    assert _rel(of, acc) < 1e-4


@pytest.mark.parametrize("splits", [0, 1, 4])
def test_wgrad_split_k(splits):
    """Weight-gradient GEMM (contraction over many rows, few output tiles) with split-K partial sums added atomically."""
    L = _lib()
    torch.manual_seed(5)
    m, n, k = 8192, 384, 256
    dy = torch.randn(m, n, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    g = torch.full((n, k), -1.0, device="cuda", dtype=torch.float32)
    L.gemm(dy, x, g, m=n, n=k, k=m, lda=n, ldb=k, ldd=k, a_major=1, b_major=1, epi=L.EPI_ACC_F32, splits=splits)
    torch.cuda.synchronize()
    L.check_error_word()
    assert _rel(g, -1.0 + dy.float().T @ x.float()) < 2e-3


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (512, 768, 320), (1000, 520, 200), (2048, 1280, 1280)])
def test_pair_gemm_nt(m, n, k):
    """CTA-pair (cta_group::2) kernel: K-major operands, ragged edges."""
    L = _lib()
    torch.manual_seed(7)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    L.gemm(x, w, out, m=m, n=n, k=k, lda=k, ldb=k, ldd=n, pair=True)
    torch.cuda.synchronize()
    L.check_error_word()
    assert _rel(out, x.float() @ w.float().T) < 6e-3


def test_pair_gemm_layouts_epilogues_batch():
    L = _lib()
    torch.manual_seed(8)
    m, n, k = 512, 384, 640
    dy = torch.randn(m, n, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    dx = torch.empty(m, k, device="cuda", dtype=torch.bfloat16)
    L.gemm(dy, w, dx, m=m, n=k, k=n, lda=n, ldb=k, ldd=k, b_major=1, pair=True)
    g = torch.full((n, k), 0.25, device="cuda", dtype=torch.float32)
    L.gemm(dy, x, g, m=n, n=k, k=m, lda=n, ldb=k, ldd=k, a_major=1, b_major=1, epi=L.EPI_ACC_F32, pair=True)
    g2 = torch.full((n, k), 0.25, device="cuda", dtype=torch.float32)
    L.gemm(dy, x, g2, m=n, n=k, k=m, lda=n, ldb=k, ldd=k, a_major=1, b_major=1, epi=L.EPI_ACC_F32, splits=2, pair=True)
    torch.cuda.synchronize()
    L.check_error_word()
    assert _rel(dx, dy.float() @ w.float()) < 6e-3
    assert _rel(g, 0.25 + dy.float().T @ x.float()) < 2e-3 and _rel(g2, 0.25 + dy.float().T @ x.float()) < 2e-3
    b = 3
    xb = torch.randn(b, 256, 320, device="cuda", dtype=torch.bfloat16)
    wb = torch.randn(b, 512, 320, device="cuda", dtype=torch.bfloat16) * 0.1
    rb = torch.randn(b, 256, 512, device="cuda", dtype=torch.bfloat16)
    o = torch.empty(b, 256, 512, device="cuda", dtype=torch.bfloat16)
    L.gemm(xb, wb, o, m=256, n=512, k=320, lda=320, ldb=320, ldd=512, batch=b, stride_a=256 * 320, stride_b=512 * 320,
           stride_d=256 * 512, epi=L.EPI_BF16_RES, r=rb, ldr=512, stride_r=256 * 512, alpha=0.5, beta=2.0, pair=True)
    torch.cuda.synchronize()
    L.check_error_word()
    acc = torch.einsum("bmk,bnk->bmn", xb.float(), wb.float())
    assert _rel(o, 0.5 * acc + 2.0 * rb.float()) < 6e-3


@pytest.mark.parametrize("pair", [False, True])
def test_gemm_softcap_epilogue(pair):
    """Logit soft-capping fused into the GEMM epilogue: ``cap * tanh(x @ w.T / cap)`` in bf16."""
    from them_bones_b200.ops import _lib as L
    torch.manual_seed(2)
    m, n, k, cap = 512, 1000, 256, 15.0
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(m, 1008, device="cuda", dtype=torch.bfloat16)
    L.gemm(x, w, out, m=m, n=n, k=k, lda=k, ldb=k, ldd=1008, epi=L.EPI_SOFTCAP, alpha=1.0 / cap, beta=cap, pair=pair)
    torch.cuda.synchronize()
    L.check_error_word()
    ref = cap * torch.tanh(x.float() @ w.float().T / cap)
    assert float((out[:, :n].float() - ref).abs().max()) < 0.08
    assert float(out[:, n:].float().abs().sum()) == 0.0
