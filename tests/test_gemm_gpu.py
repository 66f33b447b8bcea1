"""tcgen05 GEMM against fp32 torch matmul: every operand majorness, ragged shapes, batches, epilogues, fp8."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().transpose(-1, -2) if a_mn else a.float()
    B = b.float().transpose(-1, -2) if b_mn else b.float()
    return A @ B.transpose(-1, -2)


def _rel_err(x, y):
    return ((x.float() - y).norm() / (y.norm() + 1e-12)).item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 512, 256), (384, 768, 1024), (200, 136, 72), (1024, 2304, 768)])
def test_gemm_bf16_majors(a_mn, b_mn, m, n, k):
    from ml_experiments_b200.ops.gemm import gemm

    torch.manual_seed(0)
    a = torch.randn((k, m) if a_mn else (m, k), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((k, n) if b_mn else (n, k), device="cuda", dtype=torch.bfloat16)
    ref = _ref(a, b, a_mn, b_mn)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert _rel_err(out, ref) < 2e-3
    out16 = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    assert out16.dtype == torch.bfloat16
    assert _rel_err(out16, ref) < 6e-3


def test_gemm_batched_and_epilogues():
    from ml_experiments_b200.ops import gemm as G

    torch.manual_seed(1)
    a = torch.randn(3, 256, 320, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(3, 384, 320, device="cuda", dtype=torch.bfloat16)
    ref = _ref(a, b, False, False)
    assert _rel_err(G.gemm(a, b, out_dtype=torch.float32), ref) < 2e-3
    # relu^2
    out = G.gemm(a, b, epilogue=G.EPI_RELU2, alpha=0.05)
    assert _rel_err(out, torch.relu(ref * 0.05) ** 2) < 1e-2
    # alpha * acc + beta * aux
    aux = torch.randn(3, 256, 384, device="cuda", dtype=torch.bfloat16)
    out = G.gemm(a, b, epilogue=G.EPI_AXPBY, aux=aux, alpha=0.5, beta=-2.0, out_dtype=torch.float32)
    assert _rel_err(out, 0.5 * ref - 2.0 * aux.float()) < 2e-3
    # relu^2 backward: acc * 2 * sqrt(h)
    h = (torch.relu(torch.randn(3, 256, 384, device="cuda")) ** 2).bfloat16()
    out = G.gemm(a, b, epilogue=G.EPI_RELU2_BWD, aux=h, out_dtype=torch.float32)
    assert _rel_err(out, ref * 2 * h.float().sqrt()) < 2e-3


def test_gemm_split_k_and_accumulate():
    from ml_experiments_b200.ops import gemm as G

    torch.manual_seed(2)
    # weight-gradient shape: both operands MN-major, long K
    dy = torch.randn(8192, 768, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(8192, 768, device="cuda", dtype=torch.bfloat16)
    ref = dy.float().T @ x.float()
    out = G.gemm(dy, x, a_mn=True, b_mn=True, split_k=8)
    assert out.dtype == torch.float32
    assert _rel_err(out, ref) < 2e-3
    out2 = G.gemm(dy, x, a_mn=True, b_mn=True, split_k=4, out=out.clone(), accumulate=True)
    assert _rel_err(out2, 2 * ref) < 2e-3


def test_gemm_strided_views():
    from ml_experiments_b200.ops import gemm as G

    torch.manual_seed(3)
    big = torch.randn(512, 3 * 256, device="cuda", dtype=torch.bfloat16)
    a = big[:, 256:512]  # row pitch 768, K = 256
    w = torch.randn(384, 256, device="cuda", dtype=torch.bfloat16)
    outbuf = torch.zeros(512, 1024, device="cuda", dtype=torch.bfloat16)
    G.gemm(a, w, out=outbuf[:, 128:512])
    assert _rel_err(outbuf[:, 128:512], a.float() @ w.float().T) < 6e-3
    assert outbuf[:, :128].abs().max().item() == 0 and outbuf[:, 512:].abs().max().item() == 0


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_fp8(a_mn, b_mn):
    from ml_experiments_b200.ops.gemm import gemm

    torch.manual_seed(4)
    m, n, k = 512, 640, 768
    a = torch.randn((k, m) if a_mn else (m, k), device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn((k, n) if b_mn else (n, k), device="cuda").to(torch.float8_e5m2 if b_mn else torch.float8_e4m3fn)
    ref = _ref(a, b, a_mn, b_mn)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, alpha=0.25)
    assert _rel_err(out, 0.25 * ref) < 2e-3


def test_output_aliasing_an_operand_is_refused():
    """In-place products are a timing-dependent race between CTAs (one stores a tile of the operand another still
    reads); the front end rejects them instead of returning numbers that are right most of the time."""
    from ml_experiments_b200.ops import gemm as G

    x = torch.randn(4, 256, 256, device="cuda").bfloat16()
    w = torch.randn(4, 256, 256, device="cuda").bfloat16()
    with pytest.raises(ValueError, match="alias"):
        G.gemm(w, x, b_mn=True, out=x)
    with pytest.raises(ValueError, match="alias"):
        G.gemm(x, w, out=x[:, :, :])
    out = torch.empty_like(x)
    G.gemm(w, x, b_mn=True, out=out, epilogue=G.EPI_AXPBY, aux=x, alpha=1.0, beta=0.5)      # aux may be an operand
