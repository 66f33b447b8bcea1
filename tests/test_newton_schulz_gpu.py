"""Newton-Schulz orthogonalisation on the tcgen05 GEMM against its plain PyTorch restatement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _stack(b, r, c, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    X = torch.randn(b, r, c, device="cuda", generator=g)
    return (X / X.norm(dim=(1, 2), keepdim=True)).bfloat16()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


@pytest.mark.parametrize("shape", [(3, 256, 256), (2, 256, 768), (2, 768, 256)])
def test_matches_torch_restatement(shape):
    from ml_experiments_b200.ops.newton_schulz import NS5_COEFFS, newton_schulz_, newton_schulz_torch

    X = _stack(*shape, seed=1)
    want = newton_schulz_torch(X.float() , NS5_COEFFS, eps=0.0)
    got = newton_schulz_(X.clone(), NS5_COEFFS)
    assert got.shape == want.shape and _rel(got, want) < 3e-2


def test_same_buffer_every_step_never_runs_in_place():
    """An optimizer hands the same stack buffer in every step, with the same work dict. The result of an odd number of
    iterations lives in the work dict's ping-pong buffer; that buffer must stay distinct from the stack, otherwise the
    last GEMM of every iteration would write the operand that other CTAs are still reading."""
    from ml_experiments_b200.ops.newton_schulz import NS5_COEFFS, newton_schulz_, newton_schulz_torch

    work: dict = {}
    buf = torch.empty(4, 768, 768, device="cuda", dtype=torch.bfloat16)
    for step in range(4):
        X = _stack(4, 768, 768, seed=10 + step)
        buf.copy_(X)
        out = newton_schulz_(buf, NS5_COEFFS, work)
        assert out.data_ptr() != buf.data_ptr()
        assert _rel(out, newton_schulz_torch(X.float(), NS5_COEFFS, eps=0.0)) < 3e-2, step


def test_graph_replay_equals_eager():
    from ml_experiments_b200.ops.newton_schulz import NS5_COEFFS, GraphedNewtonSchulz, newton_schulz_

    buf = torch.empty(3, 256, 768, device="cuda", dtype=torch.bfloat16)
    graphed = GraphedNewtonSchulz(buf, NS5_COEFFS)
    for step in range(3):
        X = _stack(3, 256, 768, seed=20 + step)
        want = newton_schulz_(X.clone(), NS5_COEFFS).clone()
        buf.copy_(X)
        got = graphed()
        torch.cuda.synchronize()
        assert torch.equal(got, want), step
