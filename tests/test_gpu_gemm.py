"""tcgen05 GEMM against an fp32 PyTorch reference, for every operand-major combination used by the dense towers."""
import pytest
import torch

import recis_b200

pytestmark = pytest.mark.gpu
C = recis_b200.native()
DEV = "cuda:0"


def _ref(a, b, bias, relu, a_mn, b_mn):
    A = (a.t() if a_mn else a).float()
    B = (b.t() if b_mn else b).float()
    y = A @ B.t()
    if bias is not None:
        y = y + bias.float()
    return torch.relu(y) if relu else y


@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 128, 128), (300, 200, 72), (8192, 512, 16), (1000, 1024, 480), (77, 8, 8)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_matches_fp32(shape, a_mn, b_mn):
    M, N, K = shape
    torch.manual_seed(M + N + K)
    a = (torch.randn(K, M) if a_mn else torch.randn(M, K)).to(DEV, torch.bfloat16)
    b = (torch.randn(K, N) if b_mn else torch.randn(N, K)).to(DEV, torch.bfloat16)
    if (a.shape[1] % 8) or (b.shape[1] % 8):
        pytest.skip("row pitch must be a multiple of 16 bytes for TMA")
    bias = torch.randn(N, device=DEV)
    for relu, out_fp32 in ((False, True), (True, False)):
        y = C.gemm_bf16(a, b, bias, relu, a_mn, b_mn, out_fp32, None)
        ref = _ref(a, b, bias, relu, a_mn, b_mn)
        tol = 2e-2 if not out_fp32 else 2e-3
        err = (y.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1.0)
        assert err < tol, (shape, a_mn, b_mn, relu, err)
        # relative Frobenius norm: bf16 output rounding is 2^-9 per entry, fp32 output only carries accumulation order
        fro = ((y.float() - ref).norm() / ref.norm().clamp_min(1e-6)).item()
        assert fro < (4e-3 if not out_fp32 else 1e-4), (shape, a_mn, b_mn, relu, fro)
    assert C.dense_status(DEV) == 0


def test_gemm_accumulate():
    torch.manual_seed(0)
    a = torch.randn(256, 64, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(128, 64, device=DEV, dtype=torch.bfloat16)
    acc = torch.randn(256, 128, device=DEV)
    ref = acc + a.float() @ b.float().t()
    out = C.gemm_bf16(a, b, None, False, False, False, True, acc)
    assert out.data_ptr() == acc.data_ptr()
    assert torch.allclose(out, ref, atol=1e-2, rtol=1e-3)


@pytest.mark.parametrize("M,N,K,masked", [(8192, 1024, 512, True), (1000, 264, 520, True), (300, 64, 128, False), (8192, 512, 1024, True), (77, 8, 24, True)])
def test_dgrad_with_relu_mask_and_bias_gradient_in_the_epilogue(M, N, K, masked):
    """dx = (dy W) masked by the ReLU of the layer below, and its column sums, from one GEMM: against fp32 matmul + mask + sum,
    on shapes that take the one-CTA kernel and shapes that take the pair kernel."""
    C = recis_b200.native()
    g = torch.Generator().manual_seed(M + N + K)
    dy = torch.randn(M, N, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    y_below = torch.randn(M, K, generator=g).to(torch.bfloat16)
    dx, db = C.gemm_dgrad_fused(dy.to(DEV), w.to(DEV), y_below.to(DEV) if masked else None)
    ref = dy.float() @ w.float()
    if masked:
        ref = ref * (y_below.float() > 0).float()
    rel = lambda a, b: float((a.float().cpu() - b).norm() / b.norm().clamp(min=1e-12))
    assert dx.dtype == torch.bfloat16 and rel(dx, ref) < 6e-3
    if masked:
        assert float(dx.float().cpu()[(y_below.float() <= 0)].abs().max()) == 0.0       # masked entries are exact zeros
    assert rel(db, ref.sum(0)) < 2e-3
    assert C.dense_status(DEV) == 0
