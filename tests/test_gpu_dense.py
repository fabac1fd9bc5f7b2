"""Dense-tower kernels (tcgen05 Linear, interactions) against fp32 PyTorch references."""
import pytest
import torch

import recis_b200
from recis_b200.ops import dense as D

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ref_dot(x, cube):
    B, Fn, Dm = cube.shape
    z = torch.cat([x.unsqueeze(1), cube], dim=1)
    zz = torch.bmm(z, z.transpose(1, 2))
    li, lj = torch.tril_indices(Fn + 1, Fn + 1, offset=-1)
    return torch.cat([x, zz[:, li, lj]], dim=1)


@pytest.mark.parametrize("B,F,Dm", [(64, 26, 128), (33, 3, 16), (8, 1, 8)])
def test_dot_interaction_fwd_bwd(B, F, Dm):
    torch.manual_seed(0)
    x = torch.randn(B, Dm).to(torch.bfloat16)
    cube = torch.randn(B, F, Dm)
    xr = x.float().requires_grad_(True); cr = cube.clone().requires_grad_(True)
    ref = _ref_dot(xr, cr)
    xg = x.to(DEV).requires_grad_(True); cg = cube.to(DEV).requires_grad_(True)
    out = D.dot_interaction(xg, cg)
    n = ref.shape[1]
    assert out.shape[1] % 8 == 0 and out.shape[1] >= n
    assert torch.allclose(out[:, :n].float().cpu(), ref, atol=0.15, rtol=2e-2)
    assert float(out[:, n:].abs().sum()) == 0
    go = torch.randn(B, out.shape[1]).to(torch.bfloat16)
    out.backward(go.to(DEV))
    ref.backward(go[:, :n].float())
    assert torch.allclose(cg.grad.cpu(), cr.grad, atol=0.1, rtol=2e-2)
    assert torch.allclose(xg.grad.float().cpu(), xr.grad, atol=0.3, rtol=3e-2)


def test_fm_interaction():
    torch.manual_seed(0)
    cube = torch.randn(50, 7, 16)
    cr = cube.clone().requires_grad_(True)
    ref = D.fm_interaction(cr)
    cg = cube.to(DEV).requires_grad_(True)
    out = D.fm_interaction(cg)
    assert torch.allclose(out.cpu(), ref, atol=1e-4, rtol=1e-4)
    g = torch.randn(50, 1)
    ref.backward(g); out.backward(g.to(DEV))
    assert torch.allclose(cg.grad.cpu(), cr.grad, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("dims", [(13, 512, 256, 128), (480, 1024, 1024, 512, 256, 1), (16, 8)])
def test_mlp_matches_fp32(dims):
    torch.manual_seed(0)
    M = 1000
    mlp = D.MLP(list(dims), final_act=False)
    ref = D.MLP(list(dims), final_act=False, dtype=torch.float32)
    ref.load_state_dict(mlp.state_dict())
    mlp = mlp.to(DEV)
    x = torch.randn(M, dims[0])
    y = mlp(x.to(DEV)).float().cpu()
    yr = ref(x)
    assert y.shape == yr.shape
    scale = max(float(yr.abs().max()), 1.0)
    assert float((y - yr).abs().max()) / scale < 3e-2
    go = torch.randn_like(yr)
    (y_g := mlp(x.to(DEV))).backward(go.to(DEV).to(y_g.dtype))
    yr.backward(go)
    for (n1, p1), (n2, p2) in zip(mlp.named_parameters(), ref.named_parameters()):
        g1, g2 = p1.grad.float().cpu(), p2.grad
        denom = max(float(g2.abs().max()), 1e-3)
        assert float((g1 - g2).abs().max()) / denom < 6e-2, (n1, float((g1 - g2).abs().max()), denom)
    assert recis_b200.native().dense_status(DEV) == 0
