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


@pytest.mark.parametrize("B,F,Dm", [(64, 26, 128), (130, 26, 64), (5, 31, 128), (33, 3, 16), (8, 1, 8)])
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
    got = out[:, :n].detach().float().cpu()
    assert torch.allclose(got, ref.detach(), atol=0.15, rtol=2e-2)
    # relative norm: a dropped 16-column k-block of the D = 128 reduction would cost about 1/8 of every entry's terms
    assert float((got - ref.detach()).norm() / ref.detach().norm()) < 1e-2
    assert float(out[:, n:].detach().abs().sum()) == 0
    go = torch.randn(B, out.shape[1]).to(torch.bfloat16)
    out.backward(go.to(DEV))
    ref.backward(go[:, :n].float())
    assert torch.allclose(cg.grad.cpu(), cr.grad, atol=0.1, rtol=2e-2)
    assert torch.allclose(xg.grad.float().cpu(), xr.grad, atol=0.3, rtol=3e-2)
    assert float((cg.grad.cpu() - cr.grad).norm() / cr.grad.norm()) < 1e-2
    assert float((xg.grad.float().cpu() - xr.grad).norm() / xr.grad.norm()) < 1.5e-2


def test_fm_interaction():
    torch.manual_seed(0)
    for shape in [(50, 7, 16), (1000, 39, 16), (33, 5, 12), (17, 3, 128), (9, 4, 7)]:
        cube = torch.randn(*shape)
        cr = cube.clone().requires_grad_(True)
        ref = D.fm_interaction(cr)
        cg = cube.to(DEV).requires_grad_(True)
        out = D.fm_interaction(cg)
        assert torch.allclose(out.cpu(), ref, atol=2e-4, rtol=1e-4), shape
        g = torch.randn(shape[0], 1)
        ref.backward(g); out.backward(g.to(DEV))
        assert torch.allclose(cg.grad.cpu(), cr.grad, atol=1e-4, rtol=1e-4), shape


def _torch_bf16_mlp(mlp, x):
    """The same network with plain PyTorch ops and the same rounding points (bf16 operands/activations, fp32 accumulation)."""
    import torch.nn.functional as F
    params = []
    h = x.to(torch.bfloat16)
    n = len(mlp.layers)
    for i, layer in enumerate(mlp.layers):
        w = layer.weight.detach().clone().requires_grad_(True)
        b = layer.bias.detach().clone().requires_grad_(True)
        params += [w, b]
        h = (F.linear(h.float(), w.to(torch.bfloat16).float()) + b)
        if layer.act:
            h = torch.relu(h)
        h = h.to(torch.bfloat16)
    return h, params


@pytest.mark.parametrize("dims", [(13, 512, 256, 128), (480, 1024, 1024, 512, 256, 1), (16, 8)])
def test_mlp_matches_reference(dims):
    torch.manual_seed(0)
    M = 1000
    mlp = D.MLP(list(dims), final_act=False).to(DEV)
    x = torch.randn(M, dims[0], device=DEV)
    y = mlp(x)
    yr, ref_params = _torch_bf16_mlp(mlp, x)
    rel = lambda a, b: float((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12))
    assert y.shape == yr.shape
    assert rel(y, yr) < 1e-2
    # and against a pure fp32 network (no bf16 anywhere): loose, it only guards against gross errors
    ref32 = D.MLP(list(dims), final_act=False, dtype=torch.float32).to(DEV)
    ref32.load_state_dict(mlp.state_dict())
    assert rel(y, ref32(x)) < 5e-2
    go = torch.randn(M, dims[-1], device=DEV).to(torch.bfloat16)
    y.backward(go)
    yr.backward(go)
    for (name, p), r in zip(mlp.named_parameters(), ref_params):
        assert rel(p.grad, r.grad) < 3e-2, (name, rel(p.grad, r.grad))
    assert recis_b200.native().dense_status(DEV) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("decoupled", [False, True])
def test_dense_adam_matches_torch(decoupled):
    """Native multi-tensor Adam/AdamW against torch.optim on the same gradients (30 tensors: two launches, odd sizes)."""
    from recis_b200.optim import DenseAdam
    torch.manual_seed(0)
    shapes = [(37,), (128, 65), (3,), (1024, 16)] * 7 + [(5, 5), (1,)]
    ours = [torch.randn(s, device="cuda").requires_grad_() for s in shapes]
    ref = [p.detach().clone().requires_grad_() for p in ours]
    wd = 0.01
    o1 = DenseAdam(ours, lr=1e-2, weight_decay=wd, decoupled=decoupled)
    o2 = (torch.optim.AdamW if decoupled else torch.optim.Adam)(ref, lr=1e-2, weight_decay=wd)
    for _ in range(5):
        for a, b in zip(ours, ref):
            g = torch.randn_like(a)
            a.grad = g.clone()
            b.grad = g.clone()
        o1.step()
        o2.step()
    for a, b in zip(ours, ref):
        torch.testing.assert_close(a, b, rtol=2e-5, atol=2e-6)


@pytest.mark.gpu
def test_adamw_tf_native_matches_cpu_foreach():
    from recis_b200.optim import AdamWTF
    torch.manual_seed(1)
    shapes = [(33, 7), (256,), (2, 3, 5)]
    cpu = [torch.randn(s).requires_grad_() for s in shapes]
    gpu = [p.detach().cuda().requires_grad_() for p in cpu]
    o1, o2 = AdamWTF(cpu, lr=1e-2, weight_decay=0.02), AdamWTF(gpu, lr=1e-2, weight_decay=0.02)
    for _ in range(4):
        for a, b in zip(cpu, gpu):
            g = torch.randn_like(a)
            a.grad = g.clone()
            b.grad = g.cuda()
        o1.step()
        o2.step()
    for a, b in zip(cpu, gpu):
        torch.testing.assert_close(a, b.cpu(), rtol=2e-5, atol=2e-6)
