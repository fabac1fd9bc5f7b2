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


@pytest.mark.parametrize("rows,hidden,out_bf16", [(1000, 256, True), (333, 64, False), (77, 1024, True), (4097, 36, False), (5, 512, False)])
def test_layer_norm_kernels_match_fp32_reference(rows, hidden, out_bf16):
    """Forward (bf16 or fp32 output) and the one-pass backward (input gradient and both weight gradients) against torch's
    layer norm in fp32 on the CPU."""
    from recis_b200.ops.dense import LayerNorm
    g = torch.Generator().manual_seed(rows + hidden)
    x = torch.randn(rows, hidden, generator=g) * 2 + 0.5
    go = torch.randn(rows, hidden, generator=g)
    ref = torch.nn.LayerNorm(hidden)
    with torch.no_grad():
        ref.weight.copy_(torch.randn(hidden, generator=g) * 0.5 + 1)
        ref.bias.copy_(torch.randn(hidden, generator=g) * 0.1)
    ours = LayerNorm(hidden).to(DEV)
    ours.load_state_dict(ref.state_dict())
    xr = x.clone().requires_grad_(True)
    yr = ref(xr)
    yr.backward(go)
    xo = x.to(DEV).requires_grad_(True)
    yo = ours(xo, out_bf16=out_bf16)
    assert yo.dtype == (torch.bfloat16 if out_bf16 else torch.float32)
    yo.backward(go.to(DEV).to(yo.dtype))
    rel = lambda a, b: float((a.float().cpu() - b).norm() / b.norm().clamp(min=1e-12))
    tol = 6e-3 if out_bf16 else 2e-5           # bf16 output and bf16 upstream gradient round at 2^-9
    assert rel(yo.detach(), yr.detach()) < tol
    assert rel(xo.grad, xr.grad) < tol
    assert rel(ours.weight.grad, ref.weight.grad) < tol
    assert rel(ours.bias.grad, ref.bias.grad) < tol


@pytest.mark.parametrize("M,N,relu", [(5000, 256, True), (777, 1024, True), (4096, 768, False), (100, 8, True), (300, 64, True), (64, 24, True)])
def test_relu_backward_with_bias_gradient_all_widths(M, N, relu):
    """Widths served by the 16-byte kernel (powers of two below 256, multiples of 256) and one that falls back (24)."""
    C = recis_b200.native()
    g = torch.Generator().manual_seed(M + N)
    y = torch.randn(M, N, generator=g).to(torch.bfloat16)
    dout = torch.randn(M, N, generator=g).to(torch.bfloat16)
    dy, db = C.relu_bwd_bias(y.to(DEV), dout.to(DEV), relu)
    want = dout.float() * ((y.float() > 0).float() if relu else 1.0)
    assert torch.equal(dy.cpu().float(), want.to(torch.bfloat16).float())
    ref_db = want.to(torch.bfloat16).float().sum(0)
    assert float((db.cpu() - ref_db).norm() / ref_db.norm().clamp(min=1e-6)) < 1e-5


def test_linear_with_residual_in_the_epilogue_matches_fp32_reference():
    from recis_b200.ops.dense import Linear
    g = torch.Generator().manual_seed(3)
    M, K, N = 1000, 256, 256
    lin = Linear(K, N).to(DEV)
    x = torch.randn(M, K, generator=g)
    res = torch.randn(M, N, generator=g)
    go = torch.randn(M, N, generator=g)
    xo = x.to(DEV).to(torch.bfloat16).requires_grad_(True)
    ro = res.to(DEV).requires_grad_(True)
    out = lin.forward_residual(xo, ro)
    assert out.dtype == torch.float32
    out.backward(go.to(DEV))
    xb = x.to(torch.bfloat16).float().requires_grad_(True)
    rr = res.clone().requires_grad_(True)
    W, b = lin.weight.detach().cpu().to(torch.bfloat16).float().requires_grad_(True), lin.bias.detach().cpu().clone().requires_grad_(True)
    ref = rr + xb @ W.t() + b
    ref.backward(go)
    rel = lambda a, b_: float((a.float().cpu() - b_).norm() / b_.norm().clamp(min=1e-12))
    assert rel(out.detach(), ref.detach()) < 1e-5
    assert torch.equal(ro.grad.cpu(), go)
    assert rel(xo.grad, xb.grad) < 8e-3 and rel(lin.weight.grad, W.grad) < 8e-3 and rel(lin.bias.grad, b.grad) < 8e-3


def test_bf16_weight_copies_follow_the_optimizer_and_any_other_change():
    """The forward pass keeps a bf16 copy (padded to multiples of 8) of every weight; the native dense optimizer rewrites it
    together with the weight (no cast in the next forward), and a change made through torch invalidates it."""
    from recis_b200.optim import DenseAdam
    torch.manual_seed(0)
    mlp = D.MLP([64, 128, 24, 1]).to(DEV)
    opt = DenseAdam(mlp.parameters(), lr=1e-2)
    x = torch.randn(256, 64, device=DEV)
    C = recis_b200.native()
    for step in range(3):
        before = C.launch_count()
        loss = mlp(x)[:, :1].float().square().mean()
        launches_fwd = C.launch_count() - before
        opt.zero_grad()
        loss.backward()
        opt.step()
        for layer in mlp.layers:
            sh = D.bf16_shadow(layer.weight)
            N, K = layer.weight.shape
            assert sh is not None and sh.shape == ((N + 7) // 8 * 8, (K + 7) // 8 * 8)
            assert torch.equal(sh[:N, :K], layer.weight.detach().to(torch.bfloat16))            # rewritten by the optimizer
            assert float(sh[N:].abs().sum()) == 0.0 and float(sh[:, K:].abs().sum()) == 0.0     # the padding stays zero
        if step == 0:
            first = launches_fwd
        else:
            assert launches_fwd == first - 3          # no layer casts its weight any more
    with torch.no_grad():
        mlp.layers[0].weight.mul_(0.5)
    assert D.bf16_shadow(mlp.layers[0].weight) is None
    ref = torch.relu(torch.relu(x.to(torch.bfloat16).float() @ mlp.layers[0].weight.detach().to(torch.bfloat16).float().t() + mlp.layers[0].bias))
    out = mlp.layers[0](x.to(torch.bfloat16)).float()
    assert float((out - ref).norm() / ref.norm()) < 1e-2
