"""Ragged (unpadded) self-attention on the tcgen05 kernels against a plain fp32 PyTorch computation of the same thing:
per sequence and head, ``softmax(q k^T / sqrt(d)) v`` on the bf16 inputs widened to fp32. Forward and backward."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _oracle(qkv, lens, H, d_out=None):
    """fp32 reference; returns (out [T, H*64], dqkv or None)."""
    x = qkv.float().detach().requires_grad_(d_out is not None)
    T = x.shape[0]
    hidden = H * 64
    outs, s0 = [], 0
    for L in lens:
        blk = x[s0:s0 + L]
        q, k, v = (blk[:, i * hidden:(i + 1) * hidden].view(L, H, 64).transpose(0, 1) for i in range(3))   # [H, L, 64]
        att = torch.softmax(q @ k.transpose(1, 2) / 8.0, dim=-1)
        outs.append((att @ v).transpose(0, 1).reshape(L, hidden))
        s0 += L
    out = torch.cat(outs) if outs else x.new_zeros(0, hidden)
    if d_out is None:
        return out, None
    out.backward(d_out.float())
    return out.detach(), x.grad


def _case(lens, H, seed=0):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    offs = torch.zeros(len(lens) + 1, dtype=torch.int32)
    offs[1:] = torch.tensor(lens).cumsum(0)
    qkv = (torch.randn(T, 3 * H * 64, generator=g) * 0.7).to(torch.bfloat16)
    d_out = (torch.randn(T, H * 64, generator=g) * 0.2).to(torch.bfloat16)
    return qkv, offs, d_out


CASES = [([5], 1), ([128], 1), ([129], 2), ([5, 128, 129, 300, 1], 4), ([1000, 50], 2), ([64] * 7, 1), ([257, 3, 511], 3)]


@pytest.mark.parametrize("lens,H", CASES)
def test_ragged_attention_forward_matches_fp32(lens, H):
    import recis_b200
    C = recis_b200.native()
    qkv, offs, _ = _case(lens, H)
    out, lse = C.ragged_attention_fwd(qkv.to(DEV), offs.to(DEV), H, max(lens), 0.125)
    torch.cuda.synchronize()
    assert C.dense_status("cuda:0") == 0
    ref, _ = _oracle(qkv, lens, H)
    got = out.float().cpu()
    assert got.shape == ref.shape
    err = (got - ref).norm() / ref.norm()
    assert err < 1e-2 and float((got - ref).abs().max()) < 3e-2, (float(err), float((got - ref).abs().max()))


@pytest.mark.parametrize("lens,H", CASES)
def test_ragged_attention_backward_matches_fp32(lens, H):
    import recis_b200
    C = recis_b200.native()
    qkv, offs, d_out = _case(lens, H, seed=1)
    q_dev, o_dev = qkv.to(DEV), offs.to(DEV)
    out, lse = C.ragged_attention_fwd(q_dev, o_dev, H, max(lens), 0.125)
    dqkv = C.ragged_attention_bwd(q_dev, out, d_out.to(DEV), lse, o_dev, H, max(lens), 0.125)
    torch.cuda.synchronize()
    assert C.dense_status("cuda:0") == 0
    _, ref = _oracle(qkv, lens, H, d_out)
    got = dqkv.float().cpu()
    hidden = H * 64
    for name, sl in (("dq", slice(0, hidden)), ("dk", slice(hidden, 2 * hidden)), ("dv", slice(2 * hidden, 3 * hidden))):
        a, b = got[:, sl], ref[:, sl]
        err = (a - b).norm() / b.norm().clamp_min(1e-6)
        assert err < 2e-2, (name, float(err))


def test_module_path_uses_the_kernels_and_matches_the_padded_path():
    """``ragged_self_attention`` (what the sequence model calls) on the kernels against the padded SDPA path in fp32."""
    import os
    from recis_b200.ops import attention
    lens, H = [40, 200, 7], 2
    qkv, offs, d_out = _case(lens, H, seed=2)
    a = qkv.to(DEV).requires_grad_(True)
    out = attention.ragged_self_attention(a, offs.to(DEV), H, max(lens))
    out.backward(d_out.to(DEV))
    prev = os.environ.get("RECIS_ATTENTION")
    os.environ["RECIS_ATTENTION"] = "padded"
    try:
        b = qkv.float().to(DEV).requires_grad_(True)
        ref = attention.ragged_self_attention(b, offs.to(DEV), H, max(lens))
        ref.backward(d_out.float().to(DEV))
    finally:
        if prev is None:
            os.environ.pop("RECIS_ATTENTION", None)
        else:
            os.environ["RECIS_ATTENTION"] = prev
    assert (out.float() - ref).norm() / ref.norm() < 1e-2
    assert (a.grad.float() - b.grad).norm() / b.grad.norm() < 2e-2


@pytest.mark.parametrize("lens,hidden", [([5, 1, 300], 256), ([0, 17, 1000, 0, 64], 64), ([33] * 40, 128), ([700, 2], 1024), ([9], 8)])
def test_target_attention_kernels_match_tensor_ops(lens, hidden):
    """One query per sequence over packed tokens, forward and backward, against the segment-reduction formulation in fp32."""
    import os
    from recis_b200.ops import attention
    g = torch.Generator().manual_seed(len(lens) + hidden)
    T, B = sum(lens), len(lens)
    offs = torch.zeros(B + 1, dtype=torch.int32)
    offs[1:] = torch.tensor(lens).cumsum(0)
    x = torch.randn(T, hidden, generator=g)
    q = torch.randn(B, hidden, generator=g)
    go = torch.randn(B, hidden, generator=g)
    a, b = x.to(DEV).requires_grad_(True), q.to(DEV).requires_grad_(True)
    out = attention.target_attention(a, b, offs.to(DEV))
    out.backward(go.to(DEV))
    os.environ["RECIS_TARGET_ATTENTION"] = "eager"
    try:
        c, d = x.clone().requires_grad_(True), q.clone().requires_grad_(True)
        ref = attention.target_attention(c, d, offs)
        ref.backward(go)
    finally:
        os.environ.pop("RECIS_TARGET_ATTENTION", None)
    assert torch.allclose(out.cpu(), ref, atol=2e-5, rtol=1e-4), float((out.cpu() - ref).abs().max())
    assert torch.allclose(a.grad.cpu(), c.grad, atol=5e-5, rtol=1e-3), float((a.grad.cpu() - c.grad).abs().max())
    assert torch.allclose(b.grad.cpu(), d.grad, atol=5e-5, rtol=1e-3), float((b.grad.cpu() - d.grad).abs().max())
