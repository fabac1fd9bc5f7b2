"""Fused feature-engine kernels on the GPU against the CPU implementation of the same op (exact integer equality)."""
import pytest
import torch

from recis_b200.nn.functional import fused_ops, hash_ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _strings(n, seed, max_len):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(0, max_len + 1, (n,), generator=g)
    offs = torch.zeros(n + 1, dtype=torch.int32)
    offs[1:] = lens.cumsum(0)
    data = torch.randint(-128, 128, (int(offs[-1]),), generator=g, dtype=torch.int8)
    return data, offs


@pytest.mark.parametrize("kind", ["farm", "murmur"])
def test_fused_hash_matches_cpu(kind):
    fn = hash_ops.farmhash if kind == "farm" else hash_ops.murmurhash
    # sizes chosen so that chunks of 4096 strings straddle tensor boundaries, one empty tensor, long strings (> 64 bytes)
    cases = [_strings(5000, 1, 24), _strings(3, 2, 8), _strings(0, 3, 8), _strings(9000, 4, 100), _strings(4096, 5, 8)]
    ref = fn([c[0] for c in cases], [c[1] for c in cases])
    got = fn([c[0].to(DEV) for c in cases], [c[1].to(DEV) for c in cases])
    for r, g in zip(ref, got):
        assert torch.equal(r, g.cpu())


def test_fused_mod_matches_cpu_and_python():
    g = torch.Generator().manual_seed(0)
    sizes = [5000, 1, 0, 12289, 4096]
    mods = [1, 7, (1 << 47) - 115, (1 << 62) + 1, 1000003]
    vals = [torch.randint(-(1 << 62), 1 << 62, (n,), generator=g, dtype=torch.int64) for n in sizes]
    vals[3][:4] = torch.tensor([-1, 0, (1 << 63) - 1, -(1 << 63)])
    ref = fused_ops.fused_uint64_mod_gpu(vals, mods)
    got = fused_ops.fused_uint64_mod_gpu([v.to(DEV) for v in vals], mods)
    for r, o in zip(ref, got):
        assert torch.equal(r, o.cpu())
    assert got[3][:4].cpu().tolist() == [((1 << 64) - 1) % mods[3], 0, ((1 << 63) - 1) % mods[3], (1 << 63) % mods[3]]


def test_fused_bucketize_matches_cpu():
    g = torch.Generator().manual_seed(0)
    sizes = [5000, 3, 0, 9000, 4096]
    vals = [torch.randn(n, generator=g) * 2 for n in sizes]
    # 200 boundaries (shared-memory path), 3000 boundaries (beyond the shared-memory limit), a single boundary, duplicates
    bnds = [torch.linspace(-3, 3, 200), torch.linspace(-3, 3, 200), torch.tensor([0.0]), torch.sort(torch.randn(3000, generator=g))[0],
            torch.tensor([-1.0, -1.0, 0.5, 0.5, 2.0])]
    vals[3][:3] = torch.tensor([float("inf"), -float("inf"), 0.0])
    ref = fused_ops.fused_bucketize_gpu(vals, bnds)
    got = fused_ops.fused_bucketize_gpu([v.to(DEV) for v in vals], [b.to(DEV) for b in bnds])
    for r, o, v, b in zip(ref, got, vals, bnds):
        assert torch.equal(r, o.cpu())
        assert torch.equal(r, torch.bucketize(v, b, right=True))


def test_fused_multi_hash_matches_cpu():
    g = torch.Generator().manual_seed(0)
    vals = [torch.randint(-(1 << 40), 1 << 40, (n,), generator=g, dtype=torch.int64) for n in (3000, 17)]
    muls = [torch.tensor([1, 3, 5, 7]), torch.tensor([1, 3])]
    primes = [torch.tensor([29, 47, 67, 83]) * 1000 + 1, torch.tensor([2897, 4703])]
    buckets = [torch.tensor([100, 100, 100, 100]), torch.tensor([10, 10])]
    ref = fused_ops.fused_multi_hash(vals, muls, primes, buckets)
    got = fused_ops.fused_multi_hash([v.to(DEV) for v in vals], muls, primes, buckets)
    assert len(ref) == len(got) == 6
    for r, o in zip(ref, got):
        assert torch.equal(r, o.cpu())
