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


def _ragged(rows, max_len, seed, dtype=torch.int64, off_dtype=torch.int32):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(0, max_len + 1, (rows,), generator=g)
    offs = torch.zeros(rows + 1, dtype=off_dtype)
    offs[1:] = lens.cumsum(0)
    n = int(offs[-1])
    vals = torch.randint(0, 1 << 20, (n,), generator=g).to(dtype) if dtype != torch.float32 else torch.randn(n, generator=g)
    return vals, offs


def test_fused_cutoff_2d_all_features_in_three_launches():
    """Sequence truncation of many features at once: equal to the CPU implementation, three kernel launches and one host read
    for the whole call however many features there are."""
    import recis_b200
    from recis_b200.nn.functional import ragged_ops
    C = recis_b200.native()
    feats = [_ragged(300, 12, s, dtype=(torch.int64, torch.float32, torch.int32)[s % 3], off_dtype=(torch.int32, torch.int64)[s % 2])
             for s in range(40)] + [_ragged(0, 5, 99), _ragged(5000, 40, 100)]
    T = len(feats)
    keep = torch.tensor([(3, 7, 0, 100)[t % 4] for t in range(T)], dtype=torch.int32)
    drop = torch.tensor([t % 2 == 0 for t in range(T)])
    pad = torch.tensor([t % 3 == 0 for t in range(T)])
    ref = ragged_ops.fused_ragged_cutoff_2D([f[0] for f in feats], [f[1] for f in feats], keep, drop, pad)
    torch.cuda.synchronize()
    before = C.launch_count()
    got = ragged_ops.fused_ragged_cutoff_2D([f[0].to(DEV) for f in feats], [f[1].to(DEV) for f in feats], keep, drop, pad)
    assert C.launch_count() - before <= 4
    for k in range(4):                                   # values, offsets, drop_nums, pad_nums
        for r, o in zip(ref[k], got[k]):
            assert r.dtype == o.dtype and torch.equal(r, o.cpu()), k


def test_fused_cutoff_2d_thousand_features():
    import recis_b200
    from recis_b200.nn.functional import ragged_ops
    C = recis_b200.native()
    feats = [_ragged(64, 9, s) for s in range(1000)]
    keep = torch.full((1000,), 4, dtype=torch.int32)
    ref = ragged_ops.fused_ragged_cutoff_2D([f[0] for f in feats], [f[1] for f in feats], keep)
    dev_feats = [(f[0].to(DEV), f[1].to(DEV)) for f in feats]
    torch.cuda.synchronize()
    before = C.launch_count()
    got = ragged_ops.fused_ragged_cutoff_2D([f[0] for f in dev_feats], [f[1] for f in dev_feats], keep)
    assert C.launch_count() - before <= 4
    for r, o in zip(ref[0] + ref[1], got[0] + got[1]):
        assert torch.equal(r, o.cpu())


def test_fused_cutoff_3d_matches_cpu():
    import recis_b200
    from recis_b200.nn.functional import ragged_ops
    C = recis_b200.native()
    g = torch.Generator().manual_seed(7)
    vals, offs = [], []
    for t in range(12):
        B = (50, 1, 200)[t % 3]
        n_inner = torch.randint(0, 7, (B,), generator=g)
        outer = torch.zeros(B + 1, dtype=torch.int32); outer[1:] = n_inner.cumsum(0)
        v, inner = _ragged(int(outer[-1]), 5, 100 + t)
        vals.append(v); offs.append([outer, inner])
    keep = torch.tensor([(3, 1, 6, 4)[t % 4] for t in range(12)], dtype=torch.int32)
    drop = torch.tensor([t % 2 == 1 for t in range(12)])
    pad = torch.tensor([t % 3 == 1 for t in range(12)])
    ref_v, ref_o = ragged_ops.fused_ragged_cutoff_3D(vals, offs, keep, drop, pad)
    torch.cuda.synchronize()
    before = C.launch_count()
    got_v, got_o = ragged_ops.fused_ragged_cutoff_3D([v.to(DEV) for v in vals], [[o[0].to(DEV), o[1].to(DEV)] for o in offs], keep, drop, pad)
    assert C.launch_count() - before <= 4
    for r, o in zip(ref_v, got_v):
        assert torch.equal(r, o.cpu())
    for (ro, ri), (go, gi) in zip(ref_o, got_o):
        assert torch.equal(ro, go.cpu()) and torch.equal(ri, gi.cpu())


def test_feature_cross_sorted_unique_matches_cpu():
    """Per-row unique by segmented sort on the GPU: identical to the CPU implementation (both emit a row's unique values in
    ascending order; a repeated value keeps the weight of its first occurrence), including long rows full of duplicates."""
    from recis_b200.nn.functional import ragged_ops
    g = torch.Generator().manual_seed(3)

    def side(rows, max_len, n_vals, seed):
        gg = torch.Generator().manual_seed(seed)
        lens = torch.randint(0, max_len + 1, (rows,), generator=gg)
        lens[0] = 0
        lens[1] = max_len
        off = torch.zeros(rows + 1, dtype=torch.int64); off[1:] = lens.cumsum(0)
        vals = torch.randint(-n_vals, n_vals, (int(off[-1]),), generator=gg)
        return vals, off, torch.rand(int(off[-1]), generator=gg)
    xv, xo, xw = side(500, 300, 40, 1)          # up to 300 values per row drawn from 80: heavy duplication
    yv, yo, yw = side(500, 20, 1000, 2)
    ref = ragged_ops.feature_cross_ragged(xv, xo, yv, yo, xw, yw)
    got = ragged_ops.feature_cross_ragged(xv.to(DEV), xo.to(DEV), yv.to(DEV), yo.to(DEV), xw.to(DEV), yw.to(DEV))
    assert torch.equal(ref[0], got[0].cpu()) and torch.equal(ref[1], got[1].cpu()) and torch.allclose(ref[2], got[2].cpu())
    # the count per row is unique(x) * unique(y)
    for r in (1, 7, 100):
        ux = xv[xo[r]:xo[r + 1]].unique().numel(); uy = yv[yo[r]:yo[r + 1]].unique().numel()
        assert int(ref[1][r + 1] - ref[1][r]) == ux * uy
