"""GPU tests of the global point-cloud extraction (leaf counts, Halton placement, Morton order) through
the Python mirror and hence the C ABI.  The Halton placement is bit-exact against the output of the
reference's own `extract_global` (tests/golden/extract_vectors.npz); the multinomial counts are checked
by distribution (the reference uses torch's generator); the Morton order by its defining properties."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _golden():
    return np.load(Path(__file__).resolve().parent / "golden" / "extract_vectors.npz")


def test_halton_samples_reproduce_the_reference():
    from inpc_b200.sampling import halton_samples
    g = _golden()
    out = halton_samples(torch.from_numpy(g["counts"]).to(DEV), torch.from_numpy(g["centers"]).to(DEV), torch.from_numpy(g["levels"]).to(DEV),
                         float(g["initial_size"]))
    np.testing.assert_array_equal(out.cpu().numpy(), g["samples"])


def test_halton_samples_match_restatement_with_deep_sequences():
    from inpc_b200.sampling import halton_samples
    gen = torch.Generator().manual_seed(71)
    n_leaves = 3000
    counts = torch.randint(0, 4, (n_leaves,), generator=gen, dtype=torch.int32)
    counts[17] = 5000                                             # Halton indices far beyond the first few digits
    counts[1999] = 1
    centers = (torch.rand((n_leaves, 3), generator=gen) * 2 - 1)
    levels = torch.randint(0, 11, (n_leaves,), generator=gen, dtype=torch.int32)
    out = halton_samples(counts.to(DEV), centers.to(DEV), levels.to(DEV), 2.0)
    np.testing.assert_array_equal(out.cpu().numpy(), O.halton_samples(counts.numpy(), centers.numpy(), levels.numpy(), 2.0))
    empty = halton_samples(torch.zeros(n_leaves, dtype=torch.int32, device=DEV), centers.to(DEV), levels.to(DEV), 2.0)
    assert empty.shape == (0, 3)


def test_leaf_counts_follow_the_weights():
    from inpc_b200 import ProbabilityFieldSampler
    gen = torch.Generator().manual_seed(72)
    n_leaves, n = 2000, 4_000_000
    w = torch.rand(n_leaves, generator=gen) ** 3
    w[::7] = 0.0
    s = ProbabilityFieldSampler(5)
    counts = s.draw_leaf_counts(w.to(DEV), n)
    assert counts.dtype == torch.int32 and int(counts.sum()) == n
    c = counts.cpu().double()
    assert torch.all(c[w == 0] == 0)
    expected = (w.double() / w.double().sum()) * n
    # binomial standard deviation sqrt(n p (1 - p)): 6 sigma plus the CDF's fixed-point resolution
    assert torch.all((c - expected).abs() <= 6 * expected.clamp_min(1).sqrt() + 4)
    again = ProbabilityFieldSampler(5).draw_leaf_counts(w.to(DEV), n)
    assert torch.equal(again, counts)                              # same seed and call counter: same draw
    assert not torch.equal(s.draw_leaf_counts(w.to(DEV), n), counts)
    with pytest.raises(Exception):
        s.draw_leaf_counts(torch.zeros(n_leaves, device=DEV), 10)


def test_morton_order_is_a_sorted_permutation():
    from inpc_b200.sampling import morton_order
    gen = torch.Generator().manual_seed(73)
    pos = (torch.rand((300_000, 3), generator=gen) * torch.tensor([2.0, 1.0, 0.5]) - 0.7).to(DEV)
    out = morton_order(pos)
    assert out.shape == pos.shape
    # a permutation of the rows
    key = lambda p: p[:, 0].double() * 1e6 + p[:, 1].double() * 1e3 + p[:, 2].double()
    assert torch.equal(torch.sort(key(out)).values, torch.sort(key(pos)).values)
    # codes recomputed on the host are non-decreasing along the output
    lo = pos.amin(dim=0)
    extent = float((pos.amax(dim=0) - lo).max()) * (1.0 + 1e-6)
    q = (((out - lo) * (1.0 / extent)) * 1024.0).clamp(0, 1023).to(torch.int64).cpu().numpy()

    def spread(v):
        r = np.zeros_like(v)
        for b in range(10):
            r |= ((v >> b) & 1) << (3 * b)
        return r
    codes = spread(q[:, 0]) | (spread(q[:, 1]) << 1) | (spread(q[:, 2]) << 2)
    assert np.all(np.diff(codes) >= 0)
    assert morton_order(pos[:0]).shape == (0, 3)


def test_extract_global_end_to_end():
    import inpc_b200
    import synthetic_workloads as syn
    from inpc_b200.sampling import extract_global
    tree = syn.uniform_octree(4, seed=0).to(DEV)
    views = [v.to(DEV) for v in syn.orbit_views(3, seed=2, width=160, height=120, focal=140.0)]
    s = inpc_b200.ProbabilityFieldSampler(1)
    n = 200_000
    pts = extract_global(s, tree.centers, tree.levels, tree.weights, views, n, tree.initial_size, use_morton_order=True)
    assert pts.shape == (n, 3)
    # every point lies inside the root cube, and inside some leaf's cell
    assert float(pts.abs().max()) <= 1.0 + 1e-6
    plain = extract_global(inpc_b200.ProbabilityFieldSampler(1), tree.centers, tree.levels, tree.weights, views, n, tree.initial_size,
                           use_morton_order=False)
    key = lambda p: p[:, 0].double() * 1e6 + p[:, 1].double() * 1e3 + p[:, 2].double()
    assert torch.equal(torch.sort(key(pts)).values, torch.sort(key(plain)).values)
