"""GPU tests of the octree structure kernels (prune, subdivide) through the Python mirror and hence the
C ABI: bit-exact against the numpy restatement of the reference's torch code, which is itself pinned by
tests/golden/octree_vectors.npz (outputs of the reference code)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("centers", "levels", "weights", "scores")


def _golden():
    return np.load(Path(__file__).resolve().parent / "golden" / "octree_vectors.npz")


def _dev(g):
    return (torch.from_numpy(g["centers"]).to(DEV), torch.from_numpy(g["levels"]).to(DEV), torch.from_numpy(g["weights"]).to(DEV),
            torch.from_numpy(g["scores"]).to(DEV))


def _random_octree(n, seed):
    g = torch.Generator().manual_seed(seed)
    return dict(centers=(torch.rand((n, 3), generator=g) * 2 - 1).numpy(), levels=torch.randint(0, 9, (n,), generator=g, dtype=torch.int32).numpy(),
                weights=torch.rand((n,), generator=g).numpy(), scores=torch.rand((n,), generator=g).numpy())


def _assert_same(out, ref):
    assert len(out) == 4
    for a, b, name in zip(out, ref, NAMES):
        assert a.shape == b.shape, name
        np.testing.assert_array_equal(a.cpu().numpy(), b, err_msg=name)


def test_prune_and_subdivide_reproduce_the_reference_outputs():
    from inpc_b200 import probability_field as PF
    g = _golden()
    for k in range(2):
        _assert_same(PF.prune(*_dev(g), float(g[f"prune{k}_threshold"])), [g[f"prune{k}_{n}"] for n in NAMES])
        _assert_same(PF.subdivide(*_dev(g), float(g[f"subdivide{k}_threshold"]), float(g["initial_size"])),
                     [g[f"subdivide{k}_{n}"] for n in NAMES])


@pytest.mark.parametrize("n", [1, 1023, 1024, 1025, 300_001, 2_500_000])
def test_prune_and_subdivide_match_oracle_at_ragged_sizes(n):
    from inpc_b200 import probability_field as PF
    t = _random_octree(n, n)
    args = _dev(t)
    _assert_same(PF.prune(*args, 0.4), O.leaf_prune(t["centers"], t["levels"], t["weights"], t["scores"], 0.4))
    _assert_same(PF.subdivide(*args, 0.8, 2.0), O.leaf_subdivide(t["centers"], t["levels"], t["weights"], t["scores"], 0.8, 2.0))


def test_octree_edge_cases():
    from inpc_b200 import probability_field as PF
    t = _random_octree(5000, 7)
    args = _dev(t)
    none_kept = PF.prune(*args, 2.0)
    assert [x.shape[0] for x in none_kept] == [0, 0, 0, 0]
    _assert_same(PF.prune(*args, -1.0), [t[n] for n in NAMES])                         # everything kept
    _assert_same(PF.subdivide(*args, 2.0, 2.0), [t[n] for n in NAMES])                 # nothing split
    deep = (args[0], torch.full_like(args[1], 6), args[2], args[3])
    _assert_same(PF.subdivide(*deep, -1.0, 2.0), [t["centers"], np.full(5000, 6, np.int32), t["weights"], t["scores"]])   # level limit
    assert PF.subdivide(*args, -1.0, 2.0, max_level=20, max_leaves=8 * 5000 - 1) is None                                    # leaf cap
    all_split = PF.subdivide(*args, -1.0, 2.0, max_level=20)
    _assert_same(all_split, O.leaf_subdivide(t["centers"], t["levels"], t["weights"], t["scores"], -1.0, 2.0, max_level=20))
    assert all_split[0].shape[0] == 8 * 5000
    empty = (torch.empty((0, 3), device=DEV), torch.empty(0, dtype=torch.int32, device=DEV), torch.empty(0, device=DEV), torch.empty(0, device=DEV))
    assert PF.prune(*empty, 0.5)[0].shape == (0, 3) and PF.subdivide(*empty, 0.5, 2.0)[0].shape == (0, 3)
    with pytest.raises(TypeError):
        PF.prune(args[0], args[1].long(), args[2], args[3], 0.5)
    with pytest.raises(ValueError):
        PF.prune(args[0][:10], args[1], args[2], args[3], 0.5)


def test_update_reproduces_the_reference_outputs():
    from inpc_b200 import probability_field as PF
    g = _golden()
    w = torch.from_numpy(g["weights"]).to(DEV).clone()
    s = torch.from_numpy(g["scores"]).to(DEV).clone()
    PF.update_from_samples(w, s, torch.from_numpy(g["update_indices"]).to(DEV), torch.from_numpy(g["update_sample_weights"]).to(DEV))
    np.testing.assert_array_equal(w.cpu().numpy(), g["updated_weights"])
    np.testing.assert_array_equal(s.cpu().numpy(), g["updated_scores"])
