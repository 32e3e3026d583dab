"""Generates tests/golden/octree_vectors.npz: outputs of the reference's own torch code for the octree
probability field (Modules/ProbabilityField.py: update, prune, subdivide) on small seeded inputs.

Run on the CPU from the repository root, with the reference tree at hand:

    python tests/golden/generate_octree_golden.py /path/to/INPC [OUT.npz]

The reference module imports NeRFICG packages that are not installed; they are replaced by empty
stand-ins, which is enough because the three methods only touch torch and the module's own leaf
buffers.  The module object is created without running its constructor (which needs the CUDA
backend); the buffers are registered by hand as `ProbabilityField.initialize` does.
"""
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]


def load_reference_class(ref_root: Path):
    names = ["Framework", "Logging", "Datasets", "Datasets.Base", "Datasets.utils", "Methods", "Methods.INPC", "Methods.INPC.utils",
             "Methods.INPC.INPCCudaBackend", "CudaUtils", "CudaUtils.MortonEncoding"]
    for n in names:
        sys.modules.setdefault(n, types.ModuleType(n))
    sys.modules["Logging"].Logger = object
    sys.modules["Datasets.Base"].BaseDataset = object
    sys.modules["Datasets.utils"].tensor_to_string = str
    sys.modules["Datasets.utils"].View = object
    sys.modules["Methods.INPC.utils"].compute_halton_coords = None
    sys.modules["Methods.INPC.INPCCudaBackend"].ProbabilityFieldSampler = object
    sys.modules["Methods.INPC.INPCCudaBackend"].compute_viewpoint_weights = None
    sys.modules["CudaUtils.MortonEncoding"].morton_encode = None
    spec = importlib.util.spec_from_file_location("ref_probability_field", ref_root / "Modules" / "ProbabilityField.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.ProbabilityField


def make_field(cls, centers, levels, weights, scores, initial_size):
    f = cls.__new__(cls)
    torch.nn.Module.__init__(f)
    f.register_buffer("initial_cell_size", torch.tensor(initial_size, dtype=torch.float32).expand(3))
    f.register_buffer("leaf_centers", centers.clone())
    f.register_buffer("leaf_levels", levels.clone())
    f.register_buffer("leaf_weights", weights.clone())
    f.register_buffer("leaf_subdivision_scores", scores.clone())
    return f


def leaf_arrays(f, prefix):
    return {f"{prefix}_centers": f.leaf_centers.numpy().copy(), f"{prefix}_levels": f.leaf_levels.numpy().copy(),
            f"{prefix}_weights": f.leaf_weights.numpy().copy(), f"{prefix}_scores": f.leaf_subdivision_scores.numpy().copy()}


def main(ref_root, out_path):
    cls = load_reference_class(Path(ref_root))
    g = torch.Generator().manual_seed(31)
    n_leaves, n_samples, initial_size = 3000, 20000, 0.37
    centers = (torch.rand((n_leaves, 3), generator=g) * 2 - 1).contiguous()
    levels = torch.randint(0, 8, (n_leaves,), generator=g, dtype=torch.int32)
    weights = torch.rand((n_leaves,), generator=g)
    scores = torch.rand((n_leaves,), generator=g)
    out = dict(centers=centers.numpy(), levels=levels.numpy(), weights=weights.numpy(), scores=scores.numpy(),
               initial_size=np.float32(initial_size))

    # update: some leaves unsampled, some sampled once, some many times
    indices = torch.randint(0, n_leaves * 3 // 4, (n_samples,), generator=g, dtype=torch.int64)
    sample_w = torch.rand((n_samples, 1), generator=g) ** 3
    f = make_field(cls, centers, levels, weights, scores, initial_size)
    f.update(indices, sample_w)
    out.update(update_indices=indices.numpy(), update_sample_weights=sample_w.numpy(), **leaf_arrays(f, "updated"))

    for k, thr in enumerate((0.25, 0.9)):
        f = make_field(cls, centers, levels, weights, scores, initial_size)
        f.prune(thr)
        out.update({f"prune{k}_threshold": np.float32(thr), **leaf_arrays(f, f"prune{k}")})
    for k, thr in enumerate((0.5, 0.97)):
        f = make_field(cls, centers, levels, weights, scores, initial_size)
        f.subdivide(thr)
        out.update({f"subdivide{k}_threshold": np.float32(thr), **leaf_arrays(f, f"subdivide{k}")})
    np.savez_compressed(out_path, **out)
    print(f"wrote {out_path}: {len(out)} arrays")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else str(ROOT / "tests" / "golden" / "octree_vectors.npz"))
