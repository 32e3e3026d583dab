"""Generates tests/golden/extract_vectors.npz: outputs of the reference's own `extract_global`
(Modules/ProbabilityField.py:121-144) with its own Halton code (utils.py:36-64) on a small seeded
octree, run on the CPU.

    python tests/golden/generate_extract_golden.py /path/to/INPC [OUT.npz]

The multinomial draw is torch's and cannot be reproduced elsewhere, so the fixture records the counts
it produced; everything after the draw (Halton indices per leaf, placement, single-sample leaves) is
deterministic.  NeRFICG packages are replaced by empty stand-ins; the viewpoint weights of the two
"training views" are prepared arrays.
"""
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]


def load(ref_root: Path):
    for n in ["Framework", "Logging", "Datasets", "Datasets.Base", "Datasets.utils", "Methods", "Methods.INPC", "Methods.INPC.INPCCudaBackend",
              "CudaUtils", "CudaUtils.MortonEncoding", "Cameras", "Cameras.Perspective"]:
        sys.modules.setdefault(n, types.ModuleType(n))
    sys.modules["Cameras.Perspective"].PerspectiveCamera = object
    spec = importlib.util.spec_from_file_location("Methods.INPC.utils", ref_root / "utils.py")
    utils = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(utils)
    sys.modules["Methods.INPC.utils"] = utils

    class Logger:
        @staticmethod
        def log_progress(it, **kwargs):
            return it
    sys.modules["Logging"].Logger = Logger
    sys.modules["Datasets.Base"].BaseDataset = object
    sys.modules["Datasets.utils"].tensor_to_string = str
    sys.modules["Datasets.utils"].View = object
    sys.modules["Methods.INPC.INPCCudaBackend"].ProbabilityFieldSampler = object
    sys.modules["CudaUtils.MortonEncoding"].morton_encode = None
    view_weights = {}
    sys.modules["Methods.INPC.INPCCudaBackend"].compute_viewpoint_weights = lambda centers, levels, weights, view, initial_size: view_weights[view]
    spec = importlib.util.spec_from_file_location("ref_probability_field2", ref_root / "Modules" / "ProbabilityField.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.ProbabilityField, utils, view_weights


def main(ref_root, out_path):
    cls, utils, view_weights = load(Path(ref_root))
    g = torch.Generator().manual_seed(61)
    n_leaves, n_samples, initial_size = 700, 6000, 0.23
    centers = (torch.rand((n_leaves, 3), generator=g) * 2 - 1).contiguous()
    levels = torch.randint(0, 7, (n_leaves,), generator=g, dtype=torch.int32)
    weights = torch.rand((n_leaves,), generator=g) ** 6          # a few heavy leaves, many with one or no sample
    view_weights["view0"] = weights * (torch.rand((n_leaves,), generator=g) > 0.3)
    view_weights["view1"] = weights * 0.5 * (torch.rand((n_leaves,), generator=g) > 0.3)
    f = cls.__new__(cls)
    torch.nn.Module.__init__(f)
    f.register_buffer("initial_cell_size", torch.tensor(initial_size, dtype=torch.float32).expand(3))
    f.register_buffer("leaf_centers", centers)
    f.register_buffer("leaf_levels", levels)
    f.register_buffer("leaf_weights", weights)
    f.training_views = ["view0", "view1"]
    drawn = []
    real_multinomial = torch.multinomial

    def recording_multinomial(*args, **kwargs):
        out = real_multinomial(*args, **kwargs)
        drawn.append(out)
        return out
    torch.manual_seed(62)
    torch.multinomial = recording_multinomial
    try:
        samples = f.extract_global(n_samples, False)
    finally:
        torch.multinomial = real_multinomial
    counts = torch.bincount(drawn[0], minlength=n_leaves).to(torch.int32)
    halton = utils.generate_halton_sequence(40, 3)
    np.savez_compressed(out_path, centers=centers.numpy(), levels=levels.numpy(), weights=weights.numpy(), initial_size=np.float32(initial_size),
                        global_weights=torch.maximum(view_weights["view0"], view_weights["view1"]).numpy(), counts=counts.numpy(),
                        samples=samples.numpy(), halton_first_40=halton.numpy())
    print(f"wrote {out_path}: {samples.shape[0]} samples, {int((counts == 1).sum())} single-sample leaves, max count {int(counts.max())}")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else str(ROOT / "tests" / "golden" / "extract_vectors.npz"))
