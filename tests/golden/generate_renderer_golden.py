"""Generates tests/golden/renderer_vectors.npz: outputs of the reference renderer's own image
composition code (Renderer.py: render_image_train line 80, render_image_inference lines 105-125) on
small seeded images, run on the CPU.

    python tests/golden/generate_renderer_golden.py /path/to/INPC [OUT.npz]

The reference methods are called unmodified on a stand-in `self` whose rasterizer hands out prepared
(feature, depth, alpha) triples, whose U-Net is the identity and whose background model returns a
prepared image: what remains is exactly the accumulation / compose arithmetic.  NeRFICG packages the
module imports are replaced by empty stand-ins.
"""
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]


def load_renderer_class(ref_root: Path):
    for n in ["Framework", "Datasets", "Datasets.utils", "Methods", "Methods.Base", "Methods.Base.Renderer", "Methods.INPC",
              "Methods.INPC.Model", "Methods.INPC.utils", "Methods.INPC.INPCCudaBackend", "Visual", "Visual.utils"]:
        sys.modules.setdefault(n, types.ModuleType(n))

    class Configurable:
        @staticmethod
        def configure(**defaults):
            def deco(cls):
                for k, v in defaults.items():
                    setattr(cls, k, v)
                return cls
            return deco
    sys.modules["Framework"].Configurable = Configurable
    sys.modules["Datasets.utils"].View = object
    sys.modules["Methods.Base.Renderer"].BaseModel = object
    sys.modules["Methods.Base.Renderer"].BaseRenderer = object
    sys.modules["Methods.INPC.Model"].INPCModel = object
    for name in ("adjust_for_unet", "PreextractedPointCloud", "MultisamplingRingBuffer"):
        setattr(sys.modules["Methods.INPC.utils"], name, None)
    sys.modules["Methods.INPC.INPCCudaBackend"].INPCRasterizer = object
    sys.modules["Visual.utils"].apply_color_map = None
    spec = importlib.util.spec_from_file_location("ref_renderer", ref_root / "Renderer.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.INPCRenderer


class _Rasterizer:
    def __init__(self, triples):
        self.triples = list(triples)

    def render(self, *args, **kwargs):
        f, d, a = self.triples.pop(0)
        return f.clone(), d.clone(), a.clone()

    def __call__(self, *args, **kwargs):        # training forward: image, alpha, blending weights
        f, d, a = self.triples.pop(0)
        return f.clone(), a.clone(), torch.zeros(1)


def stand_in(cls, triples, background, n_multisamples, premultiplied):
    model = types.SimpleNamespace(
        background_model=lambda view, *a: background,
        probability_field=types.SimpleNamespace(generate_expected_samples=lambda *a, **k: None, generate_multisamples=lambda *a, **k: None,
                                                generate_training_samples=lambda *a, **k: (None, None)),
        appearance_field=lambda *a, **k: (None, None), unet=lambda x: x, tone_mapper=None)
    return types.SimpleNamespace(N_MULTISAMPLES=n_multisamples, N_SAMPLES=0, USE_EXPECTED_SAMPLES=True, SPLATTING_MODE=0, SIGMA_WORLD_SCALE=1.0,
                                 SIGMA_CUTOFF=3.0, AVERAGE_WITH_PREMULTIPLIED_ALHPA=premultiplied, USE_COMPILED_UNET_INFERENCE=False,
                                 USE_DISTILLED_BG_TEXTURE_INFERENCE=False, model=model, rasterizer=_Rasterizer(triples))


def main(ref_root, out_path):
    cls = load_renderer_class(Path(ref_root))
    g = torch.Generator().manual_seed(51)
    C, H, W, n = 4, 20, 24, 4
    triples = []
    for _ in range(n):
        alpha = torch.rand((1, H, W), generator=g)
        alpha[alpha < 0.15] = 0.0                       # pixels no point reached
        alpha[alpha > 0.9] = 1.0                        # saturated pixels
        feats = torch.randn((C, H, W), generator=g) * alpha
        depth = torch.rand((1, H, W), generator=g) * 5 * (alpha > 0)
        triples.append((feats, depth, alpha))
    background = torch.randn((C, H, W), generator=g)
    out = dict(background=background.numpy())
    for i, (f, d, a) in enumerate(triples):
        out.update({f"sample{i}_image": f.numpy(), f"sample{i}_depth": d.numpy(), f"sample{i}_alpha": a.numpy()})
    for n_ms in (1, 3, 4):
        for premult in (True, False):
            r = cls.render_image_inference(stand_in(cls, triples[:n_ms], background, n_ms, premult), None, True)
            tag = f"n{n_ms}_{'premultiplied' if premult else 'straight'}"
            out.update({f"{tag}_feature_image": r["feature_image"].numpy(), f"{tag}_depth": r["depth"].numpy(),
                        f"{tag}_alpha": r["alpha"].numpy(), f"{tag}_alpha_sum": r["alpha_sum"].numpy()})
    r = cls.render_image_train(stand_in(cls, triples[:1], background, 1, True), None)
    out["train_feature_image"] = r["rgb"].numpy()
    np.savez_compressed(out_path, **out)
    print(f"wrote {out_path}: {len(out)} arrays")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else str(ROOT / "tests" / "golden" / "renderer_vectors.npz"))
