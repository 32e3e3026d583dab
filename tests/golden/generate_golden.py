"""Generates tests/golden/reference_vectors.npz: outputs of the reference's own CUDA backend
(oracle/_ref/libinpc_ref.so, built unmodified from the reference tree) on small seeded inputs.

Run on a machine with a GPU from the repository root:

    python tests/golden/generate_golden.py            # writes tests/golden/reference_vectors.npz
    python tests/golden/generate_golden.py OUT.npz    # or to another path

The fixture pins the CPU oracle (tests/test_oracle_golden.py) without a GPU and without the
reference tree.  Nothing of the product is involved in producing it except the seeded input
generator and the depth-tie silencing, which needs per-point depths: those are taken from the
reference's own intermediate buffers.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path[:0] = [str(ROOT), str(ROOT / "oracle"), str(ROOT / "tests")]

import ref_backend as RB  # noqa: E402
from helpers import silence_depth_ties, small_scene  # noqa: E402
import synthetic_workloads as syn  # noqa: E402

DEV = "cuda:0"


def view_arrays(view):
    c = view.camera
    return dict(w2c=view.w2c.cpu().numpy(), cam_position=view.position.cpu().numpy(),
                cam=np.array([c.width, c.height, c.focal_x, c.focal_y, c.center_x, c.center_y, c.near_plane, c.far_plane], np.float64))


def main(out_path):
    out = {}
    # ---- rasterizer: rotated camera, culled points on all sides ---------------------------------
    view, pos, feats, opac = small_scene(n=3000, width=64, height=48, seed=3, focal=56.0)
    v = view.to(DEV)
    pos_d, feats_d = pos.to(DEV), feats.to(DEV)
    RB.forward(v, 0, pos_d, feats_d, opac.to(DEV).reshape(-1))
    first = RB.intermediates(v, pos.shape[0])
    opac_d = silence_depth_ties(first["depth"], first["n_touched"] > 0, opac.to(DEV))
    out.update({f"view_{k}": a for k, a in view_arrays(view).items()})
    out.update(positions=pos.numpy(), features=feats.numpy(), opacities=opac_d.cpu().numpy())
    g = torch.Generator().manual_seed(31)
    H, W = view.camera.height, view.camera.width
    gi = (torch.randn((4, H, W), generator=g) * 1e-3)
    ga = (torch.randn((1, H, W), generator=g) * 1e-3)
    out.update(grad_image=gi.numpy(), grad_alpha=ga.numpy())
    for mode, tag in ((0, "bil"), (1, "gau")):
        img, alpha, bw = RB.forward(v, mode, pos_d, feats_d, opac_d.reshape(-1))
        if mode == 0:
            inter = RB.intermediates(v, pos.shape[0])
            vis = inter["n_touched"] > 0
            for k in ("n_touched", "sorted_depth_keys", "ranges"):
                out[f"bil_{k}"] = inter[k]
            out["bil_bounds"] = np.where(vis[:, None], inter["bounds"], 0).astype(np.uint16)
            out["bil_depth"] = np.where(vis, inter["depth"], 0).astype(np.float32)
            out["bil_screen"] = np.where(vis[:, None], inter["screen"], 0).astype(np.float32)
            out["bil_feat_view"] = np.where(vis[:, None], inter["feat_view"], 0).astype(np.float32)
            # canonical order: ties by point id
            bits = inter["depth"].view(np.uint32).astype(np.int64)
            sp = inter["sorted_points"].astype(np.int64)
            out["bil_sorted_points"] = sp[np.argsort((bits[sp] << 32) | sp, kind="stable")].astype(np.uint32)
            ip = inter["inst_point"].astype(np.int64)
            lens = (inter["ranges"][:, 1] - inter["ranges"][:, 0]).astype(np.int64)
            tiles = np.repeat(np.arange(len(lens)), lens)
            out["bil_inst_point"] = ip[np.lexsort(((bits[ip] << 32) | ip, tiles))].astype(np.uint32)
        gf, go, gfv = RB.backward(v, mode, gi.to(DEV), ga.to(DEV), img, alpha, pos_d, opac_d.reshape(-1))
        out.update({f"{tag}_image": img.cpu().numpy(), f"{tag}_alpha": alpha.cpu().numpy(), f"{tag}_bw": bw.cpu().numpy(),
                    f"{tag}_grad_features": gf.cpu().numpy(), f"{tag}_grad_opacities": go.cpu().numpy(),
                    f"{tag}_grad_feat_view": gfv.cpu().numpy()})
        # inference variants
        g2 = torch.Generator().manual_seed(32)
        raw = torch.cat([torch.randn((pos.shape[0], 1), generator=g2).to(torch.float16), feats], dim=1).contiguous()
        raw[(opac_d.reshape(-1) == 0).cpu(), 0] = -30000.0
        scales = torch.rand((pos.shape[0],), generator=g2) * 0.01 + 0.002
        sw = 1.5 * 0.05 / view.camera.focal_y
        out["raw"] = raw.numpy()
        out["scales"] = scales.numpy()
        out["sigma"] = np.array([sw, 2.5], np.float64)
        i1 = RB.render(v, mode, pos_d, raw.to(DEV), sw, 2.5)
        i2 = RB.render_preextracted(v, mode, pos_d, feats_d, opac_d.reshape(-1), None, sw, 2.5)
        i3 = RB.render_preextracted(v, mode, pos_d, feats_d, opac_d.reshape(-1), scales.to(DEV), sw, 2.5)
        for name, trip in (("render", i1), ("pre", i2), ("pre_scales", i3)):
            for part, t in zip(("image", "depth", "alpha"), trip):
                out[f"{tag}_{name}_{part}"] = t.cpu().numpy()

    # ---- sampler --------------------------------------------------------------------------------
    tree = syn.adaptive_octree(4000, seed=7, min_level=3, max_level=6)
    sview = syn.orbit_view(0.8, -0.3, 2.2, 200, 150, 170.0)
    t, sv = tree.to(DEV), sview.to(DEV)
    out.update({f"sview_{k}": a for k, a in view_arrays(sview).items()})
    out.update(leaf_centers=tree.centers.numpy(), leaf_levels=tree.levels.numpy(), leaf_weights=tree.weights.numpy(),
               initial_size=np.array([tree.initial_size]))
    out["viewpoint_weights"] = RB.viewpoint_weights(sv, t.centers, t.levels, t.weights, tree.initial_size).cpu().numpy()
    RB.sampler_seed(2024)
    spos, cdf = RB.samples(sv, t.centers, t.levels, t.weights, 5000, tree.initial_size)
    out.update(samples_positions=spos.cpu().numpy(), samples_cdf=cdf.cpu().numpy(), samples_seed=np.array([2024]))
    epos, evw, esum = RB.expected_samples(sv, t.centers, t.levels, t.weights, 6000, 2, tree.initial_size)
    out.update(expected_positions=epos.cpu().numpy(), expected_sum=esum.cpu().numpy())
    tpos, tidx, _ = RB.training_samples(sv, t.centers, t.levels, t.weights, 20000, tree.initial_size)
    out.update(training_hist=np.bincount(tidx.cpu().numpy(), minlength=tree.centers.shape[0]).astype(np.int32))

    # ---- misc -----------------------------------------------------------------------------------
    g3 = torch.Generator().manual_seed(33)
    p = torch.randn((2000, 3), generator=g3) * 2
    a, b = torch.randn(5000, generator=g3), torch.randn(5000, generator=g3)
    w = torch.randn(30000, generator=g3)
    out.update(misc_points=p.numpy(), misc_contracted=RB.contraction(p.to(DEV)).cpu().numpy(), misc_a=a.numpy(), misc_b=b.numpy(),
               misc_cauchy=np.array([RB.cauchy(a.to(DEV), b.to(DEV)).item()]),
               misc_cauchy_grad=RB.cauchy_backward(torch.tensor([2.0], device=DEV), a.to(DEV), b.to(DEV)).cpu().numpy(),
               misc_w=w.numpy(), misc_decay=RB.weight_decay(w.to(DEV)).cpu().numpy())
    np.savez_compressed(out_path, **out)
    print(f"wrote {out_path}: {len(out)} arrays, {Path(out_path).stat().st_size / 1024:.0f} KiB")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else str(ROOT / "tests" / "golden" / "reference_vectors.npz"))
