"""TEST INFRASTRUCTURE — ctypes front-end of oracle/_ref/libinpc_ref.so, the reference's own CUDA
native layer compiled unmodified (oracle/Makefile, target `ref`) behind the shim oracle/ref_shim.cu.

Used by the GPU parity tests, the golden-vector generator (tests/golden/generate_golden.py) and the
reference arm of bench.py.  The product never imports this module.  Tensors are torch CUDA tensors;
the reference launches on the legacy default stream, so callers synchronise around these calls.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "_ref" / "libinpc_ref.so"
_lib = None


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(f"{LIB_PATH} not built (make -C oracle ref; needs the reference tree)")
        _lib = C.CDLL(str(LIB_PATH))
        _lib.inpcref_intermediate.restype = C.c_void_p
    return _lib


def _p(t):
    return C.c_void_p(0 if t is None or t.numel() == 0 else t.data_ptr())


def _cam_args(view):
    c = view.camera
    return (C.c_int(int(c.width)), C.c_int(int(c.height)), C.c_float(c.focal_x), C.c_float(c.focal_y),
            C.c_float(c.center_x), C.c_float(c.center_y), C.c_float(c.near_plane), C.c_float(c.far_plane))


def _sync():
    rc = lib().inpcref_sync()
    if rc != 0:
        raise RuntimeError(f"reference backend reported CUDA error {rc}")


def forward(view, mode, positions, features, opacities, sync=True):
    """_C.forward (torch_bindings/rasterization.py:56-61)."""
    n = positions.shape[0]
    dev = positions.device
    H, W = view.camera.height, view.camera.width
    image = torch.empty((4, H, W), dtype=torch.float32, device=dev)
    alpha = torch.empty((1, H, W), dtype=torch.float32, device=dev)
    bw = torch.empty((n,), dtype=torch.float32, device=dev)
    torch.cuda.current_stream().synchronize()
    rc = lib().inpcref_forward(C.c_int(mode), _p(positions), _p(features), _p(opacities), _p(view.w2c), _p(view.position),
                               _p(image), _p(alpha), _p(bw), C.c_int(n), *_cam_args(view))
    if rc != 0:
        raise RuntimeError("inpcref_forward failed")
    if sync:
        _sync()
    return image, alpha, bw


def backward(view, mode, grad_image, grad_alpha, image, alpha, positions, opacities, sync=True):
    """_C.backward (torch_bindings/rasterization.py:88-95); uses the blobs of the last forward."""
    n = positions.shape[0]
    dev = positions.device
    gfv = torch.empty((n, 4), dtype=torch.float32, device=dev)
    gf = torch.empty((n, 36), dtype=torch.float16, device=dev)
    go = torch.empty((n, 1), dtype=torch.float32, device=dev)
    torch.cuda.current_stream().synchronize()
    rc = lib().inpcref_backward(C.c_int(mode), _p(grad_image), _p(grad_alpha), _p(image), _p(alpha), _p(positions),
                                _p(opacities), _p(view.position), _p(gfv), _p(gf), _p(go), C.c_int(n),
                                C.c_int(int(view.camera.width)), C.c_int(int(view.camera.height)))
    if rc != 0:
        raise RuntimeError("inpcref_backward failed")
    if sync:
        _sync()
    return gf, go, gfv


def render(view, mode, positions, features_raw, sigma_world, sigma_cutoff):
    n = positions.shape[0]
    dev = positions.device
    H, W = view.camera.height, view.camera.width
    image = torch.empty((4, H, W), dtype=torch.float32, device=dev)
    depth = torch.empty((1, H, W), dtype=torch.float32, device=dev)
    alpha = torch.empty((1, H, W), dtype=torch.float32, device=dev)
    torch.cuda.current_stream().synchronize()
    rc = lib().inpcref_render(C.c_int(mode), _p(positions), _p(features_raw), _p(view.w2c), _p(view.position), _p(image),
                              _p(depth), _p(alpha), C.c_int(n), *_cam_args(view), C.c_float(sigma_world),
                              C.c_float(sigma_cutoff))
    if rc != 0:
        raise RuntimeError("inpcref_render failed")
    _sync()
    return image, depth, alpha


def render_preextracted(view, mode, positions, features, opacities, scales, sigma_world, sigma_cutoff, sync=True):
    n = positions.shape[0]
    dev = positions.device
    H, W = view.camera.height, view.camera.width
    image = torch.empty((4, H, W), dtype=torch.float32, device=dev)
    depth = torch.empty((1, H, W), dtype=torch.float32, device=dev)
    alpha = torch.empty((1, H, W), dtype=torch.float32, device=dev)
    torch.cuda.current_stream().synchronize()
    rc = lib().inpcref_render_preextracted(C.c_int(mode), _p(positions), _p(features), _p(opacities), _p(scales),
                                           _p(view.w2c), _p(view.position), _p(image), _p(depth), _p(alpha), C.c_int(n),
                                           *_cam_args(view), C.c_float(sigma_world), C.c_float(sigma_cutoff))
    if rc != 0:
        raise RuntimeError("inpcref_render_preextracted failed")
    if sync:
        _sync()
    return image, depth, alpha


_INTERMEDIATE = {"depth_keys_a": 0, "depth_keys_b": 1, "point_ids_a": 2, "point_ids_b": 3, "n_touched": 4, "bounds": 5,
                 "screen": 6, "feat_view": 7, "depth": 8, "n_visible": 9, "n_instances": 10, "ranges": 11,
                 "inst_point": 12, "inst_keys_a": 13, "inst_keys_b": 14}


def intermediates(view, n):
    """Host copies of the reference's intermediate buffers after a bilinear training forward
    (8x8 tiles).  Sorted arrays are cut to the visible / instance counts."""
    import numpy as np
    W, H = int(view.camera.width), int(view.camera.height)
    n_tiles = (-(-W // 8)) * (-(-H // 8))
    L = lib()

    def fetch(name, count, dtype):
        ptr = L.inpcref_intermediate(C.c_int(_INTERMEDIATE[name]), C.c_int(W), C.c_int(H))
        if not ptr or count == 0:
            return np.zeros(0, dtype)
        out = np.empty(count, dtype)
        nbytes = out.nbytes
        err = L.inpcref_copy_to_host(C.c_void_p(out.ctypes.data), C.c_void_p(ptr), C.c_size_t(nbytes))
        if int(err) != 0:
            raise RuntimeError(f"cudaMemcpy failed: {err}")
        return out

    nv = int(fetch("n_visible", 1, np.uint32)[0])
    ni = int(fetch("n_instances", 1, np.uint32)[0])
    out = {"n_visible": nv, "n_instances": ni}
    out["n_touched"] = fetch("n_touched", n, np.uint32)
    out["bounds"] = fetch("bounds", 4 * n, np.uint16).reshape(n, 4)
    out["screen"] = fetch("screen", 2 * n, np.float32).reshape(n, 2)
    out["feat_view"] = fetch("feat_view", 4 * n, np.float32).reshape(n, 4)
    out["depth"] = fetch("depth", n, np.float32)
    for k in ("depth_keys_a", "depth_keys_b", "point_ids_a", "point_ids_b"):
        out[k] = fetch(k, nv, np.uint32)
    out["ranges"] = fetch("ranges", 2 * n_tiles, np.uint32).reshape(n_tiles, 2)
    out["inst_point"] = fetch("inst_point", ni, np.uint32)
    out["inst_keys_a"] = fetch("inst_keys_a", ni, np.uint16)
    out["inst_keys_b"] = fetch("inst_keys_b", ni, np.uint16)
    # the depth sort leaves its result in whichever ping-pong buffer is sorted
    a_sorted = bool(np.all(out["depth_keys_a"][:-1] <= out["depth_keys_a"][1:])) if nv > 1 else True
    out["sorted_depth_keys"] = out["depth_keys_a"] if a_sorted else out["depth_keys_b"]
    out["sorted_points"] = out["point_ids_a"] if a_sorted else out["point_ids_b"]
    return out


# ---- sampler ------------------------------------------------------------------------------------

def sampler_seed(seed: int) -> None:
    lib().inpcref_sampler_seed(C.c_longlong(seed))


def viewpoint_weights(view, centers, levels, weights, initial_size):
    n = centers.shape[0]
    out = torch.empty((n,), dtype=torch.float32, device=centers.device)
    c = view.camera
    torch.cuda.current_stream().synchronize()
    lib().inpcref_viewpoint_weights(_p(centers), _p(levels), _p(weights), _p(view.w2c), _p(out), C.c_uint(n),
                                    C.c_uint(int(c.width)), C.c_uint(int(c.height)), C.c_float(c.focal_x),
                                    C.c_float(c.focal_y), C.c_float(c.center_x), C.c_float(c.center_y),
                                    C.c_float(c.near_plane), C.c_float(c.far_plane), C.c_float(initial_size))
    _sync()
    return out


def _sampler_cam(view):
    c = view.camera
    return (C.c_uint(int(c.width)), C.c_uint(int(c.height)), C.c_float(c.focal_x), C.c_float(c.focal_y),
            C.c_float(c.center_x), C.c_float(c.center_y), C.c_float(c.near_plane), C.c_float(c.far_plane))


def training_samples(view, centers, levels, weights, n_samples, initial_size, sync=True):
    n = centers.shape[0]
    dev = centers.device
    vw = torch.empty((n,), dtype=torch.float32, device=dev)
    s = torch.empty((1,), dtype=torch.float32, device=dev)
    counter = torch.zeros((1,), dtype=torch.int32, device=dev)
    pos = torch.empty((n_samples, 3), dtype=torch.float32, device=dev)
    idx = torch.empty((n_samples,), dtype=torch.int64, device=dev)
    torch.cuda.current_stream().synchronize()
    lib().inpcref_training_samples(_p(centers), _p(levels), _p(weights), _p(view.w2c), _p(vw), _p(s), _p(pos), _p(idx),
                                   _p(counter), C.c_uint(n), C.c_uint(n_samples), *_sampler_cam(view),
                                   C.c_float(initial_size))
    if sync:
        _sync()
    return pos, idx, vw


def samples(view, centers, levels, weights, n_samples, initial_size):
    """Returns (positions, cdf): the second is the reference's own CDF, left in its weight buffer."""
    n = centers.shape[0]
    dev = centers.device
    vw = torch.empty((n,), dtype=torch.float32, device=dev)
    s = torch.empty((1,), dtype=torch.float32, device=dev)
    pos = torch.empty((n_samples, 3), dtype=torch.float32, device=dev)
    torch.cuda.current_stream().synchronize()
    written = lib().inpcref_samples(_p(centers), _p(levels), _p(weights), _p(view.w2c), _p(vw), _p(s), _p(pos),
                                    C.c_uint(n), C.c_uint(n_samples), *_sampler_cam(view), C.c_float(initial_size))
    _sync()
    return pos[:written], vw


def expected_samples(view, centers, levels, weights, n_samples, n_multi, initial_size):
    n = centers.shape[0]
    dev = centers.device
    vw = torch.empty((n,), dtype=torch.float32, device=dev)
    s = torch.empty((1,), dtype=torch.float32, device=dev)
    torch.cuda.current_stream().synchronize()
    created = lib().inpcref_expected_samples_count(_p(centers), _p(levels), _p(weights), _p(view.w2c), _p(vw), _p(s),
                                                   C.c_uint(n), C.c_uint(n_samples), *_sampler_cam(view),
                                                   C.c_float(initial_size))
    _sync()
    if created == 0:
        return torch.empty((0, 3), dtype=torch.float32, device=dev), vw, s
    cells = torch.empty((created,), dtype=torch.int32, device=dev)
    pos = torch.empty((created * n_multi, 3), dtype=torch.float32, device=dev)
    lib().inpcref_expected_samples_fill(_p(centers), _p(levels), _p(cells), _p(pos), C.c_uint(created), C.c_uint(n_multi),
                                        C.c_uint(n), C.c_float(initial_size))
    _sync()
    return pos, vw, s


# ---- misc -----------------------------------------------------------------------------------------

def weight_decay(weights, grads=None):
    add = grads is not None
    out = grads if add else torch.empty_like(weights)
    torch.cuda.current_stream().synchronize()
    lib().inpcref_weight_decay(_p(weights), _p(out), C.c_uint(weights.numel()), C.c_int(int(add)))
    _sync()
    return out


def contraction(positions):
    out = torch.empty_like(positions)
    torch.cuda.current_stream().synchronize()
    lib().inpcref_contraction(_p(positions), _p(out), C.c_uint(positions.shape[0]))
    _sync()
    return out


def cauchy(inp, tgt):
    ew = torch.empty_like(inp)
    torch.cuda.current_stream().synchronize()
    lib().inpcref_cauchy(_p(inp), _p(tgt), _p(ew), C.c_uint(inp.numel()))
    _sync()
    return ew.sum()


def cauchy_backward(grad, inp, tgt):
    out = torch.empty_like(inp)
    torch.cuda.current_stream().synchronize()
    lib().inpcref_cauchy_backward(_p(grad), _p(inp), _p(tgt), _p(out), C.c_uint(inp.numel()))
    _sync()
    return out
