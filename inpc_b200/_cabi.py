"""ctypes binding of the C ABI declared in include/inpc_b200.h.

The shared library is the product; this module only loads it and declares the prototypes.  There is
no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
# INPC_B200_LIB selects another build of the same library (e.g. one compiled with different tuning macros)
LIB_PATH = Path(os.environ.get("INPC_B200_LIB", _PKG / "libinpc_b200.so"))

ALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_size_t)


class InpcError(RuntimeError):
    """Raised when an entry point of libinpc_b200 returns a non-zero status."""


class View(C.Structure):
    """struct inpc_view."""
    _fields_ = [("w2c", C.c_void_p), ("cam_position", C.c_void_p), ("width", C.c_int32), ("height", C.c_int32),
                ("fx", C.c_float), ("fy", C.c_float), ("cx", C.c_float), ("cy", C.c_float),
                ("near_plane", C.c_float), ("far_plane", C.c_float)]


class RasterState(C.Structure):
    """struct inpc_raster_state."""
    _fields_ = [("point_blob", C.c_void_p), ("instance_blob", C.c_void_p), ("n_points", C.c_int64),
                ("n_visible", C.c_int64), ("n_instances", C.c_int64), ("tile_size", C.c_int32), ("mode", C.c_int32),
                ("depth_key_base", C.c_uint32), ("depth_key_bits", C.c_int32), ("channels", C.c_int32),
                ("deferred_counts", C.c_int32)]


_P, _I, _L, _F, _Z = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t
_VP, _SP = C.POINTER(View), C.POINTER(RasterState)

# name -> (restype, argtypes); the order of the arguments is that of include/inpc_b200.h
PROTOTYPES = {
    "inpc_last_error": (C.c_char_p, []),
    "inpc_version": (_I, []),
    "inpc_launch_count": (C.c_longlong, []),
    "inpc_profile_enable": (_I, [_I]),
    "inpc_profile_read": (_I, [C.POINTER(C.c_double), C.POINTER(C.c_longlong), _I, _I]),
    "inpc_rasterize_forward": (_I, [_I, _I, _VP, _L, _P, _P, _P, _P, _P, _P, ALLOC_FN, ALLOC_FN, _P, _SP, _P]),
    "inpc_rasterize_backward": (_I, [_SP, _VP, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "inpc_render": (_I, [_I, _I, _VP, _L, _P, _P, _F, _F, _P, _P, _P, ALLOC_FN, ALLOC_FN, _P, _P]),
    "inpc_render_multi": (_I, [_I, _VP, _I, C.POINTER(_L), C.POINTER(_P), C.POINTER(_P), _P, _P, _P, ALLOC_FN, ALLOC_FN, _P, _P]),
    "inpc_render_preextracted": (_I, [_I, _I, _VP, _L, _P, _P, _P, _P, _F, _F, _P, _P, _P, ALLOC_FN, ALLOC_FN, _P, _P]),
    "inpc_rasterize_rows_forward": (_I, [_I, _VP, _L, _P, _P, _I, _P, _P, _P, _P, ALLOC_FN, ALLOC_FN, _P, _SP, _P]),
    "inpc_rasterize_rows_backward": (_I, [_SP, _VP, _P, _P, _P, _P, _P, _P, _P, _P]),
    "inpc_render_rows": (_I, [_I, _VP, _L, _P, _P, _I, _P, _P, _P, _P, ALLOC_FN, ALLOC_FN, _P, _P]),
    "inpc_raster_debug_copy": (_I, [_SP, _VP, _I, _P, _P]),
    "inpc_raster_resolve": (_I, [_SP, _P]),
    "inpc_sort_workspace_bytes": (_Z, [_L]),
    "inpc_sort_pairs": (_I, [_P, _P, _P, _P, _L, _I, _P, C.POINTER(C.c_int), _P]),
    "inpc_sort_pairs_static": (_I, [_P, _P, _P, _P, _L, _I, C.POINTER(C.c_int), _P]),
    "inpc_sort_pairs_static_status": (_I, [_P, C.POINTER(C.c_uint)]),
    "inpc_debug_sort_lookback_timeout": (_I, [_P, _P, _P, _P, _L, _I, _P, C.POINTER(C.c_longlong), _P]),
    "inpc_last_call_ticket": (C.c_longlong, []),
    "inpc_call_status": (_I, [C.c_longlong, C.POINTER(C.c_uint)]),
    "inpc_sampler_exhausted": (_I, [_P]),
    "inpc_compute_viewpoint_weights": (_I, [_VP, _L, _P, _P, _P, _F, _P, _P]),
    "inpc_sampler_create": (_P, [_L]),
    "inpc_sampler_destroy": (None, [_P]),
    "inpc_sampler_get_counter": (C.c_uint64, [_P]),
    "inpc_sampler_set_counter": (None, [_P, C.c_uint64]),
    "inpc_sampler_workspace_bytes": (_Z, [_L]),
    "inpc_generate_training_samples": (_I, [_P, _VP, _L, _P, _P, _P, _F, _L, _P, _P, _P, _P]),
    "inpc_generate_samples": (_I, [_P, _VP, _L, _P, _P, _P, _F, _L, _P, C.POINTER(_L), _P, _P]),
    "inpc_generate_expected_samples_count": (_I, [_P, _VP, _L, _P, _P, _P, _F, _L, C.POINTER(_L), _P, _P]),
    "inpc_generate_expected_samples_fill": (_I, [_P, _L, _P, _P, _F, _L, _L, _P, _P, _P]),
    "inpc_draw_leaves": (_I, [_P, _L, _P, _L, _P, _P]),
    "inpc_build_cdf": (_I, [_P, _L, _P, _P, _P, _P]),
    "inpc_weight_decay_grads": (_I, [_P, _P, _L, _I, _P]),
    "inpc_spherical_contraction": (_I, [_P, _P, _L, _P]),
    "inpc_cauchy_workspace_bytes": (_Z, [_L]),
    "inpc_cauchy_loss": (_I, [_P, _P, _L, _P, _P, _P]),
    "inpc_cauchy_loss_backward": (_I, [_P, _P, _P, _L, _P, _P]),
    "inpc_leaf_stats_reset": (_I, [_P, _L, _P]),
    "inpc_leaf_stats_accumulate": (_I, [_P, _P, _L, _P, _L, _P]),
    "inpc_leaf_update": (_I, [_P, _P, _P, _L, _F, _P]),
    "inpc_draw_leaf_counts": (_I, [_P, _L, _P, _L, _P, _P, _P]),
    "inpc_halton_samples": (_I, [_P, _L, _P, _P, _F, _L, _P, _P, _P]),
    "inpc_morton_workspace_bytes": (_Z, [_L]),
    "inpc_morton_order": (_I, [_P, _L, C.POINTER(C.c_float), _F, _P, _P, _P]),
    "inpc_compose_background": (_I, [_P, _P, _P, _I, _L, _P, _P]),
    "inpc_compose_background_backward": (_I, [_P, _P, _P, _I, _L, _P, _P, _P]),
    "inpc_multisample_accumulate": (_I, [_P, _P, _P, _P, _P, _P, _I, _L, _I, _I, _P]),
    "inpc_multisample_resolve": (_I, [_P, _P, _P, _P, _P, _I, _L, _I, _I, _P]),
    "inpc_leaf_select_workspace_bytes": (_Z, [_L]),
    "inpc_leaf_select_count": (_I, [_I, _P, _P, _L, _F, _I, _P, C.POINTER(_L), _P]),
    "inpc_leaf_prune_fill": (_I, [_P, _P, _P, _P, _L, _F, _P, _P, _P, _P, _P, _P]),
    "inpc_leaf_subdivide_fill": (_I, [_P, _P, _P, _P, _L, _F, _I, _F, _L, _P, _P, _P, _P, _P, _P]),
}

_lib = None


def lib() -> C.CDLL:
    """Loads libinpc_b200.so (once).  Raises if it has not been built: there is no other path."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise InpcError(f"{LIB_PATH} is missing: build it with `python -m inpc_b200._build` "
                            "(nvcc, sm_100a). inpc_b200 has no fallback implementation.")
        handle = C.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != 0:
        msg = lib().inpc_last_error()
        raise InpcError(f"inpc_b200 error {status}: {msg.decode() if msg else ''}")


STAGES = ("sample", "preprocess", "sort_depth", "instances", "sort_tile", "blend_fwd", "blend_bwd", "preprocess_bwd")


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib().inpc_launch_count())


def profile_enable(on: bool) -> None:
    check(lib().inpc_profile_enable(1 if on else 0))


def profile_read(reset: bool = True) -> dict:
    """Per-stage device time since the last reset: {stage: (total milliseconds, timed scopes)}."""
    ms = (C.c_double * len(STAGES))()
    calls = (C.c_longlong * len(STAGES))()
    check(lib().inpc_profile_read(ms, calls, len(STAGES), 1 if reset else 0))
    return {name: (float(ms[i]), int(calls[i])) for i, name in enumerate(STAGES)}
