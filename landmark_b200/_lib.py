"""ctypes binding of ``libgridnerf_b200.so`` (declared in ``include/gridnerf_b200.h``).

The library is the only implementation of the render path: if it is missing or does not
load, importing this module raises -- there is no Python or CPU fallback.
"""

from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libgridnerf_b200.so")

STAGE_NAMES = ("sample", "compact", "density", "weights", "compact_app", "app_gather", "mlp", "composite")
SAMPLE_STATIC_SCRATCH_BYTES = (4 << 20) + 4096
ST_OVERFLOW_VALID, ST_OVERFLOW_APP, ST_NUM_VALID, ST_NUM_APP, ST_WAIT_EXPIRED, ST_NUM_DENSITY, ST_WORDS = 0, 1, 2, 3, 4, 5, 8


class GnrConfig(C.Structure):
    _fields_ = [
        ("aabb", C.c_float * 6),
        ("inv_aabb_size", C.c_float * 3),
        ("grid", C.c_int32 * 3),
        ("near_t", C.c_float),
        ("far_t", C.c_float),
        ("step_size", C.c_float),
        ("distance_scale", C.c_float),
        ("density_shift", C.c_float),
        ("density_act", C.c_int32),
        ("ray_weight_thres", C.c_float),
        ("alpha_filter_thres", C.c_float),
        ("n_pairs", C.c_int32),
        ("n_density", C.c_int32),
        ("n_app", C.c_int32),
        ("app_dim", C.c_int32),
        ("fea_pe", C.c_int32),
        ("view_pe", C.c_int32),
        ("hidden", C.c_int32),
        ("has_bias", C.c_int32),
        ("mlp_mode", C.c_int32),
        ("sampling_mode", C.c_int32),
        ("ert_transmittance", C.c_float),
        ("app_storage", C.c_int32),
        ("den_storage", C.c_int32),
        ("unfused_appearance", C.c_int32),
        ("reserved", C.c_int32 * 3),
    ]


_P = C.c_void_p
_I64 = C.c_int64
_INT = C.c_int
_SZ = C.c_size_t

# name -> (restype, argtypes); this table is also what the symbol-export test walks.
SIGNATURES = {
    "gnr_last_error": (C.c_char_p, []),
    "gnr_version": (_INT, []),
    "gnr_create": (_INT, [C.POINTER(GnrConfig), _INT, C.POINTER(_P)]),
    "gnr_destroy": (_INT, [_P]),
    "gnr_upload_plane": (_INT, [_P, _INT, _INT, _P, _INT, _INT, _INT, _INT, _INT, _P]),
    "gnr_upload_line": (_INT, [_P, _INT, _INT, _P, _INT, _INT, _INT, _P]),
    "gnr_upload_alpha_mask": (_INT, [_P, _P, _INT, _INT, _INT, C.POINTER(C.c_float), C.POINTER(C.c_float), _P]),
    "gnr_upload_mlp": (_INT, [_P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "gnr_build_density_lattice": (_INT, [_P, _INT, _P]),
    "gnr_build_appearance_lattice": (_INT, [_P, _INT, _P]),
    "gnr_upload_hull_tables": (_INT, [_P, _INT, _P, _P, _P]),
    "gnr_generate_rays": (_INT, [C.POINTER(C.c_float), _P, _P, _INT, _INT, _P, _I64, _I64, _P, _P]),
    "gnr_generate_rays_dev": (_INT, [_P, _P, _P, _INT, _INT, _P, _I64, _I64, _P, _P]),
    "gnr_rgba8": (_INT, [_P, _I64, _P, _P]),
    "gnr_workspace_bytes": (_INT, [_P, _I64, _INT, _I64, _I64, C.POINTER(_SZ)]),
    "gnr_render_chunk": (_INT, [_P, _P, _I64, _INT, _INT, _P, _SZ, _I64, _I64, _P, _P, _P]),
    "gnr_render_host": (_INT, [_P, _P, _I64, _INT, _INT, _I64, _I64, _I64, _P, _P, C.POINTER(C.c_int32)]),
    "gnr_sample": (_INT, [_P, _P, _I64, _INT, _P, _SZ, _I64, _P, _P, _P, _P, _P, _P]),
    "gnr_sample_bits": (_INT, [_INT]),
    "gnr_sample_static": (_INT, [_P, _P, _I64, _INT, _I64, _P, _P, _P, _P, _P, _P]),
    "gnr_density": (_INT, [_P, _P, _I64, _INT, _P, _SZ, _I64, _P, _P, _P]),
    "gnr_weights": (_INT, [_P, _P, _I64, _INT, _P, _SZ, _I64, _I64, _P, _P, _P, _P, _P, _P, _P]),
    "gnr_march": (_INT, [_P, _P, _I64, _INT, _P, _SZ, _I64, _I64, _P, _P, _P, _P, _P, _P, _P]),
    "gnr_appearance": (_INT, [_P, _P, _I64, _INT, _P, _SZ, _I64, _I64, _P, _P, _P]),
    "gnr_composite": (_INT, [_P, _I64, _INT, _P, _SZ, _I64, _I64, _INT, _P, _P, _P]),
    "gnr_valid_positions": (_INT, [_P, _P, _I64, _INT, _P, _SZ, _I64, _P, _P, _P]),
    "gnr_route_blocks": (_INT, [_P, _P, _I64, _INT, _P, _SZ, _I64, _I64, _INT, _INT, _INT, _P, _P, _P, _P, _P]),
    "gnr_density_points": (_INT, [_P, _P, _I64, _P, _P, _P]),
    "gnr_weights_from_sigma": (_INT, [_P, _I64, _INT, _P, _SZ, _I64, _I64, _P, _P, _P]),
    "gnr_app_features": (_INT, [_P, _P, _I64, _INT, _P, _SZ, _I64, _I64, _P, _I64, _P]),
    "gnr_points_scratch_bytes": (_INT, [_P, _I64, C.POINTER(_SZ)]),
    "gnr_appearance_points": (_INT, [_P, _P, _P, _I64, _P, _SZ, _P, _P, _P]),
    "gnr_appearance_rows": (_INT, [_P, _P, _I64, _P, _SZ, _P, _P]),
    "gnr_weights_from_rows": (_INT, [_P, _I64, C.c_int, _P, _SZ, _I64, _I64, _P, _P, _P]),
    "gnr_route_block_ids": (_INT, [_P, _P, _I64, C.c_int, _P, _SZ, _I64, _I64, C.c_int, C.c_int, C.c_int, C.c_uint32,
                                   _P, _P, _P, _P]),
    "gnr_query_one_kernel_appearance": (_INT, [_P]),
    "gnr_density_list": (_INT, [_P, _P, _P, _P, _P, _I64, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P]),
    "gnr_appearance_list": (_INT, [_P, _P, _P, _P, _P, _I64, C.c_int, C.c_int, C.c_int, C.c_int, _P, _SZ, _P, _P]),
    "gnr_project_slice_points": (_INT, [_P, _P, C.c_int, _I64, _P, _P, _P]),
    "gnr_mlp_partial_rows": (_INT, [_P, _P, C.c_int, _I64, _P, _I64, _P, _SZ, _P, _P]),
    "gnr_sum_partials": (_INT, [_P, _P, C.c_int, _I64, _I64, _P, _P]),
    "gnr_app_features_points": (_INT, [_P, _P, _I64, _P, _SZ, _P, _P]),
    "gnr_mlp_features": (_INT, [_P, _P, _P, _I64, _P, _SZ, _P, _P]),
    "gnr_composite_rgb": (_INT, [_P, _I64, _INT, _P, _SZ, _I64, _I64, _INT, _P, _I64, _P, _P, _P]),
    "gnr_profile_enable": (_INT, [_P, _INT]),
    "gnr_profile_collect": (_INT, [_P, C.POINTER(C.c_float), C.POINTER(C.c_int64)]),
    "gnr_measure_l1_bandwidth": (_INT, [_INT, _INT, C.POINTER(C.c_float)]),
    "gnr_debug_phase_cycles": (_INT, [_P, _INT, C.POINTER(C.c_longlong)]),
    "gnr_debug_wait": (_INT, [_P, _INT, _INT]),
    "gnr_read_status": (_INT, [_P, C.POINTER(C.c_int32), _P]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m landmark_b200.build` "
            "(nvcc, sm_100a). landmark_b200 has no fallback implementation."
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class GnrError(RuntimeError):
    pass


def check(rc: int, what: str = ""):
    if rc != 0:
        msg = lib.gnr_last_error().decode(errors="replace")
        raise GnrError(f"{what or 'gridnerf_b200'} failed (rc={rc}): {msg}")
