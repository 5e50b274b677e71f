"""CPU tests of the C-ABI boundary: the library builds, loads, exports every symbol the
header declares, and refuses to work without a GPU instead of falling back."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "gridnerf_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gnr_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    for must in ("gnr_create", "gnr_render_chunk", "gnr_render_host", "gnr_sample", "gnr_density", "gnr_weights",
                 "gnr_appearance", "gnr_composite", "gnr_generate_rays"):
        assert must in names


def test_library_exports_every_declared_symbol(built_library):
    lib = C.CDLL(built_library)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_binding_table_matches_header(built_library):
    from landmark_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()
    assert _lib.lib.gnr_version() >= 100
    assert _lib.lib.gnr_sample_bits(512) == 9 and _lib.lib.gnr_sample_bits(513) == 10 and _lib.lib.gnr_sample_bits(1) == 1


def test_config_struct_size_matches_header(built_library):
    from landmark_b200 import _lib

    # 6+3 floats, 3 ints, 5 floats, 1 int, 2 floats, 9 ints, 8 reserved ints
    assert C.sizeof(_lib.GnrConfig) == 4 * (6 + 3 + 3 + 5 + 1 + 2 + 9 + 8)


def test_no_cpu_fallback(built_library):
    """Without a CUDA device model creation must fail with a message; nothing computes."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from landmark_b200 import _lib

    cfg = _lib.GnrConfig()
    cfg.n_pairs, cfg.n_density, cfg.n_app, cfg.app_dim, cfg.hidden = 3, 16, 48, 27, 128
    h = C.c_void_p(0)
    rc = _lib.lib.gnr_create(C.byref(cfg), 0, C.byref(h))
    assert rc != 0 and not h.value
    assert len(_lib.lib.gnr_last_error()) > 0
    from landmark_b200 import scenes
    from landmark_b200.gridnerf import B200GridNeRF

    spec = scenes.tiny_spec()
    with pytest.raises(RuntimeError):
        B200GridNeRF(**scenes.model_kwargs(spec), device="cpu", args=scenes.model_args(spec))


def test_host_argument_validation(built_library):
    from landmark_b200 import _lib

    lib = _lib.lib
    n = C.c_size_t(0)
    assert lib.gnr_workspace_bytes(None, 10, 16, 10, 10, C.byref(n)) != 0
    assert lib.gnr_render_chunk(None, None, 1, 16, 1, None, 0, 1, 1, None, None, None) != 0
    assert b"null model" in lib.gnr_last_error()
    pose = (C.c_float * 12)()
    assert lib.gnr_generate_rays(pose, None, None, 4, 4, None, 0, 16, None, None) != 0
