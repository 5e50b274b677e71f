"""GPU test of gnr_sample_static, the sampling entry point that allocates nothing.

Some callers cannot hand the library a workspace or tolerate an allocation: the frame loop of
an online renderer (a cudaMalloc there synchronises the device and stalls the other pipeline
stages), or a host whose device memory is entirely taken by the field's planes.  For them the
library keeps the sampler's scratch in a fixed built-in array.  This file checks, through the
C ABI, that the entry gives exactly what the workspace-based gnr_sample gives, on two calls
in a row that share the array (the second with fewer rays and fewer samples, so that anything
stale from the first would show), and that a chunk beyond the array's size is refused.

Kept in a file that sorts last so that a run which stops at the first failure has already
executed every other test.
"""
import ctypes as C

import pytest
import torch

from landmark_b200 import scenes
from tests._util import cuda_model, tiny_rays

pytestmark = pytest.mark.gpu


def _call_static(model, rays, n_samples, max_valid):
    from landmark_b200 import _lib

    n = rays.shape[0]
    dev = rays.device
    t_min = torch.full((n,), -7.0, dtype=torch.float32, device=dev)
    counts = torch.full((n,), -7, dtype=torch.int32, device=dev)
    offsets = torch.full((n + 1,), -7, dtype=torch.int32, device=dev)
    ids = torch.full((max_valid,), -7, dtype=torch.int32, device=dev)
    status = torch.full((_lib.ST_WORDS,), -7, dtype=torch.int32, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = _lib.lib.gnr_sample_static(model._handle, C.c_void_p(rays.data_ptr()), n, n_samples, max_valid,
                                    C.c_void_p(t_min.data_ptr()), C.c_void_p(counts.data_ptr()),
                                    C.c_void_p(offsets.data_ptr()), C.c_void_p(ids.data_ptr()),
                                    C.c_void_p(status.data_ptr()), stream)
    torch.cuda.synchronize()
    return rc, t_min, counts, offsets, ids, status


def _check_against_workspace_entry(model, rays, n_samples):
    from landmark_b200 import _lib

    ref = model.run_stages(rays, n_samples, True, upto="sample")
    max_valid = rays.shape[0] * n_samples
    rc, t_min, counts, offsets, ids, status = _call_static(model, rays, n_samples, max_valid)
    assert rc == 0, _lib.lib.gnr_last_error()
    assert torch.equal(t_min, ref["t_min"])
    assert torch.equal(counts, ref["counts"])
    assert torch.equal(offsets, ref["offsets"])
    m_v = ref["num_valid"]
    assert int(status[_lib.ST_NUM_VALID]) == m_v and int(status[_lib.ST_OVERFLOW_VALID]) == 0
    kbits = _lib.lib.gnr_sample_bits(n_samples)
    got = ids[:m_v].to(torch.int64) & 0xFFFFFFFF
    assert torch.equal(got >> kbits, ref["ray_index"]) and torch.equal(got & ((1 << kbits) - 1), ref["sample_index"])
    return m_v


def test_static_sampler_matches_workspace_sampler_twice():
    spec = scenes.tiny_spec().lit()
    model = cuda_model(spec)
    rays = tiny_rays(spec).cuda()
    first = _check_against_workspace_entry(model, rays, spec.n_samples)
    # second call on the same array: fewer rays, fewer samples, other rays
    second = _check_against_workspace_entry(model, rays[2500:5500].contiguous(), 96)
    assert first > 100000 and 0 < second < first


def test_static_sampler_reports_overflow_and_refuses_oversize():
    from landmark_b200 import _lib

    spec = scenes.tiny_spec().lit()
    model = cuda_model(spec)
    rays = tiny_rays(spec).cuda()
    rc, _, counts, _, _, status = _call_static(model, rays, spec.n_samples, 1000)
    assert rc == 0 and int(status[_lib.ST_OVERFLOW_VALID]) == 1 and int(status[_lib.ST_NUM_VALID]) == int(counts.sum())
    # 300k rays x 512 samples would need 19 MB of scratch: refused before anything is enqueued
    big = torch.zeros((300000, 6), dtype=torch.float32, device="cuda")
    rc, t_min, *_ = _call_static(model, big, 512, 1024)
    assert rc != 0
    msg = _lib.lib.gnr_last_error().decode()
    assert "scratch" in msg and str(_lib.SAMPLE_STATIC_SCRATCH_BYTES) in msg
    assert float(t_min[0]) == -7.0  # untouched


def test_static_sampler_size_boundary():
    """The documented limit: 65,536 rays x 512 samples fit the built-in array, one more scan
    block of rays (4,096 more) does not, and a refused call enqueues nothing."""
    from landmark_b200 import _lib

    spec = scenes.tiny_spec().lit()
    model = cuda_model(spec)
    rays = tiny_rays(spec).cuda()
    big = rays[torch.arange(65536 + 4096, device="cuda") % rays.shape[0]].contiguous()
    rc, _, counts, offsets, _, status = _call_static(model, big[:65536].contiguous(), 512, 1024)
    assert rc == 0, _lib.lib.gnr_last_error()
    assert int(status[_lib.ST_NUM_VALID]) == int(counts.sum()) == int(offsets[-1])
    rc, t_min, *_ = _call_static(model, big, 512, 1024)
    assert rc != 0 and "scratch" in _lib.lib.gnr_last_error().decode()
    assert float(t_min[0]) == -7.0


def test_static_sampler_refuses_hull_model_without_tables():
    """A hull-sampler model reads two per-sample tables on the device.  Without them (or with
    tables for another sample count) the call is refused on the host, exactly as gnr_sample
    refuses it, and no kernel is launched."""
    from landmark_b200 import _lib
    from landmark_b200.gridnerf import B200GridNeRF

    spec = scenes.tiny_spec().lit()
    ckpt = scenes.make_checkpoint(spec)
    args = scenes.model_args(spec, "cuda:0")
    args.sampling_opt, args.n_importance = 1, 64
    kw = dict(ckpt["kwargs"])
    kw.update({"device": "cuda:0", "args": args, "is_train": False})
    model = B200GridNeRF(**kw)
    model.load(ckpt)  # committed, but no hull tables have been uploaded yet
    rays = tiny_rays(spec).cuda()[:512].contiguous()
    rc, t_min, counts, *_ = _call_static(model, rays, 64, 512 * 64)
    assert rc != 0 and "hull" in _lib.lib.gnr_last_error().decode()
    assert float(t_min[0]) == -7.0 and int(counts[0]) == -7
    ref = model.run_stages(rays, -1, True, upto="sample")  # uploads the tables for 64 samples
    rc, _, counts, *_ = _call_static(model, rays, 64, 512 * 64)
    assert rc == 0 and torch.equal(counts, ref["counts"])
    rc, t_min, *_ = _call_static(model, rays, 96, 512 * 96)  # tables are for 64 samples, not 96
    assert rc != 0 and float(t_min[0]) == -7.0
