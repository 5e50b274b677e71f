"""Torch-free restatement of WHICH samples of a ray are valid.  TEST INFRASTRUCTURE ONLY.

The set of valid (ray, sample) pairs is the integer-valued result the CUDA sampler must
reproduce exactly, so it is restated here from first principles in numpy float32, one
IEEE-754 operation per line, with no fused multiply-add:

* ``valid_mask``: slab entry, uniform steps, closed-box test
  (app/models/gridnerf_sequential.py:260-281) followed by the occupancy filter
  (app/models/gridnerf_sequential.py:460-465 with app/models/alpha_mask.py:35-59).
* ``trilinear_zero_pad``: what ``F.grid_sample`` computes for a ``[1,1,D,H,W]`` volume with
  ``mode="bilinear"``, ``padding_mode="zeros"``, ``align_corners=True`` (ATen
  ``grid_sampler_3d``, published in torch's aten/src/ATen/native/GridSampler.cpp): index
  ``((q + 1) / 2) * (size - 1)``, floor, corner weights as products of differences to the
  opposite corner, eight bounds-checked taps accumulated in the order
  tnw, tne, tsw, tse, bnw, bne, bsw, bse.

``tests/test_oracle.py`` checks this file against the torch oracle on seeded inputs, and
``tests/golden/make_golden.py`` checks both against the reference itself.
"""

from __future__ import annotations

import numpy as np

f32 = np.float32


def slab_t_min(rays_o, rays_d, aabb, near, far):
    o = rays_o.astype(f32)
    d = rays_d.astype(f32)
    vec = np.where(d == 0, f32(1e-6), d).astype(f32)
    rate_a = ((aabb[1].astype(f32) - o) / vec).astype(f32)
    rate_b = ((aabb[0].astype(f32) - o) / vec).astype(f32)
    t = np.minimum(rate_a, rate_b).max(axis=-1)
    t = np.minimum(np.maximum(t, f32(near)), f32(far))
    return t.astype(f32)


def sample_points(rays_o, rays_d, t_min, step_size, n_samples):
    k = np.arange(n_samples, dtype=f32)
    step = (f32(step_size) * k).astype(f32)
    t = (t_min[:, None] + step[None, :]).astype(f32)
    prod = (rays_d.astype(f32)[:, None, :] * t[:, :, None]).astype(f32)
    pts = (rays_o.astype(f32)[:, None, :] + prod).astype(f32)
    return pts, t


def in_box(pts, aabb):
    lo, hi = aabb[0].astype(f32), aabb[1].astype(f32)
    return ~((lo > pts) | (pts > hi)).any(axis=-1)


def trilinear_zero_pad(volume, q):
    """``volume [D,H,W]`` float32, ``q [M,3]`` normalised (x, y, z) -> ``[M]`` float32."""
    dd, hh, ww = volume.shape
    ix = (((q[:, 0] + f32(1)) / f32(2)).astype(f32) * f32(ww - 1)).astype(f32)
    iy = (((q[:, 1] + f32(1)) / f32(2)).astype(f32) * f32(hh - 1)).astype(f32)
    iz = (((q[:, 2] + f32(1)) / f32(2)).astype(f32) * f32(dd - 1)).astype(f32)
    x0, y0, z0 = np.floor(ix), np.floor(iy), np.floor(iz)
    x1, y1, z1 = x0 + f32(1), y0 + f32(1), z0 + f32(1)
    wx0, wx1 = (x1 - ix).astype(f32), (ix - x0).astype(f32)
    wy0, wy1 = (y1 - iy).astype(f32), (iy - y0).astype(f32)
    wz0, wz1 = (z1 - iz).astype(f32), (iz - z0).astype(f32)
    out = np.zeros(q.shape[0], dtype=f32)
    for zc, wz in ((z0, wz0), (z1, wz1)):
        for yc, wy in ((y0, wy0), (y1, wy1)):
            for xc, wx in ((x0, wx0), (x1, wx1)):
                w = ((wx * wy).astype(f32) * wz).astype(f32)
                ok = (xc >= 0) & (xc < ww) & (yc >= 0) & (yc < hh) & (zc >= 0) & (zc < dd)
                xi = np.clip(xc, 0, ww - 1).astype(np.int64)
                yi = np.clip(yc, 0, hh - 1).astype(np.int64)
                zi = np.clip(zc, 0, dd - 1).astype(np.int64)
                tap = np.where(ok, volume[zi, yi, xi].astype(f32), f32(0))
                out = (out + (tap * w).astype(f32)).astype(f32)
    return out


def valid_mask(rays, aabb, near, far, step_size, n_samples, alpha_volume=None, alpha_aabb=None,
               alpha_thres=0.0):
    """Boolean ``[N, S]`` validity, plus ``t_min [N]``."""
    rays = np.asarray(rays, dtype=f32)
    aabb = np.asarray(aabb, dtype=f32)
    o, d = rays[:, :3], rays[:, 3:6]
    t_min = slab_t_min(o, d, aabb, near, far)
    pts, _ = sample_points(o, d, t_min, step_size, n_samples)
    valid = in_box(pts, aabb)
    if alpha_volume is not None:
        a = np.asarray(alpha_aabb, dtype=f32)
        inv = ((f32(1.0) / (a[1] - a[0]).astype(f32)).astype(f32) * f32(2)).astype(f32)
        sel = pts[valid]
        q = (((sel - a[0]).astype(f32) * inv).astype(f32) - f32(1)).astype(f32)
        alpha = trilinear_zero_pad(np.asarray(alpha_volume, dtype=f32), q)
        keep = alpha > f32(alpha_thres)
        idx = np.nonzero(valid)
        valid[idx[0][~keep], idx[1][~keep]] = False
    return valid, t_min
