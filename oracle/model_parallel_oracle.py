"""CPU oracle of the block-parallel render path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Restates, with torch CPU operators in the reference's order, how a scene cut into ``Px x Py``
blocks is rendered: global sampling and occupancy filter as in the sequential model, then
``assign_blocks_to_samples`` (app/models/gridnerf_parallel.py:296-327) gives every valid sample a
block and block-local coordinates, each block's own field supplies sigma and colour for its
samples (:765-859), and weights / compositing run over the merged values
(app/models/gridnerf_sequential.py:477-504).  ``assign_blocks`` is pinned: tests/golden/make_golden.py
runs the reference's own method on seeded points (including points on block borders) and asserts
equality bit for bit (tests/golden/assign_blocks.npz).  The one intended difference lies outside that
set: a sample with x or y exactly 1 is given to the last block here (the reference's CUDA kernel drops
such a sample, its torch path gives it an index past the last block).

The channel-parallel layout needs no oracle of its own: the sum of the ranks' partial basis
projections is the projection of the unsplit model, so ``gridnerf_oracle.render_chunk`` on the
unsplit field is its oracle.
"""

from __future__ import annotations

from typing import List, Tuple

import torch

from oracle import gridnerf_oracle as orc


def assign_blocks(xyz: torch.Tensor, division: Tuple[int, int]):
    px, py = division
    plane_width, plane_height = 2 / px, 2 / py
    xyzb = torch.zeros(xyz.shape[0], 4)
    xyzb[:, :3] = xyz
    xyzb[:, :2] += 1
    xyzb[:, 0] /= plane_width
    xyzb[:, 1] /= plane_height
    bx = torch.floor(xyzb[:, 0]).clamp(0, px - 1)
    by = torch.floor(xyzb[:, 1]).clamp(0, py - 1)
    xyzb[:, 3] = bx * py + by
    xyzb[:, :3] = xyz
    coord_min = torch.stack([-1 + (xyzb[:, 3] // py) * plane_width, -1 + (xyzb[:, 3] % py) * plane_height], dim=-1)
    coord_max = torch.stack([-1 + (xyzb[:, 3] // py + 1) * plane_width, -1 + (xyzb[:, 3] % py + 1) * plane_height], dim=-1)
    xyzb[:, :2] = (xyzb[:, :2] - coord_min) * 2 / (coord_max - coord_min) - 1
    return xyzb[:, 3].to(torch.int64), xyzb[:, :3]


@torch.no_grad()
def render_chunk_blocks(global_field: orc.Field, block_fields: List[orc.Field], division: Tuple[int, int],
                        rays: torch.Tensor, n_samples: int, white_bg: bool = True):
    f = global_field
    rays = rays.float()
    rays_o, viewdirs = rays[:, :3], rays[:, 3:6]
    pts, z_vals, ray_valid, _ = orc.sample_ray(f, rays_o, viewdirs, n_samples)
    dists = torch.cat((z_vals[:, 1:] - z_vals[:, :-1], torch.zeros_like(z_vals[:, :1])), dim=-1)
    view_exp = viewdirs.view(-1, 1, 3).expand(pts.shape)
    if f.alpha_volume is not None:
        alphas = orc.sample_alpha(f, pts[ray_valid])
        ray_invalid = ~ray_valid
        ray_invalid[ray_valid] |= ~(alphas > f.alpha_filter_thres)
        ray_valid = ~ray_invalid
    xyz = (pts - f.aabb[0]) * f.inv_aabb_size - 1
    block, local = assign_blocks(xyz[ray_valid], division)
    sig_v = torch.zeros(local.shape[0])
    for b, bf in enumerate(block_fields):
        sel = block == b
        if sel.any():
            sig_v[sel] = orc.feature2density(bf, orc.density_feature(bf, local[sel]))
    sigma = torch.zeros(pts.shape[:-1])
    sigma[ray_valid] = sig_v
    _, weight, _ = orc.raw2alpha(sigma, dists * f.distance_scale)
    app_mask = weight > f.ray_weight_thres
    rgb = torch.zeros((*pts.shape[:2], 3))
    if app_mask.any():
        in_valid = app_mask[ray_valid]
        rgb_v = torch.zeros((int(in_valid.sum()), 3))
        blk_a, loc_a, view_a = block[in_valid], local[in_valid], view_exp[app_mask]
        for b, bf in enumerate(block_fields):
            sel = blk_a == b
            if sel.any():
                rgb_v[sel] = orc.mlp_render(bf, view_a[sel], orc.app_feature(bf, loc_a[sel]))
        rgb[app_mask] = rgb_v
    acc = torch.sum(weight, -1)
    rgb_map = torch.sum(weight[..., None] * rgb, -2)
    if white_bg:
        rgb_map = rgb_map + (1.0 - acc[..., None])
    return {"rgb_map": rgb_map.clamp(0, 1), "depth_map": torch.sum(weight * z_vals, -1), "ray_valid": ray_valid,
            "app_mask": app_mask, "block": block}
