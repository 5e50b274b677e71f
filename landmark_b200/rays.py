"""Ray generation for the online renderer: ``generate_rays`` of dist_render/dataset/utils.py.

``get_ray_directions_blender_faster`` (:57-70) builds two 1-D tables with ``torch.arange``
(x direction per column, y direction per row); ``get_rays_with_directions`` (:73-89) rotates
``(dir_x[i], dir_y[j], -1)`` by the pose and takes the pose's translation as origin.  The tables
are W + H floats and are produced here by the very same ``torch.arange`` calls (on the CPU,
so that they have the bits of the CPU reference); the per-pixel work runs in the library's
ray-generation kernel, which can also emit the rays of an arbitrary pixel list (image tiles).
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from ._lib import check, lib


def direction_tables(H: int, W: int, focal: float):
    cx, cy = W / 2, H / 2
    dir_x = torch.arange(-cx / focal, (W - cx - 1e-5) / focal, 1 / focal, dtype=torch.float32)
    dir_y = torch.arange(cy / focal, (cy - H + 1e-5) / focal, -1 / focal, dtype=torch.float32)
    if dir_x.numel() != W or dir_y.numel() != H:
        raise ValueError(f"direction tables have {dir_x.numel()}x{dir_y.numel()} entries for a {W}x{H} image")
    return dir_x, dir_y


_table_cache = {}


def generate_rays(single_pose, H, W, focal=None, device="cuda", pixel_ids: Optional[torch.Tensor] = None,
                  first_pixel: int = 0, n: Optional[int] = None) -> torch.Tensor:
    """Rays ``[n, 6]`` (origin, un-normalised direction) on ``device``.

    ``single_pose`` is ``[3, 4]`` or ``[3, 5]`` (focal in the last column, as the reference's
    pose files have it).  Without ``pixel_ids`` the rays of pixels ``first_pixel ... first_pixel+n``
    (row-major) are produced, by default the whole image.
    """
    pose = np.asarray(single_pose.cpu() if isinstance(single_pose, torch.Tensor) else single_pose, dtype=np.float32)
    if focal is None:
        focal = float(pose[-1, -1])
    if isinstance(focal, torch.Tensor):
        focal = focal.item()
    H, W = int(H), int(W)
    dev = torch.device(device)
    key = (H, W, float(focal), str(dev))
    if key not in _table_cache:
        if len(_table_cache) > 8:
            _table_cache.clear()
        dx, dy = direction_tables(H, W, float(focal))
        _table_cache[key] = (dx.to(dev), dy.to(dev))
    dx, dy = _table_cache[key]
    if pixel_ids is not None:
        pixel_ids = pixel_ids.to(device=dev, dtype=torch.int32).contiguous()
        n = pixel_ids.numel()
    elif n is None:
        n = H * W - first_pixel
    rays = torch.empty((n, 6), dtype=torch.float32, device=dev)
    pose_c = (C.c_float * 12)(*[float(v) for v in pose[:3, :4].reshape(-1)])
    with torch.cuda.device(dev):
        check(lib.gnr_generate_rays(pose_c, C.c_void_p(dx.data_ptr()), C.c_void_p(dy.data_ptr()), H, W,
                                    C.c_void_p(pixel_ids.data_ptr() if pixel_ids is not None else 0), first_pixel, n,
                                    C.c_void_p(rays.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)),
              "gnr_generate_rays")
    return rays
