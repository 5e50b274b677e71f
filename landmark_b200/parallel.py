"""Image-tile data parallelism for a replicated model.

The reference splits a frame's rays into contiguous ranges, scatters them from rank 0 and
gathers the colours back (dist_render/ddp_infer/nerf_inferer.py:58-72,300-305,337-339; offline:
app/tools/render_utils.py:126-170).  Here every rank derives its own rays from the pose, so
nothing is scattered: the frame is cut into ``tile x tile`` pixel tiles, tile ``k`` belongs to
rank ``k % world`` (round-robin balances empty sky against dense ground), and one
``all_gather_into_tensor`` of the per-rank colour buffers (padded to a common length) brings
the frame together.  Works with any ``torch.distributed`` backend (NCCL on GPUs, gloo in tests).
"""

from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

TILE = 64


PATCH = (8, 4)  # pixels of one warp: 8 wide, 4 high


def _patch_order(ys: np.ndarray, xs: np.ndarray, W: int, patch) -> np.ndarray:
    """Pixel ids of the region ys x xs, in patches of ``patch`` = (width, height) pixels: patches
    row-major over the region, pixels row-major inside a patch."""
    pw, ph = patch
    grid = ys[:, None] * W + xs[None, :]
    h, w = grid.shape
    if h % ph == 0 and w % pw == 0:
        return grid.reshape(h // ph, ph, w // pw, pw).transpose(0, 2, 1, 3).reshape(-1)
    out = []
    for y0 in range(0, h, ph):
        for x0 in range(0, w, pw):
            out.append(grid[y0:y0 + ph, x0:x0 + pw].reshape(-1))
    return np.concatenate(out)


def tile_pixel_ids(H: int, W: int, rank: int, world: int, tile: int = TILE, patch=PATCH) -> np.ndarray:
    """Pixel ids (row-major ``y * W + x``) of the tiles owned by ``rank``, tiles clipped at the image
    border.  Inside a tile the pixels come in 8 x 4 patches (``patch``; ``None`` = plain row-major):
    the render kernels give 32 consecutive rays to one warp, and the rays of a compact patch stay
    within a voxel of each other, so the lanes of a load read the same few texels."""
    tx, ty = (W + tile - 1) // tile, (H + tile - 1) // tile
    ids = []
    for k in range(rank, tx * ty, world):
        y0, x0 = (k // tx) * tile, (k % tx) * tile
        ys = np.arange(y0, min(y0 + tile, H))
        xs = np.arange(x0, min(x0 + tile, W))
        if patch is None:
            ids.append((ys[:, None] * W + xs[None, :]).reshape(-1))
        else:
            ids.append(_patch_order(ys, xs, W, patch))
    return np.concatenate(ids).astype(np.int32) if ids else np.zeros((0,), np.int32)


class TileSharding:
    """Per-rank pixel list plus what rank 0 needs to put the gathered colours back in place."""

    def __init__(self, H: int, W: int, rank: int, world: int, device, tile: int = TILE, group=None):
        import torch.distributed as dist

        self.H, self.W, self.rank, self.world, self.group = H, W, rank, world, group
        ids = tile_pixel_ids(H, W, rank, world, tile)
        self.n_local = int(ids.shape[0])
        self.pixel_ids = torch.from_numpy(ids).to(device)
        self.n_pad = self.n_local
        if world > 1:
            cnt = torch.tensor([self.n_local], device=device, dtype=torch.int64)
            dist.all_reduce(cnt, op=dist.ReduceOp.MAX, group=group)
            self.n_pad = int(cnt.item())
            pad = torch.full((self.n_pad,), -1, dtype=torch.int64, device=device)
            pad[: self.n_local] = self.pixel_ids.to(torch.int64)
            all_pix = torch.empty((world * self.n_pad,), dtype=torch.int64, device=device)
            dist.all_gather_into_tensor(all_pix, pad, group=group)
            self.keep = all_pix >= 0
            self.all_pixels = all_pix[self.keep]
            rows = self.keep.nonzero(as_tuple=True)[0]
            self.gathered = torch.empty((world * self.n_pad, 3), dtype=torch.float32, device=device)
        else:
            self.keep = None
            self.all_pixels = self.pixel_ids.to(torch.int64)
            rows = torch.arange(self.n_local, dtype=torch.int64, device=device)
            self.gathered = None
        # pixel -> row of the gathered colour buffer: assembling a frame is one gather with
        # coalesced writes and no host synchronisation
        self.src_for_pixel = torch.empty((H * W,), dtype=torch.int64, device=device)
        self.src_for_pixel[self.all_pixels] = rows

    def assemble(self, rgb_padded: torch.Tensor, image: torch.Tensor) -> torch.Tensor:
        """``rgb_padded [n_pad, 3]`` of this rank -> ``image [H*W, 3]`` (complete on every rank
        after the all-gather; callers usually only read it on rank 0)."""
        import torch.distributed as dist

        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered, rgb_padded, group=self.group)
            torch.index_select(self.gathered, 0, self.src_for_pixel, out=image)
        else:
            torch.index_select(rgb_padded, 0, self.src_for_pixel, out=image)
        return image


def split_contiguous(n_rays: int, world: int) -> Tuple[int, int]:
    """The reference's split: ``ceil(n / world)`` rays per rank and the padding that makes the
    total divisible (nerf_inferer.py:58-72)."""
    per = -(-n_rays // world)
    return per, per * world - n_rays
