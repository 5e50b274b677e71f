"""Ingest of the reference's multi-block checkpoint files.

The branch-parallel trainer saves one ``<exp>-sub<b>.th`` per block and ``merge_ckpts``
(app/models/gridnerf_branch_parallel.py:465-546) stacks them into ``<exp>-merged-stack.th``:

* every plane ``[1, C, H, W]`` of the sub checkpoints becomes ``[1, C, n_blocks, H, W]``
  (block index on dim 2),
* every line ``[1, C, L, 1]`` becomes ``[1, C, L, n_blocks]`` (block index on the last dim),
* ``basis_mat``, the MLP, ``kwargs`` and the occupancy mask are those of block 0 / the whole scene,
* ``kwargs["gridSize"]`` is the per-block resolution ``[W, H, L]``, ``gridShape`` records the stacked
  shapes,

and two sidecars: ``-wo_plane.th`` (the same without the plane tensors, for renderers that fetch
planes on demand) and ``-wo_state_dict.th`` (kwargs only).

``split_merged_stack`` turns such a file back into one checkpoint per block, which is what the
block-parallel renderer's owners load (block ``b`` of a ``Px x Py`` division is
``floor((x_n + 1) / (2 / Px)) * Py + floor((y_n + 1) / (2 / Py))``, the order ``merge_ckpts`` stacks
in), and ``sampler_checkpoint`` keeps what the ray owners need (box, step, occupancy mask).
``merge_stack`` is the inverse, in the reference's format.
"""

from __future__ import annotations

import copy
from typing import Dict, List, Sequence

import torch

PLANE_NAMES = ("density_plane", "app_plane")
LINE_NAMES = ("density_line", "app_line")
MASK_KEYS = ("alphaMask.shape", "alphaMask.mask", "alphaMask.aabb")


def _is_plane(key: str) -> bool:
    return any(n in key for n in PLANE_NAMES)


def _is_line(key: str) -> bool:
    return any(n in key for n in LINE_NAMES)


def is_merged_stack(ckpt: Dict) -> bool:
    """True if ``ckpt`` holds stacked (5-D) planes or stacked lines."""
    sd = ckpt.get("state_dict", {})
    for k, v in sd.items():
        if _is_plane(k) and v.dim() == 5:
            return True
    return bool(ckpt.get("gridShape")) and any(_is_line(k) and v.shape[-1] > 1 for k, v in sd.items())


def n_blocks_of(ckpt: Dict) -> int:
    sd = ckpt["state_dict"]
    for k, v in sd.items():
        if _is_plane(k) and v.dim() == 5:
            return int(v.shape[2])
    for k, v in sd.items():
        if _is_line(k):
            return int(v.shape[-1])
    raise ValueError("checkpoint holds neither planes nor lines")


def split_merged_stack(ckpt: Dict, planes: Dict[str, torch.Tensor] | None = None) -> List[Dict]:
    """One checkpoint per block from a ``-merged-stack.th`` dict.

    ``planes`` supplies the plane tensors when ``ckpt`` is a ``-wo_plane.th`` sidecar (keys as in
    the state dict, stacked ``[1, C, n_blocks, H, W]``).  Shared tensors (``basis_mat``, the MLP)
    are referenced, not copied; the occupancy mask stays with ``sampler_checkpoint``.
    """
    sd = dict(ckpt["state_dict"])
    if planes:
        sd.update(planes)
    if not any(_is_plane(k) for k in sd):
        raise ValueError("no plane tensors: pass the planes of a -wo_plane sidecar through `planes`")
    nb = n_blocks_of({"state_dict": sd})
    out = []
    for b in range(nb):
        bsd = {}
        for k, v in sd.items():
            if _is_plane(k):
                if v.dim() != 5 or v.shape[2] != nb:
                    raise ValueError(f"{k}: expected a stacked plane [1, C, {nb}, H, W], got {tuple(v.shape)}")
                bsd[k] = v[:, :, b].contiguous()
            elif _is_line(k):
                if v.dim() != 4 or v.shape[-1] != nb:
                    raise ValueError(f"{k}: expected a stacked line [1, C, L, {nb}], got {tuple(v.shape)}")
                bsd[k] = v[..., b:b + 1].contiguous()
            else:
                bsd[k] = v
        kwargs = {k: v for k, v in ckpt["kwargs"].items() if k not in ("device", "args")}
        out.append({"kwargs": kwargs, "state_dict": bsd})
    return out


def sampler_checkpoint(ckpt: Dict) -> Dict:
    """What a ray owner loads: kwargs and the occupancy mask, no field tensors."""
    out = {"kwargs": {k: v for k, v in ckpt["kwargs"].items() if k not in ("device", "args")}, "state_dict": {}}
    for k in MASK_KEYS:
        if k in ckpt:
            out[k] = ckpt[k]
    return out


def merge_stack(blocks: Sequence[Dict]) -> Dict:
    """Stack per-block checkpoints the way ``merge_ckpts`` does (block 0 supplies everything that
    is not a plane or a line)."""
    if not blocks:
        raise ValueError("no blocks")
    nb = len(blocks)
    merged = {k: (copy.copy(v) if k != "state_dict" else None) for k, v in blocks[0].items()}
    sd0 = blocks[0]["state_dict"]
    sd, shapes = {}, {}
    for k in sorted(sd0.keys()):
        v = sd0[k]
        if _is_plane(k):
            t = torch.zeros((1, v.shape[1], nb, v.shape[2], v.shape[3]), dtype=v.dtype)
            for b in range(nb):
                t[:, :, b] = blocks[b]["state_dict"][k]
            sd[k], shapes[k] = t, t.shape
        elif _is_line(k):
            t = torch.zeros((*v.shape[:3], nb), dtype=v.dtype)
            for b in range(nb):
                t[..., b] = blocks[b]["state_dict"][k][..., 0]
            sd[k], shapes[k] = t, t.shape
        else:
            sd[k] = v
    merged["state_dict"] = sd
    kwargs = dict(blocks[0]["kwargs"])
    kwargs["gridSize"] = [int(sd["density_plane.0"].shape[-1]), int(sd["density_plane.0"].shape[-2]),
                          int(sd["density_line.0"].shape[-2])]
    merged["kwargs"] = kwargs
    merged["gridShape"] = shapes
    return merged


def without_planes(merged: Dict) -> Dict:
    """The ``-wo_plane.th`` sidecar of a merged checkpoint (plane tensors removed)."""
    out = {k: v for k, v in merged.items() if k != "state_dict"}
    out["state_dict"] = {k: v for k, v in merged["state_dict"].items() if not _is_plane(k)}
    return out
