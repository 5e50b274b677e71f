"""Multi-process drivers of the two model-parallel layouts on the city scene.

Used by ``bench.py --workload city_blocks | city_channels`` under torchrun (one rank per GPU,
NCCL).  Both build seeded synthetic scenes on the fly:

* ``city_blocks``: ``Px x Py`` blocks (world 1/2/4/8 -> 1x1, 2x1, 2x2, 4x2), every block a full
  city-block field (grid 2048x2048x256, 16/48 channels, its own seed) owned by one rank; global
  box ``[-8 Px, 8 Px] x [-8 Py, 8 Py] x [-1, 1]`` with a ``512 Px x 512 Py x 64`` occupancy
  heightfield.  The 1080p frame's rays are tile-sharded over the ranks; samples are routed to
  block owners by all-to-all.
* ``city_channels``: one city block whose appearance planes have ``48 x world`` channels, 48 per
  rank; every rank samples its share of the rays of a chunk, the appearance points are all-gathered,
  partial projections are reduce-scattered back to the rank that owns the points.
"""

from __future__ import annotations

import time
from typing import Dict, Tuple

import numpy as np
import torch

from . import scenes
from .gridnerf import B200GridNeRF
from .model_parallel import BlockParallelRenderer, ChannelParallelRenderer, DistComm, LoopbackComm
from .parallel import TileSharding
from .rays import generate_rays

# (the camera of the block scene looks along +x across the y = 0 plane: every division here cuts y, so that at
# least two owners carry visible samples)
DIVISIONS = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (4, 2)}


def _model(spec, ckpt, device, mlp_mode, **extra):
    kw = dict(ckpt["kwargs"])
    kw.update({"device": device, "args": scenes.model_args(spec, device), "is_train": False})
    m = B200GridNeRF(**kw, mlp_mode=mlp_mode, **extra)
    m.load(ckpt)
    m.release_torch_planes()
    return m


def build_blocks(world: int, rank_list, device: str, mlp_mode: int, grid_scale: int = 1, **model_extra):
    """Sampler (global box + mask) and the owned block fields for the ranks in ``rank_list``."""
    px, py = DIVISIONS[world]
    block = scenes.city_spec(scale=grid_scale).lit()
    gspec = scenes.city_spec(scale=grid_scale).lit()
    gspec.name = f"city_blocks_{px}x{py}"
    gspec.aabb = ((-8.0 * px, -8.0 * py, -1.0), (8.0 * px, 8.0 * py, 1.0))
    gspec.grid = (block.grid[0] * px, block.grid[1] * py, block.grid[2])
    gspec.mask_shape = (block.mask_shape[0], block.mask_shape[1] * py, block.mask_shape[2] * px)
    gspec.mask_boxes = block.mask_boxes * px * py
    vol = scenes.make_alpha_volume(gspec)
    gck = {"kwargs": scenes.model_kwargs(gspec), "state_dict": {}, "alphaMask.shape": tuple(vol.shape),
           "alphaMask.mask": np.packbits(vol.numpy().reshape(-1)), "alphaMask.aabb": torch.tensor(gspec.aabb)}
    samplers, owners = [], []
    for r in rank_list:
        samplers.append(_model(gspec, gck, device, 0, field_grid=(2, 2, 2)))
        sd = scenes.make_state_dict(block, seed=scenes.FIELD_SEED + 1000 * (r + 1), device=device)
        owners.append(_model(block, {"kwargs": scenes.model_kwargs(block), "state_dict": sd}, device, mlp_mode, **model_extra))
        del sd
        torch.cuda.empty_cache()
    pose = scenes.make_pose(gspec, vol)
    return gspec, pose, samplers, owners, (px, py)


def build_channels(world: int, rank_list, device: str, mlp_mode: int, grid_scale: int = 1, **model_extra):
    """Channel-sliced models (48 appearance channels each) for the ranks in ``rank_list``."""
    spec = scenes.city_spec(scale=grid_scale).lit()
    vol = scenes.make_alpha_volume(spec)
    models = []
    for r in rank_list:
        # density and the MLP are replicated (same seed on every rank); the appearance slice of
        # rank r and its basis columns are drawn from a rank-specific seed
        sd = scenes.make_state_dict(spec, device=device)
        gen = torch.Generator(device=device).manual_seed(scenes.FIELD_SEED + 77 * (r + 1))
        for k in list(sd):
            if k.startswith("app_plane") or k.startswith("app_line"):
                sd[k] = 0.1 * torch.randn(sd[k].shape, generator=gen, device=device)
        gw = torch.Generator().manual_seed(scenes.FIELD_SEED + 78 * (r + 1))
        bound = 1.0 / np.sqrt(3 * 48 * world)
        sd["basis_mat.weight"] = ((torch.rand((spec.app_dim, 3 * 48), generator=gw) * 2 - 1) * bound).to(device)
        ck = {"kwargs": scenes.model_kwargs(spec), "state_dict": sd, "alphaMask.shape": tuple(vol.shape),
              "alphaMask.mask": np.packbits(vol.numpy().reshape(-1)), "alphaMask.aabb": torch.tensor(spec.aabb)}
        models.append(_model(spec, ck, device, mlp_mode, **model_extra))
        del sd
        torch.cuda.empty_cache()
    return spec, scenes.make_pose(spec, vol), models


def run(workload: str, steps: int, warmup: int, chunk: int, mlp_mode: int, rank: int, world: int, device: str,
        grid_scale: int = 1, check: bool = False, ert: float = 0.0, app_fp16: bool = False, den_lattice: bool = True,
        lanes: int = 2) -> Dict:
    """Render ``steps`` frames; returns timing and sample statistics (rank 0's view).  ``lanes``: chunks in flight."""
    import torch.distributed as dist

    comm = DistComm() if world > 1 else LoopbackComm(1)
    H, W = 1080, 1920
    if workload == "city_blocks":
        extra = {"app_plane_fp16": bool(app_fp16 and mlp_mode == 2), "density_lattice": bool(den_lattice)}
        spec, pose, samplers, owners, division = build_blocks(world, [rank], device, mlp_mode, grid_scale, **extra)
        ren = BlockParallelRenderer(samplers, owners, comm, division)
        shard = TileSharding(H, W, rank, world, device)
        rays = generate_rays(pose, H, W, spec.focal, device=device, pixel_ids=shard.pixel_ids)
        parallelism = f"blocks {division[0]}x{division[1]} (all-to-all sample routing) + ray tiles x{world}"
    elif workload == "city_channels":
        extra = {"app_plane_fp16": bool(app_fp16 and mlp_mode == 2), "ert_transmittance": float(ert),
                 "density_lattice": bool(den_lattice)}
        spec, pose, models = build_channels(world, [rank], device, mlp_mode, grid_scale, **extra)
        ren = ChannelParallelRenderer(models, comm)
        shard = TileSharding(H, W, 0, 1, device)  # every rank walks the whole frame
        rays = generate_rays(pose, H, W, spec.focal, device=device, pixel_ids=shard.pixel_ids)
        parallelism = f"appearance channels 48 x {world} (reduce-scatter of partial projections)"
    else:
        raise ValueError(workload)
    S = spec.n_samples
    n_local = rays.shape[0]
    # every rank must make the same number of collective calls: pad the chunk count
    n_chunks = -(-n_local // chunk)
    if world > 1:
        t = torch.tensor([n_chunks], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        n_chunks = int(t.item())
    rgb = torch.zeros((shard.n_pad if workload == "city_blocks" else n_local, 3), dtype=torch.float32, device=device)
    image = torch.zeros((H * W, 3), dtype=torch.float32, device=device)
    stats = {"valid": 0, "app": 0}

    def parts_of_frame():
        out = []
        for c in range(n_chunks):
            lo, hi = min(c * chunk, n_local), min((c + 1) * chunk, n_local)
            out.append((lo, hi, rays[lo:hi] if hi > lo else rays[:1]))  # an idle rank still takes part in the exchange
        return out

    def frame_blocks(lanes=lanes):
        """Block layout: the chunks of the frame go through the renderer's two-lane pipeline."""
        parts = parts_of_frame()
        res = ren.render_frame([[p[2]] for p in parts], S, True, lanes=lanes)
        for (lo, hi, _), per_chunk in zip(parts, res):
            if hi > lo:
                rgb[lo:hi] = per_chunk[0][0]
        shard.assemble(rgb, image)
        stats["valid"], stats["app"] = ren.samples["valid"], ren.samples["app"]

    def frame_channels(lanes=lanes):
        """Channel layout: every rank walks the whole frame; the chunks go through the renderer's two-lane pipeline."""
        parts = parts_of_frame()
        res = ren.render_frame([[p[2]] for p in parts], S, True, lanes=lanes)
        stats["valid"], stats["app"] = ren.samples["valid"], ren.samples["app"]
        for (lo, hi, _), per_chunk in zip(parts, res):
            if hi > lo:
                rgb[lo:hi] = per_chunk[0][0]
        image[shard.all_pixels] = rgb

    def frame():
        if workload == "city_blocks":
            return frame_blocks()
        if ren._fp16_exchange():
            return frame_channels()
        stats["valid"] = stats["app"] = 0
        for c in range(n_chunks):
            lo, hi = min(c * chunk, n_local), min((c + 1) * chunk, n_local)
            part = rays[lo:hi] if hi > lo else rays[:1]  # an idle rank still takes part in the exchange
            (out_rgb, _), = ren.render_chunk([part], S, True)
            if hi > lo:
                rgb[lo:hi] = out_rgb
            s = ren.samplers[0] if workload == "city_blocks" else ren.models[0]
            stats["valid"] += int(s.last_status[2]) if hi > lo else 0
            stats["app"] += int(s.last_status[3]) if hi > lo else 0
        if workload == "city_blocks":
            shard.assemble(rgb, image)
        else:
            image[shard.all_pixels] = rgb

    for _ in range(max(warmup, 1)):
        frame()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        frame()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
    # one more frame with a CUDA-event stopwatch around every section (rank 0's view; its extra events and the
    # synchronisation at the end are why this frame is not part of the timed ones)
    ren.timer.enabled = True
    if workload == "city_blocks":
        frame_blocks(lanes=1)  # one lane: the sections of a chunk follow each other on one stream
    elif ren._fp16_exchange():
        frame_channels(lanes=1)
    else:
        frame()
    sections = {k: round(v, 3) for k, v in ren.timer.collect().items()}
    ren.timer.enabled = False
    tot = torch.tensor([float(stats["valid"]), float(stats["app"])], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot)  # every rank sampled its own share of the rays (both layouts)
    res = {"ms_per_frame": float(ms.item()), "wall_ms_per_frame": (time.perf_counter() - t0) * 1e3 / steps,
           "valid": float(tot[0].item()), "appearance": float(tot[1].item()), "parallelism": parallelism,
           "image_mean": float(image.mean().item()), "rays": H * W, "sections_ms": sections, "chunks_per_rank": n_chunks}
    if check and workload == "city_blocks" and rank == 0 and world > 1:
        # rank 0 re-renders its own rays with every block held locally (loopback); the bits must agree
        _, _, s_all, o_all, division = build_blocks(world, list(range(world)), device, mlp_mode, grid_scale, **extra)
        lb = BlockParallelRenderer(s_all, o_all, LoopbackComm(world), division)
        sub = rays[: min(n_local, 20000)]
        parts = [sub] + [sub[:1]] * (world - 1)
        ref_rgb = lb.render_chunk(parts, S, True)[0][0]
        res["check_max_abs_diff_vs_single_process"] = float((ref_rgb - rgb[: sub.shape[0]]).abs().max().item())
    return res
