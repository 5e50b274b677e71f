"""Pin the oracle against the reference and write the golden fixtures.

Run once, in a container that has the reference checked out (it is NOT needed to run the
tests): ``python tests/golden/make_golden.py --reference /path/to/LandMark``.

What it does, per scene:
  1. builds the seeded synthetic scene (``landmark_b200.scenes``) as a reference-format
     checkpoint and loads it into the reference's own ``GridNeRF`` on CPU;
  2. runs the reference's own methods stage by stage (``sample_ray``, ``sample_alpha``,
     ``compute_densityfeature``, ``feature2density``, ``raw2alpha``, ``compute_appfeature``,
     ``renderModule``) and its ``forward``;
  3. asserts that the torch oracle (``oracle/gridnerf_oracle.py``) reproduces every stage
     EXACTLY (``torch.equal``) and that the numpy sampler (``oracle/sampling_numpy.py``)
     reproduces the valid-sample set exactly;
  4. writes compact ``.npz`` fixtures (bit-packed masks, per-ray counts, images, strided
     subsets of per-sample values) that the tests compare the oracle and the CUDA path with.
"""

from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from landmark_b200 import scenes  # noqa: E402
from oracle import gridnerf_oracle as orc  # noqa: E402
from oracle import sampling_numpy as snp  # noqa: E402

SUBSET_STRIDE = 97


def import_reference(path):
    """The reference imports two packages this image lacks for training-only symbols."""
    sys.path.insert(0, path)
    m = types.ModuleType("torch_efficient_distloss")
    m.eff_distloss = lambda *a, **k: None
    sys.modules["torch_efficient_distloss"] = m
    k = types.ModuleType("kornia")
    k.create_meshgrid = lambda *a, **kw: None
    sys.modules["kornia"] = k
    from app.models.gridnerf_sequential import GridNeRF
    from app.tools.utils import raw2alpha
    from dist_render.dataset import utils as ray_utils

    return GridNeRF, raw2alpha, ray_utils


def reference_model(GridNeRF, spec, ckpt, sampling_opt=0, n_importance=None):
    args = scenes.model_args(spec)
    args.sampling_opt = sampling_opt
    if n_importance is not None:
        args.n_importance = n_importance
    kwargs = dict(ckpt["kwargs"])
    kwargs.update({"device": "cpu", "args": args, "is_train": False})
    model = GridNeRF(**kwargs)
    model.load(ckpt)
    return model


def reference_stages(model, raw2alpha, rays, n_samples, app_code=None):
    """Re-trace app/models/gridnerf_sequential.py:448-504 (or :522-576 when the model was built
    with sampling_opt) with the model's own methods."""
    rays_o, viewdirs = rays[:, :3], rays[:, 3:6]
    if model.sampling_opt:
        pts, _, z_vals, ray_valid = model.sample_ray_within_hull(rays_o, viewdirs, is_train=False, N_samples=n_samples)
    else:
        pts, _, z_vals, ray_valid = model.sample_ray(rays_o, viewdirs, is_train=False, N_samples=n_samples)
    in_box = ray_valid.clone()
    dists = torch.cat((z_vals[:, 1:] - z_vals[:, :-1], torch.zeros_like(z_vals[:, :1])), dim=-1)
    alphas = model.alphaMask.sample_alpha(pts[ray_valid])
    alpha_mask = alphas > model.alpha_mask_filter_thre
    ray_invalid = ~ray_valid
    ray_invalid[ray_valid] |= ~alpha_mask
    ray_valid = ~ray_invalid
    sigma = torch.zeros(pts.shape[:-1])
    xyz = model.normalize_coord(pts)
    sigma_feat = model.compute_densityfeature(xyz[ray_valid])
    sigma[ray_valid] = model.feature2density(sigma_feat)
    _, weight, _ = raw2alpha(sigma, dists * model.distance_scale)
    app_mask = weight > model.rayMarch_weight_thres
    feats = rgb_s = None
    if app_mask.any():
        feats = model.compute_appfeature(xyz[app_mask])
        view_exp = viewdirs.view(-1, 1, 3).expand(pts.shape)
        latent = model.compute_app_latent(xyz, app_mask, app_code) if model.args.encode_app else None
        rgb_s = model.renderModule(view_exp[app_mask], feats, latent)
    return {"in_box": in_box, "ray_valid": ray_valid, "sigma_feature": sigma_feat, "sigma": sigma,
            "weight": weight, "app_mask": app_mask, "app_features": feats, "rgb_samples": rgb_s,
            "z_vals": z_vals}


def check_equal(name, a, b):
    if a is None and b is None:
        return
    assert torch.equal(a, b), f"oracle != reference at stage {name}: max diff {(a.float() - b.float()).abs().max()}"


def pin_and_dump(GridNeRF, raw2alpha, ray_utils, spec, rays, out_name, n_samples, note, sampling_opt=0, app_code=None):
    ckpt = scenes.make_checkpoint(spec)
    digest = scenes.state_dict_digest(ckpt["state_dict"])
    with torch.no_grad():
        model = reference_model(GridNeRF, spec, ckpt, sampling_opt, n_samples)
        ref = reference_stages(model, raw2alpha, rays, n_samples, app_code)
        ref_out, _ = model(rays, app_code=app_code, white_bg=True, is_train=False, N_samples=n_samples)
    field = orc.field_from_checkpoint(ckpt, spec.alpha_filter_thres)
    assert torch.equal(field.step_size, model.stepSize)
    assert field.n_samples_default == model.nSamples
    mine = orc.render_chunk(field, rays, n_samples, True, keep_stages=True, sampling_opt=bool(sampling_opt), app_code=app_code)
    for k in ("in_box", "ray_valid", "sigma_feature", "sigma", "weight", "app_mask", "app_features", "z_vals"):
        check_equal(k, mine[k], ref[k])
    if ref["rgb_samples"] is not None:
        check_equal("rgb_samples", mine["rgb"][mine["app_mask"]], ref["rgb_samples"])
    check_equal("rgb_map", mine["rgb_map"], ref_out["rgb_map"])
    check_equal("depth_map", mine["depth_map"], ref_out["depth_map"])
    # torch-free sampler against the reference (dense sampler only)
    if not sampling_opt:
        vol = field.alpha_volume[0, 0].numpy()
        v_np, t_np = snp.valid_mask(rays.numpy(), field.aabb.numpy(), field.near, field.far,
                                    field.step_size.item(), n_samples, vol, field.alpha_aabb.numpy(),
                                    spec.alpha_filter_thres)
        assert np.array_equal(v_np, ref["ray_valid"].numpy()), "numpy sampler != reference ray_valid"
        assert np.array_equal(t_np, mine["t_min"].numpy())

    valid = ref["ray_valid"].numpy()
    app = ref["app_mask"].numpy()
    sub = slice(0, None, SUBSET_STRIDE)
    fx = {
        "note": np.array(note),
        "scene": np.array(spec.name),
        "state_dict_digest": np.array(digest),
        "torch_version": np.array(torch.__version__),
        "n_samples": np.array(n_samples),
        "rays": rays.numpy(),
        "step_size": np.array(field.step_size.item(), dtype=np.float32),
        "t_min": mine["t_min"].numpy(),
        "valid_bits": np.packbits(valid, axis=1),
        "valid_counts": valid.sum(1).astype(np.int32),
        "in_box_counts": ref["in_box"].numpy().sum(1).astype(np.int32),
        "app_bits": np.packbits(app, axis=1),
        "app_counts": app.sum(1).astype(np.int32),
        "sigma_feature_sub": ref["sigma_feature"].numpy()[sub],
        "weight_sub": ref["weight"].numpy()[valid][sub],
        "acc": ref["weight"].sum(-1).numpy(),
        "rgb_map": ref_out["rgb_map"].numpy(),
        "depth_map": ref_out["depth_map"].numpy(),
        "subset_stride": np.array(SUBSET_STRIDE),
        "app_code": np.array(-1 if app_code is None else int(app_code)),
    }
    if ref["app_features"] is not None:
        fx["app_features_sub"] = ref["app_features"].numpy()[sub]
        fx["rgb_samples_sub"] = ref["rgb_samples"].numpy()[sub]
    path = os.path.join(HERE, out_name)
    np.savez_compressed(path, **fx)
    print(f"{out_name}: rays {rays.shape[0]} valid {int(valid.sum())} app {int(app.sum())} "
          f"rgb_mean {float(ref_out['rgb_map'].mean()):.4f} digest {digest} "
          f"size {os.path.getsize(path) / 1e3:.0f} kB", flush=True)


def block_checkpoints(n_blocks=2, grid=8):
    """Seeded per-block checkpoints (what the branch-parallel trainer saves as <exp>-sub<b>.th)."""
    spec = scenes.tiny_spec(grid=grid).lit()
    return [scenes.make_checkpoint(spec, seed=500 + b) for b in range(n_blocks)]


def pin_merged_stack():
    """Run the reference's merge_ckpts (gridnerf_branch_parallel.py:465-546) on two small block
    checkpoints and keep what it stacked, as the pin of landmark_b200.checkpoints."""
    import tempfile

    from app.models.gridnerf_branch_parallel import GridNeRFBranchParallel
    from landmark_b200 import checkpoints

    blocks = block_checkpoints()
    orig_load = torch.load
    torch.load = lambda *x, **k: orig_load(*x, **{**k, "weights_only": False})  # our own files; torch>=2.6 default differs
    try:
        with tempfile.TemporaryDirectory() as d:
            for b, ck in enumerate(blocks):
                torch.save(ck, f"{d}/exp-sub{b}.th")
            fake = types.SimpleNamespace(args=types.SimpleNamespace(rank=0, expname="exp", model_parallel_degree=len(blocks),
                                                                    plane_division=[len(blocks), 1], device="cpu"))
            GridNeRFBranchParallel.merge_ckpts(fake, d)
            ref = torch.load(f"{d}/exp-merged-stack.th", map_location="cpu")
            wo = torch.load(f"{d}/exp-merged-stack-wo_plane.th", map_location="cpu")
    finally:
        torch.load = orig_load
    mine = checkpoints.merge_stack(blocks)
    assert set(ref["state_dict"]) == set(mine["state_dict"])
    for k, v in ref["state_dict"].items():
        assert torch.equal(v, mine["state_dict"][k]), k
    assert list(ref["kwargs"]["gridSize"]) == list(mine["kwargs"]["gridSize"])
    assert {k: tuple(v) for k, v in ref["gridShape"].items()} == {k: tuple(v) for k, v in mine["gridShape"].items()}
    assert set(wo["state_dict"]) == set(checkpoints.without_planes(mine)["state_dict"])
    fx = {"grid_size": np.array(ref["kwargs"]["gridSize"], dtype=np.int64), "n_blocks": np.int64(len(blocks))}
    for k, v in ref["state_dict"].items():
        if any(n in k for n in checkpoints.PLANE_NAMES + checkpoints.LINE_NAMES):
            fx["sd." + k] = v.numpy()
    path = os.path.join(HERE, "merged_stack_tiny.npz")
    np.savez_compressed(path, **fx)
    print(f"merged_stack_tiny.npz: merge_ckpts of {len(blocks)} blocks pinned, size {os.path.getsize(path) / 1e3:.0f} kB", flush=True)


def pin_assign_blocks():
    """Run the reference's own assign_blocks_to_samples (app/models/gridnerf_parallel.py:279-338) with a
    stand-in ``self`` on seeded points and keep block ids and block-local coordinates; the oracle's
    restatement (oracle/model_parallel_oracle.py) must reproduce both bit for bit.  The one intended
    difference is outside the compared set: a point with x or y exactly 1 gets the block index
    ``px * py + ...`` from the reference (past the last block, so none of its masks selects it), while
    the restatement clamps it into the last block; the points here lie in [-1, 1)."""
    from app.models.gridnerf_parallel import GridBaseParallel
    from oracle import model_parallel_oracle as mpo

    g = torch.Generator().manual_seed(4242)
    xyz = torch.rand((4096, 3), generator=g) * 2 - 1
    xyz[:64, 0] = -1.0                      # on the lower faces
    xyz[64:128, 1] = -1.0
    xyz[128:192, 0] = torch.linspace(-1, 1, 65)[:-1]  # on interior block borders for every division below
    xyz[192:256, 1] = torch.linspace(-1, 1, 65)[:-1]
    xyz[:, :2] = xyz[:, :2].clamp(max=float(np.nextafter(np.float32(1.0), np.float32(0.0))))
    fx = {"xyz": xyz.numpy()}
    for division in ((2, 1), (2, 2), (4, 2), (3, 5)):
        fake = types.SimpleNamespace(args=types.SimpleNamespace(plane_division=list(division), ckpt_type="sub"), device="cpu")
        masks, xyzb = GridBaseParallel.assign_blocks_to_samples(fake, xyz, None, False)
        block = torch.full((xyz.shape[0],), -1, dtype=torch.int64)
        for b, m in enumerate(masks):
            assert not (block[m] >= 0).any()
            block[m] = b
        assert (block >= 0).all()
        mine_block, mine_local = mpo.assign_blocks(xyz, division)
        assert torch.equal(mine_block, block), division
        assert torch.equal(mine_local, xyzb[:, :3]), division
        tag = f"{division[0]}x{division[1]}"
        fx[f"block_{tag}"] = block.numpy().astype(np.int32)
        fx[f"local_{tag}"] = xyzb[:, :3].numpy()
    path = os.path.join(HERE, "assign_blocks.npz")
    np.savez_compressed(path, **fx)
    print(f"assign_blocks.npz: assign_blocks_to_samples pinned for 4 divisions on {xyz.shape[0]} points, "
          f"size {os.path.getsize(path) / 1e3:.0f} kB", flush=True)


def pin_multires(GridNeRF, raw2alpha):
    """The multi-resolution single-dimension layout of the reference's city configs (``ndims=1``,
    ``resMode=[1,2,4]``: three xy planes at 1x/2x/4x the grid with z lines) rendered by the reference
    class itself, every stage compared with the oracle, through rgb_map."""
    spec = scenes.tiny_spec(height=40, width=40, n_samples=64, grid=32).lit()
    spec.name = "tiny_multires"
    res_mode = [1, 2, 4]
    ckpt = scenes.make_checkpoint(spec)
    ckpt["state_dict"] = scenes.multires_state_dict(spec, res_mode)
    args = scenes.model_args(spec)
    args.ndims, args.resMode = 1, res_mode
    kwargs = dict(ckpt["kwargs"])
    kwargs.update({"device": "cpu", "args": args, "is_train": False})
    pose = torch.from_numpy(scenes.make_pose(spec))
    rays = orc.generate_rays(pose, spec.height, spec.width, spec.focal)
    with torch.no_grad():
        model = GridNeRF(**kwargs)
        model.load(ckpt)
        assert len(model.density_plane) == 3 and tuple(model.app_plane[2].shape[-2:]) == (128, 128)
        ref = reference_stages(model, raw2alpha, rays, spec.n_samples)
        ref_out, _ = model(rays, white_bg=True, is_train=False, N_samples=spec.n_samples)
    field = orc.field_from_checkpoint(ckpt, 0.0, ndims=1, res_mode=res_mode)
    mine = orc.render_chunk(field, rays, spec.n_samples, True, keep_stages=True)
    for k in ("in_box", "ray_valid", "sigma_feature", "sigma", "weight", "app_mask", "app_features", "z_vals"):
        check_equal(k, mine[k], ref[k])
    check_equal("rgb_samples", mine["rgb"][mine["app_mask"]], ref["rgb_samples"])
    check_equal("rgb_map", mine["rgb_map"], ref_out["rgb_map"])
    check_equal("depth_map", mine["depth_map"], ref_out["depth_map"])
    valid, app = ref["ray_valid"].numpy(), ref["app_mask"].numpy()
    fx = {"note": np.array("ndims=1, resMode=[1,2,4], grid 32, 40x40 rays, 64 samples; rendered by the reference's GridNeRF"),
          "state_dict_digest": np.array(scenes.state_dict_digest(ckpt["state_dict"])), "n_samples": np.array(spec.n_samples),
          "rays": rays.numpy(), "valid_bits": np.packbits(valid, axis=1), "valid_counts": valid.sum(1).astype(np.int32),
          "app_counts": app.sum(1).astype(np.int32), "sigma_feature": ref["sigma_feature"].numpy(),
          "app_features_sub": ref["app_features"].numpy()[::7], "rgb_map": ref_out["rgb_map"].numpy(),
          "depth_map": ref_out["depth_map"].numpy()}
    path = os.path.join(HERE, "tiny_multires.npz")
    np.savez_compressed(path, **fx)
    print(f"tiny_multires.npz: rays {rays.shape[0]} valid {int(valid.sum())} app {int(app.sum())} "
          f"rgb_mean {float(ref_out['rgb_map'].mean()):.4f} size {os.path.getsize(path) / 1e3:.0f} kB", flush=True)


def pin_update_alpha_mask(GridNeRF, grid=(40, 36, 28)):
    """updateAlphaMask of the reference (gridnerf_sequential.py:321-384) on the tiny lit scene, with
    and without an existing mask; the oracle's restatement must give the same volume and box."""
    spec = scenes.tiny_spec().lit()
    ckpt = scenes.make_checkpoint(spec)
    fx = {"grid": np.array(grid, dtype=np.int64), "state_dict_digest": scenes.state_dict_digest(ckpt["state_dict"])}
    # "threshold": no mask, and a threshold in the middle of the scene's alpha values, so that the
    # outcome depends on the density itself
    for tag, with_mask, thres in (("masked", True, None), ("unmasked", False, None), ("threshold", False, 0.00575)):
        ck = ckpt if with_mask else {k: v for k, v in ckpt.items() if not k.startswith("alphaMask")}
        if thres is not None:
            ck = dict(ck)
            ck["kwargs"] = dict(ck["kwargs"], alphaMask_thres=thres)
        model = reference_model(GridNeRF, spec, ck)
        new_aabb = model.updateAlphaMask(tuple(grid))
        ref_vol = model.alphaMask.alpha_volume[0, 0] > 0.5
        field = orc.field_from_checkpoint(ck)
        vol, box = orc.update_alpha_mask(field, grid, alpha_mask_thres=model.alphaMask_thres)
        assert torch.equal(vol, ref_vol), tag
        assert torch.equal(box, new_aabb), tag
        fx[f"{tag}_volume_bits"] = np.packbits(ref_vol.numpy().reshape(-1))
        fx[f"{tag}_aabb"] = new_aabb.numpy()
        fx[f"{tag}_occupied"] = np.int64(int(ref_vol.sum()))
    fx["threshold_value"] = np.float64(0.00575)
    path = os.path.join(HERE, "tiny_lit_update_mask.npz")
    np.savez_compressed(path, **fx)
    print(f"tiny_lit_update_mask.npz: updateAlphaMask{tuple(grid)} pinned, occupied masked/unmasked/threshold "
          f"{int(fx['masked_occupied'])}/{int(fx['unmasked_occupied'])}/{int(fx['threshold_occupied'])} of {int(np.prod(grid))}",
          flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a LandMark checkout")
    ap.add_argument("--skip-city", action="store_true")
    a = ap.parse_args()
    GridNeRF, raw2alpha, ray_utils = import_reference(a.reference)
    torch.set_num_threads(os.cpu_count())

    # ray generation: the reference's two device-agnostic helpers vs the oracle's restatement
    for spec in (scenes.tiny_spec(), scenes.city_spec()):
        pose = torch.from_numpy(scenes.make_pose(spec, scenes.make_alpha_volume(spec)))
        dirs = ray_utils.get_ray_directions_blender_faster(spec.height, spec.width, spec.focal, device="cpu")
        ro, rd = ray_utils.get_rays_with_directions(dirs, pose)
        ref_rays = torch.cat([ro, rd], 1)
        assert torch.equal(ref_rays, orc.generate_rays(pose, spec.height, spec.width, spec.focal))
        print(f"generate_rays pinned for {spec.name}: {tuple(ref_rays.shape)}")

    tiny = scenes.tiny_spec()
    pose = torch.from_numpy(scenes.make_pose(tiny))
    rays = orc.generate_rays(pose, tiny.height, tiny.width, tiny.focal)
    pin_and_dump(GridNeRF, raw2alpha, ray_utils, tiny, rays, "tiny_literal.npz", tiny.n_samples,
                 "config[0], density_shift=-10 (no appearance samples)")
    pin_and_dump(GridNeRF, raw2alpha, ray_utils, tiny.lit(), rays, "tiny_lit.npz", tiny.n_samples,
                 "config[0] with density_shift=0 (appearance path active)")
    # a threshold > 0 exercises the trilinear sum rather than the any-corner test
    thr = scenes.tiny_spec().lit()
    thr.name = "tiny_lit_thr05"
    thr.alpha_filter_thres = 0.5
    pin_and_dump(GridNeRF, raw2alpha, ray_utils, thr, rays[::7].contiguous(), "tiny_lit_thr05.npz",
                 thr.n_samples, "config[0] lit, alpha_mask_filter_thre=0.5, every 7th ray")

    # the hull sampler of the online renderer (sampling_opt=1, n_importance samples per ray)
    pin_and_dump(GridNeRF, raw2alpha, ray_utils, tiny.lit(), rays[::3].contiguous(), "tiny_lit_hull.npz", 128,
                 "config[0] lit, sampling_opt=1 (sample_ray_within_hull), n_importance=128, every 3rd ray",
                 sampling_opt=1)

    # appearance latent (encode_app=1): embedding row `app_code` appended to the MLP input
    enc = scenes.tiny_spec().lit()
    enc.name, enc.encode_app = "tiny_lit_encode_app", True
    pin_and_dump(GridNeRF, raw2alpha, ray_utils, enc, rays[::5].contiguous(), "tiny_lit_encode_app.npz", enc.n_samples,
                 "config[0] lit, encode_app=1, app_code=1234, every 5th ray", app_code=torch.tensor(1234))

    pin_merged_stack()
    pin_assign_blocks()
    pin_multires(GridNeRF, raw2alpha)
    pin_update_alpha_mask(GridNeRF)

    if not a.skip_city:
        city = scenes.city_spec().lit()
        vol = scenes.make_alpha_volume(city)
        pose = torch.from_numpy(scenes.make_pose(city, vol))
        rays = orc.generate_rays(pose, city.height, city.width, city.focal)
        # 64-ray slices: image rows 100, 540 and 1000, columns spread over the row
        pick = torch.cat([torch.arange(r * city.width + 7, (r + 1) * city.width, 30)[:64] for r in (100, 540, 1000)])
        pin_and_dump(GridNeRF, raw2alpha, ray_utils, city, rays[pick].contiguous(), "city_lit_slices.npz",
                     city.n_samples, "config[1] lit, 3 x 64 rays from rows 100/540/1000; ray ids in 'pick'")
        d = dict(np.load(os.path.join(HERE, "city_lit_slices.npz")))
        d["pick"] = pick.numpy()
        np.savez_compressed(os.path.join(HERE, "city_lit_slices.npz"), **d)


if __name__ == "__main__":
    main()
