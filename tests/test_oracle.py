"""CPU tests: the oracle against the committed golden fixtures (which were produced by the
reference itself, see tests/golden/make_golden.py) and against its torch-free sibling."""
import numpy as np
import pytest
import torch

from landmark_b200 import scenes
from oracle import gridnerf_oracle as orc
from oracle import sampling_numpy as snp
from tests._util import load_golden, oracle_field, tiny_rays


@pytest.fixture(scope="module")
def tiny_lit():
    spec = scenes.tiny_spec().lit()
    field, ckpt = oracle_field(spec)
    return spec, field, ckpt


def test_scene_bits_match_fixture(tiny_lit):
    spec, field, ckpt = tiny_lit
    fx = load_golden("tiny_lit.npz")
    assert scenes.state_dict_digest(ckpt["state_dict"]) == str(fx["state_dict_digest"])
    assert np.float32(field.step_size.item()) == fx["step_size"]


def test_generate_rays_matches_fixture():
    spec = scenes.tiny_spec()
    fx = load_golden("tiny_lit.npz")
    assert np.array_equal(tiny_rays(spec).numpy(), fx["rays"])


@pytest.mark.parametrize("name,lit", [("tiny_literal.npz", False), ("tiny_lit.npz", True)])
def test_oracle_reproduces_reference_fixture(name, lit):
    spec = scenes.tiny_spec()
    if lit:
        spec = spec.lit()
    field, _ = oracle_field(spec)
    fx = load_golden(name)
    rays = torch.from_numpy(fx["rays"])
    out = orc.render_chunk(field, rays, int(fx["n_samples"]), True, keep_stages=True)
    valid = out["ray_valid"].numpy()
    assert np.array_equal(np.packbits(valid, axis=1), fx["valid_bits"])
    assert np.array_equal(valid.sum(1).astype(np.int32), fx["valid_counts"])
    assert np.array_equal(np.packbits(out["app_mask"].numpy(), axis=1), fx["app_bits"])
    assert np.array_equal(out["t_min"].numpy(), fx["t_min"])
    stride = int(fx["subset_stride"])
    assert np.array_equal(out["sigma_feature"].numpy()[::stride], fx["sigma_feature_sub"])
    assert np.array_equal(out["rgb_map"].numpy(), fx["rgb_map"])
    assert np.array_equal(out["depth_map"].numpy(), fx["depth_map"])
    if lit:
        assert np.array_equal(out["app_features"].numpy()[::stride], fx["app_features_sub"])
        assert np.array_equal(out["rgb"][out["app_mask"]].numpy()[::stride], fx["rgb_samples_sub"])
        assert int(fx["app_counts"].sum()) > 100000
    else:
        assert int(fx["app_counts"].sum()) == 0  # density_shift=-10: nothing passes w > 1e-3


def test_threshold_fixture():
    spec = scenes.tiny_spec().lit()
    spec.alpha_filter_thres = 0.5
    field, _ = oracle_field(spec)
    fx = load_golden("tiny_lit_thr05.npz")
    out = orc.render_chunk(field, torch.from_numpy(fx["rays"]), int(fx["n_samples"]), True, keep_stages=True)
    assert np.array_equal(np.packbits(out["ray_valid"].numpy(), axis=1), fx["valid_bits"])
    assert np.array_equal(out["rgb_map"].numpy(), fx["rgb_map"])


def test_numpy_sampler_equals_fixture_and_oracle(tiny_lit):
    spec, field, _ = tiny_lit
    fx = load_golden("tiny_lit.npz")
    rays = fx["rays"][::5]
    vol = field.alpha_volume[0, 0].numpy()
    valid, t_min = snp.valid_mask(rays, field.aabb.numpy(), field.near, field.far, field.step_size.item(),
                                  int(fx["n_samples"]), vol, field.alpha_aabb.numpy(), 0.0)
    bits = np.unpackbits(fx["valid_bits"][::5], axis=1)[:, : int(fx["n_samples"])].astype(bool)
    assert np.array_equal(valid, bits)
    assert np.array_equal(t_min, fx["t_min"][::5])


def test_numpy_sampler_random_rays_with_threshold(tiny_lit):
    """Random origins inside and outside the box, axis-parallel directions (d component 0),
    and a trilinear threshold of 0.5: torch oracle and numpy restatement agree exactly."""
    spec, field, ckpt = tiny_lit
    g = torch.Generator().manual_seed(5)
    o = (torch.rand((400, 3), generator=g) * 3.0 - 1.5)
    d = torch.randn((400, 3), generator=g)
    d[::7, 0] = 0.0
    d[::11, 2] = 0.0
    d[3::50] = torch.tensor([0.0, 0.0, -1.0])
    rays = torch.cat([o, d], 1)
    f2 = orc.field_from_checkpoint(ckpt, 0.5)
    out = orc.render_chunk(f2, rays, 96, True, keep_stages=True)
    valid, _ = snp.valid_mask(rays.numpy(), f2.aabb.numpy(), f2.near, f2.far, f2.step_size.item(), 96,
                              f2.alpha_volume[0, 0].numpy(), f2.alpha_aabb.numpy(), 0.5)
    assert np.array_equal(valid, out["ray_valid"].numpy())
    assert valid.sum() > 1000


def test_empty_and_single_ray(tiny_lit):
    spec, field, _ = tiny_lit
    out = orc.render_chunk(field, torch.zeros((0, 6)), 16)
    assert out["rgb_map"].shape == (0, 3)
    ray = torch.tensor([[3.0, 3.0, 3.0, 1.0, 0.0, 0.0]])  # never enters the box
    out = orc.render_chunk(field, ray, 16, True, keep_stages=True)
    assert not out["ray_valid"].any()
    assert torch.equal(out["rgb_map"], torch.ones((1, 3)))


def test_city_slice_fixture_is_self_consistent():
    fx = load_golden("city_lit_slices.npz")
    assert fx["rays"].shape == (192, 6)
    assert int(fx["valid_counts"].sum()) == 42671 and int(fx["app_counts"].sum()) == 11374
    assert fx["pick"].shape == (192,)


def test_hull_sampler_fixture():
    """sampling_opt=1 (sample_ray_within_hull): the oracle reproduces what the reference gave."""
    spec = scenes.tiny_spec().lit()
    field, _ = oracle_field(spec)
    fx = load_golden("tiny_lit_hull.npz")
    out = orc.render_chunk(field, torch.from_numpy(fx["rays"]), int(fx["n_samples"]), True, keep_stages=True,
                           sampling_opt=True)
    assert np.array_equal(np.packbits(out["ray_valid"].numpy(), axis=1), fx["valid_bits"])
    assert np.array_equal(out["t_min"].numpy(), fx["t_min"])
    assert np.array_equal(out["rgb_map"].numpy(), fx["rgb_map"])
    assert np.array_equal(out["depth_map"].numpy(), fx["depth_map"])


def test_encode_app_fixture():
    spec = scenes.tiny_spec().lit()
    spec.encode_app = True
    field, _ = oracle_field(spec)
    fx = load_golden("tiny_lit_encode_app.npz")
    out = orc.render_chunk(field, torch.from_numpy(fx["rays"]), int(fx["n_samples"]), True, app_code=int(fx["app_code"]))
    assert np.array_equal(out["rgb_map"].numpy(), fx["rgb_map"])


def test_update_alpha_mask_fixture():
    """updateAlphaMask: the oracle against what the reference produced (existing mask kept, no mask,
    and a threshold in the middle of the scene's alpha values)."""
    spec = scenes.tiny_spec().lit()
    ckpt = scenes.make_checkpoint(spec)
    fx = load_golden("tiny_lit_update_mask.npz")
    grid = tuple(int(g) for g in fx["grid"])
    n = int(np.prod(grid))
    bare = {k: v for k, v in ckpt.items() if not k.startswith("alphaMask")}
    for tag, ck, thres in (("masked", ckpt, 1e-3), ("threshold", bare, float(fx["threshold_value"]))):
        vol, box = orc.update_alpha_mask(orc.field_from_checkpoint(ck), grid, alpha_mask_thres=thres)
        assert vol.shape == grid[::-1]
        assert np.array_equal(np.packbits(vol.numpy().reshape(-1)), fx[f"{tag}_volume_bits"])
        assert np.array_equal(box.numpy(), fx[f"{tag}_aabb"])
        assert 0 < int(vol.sum()) == int(fx[f"{tag}_occupied"]) < n


def test_assign_blocks_fixture():
    """The block assignment of the block-parallel oracle against what the reference's own
    assign_blocks_to_samples returned for the same points (pinned by make_golden.py)."""
    from oracle import model_parallel_oracle as mpo

    fx = load_golden("assign_blocks.npz")
    xyz = torch.from_numpy(fx["xyz"])
    for division in ((2, 1), (2, 2), (4, 2), (3, 5)):
        tag = f"{division[0]}x{division[1]}"
        b, local = mpo.assign_blocks(xyz, division)
        assert np.array_equal(b.numpy(), fx[f"block_{tag}"].astype(np.int64))
        assert np.array_equal(local.numpy(), fx[f"local_{tag}"])


def test_multires_fixture():
    """ndims=1, resMode=[1,2,4]: the oracle against the fixture the reference's GridNeRF class rendered."""
    fx = load_golden("tiny_multires.npz")
    spec = scenes.tiny_spec(height=40, width=40, n_samples=64, grid=32).lit()
    ckpt = scenes.make_checkpoint(spec)
    ckpt["state_dict"] = scenes.multires_state_dict(spec)
    assert scenes.state_dict_digest(ckpt["state_dict"]) == str(fx["state_dict_digest"])
    field = orc.field_from_checkpoint(ckpt, 0.0, ndims=1, res_mode=[1, 2, 4])
    out = orc.render_chunk(field, torch.from_numpy(fx["rays"]), int(fx["n_samples"]), True, keep_stages=True)
    assert np.array_equal(np.packbits(out["ray_valid"].numpy(), axis=1), fx["valid_bits"])
    assert np.array_equal(out["sigma_feature"].numpy(), fx["sigma_feature"])
    assert np.array_equal(out["rgb_map"].numpy(), fx["rgb_map"]) and np.array_equal(out["depth_map"].numpy(), fx["depth_map"])
