"""Seeded synthetic GridNeRF scenes.

The reference renders trained city checkpoints that are not redistributable, so every
test and benchmark of this package runs on synthetic fields with the same shapes, value
distributions and checkpoint layout as a reference checkpoint:

* state-dict keys and tensor shapes follow ``GridNeRF.init_one_svd`` / ``init_svd_volume``
  (app/models/gridnerf_sequential.py:669-747): plane ``i`` is ``[1, C, G[mat1], G[mat0]]`` and
  line ``i`` is ``[1, C, G[vec], 1]`` with ``matMode = [[0,1],[0,2],[1,2]]``, ``vecMode = [2,1,0]``,
  values ``0.1 * randn``;
* ``basis_mat`` and the three ``renderModule.mlp`` layers are ``nn.Linear`` tensors drawn
  U(-1/sqrt(fan_in), 1/sqrt(fan_in)), which is what ``nn.Linear`` draws by default
  (app/models/mlp_render_fea.py:29-31);
* the occupancy volume is a boolean ``[D, H, W]`` (z, y, x) array as unpacked by
  ``GridBaseSequential.load`` (app/models/gridnerf_sequential.py:232-241).

All draws use CPU generators so that the same seed gives the same bits on every machine
with the same torch build.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import numpy as np
import torch

MAT_MODE = ((0, 1), (0, 2), (1, 2))
VEC_MODE = (2, 1, 0)

FIELD_SEED = 20211202  # the reference's default --random_seed (app/tools/config_parser.py:343)
MASK_SEED = 20211203


@dataclass
class SceneSpec:
    """Everything needed to rebuild one synthetic scene bit for bit."""

    name: str
    aabb: Tuple[Tuple[float, float, float], Tuple[float, float, float]]
    grid: Tuple[int, int, int]
    mask_shape: Tuple[int, int, int]  # (D, H, W) = (z, y, x)
    near_far: Tuple[float, float]
    height: int
    width: int
    focal: float
    n_samples: int
    density_n_comp: Tuple[int, int, int] = (16, 16, 16)
    app_n_comp: Tuple[int, int, int] = (48, 48, 48)
    app_dim: int = 27
    view_pe: int = 2
    fea_pe: int = 2
    feature_c: int = 128
    step_ratio: float = 0.5
    density_shift: float = -10.0
    distance_scale: float = 25.0
    ray_weight_thres: float = 1e-3
    alpha_filter_thres: float = 0.0
    bias_enable: bool = True
    encode_app: bool = False  # 48-d appearance latent per image (embedding_app), gridnerf_sequential.py:681-682
    fea2dense_act: str = "softplus"
    mask_kind: str = "boxes"  # "boxes" (free 3-D boxes) | "heightfield" (columns from z=0)
    mask_boxes: int = 60
    mask_edge: Tuple[int, int] = (4, 16)
    mask_height: Tuple[int, int] = (2, 32)
    extras: Dict[str, float] = field(default_factory=dict)

    def lit(self) -> "SceneSpec":
        """Same scene with ``density_shift = 0`` so that weights exceed the appearance
        threshold and the appearance gather + MLP actually run (with ``-10`` and 0.1*randn
        planes every sigma is ~4.5e-5 and the image is pure background)."""
        import copy

        s = copy.deepcopy(self)
        s.name = self.name + "_lit"
        s.density_shift = 0.0
        return s


def tiny_spec(height: int = 100, width: int = 100, n_samples: int = 128, grid: int = 128) -> SceneSpec:
    """The CPU-runnable case: AABB [-1,1]^3, grid 128^3, 64^3 mask of 60 boxes, 100x100 pinhole
    image with a 60 degree field of view from radius 2."""
    return SceneSpec(
        name="tiny",
        aabb=((-1.0, -1.0, -1.0), (1.0, 1.0, 1.0)),
        grid=(grid, grid, grid),
        mask_shape=(64, 64, 64),
        near_far=(0.1, 6.0),
        height=height,
        width=width,
        focal=0.5 * width / math.tan(math.radians(30.0)),
        n_samples=n_samples,
        mask_kind="boxes",
        mask_boxes=60,
        mask_edge=(4, 16),
    )


def city_spec(height: int = 1080, width: int = 1920, n_samples: int = 512, scale: int = 1) -> SceneSpec:
    """The city-block case: AABB [-8,8]x[-8,8]x[-1,1], grid 2048x2048x256, 512x512x64 heightfield
    mask, 1920x1080 camera with the online renderer's focal length
    (dist_render/ddp_infer/nerf_inferer.py:404). ``scale`` divides the grid and mask resolution
    (and nothing else) to give a structurally identical but smaller scene for tests."""
    assert 2048 % scale == 0 and scale >= 1
    return SceneSpec(
        name="city" if scale == 1 else f"city_div{scale}",
        aabb=((-8.0, -8.0, -1.0), (8.0, 8.0, 1.0)),
        grid=(2048 // scale, 2048 // scale, 256 // scale),
        mask_shape=(64 // min(scale, 8), 512 // scale, 512 // scale),
        near_far=(0.05, 40.0),
        height=height,
        width=width,
        focal=1483.6378 * width / 1920.0,
        n_samples=n_samples,
        mask_kind="heightfield",
        mask_boxes=3000,
        mask_edge=(4, 24),
        mask_height=(2, 26),  # tuned once so that occupancy is 0.251 at full resolution
    )


# ----------------------------------------------------------------------------------------------
# fields
# ----------------------------------------------------------------------------------------------


def _linear(gen: torch.Generator, out_f: int, in_f: int, bias: bool):
    bound = 1.0 / math.sqrt(in_f)
    w = (torch.rand((out_f, in_f), generator=gen, dtype=torch.float32) * 2.0 - 1.0) * bound
    b = (torch.rand((out_f,), generator=gen, dtype=torch.float32) * 2.0 - 1.0) * bound if bias else None
    return w, b


def mlp_in_dim(spec: SceneSpec) -> int:
    """Width of the appearance MLP input (app/models/mlp_render_fea.py:24-26, encode_app off)."""
    return (2 * max(spec.view_pe, 0) * 3 + 2 * spec.fea_pe * spec.app_dim + 3 * (spec.view_pe > -1) + spec.app_dim
            + (48 if spec.encode_app else 0))


def make_state_dict(spec: SceneSpec, seed: int = FIELD_SEED, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Draw all learnable tensors of one scene. With ``device="cpu"`` the bits depend only on
    (spec, seed, torch build). With a CUDA device the planes are drawn by the CUDA generator
    (fast, used by the benchmark, not comparable with fixtures)."""
    sd: Dict[str, torch.Tensor] = {}
    gx = spec.grid
    if device == "cpu":
        gen = torch.Generator(device="cpu").manual_seed(seed)

        def randn(shape):
            return torch.randn(shape, generator=gen, dtype=torch.float32)

    else:
        gen_d = torch.Generator(device=device).manual_seed(seed)

        def randn(shape):
            return torch.randn(shape, generator=gen_d, dtype=torch.float32, device=device)

    for prefix, comps in (("density", spec.density_n_comp), ("app", spec.app_n_comp)):
        for i in range(3):
            m0, m1 = MAT_MODE[i]
            sd[f"{prefix}_plane.{i}"] = 0.1 * randn((1, comps[i], gx[m1], gx[m0]))
            sd[f"{prefix}_line.{i}"] = 0.1 * randn((1, comps[i], gx[VEC_MODE[i]], 1))
    gen_w = torch.Generator(device="cpu").manual_seed(seed + 7)
    w, _ = _linear(gen_w, spec.app_dim, sum(spec.app_n_comp), False)
    sd["basis_mat.weight"] = w
    dims = [(spec.feature_c, mlp_in_dim(spec)), (spec.feature_c, spec.feature_c), (3, spec.feature_c)]
    for layer, (o, i_) in zip((0, 2, 4), dims):
        w, b = _linear(gen_w, o, i_, spec.bias_enable)
        sd[f"renderModule.mlp.{layer}.weight"] = w
        if b is not None:
            sd[f"renderModule.mlp.{layer}.bias"] = b
    if spec.bias_enable:
        sd["renderModule.mlp.4.bias"].zero_()  # app/models/mlp_render_fea.py:41-42
    if spec.encode_app:
        sd["embedding_app.weight"] = torch.randn((11500, 48), generator=gen_w, dtype=torch.float32)
    if device != "cpu":
        sd = {k: v.to(device) for k, v in sd.items()}
    return sd


def make_alpha_volume(spec: SceneSpec, seed: int = MASK_SEED) -> torch.Tensor:
    """Boolean occupancy volume ``[D, H, W]`` (z, y, x), numpy-generated from ``seed``."""
    rng = np.random.RandomState(seed)
    d, h, w = spec.mask_shape
    vol = np.zeros((d, h, w), dtype=bool)
    lo, hi = spec.mask_edge
    for _ in range(spec.mask_boxes):
        ex, ey = rng.randint(lo, hi + 1, size=2)
        ex, ey = min(int(ex), w), min(int(ey), h)
        x0 = rng.randint(0, w - ex + 1)
        y0 = rng.randint(0, h - ey + 1)
        if spec.mask_kind == "heightfield":
            zl, zh = spec.mask_height  # heights are given in 1/64ths of the z extent
            ez = max(1, min(d, int(rng.randint(zl, zh + 1)) * d // 64))
            z0 = 0
        else:
            ez = min(int(rng.randint(lo, hi + 1)), d)
            z0 = rng.randint(0, d - ez + 1)
        vol[z0 : z0 + ez, y0 : y0 + ey, x0 : x0 + ex] = True
    return torch.from_numpy(vol)


def model_kwargs(spec: SceneSpec) -> Dict[str, object]:
    """``ckpt["kwargs"]`` of this scene (app/models/gridnerf_sequential.py:171-189)."""
    return {
        "aabb": torch.tensor(spec.aabb, dtype=torch.float32),
        "gridSize": list(spec.grid),
        "density_n_comp": list(spec.density_n_comp),
        "appearance_n_comp": list(spec.app_n_comp),
        "app_dim": spec.app_dim,
        "density_shift": spec.density_shift,
        "alphaMask_thres": 0.001,
        "distance_scale": spec.distance_scale,
        "rayMarch_weight_thres": spec.ray_weight_thres,
        "fea2denseAct": spec.fea2dense_act,
        "near_far": list(spec.near_far),
        "step_ratio": spec.step_ratio,
        "pos_pe": 6,
        "view_pe": spec.view_pe,
        "fea_pe": spec.fea_pe,
        "featureC": spec.feature_c,
    }


def model_args(spec: SceneSpec, device: str = "cpu"):
    """The ``args`` namespace the model constructor reads
    (app/models/gridnerf_sequential.py:75-132, 650-657, 698)."""
    from types import SimpleNamespace

    return SimpleNamespace(
        distributed=False,
        run_nerf=False,
        nonlinear_density=False,
        ndims=3,
        TV_weight_density=0.0,
        TV_weight_app=0.0,
        Ortho_weight=0.0,
        L1_weight_inital=0.0,
        resMode=[1],
        sampling_opt=0,
        bias_enable=int(spec.bias_enable),
        encode_app=bool(spec.encode_app),
        n_importance=spec.n_samples,
        alpha_mask_filter_thre=spec.alpha_filter_thres,
        ckpt=None,
        device=device,
        render_batch_size=8192,
    )


def multires_state_dict(spec: SceneSpec, res_mode=(1, 2, 4), seed: int = 11) -> Dict[str, torch.Tensor]:
    """State dict of the single-dimension multi-resolution layout the reference's city configs use
    (``ndims=1``, ``resMode=[1,2,4]``: pair ``j`` is an xy plane and a z line at ``resMode[j]`` times the
    grid, app/models/gridnerf_sequential.py:684-718), seeded; basis_mat and the MLP are those of
    ``make_state_dict(spec)``."""
    g = torch.Generator().manual_seed(seed)
    gx, gy, gz = spec.grid
    sd = {}
    for j, r in enumerate(res_mode):
        sd[f"density_plane.{j}"] = 0.1 * torch.randn((1, spec.density_n_comp[0], gy * r, gx * r), generator=g)
        sd[f"density_line.{j}"] = 0.1 * torch.randn((1, spec.density_n_comp[0], gz * r, 1), generator=g)
        sd[f"app_plane.{j}"] = 0.1 * torch.randn((1, spec.app_n_comp[0], gy * r, gx * r), generator=g)
        sd[f"app_line.{j}"] = 0.1 * torch.randn((1, spec.app_n_comp[0], gz * r, 1), generator=g)
    base = make_state_dict(spec)
    sd.update({k: v for k, v in base.items() if k.startswith(("renderModule", "basis_mat"))})
    return sd


def make_checkpoint(spec: SceneSpec, seed: int = FIELD_SEED, mask_seed: int = MASK_SEED, device: str = "cpu"):
    """A dict in the reference's on-disk checkpoint format
    (app/models/gridnerf_sequential.py:209-223): kwargs, state_dict, bit-packed alpha mask."""
    vol = make_alpha_volume(spec, mask_seed).numpy()
    return {
        "kwargs": model_kwargs(spec),
        "state_dict": make_state_dict(spec, seed, device),
        "alphaMask.shape": vol.shape,
        "alphaMask.mask": np.packbits(vol.reshape(-1)),
        "alphaMask.aabb": torch.tensor(spec.aabb, dtype=torch.float32),
    }


# ----------------------------------------------------------------------------------------------
# cameras (OpenGL convention: camera looks along -z, x right, y up; c2w is [3, 4])
# ----------------------------------------------------------------------------------------------


def look_at(eye, target, up=(0.0, 0.0, 1.0)) -> np.ndarray:
    eye = np.asarray(eye, dtype=np.float64)
    fwd = np.asarray(target, dtype=np.float64) - eye
    fwd /= np.linalg.norm(fwd)
    right = np.cross(fwd, np.asarray(up, dtype=np.float64))
    right /= np.linalg.norm(right)
    true_up = np.cross(right, fwd)
    c2w = np.stack([right, true_up, -fwd, eye], axis=1)
    return c2w.astype(np.float32)


def pitched_pose(eye, yaw_deg: float, pitch_deg: float) -> np.ndarray:
    yaw, pitch = math.radians(yaw_deg), math.radians(pitch_deg)
    fwd = np.array([math.cos(pitch) * math.cos(yaw), math.cos(pitch) * math.sin(yaw), math.sin(pitch)])
    return look_at(eye, np.asarray(eye, dtype=np.float64) + fwd)


def make_pose(spec: SceneSpec, alpha_volume: torch.Tensor | None = None) -> np.ndarray:
    """Camera pose ``[3, 4]`` of the scene's benchmark view."""
    if spec.mask_kind == "heightfield":
        # 0.5 units above the tallest occupied voxel under the camera, pitched 30 degrees down.
        z_top = spec.aabb[0][2]
        if alpha_volume is not None:
            d, h, w = alpha_volume.shape
            col = alpha_volume[:, h // 2, w // 2].nonzero()
            if col.numel() > 0:
                k = int(col.max()) + 1
                z_top = spec.aabb[0][2] + (spec.aabb[1][2] - spec.aabb[0][2]) * k / d
        return pitched_pose((0.0, 0.0, z_top + 0.5), yaw_deg=0.0, pitch_deg=-30.0)
    r = 2.0
    el, az = math.radians(30.0), math.radians(45.0)
    eye = (r * math.cos(el) * math.cos(az), r * math.cos(el) * math.sin(az), r * math.sin(el))
    return look_at(eye, (0.0, 0.0, 0.0))


def state_dict_digest(sd: Dict[str, torch.Tensor]) -> str:
    """Short content hash used by the fixtures to prove that a regenerated scene has the bits
    the fixture was made from."""
    import hashlib

    h = hashlib.sha256()
    for k in sorted(sd):
        h.update(k.encode())
        h.update(sd[k].detach().cpu().contiguous().numpy().tobytes())
    return h.hexdigest()[:16]


def scene_tensor_bytes(spec: SceneSpec) -> int:
    gx = spec.grid
    n = 0
    for comps in (spec.density_n_comp, spec.app_n_comp):
        for i in range(3):
            m0, m1 = MAT_MODE[i]
            n += comps[i] * (gx[m0] * gx[m1] + gx[VEC_MODE[i]])
    return 4 * n


def spec_names() -> List[str]:
    return ["tiny", "city"]
