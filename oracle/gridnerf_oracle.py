"""CPU oracle for the GridNeRF render path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this
module; the package itself never does.

This is a functional restatement (no ``nn.Module``, no checkpoint classes) of what the
reference's torch renderer computes for one chunk of rays, written with the same torch
operators in the same order so that on the same torch build it reproduces the reference
bit for bit on CPU.  Each function names the reference lines it follows.  The arithmetic of
``F.grid_sample``, ``cumprod``, ``softplus``, ``sin``/``cos``, ``sigmoid`` and ``linear`` lives in
torch itself (ATen, here torch 2.11.0; the reference pins 1.13.1), which is why a second,
torch-free restatement of the integer-valued part (which samples are valid) is kept next
to it in ``sampling_numpy.py``.

Pinning: the reference's own tests hold no golden vectors for this path (they compare PSNR
against photographs on a cluster), so the oracle is pinned against the reference itself:
``tests/golden/make_golden.py`` imports the reference model, loads the same seeded scene,
asserts that every stage below equals the reference's tensors exactly, and writes the
fixtures under ``tests/golden/``.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn.functional as F

MAT_MODE = ((0, 1), (0, 2), (1, 2))
VEC_MODE = (2, 1, 0)


class Field:
    """Plain container of one scene's tensors in the reference's native layout."""

    def __init__(self, state_dict: Dict[str, torch.Tensor], kwargs: Dict[str, object],
                 alpha_volume: Optional[torch.Tensor], alpha_aabb: Optional[torch.Tensor],
                 alpha_filter_thres: float = 0.0, ndims: int = 3, res_mode=(1,)):
        sd = state_dict
        # args.ndims dimensions x len(args.resMode) resolutions: pair idx belongs to dimension
        # idx // len(resMode) (app/models/gridnerf_sequential.py:106-110,698-718,801-802)
        self.ndims, self.n_res = int(ndims), len(res_mode)
        n_pairs = self.ndims * self.n_res
        self.density_plane = [sd[f"density_plane.{i}"].float() for i in range(n_pairs)]
        self.density_line = [sd[f"density_line.{i}"].float() for i in range(n_pairs)]
        self.app_plane = [sd[f"app_plane.{i}"].float() for i in range(n_pairs)]
        self.app_line = [sd[f"app_line.{i}"].float() for i in range(n_pairs)]
        self.basis_w = sd["basis_mat.weight"].float()
        self.mlp_w = [sd[f"renderModule.mlp.{j}.weight"].float() for j in (0, 2, 4)]
        self.mlp_b = [sd.get(f"renderModule.mlp.{j}.bias") for j in (0, 2, 4)]
        self.embedding_app = sd.get("embedding_app.weight")  # present iff encode_app
        self.aabb = torch.as_tensor(kwargs["aabb"], dtype=torch.float32)
        self.near, self.far = [float(v) for v in kwargs["near_far"]]
        self.density_shift = float(kwargs["density_shift"])
        self.distance_scale = float(kwargs["distance_scale"])
        self.ray_weight_thres = float(kwargs["rayMarch_weight_thres"])
        self.act = kwargs.get("fea2denseAct", "softplus")
        self.view_pe = int(kwargs["view_pe"])
        self.fea_pe = int(kwargs["fea_pe"])
        self.alpha_filter_thres = float(alpha_filter_thres)
        # update_stepSize, app/models/gridnerf_sequential.py:149-164
        self.aabb_size = self.aabb[1] - self.aabb[0]
        self.inv_aabb_size = 2.0 / self.aabb_size
        grid = torch.tensor(kwargs["gridSize"])
        units = self.aabb_size / (grid - 1)
        self.step_size = torch.mean(units) * float(kwargs["step_ratio"])
        diag = torch.sqrt(torch.sum(torch.square(self.aabb_size)))
        self.n_samples_default = int((diag / self.step_size).item()) + 1
        if alpha_volume is not None:
            # AlphaGridMask.__init__, app/models/alpha_mask.py:16-26
            self.alpha_aabb = torch.as_tensor(alpha_aabb, dtype=torch.float32)
            self.alpha_inv = 1.0 / (self.alpha_aabb[1] - self.alpha_aabb[0]) * 2
            self.alpha_volume = alpha_volume.float().view(1, 1, *alpha_volume.shape[-3:])
        else:
            self.alpha_volume = None

    def to(self, device):
        """Move every tensor of the field (the same torch operators then run on that device: the
        benchmark times this port on the GPU as a same-hardware reference point)."""
        for k, v in list(vars(self).items()):
            if isinstance(v, torch.Tensor):
                setattr(self, k, v.to(device))
            elif isinstance(v, list) and v and all(isinstance(t, torch.Tensor) or t is None for t in v):
                setattr(self, k, [t.to(device) if t is not None else None for t in v])
        return self


def generate_rays(pose: torch.Tensor, height: int, width: int, focal: float) -> torch.Tensor:
    """Pinhole rays ``[H*W, 6]`` (origin, un-normalised direction) for a ``[3, 4]`` pose.
    Follows dist_render/dataset/utils.py:57-70 (direction tables by ``torch.arange``),
    :73-89 (rotate by the pose) and :92-113 (concatenate)."""
    cx, cy = width / 2, height / 2
    d = torch.empty((3, height, width), dtype=torch.float32)
    d[0] = torch.arange(-cx / focal, (width - cx - 1e-5) / focal, 1 / focal, dtype=torch.float32).view(1, width)
    d[1] = torch.arange(cy / focal, (cy - height + 1e-5) / focal, -1 / focal, dtype=torch.float32).view(height, 1)
    d[2] = -1
    d = d.permute(1, 2, 0)
    pose = torch.as_tensor(pose, dtype=torch.float32)
    rays_d = (d @ pose[:3, :3].T).reshape(-1, 3)
    rays_o = pose[:3, 3].expand(rays_d.shape)
    return torch.cat([rays_o, rays_d], 1)


def sample_ray(f: Field, rays_o, rays_d, n_samples: int):
    """Uniform samples from the slab entry point.  app/models/gridnerf_sequential.py:260-281
    (``is_train=False`` branch)."""
    vec = torch.where(rays_d == 0, torch.full_like(rays_d, 1e-6), rays_d)
    rate_a = (f.aabb[1] - rays_o) / vec
    rate_b = (f.aabb[0] - rays_o) / vec
    t_min = torch.minimum(rate_a, rate_b).amax(-1).clamp(min=f.near, max=f.far)
    rng = torch.arange(n_samples, device=rays_o.device)[None].float()
    step = f.step_size * rng
    interpx = t_min[..., None] + step
    pts = rays_o[..., None, :] + rays_d[..., None, :] * interpx[..., None]
    outside = ((f.aabb[0] > pts) | (pts > f.aabb[1])).any(dim=-1)
    return pts, interpx, ~outside, t_min


def sample_ray_within_hull(f: Field, rays_o, rays_d, n_samples: int):
    """Samples between ``near`` and the ray's hit with the ground plane ``z = aabb_min_z``.
    app/models/gridnerf_sequential.py:298-319 (``is_train=False`` branch)."""
    near = f.near
    o_z = rays_o[:, -1:] - f.aabb[0, 2].item()
    d_z = rays_d[:, -1:]
    far = -(o_z / d_z)
    far[rays_d[:, 2] >= 0] = f.far
    t_vals = torch.linspace(0.0, 1.0, steps=n_samples, device=rays_o.device)
    z_vals = near * (1.0 - t_vals) + far * (t_vals)
    pts = rays_o[..., None, :] + rays_d[..., None, :] * z_vals[..., :, None]
    outside = ((f.aabb[0] > pts) | (pts > f.aabb[1])).any(dim=-1)
    return pts, z_vals, ~outside, far[:, 0]


def sample_alpha(f: Field, pts):
    """Trilinear occupancy lookup.  app/models/alpha_mask.py:35-59."""
    q = (pts - f.alpha_aabb[0]) * f.alpha_inv - 1
    return F.grid_sample(f.alpha_volume, q.view(1, -1, 1, 1, 3), align_corners=True).view(-1)


def _coords(xyz, n: int = 3):
    plane = torch.stack([xyz[..., list(MAT_MODE[i])] for i in range(n)]).view(n, -1, 1, 2)
    line = torch.stack([xyz[..., VEC_MODE[i]] for i in range(n)])
    line = torch.stack((torch.zeros_like(line), line), dim=-1).view(n, -1, 1, 2)
    return plane, line


def density_feature(f: Field, xyz):
    """Sum over planes and channels of plane x line.  app/models/gridnerf_sequential.py:779-827."""
    cp, cl = _coords(xyz, f.ndims)
    sigma = torch.zeros((xyz.shape[0],), device=xyz.device)
    for i in range(len(f.density_plane)):
        d = i // f.n_res
        p = F.grid_sample(f.density_plane[i], cp[[d]], align_corners=True).view(-1, xyz.shape[0])
        l = F.grid_sample(f.density_line[i], cl[[d]], align_corners=True).view(-1, xyz.shape[0])
        sigma = sigma + torch.sum(p * l, dim=0)
    return sigma


def feature2density(f: Field, feat):
    """app/models/gridnerf_sequential.py:386-399."""
    if f.act == "softplus":
        return F.softplus(feat + f.density_shift)
    return F.relu(feat)


def app_feature(f: Field, xyz):
    """Plane x line products, concatenated and projected by ``basis_mat``.
    app/models/gridnerf_sequential.py:829-871."""
    cp, cl = _coords(xyz, f.ndims)
    ps, ls = [], []
    for i in range(len(f.app_plane)):
        d = i // f.n_res
        ps.append(F.grid_sample(f.app_plane[i], cp[[d]], align_corners=True).view(-1, xyz.shape[0]))
        ls.append(F.grid_sample(f.app_line[i], cl[[d]], align_corners=True).view(-1, xyz.shape[0]))
    prod = (torch.cat(ps) * torch.cat(ls)).T
    return F.linear(prod, f.basis_w)


def positional_encoding(x, freqs: int):
    """app/tools/utils.py:42-48."""
    bands = 2 ** torch.arange(freqs, dtype=torch.float, device=x.device)
    pts = (x[..., None] * bands).reshape(x.shape[:-1] + (freqs * x.shape[-1],))
    return torch.cat([torch.sin(pts), torch.cos(pts)], dim=-1)


def mlp_render(f: Field, viewdirs, feats, latent=None):
    """Appearance MLP.  app/models/mlp_render_fea.py:44-68; ``latent [M, 48]`` is the appearance
    embedding when the model was built with encode_app."""
    parts = [feats] if latent is None else [feats, latent]
    if f.view_pe > -1:
        parts.append(viewdirs)
    if f.fea_pe > 0:
        parts.append(positional_encoding(feats, f.fea_pe))
    if f.view_pe > 0:
        parts.append(positional_encoding(viewdirs, f.view_pe))
    x = torch.cat(parts, dim=-1)
    x = torch.relu(F.linear(x, f.mlp_w[0], f.mlp_b[0]))
    x = torch.relu(F.linear(x, f.mlp_w[1], f.mlp_b[1]))
    return torch.sigmoid(F.linear(x, f.mlp_w[2], f.mlp_b[2]))


def raw2alpha(sigma, dist):
    """app/tools/utils.py:51-64."""
    alpha = 1.0 - torch.exp(-sigma * dist)
    trans = torch.cumprod(torch.cat([torch.ones(alpha.shape[0], 1, device=alpha.device), 1.0 - alpha + 1e-10], -1), -1)
    return alpha, alpha * trans[:, :-1], trans[:, -1:]


@torch.no_grad()
def render_chunk(f: Field, rays: torch.Tensor, n_samples: int = -1, white_bg: bool = True,
                 keep_stages: bool = False, sampling_opt: bool = False, app_code=None):
    """One chunk through ``GridBaseSequential.forward``: the dense-sampling branch
    (app/models/gridnerf_sequential.py:448-504) or, with ``sampling_opt``, the hull-sampling
    branch (:522-576, ``n_samples`` playing the role of ``n_importance``).  Returns ``rgb_map [N,3]``,
    ``depth_map [N]`` and, with ``keep_stages``, every intermediate the parity tests compare."""
    rays = rays.float()
    rays_o, viewdirs = rays[:, :3], rays[:, 3:6]
    n_samples = n_samples if n_samples > 0 else f.n_samples_default
    if sampling_opt:
        pts, z_vals, ray_valid, t_min = sample_ray_within_hull(f, rays_o, viewdirs, n_samples)
    else:
        pts, z_vals, ray_valid, t_min = sample_ray(f, rays_o, viewdirs, n_samples)
    in_box = ray_valid.clone()
    dists = torch.cat((z_vals[:, 1:] - z_vals[:, :-1], torch.zeros_like(z_vals[:, :1])), dim=-1)
    view_exp = viewdirs.view(-1, 1, 3).expand(pts.shape)
    if f.alpha_volume is not None:
        alphas = sample_alpha(f, pts[ray_valid])
        alpha_mask = alphas > f.alpha_filter_thres
        ray_invalid = ~ray_valid
        ray_invalid[ray_valid] |= ~alpha_mask
        ray_valid = ~ray_invalid
    sigma = torch.zeros(pts.shape[:-1], device=pts.device)
    rgb = torch.zeros((*pts.shape[:2], 3), device=pts.device)
    xyz = pts
    sigma_feat = None
    if ray_valid.any():
        xyz = (pts - f.aabb[0]) * f.inv_aabb_size - 1
        sigma_feat = density_feature(f, xyz[ray_valid])
        sigma[ray_valid] = feature2density(f, sigma_feat)
    _, weight, _ = raw2alpha(sigma, dists * f.distance_scale)
    app_mask = weight > f.ray_weight_thres
    feats = None
    if app_mask.any():
        feats = app_feature(f, xyz[app_mask])
        latent = None
        if f.embedding_app is not None:
            # compute_app_latent, app/models/gridnerf_sequential.py:429-437: the same row for every sample
            idx = torch.ones(pts.shape[:-1], dtype=torch.long, device=pts.device) * torch.as_tensor(app_code).long().to(pts.device)
            latent = F.embedding(idx[app_mask], f.embedding_app)
        rgb[app_mask] = mlp_render(f, view_exp[app_mask], feats, latent)
    acc = torch.sum(weight, -1)
    rgb_map = torch.sum(weight[..., None] * rgb, -2)
    if white_bg:
        rgb_map = rgb_map + (1.0 - acc[..., None])
    rgb_map = rgb_map.clamp(0, 1)
    depth_map = torch.sum(weight * z_vals, -1)
    out = {"rgb_map": rgb_map, "depth_map": depth_map}
    if keep_stages:
        out.update({
            "t_min": t_min, "in_box": in_box, "ray_valid": ray_valid, "sigma": sigma,
            "sigma_feature": sigma_feat, "weight": weight, "app_mask": app_mask,
            "app_features": feats, "rgb": rgb, "acc": acc, "z_vals": z_vals,
        })
    return out


@torch.no_grad()
def render_rays(f: Field, rays: torch.Tensor, n_samples: int = -1, white_bg: bool = True,
                chunk: int = 8192):
    """Host chunk loop.  dist_render/ddp_infer/inferer_impl.py:95-120."""
    rgbs, depths = [], []
    for s in range(0, rays.shape[0], chunk):
        o = render_chunk(f, rays[s:s + chunk], n_samples, white_bg)
        rgbs.append(o["rgb_map"])
        depths.append(o["depth_map"])
    return torch.cat(rgbs, 0), torch.cat(depths, 0)


def compute_alpha(f: Field, xyz_locs, length):
    """alpha of free points over a segment of ``length``.  app/models/gridnerf_sequential.py:401-427."""
    if f.alpha_volume is not None:
        alpha_mask = sample_alpha(f, xyz_locs) > 0
    else:
        alpha_mask = torch.ones_like(xyz_locs[:, 0], dtype=torch.bool)
    sigma = torch.zeros(xyz_locs.shape[:-1])
    if alpha_mask.any():
        xyz = (xyz_locs[alpha_mask] - f.aabb[0]) * f.inv_aabb_size - 1
        sigma[alpha_mask] = feature2density(f, density_feature(f, xyz))
    return 1 - torch.exp(-sigma * length)


def update_alpha_mask(f: Field, grid_size, alpha_mask_thres: float = 1e-3, increase_alpha_thresh: int = 0):
    """getDenseAlpha + updateAlphaMask, app/models/gridnerf_sequential.py:321-384: alpha on a dense
    lattice of the box, 3x3x3 max pooling, threshold.  Returns the new 0/1 volume ``[D, H, W]`` and
    the bounding box of its occupied lattice points."""
    gx, gy, gz = [int(g) for g in grid_size]
    samples = torch.stack(torch.meshgrid(torch.linspace(0, 1, gx), torch.linspace(0, 1, gy), torch.linspace(0, 1, gz),
                                         indexing="ij"), -1)
    dense_xyz = f.aabb[0] * (1 - samples) + f.aabb[1] * samples
    alpha = torch.zeros_like(dense_xyz[..., 0])
    for i in range(gx):
        alpha[i] = compute_alpha(f, dense_xyz[i].view(-1, 3), f.step_size).view(gy, gz)
    dense_xyz = dense_xyz.transpose(0, 2).contiguous()
    alpha = alpha.clamp(0, 1).transpose(0, 2).contiguous()[None, None]
    alpha = F.max_pool3d(alpha, kernel_size=3, padding=1, stride=1).view(gz, gy, gx)
    thres = alpha_mask_thres * (10 ** increase_alpha_thresh)
    volume = alpha >= thres
    valid_xyz = dense_xyz[volume]
    return volume, torch.stack((valid_xyz.amin(0), valid_xyz.amax(0)))


def field_from_checkpoint(ckpt: Dict[str, object], alpha_filter_thres: float = 0.0, ndims: int = 3, res_mode=(1,)) -> Field:
    """Unpack a checkpoint dict the way ``GridBaseSequential.load`` does
    (app/models/gridnerf_sequential.py:225-242)."""
    import numpy as np

    vol = aabb = None
    if "alphaMask.aabb" in ckpt:
        shape = tuple(ckpt["alphaMask.shape"])
        n = int(np.prod(shape))
        vol = torch.from_numpy(np.unpackbits(ckpt["alphaMask.mask"])[:n].reshape(shape))
        aabb = ckpt["alphaMask.aabb"]
    sd = {k: v.detach().cpu() for k, v in ckpt["state_dict"].items()}
    return Field(sd, ckpt["kwargs"], vol, aabb, alpha_filter_thres, ndims, res_mode)
