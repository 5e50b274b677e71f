"""``B200GridNeRF``: the reference's ``GridNeRF`` model API on top of ``libgridnerf_b200.so``.

Same constructor arguments, state-dict keys, checkpoint format, ``load`` and ``forward``
signature as ``app/models/gridnerf_sequential.py`` (``GridBaseSequential.__init__`` :46-132,
``save``/``load`` :209-242, ``forward`` :439-658, ``GridNeRF`` :661-747), so that
``GridNeRF(**ckpt["kwargs"], device=..., args=..., is_train=False); model.load(ckpt)`` and the
``renderer_fn`` chunk loops (app/tools/render_utils.py:15-63,
dist_render/ddp_infer/inferer_impl.py:95-120) work unchanged.  All device work of ``forward``
happens in the CUDA library; torch only owns the tensors.

Rendering only: ``is_train=True`` and the NeRF refinement branch (``run_nerf``) raise
``NotImplementedError``.  With ``args.encode_app`` the 48-d appearance latent of ``app_code``
(``embedding_app``, gridnerf_sequential.py:429-437,681-682) is the same for every sample of a call, so
its layer-1 contribution ``W1[:, 27:75] @ latent`` is folded into the layer-1 bias when ``app_code``
changes; the kernels keep their 150-wide input.  Both samplers are supported: the dense
``sample_ray`` and, with ``args.sampling_opt``, ``sample_ray_within_hull`` with ``n_importance`` samples.
"""

from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import numpy as np
import torch

from . import _lib
from ._lib import GnrConfig, check, lib

MAT_MODE = [[0, 1], [0, 2], [1, 2]]
VEC_MODE = [2, 1, 0]


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class AlphaGridMask(torch.nn.Module):
    """Occupancy volume holder with the attributes of app/models/alpha_mask.py:16-26."""

    def __init__(self, device, aabb, alpha_volume):
        super().__init__()
        self.device = device
        aabb_cpu = aabb.detach().cpu().float()
        size_cpu = aabb_cpu[1] - aabb_cpu[0]
        self.aabb = aabb_cpu.to(device)
        self.aabbSize = size_cpu.to(device)
        self.invgridSize = (1.0 / size_cpu * 2).to(device)  # evaluated on the CPU, see update_stepSize
        self.alpha_volume = alpha_volume.view(1, 1, *alpha_volume.shape[-3:])
        self.gridSize = torch.LongTensor(
            [alpha_volume.shape[-1], alpha_volume.shape[-2], alpha_volume.shape[-3]]
        ).to(device)


class _MLPRenderFea(torch.nn.Module):
    """Parameter holder with the layout of app/models/mlp_render_fea.py:20-42."""

    def __init__(self, in_chanel, viewpe, feape, feature_c, bias_enable, encode_app=False):
        super().__init__()
        self.encode_app = bool(encode_app)
        self.in_mlpC = (2 * max(viewpe, 0) * 3 + 2 * feape * in_chanel + 3 * (viewpe > -1) + in_chanel
                        + (48 if self.encode_app else 0))
        self.viewpe, self.feape = viewpe, feape
        self.mlp = torch.nn.Sequential(
            torch.nn.Linear(self.in_mlpC, feature_c, bias=bool(bias_enable)),
            torch.nn.ReLU(inplace=True),
            torch.nn.Linear(feature_c, feature_c, bias=bool(bias_enable)),
            torch.nn.ReLU(inplace=True),
            torch.nn.Linear(feature_c, 3, bias=bool(bias_enable)),
        )
        if bias_enable:
            torch.nn.init.constant_(self.mlp[-1].bias, 0)


class B200GridNeRF(torch.nn.Module):
    # MLP precision modes of the library (GnrConfig.mlp_mode)
    MLP_FP32, MLP_TC_SPLIT, MLP_TC_BF16 = 0, 1, 2

    def __init__(  # noqa: PLR0913 -- the reference's signature
        self,
        aabb,
        gridSize,
        device,
        density_n_comp=8,
        appearance_n_comp=24,
        app_dim=27,
        alphaMask=None,
        near_far=(2.0, 6.0),
        density_shift=-10,
        alphaMask_thres=0.001,
        distance_scale=25,
        rayMarch_weight_thres=0.001,
        pos_pe=6,
        view_pe=6,
        fea_pe=6,
        featureC=128,
        step_ratio=2.0,
        fea2denseAct="softplus",
        use_plane_split=True,
        args=None,
        group=None,
        is_train=False,
        mlp_mode: int = 0,
        field_grid=None,
        ert_transmittance: float = 0.0,
        app_plane_fp16: bool = False,
        density_plane_fp16: bool = False,
        density_lattice: bool = False,
        fused_appearance: bool = True,
        appearance_lattice: bool = False,
        **_ignored,
    ):
        super().__init__()
        if args is None:
            raise ValueError("args namespace required (same attributes as the reference's ArgsConfig)")
        if is_train:
            raise NotImplementedError("B200GridNeRF renders only; training stays with the reference model")
        if getattr(args, "run_nerf", False):
            raise NotImplementedError("run_nerf (NeRF refinement branch) is not part of the render path")
        if getattr(args, "nonlinear_density", False):
            raise NotImplementedError("nonlinear_density is not supported")
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("B200GridNeRF needs a CUDA device (sm_100a); there is no CPU path")
        self.device = dev
        self.args = args
        self.ndims = int(getattr(args, "ndims", 3))
        self.resMode = list(args.resMode) if getattr(args, "resMode", None) is not None else [1]
        if isinstance(density_n_comp, int):
            density_n_comp = [density_n_comp] * 3
        if isinstance(appearance_n_comp, int):
            appearance_n_comp = [appearance_n_comp] * 3
        self.density_n_comp = list(density_n_comp)[: self.ndims]
        self.app_n_comp = list(appearance_n_comp)[: self.ndims]
        if len(set(self.density_n_comp)) != 1 or len(set(self.app_n_comp)) != 1:
            raise NotImplementedError("planes of one kind must share a channel count")
        self.app_dim = app_dim
        self.aabb = torch.as_tensor(aabb, dtype=torch.float32).to(dev)
        self.alphaMask = alphaMask
        self.density_shift = density_shift
        self.alphaMask_thres = alphaMask_thres
        self.distance_scale = distance_scale
        self.rayMarch_weight_thres = rayMarch_weight_thres
        self.fea2denseAct = fea2denseAct
        self.near_far = list(near_far)
        self.step_ratio = step_ratio
        self.pos_pe, self.view_pe, self.fea_pe, self.featureC = pos_pe, view_pe, fea_pe, featureC
        self.matMode = MAT_MODE[: self.ndims]
        self.vecMode = VEC_MODE[: self.ndims]
        self.sampling_opt = getattr(args, "sampling_opt", 0)
        self.n_importance = getattr(args, "n_importance", 128)
        self.alpha_mask_filter_thre = getattr(args, "alpha_mask_filter_thre", 0.0) or 0.0
        self.mlp_mode = int(mlp_mode)
        # early ray termination of the density pass (see GnrConfig.ert_transmittance); 0 = exact
        self.ert_transmittance = float(ert_transmittance)
        # Appearance planes and lines held as fp16 in the library (GnrConfig.app_storage); mlp_mode 2 only.
        # args.half_precision_param is the reference's switch for half planes (inferer_impl.py:251,263-267:
        # density_plane and app_plane become fp16, the lines stay fp32).  Here it selects fp16 appearance
        # storage when the tensor-core MLP is in use (planes AND lines: the gather interpolates in packed
        # fp16) and leaves the density field in fp32: fp16 density moves weights across the w > 1e-3
        # appearance threshold, so it is only ever switched on explicitly (density_plane_fp16=True).
        self.app_plane_fp16 = bool(app_plane_fp16) or (bool(getattr(args, "half_precision_param", False))
                                                       and int(mlp_mode) == 2)
        self.density_plane_fp16 = bool(density_plane_fp16)
        # Density from the pre-summed lattice (gnr_build_density_lattice): one fp32 scalar per grid point,
        # built on the device from the planes and lines at commit(); the same function of position, 8
        # scalar taps per sample instead of 18 texels x 16 channels.  Costs 4 bytes per grid point of HBM.
        self.density_lattice = bool(density_lattice)
        # Appearance features from a baked lattice (gnr_build_appearance_lattice): 64 bytes per grid point of HBM
        # (69 GB for the city block), 8 taps per sample, no plane gather and no projection GEMM; mlp_mode 2 only
        self.appearance_lattice = bool(appearance_lattice)
        # forward() runs appearance gather + basis projection + MLP as one kernel when the library can
        # (mlp_mode 2 with fp16 appearance planes); False keeps the separate kernels (GnrConfig.unfused_appearance)
        # ("groups" = True: three groups of warps share two accumulators; "two_groups": two groups, one accumulator
        # each; "stream": dedicated gather warps)
        self.fused_appearance = (fused_appearance if fused_appearance in ("stream", "groups", "two_groups")
                                 else bool(fused_appearance))
        self.update_stepSize(gridSize)

        # learnable tensors, reference layout and names (gridnerf_sequential.py:669-747)
        # ``field_grid``: resolution of the stored planes when it differs from ``gridSize`` (which
        # fixes the step size); a model that only samples and composites keeps 2x2 planes.
        g = [int(v) for v in (field_grid if field_grid is not None else self.gridSize.tolist())]
        dp, dl, ap, al = [], [], [], []
        for i in range(len(self.vecMode)):
            m0, m1 = self.matMode[i]
            for j in self.resMode:
                dp.append(torch.nn.Parameter(torch.zeros((1, self.density_n_comp[i], g[m1] * j, g[m0] * j), device=dev), requires_grad=False))
                dl.append(torch.nn.Parameter(torch.zeros((1, self.density_n_comp[i], g[self.vecMode[i]] * j, 1), device=dev), requires_grad=False))
                ap.append(torch.nn.Parameter(torch.zeros((1, self.app_n_comp[i], g[m1] * j, g[m0] * j), device=dev), requires_grad=False))
                al.append(torch.nn.Parameter(torch.zeros((1, self.app_n_comp[i], g[self.vecMode[i]] * j, 1), device=dev), requires_grad=False))
        self.density_plane = torch.nn.ParameterList(dp)
        self.density_line = torch.nn.ParameterList(dl)
        self.app_plane = torch.nn.ParameterList(ap)
        self.app_line = torch.nn.ParameterList(al)
        self.basis_mat = torch.nn.Linear(sum(self.app_n_comp) * len(self.resMode), self.app_dim, bias=False).to(dev)
        self.encode_app = bool(getattr(args, "encode_app", False))
        if self.encode_app:
            self.embedding_app = torch.nn.Embedding(11500, 48).to(dev)
        self._app_code = None  # the appearance code whose latent is currently folded into the uploaded bias
        self.renderModule = _MLPRenderFea(self.app_dim, view_pe, fea_pe, featureC, getattr(args, "bias_enable", 0),
                                          self.encode_app).to(dev)
        for p in self.parameters():
            p.requires_grad_(False)

        self._handle = C.c_void_p(0)
        self._committed = False
        self._hull_tables_for = -1
        self._ws: Dict[int, torch.Tensor] = {}        # chunk slot -> scratch buffer (grows, never shrinks)
        self._ws_bytes: Dict[tuple, int] = {}          # chunk shape -> bytes the library asks for
        self._last_workspaces: list = []               # buffers the last render_rays call used
        # capacities of the two compacted sample lists, per ray of a chunk
        self.valid_capacity_per_ray: Optional[int] = None  # None = n_samples (can never overflow)
        self.app_capacity_per_ray = 192
        self.check_status_every_call = True
        self.last_status: Optional[np.ndarray] = None

    # -- geometry scalars (:149-164) -------------------------------------------------------------
    def update_stepSize(self, gridSize):
        """Same expressions as the reference, evaluated on CPU tensors: torch's CUDA ``mean``
        multiplies by 1/N where the CPU divides by N, which moves ``stepSize`` by one ulp for
        anisotropic grids and with it every sample position.  The CPU values are the ones the
        sampler's bit-exactness is defined against; device copies are kept for API parity."""
        aabb = self.aabb.detach().cpu()
        aabb_size = aabb[1] - aabb[0]
        grid = torch.tensor(gridSize)
        units = aabb_size / (grid - 1)
        step = torch.mean(units) * self.step_ratio
        diag = torch.sqrt(torch.sum(torch.square(aabb_size)))
        dev = self.aabb.device
        self.aabbSize = aabb_size.to(dev)
        self.invaabbSize = (2.0 / aabb_size).to(dev)
        self.gridSize = grid.to(dev)
        self.units = units.to(dev)
        self.stepSize = step.to(dev)
        self.aabbDiag = diag.to(dev)
        self.nSamples = int((diag / step).item()) + 1

    def get_kwargs(self):
        return {
            "aabb": self.aabb,
            "gridSize": self.gridSize.tolist(),
            "density_n_comp": self.density_n_comp,
            "appearance_n_comp": self.app_n_comp,
            "app_dim": self.app_dim,
            "density_shift": self.density_shift,
            "alphaMask_thres": self.alphaMask_thres,
            "distance_scale": self.distance_scale,
            "rayMarch_weight_thres": self.rayMarch_weight_thres,
            "fea2denseAct": self.fea2denseAct,
            "near_far": self.near_far,
            "step_ratio": self.step_ratio,
            "pos_pe": self.pos_pe,
            "view_pe": self.view_pe,
            "fea_pe": self.fea_pe,
            "featureC": self.featureC,
        }

    def normalize_coord(self, xyz_sampled):
        return (xyz_sampled - self.aabb[0]) * self.invaabbSize - 1

    # -- checkpoint I/O (:209-242) -----------------------------------------------------------------
    def save(self, path):
        ckpt = {"kwargs": self.get_kwargs(), "state_dict": self.state_dict()}
        if self.alphaMask is not None:
            alpha_volume = self.alphaMask.alpha_volume.bool().cpu().numpy()
            ckpt.update({"alphaMask.shape": alpha_volume.shape})
            ckpt.update({"alphaMask.mask": np.packbits(alpha_volume.reshape(-1))})
            ckpt.update({"alphaMask.aabb": self.alphaMask.aabb.cpu()})
        torch.save(ckpt, path)

    def load(self, ckpt):
        if "alphaMask.aabb" in ckpt.keys():
            length = int(np.prod(ckpt["alphaMask.shape"]))
            alpha_volume = torch.from_numpy(
                np.unpackbits(ckpt["alphaMask.mask"])[:length].reshape(ckpt["alphaMask.shape"])
            )
            self.alphaMask = AlphaGridMask(self.device, ckpt["alphaMask.aabb"].to(self.device),
                                           alpha_volume.float().to(self.device))
        self.load_state_dict(ckpt["state_dict"], strict=False)
        self.commit()

    # -- library handle ----------------------------------------------------------------------------
    def _config(self) -> GnrConfig:
        cfg = GnrConfig()
        aabb = self.aabb.detach().cpu().numpy().astype(np.float32)
        inv = self.invaabbSize.detach().cpu().numpy().astype(np.float32)
        for a in range(3):
            cfg.aabb[a] = float(aabb[0, a])
            cfg.aabb[3 + a] = float(aabb[1, a])
            cfg.inv_aabb_size[a] = float(inv[a])
            cfg.grid[a] = int(self.gridSize[a])
        cfg.near_t, cfg.far_t = float(self.near_far[0]), float(self.near_far[1])
        cfg.step_size = float(self.stepSize.item())
        cfg.distance_scale = float(self.distance_scale)
        cfg.density_shift = float(self.density_shift)
        if self.fea2denseAct not in ("softplus", "relu"):
            raise ValueError(f"fea2denseAct {self.fea2denseAct!r} (softplus|relu)")
        cfg.density_act = 0 if self.fea2denseAct == "softplus" else 1
        cfg.ray_weight_thres = float(self.rayMarch_weight_thres)
        cfg.alpha_filter_thres = float(self.alpha_mask_filter_thre)
        cfg.n_pairs = len(self.density_plane)
        cfg.n_density = int(self.density_n_comp[0])
        cfg.n_app = int(self.app_n_comp[0])
        cfg.app_dim = int(self.app_dim)
        cfg.fea_pe, cfg.view_pe = int(self.fea_pe), int(self.view_pe)
        cfg.hidden = int(self.featureC)
        cfg.has_bias = int(self.renderModule.mlp[0].bias is not None or self.encode_app)
        cfg.mlp_mode = self.mlp_mode
        cfg.sampling_mode = 1 if self.sampling_opt else 0
        cfg.ert_transmittance = self.ert_transmittance
        cfg.app_storage = 1 if self.app_plane_fp16 else 0
        cfg.den_storage = 1 if self.density_plane_fp16 else 0
        # True / "groups": three groups of warps that each gather and run the MLP of their tile; "stream": gather warps
        # feed MLP warps through tensor memory; False: separate kernels
        cfg.unfused_appearance = {True: 0, "groups": 0, "stream": 2, "two_groups": 3, False: 1}[self.fused_appearance]
        return cfg

    def commit(self, release_torch_planes: bool = False):
        """(Re)create the library model from the current parameters: converts planes and
        lines to channel-last, bit-packs the occupancy volume, re-tiles the MLP weights."""
        self._release()
        self._hull_tables_for = -1
        dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        cfg = self._config()
        h = C.c_void_p(0)
        check(lib.gnr_create(C.byref(cfg), dev_index, C.byref(h)), "gnr_create")
        self._handle = h
        st = _stream()
        n_res = len(self.resMode)
        with torch.cuda.device(self.device):
            for kind, planes, lines in ((0, self.density_plane, self.density_line), (1, self.app_plane, self.app_line)):
                for idx in range(len(planes)):
                    dim = idx // n_res
                    p = planes[idx].detach().float().contiguous()
                    l_ = lines[idx].detach().float().contiguous()
                    check(lib.gnr_upload_plane(h, kind, idx, _ptr(p), p.shape[1], p.shape[2], p.shape[3],
                                               self.matMode[dim][0], self.matMode[dim][1], st), "gnr_upload_plane")
                    check(lib.gnr_upload_line(h, kind, idx, _ptr(l_), l_.shape[1], l_.shape[2], self.vecMode[dim], st),
                          "gnr_upload_line")
            if self.density_lattice:
                check(lib.gnr_build_density_lattice(h, 1, st), "gnr_build_density_lattice")
            self._upload_alpha_mask(st)
            self._upload_mlp(st)
            if self.appearance_lattice:
                check(lib.gnr_build_appearance_lattice(h, 1, st), "gnr_build_appearance_lattice")
            torch.cuda.current_stream().synchronize()
        self._committed = True
        if release_torch_planes:
            self.release_torch_planes()

    def _upload_alpha_mask(self, st=None):
        """Occupancy volume -> library (bit-packed there, with its coarse grid)."""
        if self.alphaMask is None:
            return
        with torch.cuda.device(self.device):
            vol = (self.alphaMask.alpha_volume[0, 0] > 0).to(torch.uint8).contiguous().to(self.device)
            d_, h_, w_ = vol.shape
            a = self.alphaMask.aabb.detach().cpu().numpy().astype(np.float32)
            inv = self.alphaMask.invgridSize.detach().cpu().numpy().astype(np.float32)
            a_c = (C.c_float * 6)(*[float(v) for v in a.reshape(-1)])
            i_c = (C.c_float * 3)(*[float(v) for v in inv])
            check(lib.gnr_upload_alpha_mask(self._handle, _ptr(vol), d_, h_, w_, a_c, i_c, st if st is not None else _stream()),
                  "gnr_upload_alpha_mask")
            torch.cuda.current_stream(self.device).synchronize()  # `vol` must outlive the packing kernels

    def _upload_mlp(self, st=None):
        """basis_mat and the three MLP layers -> library.  With encode_app the latent columns
        (27..74) of layer 1 are removed and their product with the current latent joins the bias."""
        mlp = self.renderModule.mlp
        ws = [mlp[i].weight.detach().float().contiguous() for i in (0, 2, 4)]
        bs = [mlp[i].bias.detach().float().contiguous() if mlp[i].bias is not None else None for i in (0, 2, 4)]
        if self.encode_app:
            a = self.app_dim
            w1 = ws[0]
            b1 = bs[0] if bs[0] is not None else torch.zeros(w1.shape[0], device=self.device)
            if self._app_code is not None:
                latent = self.embedding_app.weight.detach()[int(self._app_code)].float()
                b1 = b1 + w1[:, a:a + 48] @ latent
            ws[0] = torch.cat([w1[:, :a], w1[:, a + 48:]], dim=1).contiguous()
            bs[0] = b1.contiguous()
        bw = self.basis_mat.weight.detach().float().contiguous()
        check(lib.gnr_upload_mlp(self._handle, _ptr(bw), _ptr(ws[0]), _ptr(bs[0]), _ptr(ws[1]), _ptr(bs[1]), _ptr(ws[2]),
                                 _ptr(bs[2]), st if st is not None else _stream()), "gnr_upload_mlp")
        torch.cuda.current_stream(self.device).synchronize()  # the temporaries above must outlive the copy kernels

    def set_app_code(self, app_code):
        """Select the appearance embedding row used by the following renders (encode_app models)."""
        if not self.encode_app:
            return
        if app_code is None:
            raise ValueError("this model was built with encode_app: forward needs an app_code")
        code = int(app_code.item()) if isinstance(app_code, torch.Tensor) else int(app_code)
        if code != self._app_code:
            self._app_code = code
            with torch.cuda.device(self.device):
                self._upload_mlp()
                if self.appearance_lattice:  # (the latent only moves the layer-1 bias, but an MLP upload marks the lattice stale)
                    check(lib.gnr_build_appearance_lattice(self._handle, 1, _stream()), "gnr_build_appearance_lattice")

    @torch.no_grad()
    def updateAlphaMask(self, gridSize=(200, 200, 200), increase_alpha_thresh=0):
        """Regenerate the occupancy mask from the current density field, as
        app/models/gridnerf_sequential.py:321-384 does: alpha over one step at the points of a dense
        lattice of the box (points the current mask already rules out keep alpha 0), 3x3x3 max
        pooling, threshold ``alphaMask_thres * 10**increase_alpha_thresh``.  The density of the
        lattice points comes from the library's point-mode entry; the new mask is uploaded to the
        library.  Returns the bounding box of the occupied lattice points."""
        if not self._committed:
            self.commit()
        from .model_parallel import density_points  # point-mode wrapper over gnr_density_points

        gx, gy, gz = [int(g) for g in gridSize]
        dev = self.device
        samples = torch.stack(torch.meshgrid(torch.linspace(0, 1, gx), torch.linspace(0, 1, gy), torch.linspace(0, 1, gz),
                                             indexing="ij"), -1).to(dev)
        dense_xyz = self.aabb[0] * (1 - samples) + self.aabb[1] * samples
        alpha = torch.zeros_like(dense_xyz[..., 0])
        for i in range(gx):
            pts = dense_xyz[i].view(-1, 3)
            if self.alphaMask is not None:
                q = (pts - self.alphaMask.aabb[0]) * self.alphaMask.invgridSize - 1
                keep = torch.nn.functional.grid_sample(self.alphaMask.alpha_volume, q.view(1, -1, 1, 1, 3),
                                                       align_corners=True).view(-1) > 0
            else:
                keep = torch.ones(pts.shape[0], dtype=torch.bool, device=dev)
            sigma = torch.zeros(pts.shape[0], device=dev)
            if bool(keep.any()):
                xyz = ((pts[keep] - self.aabb[0]) * self.invaabbSize - 1).contiguous()
                sigma[keep] = density_points(self, xyz)
            alpha[i] = (1 - torch.exp(-sigma * self.stepSize)).view(gy, gz)
        dense_xyz = dense_xyz.transpose(0, 2).contiguous()
        alpha = alpha.clamp(0, 1).transpose(0, 2).contiguous()[None, None]
        alpha = torch.nn.functional.max_pool3d(alpha, kernel_size=3, padding=1, stride=1).view(gz, gy, gx)
        thres = self.alphaMask_thres * (10 ** increase_alpha_thresh)
        volume = (alpha >= thres).float()
        self.alphaMask = AlphaGridMask(dev, self.aabb, volume)
        self._upload_alpha_mask()
        valid_xyz = dense_xyz[volume > 0.5]
        return torch.stack((valid_xyz.amin(0), valid_xyz.amax(0)))

    @torch.no_grad()
    def reload_field_async(self, state_dict, stream=None):
        """Replace the planes and lines by those of ``state_dict`` (same shapes; pinned host or device
        tensors), everything enqueued on ``stream``: no allocation, no host or device-wide
        synchronisation, so that a copy stream can refill a spare model while another one renders.
        The torch parameters serve as the staging copy, so they must not have been released.
        The caller orders later use after this work (event / wait_stream)."""
        if not self._committed:
            raise RuntimeError("reload_field_async needs a committed model (load a first block with load())")
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        n_res = len(self.resMode)
        with torch.cuda.device(self.device), torch.cuda.stream(st):
            raw = C.c_void_p(st.cuda_stream)
            for kind, planes, lines, pn, ln in ((0, self.density_plane, self.density_line, "density_plane", "density_line"),
                                                (1, self.app_plane, self.app_line, "app_plane", "app_line")):
                for idx in range(len(planes)):
                    p, l_ = planes[idx].data, lines[idx].data
                    if p.numel() == 0 or p.dtype != torch.float32 or not p.is_contiguous():
                        raise RuntimeError("the torch planes were released or are not plain fp32 tensors")
                    src_p, src_l = state_dict[f"{pn}.{idx}"], state_dict[f"{ln}.{idx}"]
                    if tuple(src_p.shape) != tuple(p.shape) or tuple(src_l.shape) != tuple(l_.shape):
                        raise ValueError(f"{pn}.{idx}: block shape {tuple(src_p.shape)} does not fit this model's {tuple(p.shape)}")
                    p.copy_(src_p, non_blocking=True)
                    l_.copy_(src_l, non_blocking=True)
                    dim = idx // n_res
                    check(lib.gnr_upload_plane(self._handle, kind, idx, _ptr(p), p.shape[1], p.shape[2], p.shape[3],
                                               self.matMode[dim][0], self.matMode[dim][1], raw), "gnr_upload_plane")
                    check(lib.gnr_upload_line(self._handle, kind, idx, _ptr(l_), l_.shape[1], l_.shape[2], self.vecMode[dim], raw),
                          "gnr_upload_line")
            if self.density_lattice:  # same size as before: rebuilt in place, stream-ordered
                check(lib.gnr_build_density_lattice(self._handle, 1, raw), "gnr_build_density_lattice")

    def release_torch_planes(self):
        """Drop the torch (NCHW) copies of the planes once the library holds its own
        channel-last copies; ``state_dict()`` no longer contains them afterwards."""
        for plist in (self.density_plane, self.app_plane):
            for p in plist:
                p.data = torch.empty(0, device=self.device)

    def _release(self):
        if getattr(self, "_handle", None) is not None and self._handle.value:
            lib.gnr_destroy(self._handle)
        self._handle = C.c_void_p(0)
        self._committed = False

    def __del__(self):
        try:
            self._release()
        except Exception:
            pass

    # -- chunk plumbing ----------------------------------------------------------------------------
    def capacities(self, n_rays: int, n_samples: int):
        per_valid = n_samples if self.valid_capacity_per_ray is None else min(n_samples, self.valid_capacity_per_ray)
        per_app = min(n_samples, self.app_capacity_per_ray)
        return max(1, n_rays * per_valid), max(1, n_rays * per_app)

    def workspace(self, n_rays: int, n_samples: int, slot: int = 0):
        """Scratch buffer of chunk slot ``slot`` (one per stream that renders chunks concurrently).

        A slot keeps ONE buffer and only ever replaces it by a larger one: the library derives the
        layout from the call's arguments, so a larger buffer serves every smaller shape.  Before a
        buffer is replaced the device is synchronised, because kernels on a side stream may still
        be using it and the caching allocator would hand its memory out again at once.  Callers
        that bake the pointer into a CUDA graph keep their own reference to the returned tensor
        (``GraphedFrameRenderer`` does), which keeps that memory out of the allocator for as long
        as the graph lives."""
        max_valid, max_app = self.capacities(n_rays, n_samples)
        key = (n_rays, n_samples, max_valid, max_app)
        need = self._ws_bytes.get(key)
        if need is None:
            nbytes = C.c_size_t(0)
            check(lib.gnr_workspace_bytes(self._handle, n_rays, n_samples, max_valid, max_app, C.byref(nbytes)),
                  "gnr_workspace_bytes")
            if len(self._ws_bytes) > 256:
                self._ws_bytes.clear()
            need = self._ws_bytes[key] = int(nbytes.value)
        buf = self._ws.get(slot)
        if buf is None or buf.numel() < need + 256:
            if buf is not None:
                torch.cuda.synchronize(self.device)
            buf = torch.empty(need + 256, dtype=torch.uint8, device=self.device)
            self._ws[slot] = buf
        off = (-buf.data_ptr()) % 256
        return buf, C.c_void_p(buf.data_ptr() + off), buf.numel() - off, max_valid, max_app

    def release_workspaces(self):
        """Give the chunk scratch buffers back to the allocator (they are made again on the next render).
        Synchronises the device first: kernels on a side stream may still be using them."""
        torch.cuda.synchronize(self.device)
        self._ws.clear()
        self._last_workspaces = []
        torch.cuda.empty_cache()

    def _samples(self, N_samples: int) -> int:
        if self.sampling_opt:
            # the hull branch ignores N_samples and takes n_importance samples (:528-530)
            s = int(self.n_importance)
            if self._hull_tables_for != s:
                t_vals = torch.linspace(0.0, 1.0, steps=s)  # CPU: the bits of the CPU reference
                near_term = (float(self.near_far[0]) * (1.0 - t_vals)).to(self.device)
                u = t_vals.to(self.device)
                check(lib.gnr_upload_hull_tables(self._handle, s, _ptr(near_term), _ptr(u), _stream()),
                      "gnr_upload_hull_tables")
                torch.cuda.current_stream(self.device).synchronize()
                self._hull_tables_for = s
            return s
        return int(N_samples) if N_samples > 0 else self.nSamples

    def _prepare(self, rays_chunk):
        if not self._committed:
            raise RuntimeError("model parameters were never committed: call load(ckpt) or commit()")
        if rays_chunk.device != self.device and rays_chunk.device.type != "cuda":
            raise RuntimeError("rays must live on the model's CUDA device")
        return rays_chunk.detach().to(torch.float32).contiguous()

    def read_status(self, ws_ptr) -> np.ndarray:
        st = (C.c_int32 * _lib.ST_WORDS)()
        check(lib.gnr_read_status(ws_ptr, st, _stream()), "gnr_read_status")
        self.last_status = np.array(list(st), dtype=np.int64)
        return self.last_status

    def raise_on_status(self, status):
        if status[_lib.ST_OVERFLOW_VALID]:
            raise RuntimeError(f"valid-sample list overflow ({status[_lib.ST_NUM_VALID]} samples): "
                               "raise valid_capacity_per_ray (None = worst case)")
        if status[_lib.ST_OVERFLOW_APP]:
            raise RuntimeError(f"appearance-sample list overflow ({status[_lib.ST_NUM_APP]} samples): "
                               "raise app_capacity_per_ray")
        if status[_lib.ST_WAIT_EXPIRED]:
            raise RuntimeError("a bounded device-side wait expired in the tensor-core MLP kernel")

    # -- the reference's forward (:439-658), rendering branch ---------------------------------------
    def forward(self, rays_chunk, app_code=None, white_bg=True, is_train=False, N_samples=-1, idxs_chunk=None):
        if is_train:
            raise NotImplementedError("is_train=True: training is not part of this package")
        rays = self._prepare(rays_chunk)
        self.set_app_code(app_code)
        n = rays.shape[0]
        s = self._samples(N_samples)
        rgb = torch.empty((n, 3), dtype=torch.float32, device=self.device)
        depth = torch.empty((n,), dtype=torch.float32, device=self.device)
        if n == 0:
            return {"rgb_map": rgb, "depth_map": depth}, {}
        with torch.cuda.device(self.device):
            keep, ws_ptr, ws_bytes, max_valid, max_app = self.workspace(n, s)
            check(lib.gnr_render_chunk(self._handle, _ptr(rays), n, s, int(bool(white_bg)), ws_ptr, ws_bytes,
                                       max_valid, max_app, _ptr(rgb), _ptr(depth), _stream()), "gnr_render_chunk")
            if self.check_status_every_call:
                self.raise_on_status(self.read_status(ws_ptr))
        return {"rgb_map": rgb, "depth_map": depth}, {}

    # -- stage-wise access for parity tests and profiling --------------------------------------------
    @torch.no_grad()
    def run_stages(self, rays_chunk, N_samples=-1, white_bg=True, upto: str = "composite"):
        """Run the chunk stage by stage through the stage-wise C entry points and return every
        intermediate as torch tensors (lists are trimmed to their true lengths)."""
        order = ["sample", "density", "weights", "appearance", "composite"]
        stop = order.index(upto)
        rays = self._prepare(rays_chunk)
        n, s = rays.shape[0], self._samples(N_samples)
        dev = self.device
        out = {}
        with torch.cuda.device(dev):
            keep, ws_ptr, ws_bytes, max_valid, max_app = self.workspace(n, s)
            words = (s + 31) // 32
            t_min = torch.empty(n, dtype=torch.float32, device=dev)
            counts = torch.empty(n, dtype=torch.int32, device=dev)
            offsets = torch.empty(n + 1, dtype=torch.int32, device=dev)
            mask_words = torch.empty((n, words), dtype=torch.int32, device=dev)
            ids = torch.empty(max_valid, dtype=torch.int32, device=dev)
            st = _stream()
            check(lib.gnr_sample(self._handle, _ptr(rays), n, s, ws_ptr, ws_bytes, max_valid, _ptr(t_min), _ptr(counts),
                                 _ptr(offsets), _ptr(mask_words), _ptr(ids), st), "gnr_sample")
            status = self.read_status(ws_ptr)
            self.raise_on_status(status)
            m_v = int(offsets[-1].item())
            kbits = lib.gnr_sample_bits(s)
            ids64 = ids[:m_v].to(torch.int64) & 0xFFFFFFFF
            out.update({"t_min": t_min, "counts": counts, "offsets": offsets, "mask_words": mask_words,
                        "ray_index": ids64 >> kbits, "sample_index": ids64 & ((1 << kbits) - 1), "num_valid": m_v})
            if stop >= 1:
                sf = torch.empty(max_valid, dtype=torch.float32, device=dev)
                sg = torch.empty(max_valid, dtype=torch.float32, device=dev)
                check(lib.gnr_density(self._handle, _ptr(rays), n, s, ws_ptr, ws_bytes, max_valid, _ptr(sf), _ptr(sg), st),
                      "gnr_density")
                out.update({"sigma_feature": sf[:m_v], "sigma": sg[:m_v]})
            if stop >= 2:
                w = torch.empty(max_valid, dtype=torch.float32, device=dev)
                acc = torch.empty(n, dtype=torch.float32, device=dev)
                dep = torch.empty(n, dtype=torch.float32, device=dev)
                ac = torch.empty(n, dtype=torch.int32, device=dev)
                ao = torch.empty(n + 1, dtype=torch.int32, device=dev)
                ai = torch.empty(max_app, dtype=torch.int32, device=dev)
                check(lib.gnr_weights(self._handle, _ptr(rays), n, s, ws_ptr, ws_bytes, max_valid, max_app, _ptr(w),
                                      _ptr(acc), _ptr(dep), _ptr(ac), _ptr(ao), _ptr(ai), st), "gnr_weights")
                self.raise_on_status(self.read_status(ws_ptr))
                m_a = int(ao[-1].item())
                out.update({"weight": w[:m_v], "acc": acc, "depth": dep, "app_counts": ac, "app_offsets": ao,
                            "app_index": ai[:m_a].to(torch.int64), "num_app": m_a})
            if stop >= 3:
                feat = torch.empty((max_app, self.app_dim), dtype=torch.float32, device=dev)
                rgb_s = torch.empty((max_app, 3), dtype=torch.float32, device=dev)
                check(lib.gnr_appearance(self._handle, _ptr(rays), n, s, ws_ptr, ws_bytes, max_valid, max_app, _ptr(feat),
                                         _ptr(rgb_s), st), "gnr_appearance")
                out.update({"app_features": feat[: out["num_app"]], "rgb_samples": rgb_s[: out["num_app"]]})
            if stop >= 4:
                rgb = torch.empty((n, 3), dtype=torch.float32, device=dev)
                depth = torch.empty(n, dtype=torch.float32, device=dev)
                check(lib.gnr_composite(self._handle, n, int(bool(white_bg)), ws_ptr, ws_bytes, max_valid, max_app, s,
                                        _ptr(rgb), _ptr(depth), st), "gnr_composite")
                self.raise_on_status(self.read_status(ws_ptr))
                out.update({"rgb_map": rgb, "depth_map": depth})
            torch.cuda.current_stream().synchronize()
        return out

    def debug_wait(self, expire: bool = False, wait_limit: int = 0):
        """Test hook (gnr_debug_wait): make one bounded device-side wait of the next tensor-core launches
        run out, with ``wait_limit`` polls per wait; ``debug_wait()`` restores normal operation."""
        check(lib.gnr_debug_wait(self._handle, int(bool(expire)), int(wait_limit)), "gnr_debug_wait")

    def profile_enable(self, on: bool = True):
        check(lib.gnr_profile_enable(self._handle, int(on)), "gnr_profile_enable")

    def profile_collect(self):
        """Milliseconds and kernel launches per stage since the last collect."""
        ms = (C.c_float * len(_lib.STAGE_NAMES))()
        launches = (C.c_int64 * len(_lib.STAGE_NAMES))()
        check(lib.gnr_profile_collect(self._handle, ms, launches), "gnr_profile_collect")
        return ({k: float(v) for k, v in zip(_lib.STAGE_NAMES, ms)},
                {k: int(v) for k, v in zip(_lib.STAGE_NAMES, launches)})

    @torch.no_grad()
    def render_rays(self, rays: torch.Tensor, N_samples=-1, white_bg=True, chunk: int = 262144,
                    rgb_out: Optional[torch.Tensor] = None, depth_out: Optional[torch.Tensor] = None,
                    overlap=False, after: Optional["torch.cuda.Event"] = None):
        """Device-resident chunk loop: ``rays [N, 6]`` on the GPU -> ``rgb [N, 3]``, ``depth [N]``
        written in place, one status check at the end instead of one per chunk.
        With ``overlap`` consecutive chunks rotate over that many side streams (``True`` = 2), each
        with its own workspace, so that one chunk's kernels run beside the other's: the stages are
        bound by different units (issue slots, L1, tensor pipe).
        ``after`` (with ``overlap``): the side streams wait for this event instead of for everything queued on the
        current stream.  A caller that keeps several frames in flight passes the event that marks its output
        buffers free (and makes sure the rays were ready before it): the next frame's first chunks then run
        beside the previous frame's last chunk and its assembly instead of behind them."""
        rays = self._prepare(rays)
        n, s = rays.shape[0], self._samples(N_samples)
        if rgb_out is None:
            rgb_out = torch.empty((n, 3), dtype=torch.float32, device=self.device)
        if depth_out is None:
            depth_out = torch.empty((n,), dtype=torch.float32, device=self.device)
        chunk = max(1, min(chunk, n))
        n_chunks = max(1, (n + chunk - 1) // chunk)
        status = torch.zeros((n_chunks, _lib.ST_WORDS), dtype=torch.int32, device=self.device)
        n_side = 2 if overlap is True else int(overlap or 0)
        use_side = n_side > 1 and n_chunks > 1
        with torch.cuda.device(self.device):
            main = torch.cuda.current_stream()
            if use_side:
                if len(getattr(self, "_side_streams", None) or ()) < n_side:
                    self._side_streams = [torch.cuda.Stream(device=self.device) for _ in range(n_side)]
                for st_ in self._side_streams[:n_side]:
                    if after is not None:
                        st_.wait_event(after)
                    else:
                        st_.wait_stream(main)
            used = {}
            for ci, first in enumerate(range(0, n, chunk)):
                m = min(chunk, n - first)
                slot = ci % n_side if use_side else 0
                keep, ws_ptr, ws_bytes, max_valid, max_app = self.workspace(chunk, s, slot)
                used[slot] = keep
                stream = self._side_streams[slot] if use_side else main
                with torch.cuda.stream(stream):
                    check(lib.gnr_render_chunk(self._handle, C.c_void_p(rays.data_ptr() + first * 24), m, s,
                                               int(bool(white_bg)), ws_ptr, ws_bytes, max_valid, max_app,
                                               C.c_void_p(rgb_out.data_ptr() + first * 12),
                                               C.c_void_p(depth_out.data_ptr() + first * 4),
                                               C.c_void_p(stream.cuda_stream)), "gnr_render_chunk")
                    status[ci].copy_(keep[(-keep.data_ptr()) % 256:][: 4 * _lib.ST_WORDS].view(torch.int32))
            if use_side:
                for st_ in self._side_streams[:n_side]:
                    main.wait_stream(st_)
        self._pending_status = status
        self._last_workspaces = list(used.values())
        return rgb_out, depth_out

    def check_pending_status(self):
        """Synchronise and raise if any chunk of the last ``render_rays`` overflowed a list."""
        st = getattr(self, "_pending_status", None)
        if st is None:
            return None
        h = st.cpu().numpy().astype(np.int64)
        agg = np.zeros(_lib.ST_WORDS, dtype=np.int64)
        agg[[0, 1, 4]] = h[:, [0, 1, 4]].max(0)
        agg[[2, 3, 5]] = h[:, [2, 3, 5]].sum(0)
        self.last_status = agg
        self._pending_status = None
        self.raise_on_status(agg)
        return agg

    @torch.no_grad()
    def render_host(self, rays_host: torch.Tensor, N_samples=-1, white_bg=True, chunk: int = 262144,
                    rgb_out: Optional[torch.Tensor] = None, depth_out: Optional[torch.Tensor] = None):
        """Whole chunk loop with HOST buffers (pinned recommended): rays are copied to the
        device chunk by chunk and rgb/depth copied back, all inside the library call."""
        if rays_host.device.type != "cpu" or rays_host.dtype != torch.float32 or not rays_host.is_contiguous():
            raise ValueError("rays_host must be a contiguous float32 CPU tensor [N, 6]")
        n, s = rays_host.shape[0], self._samples(N_samples)
        if rgb_out is None:
            rgb_out = torch.empty((n, 3), dtype=torch.float32).pin_memory()
        if depth_out is None:
            depth_out = torch.empty((n,), dtype=torch.float32).pin_memory()
        chunk = min(chunk, max(n, 1))
        max_valid, max_app = self.capacities(chunk, s)
        st = (C.c_int32 * _lib.ST_WORDS)()
        check(lib.gnr_render_host(self._handle, _ptr(rays_host), n, s, int(bool(white_bg)), chunk, max_valid, max_app,
                                  _ptr(rgb_out), _ptr(depth_out), st), "gnr_render_host")
        self.last_status = np.array(list(st), dtype=np.int64)
        self.raise_on_status(self.last_status)
        return rgb_out, depth_out


# The reference's class name, so that ``eval(args.model_name)(**kwargs)``-style construction
# (app/tools/render_utils.py:452-462) can be pointed at this module.
GridNeRF = B200GridNeRF
