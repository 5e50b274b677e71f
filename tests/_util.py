"""Shared helpers of the test-suite (scene -> oracle field / CUDA model, fixture loading)."""
import os

import numpy as np
import torch

from landmark_b200 import scenes
from oracle import gridnerf_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name), allow_pickle=False))


def oracle_field(spec, ckpt=None):
    ckpt = ckpt or scenes.make_checkpoint(spec)
    return orc.field_from_checkpoint(ckpt, spec.alpha_filter_thres), ckpt


def cuda_model(spec, ckpt=None, mlp_mode=0, device="cuda:0", **extra):
    from landmark_b200.gridnerf import B200GridNeRF

    ckpt = ckpt or scenes.make_checkpoint(spec)
    kwargs = dict(ckpt["kwargs"])
    kwargs.update({"device": device, "args": scenes.model_args(spec, device), "is_train": False})
    model = B200GridNeRF(**kwargs, mlp_mode=mlp_mode, **extra)
    model.load(ckpt)
    return model


def tiny_rays(spec):
    pose = torch.from_numpy(scenes.make_pose(spec))
    return orc.generate_rays(pose, spec.height, spec.width, spec.focal)


def valid_bits_from_words(mask_words, n_samples):
    """[N, words] int32 little-endian bit words -> bool [N, S]."""
    w = mask_words.cpu().numpy().astype(np.uint32)
    bits = ((w[:, :, None] >> np.arange(32, dtype=np.uint32)[None, None, :]) & 1).astype(bool)
    return bits.reshape(w.shape[0], -1)[:, :n_samples]
