"""CPU tests of the multi-block checkpoint ingest against what the reference's merge_ckpts wrote
(tests/golden/merged_stack_tiny.npz, produced by tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from landmark_b200 import checkpoints, scenes
from tests._util import load_golden


def _blocks(n=2, grid=8):
    spec = scenes.tiny_spec(grid=grid).lit()
    return [scenes.make_checkpoint(spec, seed=500 + b) for b in range(n)]


def test_merge_stack_equals_reference_merge_ckpts():
    fx = load_golden("merged_stack_tiny.npz")
    blocks = _blocks(int(fx["n_blocks"]))
    merged = checkpoints.merge_stack(blocks)
    assert list(merged["kwargs"]["gridSize"]) == fx["grid_size"].tolist()
    keys = [k[3:] for k in fx if k.startswith("sd.")]
    assert len(keys) == 12  # 3 pairs x (density, appearance) x (plane, line)
    for k in keys:
        assert np.array_equal(merged["state_dict"][k].numpy(), fx["sd." + k]), k
    assert merged["state_dict"]["density_plane.0"].shape == (1, 16, 2, 8, 8)
    assert merged["state_dict"]["app_line.2"].shape == (1, 48, 8, 2)
    assert checkpoints.is_merged_stack(merged) and not checkpoints.is_merged_stack(blocks[0])
    assert checkpoints.n_blocks_of(merged) == 2


def test_split_restores_every_block():
    blocks = _blocks(3)
    merged = checkpoints.merge_stack(blocks)
    parts = checkpoints.split_merged_stack(merged)
    assert len(parts) == 3
    for b, part in enumerate(parts):
        for k, v in blocks[b]["state_dict"].items():
            if any(n in k for n in checkpoints.PLANE_NAMES + checkpoints.LINE_NAMES):
                assert torch.equal(part["state_dict"][k], v), (b, k)
            else:  # basis_mat and the MLP are block 0's, as in the reference's merged file
                assert torch.equal(part["state_dict"][k], blocks[0]["state_dict"][k]), (b, k)
        assert "device" not in part["kwargs"] and "args" not in part["kwargs"]
    sampler = checkpoints.sampler_checkpoint(merged)
    assert sampler["state_dict"] == {} and "alphaMask.mask" in sampler


def test_sidecar_without_planes():
    blocks = _blocks(2)
    merged = checkpoints.merge_stack(blocks)
    sidecar = checkpoints.without_planes(merged)
    assert not any("plane" in k for k in sidecar["state_dict"])
    with pytest.raises(ValueError, match="planes"):
        checkpoints.split_merged_stack(sidecar)
    planes = {k: v for k, v in merged["state_dict"].items() if "plane" in k}
    parts = checkpoints.split_merged_stack(sidecar, planes)
    assert torch.equal(parts[1]["state_dict"]["app_plane.1"], blocks[1]["state_dict"]["app_plane.1"])
    bad = dict(merged)
    bad["state_dict"] = dict(merged["state_dict"])
    bad["state_dict"]["density_line.0"] = bad["state_dict"]["density_line.0"][..., :1]
    with pytest.raises(ValueError, match="stacked line"):
        checkpoints.split_merged_stack(bad)


def test_dynamic_window_blocks():
    from landmark_b200.dynamic import window_blocks

    assert window_blocks(0, (4, 2), 1) == [0, 1, 2, 3]
    assert window_blocks(5, (4, 2), 1) == [2, 3, 4, 5, 6, 7]
    assert window_blocks(5, (4, 2), 0) == [5]
    assert window_blocks(12, (5, 5), 1) == [6, 7, 8, 11, 12, 13, 16, 17, 18]
    assert window_blocks(3, (4, 2), 9) == list(range(8))
