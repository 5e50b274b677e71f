"""CPU tests of the multi-GPU host logic: tile ownership, and the gather/assemble step run
with two real ranks over gloo."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from landmark_b200.parallel import TileSharding, split_contiguous, tile_pixel_ids


def test_tiles_partition_the_frame():
    H, W = 1080, 1920
    for world in (1, 2, 3, 8):
        parts = [tile_pixel_ids(H, W, r, world) for r in range(world)]
        allp = np.concatenate(parts)
        assert allp.shape[0] == H * W and np.array_equal(np.sort(allp), np.arange(H * W))
        sizes = [p.shape[0] for p in parts]
        assert max(sizes) - min(sizes) <= 64 * 64 * 2  # round-robin keeps ranks within two tiles of each other
    # a ragged image: tiles clipped at both borders
    parts = [tile_pixel_ids(70, 130, r, 4) for r in range(4)]
    assert np.array_equal(np.sort(np.concatenate(parts)), np.arange(70 * 130))
    first = tile_pixel_ids(70, 130, 0, 4)
    assert list(first[:3]) == [0, 1, 2] and first[64] == 130  # row-major inside a tile


def test_reference_contiguous_split():
    assert split_contiguous(2073600, 8) == (259200, 0)
    assert split_contiguous(10, 4) == (3, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, H, W, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = TileSharding(H, W, rank, world, "cpu", tile=16)
        # a fake renderer: colour is a function of the pixel id
        pid = sh.pixel_ids.to(torch.float32)
        rgb = torch.zeros((sh.n_pad, 3))
        rgb[: sh.n_local] = torch.stack([pid, pid * 2, pid + 0.5], 1)
        image = torch.zeros((H * W, 3))
        sh.assemble(rgb, image)
        if rank == 0:
            torch.save(image, out)
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_over_gloo(tmp_path):
    H, W = 50, 70  # not multiples of the tile, unequal per-rank counts -> padding path
    out = str(tmp_path / "image.pt")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, H, W, out), nprocs=2, join=True)
    image = torch.load(out)
    pid = torch.arange(H * W, dtype=torch.float32)
    assert torch.equal(image, torch.stack([pid, pid * 2, pid + 0.5], 1))
