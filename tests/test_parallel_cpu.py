"""CPU tests of the multi-GPU host logic: tile ownership, and the gather/assemble step run
with two real ranks over gloo."""
import os
import socket

import numpy as np
import pytest
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
    first = tile_pixel_ids(70, 130, 0, 4, patch=None)
    assert list(first[:3]) == [0, 1, 2] and first[64] == 130  # plain row-major inside a tile
    first = tile_pixel_ids(70, 130, 0, 4)  # default: 8 x 4 patches, one warp's rays each
    assert list(first[:9]) == [0, 1, 2, 3, 4, 5, 6, 7, 130] and first[32] == 8 and first[8 * 32] == 4 * 130


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


class _FakeRenderer:
    """CPU stand-in for FrameRenderer: colour = f(pose, pixel), rgba by torch ops."""

    device = "cpu"

    def render_pixels(self, pose, H, W, focal, pixel_ids, rgb_out):
        pid = pixel_ids.to(torch.float32)
        base = float(np.asarray(pose).sum()) + focal
        rgb_out[:, 0] = (pid % 251) / 251.0
        rgb_out[:, 1] = ((pid * 7 + base) % 13) / 13.0
        rgb_out[:, 2] = 0.5

    def finish(self):
        pass

    def to_rgba8(self, image, out):
        out[:, :3] = (image * 255).clamp(0, 255).to(torch.uint8)
        out[:, 3] = 255


def _expected(pose, focal, H, W):
    pid = torch.arange(H * W, dtype=torch.float32)
    base = float(np.asarray(pose, dtype=np.float32)[:3, :4].sum()) + focal
    img = torch.stack([(pid % 251) / 251.0, ((pid * 7 + base) % 13) / 13.0, torch.full_like(pid, 0.5)], 1)
    out = torch.full((H * W, 4), 255, dtype=torch.uint8)
    out[:, :3] = (img * 255).clamp(0, 255).to(torch.uint8)
    return out.view(H, W, 4).numpy()


def _engine_worker(rank, world, port, H, W, out):
    from landmark_b200.engine import MainRankDDPRenderEngine, NerfDDPRunner, OtherRankRenderEngine

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        factory = lambda: NerfDDPRunner(_FakeRenderer(), H, W, focal=100.0, rank=rank, world=world)  # noqa: E731
        poses = [np.eye(4, dtype=np.float32)[:3] * (k + 1) for k in range(3)]
        if rank == 0:
            eng = MainRankDDPRenderEngine(factory, poses=poses)
            eng.start()
            imgs = [eng.submit(p) for p in poses]
            eng.stop()
            torch.save(imgs, out)
        else:
            eng = OtherRankRenderEngine(factory)
            eng.start()
            assert eng.frames == 3
    finally:
        dist.destroy_process_group()


def test_engine_protocol_two_ranks_over_gloo(tmp_path):
    """Main-rank engine submits three poses; the other rank sits in its serve loop, renders its
    tiles for each broadcast pose and is released by the stop message."""
    H, W = 40, 72
    out = str(tmp_path / "imgs.pt")
    mp.spawn(_engine_worker, args=(2, _free_port(), H, W, out), nprocs=2, join=True)
    imgs = torch.load(out, weights_only=False)
    for k, img in enumerate(imgs):
        pose = np.eye(4, dtype=np.float32)[:3] * (k + 1)
        assert img.shape == (H, W, 4) and img.dtype == np.uint8
        assert np.array_equal(img, _expected(pose, 100.0, H, W))


def test_engine_single_rank_cpu_fake():
    from landmark_b200.engine import MainRankDDPRenderEngine, NerfDDPRunner

    eng = MainRankDDPRenderEngine(lambda: NerfDDPRunner(_FakeRenderer(), 30, 50, focal=None),
                                  poses=[np.concatenate([np.eye(3), np.zeros((3, 1)), np.full((3, 1), 80.0)], 1)])
    eng.start(test=True)
    assert len(eng.latency) == 1
    img = eng.submit(eng.poses[0])
    assert np.array_equal(img, _expected(eng.poses[0], 80.0, 30, 50))


def _rank_rows(rank, world):
    """Deterministic per-rank payload and owners for the routing test."""
    g = torch.Generator().manual_seed(100 + rank)
    n = 1000 + 37 * rank
    owner = torch.randint(0, world, (n,), generator=g)
    owner[:50] = 0  # an uneven split
    x = torch.randn((n, 4), generator=g)
    return owner, x


def _route_worker(rank, world, port, out):
    from landmark_b200.model_parallel import DistComm, _route

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        comm = DistComm()
        owner, x = _rank_rows(rank, world)
        order, counts = _route(owner, world)
        got, rc = comm.all_to_all_rows([x[order]], [counts])
        # the reply travels the reverse way and is put back in sample order
        back, _ = comm.all_to_all_rows([got[0] * 2], [rc[0]])
        restored = torch.empty_like(x)
        restored[order] = back[0]
        gathered = comm.all_gather_rows([x[:8]])
        # the channel-parallel renderer's exchange: partial feature rows summed and dealt out by rows
        part = comm.reduce_scatter_rows([x[:64]])
        # the pipelined block renderer's form: device-side counts gathered into one [source, destination] matrix,
        # exchanges into caller-held buffers of list capacity, return trip with the transposed matrix
        matrix = comm.gather_counts([torch.tensor(counts, dtype=torch.int32)])
        known = comm.all_to_all_known([x[order]], matrix, [torch.zeros((4000, 4))])
        known_back = comm.all_to_all_known([known[0] * 2], matrix.T, [torch.zeros((4000, 4))])
        restored2 = torch.empty_like(x)
        restored2[order] = known_back[0]
        torch.save({"recv": got[0], "rc": rc[0], "restored": restored, "gathered": gathered[0], "part": part[0],
                    "matrix": torch.from_numpy(matrix.copy()), "known": known[0].clone(), "restored2": restored2},
                   f"{out}.{rank}")
    finally:
        dist.destroy_process_group()


def test_sample_routing_two_ranks_over_gloo_equals_loopback(tmp_path):
    """The block-parallel renderer's exchange (group samples by owner, counts first, variable
    all-to-all, reverse trip) through torch.distributed on two gloo ranks gives what the
    in-process LoopbackComm, which the GPU tests use, gives for the same rows."""
    from landmark_b200.model_parallel import LoopbackComm, _route

    world = 2
    out = str(tmp_path / "route")
    mp.spawn(_route_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    rows = [_rank_rows(r, world) for r in range(world)]
    routed = [_route(o, world) for o, _ in rows]
    lb = LoopbackComm(world)
    recv, rcs = lb.all_to_all_rows([rows[r][1][routed[r][0]] for r in range(world)], [routed[r][1] for r in range(world)])
    gathered = lb.all_gather_rows([rows[r][1][:8] for r in range(world)])
    parts = lb.reduce_scatter_rows([rows[r][1][:64] for r in range(world)])
    matrix = lb.gather_counts([torch.tensor(routed[r][1], dtype=torch.int32) for r in range(world)])
    known = lb.all_to_all_known([rows[r][1][routed[r][0]] for r in range(world)], matrix,
                                [torch.zeros((4000, 4)) for _ in range(world)])
    for r in range(world):
        got = torch.load(f"{out}.{r}")
        assert np.array_equal(got["matrix"].numpy(), matrix) and matrix[r].tolist() == routed[r][1]
        assert torch.equal(got["known"], known[r]) and torch.equal(known[r], recv[r])
        assert torch.equal(got["restored2"], rows[r][1] * 2)
        assert torch.equal(got["part"], parts[r])
        assert got["rc"] == rcs[r]
        assert torch.equal(got["recv"], recv[r])
        assert torch.equal(got["restored"], rows[r][1] * 2)
        assert torch.equal(got["gathered"], gathered[r])
        # stable grouping: inside one owner the samples keep their order
        order, counts = routed[r]
        assert sum(counts) == rows[r][0].numel()
        start = 0
        for d in range(world):
            seg = order[start:start + counts[d]]
            assert torch.all(rows[r][0][seg] == d) and torch.all(seg[1:] > seg[:-1])
            start += counts[d]


def test_pipe_engine_submit_get_result_wait_stop_cpu():
    """The asynchronous engine interface (submit -> uid, get_result in submission order, wait(uid) in any
    order, more frames submitted than slots, stop) with a CPU frame backend, and through NerfDDPRunner's
    enqueue with the fake renderer."""
    from queue import Empty

    from landmark_b200.engine import NerfDDPRunner
    from landmark_b200.pipe_engine import CpuFrameBackend, MainRankPipeRenderEngine, PipeRunner, RunnerFrameBackend

    H, W = 24, 40
    poses = [np.eye(4, dtype=np.float32)[:3] * (k + 1) for k in range(7)]
    frame = lambda pose: _expected(pose, 100.0, H, W)  # noqa: E731

    eng = MainRankPipeRenderEngine(lambda: PipeRunner(CpuFrameBackend(frame, H, W), depth=2), poses=poses, async_=True)
    eng.start()
    uids = [eng.submit(p) for p in poses]          # 7 frames through 2 slots
    assert len(set(uids)) == 7
    for k in (3, 0, 6):                            # by uid, any order
        assert np.array_equal(eng.wait(uids[k]), frame(poses[k]))
    assert np.array_equal(eng.get_result(), frame(poses[1]))   # the rest in submission order
    assert np.array_equal(eng.get_result(), frame(poses[2]))
    with pytest.raises(KeyError):
        eng.wait(uids[3])                          # handed out already
    assert np.array_equal(eng.get_result(), frame(poses[4])) and np.array_equal(eng.get_result(), frame(poses[5]))
    with pytest.raises(Empty):
        eng.runner.get_result_task(block=False)
    eng.run_for_latency()
    eng.run_for_throughput()
    assert len(eng.latency) == 7 and eng.throughput > 0
    eng.stop()
    with pytest.raises(RuntimeError):
        eng.submit(poses[0])

    # the same interface over the tile-sharded runner (single rank, fake renderer)
    eng2 = MainRankPipeRenderEngine(
        lambda: PipeRunner(RunnerFrameBackend(NerfDDPRunner(_FakeRenderer(), H, W, focal=100.0)), depth=3), poses=poses[:3])
    eng2.start(test=True)  # warm-up, latency run, stop
    assert len(eng2.latency) == 3
