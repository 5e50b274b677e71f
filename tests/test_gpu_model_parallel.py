"""GPU tests of the two model-parallel renderers.  All ranks of a group run inside this one
process in lock step (LoopbackComm), with the real kernels, against the CPU oracles."""
import numpy as np
import pytest
import torch

from landmark_b200 import scenes
from oracle import gridnerf_oracle as orc
from oracle import model_parallel_oracle as mpo
from tests._util import cuda_model, oracle_field, tiny_rays

pytestmark = pytest.mark.gpu
RGB_TOL, FLIP_RGB_TOL = 1e-4, 2.5e-3


def _check(rgb, depth, ref, max_flips=3):
    err = (rgb.cpu() - ref["rgb_map"]).abs().max(dim=1).values
    assert (err > RGB_TOL).sum().item() <= max_flips, f"{int((err > RGB_TOL).sum())} rays above 1e-4 (max {err.max():.2e})"
    assert err.max().item() <= FLIP_RGB_TOL
    assert (depth.cpu() - ref["depth_map"]).abs().max().item() <= 2e-4


@pytest.mark.parametrize("world,mlp_mode", [(2, 0), (3, 2), (1, 2), (1, "fp16"), (2, "fp16"), (3, "fp16")])
def test_channel_parallel_matches_unsplit_oracle(world, mlp_mode):
    """``"fp16"``: fp16 appearance planes + mlp_mode 2 on every rank, which selects the tensor-core form of the
    exchange (slices of 48, 24 and 16 channels: three, two and one round of 16 per pair)."""
    from landmark_b200.model_parallel import ChannelParallelRenderer, LoopbackComm, slice_checkpoint_channels

    extra = {}
    if mlp_mode == "fp16":
        mlp_mode, extra = 2, {"app_plane_fp16": True, "ert_transmittance": 0.0}

    spec = scenes.tiny_spec(grid=64).lit()
    field, ckpt = oracle_field(spec)
    rays = tiny_rays(spec)[3000:7000].contiguous()
    ref = orc.render_chunk(field, rays, spec.n_samples, True)
    models = []
    for r in range(world):
        sl = slice_checkpoint_channels(ckpt, r, world)
        assert sl["state_dict"]["app_plane.0"].shape[1] == 48 // world
        sspec = scenes.tiny_spec(grid=64).lit()
        sspec.app_n_comp = (48 // world,) * 3
        models.append(cuda_model(sspec, sl, mlp_mode=mlp_mode, **extra))
    ren = ChannelParallelRenderer(models, LoopbackComm(world))
    assert ren._fp16_exchange() == bool(extra)
    outs = ren.render_chunk([rays.cuda()] * world, spec.n_samples, True)
    assert len(outs) == world
    for rgb, depth in outs:
        _check(rgb, depth, ref)
    for rgb, depth in outs[1:]:
        assert torch.equal(rgb, outs[0][0])  # every rank ends with the same image
    # the frame form (two chunks in flight with the fp16 exchange) gives the bits of chunk-by-chunk calls
    cuts = [0, 1500, 2600, rays.shape[0]]
    chunk_list = [[rays[lo:hi].cuda()] * world for lo, hi in zip(cuts[:-1], cuts[1:])]
    want = [ren.render_chunk(c, spec.n_samples, True) for c in chunk_list]
    res = ren.render_frame(chunk_list, spec.n_samples, True, lanes=2)
    torch.cuda.synchronize()
    for w_c, r_c in zip(want, res):
        for (a, b), (c, d) in zip(w_c, r_c):
            assert torch.equal(a, c) and torch.equal(b, d)


def _block_scene(division, grid=32, seed0=100):
    """Global box split in x-y; every block has its own seeded field of ``grid``^3."""
    px, py = division
    gspec = scenes.tiny_spec(grid=grid).lit()
    gspec.name = "blocks_global"
    gspec.aabb = ((-1.0 * px, -1.0 * py, -1.0), (1.0 * px, 1.0 * py, 1.0))
    gspec.grid = (grid * px, grid * py, grid)
    gspec.mask_shape = (32, 32 * py, 32 * px)
    gspec.near_far = (0.1, 12.0)
    gspec.mask_boxes = 40 * px * py
    blocks = []
    for b in range(px * py):
        bs = scenes.tiny_spec(grid=grid).lit()
        blocks.append((bs, scenes.make_checkpoint(bs, seed=seed0 + b)))
    gck = scenes.make_checkpoint(gspec)
    return gspec, gck, blocks


@pytest.mark.parametrize("division,mlp_mode", [((2, 1), 0), ((2, 2), 2), ((2, 2), "bench"), ((4, 2), "bench")])
def test_block_parallel_matches_oracle(division, mlp_mode):
    from landmark_b200.gridnerf import B200GridNeRF
    from landmark_b200.model_parallel import BlockParallelRenderer, LoopbackComm

    world = division[0] * division[1]
    gspec, gck, blocks = _block_scene(division)
    gfield = orc.field_from_checkpoint(gck)
    bfields = [orc.field_from_checkpoint(ck) for _, ck in blocks]
    # camera above the middle of the scene looking down at an angle, so that rays cross block seams
    pose = scenes.pitched_pose((0.1, -0.2, 2.5), yaw_deg=20.0, pitch_deg=-65.0)
    rays = orc.generate_rays(torch.from_numpy(pose), 48, 64, 40.0)
    ref = mpo.render_chunk_blocks(gfield, bfields, division, rays, 160, True)
    # (the 4 x 2 scene is wider than the camera's view: six of its eight blocks hold samples, the other owners idle)
    assert len(torch.unique(ref["block"])) >= min(world, 6) and int(ref["app_mask"].sum()) > 2000
    # samplers: global box / step / mask, planes never read -> keep them 2x2
    samplers, owners = [], []
    for r in range(world):
        kw = dict(gck["kwargs"])
        kw.update({"device": "cuda:0", "args": scenes.model_args(gspec, "cuda:0"), "is_train": False})
        s = B200GridNeRF(**kw, mlp_mode=0, field_grid=(2, 2, 2))
        s.load({k: v for k, v in gck.items() if k != "state_dict"} | {"state_dict": {}})
        samplers.append(s)
        if mlp_mode == "bench":  # what the benchmark's owners run: density lattice, fused appearance kernel in point mode
            owners.append(cuda_model(blocks[r][0], blocks[r][1], mlp_mode=2, app_plane_fp16=True, density_lattice=True))
        else:
            owners.append(cuda_model(blocks[r][0], blocks[r][1], mlp_mode=mlp_mode))
    ren = BlockParallelRenderer(samplers, owners, LoopbackComm(world), division)
    # data parallel over rays: rank r renders rows r, r + world, ...
    parts = [torch.arange(r, rays.shape[0], world) for r in range(world)]
    outs = ren.render_chunk([rays[p].cuda() for p in parts], 160, True)
    rgb = torch.zeros((rays.shape[0], 3))
    depth = torch.zeros(rays.shape[0])
    for p, (c, d) in zip(parts, outs):
        rgb[p], depth[p] = c.cpu(), d.cpu()
    _check(rgb, depth, ref)
    # the frame form: three chunks per rank through the two-lane pipeline give the bits of chunk-by-chunk calls
    n_min = min(p.numel() for p in parts)
    cuts = [0, n_min // 4, (5 * n_min) // 8, 10 ** 9]  # three uneven, non-empty chunks per rank
    chunk_list = [[rays[p][lo:hi].cuda() for p in parts] for lo, hi in zip(cuts[:-1], cuts[1:])]
    for lanes in (1, 2):
        res = ren.render_frame(chunk_list, 160, True, lanes=lanes)
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(torch.cat([res[c][r][0] for c in range(3)]), outs[r][0]), (lanes, r)
            assert torch.equal(torch.cat([res[c][r][1] for c in range(3)]), outs[r][1]), (lanes, r)
    assert ren.samples["valid"] > 0 and ren.samples["app"] > 2000
    if mlp_mode == "bench":
        # ids on the wire (owners recompute the positions from the gathered rays) against points on the wire: same bits
        assert ren.ship_ids
        ren.ship_ids = False
        pts = ren.render_chunk([rays[p].cuda() for p in parts], 160, True)
        for (a, b), (c, d) in zip(outs, pts):
            assert torch.equal(a, c) and torch.equal(b, d)
    else:
        assert not ren.ship_ids


def test_assign_blocks_matches_oracle_restatement():
    from landmark_b200.model_parallel import assign_blocks

    g = torch.Generator().manual_seed(3)
    xyz = torch.rand((5000, 3), generator=g) * 2 - 1
    xyz[0] = torch.tensor([1.0, 1.0, 0.0])   # upper faces
    xyz[1] = torch.tensor([-1.0, -1.0, 0.0])
    xyz[2] = torch.tensor([0.0, 0.0, 0.5])   # exactly on a seam
    for division in ((4, 2), (2, 1), (3, 3)):
        b0, l0 = mpo.assign_blocks(xyz, division)
        b1, l1 = assign_blocks(xyz.cuda(), division)
        assert torch.equal(b0, b1.cpu()) and torch.equal(l0, l1.cpu())
        assert int(b0.max()) == division[0] * division[1] - 1 and int(b0.min()) == 0


def test_assign_blocks_matches_the_reference_fixture():
    """Block ids and block-local coordinates the reference's own assign_blocks_to_samples produced
    (tests/golden/assign_blocks.npz, written by make_golden.py), against the device arithmetic."""
    from landmark_b200.model_parallel import assign_blocks
    from tests._util import load_golden

    fx = load_golden("assign_blocks.npz")
    xyz = torch.from_numpy(fx["xyz"]).cuda()
    for division in ((2, 1), (2, 2), (4, 2), (3, 5)):
        tag = f"{division[0]}x{division[1]}"
        b, local = assign_blocks(xyz, division)
        assert np.array_equal(b.cpu().numpy(), fx[f"block_{tag}"].astype(np.int64)), tag
        assert np.array_equal(local.cpu().numpy(), fx[f"local_{tag}"]), tag


@pytest.mark.parametrize("division", [(2, 1), (2, 2), (4, 2), (3, 5)])
def test_route_blocks_kernel_equals_torch_assignment_and_stable_grouping(division):
    """gnr_route_blocks (block assignment + grouping by owner in one pass on the device) against the torch
    arithmetic (pinned to the reference's method by the fixture test above) followed by a stable per-owner
    grouping: same rows in the same order, same counts, for the valid list and for the appearance list."""
    from landmark_b200.model_parallel import _Chunk, _route, assign_blocks

    spec = scenes.tiny_spec().lit()
    model = cuda_model(spec)
    rays = tiny_rays(spec).cuda()[2000:6000].contiguous()
    ch = _Chunk(model, rays, spec.n_samples)
    ch.sample()
    xyz, ray = ch.positions()
    b, loc = assign_blocks(xyz, division)
    order, cnt = _route(b, division[0] * division[1])
    send, dest, counts = ch.route(0, division)
    assert counts == cnt and sum(counts) == ch.num_valid > 50000
    assert torch.equal(send, loc[order])
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    assert torch.equal(dest.to(torch.int64), inv)
    # appearance list: rows carry the view direction as well
    ch.density()
    ch.weights()
    ids = ch.ids[: ch.num_valid].to(torch.int64) & 0xFFFFFFFF
    ai = ch.app_index
    b_a, loc_a = b[ai], loc[ai]
    view = rays[ids[ai] >> ch.kbits, 3:6]
    order_a, cnt_a = _route(b_a, division[0] * division[1])
    send_a, dest_a, counts_a = ch.route(1, division)
    assert counts_a == cnt_a and sum(counts_a) == ch.num_app > 10000
    assert torch.equal(send_a, torch.cat([loc_a, view], dim=1)[order_a])
    inv_a = torch.empty_like(order_a)
    inv_a[order_a] = torch.arange(order_a.numel(), device=order_a.device)
    assert torch.equal(dest_a.to(torch.int64), inv_a)


def test_point_mode_entries_match_list_mode():
    """gnr_density_points / gnr_appearance_points on explicit coordinates give what the list-mode
    stages give for the same samples."""
    from landmark_b200.model_parallel import _Chunk, appearance_points, density_points

    spec = scenes.tiny_spec(grid=64).lit()
    for mode in (0, 2):
        model = cuda_model(spec, mlp_mode=mode)
        rays = tiny_rays(spec)[4000:6000].cuda()
        got = model.run_stages(rays, spec.n_samples, True)
        ch = _Chunk(model, rays, spec.n_samples)
        ch.sample()
        xyz, ray = ch.positions()
        assert torch.equal(ray, got["ray_index"])
        sig = density_points(model, xyz)
        assert torch.equal(sig, got["sigma"])
        ai = got["app_index"]
        rgb = appearance_points(model, xyz[ai], rays[ray[ai], 3:6])
        assert torch.equal(rgb, got["rgb_samples"])
    # fp16 appearance planes: point mode runs the one-kernel form (gather + basis + MLP), list-mode stages the
    # separate kernels; same products and GEMMs, another K order in layer 1 (a last-bit difference of a
    # pre-activation can flip the fp16 rounding of a hidden unit, which moves a colour by a few 1e-6)
    model = cuda_model(spec, mlp_mode=2, app_plane_fp16=True)
    got = model.run_stages(rays, spec.n_samples, True)
    ai = got["app_index"]
    rgb = appearance_points(model, xyz[ai], rays[ray[ai], 3:6])
    assert (rgb - got["rgb_samples"]).abs().max().item() <= 5e-5
    assert (rgb - got["rgb_samples"]).abs().mean().item() <= 2e-6


def test_block_renderer_from_merged_stack_checkpoint():
    """Blocks split out of a merged-stack checkpoint (the reference's single-file export of a
    branch-parallel model) render exactly what the per-block checkpoints render."""
    from landmark_b200 import checkpoints
    from landmark_b200.gridnerf import B200GridNeRF
    from landmark_b200.model_parallel import BlockParallelRenderer, LoopbackComm

    division = (2, 1)
    gspec, gck, blocks = _block_scene(division)
    # the trainer keeps basis_mat and the MLP identical across blocks; the merged file holds block 0's
    shared = {k: v for k, v in blocks[0][1]["state_dict"].items()
              if not any(n in k for n in checkpoints.PLANE_NAMES + checkpoints.LINE_NAMES)}
    for _, ck in blocks[1:]:
        ck["state_dict"].update(shared)
    merged = checkpoints.merge_stack([ck for _, ck in blocks])
    merged.update({k: gck[k] for k in checkpoints.MASK_KEYS})
    parts = checkpoints.split_merged_stack(merged)
    pose = scenes.pitched_pose((0.1, -0.2, 2.5), yaw_deg=20.0, pitch_deg=-65.0)
    rays = orc.generate_rays(torch.from_numpy(pose), 32, 48, 30.0).cuda()

    def renderer(block_ckpts):
        samplers, owners = [], []
        for r in range(2):
            kw = dict(gck["kwargs"])
            kw.update({"device": "cuda:0", "args": scenes.model_args(gspec, "cuda:0"), "is_train": False})
            s = B200GridNeRF(**kw, mlp_mode=0, field_grid=(2, 2, 2))
            s.load({k: v for k, v in gck.items() if k != "state_dict"} | {"state_dict": {}})
            samplers.append(s)
            owners.append(cuda_model(blocks[r][0], block_ckpts[r], mlp_mode=2))
        return BlockParallelRenderer(samplers, owners, LoopbackComm(2), division)

    halves = [rays[0::2].contiguous(), rays[1::2].contiguous()]
    a = renderer([ck for _, ck in blocks]).render_chunk(halves, 160, True)
    b = renderer(parts).render_chunk(halves, 160, True)
    for (rgb_a, dep_a), (rgb_b, dep_b) in zip(a, b):
        assert torch.equal(rgb_a, rgb_b) and torch.equal(dep_a, dep_b)
    assert float(a[0][0].std()) > 0.05


def test_dynamic_block_window_follows_the_camera():
    """Blocks wait in pinned host memory; a 3x3 window around the camera is resident.  While the
    camera stays inside the window's reach the windowed render equals the render with every block
    resident, bit for bit; a move into another block starts an asynchronous load into spare slots,
    frames keep coming from the old window, and after the switch the pictures agree again."""
    from landmark_b200.dynamic import DynamicBlockRenderer, LoadStatus, pin_block, window_blocks
    from landmark_b200.gridnerf import B200GridNeRF

    division = (4, 2)
    gspec, gck, blocks = _block_scene(division, grid=16)
    kw = dict(gck["kwargs"])
    kw.update({"device": "cuda:0", "args": scenes.model_args(gspec, "cuda:0"), "is_train": False})
    sampler = B200GridNeRF(**kw, mlp_mode=0, field_grid=(2, 2, 2))
    sampler.load({k: v for k, v in gck.items() if k != "state_dict"} | {"state_dict": {}})
    host = [pin_block(ck) for _, ck in blocks]
    assert all(t.is_pinned() for t in host[0].values())

    def factory(b):
        return cuda_model(blocks[b][0], blocks[b][1], mlp_mode=2)

    # basis_mat and the MLP are per model here; give every block the same ones, as a trained scene has
    shared = {k: v for k, v in blocks[0][1]["state_dict"].items() if "plane" not in k and "line" not in k}
    for _, ck in blocks[1:]:
        ck["state_dict"].update(shared)

    def frame_rays(x, y):
        pose = scenes.pitched_pose((x, y, 1.6), yaw_deg=10.0, pitch_deg=-88.0)  # looking almost straight down
        return orc.generate_rays(torch.from_numpy(pose), 40, 40, 60.0).cuda()

    everything = DynamicBlockRenderer(sampler, host, division, factory, radius=4).start((-3.0, -1.0, 1.6))
    assert sorted(everything.block_to_slot) == list(range(8))
    windowed = DynamicBlockRenderer(sampler, host, division, factory, radius=1).start((-3.0, -1.0, 1.6))
    assert sorted(windowed.block_to_slot) == window_blocks(0, division, 1) == [0, 1, 2, 3]
    assert windowed.n_slots == 8 and windowed.loads == 0

    rays = frame_rays(-3.0, -1.0)
    a, da = everything.render_rays(rays, 160, True, chunk=700)
    b, db = windowed.render_rays(rays, 160, True, chunk=700)
    assert torch.equal(a, b) and torch.equal(da, db) and float(a.std()) > 0.002
    assert windowed.update((-3.2, -0.8, 1.6)) is LoadStatus.IDLE  # same block: nothing to do

    # the camera flies to block 5 (x in [0, 2), y in [0, 2)): its window is blocks 2..7
    assert windowed.update((1.0, 1.0, 1.6)) is LoadStatus.LOADING
    assert sorted(windowed.block_to_slot) == [0, 1, 2, 3]  # frames still see the old window
    b_old, _ = windowed.render_rays(rays, 160, True, chunk=700)
    assert torch.equal(b_old, b)
    windowed.wait_loaded()
    assert windowed.update((1.0, 1.0, 1.6)) is LoadStatus.IDLE
    assert sorted(windowed.block_to_slot) == window_blocks(5, division, 1) == [2, 3, 4, 5, 6, 7]
    # blocks 4..7 had been parked in the spare slots at start-up, so nothing came from the host yet
    rays2 = frame_rays(1.0, 1.0)
    a2, da2 = everything.render_rays(rays2, 160, True, chunk=700)
    b2, db2 = windowed.render_rays(rays2, 160, True, chunk=700)
    assert torch.equal(a2, b2) and torch.equal(da2, db2)
    assert not torch.equal(a2, a)

    # a one-block window with three slots: the block under the camera really comes from the host
    small = DynamicBlockRenderer(sampler, host, division, factory, radius=0, n_slots=3).start((1.0, 1.0, 1.6))
    assert sorted(small.block_to_slot) == [5] and small.slot_block == [5, 0, 1] and small.loads == 0
    assert small.update((-1.0, 1.0, 1.6)) is LoadStatus.LOADING  # block 3
    assert sorted(small.block_to_slot) == [5]
    small.wait_loaded()
    assert small.update((-1.0, 1.0, 1.6)) is LoadStatus.IDLE
    assert sorted(small.block_to_slot) == [3] and small.loads == 1
    rays3 = frame_rays(-1.0, 1.0)  # straight down on the middle of block 3: no ray leaves the block
    c, dc = small.render_rays(rays3, 160, True, chunk=700)
    a3, da3 = everything.render_rays(rays3, 160, True, chunk=700)
    assert torch.equal(c, a3) and torch.equal(dc, da3)
    # an oblique view through the one-block window lacks the other blocks
    far = scenes.pitched_pose((-3.0, -1.0, 2.5), yaw_deg=0.0, pitch_deg=-30.0)
    rays4 = orc.generate_rays(torch.from_numpy(far), 32, 48, 30.0).cuda()
    full4, _ = everything.render_rays(rays4, 200, True)
    part4, _ = small.render_rays(rays4, 200, True)
    assert not torch.equal(full4, part4)


def test_slice_projection_bounded_wait_expires_and_the_context_survives():
    """The slice-projection kernel bounds its waits like the other tensor-core kernels: with the test hook one group
    skips the commit its wait depends on, the status word reports the expired wait, the kernel frees its tensor
    memory and returns, and the same call then gives the same rows as before."""
    from landmark_b200._lib import check, lib
    from landmark_b200.gridnerf import _ptr, _stream

    spec = scenes.tiny_spec(grid=64).lit()
    model = cuda_model(spec, mlp_mode=2, app_plane_fp16=True)
    g = torch.Generator().manual_seed(3)
    xyz = (torch.rand((5000, 3), generator=g) * 1.8 - 0.9).cuda()

    def project():
        out = torch.zeros((xyz.shape[0], 32), dtype=torch.float16, device="cuda:0")
        st = torch.zeros(8, dtype=torch.int32, device="cuda:0")
        check(lib.gnr_project_slice_points(model._handle, _ptr(xyz), 3, xyz.shape[0], _ptr(out), _ptr(st), _stream()),
              "gnr_project_slice_points")
        torch.cuda.synchronize()
        return out, st.cpu().tolist()

    good, st = project()
    assert st[4] == 0 and good.abs().max().item() > 0
    model.debug_wait(expire=True, wait_limit=2000)
    _, st = project()
    assert st[4] == 1  # GNR_ST_WAIT_EXPIRED
    model.debug_wait()
    again, st = project()
    assert st[4] == 0 and torch.equal(again, good)


def test_partial_rows_summed_inside_the_mlp_kernel_equal_sum_then_mlp():
    """gnr_mlp_partial_rows (the W fp16 partial rows of a sample summed in fp32 inside the one-kernel appearance path)
    against gnr_sum_partials followed by gnr_mlp_features on the same rows: the same additions in the same order and the
    same network, so the colours agree bit for bit."""
    from landmark_b200._lib import check, lib
    from landmark_b200.gridnerf import _ptr, _stream
    from landmark_b200.model_parallel import _scratch, mlp_features

    spec = scenes.tiny_spec(grid=64).lit()
    model = cuda_model(spec, mlp_mode=2, app_plane_fp16=True)
    n, W, per = 3001, 3, 3200
    g = torch.Generator().manual_seed(5)
    parts = (torch.randn((W * per, 32), generator=g) * 0.3).to(torch.float16).cuda()
    parts[:, 27:] = 0
    rows6 = torch.randn((n, 6), generator=g).cuda()
    rows6[:, 3:6] = torch.nn.functional.normalize(rows6[:, 3:6], dim=1)
    feats = torch.empty((n, model.app_dim), dtype=torch.float32, device="cuda:0")
    check(lib.gnr_sum_partials(model._handle, _ptr(parts), W, n, per, _ptr(feats), _stream()), "gnr_sum_partials")
    want_f = parts.view(W, per, 32)[:, :n, :27].float().sum(0)
    assert torch.allclose(feats, want_f, atol=1e-6)
    want = mlp_features(model, feats, rows6[:, 3:6].contiguous())
    got = torch.empty((n, 3), dtype=torch.float32, device="cuda:0")
    keep, sc, nbytes = _scratch(model, n)
    check(lib.gnr_mlp_partial_rows(model._handle, _ptr(parts), W, per, _ptr(rows6), n, sc, nbytes, _ptr(got), _stream()),
          "gnr_mlp_partial_rows")
    torch.cuda.synchronize()
    assert torch.equal(got, want)
