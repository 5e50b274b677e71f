#!/usr/bin/env python
"""Benchmark of the GridNeRF render path: Mrays/s and ms per 1080p frame.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One *step* renders one 1920x1080 frame of the city-block scene (AABB [-8,8]^2x[-1,1], grid
2048x2048x256, 16/48-channel VM planes, 512x512x64 occupancy heightfield, 512 samples per
ray, 150->128->128->3 MLP).  The fields are seeded synthetic tensors with the shapes and
value distribution of a reference checkpoint (no trained checkpoint is redistributable).
Two variants of the scene exist; the headline is ``city_lit`` (``density_shift = 0``), in which
the appearance gather and the MLP actually run; with the literal ``density_shift = -10`` every
weight stays below the appearance threshold and only sampling, density and compositing run
(``--workload city`` measures that).

With N > 1 (launched by torchrun, one rank per GPU) the frame is split into 64x64 pixel
tiles dealt round-robin to the ranks (replicated model), each rank renders its tiles and
the colours are all-gathered over NCCL; ``value`` is the whole frame's rays divided by the
slowest rank's device time (strong scaling).

``--impl reference`` times the reference's CPU torch path (the oracle port of it) on a
bounded sample of the same frame with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

DENSITY_BYTES_PER_SAMPLE = 784      # 3 planes x 4 corners x 16 ch x 4 B + 12 B coordinate + 4 B sigma
APP_BYTES_PER_SAMPLE = 2316         # 3 planes x 4 corners x 48 ch x 4 B + 12 B coordinate (fp16 storage: 1164)
# What actually bounds the two gathers: every tap of a sample is delivered from L1 into registers
# (the texels themselves are cache-resident, a frame oversamples the grid), and an SM's L1 hands
# 128 B per clock to its register files.
DENSITY_L1_BYTES_PER_SAMPLE = 18 * 16 * 4   # (4 plane + 2 line taps) x 3 pairs x 16 ch x 4 B
APP_L1_BYTES_PER_SAMPLE = 18 * 48 * 4       # halved by fp16 storage
# fp16 weight operands a 128-sample tile's GEMMs read from shared memory: basis 144x32, W1 160x128, W2 144x128, W3 128x16
FUSED_WEIGHT_OPERAND_BYTES_PER_TILE = 2 * (144 * 32 + 160 * 128 + 144 * 128 + 128 * 16)
L1_BYTES_PER_CLOCK_PER_SM = 128
MLP_FLOP_PER_SAMPLE = 71936         # 2 * (150*128 + 128*128 + 128*3)
BASIS_FLOP_PER_SAMPLE = 7776        # 2 * 144 * 27 (done inside the appearance gather kernel)
CPU_SAMPLE_RAYS = 65536
REFERENCE_BUDGET_S = 150.0  # the reference arm sizes its per-step sample so that K steps take about this long


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks/throttle reasons of one GPU, sampled every 200 ms in the background."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


FRAMES = {"1080p": (1080, 1920), "4k": (2160, 3840)}


def build_scene(workload, device, frame="1080p"):
    from landmark_b200 import scenes

    spec = scenes.city_spec(*FRAMES[frame])
    if workload == "city_lit":
        spec = spec.lit()
    vol = scenes.make_alpha_volume(spec)
    sd = scenes.make_state_dict(spec, device=device)  # CUDA generator: fast, seeded
    ckpt = {"kwargs": scenes.model_kwargs(spec), "state_dict": sd, "alphaMask.shape": tuple(vol.shape),
            "alphaMask.mask": np.packbits(vol.numpy().reshape(-1)),
            "alphaMask.aabb": torch.tensor(spec.aabb, dtype=torch.float32)}
    pose = scenes.make_pose(spec, vol)
    return spec, ckpt, pose


def run_reference(a):
    """CPU arm: the oracle port of the reference's torch path, all host threads, one bounded
    sample per step (at most CPU_SAMPLE_RAYS rays starting at image row 536 of the same frame, fewer
    when K steps of that size would take longer than REFERENCE_BUDGET_S)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from landmark_b200 import scenes
    from oracle import gridnerf_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    spec = scenes.city_spec()
    if a.workload == "city_lit":
        spec = spec.lit()
    vol = scenes.make_alpha_volume(spec)
    ckpt = scenes.make_checkpoint(spec)
    field = orc.field_from_checkpoint(ckpt)
    pose = torch.from_numpy(scenes.make_pose(spec, vol))
    rays = orc.generate_rays(pose, spec.height, spec.width, spec.focal)
    first = 536 * spec.width
    # one untimed pass over a small piece of the sample warms the threads up and gives the rate
    # that bounds the run: the K timed steps together stay near REFERENCE_BUDGET_S seconds
    probe = rays[first:first + 8192].contiguous()
    n_warm = max(a.warmup, 1)
    for _ in range(n_warm):
        t0 = time.perf_counter()
        orc.render_chunk(field, probe, spec.n_samples, True)
        rate = probe.shape[0] / (time.perf_counter() - t0)
    n_sample = int(min(CPU_SAMPLE_RAYS, max(8192, rate * REFERENCE_BUDGET_S / max(a.steps, 1))) // 4096 * 4096)
    sample = rays[first:first + n_sample].contiguous()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        orc.render_chunk(field, sample, spec.n_samples, True)
    dt = (time.perf_counter() - t0) / a.steps
    value = n_sample / dt / 1e6
    line = {
        "impl": "reference", "metric": "Mrays/s", "value": value, "unit": "Mrays/s", "n_gpus": a.gpus,
        "steps": a.steps, "warmup": n_warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{a.workload}: 1920x1080 frame, 512 samples/ray", "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": value, "unit": "Mrays/s", "cores": cores, "kind": "port",
                         "sample": f"{n_sample} rays (from image row 536 on) per step (warm-up passes: 8192 rays each), torch {torch.__version__} CPU"},
        "e2e": {"value": value, "unit": "Mrays/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "ms_per_frame_extrapolated": dt * 1e3 * spec.height * spec.width / n_sample,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="city_lit", choices=["city_lit", "city", "city_blocks", "city_channels"],
                    help="city_lit (headline) | city (density_shift=-10) | city_blocks (block-partitioned field, "
                         "all-to-all routing) | city_channels (channel-parallel appearance, reduce-scatter)")
    ap.add_argument("--grid-scale", type=int, default=1, help="divide grid and mask resolution (model-parallel workloads)")
    ap.add_argument("--check", action="store_true", help="city_blocks: compare rank 0 with a single-process render")
    ap.add_argument("--chunk", type=int, default=262144,
                    help="rays per library call (lowered so that every stream of a rank has a chunk)")
    ap.add_argument("--mlp-mode", type=int, default=2,
                    help="0 fp32 CUDA cores, 1 tcgen05 fp16 hi+lo activations, 2 tcgen05 fp16 (default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--frame", choices=sorted(FRAMES), default="1080p",
                    help="frame size (the focal length scales with the width); 4k is the tile-parallel configuration's frame")
    ap.add_argument("--reload-test", action="store_true",
                    help="time the refill of one resident block from pinned host memory (dynamic block window) and exit")
    ap.add_argument("--no-graph", action="store_true", help="skip the CUDA-graph replay measurement")
    ap.add_argument("--no-strict", action="store_true",
                    help="skip the second measurement with every approximation off (fp32 MLP, fp32 planes, no termination)")
    ap.add_argument("--app-fp16", type=int, default=1, choices=(0, 1),
                    help="hold the appearance planes as fp16 in HBM (mlp_mode 2 only)")
    ap.add_argument("--den-fp16", type=int, default=0, choices=(0, 1),
                    help="hold the density planes and lines as fp16 in HBM as well")
    ap.add_argument("--den-lattice", type=int, default=1, choices=(0, 1),
                    help="density from the pre-summed scalar lattice (4 B per grid point of HBM, 8 taps per sample) "
                         "instead of the 3 x (plane x line) x 16-channel gather")
    ap.add_argument("--app-fusion", type=int, default=1, choices=(0, 1),
                    help="appearance gather + basis projection + MLP as one kernel (needs --mlp-mode 2 --app-fp16 1)")
    ap.add_argument("--ert", type=float, default=2e-5,
                    help="early ray termination threshold of the density pass (rgb error bound); 0 = exact, "
                         "-1 = separate density and weights kernels")
    ap.add_argument("--no-model-parallel", action="store_true",
                    help="N > 1: skip the block-partitioned and channel-parallel renders of the same frame")
    ap.add_argument("--chunk-model-parallel", type=int, default=262144, help="rays per exchange of the model-parallel renderers")
    ap.add_argument("--no-variants", action="store_true", help="skip the extra configurations (literal scene, T < 1e-3, mlp_mode 1, ...)")
    ap.add_argument("--no-overlap", action="store_true", help="render the chunks of a frame on one stream only")
    ap.add_argument("--streams", type=int, default=2, help="streams the chunks of a frame rotate over")
    ap.add_argument("--frames-in-flight", type=int, default=2, choices=(1, 2),
                    help="2 (default): a frame's first chunks may start while the previous frame's last chunk, assembly and "
                         "tile gather still run (two output buffer sets; the throughput form of the reference's pipe engine; "
                         "about 0.1 ms per frame at any N: 19.51 against 19.64 ms on one GPU, 2.65 against 2.74 ms for one "
                         "rank's eighth of the frame); 1: every frame waits for the one before it.  `e2e` is always one "
                         "frame at a time")
    ap.add_argument("--order", default="tiles", choices=["tiles", "rows"], help="ray order at N=1")
    ap.add_argument("--profile-case", type=int, default=0, metavar="RAYS",
                    help="render one chunk of RAYS rays from the middle of the frame twice and exit "
                         "(a small, self-terminating case for ncu captures)")
    a = ap.parse_args()
    if a.impl == "reference":
        run_reference(a)
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the render path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = f"cuda:{local_rank}"
    import torch.distributed as dist

    if world > 1:
        # The model-parallel layouts move their samples with counted all-to-alls (point-to-point copies between
        # GPU pairs).  NCCL's default channel count gave 317 GB/s per direction between two B200s; 64 channels gave
        # 532 GB/s (456 MB per rank, measured).  Set before the communicator is made; an outer setting wins.
        for key in ("NCCL_MIN_P2P_NCHANNELS", "NCCL_MAX_P2P_NCHANNELS", "NCCL_MAX_NCHANNELS"):
            os.environ.setdefault(key, "64")
        dist.init_process_group("nccl", device_id=torch.device(device))
    if a.workload in ("city_blocks", "city_channels"):
        from landmark_b200.model_parallel_run import run as run_model_parallel

        sampler = ClockSampler(local_rank) if rank == 0 else None
        res = run_model_parallel(a.workload, a.steps, max(a.warmup, 3), a.chunk, a.mlp_mode, rank, world, device,
                                 a.grid_scale, a.check, ert=a.ert, app_fp16=bool(a.app_fp16), den_lattice=bool(a.den_lattice))
        clocks = sampler.stop() if sampler else None
        if rank == 0:
            line = {"metric": "Mrays/s", "value": res["rays"] / (res["ms_per_frame"] * 1e-3) / 1e6, "unit": "Mrays/s",
                    "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": res["ms_per_frame"],
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                    "dtype": "f32 + f16 operands / f32 accumulate (tcgen05 MLP)" if a.mlp_mode else "f32", "data": "synthetic",
                    "config": {"workload": f"{a.workload}: 1920x1080 frame, 512 samples/ray", "parallelism": res["parallelism"],
                               "chunk_rays": a.chunk, "mlp_mode": a.mlp_mode, "chunk_overlap": f"{a.streams} streams" if not a.no_overlap else "none",
                   "ert_transmittance": a.ert, "grid_scale": a.grid_scale,
                               "l2": "inputs larger than L2"},
                    "ms_per_frame": res["ms_per_frame"], "clocks": clocks,
                    "samples_per_frame": {"valid": res["valid"], "appearance": res["appearance"]}, "detail": res}
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    from landmark_b200 import scenes
    from landmark_b200.gridnerf import B200GridNeRF
    from landmark_b200.parallel import TILE, TileSharding, tile_pixel_ids
    from landmark_b200.rays import generate_rays

    spec, ckpt, pose = build_scene(a.workload, device, a.frame)
    kwargs = dict(ckpt["kwargs"])
    kwargs.update({"device": device, "args": scenes.model_args(spec, device), "is_train": False})
    model = B200GridNeRF(**kwargs, mlp_mode=a.mlp_mode, ert_transmittance=a.ert, app_plane_fp16=bool(a.app_fp16),
                         density_plane_fp16=bool(a.den_fp16), density_lattice=bool(a.den_lattice),
                         fused_appearance=bool(a.app_fusion))
    model.load(ckpt)
    if a.reload_test:
        from landmark_b200.dynamic import pin_block

        host = pin_block(ckpt)
        nbytes = sum(t.numel() * 4 for t in host.values())
        load_stream = torch.cuda.Stream(device=device)
        times = []
        for _ in range(4):
            torch.cuda.synchronize()
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r0.record(load_stream)
            model.reload_field_async(host, load_stream)
            r1.record(load_stream)
            torch.cuda.synchronize()
            times.append(r0.elapsed_time(r1))
        ms = sorted(times[1:])[1]
        print(json.dumps({"reload_block": {"bytes_from_host": nbytes, "ms": ms, "gb_per_s": nbytes / ms / 1e6,
                                           "what": "pinned host planes/lines -> device staging -> channel-last (fp16 for appearance) "
                                                   "on a copy stream, no allocation, median of 3"}}))
        return
    cpu_sd = None
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        cpu_sd = {k: v.cpu() for k, v in ckpt["state_dict"].items()}
    model.release_torch_planes()
    del ckpt["state_dict"]
    torch.cuda.empty_cache()

    H, W, S = spec.height, spec.width, spec.n_samples
    if a.profile_case:
        ids_np = tile_pixel_ids(H, W, 0, 1)
        mid = (ids_np.shape[0] // 2 // (TILE * TILE)) * TILE * TILE
        pix = torch.from_numpy(ids_np[mid:mid + a.profile_case]).to(device)
        rays = generate_rays(pose, H, W, spec.focal, device=device, pixel_ids=pix)
        for _ in range(2):
            model.render_rays(rays, S, True, chunk=a.profile_case)
            st = model.check_pending_status()
        torch.cuda.synchronize()
        print(json.dumps({"profile_case_rays": int(rays.shape[0]), "valid": int(st[2]), "appearance": int(st[3]),
                          "density_evaluated": int(st[5])}))
        return
    if world == 1 and a.order == "rows":
        shard = TileSharding(H, W, 0, 1, device, tile=max(H, W))  # one tile = the whole image, row-major
    else:
        shard = TileSharding(H, W, rank, world, device)
    n_local, n_pad, pix = shard.n_local, shard.n_pad, shard.pixel_ids
    rays = generate_rays(pose, H, W, spec.focal, device=device, pixel_ids=pix)
    if not a.no_overlap and a.streams > 1:
        # at least one chunk per stream: a rank of an 8-GPU run owns ~259 k rays
        per_stream = -(-n_local // a.streams)
        a.chunk = max(4096, min(a.chunk, -(-per_stream // 4096) * 4096))
    rgb = torch.zeros((n_pad, 3), dtype=torch.float32, device=device)
    depth = torch.zeros((n_pad,), dtype=torch.float32, device=device)
    image = torch.zeros((H * W, 3), dtype=torch.float32, device=device)

    # Two frames in flight (the throughput form of the reference's pipe engine, dist_render/engine/pipe_engine.py):
    # frame k writes buffer set k % 2; its chunk streams wait only for the assembly of frame k - 2, which freed that
    # set, so the first chunks of a frame run beside the last chunk and the tile gather of the frame before it.
    # `rgb`, `depth`, `image` are set 0 (both sets end with the same pixels: every step renders the same rays).
    pipelined = a.frames_in_flight > 1 and not a.no_overlap and a.streams > 1
    sets = [(rgb, depth, image)]
    if pipelined:
        sets.append((torch.zeros_like(rgb), torch.zeros_like(depth), torch.zeros_like(image)))
    set_free = [None] * len(sets)
    frame_no = [0]

    def step(overlap=(0 if a.no_overlap else a.streams)):
        b = frame_no[0] % len(sets) if (pipelined and overlap) else 0
        frame_no[0] += 1
        rgb_b, depth_b, image_b = sets[b]
        model.render_rays(rays, S, True, chunk=a.chunk, rgb_out=rgb_b[:n_local], depth_out=depth_b[:n_local], overlap=overlap,
                          after=set_free[b] if (pipelined and overlap) else None)
        shard.assemble(rgb_b, image_b)
        if pipelined and overlap:
            set_free[b] = torch.cuda.Event()
            set_free[b].record()

    for _ in range(max(a.warmup, 3)):
        step()
    model.check_pending_status()
    torch.cuda.synchronize()
    stats = model.last_status.copy()

    # ---- timed region: device-resident inputs -----------------------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([ms_total], device=device, dtype=torch.float64)
    per_rank_ms = [ms_total / a.steps]
    if world > 1:
        allt = torch.zeros(world, device=device, dtype=torch.float64)
        dist.all_gather_into_tensor(allt, t)
        per_rank_ms = [float(v) / a.steps for v in allt.tolist()]
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / a.steps
    model.check_pending_status()
    # ---- per-kernel times: the same K frames once more on ONE stream, CUDA events around every
    # stage (chunks of a frame run back to back, so a span times its kernels alone) -------------
    model.profile_enable(True)
    model.profile_collect()
    torch.cuda.synchronize()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(a.steps):
        step(overlap=False)
    e3.record()
    torch.cuda.synchronize()
    ms_step_single = e2.elapsed_time(e3) / a.steps
    stage_ms, stage_launches = model.profile_collect()
    model.profile_enable(False)
    model.check_pending_status()

    # ---- end to end through the runner API: pose on the host in, uint8 [H, W, 4] image on rank 0's host out.
    # Inside the timed region, every frame: pose broadcast to the ranks, ray generation, the chunk loop,
    # the NCCL all-gather of the tiles, frame assembly, RGBA8 conversion, the device->host copy of the
    # image into pinned memory and the status read (dist_render/runner/ddp_runner/nerf_ddp_runner.py:25-42,
    # dist_render/ddp_infer/nerf_inferer.py:345-378). -------------------------------------------------
    from landmark_b200.engine import FrameRenderer, NerfDDPRunner

    runner = NerfDDPRunner(FrameRenderer(model, S, True, chunk=a.chunk, streams=(1 if a.no_overlap else a.streams)),
                           H, W, focal=spec.focal, rank=rank, world=world)
    n_e2e_warm = 2

    def e2e_frames(k):
        if rank == 0:
            for _ in range(k):
                img = runner.run_batch(pose)
            return img
        runner.serve(max_frames=k)
        return None

    e2e_frames(n_e2e_warm)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    img_host = e2e_frames(a.steps)
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / a.steps
    t = torch.tensor([e2e_s], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    e2e_same = None
    if rank == 0:
        want = (image.clamp(0, 1) * 255).to(torch.uint8).view(H, W, 3).cpu().numpy()
        e2e_same = bool(np.array_equal(img_host[..., :3], want))
    del runner

    # ---- the previous end-to-end figure, kept as an extra key: host rays in, host rgb/depth out through
    # gnr_render_host (this rank's rays only, no gather) --------------------------------------------------
    rays_h = rays.cpu().pin_memory()
    rgb_h = torch.empty((n_local, 3), dtype=torch.float32).pin_memory()
    depth_h = torch.empty((n_local,), dtype=torch.float32).pin_memory()
    for _ in range(2):
        model.render_host(rays_h, S, True, chunk=a.chunk, rgb_out=rgb_h, depth_out=depth_h)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        model.render_host(rays_h, S, True, chunk=a.chunk, rgb_out=rgb_h, depth_out=depth_h)
    rays_e2e_s = (time.perf_counter() - t0) / a.steps
    t = torch.tensor([rays_e2e_s], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    rays_e2e_s = float(t.item())
    same = bool(torch.equal(rgb_h, rgb[:n_local].cpu()))
    del rays_h, rgb_h, depth_h

    # ---- the frame as one replayed CUDA graph: pose in, RGBA8 pixels out (device) -----------------
    graphed = None
    if world == 1 and not a.no_graph:
        from landmark_b200.engine import GraphedFrameRenderer

        gr = GraphedFrameRenderer(model, H, W, spec.focal, pixel_ids=pix, n_samples=S, chunk=a.chunk,
                                  streams=(1 if a.no_overlap else a.streams)).capture(pose)
        for _ in range(2):
            gr.render(pose)
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        g0.record()
        for _ in range(a.steps):
            gr.render(pose)
        host_ms = (time.perf_counter() - t0) * 1e3 / a.steps  # host time to submit a frame
        g1.record()
        torch.cuda.synchronize()
        gr.finish()
        ms_g = g0.elapsed_time(g1) / a.steps
        graphed = {"value": H * W / (ms_g * 1e-3) / 1e6, "unit": "Mrays/s", "ms_per_frame": ms_g,
                   "host_submit_ms_per_frame": host_ms, "same_pixels_as_eager": bool(torch.equal(gr.rgb, rgb[:n_local])),
                   "what": "pose upload + ray generation + chunk loop + RGBA8 as one CUDA graph replay per frame"}
        del gr
        torch.cuda.empty_cache()

    # ---- the same frame with every approximation off: fp32 CUDA-core MLP, fp32 planes, no early
    # termination.  Its image is the full-frame check of the fast configuration. -----------------
    strict = None
    if world == 1 and not a.no_strict:
        _, ckpt2, _ = build_scene(a.workload, device, a.frame)
        m2 = B200GridNeRF(**kwargs, mlp_mode=0, ert_transmittance=0.0, app_plane_fp16=False, density_plane_fp16=False)
        m2.load(ckpt2)
        m2.release_torch_planes()
        del ckpt2
        torch.cuda.empty_cache()
        rgb2, depth2 = torch.zeros_like(rgb), torch.zeros_like(depth)

        def step2():
            m2.render_rays(rays, S, True, chunk=a.chunk, rgb_out=rgb2[:n_local], depth_out=depth2[:n_local],
                           overlap=(0 if a.no_overlap else a.streams))

        for _ in range(3):
            step2()
        m2.check_pending_status()
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(a.steps):
            step2()
        s1.record()
        torch.cuda.synchronize()
        st2 = m2.check_pending_status()
        ms2 = s0.elapsed_time(s1) / a.steps
        err2 = (rgb2[:n_local] - rgb[:n_local]).abs().max(dim=1).values
        strict = {"value": H * W / (ms2 * 1e-3) / 1e6, "unit": "Mrays/s", "ms_per_step": ms2,
                  "config": "mlp_mode 0 (fp32 CUDA-core MLP), fp32 planes, ert_transmittance 0",
                  "density_evaluated": float(st2[5]),
                  "fast_vs_strict_max_abs_rgb_diff": float(err2.max()), "fast_vs_strict_rays_above_1e-4": int((err2 > 1e-4).sum()),
                  "rays_compared": int(n_local)}
        del m2, rgb2, depth2
        torch.cuda.empty_cache()

    # ---- other configurations of the same frame, a few frames each (N = 1): the literal density_shift = -10
    # scene, the coarser termination the scene description names (T < 1e-3), the split-precision
    # tensor-core mode, and the defaults with one optimisation switched off at a time ---------------------
    variants = None
    if world == 1 and not a.no_variants:
        variants = {}

        def measure(label, what, workload=None, **opts):
            _, ck, _ = build_scene(workload or a.workload, device, a.frame)
            kw = dict(ck["kwargs"])
            kw.update({"device": device, "args": scenes.model_args(spec, device), "is_train": False})
            base = {"mlp_mode": a.mlp_mode, "ert_transmittance": a.ert, "app_plane_fp16": bool(a.app_fp16),
                    "density_plane_fp16": bool(a.den_fp16), "density_lattice": bool(a.den_lattice),
                    "fused_appearance": bool(a.app_fusion)}
            base.update(opts)
            mv = B200GridNeRF(**kw, **base)
            mv.load(ck)
            mv.release_torch_planes()
            del ck
            torch.cuda.empty_cache()
            out_rgb, out_depth = torch.zeros_like(rgb), torch.zeros_like(depth)

            def one():
                mv.render_rays(rays, S, True, chunk=a.chunk, rgb_out=out_rgb[:n_local], depth_out=out_depth[:n_local],
                               overlap=(0 if a.no_overlap else a.streams))

            for _ in range(3):
                one()
            mv.check_pending_status()
            torch.cuda.synchronize()
            v0, v1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            v0.record()
            for _ in range(3):
                one()
            v1.record()
            torch.cuda.synchronize()
            stv = mv.check_pending_status()
            ms_v = v0.elapsed_time(v1) / 3
            diff = (out_rgb[:n_local] - rgb[:n_local]).abs().max(dim=1).values
            variants[label] = {"what": what, "ms_per_frame": ms_v, "Mrays_per_s": H * W / (ms_v * 1e-3) / 1e6,
                               "appearance_samples": float(stv[3]), "density_evaluated": float(stv[5]),
                               "max_abs_rgb_diff_vs_headline": float(diff.max()), "rays_above_1e-4_vs_headline": int((diff > 1e-4).sum())}
            del mv, out_rgb, out_depth
            torch.cuda.empty_cache()

        if a.workload == "city_lit":
            measure("city_literal", "the scene with its literal density_shift = -10: no sample passes the appearance "
                    "threshold, only sampling, density and compositing run (rgb is not comparable with the headline)", workload="city")
        measure("ert_1e-3", "rays stop at transmittance < 1e-3 (the scene description's own termination)", ert_transmittance=1e-3)
        measure("mlp_mode_1", "tcgen05 MLP with activations and products as fp16 hi + lo, fp32 appearance planes, separate kernels",
                mlp_mode=1, app_plane_fp16=False)
        measure("separate_appearance_kernels", "appearance gather and MLP as two kernels (product tiles through HBM)",
                fused_appearance=False)
        measure("density_from_planes", "density from the three plane x line pairs instead of the pre-summed lattice",
                density_lattice=False)
        # the baked appearance lattice takes 69 GB next to its own chunk scratch: the headline model's scratch
        # buffers go back to the allocator first (they are made again when that model renders next)
        model.release_workspaces()
        free_b, _ = torch.cuda.mem_get_info(device)
        if free_b > 125e9:
            measure("appearance_lattice", "appearance features from a baked lattice (27 projected features as 32 fp16 channels per "
                    "grid point, 69 GB): 8 taps per sample, no plane gather, no projection GEMM; a trade of memory for time, opt-in",
                    appearance_lattice=True)
        else:
            variants["appearance_lattice"] = {"skipped": f"{free_b / 1e9:.0f} GB of device memory free, 125 GB needed"}

    l1_measured = None
    if world == 1:
        from landmark_b200._lib import check as _check, lib as _glib
        import ctypes as _C

        val = _C.c_float(0.0)
        _check(_glib.gnr_measure_l1_bandwidth(local_rank, 4000, _C.byref(val)), "gnr_measure_l1_bandwidth")
        l1_measured = float(val.value)

    # what every rank did: its share of the samples and the time its kernels took on one stream (separates an
    # uneven split of the work from kernels that lose efficiency on small chunks)
    mine = torch.tensor([float(stats[2]), float(stats[3]), float(stats[5]), float(n_local), ms_step_single] +
                        [stage_ms[k] / a.steps for k in sorted(stage_ms)], device=device, dtype=torch.float64)
    rank_table = mine[None]
    if world > 1:
        rank_table = torch.zeros((world, mine.numel()), device=device, dtype=torch.float64)
        dist.all_gather_into_tensor(rank_table, mine)
    tot = torch.tensor([float(stats[2]), float(stats[3]), float(n_local), float(stats[5])], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tot)
    # ---- the two model-parallel layouts of the same frame on these N GPUs, a few frames each: the field cut
    # into N spatial blocks (samples routed to their owners by all-to-all) and the appearance channels split
    # N ways (partial projections reduce-scattered).  Every rank takes part. ----------------------------------
    model_parallel = None
    if world > 1 and not a.no_model_parallel:
        from landmark_b200.model_parallel_run import run as run_model_parallel

        del model, shard, rays, rgb, depth, image
        torch.cuda.empty_cache()
        model_parallel = {}
        for wl in ("city_blocks", "city_channels"):
            try:
                chunk_mp = a.chunk_model_parallel
                if wl == "city_blocks":  # rays are tile-sharded there: at least four chunks per rank for the two-lane pipeline
                    chunk_mp = min(chunk_mp, max(65536, -(-(H * W // world) // 4 // 4096) * 4096))
                res = run_model_parallel(wl, 3, 1, chunk_mp, a.mlp_mode, rank, world, device, 1, False, ert=a.ert,
                                         app_fp16=bool(a.app_fp16), den_lattice=bool(a.den_lattice))
                model_parallel[wl] = {"ms_per_frame": res["ms_per_frame"], "Mrays_per_s": res["rays"] / (res["ms_per_frame"] * 1e-3) / 1e6,
                                      "parallelism": res["parallelism"], "valid_samples": res["valid"],
                                      "appearance_samples": res["appearance"], "steps": 3, "warmup": 1,
                                      "chunks_per_rank": res["chunks_per_rank"], "sections_ms_rank0": res["sections_ms"]}
            except RuntimeError as exc:  # reported, never fatal for the headline line
                model_parallel[wl] = {"failed": str(exc).splitlines()[0][:300]}
            torch.cuda.empty_cache()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pk = peaks()
    n_valid, n_app = float(stats[2]), float(stats[3])  # this rank's samples per frame
    n_density = float(stats[5]) if stats[5] > 0 else n_valid  # samples whose density was actually gathered
    per_launch = {k: (stage_ms[k] / a.steps) for k in stage_ms}  # ms per frame per stage (all chunks)
    roof = {}
    sm_mhz = float((clocks or {}).get("sm_mhz") or 1965.0)
    l1_nominal = L1_BYTES_PER_CLOCK_PER_SM * torch.cuda.get_device_properties(device).multi_processor_count * sm_mhz * 1e6 / 1e9
    l1_peak = l1_measured if l1_measured else l1_nominal
    l1_peak_is = ("measured on this GPU in this run: L1-resident 256-bit loads into registers (gnr_measure_l1_bandwidth)"
                  if l1_measured else "128 B/clk/SM x SMs x median SM clock (nominal)")
    dram = {}
    tpath = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    if os.path.exists(tpath):
        with open(tpath) as fh:
            dram = json.load(fh)

    def l1_roof(bytes_per_sample, samples, ms):
        ach_l1 = samples * bytes_per_sample / (ms * 1e-3) / 1e9
        return {"achieved": ach_l1, "peak": l1_peak, "unit": "GB/s", "frac": ach_l1 / l1_peak, "peak_is": l1_peak_is,
                "bytes_per_sample": bytes_per_sample}

    def hbm_part(key, samples, ms):
        """DRAM traffic of the kernel (ncu, per sample, scaled to this frame) against the measured copy bandwidth."""
        if key not in dram:
            return None
        tb = dram[key]["dram_bytes_per_sample"] * samples
        ach_d = tb / (ms * 1e-3) / 1e9
        return {"traffic_bytes": tb, "achieved": ach_d, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach_d / pk["hbm_gbs"],
                "source": dram[key].get("source")}

    app_l1_bytes = APP_L1_BYTES_PER_SAMPLE // (2 if a.app_fp16 else 1)
    if per_launch["density"] > 0:
        if a.den_lattice:
            key, l1b = "march_lattice_kernel", 8 * 4  # eight scalar taps of the pre-summed lattice
            note = "fused density (8-tap lattice) + transmittance product + termination (march_kernel, LAT)"
        else:
            key, l1b = "density_kernel", DENSITY_L1_BYTES_PER_SAMPLE // (2 if a.den_fp16 else 1)
            note = "fused density gather (18 taps x 16 ch) + transmittance product (march_kernel)"
        r = l1_roof(l1b, n_density, per_launch["density"])
        roof["density_kernel"] = {"bound": "l1", **r, "ms_per_frame": per_launch["density"], "samples_gathered": n_density,
                                  "hbm": hbm_part(key, n_density, per_launch["density"]), "note": note}
    if per_launch["app_gather"] > 0 and n_app > 0:
        r = l1_roof(app_l1_bytes, n_app, per_launch["app_gather"])
        roof["app_gather_kernel"] = {"bound": "l1", **r, "ms_per_frame": per_launch["app_gather"],
                                     "hbm": hbm_part("app_gather_kernel", n_app, per_launch["app_gather"])}
    if per_launch["mlp"] > 0 and n_app > 0:
        fused_app = per_launch["app_gather"] == 0 and a.mlp_mode == 2  # gather + basis + MLP in one kernel
        flop = MLP_FLOP_PER_SAMPLE + (BASIS_FLOP_PER_SAMPLE if a.mlp_mode else 0)
        ach = n_app * flop / (per_launch["mlp"] * 1e-3) / 1e12
        key = "app_mlp_fused_kernel" if fused_app else "mlp_kernel"
        roof["mlp_kernel"] = {"bound": "tensor", "achieved": ach, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                              "frac": ach / pk["bf16_tflops"], "ms_per_frame": per_launch["mlp"], "flop_per_sample": flop,
                              "hbm": hbm_part(key, n_app, per_launch["mlp"]),
                              "note": "fp32 CUDA-core kernel" if a.mlp_mode == 0 else
                                      ("tcgen05 kernel with the appearance gather inside (app_mlp_fused_kernel)" if fused_app
                                       else "tcgen05 kernel (basis + MLP)")}
        if fused_app:
            roof["mlp_kernel"]["l1_to_register"] = l1_roof(app_l1_bytes, n_app, per_launch["mlp"])
            # everything the SM's L1 / shared-memory port moves for a sample: its texels into registers plus its share
            # (1/128) of the 91 KB of weight operands the four GEMMs of a 128-sample tile fetch from shared memory
            port = l1_roof(app_l1_bytes + FUSED_WEIGHT_OPERAND_BYTES_PER_TILE // 128, n_app, per_launch["mlp"])
            port["what"] = ("texel bytes into registers + weight-operand bytes of the tile's MMAs out of shared memory, against "
                            "the measured L1->register rate (the operand fetch shares that port; its own ceiling is not measured)")
            roof["mlp_kernel"]["l1_port"] = port
    dominant = max(roof, key=lambda k: roof[k]["ms_per_frame"]) if roof else None
    roofline = None
    if dominant:
        roofline = dict(roof[dominant])
        roofline["kernel"] = dominant
        roofline["peak_source"] = f"of {pk['source']}" if roofline["bound"] == "tensor" else roofline.get("peak_is")
        roofline["traffic"] = (roofline.get("hbm") or {}).get("traffic_bytes")
        roofline["per"] = "frame (sum over the chunk launches of this kernel)"
        roofline["timing"] = "CUDA events around the kernel on its stream, single-stream pass of the same K frames"

    line = {
        "metric": "Mrays/s", "value": H * W / (ms_step * 1e-3) / 1e6, "unit": "Mrays/s", "n_gpus": world,
        "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32 (gathers, compositing) + f16 operands / f32 accumulate (tcgen05 MLP)" if a.mlp_mode else "f32", "data": "synthetic",
        "config": {"workload": f"{a.workload}: {W}x{H} frame, 512 samples/ray, grid 2048x2048x256, 16/48 ch",
                   "parallelism": f"tiles{TILE}x{TILE} round-robin x{world}" if world > 1 or a.order == "tiles" else "rows",
                   "chunk_rays": a.chunk, "mlp_mode": a.mlp_mode, "chunk_overlap": f"{a.streams} streams" if not a.no_overlap else "none",
                   "ert_transmittance": a.ert, "app_plane_storage": "fp16" if a.app_fp16 else "fp32",
                   "density_plane_storage": "fp16" if a.den_fp16 else "fp32",
                   "density_lattice": bool(a.den_lattice), "fused_appearance": bool(a.app_fusion),
                   "frames_in_flight": 2 if pipelined else 1,
                   "l2": "inputs larger than L2 (1.34 GB of planes, >0.5 GB of per-frame sample lists)"},
        "ms_per_frame": ms_step, "fps": 1e3 / ms_step,
        "ms_per_frame_single_stream": ms_step_single,
        "per_rank": {"ms_per_frame": per_rank_ms,
                     "columns": ["valid", "appearance", "density_evaluated", "rays", "ms_single_stream"] + [f"ms_{k}" for k in sorted(stage_ms)],
                     "rows": [[round(float(v), 3) for v in r] for r in rank_table.tolist()]},
        "e2e": {"value": H * W / e2e_s / 1e6, "unit": "Mrays/s", "ms_per_frame": e2e_s * 1e3,
                "h2d_bytes_per_step": 56, "d2h_bytes_per_step": int(H * W * 4),
                "api": "NerfDDPRunner.run_batch(pose) -> uint8 [H, W, 4] on rank 0's host: pose broadcast, ray generation, "
                       "chunk loop, tile all-gather, frame assembly, RGBA8, pinned device->host copy, status read",
                "same_pixels_as_device_path": e2e_same},
        "e2e_ray_buffers": {"value": H * W / rays_e2e_s / 1e6, "unit": "Mrays/s", "ms_per_frame": rays_e2e_s * 1e3,
                            "h2d_bytes_per_step": int(n_local * 24), "d2h_bytes_per_step": int(n_local * 16),
                            "api": "gnr_render_host: this rank's host rays in, host rgb + depth out (no gather)",
                            "matches_device_path": same},
        "gpu_launches": int(sum(stage_launches.values())),
        "clocks": clocks,
        "roofline": roofline,
        "roofline_all": roof,
        "stage_ms_per_frame": per_launch,
        "samples_per_frame": {"valid": float(tot[0].item()), "appearance": float(tot[1].item()),
                              "rays": float(tot[2].item()), "density_evaluated": float(tot[3].item())},
    }
    if graphed is not None:
        line["graph_replay"] = graphed
    if strict is not None:
        line["strict_fp32"] = strict
    if variants is not None:
        line["variants"] = variants
    if model_parallel is not None:
        line["model_parallel"] = model_parallel
    if cpu_sd is not None:
        from oracle import gridnerf_oracle as orc

        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        vol = scenes.make_alpha_volume(spec)
        field = orc.Field(cpu_sd, scenes.model_kwargs(spec), vol, torch.tensor(spec.aabb), 0.0)
        first = 536 * W
        sample = generate_rays(pose, H, W, spec.focal, device=device, first_pixel=first, n=CPU_SAMPLE_RAYS).cpu()
        t0 = time.perf_counter()
        ref = orc.render_chunk(field, sample, S, True)
        dt = time.perf_counter() - t0
        got, _ = model(sample.to(device), N_samples=S)
        err = (got["rgb_map"].cpu() - ref["rgb_map"]).abs().max(dim=1).values
        line["cpu_baseline"] = {"value": CPU_SAMPLE_RAYS / dt / 1e6, "unit": "Mrays/s", "cores": cores, "kind": "port",
                                "sample": f"{CPU_SAMPLE_RAYS} rays (image rows 536-570), one pass, torch {torch.__version__} CPU",
                                "rays_above_1e-4_vs_gpu": int((err > 1e-4).sum()), "max_abs_rgb_diff": float(err.max())}
        # the same torch port on this GPU (the reference's torch path with device="cuda"): a same-hardware
        # reference point between the CPU baseline and the CUDA path
        try:
            gfield = orc.Field(cpu_sd, scenes.model_kwargs(spec), vol, torch.tensor(spec.aabb), 0.0).to(device)
            gs = sample.to(device)
            chunk_t = 8192  # the reference's render_batch_size
            orc.render_rays(gfield, gs[:chunk_t], S, True, chunk=chunk_t)
            torch.cuda.synchronize()
            ms_t = float("inf")
            for _ in range(2):  # best of two passes (the first still grows torch's allocator pools)
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0.record()
                g_rgb, _ = orc.render_rays(gfield, gs, S, True, chunk=chunk_t)
                c1.record()
                torch.cuda.synchronize()
                ms_t = min(ms_t, c0.elapsed_time(c1))
            errg = (got["rgb_map"] - g_rgb).abs().max(dim=1).values
            line["torch_cuda_baseline"] = {"value": CPU_SAMPLE_RAYS / (ms_t * 1e-3) / 1e6, "unit": "Mrays/s",
                                           "ms_per_frame_extrapolated": ms_t * H * W / CPU_SAMPLE_RAYS,
                                           "what": f"the same torch port with every tensor on {torch.cuda.get_device_name(device)} "
                                                   f"(grid_sample, cumprod, linear: stock torch {torch.__version__} kernels), "
                                                   f"{CPU_SAMPLE_RAYS} rays in chunks of {chunk_t}",
                                           "rays_above_1e-4_vs_cuda_path": int((errg > 1e-4).sum())}
            del gfield, gs, g_rgb
        except RuntimeError as exc:  # e.g. out of memory on a smaller GPU: report, do not fail the bench
            line["torch_cuda_baseline"] = {"unavailable": str(exc).splitlines()[0][:200]}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
