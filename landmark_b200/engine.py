"""Runner and engines of the online renderer: pose in, ``uint8 [H, W, 4]`` image out.

Mirrors the entry points of the reference's ``dist_render``:

* ``NerfDDPRunner.run_batch(pose)`` (dist_render/runner/ddp_runner/nerf_ddp_runner.py) =
  ``model_infer_preprocess`` (pose -> rays, dist_render/ddp_infer/nerf_inferer.py:393-410) +
  ``infer`` (:267-341) + ``model_infer_postprocess`` (:345-378: x255, alpha 255, ``.byte()``, pinned
  device->host copy, numpy image);
* ``MainRankDDPRenderEngine.start / submit / warm_up / run_for_latency``
  (dist_render/engine/ddp_engine.py:18-75) on rank 0;
* ``OtherRankRenderEngine.start`` (dist_render/engine/render_engine.py:99-120): the loop the
  other ranks sit in (``render_other_rank``, nerf_inferer.py:126-193).

Differences in mechanism, not in interface: rank 0 broadcasts the pose (12 floats + focal +
a stop flag) instead of scattering H*W rays, every rank generates the rays of its own 64x64
tiles and the colours come together with one all-gather (``landmark_b200.parallel``).
"""

from __future__ import annotations

import ctypes as C
import time
from typing import Callable, List, Optional

import numpy as np
import torch

from .parallel import TileSharding

RENDER_1080P = (1080, 1920, 1483.6378)  # H, W, focal of the online renderer (nerf_inferer.py:385-404)


class FrameRenderer:
    """Renders the pixels a rank owns.  The default implementation drives ``B200GridNeRF``; tests
    substitute a CPU fake with the same two methods to exercise the multi-rank protocol."""

    def __init__(self, model, n_samples: int = -1, white_bg: bool = True, chunk: int = 131072, streams: int = 2):
        self.model, self.n_samples, self.white_bg, self.chunk = model, n_samples, white_bg, chunk
        self.streams = streams  # consecutive chunks of a frame rotate over this many streams
        self.device = model.device

    def render_pixels(self, pose: np.ndarray, H: int, W: int, focal: float, pixel_ids: torch.Tensor,
                      rgb_out: torch.Tensor) -> None:
        from .rays import generate_rays

        rays = generate_rays(pose, H, W, focal, device=self.device, pixel_ids=pixel_ids)
        self.model.render_rays(rays, self.n_samples, self.white_bg, chunk=self.chunk, rgb_out=rgb_out,
                               overlap=self.streams if self.streams > 1 else False)

    def finish(self):
        self.model.check_pending_status()

    def to_rgba8(self, image: torch.Tensor, out: torch.Tensor) -> None:
        from ._lib import check, lib

        with torch.cuda.device(self.device):
            check(lib.gnr_rgba8(C.c_void_p(image.data_ptr()), image.shape[0], C.c_void_p(out.data_ptr()),
                                C.c_void_p(torch.cuda.current_stream().cuda_stream)), "gnr_rgba8")


class GraphedFrameRenderer:
    """One frame of a fixed shape as a replayable CUDA graph.

    Ray generation for this rank's pixels (from a pose in device memory), the chunk loop of
    ``render_rays`` on its streams, and the RGBA8 conversion are captured once; ``render(pose)`` copies
    the 12 pose floats through a pinned slot into that device buffer and replays the graph, so a frame costs one launch on the host instead
    of some 400 (the three-stage overlap of dist_render/runner/pipe_runner/nerf_pipe_runner.py:102-140
    then needs no host thread per stage).  Every buffer the graph touches is allocated before the
    capture and kept alive here.  List overflow / expired waits are read from the status blocks
    with ``finish()``.
    """

    def __init__(self, model, H: int, W: int, focal: float, pixel_ids: Optional[torch.Tensor] = None,
                 n_samples: int = -1, white_bg: bool = True, chunk: int = 131072, streams: int = 2):
        from .rays import direction_tables

        self.model, self.H, self.W, self.focal = model, int(H), int(W), float(focal)
        self.n_samples, self.white_bg, self.chunk, self.streams = n_samples, white_bg, chunk, streams
        dev = self.device = model.device
        self.pixel_ids = None if pixel_ids is None else pixel_ids.to(device=dev, dtype=torch.int32).contiguous()
        n = self.n = self.H * self.W if pixel_ids is None else int(self.pixel_ids.numel())
        dx, dy = direction_tables(self.H, self.W, self.focal)
        self.dir_x, self.dir_y = dx.to(dev), dy.to(dev)
        # pinned pose slots: a frame's pose copy reads its slot when the stream gets there, so frames
        # submitted before earlier ones have run each need their own (8 frames may be in flight)
        self.pose_ring = torch.zeros((8, 12), dtype=torch.float32).pin_memory()
        self._pose_slot = 0
        self.pose_dev = torch.zeros(12, dtype=torch.float32, device=dev)
        self.rays = torch.empty((n, 6), dtype=torch.float32, device=dev)
        self.rgb = torch.empty((n, 3), dtype=torch.float32, device=dev)
        self.depth = torch.empty((n,), dtype=torch.float32, device=dev)
        self.rgba = torch.empty((n, 4), dtype=torch.uint8, device=dev)
        # with a pixel list that covers the whole frame (e.g. tile order, which the kernels prefer) the graph
        # also scatters the pixels back into row-major order: ``rgba_frame`` is the image
        self.rgba_frame = None
        if self.pixel_ids is not None and n == self.H * self.W:
            self._pixel_ids64 = self.pixel_ids.to(torch.int64)
            self.rgba_frame = torch.zeros((n, 4), dtype=torch.uint8, device=dev)
        self.graph = None

    def _enqueue(self):
        from ._lib import check, lib

        with torch.cuda.device(self.device):
            st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            check(lib.gnr_generate_rays_dev(C.c_void_p(self.pose_dev.data_ptr()), C.c_void_p(self.dir_x.data_ptr()),
                                            C.c_void_p(self.dir_y.data_ptr()), self.H, self.W,
                                            C.c_void_p(self.pixel_ids.data_ptr() if self.pixel_ids is not None else 0),
                                            0, self.n, C.c_void_p(self.rays.data_ptr()), st), "gnr_generate_rays_dev")
            self.model.render_rays(self.rays, self.n_samples, self.white_bg, chunk=self.chunk, rgb_out=self.rgb,
                                   depth_out=self.depth, overlap=self.streams)
            self._status = self.model._pending_status
            # the captured launches carry these buffers' addresses: hold them for the graph's lifetime
            self._workspaces = list(self.model._last_workspaces)
            check(lib.gnr_rgba8(C.c_void_p(self.rgb.data_ptr()), self.n, C.c_void_p(self.rgba.data_ptr()),
                                C.c_void_p(torch.cuda.current_stream().cuda_stream)), "gnr_rgba8")
            if self.rgba_frame is not None:
                self.rgba_frame.view(torch.int32).view(-1).index_copy_(0, self._pixel_ids64, self.rgba.view(torch.int32).view(-1))

    def capture(self, pose: np.ndarray):
        """Warm up (creates workspaces and side streams) and capture the frame."""
        self._set_pose(pose)
        with torch.cuda.device(self.device):
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._enqueue()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize(self.device)
            self.model.check_pending_status()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._enqueue()
            self.graph = g
        return self

    def _set_pose(self, pose):
        """Pose -> next pinned slot -> device pose buffer (an asynchronous copy on the current stream,
        in front of the graph, which reads the pose from device memory)."""
        p = np.asarray(pose.cpu() if isinstance(pose, torch.Tensor) else pose, dtype=np.float32)[:3, :4].reshape(-1)
        slot = self.pose_ring[self._pose_slot]
        self._pose_slot = (self._pose_slot + 1) % self.pose_ring.shape[0]
        slot.copy_(torch.from_numpy(np.ascontiguousarray(p)))
        with torch.cuda.device(self.device):
            self.pose_dev.copy_(slot, non_blocking=True)

    def render(self, pose) -> torch.Tensor:
        """Replay for ``pose``; returns the RGBA8 pixels ``[n, 4]`` (device, valid after the stream
        work completes; the same buffer every frame)."""
        if self.graph is None:
            raise RuntimeError("capture() has not been called")
        self._set_pose(pose)
        self.graph.replay()
        return self.rgba

    def finish(self):
        self.model._pending_status = self._status
        return self.model.check_pending_status()

    # frame backend of pipe_engine.PipeRunner (single process)
    def enqueue(self, pose, host_image: torch.Tensor):
        """Replay for ``pose`` and copy the RGBA8 frame into ``host_image`` (``uint8 [H, W, 4]``, pinned;
        needs a graph over the whole image in row-major pixel order).  Returns an event behind the copy."""
        if self.pixel_ids is not None and self.rgba_frame is None:
            raise RuntimeError("enqueue needs a renderer over the whole frame (no pixel list, or one that covers it)")
        self.render(pose)
        frame = self.rgba_frame if self.rgba_frame is not None else self.rgba
        with torch.cuda.device(self.device):
            host_image.copy_(frame.view(self.H, self.W, 4), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        return ev

    def stop(self):
        return None


class NerfDDPRunner:
    """``run_batch(single_pose) -> numpy uint8 [H, W, 4]``.  ``single_pose`` is ``[3, 4]`` or ``[3, 5]``
    (focal in the last column); without a focal column the ``focal`` given here is used."""

    def __init__(self, renderer, H: int = RENDER_1080P[0], W: int = RENDER_1080P[1], focal: Optional[float] = RENDER_1080P[2],
                 rank: int = 0, world: int = 1, group=None):
        self.renderer, self.H, self.W, self.focal = renderer, int(H), int(W), focal
        self.rank, self.world, self.group = rank, world, group
        dev = renderer.device
        self.shard = TileSharding(self.H, self.W, rank, world, dev, group=group)
        self.rgb = torch.zeros((self.shard.n_pad, 3), dtype=torch.float32, device=dev)
        self.image = torch.zeros((self.H * self.W, 3), dtype=torch.float32, device=dev)
        self.rgba = torch.zeros((self.H * self.W, 4), dtype=torch.uint8, device=dev)
        self.img_cpu = torch.zeros((self.H, self.W, 4), dtype=torch.uint8)
        if torch.device(dev).type == "cuda":
            self.img_cpu = self.img_cpu.pin_memory()
        # pose (12), focal, stop flag; float64 so that a double focal length reaches the other ranks unrounded
        self._msg = torch.zeros(14, dtype=torch.float64, device=dev)

    # -- rank 0 <-> other ranks -------------------------------------------------------------------
    def _broadcast(self, pose: Optional[np.ndarray], focal: float, stop: bool):
        import torch.distributed as dist

        if self.world == 1:
            return pose, focal, stop
        if self.rank == 0:
            m = np.zeros(14, dtype=np.float64)
            if pose is not None:
                m[:12] = np.asarray(pose, dtype=np.float32)[:3, :4].reshape(-1)
            m[12], m[13] = focal, 1.0 if stop else 0.0
            self._msg.copy_(torch.from_numpy(m))
        dist.broadcast(self._msg, src=0, group=self.group)
        m = self._msg.cpu().numpy()
        return m[:12].astype(np.float32).reshape(3, 4).copy(), float(m[12]), bool(m[13] > 0.5)

    def _focal_of(self, pose) -> float:
        pose = np.asarray(pose)
        if pose.shape[-1] >= 5 and self.focal is None:
            return float(pose[-1, -1])
        if self.focal is None:
            raise ValueError("no focal length: pass focal= or a [3, 5] pose")
        return float(self.focal)

    def _render_and_gather(self, pose, focal):
        self.renderer.render_pixels(pose, self.H, self.W, focal, self.shard.pixel_ids, self.rgb[: self.shard.n_local])
        self.shard.assemble(self.rgb, self.image)
        self.renderer.finish()

    def enqueue(self, single_pose, host_image: torch.Tensor):
        """Everything ``run_batch`` does for one frame except waiting for it: broadcast, render, gather,
        RGBA8, and the copy of the image into ``host_image`` (``uint8 [H, W, 4]``, pinned for an
        asynchronous copy).  Returns an event recorded behind that copy; frames enqueued one after the
        other share this runner's device buffers and are ordered by the stream."""
        if self.rank != 0:
            raise RuntimeError("enqueue / run_batch is the main rank's call; other ranks run serve()")
        pose = np.asarray(single_pose.cpu() if isinstance(single_pose, torch.Tensor) else single_pose, dtype=np.float32)
        focal = self._focal_of(pose)
        pose, focal, _ = self._broadcast(pose[:3, :4], focal, False)
        self.renderer.render_pixels(pose, self.H, self.W, focal, self.shard.pixel_ids, self.rgb[: self.shard.n_local])
        self.shard.assemble(self.rgb, self.image)
        # postprocess (nerf_inferer.py:345-378)
        self.renderer.to_rgba8(self.image, self.rgba)
        host_image.copy_(self.rgba.view(self.H, self.W, 4), non_blocking=True)
        if torch.device(self.renderer.device).type != "cuda":
            return None
        with torch.cuda.device(self.renderer.device):
            ev = torch.cuda.Event()
            ev.record()
        return ev

    HOST_RING = 4  # pinned host images run_batch rotates over

    def run_batch(self, single_pose) -> np.ndarray:
        """One frame, synchronously.  The returned array is a view of one of ``HOST_RING`` pinned host images that
        take turns: it stays untouched until ``HOST_RING - 1`` further frames have been rendered (copy it to keep it
        longer).  Handing out the pinned image itself saves an 8 MB host copy per frame."""
        ring = self.__dict__.get("_host_ring")
        if ring is None:  # pinned once, on the first frame
            ring = [self.img_cpu]
            for _ in range(self.HOST_RING - 1):
                img = torch.zeros((self.H, self.W, 4), dtype=torch.uint8)
                ring.append(img.pin_memory() if torch.device(self.renderer.device).type == "cuda" else img)
            self._host_ring = ring
        turn = self.__dict__.get("_host_turn", 0)
        host = ring[turn]
        self._host_turn = (turn + 1) % self.HOST_RING
        ev = self.enqueue(single_pose, host)
        if ev is not None:
            ev.synchronize()
        self.renderer.finish()
        return host.numpy()

    def serve(self, max_frames: int = -1) -> int:
        """Loop of a non-main rank: render every broadcast pose until the stop message (or
        ``max_frames``, the role of the reference's CI_TEST_PICTURES).  Returns frames rendered."""
        n = 0
        while max_frames < 0 or n < max_frames:
            pose, focal, stop = self._broadcast(None, 0.0, False)
            if stop:
                break
            self._render_and_gather(pose, focal)
            n += 1
        return n

    def stop(self):
        """Main rank: release the other ranks from ``serve``."""
        if self.rank == 0 and self.world > 1:
            self._broadcast(None, 0.0, True)


class MainRankDDPRenderEngine:
    """Rank-0 engine around a runner (dist_render/engine/ddp_engine.py:18-75)."""

    def __init__(self, runner_factory: Callable[[], NerfDDPRunner], poses: Optional[List[np.ndarray]] = None,
                 save_png: bool = False, save_path: str = ".", pose_num: int = -1):
        self._factory, self.runner = runner_factory, None
        self.poses, self.save_png, self.save_path, self.pose_num = poses, save_png, save_path, pose_num
        self.latency: List[float] = []

    def start(self, test: bool = False):
        self.runner = self._factory()
        if test:
            self.run_test()

    def warm_up(self, pose_num: int = 60):
        for pose in (self.poses or [])[:pose_num]:
            self.runner.run_batch(pose)

    def run_for_latency(self):
        self.latency = []
        for i, pose in enumerate(self.poses or []):
            t0 = time.time()
            out = self.runner.run_batch(pose)
            self.latency.append(time.time() - t0)
            if self.save_png:
                from PIL import Image

                Image.fromarray(out).save(f"{self.save_path}/{i}.png")
        if self.latency:
            avg = sum(self.latency) / len(self.latency)
            print("Latency:", avg, flush=True)
            print("Throughput:", 1 / avg, flush=True)

    def run_test(self):
        if self.pose_num > 0 and self.poses:
            self.poses = self.poses[: self.pose_num]
        self.warm_up()
        self.run_for_latency()

    def submit(self, pose):
        return self.runner.run_batch(pose)

    def stop(self):
        if self.runner is not None:
            self.runner.stop()


class OtherRankRenderEngine:
    """Engine of ranks > 0 (dist_render/engine/render_engine.py:99-120)."""

    def __init__(self, runner_factory: Callable[[], NerfDDPRunner], max_frames: int = -1):
        self._factory, self.max_frames, self.frames = runner_factory, max_frames, 0

    def start(self, test: bool = False):
        runner = self._factory()
        self.frames = runner.serve(self.max_frames)
