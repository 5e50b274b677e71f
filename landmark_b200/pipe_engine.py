"""Asynchronous frame engine: ``submit(pose) -> uid`` now, the image later.

Mirrors the interface of the reference's pipeline engine and runner
(``MainRankPipeRenderEngine.start / submit / get_result / wait / warm_up / run_for_latency /
run_for_throughput / stop``, dist_render/engine/pipe_engine.py:27-203; ``run_batch`` returning a
uid, ``get_result`` and ``get_result_task``, dist_render/runner/pipe_runner/nerf_pipe_runner.py).

The reference overlaps its three stages (rays, render, post-process) with one host thread and two
queues per stage.  Here a frame is a sequence of launches on CUDA streams that the host never
waits for: ``submit`` writes the pose into a pinned slot, enqueues the frame (pose upload, ray
generation, chunk loop, tile gather, RGBA8, device->host copy into a pinned image slot) and an
event, and returns.  Up to ``depth`` frames are in flight; results are taken in submission order
(``get_result``) or by uid (``wait``).  Nothing here needs a GPU: the frame backend is an object
with ``enqueue(pose, host_image) -> handle`` (``handle.synchronize()``), and the tests drive the
engine with a CPU backend.
"""

from __future__ import annotations

import itertools
import time
from collections import OrderedDict, deque
from queue import Empty
from typing import Callable, List, Optional

import numpy as np
import torch


class ResultTask:
    """What ``get_result_task`` hands out: the uid ``run_batch`` returned and the image."""

    def __init__(self, uid: str, value: np.ndarray):
        self.uid, self.value = uid, value


class _Done:
    def synchronize(self):
        return None


class CpuFrameBackend:
    """Frame backend without a device: ``fn(pose) -> uint8 [H, W, 4]`` evaluated at enqueue time."""

    def __init__(self, fn: Callable[[np.ndarray], np.ndarray], H: int, W: int):
        self.fn, self.H, self.W, self.device = fn, H, W, "cpu"

    def enqueue(self, pose, host_image: torch.Tensor):
        host_image.copy_(torch.from_numpy(np.ascontiguousarray(self.fn(np.asarray(pose, dtype=np.float32)))))
        return _Done()

    def finish(self):
        return None

    def stop(self):
        return None


class RunnerFrameBackend:
    """Frames through ``NerfDDPRunner.enqueue`` (every rank renders its tiles, NCCL all-gather, RGBA8,
    asynchronous copy to the host slot)."""

    def __init__(self, runner):
        self.runner, self.H, self.W, self.device = runner, runner.H, runner.W, runner.renderer.device

    def enqueue(self, pose, host_image: torch.Tensor):
        return self.runner.enqueue(pose, host_image) or _Done()  # a CPU runner has finished when it returns

    def finish(self):
        self.runner.renderer.finish()

    def stop(self):
        self.runner.stop()


class PipeRunner:
    """``run_batch(pose) -> uid``; ``get_result()`` (oldest first); ``get_result_task(block)``."""

    def __init__(self, backend, depth: int = 3):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.backend, self.depth = backend, depth
        pin = torch.device(backend.device).type == "cuda"
        self._slots = [torch.zeros((backend.H, backend.W, 4), dtype=torch.uint8) for _ in range(depth)]
        if pin:
            self._slots = [s.pin_memory() for s in self._slots]
        self._free = deque(range(depth))
        self._in_flight: deque = deque()              # (uid, slot, handle) in submission order
        self._done: "OrderedDict[str, np.ndarray]" = OrderedDict()
        self._ids = itertools.count()
        self._stopped = False

    def _retire_oldest(self):
        uid, slot, handle = self._in_flight.popleft()
        handle.synchronize()
        self._done[uid] = self._slots[slot].numpy().copy()
        self._free.append(slot)

    def run_batch(self, single_pose) -> str:
        if self._stopped:
            raise RuntimeError("the runner has been stopped")
        if not self._free:
            self._retire_oldest()  # all slots busy: the oldest frame finishes first (bounded frames in flight)
        slot = self._free.popleft()
        uid = f"frame-{next(self._ids)}"
        handle = self.backend.enqueue(single_pose, self._slots[slot])
        self._in_flight.append((uid, slot, handle))
        return uid

    def _poll(self):
        """Move every frame whose work has completed to the done map without blocking."""
        while self._in_flight:
            h = self._in_flight[0][2]
            query = getattr(h, "query", None)
            if query is not None and not query():
                break
            self._retire_oldest()

    def get_result_task(self, block: bool = True) -> ResultTask:
        if not self._done:
            if block and self._in_flight:
                self._retire_oldest()
            else:
                self._poll()
        if not self._done:
            raise Empty
        uid, value = self._done.popitem(last=False)
        return ResultTask(uid, value)

    def get_result(self) -> np.ndarray:
        return self.get_result_task(block=True).value

    def take(self, uid: str) -> Optional[np.ndarray]:
        """The image of ``uid`` if its frame has been submitted and not handed out yet (blocks until
        that frame is complete); ``None`` for an unknown uid."""
        while uid not in self._done and any(u == uid for u, _, _ in self._in_flight):
            self._retire_oldest()
        return self._done.pop(uid, None)

    def stop(self):
        while self._in_flight:
            self._retire_oldest()
        self.backend.finish()
        self.backend.stop()
        self._stopped = True

    def wait_stop(self):
        return None


class MainRankPipeRenderEngine:
    """Rank-0 engine with the reference's asynchronous interface (pipe_engine.py:27-203)."""

    def __init__(self, runner_factory: Callable[[], PipeRunner], poses: Optional[List[np.ndarray]] = None,
                 save_png: bool = False, save_path: str = ".", async_: bool = False, pose_num: int = -1):
        self._factory, self.runner = runner_factory, None
        self.poses, self.save_png, self.save_path, self.pose_num = poses, save_png, save_path, pose_num
        self.async_ = async_
        self.latency: List[float] = []
        self.throughput: Optional[float] = None

    def start(self, test: bool = False):
        self.runner = self._factory()
        if test:
            self.run_test()

    def submit(self, single_pose) -> str:
        return self.runner.run_batch(single_pose)

    def get_result(self) -> np.ndarray:
        return self.runner.get_result()

    def wait(self, uid: str) -> np.ndarray:
        out = self.runner.take(uid)
        if out is None:
            raise KeyError(f"no pending frame with uid {uid!r}")
        return out

    def _collect(self, uid):
        return self.wait(uid) if self.async_ else self.get_result()

    def warm_up(self, pose_num: int = 60):
        if not self.poses:
            return
        for _ in range(pose_num):
            self._collect(self.submit(self.poses[0]))

    def _save(self, idx, image):
        if self.save_png:
            from PIL import Image

            Image.fromarray(image).save(f"{self.save_path}/{idx}.png")

    def run_for_latency(self):
        self.latency = []
        for idx, pose in enumerate((self.poses or [])[:100]):
            t0 = time.time()
            image = self._collect(self.submit(pose))
            self.latency.append(time.time() - t0)
            self._save(idx, image)
        if self.latency:
            print("Latency:", sum(self.latency) / len(self.latency), flush=True)

    def run_for_throughput(self):
        poses = self.poses or []
        t0 = time.time()
        uids = [self.submit(p) for p in poses]
        for idx, uid in enumerate(uids):
            self._save(idx, self._collect(uid))
        total = time.time() - t0
        if poses:
            self.throughput = len(poses) / total
            print("Total time = ", total, flush=True)
            print("Throughput = ", self.throughput, flush=True)

    def run_test(self):
        if self.pose_num > 0 and self.poses:
            self.poses = self.poses[: self.pose_num]
        self.warm_up()
        self.run_for_latency()
        self.stop()

    def stop(self):
        if self.runner is not None:
            self.runner.stop()
            self.runner.wait_stop()
