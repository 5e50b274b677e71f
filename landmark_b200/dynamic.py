"""Rendering a block-partitioned scene that does not fit the GPU: a window of blocks around the
camera is resident, the rest waits in pinned host memory.

The reference's dynamic fetching (dist_render/comm/dynamic_loader.py:91-171,
app/models/gridnerf_elastic_cuda.py:274-303,615-660) keeps the planes of the camera's
neighbourhood on the device in one of two buffers, starts a load thread when the camera crosses a
threshold (``meet_load_threshold``), and switches buffers once the load is done
(``LoadStatus`` Init -> IDLE -> Loading -> LoadDone -> IDLE).  Here the same protocol runs on
streams instead of threads:

* every block of the scene is a pinned host state dict (e.g. from
  ``checkpoints.split_merged_stack``); ``n_slots`` owner models live on the GPU, each holding one
  block (``B200GridNeRF.reload_field_async`` refills a slot on the copy stream without an
  allocation or a device-wide synchronisation);
* the resident window is the ``(2 r + 1)^2`` blocks around the camera's block, clipped to the
  scene; ``update(camera_position)`` is called once per frame: when the camera's block changes it
  enqueues the missing blocks into spare slots (slots whose block is in neither the old nor the
  new window) and records an event; frames keep rendering from the old window; once the event
  has completed the block -> slot map is switched between two frames;
* a sample whose block is not resident has density 0 (it is outside what the window can show), so
  no appearance sample can fall there.

Per chunk the ray owner samples against the global box and occupancy mask, assigns blocks with the
reference's arithmetic (``model_parallel.assign_blocks``), runs the point-mode density and
appearance entries of the slot that holds each block, and composites.
"""

from __future__ import annotations

import enum
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .gridnerf import B200GridNeRF
from .model_parallel import _Chunk, appearance_points, assign_blocks, density_points


class LoadStatus(enum.Enum):
    IDLE = 0
    LOADING = 1
    LOAD_DONE = 2


def window_blocks(center: int, division: Tuple[int, int], radius: int) -> List[int]:
    """Blocks within ``radius`` (Chebyshev) of block ``center``; block b = ix * Py + iy."""
    px, py = division
    cx, cy = divmod(int(center), py)
    return [ix * py + iy for ix in range(max(0, cx - radius), min(px, cx + radius + 1))
            for iy in range(max(0, cy - radius), min(py, cy + radius + 1))]


def pin_block(ckpt: Dict) -> Dict:
    """The planes and lines of a block checkpoint as pinned host tensors."""
    out = {}
    for k, v in ckpt["state_dict"].items():
        if "plane" in k or "line" in k:
            out[k] = v.detach().float().contiguous().cpu().pin_memory()
    return out


class DynamicBlockRenderer:
    def __init__(self, sampler: B200GridNeRF, blocks_host: Sequence[Dict], division: Tuple[int, int],
                 slot_factory: Callable[[int], B200GridNeRF], radius: int = 1, n_slots: Optional[int] = None):
        """``sampler``: a model with the global box, step and occupancy mask (its planes are never read).
        ``blocks_host``: per block, pinned host planes/lines (``pin_block``).
        ``slot_factory(block)``: builds a committed owner model holding ``block`` (used ``n_slots``
        times at start-up; later the slots are only refilled)."""
        px, py = division
        if len(blocks_host) != px * py:
            raise ValueError(f"{len(blocks_host)} blocks for a {px}x{py} division")
        self.sampler, self.blocks_host, self.division, self.radius = sampler, list(blocks_host), (px, py), int(radius)
        self.device = sampler.device
        full = (2 * radius + 1) ** 2
        # spare slots: what one move of the window by one block (also diagonally) can bring in
        self.n_slots = int(n_slots) if n_slots is not None else min(px * py, full + 4 * radius + 1)
        self.load_stream = torch.cuda.Stream(device=self.device)
        self.status = LoadStatus.IDLE
        self.center: Optional[int] = None
        self.block_to_slot: Dict[int, int] = {}
        self.slot_block: List[Optional[int]] = [None] * self.n_slots
        self.slots: List[B200GridNeRF] = []
        self._slot_factory = slot_factory
        self._pending: Dict[int, int] = {}
        self._pending_center: Optional[int] = None
        self._event: Optional[torch.cuda.Event] = None
        self.loads = 0  # blocks fetched from the host so far

    # ---- window management ------------------------------------------------------------------------
    def camera_block(self, position) -> int:
        """Block under the camera: the x/y arithmetic of assign_blocks on the clamped position."""
        p = torch.as_tensor(np.asarray(position, dtype=np.float32)).view(1, 3).to(self.device)
        aabb = self.sampler.aabb
        xyz = ((p - aabb[0]) * self.sampler.invaabbSize - 1).clamp(-1.0, 1.0)
        b, _ = assign_blocks(xyz, self.division)
        return int(b.item())

    def start(self, position) -> "DynamicBlockRenderer":
        """Initial fill (the reference's LoadStatus.Init): creates the slots and loads the first window."""
        c = self.camera_block(position)
        want = window_blocks(c, self.division, self.radius)
        if len(want) > self.n_slots:
            raise ValueError(f"a window of {len(want)} blocks needs more than {self.n_slots} slots")
        fill = want + [b for b in range(len(self.blocks_host)) if b not in want]
        for s in range(self.n_slots):
            b = fill[s % len(fill)]
            self.slots.append(self._slot_factory(b))
            self.slot_block[s] = b
        self.block_to_slot = {b: s for s, b in enumerate(self.slot_block[: len(want)])}
        self.center = c
        torch.cuda.synchronize(self.device)
        return self

    def update(self, position) -> LoadStatus:
        """Once per frame, between two frames.  Returns the status after the call."""
        if self.center is None:
            raise RuntimeError("start() has not been called")
        if self.status is LoadStatus.LOADING and self._event is not None and self._event.query():
            self.status = LoadStatus.LOAD_DONE
        if self.status is LoadStatus.LOAD_DONE:
            # switch: the new blocks become visible, blocks outside the new window give up their slots
            want = set(window_blocks(self._pending_center, self.division, self.radius))
            self.block_to_slot.update(self._pending)
            for b in [b for b in self.block_to_slot if b not in want]:
                del self.block_to_slot[b]
            torch.cuda.current_stream(self.device).wait_event(self._event)
            self.center, self._pending, self._pending_center, self._event = self._pending_center, {}, None, None
            self.status = LoadStatus.IDLE
        if self.status is LoadStatus.IDLE:
            c = self.camera_block(position)
            if c != self.center:  # the load threshold: the camera entered another block
                want = window_blocks(c, self.division, self.radius)
                missing = [b for b in want if b not in self.block_to_slot]
                in_use = set(self.block_to_slot.values())
                free = [s for s in range(self.n_slots) if s not in in_use]
                reuse = {self.slot_block[s]: s for s in free if self.slot_block[s] is not None}
                if len(missing) > len(free):
                    raise RuntimeError(f"{len(missing)} blocks to load but only {len(free)} spare slots")
                self._pending, self._pending_center = {}, c
                # the frames in flight read the resident slots only; the spare ones are refilled behind them
                self.load_stream.wait_stream(torch.cuda.current_stream(self.device))
                for b in missing:
                    if b in reuse:  # still sitting in a spare slot from an earlier window
                        s = reuse[b]
                        free.remove(s)
                    else:
                        s = next(x for x in free if self.slot_block[x] not in missing)
                        free.remove(s)
                        self.slots[s].reload_field_async(self.blocks_host[b], self.load_stream)
                        self.slot_block[s] = b
                        self.loads += 1
                    self._pending[b] = s
                self._event = torch.cuda.Event()
                self._event.record(self.load_stream)
                self.status = LoadStatus.LOADING
        return self.status

    def wait_loaded(self):
        """Block the host until a running load has finished (tests, start-up)."""
        if self._event is not None:
            self._event.synchronize()

    # ---- rendering --------------------------------------------------------------------------------
    @torch.no_grad()
    def render_chunk(self, rays: torch.Tensor, n_samples: int = -1, white_bg: bool = True):
        ch = _Chunk(self.sampler, rays, n_samples)
        ch.sample()
        xyz, ray = ch.positions()
        block, local = assign_blocks(xyz, self.division)
        sigma = torch.zeros(ch.num_valid, dtype=torch.float32, device=self.device)
        present = torch.unique(block).tolist() if ch.num_valid else []
        for b in present:
            s = self.block_to_slot.get(int(b))
            if s is None:
                continue  # not resident: empty space
            idx = (block == b).nonzero(as_tuple=True)[0]
            sigma[idx] = density_points(self.slots[s], local[idx])
        ch.weights(sigma)
        ai = ch.app_index
        rgb_s = torch.zeros((ch.num_app, 3), dtype=torch.float32, device=self.device)
        if ch.num_app:
            a_block, a_local = block[ai], local[ai]
            view = ch.rays[ray[ai], 3:6]
            for b in torch.unique(a_block).tolist():
                s = self.block_to_slot.get(int(b))
                if s is None:
                    continue
                idx = (a_block == b).nonzero(as_tuple=True)[0]
                rgb_s[idx] = appearance_points(self.slots[s], a_local[idx], view[idx])
        return ch.composite(rgb_s, white_bg)

    def render_rays(self, rays: torch.Tensor, n_samples: int = -1, white_bg: bool = True, chunk: int = 65536):
        outs = [self.render_chunk(rays[i:i + chunk], n_samples, white_bg) for i in range(0, rays.shape[0], chunk)]
        return torch.cat([o[0] for o in outs]), torch.cat([o[1] for o in outs])
