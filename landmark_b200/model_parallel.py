"""Renderers that spread ONE field over several GPUs.

Two layouts of the reference are covered, both composed from the library's split-stage and
point-mode entries plus ``torch.distributed`` collectives:

* ``ChannelParallelRenderer`` -- tensor (channel) parallel rendering
  (app/models/gridnerf_tensor_parallel.py:198-217,284-330; dist_render/kernel/cuda_render_extend.py:552-632):
  every rank holds all density planes and a slice of the appearance channels with the matching
  columns of ``basis_mat``.  All ranks sample the same rays; each computes its partial
  ``[M_a, app_dim]`` projection; a reduce-scatter sums them and leaves every rank with the complete
  features of ``M_a / W`` samples, on which it runs the MLP; an all-gather returns the colours.
  (The reference all-gathers the products and sums; reduce-scatter moves W times fewer bytes.)

* ``BlockParallelRenderer`` -- branch (block) parallel rendering
  (app/models/gridnerf_parallel.py:279-338,765-859): the scene is cut into ``Px x Py`` blocks in
  x-y, rank ``b`` owns the field of block ``b``.  Rays are data-parallel (each rank renders its
  own rays); every rank samples its rays against the global box and occupancy mask, assigns each
  valid sample to a block (``assign_blocks_to_samples``), and routes it to the owner with an
  all-to-all.  Owners evaluate density (then, in a second round trip, colour) at the received
  block-local points and send the values back; weights and compositing happen at the ray's rank.
  (The reference replicates the sampling on every rank and all-gathers sigma and rgb.)

Collectives go through a small ``Comm`` interface.  ``DistComm`` is the real thing (one rank per
process).  ``LoopbackComm`` runs all ranks of a group inside one process in lock step, which is how
the multi-rank logic is tested on a single GPU.
"""

from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import check, lib
from .gridnerf import B200GridNeRF, _ptr, _stream


# ----------------------------------------------------------------------------------------------
# collectives
# ----------------------------------------------------------------------------------------------
class DistComm:
    """One rank per process over ``torch.distributed`` (NCCL on GPUs).  Every method takes and
    returns a one-element list: the value of the local rank."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self.dist, self.group = dist, group
        self.world = dist.get_world_size(group)
        self.local_ranks = [dist.get_rank(group)]

    def reduce_scatter_rows(self, xs: List[torch.Tensor]) -> List[torch.Tensor]:
        x = xs[0]
        out = torch.empty((x.shape[0] // self.world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        self.dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        return [out]

    def all_gather_rows(self, xs: List[torch.Tensor]) -> List[torch.Tensor]:
        x = xs[0]
        out = torch.empty((x.shape[0] * self.world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        self.dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return [out]

    def all_to_all_rows(self, xs: List[torch.Tensor], send_counts: List[List[int]]):
        """Rows of ``xs[0]`` are grouped by destination rank (``send_counts[0][d]`` rows for rank d).
        Returns the received rows (grouped by source rank) and the receive counts."""
        x, sc = xs[0], send_counts[0]
        cnt = torch.tensor(sc, dtype=torch.int64, device=x.device)
        rcnt = torch.empty_like(cnt)
        self.dist.all_to_all_single(rcnt, cnt, group=self.group)
        rc = [int(v) for v in rcnt.cpu().tolist()]
        out = torch.empty((sum(rc),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        self.dist.all_to_all_single(out, x.contiguous(), output_split_sizes=rc, input_split_sizes=sc, group=self.group)
        return [out], [rc]


    def all_gather_into(self, xs: List[torch.Tensor], outs: List[torch.Tensor]) -> List[torch.Tensor]:
        """``outs[0]`` (world x the rows of ``xs[0]``) receives every rank's rows, rank r's first row at r * rows."""
        self.dist.all_gather_into_tensor(outs[0], xs[0], group=self.group)
        return outs

    def all_to_all_equal(self, xs: List[torch.Tensor], outs: List[torch.Tensor]) -> List[torch.Tensor]:
        """Equal split: part d of ``xs[0]`` (world equal parts) goes to rank d; ``outs[0]`` holds the parts received,
        by source."""
        self.dist.all_to_all_single(outs[0], xs[0], group=self.group)
        return outs

    def gather_counts(self, cs: List[torch.Tensor]) -> np.ndarray:
        """``cs[0]``: this rank's per-destination counts on the device.  Returns the whole [source, destination]
        matrix on the host; the one host read of an exchange (the device counts are never read on their own)."""
        c = cs[0].to(torch.int64)
        out = torch.empty((self.world * c.numel(),), dtype=torch.int64, device=c.device)
        self.dist.all_gather_into_tensor(out, c.contiguous(), group=self.group)
        return out.view(self.world, c.numel()).cpu().numpy()

    def all_to_all_known(self, xs: List[torch.Tensor], matrix: np.ndarray, outs: List[torch.Tensor]) -> List[torch.Tensor]:
        """Counted all-to-all with the [source, destination] matrix known on every rank: the first
        ``matrix[r].sum()`` rows of ``xs[0]`` go out grouped by destination, the rows for this rank (grouped by
        source) land in the front of ``outs[0]``, whose used part is returned."""
        r = self.local_ranks[0]
        sc, rc = [int(v) for v in matrix[r]], [int(v) for v in matrix[:, r]]
        x, out = xs[0][: sum(sc)], outs[0][: sum(rc)]
        self.dist.all_to_all_single(out, x, output_split_sizes=rc, input_split_sizes=sc, group=self.group)
        return [out]


class LoopbackComm:
    """All ranks of the group live in this process; element ``r`` of every list is rank ``r``'s."""

    def __init__(self, world: int):
        self.world = world
        self.local_ranks = list(range(world))

    def reduce_scatter_rows(self, xs):
        total = xs[0].clone()
        for x in xs[1:]:
            total = total + x
        n = total.shape[0] // self.world
        return [total[r * n:(r + 1) * n].clone() for r in range(self.world)]

    def all_gather_rows(self, xs):
        cat = torch.cat(list(xs), 0)
        return [cat.clone() for _ in range(self.world)]

    def all_to_all_rows(self, xs, send_counts):
        outs, rcs = [], []
        starts = [np.concatenate([[0], np.cumsum(sc)]) for sc in send_counts]
        for d in range(self.world):
            parts = [xs[s][starts[s][d]:starts[s][d + 1]] for s in range(self.world)]
            outs.append(torch.cat(parts, 0))
            rcs.append([int(send_counts[s][d]) for s in range(self.world)])
        return outs, rcs


    def all_gather_into(self, xs, outs):
        n = xs[0].shape[0]
        for out in outs:
            for r, x in enumerate(xs):
                out[r * n:(r + 1) * n] = x
        return outs

    def all_to_all_equal(self, xs, outs):
        n = xs[0].shape[0] // self.world
        for d, out in enumerate(outs):
            for src, x in enumerate(xs):
                out[src * n:(src + 1) * n] = x[d * n:(d + 1) * n]
        return outs

    def gather_counts(self, cs):
        return torch.stack([c.to(torch.int64) for c in cs], 0).cpu().numpy()

    def all_to_all_known(self, xs, matrix, outs):
        starts = np.concatenate([np.zeros((self.world, 1), dtype=np.int64), np.cumsum(matrix, axis=1)], axis=1)
        res = []
        for d in range(self.world):
            at = 0
            for src in range(self.world):
                n = int(matrix[src, d])
                outs[d][at:at + n] = xs[src][int(starts[src, d]):int(starts[src, d]) + n]
                at += n
            res.append(outs[d][:at])
        return res


class SectionTimer:
    """CUDA-event stopwatch for the sections of a model-parallel frame (off unless ``enabled``): ``mark(name)``
    closes the section that started at the previous mark; ``collect()`` returns milliseconds per name."""

    def __init__(self, enabled: bool = False):
        self.enabled, self._events, self._last = enabled, [], None

    def start(self):
        if self.enabled:
            self._last = torch.cuda.Event(enable_timing=True)
            self._last.record()

    def mark(self, name: str):
        if self.enabled and self._last is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._events.append((name, self._last, e))
            self._last = e

    def collect(self) -> Dict[str, float]:
        out: Dict[str, float] = {}
        if self.enabled:
            torch.cuda.synchronize()
            for name, a, b in self._events:
                out[name] = out.get(name, 0.0) + a.elapsed_time(b)
            self._events = []
        return out


# ----------------------------------------------------------------------------------------------
# thin stage wrappers (no output copies, no host syncs except where a count is needed)
# ----------------------------------------------------------------------------------------------
class _Chunk:
    """One model's view of one chunk of rays: workspace + the list sizes read back so far."""

    def __init__(self, model: B200GridNeRF, rays: torch.Tensor, n_samples: int, slot: int = 0):
        self.m = model
        self.rays = model._prepare(rays)
        self.n = self.rays.shape[0]
        self.s = model._samples(n_samples)
        self.keep, self.ws, self.ws_bytes, self.max_valid, self.max_app = model.workspace(self.n, self.s, slot)
        self.kbits = lib.gnr_sample_bits(self.s)
        self.num_valid = self.num_app = 0
        self.ids = self.app_index = None

    def sample(self, keep_ids: bool = True):
        """``keep_ids``: also copy the compacted id list out of the workspace (callers that index it with torch)."""
        self.ids = torch.empty(self.max_valid, dtype=torch.int32, device=self.m.device) if keep_ids else None
        check(lib.gnr_sample(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                             None, None, None, None, _ptr(self.ids), _stream()), "gnr_sample")
        st = self.m.read_status(self.ws)
        self.m.raise_on_status(st)
        self.num_valid = int(st[_lib.ST_NUM_VALID])

    # -- launch-only forms (no host read: the caller reads status and counts together, once per exchange) --
    def launch_sample(self, t_min: Optional[torch.Tensor] = None):
        """``t_min``: also copy the rays' entry distances out (``[n]``; a block owner recomputes positions from them)."""
        check(lib.gnr_sample(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                             _ptr(t_min), None, None, None, None, _stream()), "gnr_sample")

    def launch_route_ids(self, which_list: int, division: Tuple[int, int], ray_base: int, send_ids: torch.Tensor,
                         dest: torch.Tensor, counts: torch.Tensor):
        """gnr_route_block_ids: like ``launch_route`` with one 32-bit id per row instead of the point."""
        counts.zero_()
        check(lib.gnr_route_block_ids(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                                      self.max_app, which_list, division[0], division[1], int(ray_base), _ptr(send_ids),
                                      _ptr(dest), _ptr(counts), _stream()), "gnr_route_block_ids")

    def launch_route(self, which_list: int, division: Tuple[int, int], send: torch.Tensor, dest: torch.Tensor,
                     counts: torch.Tensor):
        """gnr_route_blocks into caller-held buffers of list capacity; the list length is read on the device."""
        counts.zero_()
        check(lib.gnr_route_blocks(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                                   self.max_app, which_list, division[0], division[1], _ptr(send), _ptr(dest),
                                   _ptr(counts), None, _stream()), "gnr_route_blocks")

    def launch_weights(self, sigma_back: torch.Tensor, dest: torch.Tensor):
        """Weights and the appearance list from the owners' answers, read in place (send-buffer order) through the row
        every list entry went to."""
        if sigma_back.numel() == 0:  # no valid sample in this chunk (an empty view has no address): nothing will be read
            sigma_back = torch.zeros(1, dtype=torch.float32, device=self.m.device)
        check(lib.gnr_weights_from_rows(self.m._handle, self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                                        self.max_app, _ptr(sigma_back), _ptr(dest), _stream()), "gnr_weights_from_rows")

    def launch_march(self):
        check(lib.gnr_march(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                            self.max_app, None, None, None, None, None, None, _stream()), "gnr_march")

    def checked_status(self):
        st = self.m.read_status(self.ws)
        self.m.raise_on_status(st)
        self.num_valid, self.num_app = int(st[_lib.ST_NUM_VALID]), int(st[_lib.ST_NUM_APP])
        return st

    def density(self):
        check(lib.gnr_density(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                              None, None, _stream()), "gnr_density")

    def march(self):
        """Density + weights + appearance compaction in the fused pass (a field held whole by this model)."""
        self.app_index = torch.empty(self.max_app, dtype=torch.int32, device=self.m.device)
        check(lib.gnr_march(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                            self.max_app, None, None, None, None, None, _ptr(self.app_index), _stream()), "gnr_march")
        st = self.m.read_status(self.ws)
        self.m.raise_on_status(st)
        self.num_app = int(st[_lib.ST_NUM_APP])
        self.app_index = self.app_index[: self.num_app].to(torch.int64)

    def positions(self):
        xyz = torch.empty((self.max_valid, 3), dtype=torch.float32, device=self.m.device)
        ray = torch.empty((self.max_valid,), dtype=torch.int32, device=self.m.device)
        check(lib.gnr_valid_positions(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes,
                                      self.max_valid, _ptr(xyz), _ptr(ray), _stream()), "gnr_valid_positions")
        return xyz[: self.num_valid], ray[: self.num_valid].to(torch.int64)

    def route(self, which_list: int, division: Tuple[int, int]):
        """Block assignment + grouping by owner of the valid list (``which_list`` 0) or the appearance list
        (1) in one library call (gnr_route_blocks).  Returns the send buffer (block-local points, with view
        directions for the appearance list, grouped by block), the row every list entry went to, and the
        per-block counts (the only host read of the exchange)."""
        n_items = self.num_valid if which_list == 0 else self.num_app
        dev = self.m.device
        send = torch.empty((max(n_items, 1), 3 if which_list == 0 else 6), dtype=torch.float32, device=dev)
        dest = torch.empty((max(n_items, 1),), dtype=torch.int32, device=dev)
        counts = torch.zeros((division[0] * division[1],), dtype=torch.int32, device=dev)
        if n_items:
            check(lib.gnr_route_blocks(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                                       self.max_app, which_list, division[0], division[1], _ptr(send), _ptr(dest),
                                       _ptr(counts), None, _stream()), "gnr_route_blocks")
        return send[:n_items], dest[:n_items], [int(v) for v in counts.cpu().tolist()]

    def weights(self, sigma: Optional[torch.Tensor] = None, sigma_rows: Optional[torch.Tensor] = None):
        """``sigma``: one value per valid sample in list order, or, with ``sigma_rows``, the owners' answers
        in send-buffer order plus the row of every list entry (gathered here, no intermediate copy)."""
        self.app_index = torch.empty(self.max_app, dtype=torch.int32, device=self.m.device)
        if sigma is not None and sigma_rows is not None:
            full = torch.empty(self.max_valid, dtype=torch.float32, device=self.m.device)  # entries past num_valid are never read
            if self.num_valid:
                torch.index_select(sigma, 0, sigma_rows, out=full[: self.num_valid])
            check(lib.gnr_weights_from_sigma(self.m._handle, self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                                             self.max_app, _ptr(full), _ptr(self.app_index), _stream()),
                  "gnr_weights_from_sigma")
        elif sigma is None:
            check(lib.gnr_weights(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                                  self.max_app, None, None, None, None, None, _ptr(self.app_index), _stream()),
                  "gnr_weights")
        else:
            full = torch.zeros(self.max_valid, dtype=torch.float32, device=self.m.device)
            full[: self.num_valid] = sigma
            check(lib.gnr_weights_from_sigma(self.m._handle, self.n, self.s, self.ws, self.ws_bytes, self.max_valid,
                                             self.max_app, _ptr(full), _ptr(self.app_index), _stream()),
                  "gnr_weights_from_sigma")
        st = self.m.read_status(self.ws)
        self.m.raise_on_status(st)
        self.num_app = int(st[_lib.ST_NUM_APP])
        self.app_index = self.app_index[: self.num_app].to(torch.int64)

    def app_ray_index(self) -> torch.Tensor:
        ids = self.ids[: self.num_valid].to(torch.int64) & 0xFFFFFFFF
        return (ids[self.app_index] >> self.kbits)

    def app_features(self) -> torch.Tensor:
        feat = torch.empty((self.num_app, self.m.app_dim), dtype=torch.float32, device=self.m.device)
        if self.num_app:
            check(lib.gnr_app_features(self.m._handle, _ptr(self.rays), self.n, self.s, self.ws, self.ws_bytes,
                                       self.max_valid, self.max_app, _ptr(feat), self.num_app, _stream()), "gnr_app_features")
        return feat

    def composite(self, rgb_samples: torch.Tensor, white_bg: bool):
        rgb = torch.empty((self.n, 3), dtype=torch.float32, device=self.m.device)
        depth = torch.empty((self.n,), dtype=torch.float32, device=self.m.device)
        rgb_samples = rgb_samples.contiguous()
        check(lib.gnr_composite_rgb(self.m._handle, self.n, int(bool(white_bg)), self.ws, self.ws_bytes, self.max_valid,
                                    self.max_app, self.s, _ptr(rgb_samples) if rgb_samples.numel() else None,
                                    rgb_samples.shape[0], _ptr(rgb), _ptr(depth), _stream()), "gnr_composite_rgb")
        return rgb, depth


def _scratch(model: B200GridNeRF, n: int, lane: int = 0):
    """Scratch of the point-mode entries, kept on the model (one per lane: calls of different lanes may be in
    flight on different streams) and only ever grown: calls on one stream reuse it in order, so no call has
    to wait for the previous one."""
    nb = C.c_size_t(0)
    check(lib.gnr_points_scratch_bytes(model._handle, n, C.byref(nb)), "gnr_points_scratch_bytes")
    store = model.__dict__.setdefault("_point_scratch", {})
    buf = store.get(lane)
    if buf is None or buf.numel() < nb.value + 256:
        if buf is not None:
            torch.cuda.synchronize(model.device)  # kernels may still be using the smaller buffer
        buf = torch.empty(int(nb.value * 1.25) + 256, dtype=torch.uint8, device=model.device)
        store[lane] = buf
    off = (-buf.data_ptr()) % 256
    return buf, C.c_void_p(buf.data_ptr() + off), buf.numel() - off


def mlp_features(model: B200GridNeRF, feats: torch.Tensor, view: torch.Tensor, lane: int = 0) -> torch.Tensor:
    n = feats.shape[0]
    rgb = torch.empty((n, 3), dtype=torch.float32, device=model.device)
    if n == 0:
        return rgb
    keep, sc, nb = _scratch(model, n, lane)
    feats, view = feats.contiguous(), view.contiguous()
    with torch.cuda.device(model.device):
        check(lib.gnr_mlp_features(model._handle, _ptr(feats), _ptr(view), n, sc, nb, _ptr(rgb), _stream()), "gnr_mlp_features")
    return rgb


def app_features_points(model: B200GridNeRF, xyz: torch.Tensor) -> torch.Tensor:
    """Partial (or complete) basis projection of this model's appearance channels at explicit points."""
    n = xyz.shape[0]
    feat = torch.empty((n, model.app_dim), dtype=torch.float32, device=model.device)
    if n == 0:
        return feat
    keep, sc, nb = _scratch(model, n)
    xyz = xyz.contiguous()
    with torch.cuda.device(model.device):
        check(lib.gnr_app_features_points(model._handle, _ptr(xyz), n, sc, nb, _ptr(feat), _stream()), "gnr_app_features_points")
    return feat


def density_points(model: B200GridNeRF, xyz: torch.Tensor) -> torch.Tensor:
    n = xyz.shape[0]
    sigma = torch.empty((n,), dtype=torch.float32, device=model.device)
    if n:
        xyz = xyz.contiguous()
        with torch.cuda.device(model.device):
            check(lib.gnr_density_points(model._handle, _ptr(xyz), n, None, _ptr(sigma), _stream()), "gnr_density_points")
    return sigma


def appearance_points(model: B200GridNeRF, xyz: torch.Tensor, view: torch.Tensor) -> torch.Tensor:
    n = xyz.shape[0]
    rgb = torch.empty((n, 3), dtype=torch.float32, device=model.device)
    if n == 0:
        return rgb
    keep, sc, nb = _scratch(model, n)
    xyz, view = xyz.contiguous(), view.contiguous()
    with torch.cuda.device(model.device):
        check(lib.gnr_appearance_points(model._handle, _ptr(xyz), _ptr(view), n, sc, nb, None, _ptr(rgb), _stream()),
              "gnr_appearance_points")
    return rgb


# ----------------------------------------------------------------------------------------------
# channel (tensor) parallel
# ----------------------------------------------------------------------------------------------
def slice_checkpoint_channels(ckpt: Dict, rank: int, world: int) -> Dict:
    """The checkpoint of tensor-parallel rank ``rank``: density untouched, appearance planes and
    lines chunked on the channel dimension (inferer_impl.py:259-261), ``basis_mat.weight`` viewed as
    ``[app_dim, pairs, C]`` and sliced on ``C`` (cuda_render_extend.py:552-562)."""
    sd = dict(ckpt["state_dict"])
    n_pairs = sum(1 for k in sd if k.startswith("app_plane."))
    c_full = sd["app_plane.0"].shape[1]
    if c_full % world:
        raise ValueError(f"{c_full} appearance channels do not split over {world} ranks")
    c = c_full // world
    for i in range(n_pairs):
        sd[f"app_plane.{i}"] = sd[f"app_plane.{i}"][:, rank * c:(rank + 1) * c].contiguous()
        sd[f"app_line.{i}"] = sd[f"app_line.{i}"][:, rank * c:(rank + 1) * c].contiguous()
    w = sd["basis_mat.weight"]
    sd["basis_mat.weight"] = w.view(w.shape[0], n_pairs, c_full)[:, :, rank * c:(rank + 1) * c].reshape(w.shape[0], -1).contiguous()
    out = dict(ckpt)
    out["state_dict"] = sd
    kw = dict(ckpt["kwargs"])
    kw["appearance_n_comp"] = [c] * len(kw["appearance_n_comp"])
    out["kwargs"] = kw
    return out


def _run_lanes(make_steps, n_chunks: int, lanes: int, device, streams: Dict[tuple, "torch.cuda.Stream"], steps_per_turn: int):
    """Drive ``n_chunks`` step generators (``make_steps(chunk, lane, result_list)``) with up to ``lanes`` of them in
    flight, each on its own CUDA stream; a lane's turn is ``steps_per_turn`` steps (one that ends in a host read and
    the launches that follow it), then the next lane's turn: while the host waits for one lane's read the GPU has
    the other lanes' queued work, and a lane's collectives (NCCL's stream) run beside the other lanes' kernels.
    Every rank of a group must call this with the same ``n_chunks`` and ``lanes`` (the collectives interleave in
    the same order).  Returns the result list of every chunk."""
    results = [[] for _ in range(n_chunks)]
    if n_chunks == 0:
        return results
    cur = torch.cuda.current_stream(device)
    lanes = max(1, min(lanes, n_chunks))
    lane_streams = []
    for l in range(lanes):
        key = (l, str(device))
        if key not in streams:
            streams[key] = torch.cuda.Stream(device=device)
        streams[key].wait_stream(cur)
        lane_streams.append(streams[key])
    gens = [None] * lanes
    nxt = 0
    active = True
    while active:
        active = False
        for l in range(lanes):
            if gens[l] is None and nxt < n_chunks:
                gens[l] = make_steps(nxt, l, results[nxt])
                nxt += 1
            if gens[l] is not None:
                with torch.cuda.stream(lane_streams[l]):
                    for _ in range(steps_per_turn):
                        try:
                            next(gens[l])
                        except StopIteration:
                            gens[l] = None
                            break
                active = True
        active = active or nxt < n_chunks
    for st in lane_streams:
        cur.wait_stream(st)
    for per_chunk in results:  # made on a lane's stream, read by the caller on the current one
        for rgb, depth in per_chunk:
            rgb.record_stream(cur)
            depth.record_stream(cur)
    return results


class ChannelParallelRenderer:
    """``models[i]`` is the channel-sliced model of ``comm.local_ranks[i]``."""

    def __init__(self, models: Sequence[B200GridNeRF], comm):
        assert len(models) == len(comm.local_ranks)
        self.models, self.comm = list(models), comm
        self.timer = SectionTimer(False)

    RAY_GROUP = 1024  # rays are dealt to the ranks in groups of this many consecutive rays

    def _ray_share(self, n: int, rank: int, device) -> torch.Tensor:
        """Indices of the rays of a chunk that ``rank`` samples: groups of RAY_GROUP consecutive rays dealt
        round-robin (consecutive rays are neighbouring pixels: a group keeps the kernels' locality, the
        round-robin balances sky against ground)."""
        key = (n, rank, str(device))
        cache = self.__dict__.setdefault("_shares", {})
        if key not in cache:  # (boolean indexing reads a count back: once per chunk size, not once per chunk)
            if len(cache) > 64:
                cache.clear()
            idx = torch.arange(n, device=device)
            cache[key] = idx[(idx // self.RAY_GROUP) % self.comm.world == rank]
        return cache[key]

    def _buf(self, i, name: str, rows: int, cols: int, dtype, device) -> torch.Tensor:
        """Grow-only buffer ``name`` of (lane, local rank) ``i``, at least [rows, cols] (flat when cols == 0)."""
        key = (i, name)
        need = max(rows, 1) * max(cols, 1)
        store = self.__dict__.setdefault("_bufs", {})
        buf = store.get(key)
        if buf is None or buf.numel() < need:
            if buf is not None:
                torch.cuda.synchronize(device)
            buf = torch.zeros(int(need * 1.25) + 16, dtype=dtype, device=device)
            store[key] = buf
        return buf[:need].view(max(rows, 1), cols) if cols else buf[:need]

    def _fp16_exchange(self) -> bool:
        """The tensor-core form of the exchange: fp16 appearance planes and the single-fp16 MLP on every rank."""
        return all(m.mlp_mode == 2 and m.app_plane_fp16 and m.ert_transmittance >= 0.0 for m in self.models)

    @torch.no_grad()
    def render_chunk(self, rays: Sequence[torch.Tensor], n_samples: int = -1, white_bg: bool = True):
        """``rays[i]``: the same chunk on each local rank's device.  Returns per local rank ``(rgb_map, depth_map)``;
        all ranks end up with the full result.  With fp16 appearance planes and mlp_mode 2 on every rank the
        partial projections are computed on the tensor cores and travel as fp16 (``_render_chunk_fp16``); otherwise
        they are fp32 rows summed by a reduce-scatter (``_render_chunk_fp32``)."""
        if self._fp16_exchange():
            self.timer.start()
            out: list = []
            for _ in self._steps_fp16(rays, n_samples, white_bg, 0, out):
                pass
            return out
        return self._render_chunk_fp32(rays, n_samples, white_bg)

    @torch.no_grad()
    def render_frame(self, chunk_list: Sequence[Sequence[torch.Tensor]], n_samples: int = -1, white_bg: bool = True,
                     lanes: int = 2):
        """``chunk_list[c][i]``: chunk c on local rank i's device.  With the fp16 exchange two chunks are in flight on two
        streams (a chunk has one host read, the list lengths, then only launches and collectives); returns per chunk
        what ``render_chunk`` returns."""
        if not self._fp16_exchange():
            return [self.render_chunk(c, n_samples, white_bg) for c in chunk_list]
        self.timer.start()
        self.samples = {"valid": 0, "app": 0}  # list lengths of the local ranks' shares since this call began
        streams = self.__dict__.setdefault("_streams", {})
        return _run_lanes(lambda c, lane, out: self._steps_fp16(chunk_list[c], n_samples, white_bg, lane, out), len(chunk_list),
                          lanes, self.models[0].device, streams, 2)

    def _steps_fp16(self, rays, n_samples, white_bg, lane, result):
        """Every rank samples and marches ITS share of the rays (one host read: the list lengths); the positions of
        all appearance samples are all-gathered (12 bytes each); every rank projects all of them through its channel
        slice on the tensor cores (``gnr_project_slice_points``: products from registers into tensor memory, one
        small GEMM, fp16 rows of 64 bytes); an all-to-all hands every rank the W partial rows of its OWN samples,
        which it sums in fp32 (``gnr_sum_partials``), runs through the MLP (``gnr_mlp_features``, the one-kernel
        form on given features) and composites; the pixels are all-gathered.  Against the fp32 form: half the
        bytes on the wire, no fp32 feature rows in memory, and the sum over the ranks in fp32 at the receiver."""
        W = self.comm.world
        tm = self.timer
        tm.start()
        chunks, shares, rows6 = [], [], []
        for i, (m, r, rank) in enumerate(zip(self.models, rays, self.comm.local_ranks)):
            with torch.cuda.device(m.device):
                share = self._ray_share(r.shape[0], rank, m.device)
                mine = r[share] if share.numel() else r[:1]  # a rank without rays still takes part in the collectives
                ch = _Chunk(m, mine, n_samples, slot=lane)
                ch.launch_sample()
                ch.launch_march()
                tm.mark("sample + march (own rays)")
                pts = self._buf((lane, i), "rows6", ch.max_app, 6, torch.float32, m.device)
                dest = self._buf((lane, i), "dest", ch.max_app, 0, torch.int32, m.device)
                cnt = self._buf((lane, i), "cnt", 1, 0, torch.int32, m.device)
                ch.launch_route(1, (1, 1), pts, dest, cnt)  # one block: the appearance list as (point, view) rows in list order
                tm.mark("appearance points")
                chunks.append(ch)
                shares.append(share)
                rows6.append(pts)
        counts = self.comm.gather_counts([self._buf((lane, i), "cnt", 1, 0, torch.int32, ch.m.device) for i, ch in enumerate(chunks)])
        for ch in chunks:
            with torch.cuda.device(ch.m.device):
                ch.checked_status()
        per = max(1, int(counts.max()))  # rows per rank in the gathered list (padded to the largest)
        tm.mark("counts")
        tally = self.__dict__.setdefault("samples", {"valid": 0, "app": 0})
        tally["valid"] += sum(ch.num_valid for ch in chunks)
        tally["app"] += sum(ch.num_app for ch in chunks)
        yield
        own_xyz, all_xyz = [], []
        for i, (ch, pts) in enumerate(zip(chunks, rows6)):
            with torch.cuda.device(ch.m.device):
                x = self._buf((lane, i), "xyz_own", per, 3, torch.float32, ch.m.device)
                x[: ch.num_app] = pts[: ch.num_app, :3]  # (rows past the list keep older positions: any point will do)
                own_xyz.append(x)
                all_xyz.append(self._buf((lane, i), "xyz_all", W * per, 3, torch.float32, ch.m.device))
        self.comm.all_gather_into(own_xyz, all_xyz)
        tm.mark("all-gather points")
        parts = []
        for i, (ch, allp) in enumerate(zip(chunks, all_xyz)):
            with torch.cuda.device(ch.m.device):
                part = self._buf((lane, i), "part_h", W * per, 32, torch.float16, ch.m.device)
                st = self._buf((lane, i), "slice_status", 8, 0, torch.int32, ch.m.device)
                check(lib.gnr_project_slice_points(ch.m._handle, _ptr(allp), 3, W * per, _ptr(part), _ptr(st), _stream()),
                      "gnr_project_slice_points")
                parts.append(part)
        tm.mark("partial projection (all points)")
        recvs = [self._buf((lane, i), "recv_h", W * per, 32, torch.float16, ch.m.device) for i, ch in enumerate(chunks)]
        self.comm.all_to_all_equal(parts, recvs)
        tm.mark("all-to-all of fp16 partial rows")
        pix = []
        for i, (ch, recv, pts) in enumerate(zip(chunks, recvs, rows6)):
            with torch.cuda.device(ch.m.device):
                na = ch.num_app
                rgb_s = self._buf((lane, i), "rgb_list", na, 3, torch.float32, ch.m.device)[:na]
                if na:  # the W partial rows of every own sample are summed inside the MLP kernel
                    keep, sc, nbytes = _scratch(ch.m, na, lane)
                    check(lib.gnr_mlp_partial_rows(ch.m._handle, _ptr(recv), W, per, _ptr(pts), na, sc, nbytes, _ptr(rgb_s),
                                                   _stream()), "gnr_mlp_partial_rows")
                pix.append(ch.composite(rgb_s, white_bg))
        tm.mark("sum + MLP + composite (own rays)")
        result.extend(self._gather_pixels(rays, chunks, shares, pix, lane))

    def _pixel_source(self, n: int, device):
        """For a chunk of ``n`` rays: rows per rank in the gathered pixel list, and for every ray the row that holds
        it (rank r's share starts at row r * per_rays; inside a share the rays keep their order)."""
        key = ("pix", n, str(device))
        cache = self.__dict__.setdefault("_shares", {})
        if key not in cache:
            W, G = self.comm.world, self.RAY_GROUP
            j = torch.arange(n, device=device)
            group = j // G
            n_groups = -(-n // G)
            # a rank's share: its full groups, and the last (possibly short) group if that one is its own
            sizes = [sum(min(G, n - g * G) for g in range(r, n_groups, W)) for r in range(W)]
            per_rays = max(1, max(sizes))
            cache[key] = (per_rays, (group % W) * per_rays + (group // W) * G + j % G)
        return cache[key]

    def _gather_pixels(self, rays, chunks, shares, pix, lane: int = 0):
        """Pixels of every rank -> every rank: one all-gather of (rgb, depth) rows padded to the largest share, one
        indexed read that puts them back in ray order."""
        W = self.comm.world
        n = rays[0].shape[0]
        packed, gathered, sources = [], [], []
        for i, (ch, share, (rgb, depth)) in enumerate(zip(chunks, shares, pix)):
            with torch.cuda.device(ch.m.device):
                per_rays, src = self._pixel_source(n, ch.m.device)
                buf = self._buf((lane, i), "pix_own", per_rays, 4, torch.float32, ch.m.device)
                k = share.numel()
                buf[:k, :3] = rgb[:k]
                buf[:k, 3] = depth[:k]
                packed.append(buf)
                gathered.append(self._buf((lane, i), "pix_all", W * per_rays, 4, torch.float32, ch.m.device))
                sources.append(src)
        self.comm.all_gather_into(packed, gathered)
        out = []
        for ch, g, src in zip(chunks, gathered, sources):
            with torch.cuda.device(ch.m.device):
                sel = torch.index_select(g, 0, src)
                out.append((sel[:, :3].contiguous(), sel[:, 3].contiguous()))
        self.timer.mark("all-gather pixels")
        return out

    def _render_chunk_fp32(self, rays: Sequence[torch.Tensor], n_samples: int = -1, white_bg: bool = True):
        """The fp32 form of the exchange (any precision mode of the models).

        Work split (app/models/gridnerf_tensor_parallel.py:198-217,284-330 divides the density work and the
        samples over the group as well): every rank samples and marches only ITS share of the rays; the
        appearance points of all ranks are all-gathered (24 bytes each); every rank projects all of them
        through its channel slice; the reduce-scatter hands each rank the complete features of its OWN
        points, on which it runs the MLP and composites its own rays; the pixels are all-gathered."""
        W = self.comm.world
        chunks, shares, points = [], [], []
        tm = self.timer
        tm.start()
        for m, r, rank in zip(self.models, rays, self.comm.local_ranks):
            with torch.cuda.device(m.device):
                share = self._ray_share(r.shape[0], rank, m.device)
                mine = r[share] if share.numel() else r[:1]  # a rank without rays still takes part in the collectives
                ch = _Chunk(m, mine, n_samples)
                ch.sample(keep_ids=False)
                if m.ert_transmittance >= 0.0:
                    ch.march()  # the fused pass of the single-GPU renderer
                else:
                    ch.density()
                    ch.weights()
                tm.mark("sample + march (own rays)")
                pts, _, _ = ch.route(1, (1, 1))  # one block: the appearance list as (point, view) rows in list order
                tm.mark("appearance points")
                chunks.append(ch)
                shares.append(share)
                points.append(pts)
        counts = self.comm.all_gather_rows([torch.tensor([ch.num_app], dtype=torch.int64, device=ch.m.device) for ch in chunks])
        per = max(1, int(counts[0].max().item()))  # rows per rank in the gathered list (padded to the largest)
        padded = []
        for ch, pts in zip(chunks, points):
            with torch.cuda.device(ch.m.device):
                buf = torch.zeros((per, 6), dtype=torch.float32, device=ch.m.device)
                buf[: ch.num_app] = pts
                padded.append(buf)
        everyone = self.comm.all_gather_rows(padded)  # [W * per, 6], rank r's points in rows r * per ..
        tm.mark("all-gather points")
        partial = []
        for ch, allp in zip(chunks, everyone):
            with torch.cuda.device(ch.m.device):
                partial.append(app_features_points(ch.m, allp[:, :3].contiguous()))
        tm.mark("partial projection (all points)")
        feats = self.comm.reduce_scatter_rows(partial)  # [per, app_dim]: the complete features of this rank's own points
        tm.mark("reduce-scatter features")
        pix = []
        for ch, share, f, pts in zip(chunks, shares, feats, points):
            with torch.cuda.device(ch.m.device):
                rgb_s = mlp_features(ch.m, f[: ch.num_app], pts[:, 3:6].contiguous())
                rgb, depth = ch.composite(rgb_s, white_bg)
                pix.append((rgb, depth))
        tm.mark("MLP + composite (own rays)")
        return self._gather_pixels(rays, chunks, shares, pix)


# ----------------------------------------------------------------------------------------------
# block (branch) parallel
# ----------------------------------------------------------------------------------------------
def assign_blocks(xyz: torch.Tensor, division: Tuple[int, int]):
    """Block index and block-local coordinates of normalised samples; the arithmetic of
    ``assign_blocks_to_samples`` (app/models/gridnerf_parallel.py:296-327) with torch ops in the
    same order.  A sample exactly on the upper face of the box (x or y == 1) is given to the last
    block instead of an out-of-range index."""
    px, py = division
    pw, ph = 2 / px, 2 / py
    t = xyz[:, :2] + 1
    u, v = t[:, 0] / pw, t[:, 1] / ph
    bx = torch.floor(u).clamp_(0, px - 1)
    by = torch.floor(v).clamp_(0, py - 1)
    b = bx * py + by
    coord_min = torch.stack([-1 + (b // py) * pw, -1 + (b % py) * ph], dim=-1)
    coord_max = torch.stack([-1 + (b // py + 1) * pw, -1 + (b % py + 1) * ph], dim=-1)
    local = xyz.clone()
    local[:, :2] = (xyz[:, :2] - coord_min) * 2 / (coord_max - coord_min) - 1
    return b.to(torch.int64), local


def _route(owner: torch.Tensor, world: int):
    """Stable grouping of the samples by owner: ``order`` lists the sample indices owner by owner,
    ``counts[d]`` how many go to rank ``d``.  A handful of owners: one compaction per owner beats a
    radix sort plus an atomics histogram (one bin takes most samples when a camera looks at one block)."""
    if world > 16:
        order = torch.argsort(owner, stable=True)
        return order, [int(c) for c in torch.bincount(owner, minlength=world).cpu().tolist()]
    parts = [(owner == d).nonzero(as_tuple=True)[0] for d in range(world)]
    return (torch.cat(parts) if world > 1 else parts[0]), [int(p.numel()) for p in parts]


class BlockParallelRenderer:
    """``samplers[i]``: a model carrying the global box, step size and occupancy mask (its planes
    are never read); ``owners[i]``: the field of the block that ``comm.local_ranks[i]`` owns.
    Block ``b`` lives on rank ``b``; ``division[0] * division[1]`` must equal the world size.

    A chunk goes through four steps, two of which end in the only host reads of the chunk (status + the
    [source, destination] count matrix of an exchange, one synchronisation each):

      1. sample, route the valid list by owner (``gnr_route_blocks``), gather the counts             [host read]
      2. all-to-all of the points, density at the owners, all-to-all of sigma back                      [no read]
      3. weights + appearance list, route it by owner, gather the counts                             [host read]
      4. all-to-all of (point, view) rows, colour at the owners, all-to-all back, composite            [no read]

    ``render_frame`` keeps two chunks in flight on two streams (lanes), alternating (1, 2) of one with (3, 4)
    of the other: while the host waits for one lane's counts, the GPU runs the other lane's exchange and
    owner-side kernels, and a lane's all-to-all (NCCL's stream) overlaps the other lane's kernels.  Every
    buffer of a lane is kept and only grown, so a frame allocates nothing after the first."""

    def __init__(self, samplers: Sequence[B200GridNeRF], owners: Sequence[B200GridNeRF], comm, division: Tuple[int, int]):
        if division[0] * division[1] != comm.world:
            raise ValueError(f"{division[0]}x{division[1]} blocks need {division[0] * division[1]} ranks, have {comm.world}")
        self.samplers, self.owners, self.comm, self.division = list(samplers), list(owners), comm, division
        self.timer = SectionTimer(False)  # set ``timer.enabled`` to get a per-section breakdown of a frame
        self._bufs: Dict[tuple, torch.Tensor] = {}
        self._streams: Dict[tuple, torch.cuda.Stream] = {}
        self.samples = {"valid": 0, "app": 0}  # list lengths of the local ranks' chunks since the last render_frame began
        # ids instead of points on the wire whenever the owners can evaluate colour from the ray (set False to force points)
        self.ship_ids = self.ships_ids()

    def _buf(self, lane: int, i: int, name: str, rows: int, cols: int, dtype, device) -> torch.Tensor:
        """Grow-only buffer ``name`` of lane ``lane`` and local rank ``i``, at least [rows, cols] (flat when cols == 0)."""
        key = (lane, i, name)
        need = max(rows, 1) * max(cols, 1)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < need:
            if buf is not None:
                torch.cuda.synchronize(device)  # kernels of this lane may still be using the smaller one
            buf = torch.empty(int(need * 1.25) + 16, dtype=dtype, device=device)
            self._bufs[key] = buf
        return buf[:need].view(max(rows, 1), cols) if cols else buf[:need]

    def ships_ids(self) -> bool:
        """True if the exchange can ship ids instead of points: every local owner runs the one-kernel appearance path
        (it evaluates colour in list mode, from the ray) -- all ranks of a group must be configured alike."""
        return all(bool(lib.gnr_query_one_kernel_appearance(o._handle)) for o in self.owners)

    def _agree_ray_capacity(self, n_local_max: int) -> int:
        """Rows per rank in the chunk's table of rays (the largest chunk of any rank), agreed once per call."""
        dev = self.samplers[0].device
        m = self.comm.gather_counts([torch.tensor([n_local_max], dtype=torch.int32, device=s_.device) for s_ in self.samplers])
        return max(1, int(m.max()))

    def _steps_ids(self, rays: Sequence[torch.Tensor], n_samples: int, white_bg: bool, lane: int, result: list, cap: int):
        """The four steps with ids on the wire: a valid sample travels as 4 bytes (ray << bits | sample) instead of 12,
        an appearance sample as 4 instead of 24; every rank's rays and entry distances of the chunk are all-gathered
        (28 bytes per ray) and the owners recompute the positions (``gnr_density_list`` / ``gnr_appearance_list``)."""
        tm, div, nb, W = self.timer, self.division, self.comm.world, self.comm.world
        chunks, sends, dests, cnts, rays_pad, tmins = [], [], [], [], [], []
        for i, (s_, r, rank) in enumerate(zip(self.samplers, rays, self.comm.local_ranks)):
            with torch.cuda.device(s_.device):
                ch = _Chunk(s_, r, n_samples, slot=lane)
                if ch.n > cap:
                    raise ValueError(f"a chunk of {ch.n} rays exceeds the agreed ray capacity {cap}")
                rp = self._buf(lane, i, "rays_pad", cap, 6, torch.float32, s_.device)
                rp[: ch.n] = ch.rays
                tmn = self._buf(lane, i, "tmin_own", cap, 0, torch.float32, s_.device)
                ch.launch_sample(tmn)
                tm.mark("sample")
                send = self._buf(lane, i, "send_ids", ch.max_valid, 0, torch.int32, s_.device)
                dest = self._buf(lane, i, "dest", ch.max_valid, 0, torch.int32, s_.device)
                cnt = self._buf(lane, i, "cnt", nb, 0, torch.int32, s_.device)
                ch.launch_route_ids(0, div, rank * cap, send, dest, cnt)
                tm.mark("route valid")
                chunks.append(ch)
                sends.append(send)
                dests.append(dest)
                cnts.append(cnt)
                rays_pad.append(rp)
                tmins.append(tmn)
        matrix = self.comm.gather_counts(cnts)
        for ch in chunks:
            with torch.cuda.device(ch.m.device):
                ch.checked_status()
        tm.mark("counts of the valid lists")
        yield
        rays_all = self.comm.all_gather_into(rays_pad, [self._buf(lane, i, "rays_all", W * cap, 6, torch.float32, o.device)
                                                        for i, o in enumerate(self.owners)])
        tmin_all = self.comm.all_gather_into(tmins, [self._buf(lane, i, "tmin_all", W * cap, 0, torch.float32, o.device)
                                                     for i, o in enumerate(self.owners)])
        tm.mark("all-gather rays")
        n_in = [int(matrix[:, r].sum()) for r in self.comm.local_ranks]
        recv = self.comm.all_to_all_known(sends, matrix, [self._buf(lane, i, "recv_ids", n, 0, torch.int32, o.device)
                                                          for i, (o, n) in enumerate(zip(self.owners, n_in))])
        tm.mark("all-to-all ids")
        sig = []
        for i, (o, s_, x, rank) in enumerate(zip(self.owners, self.samplers, recv, self.comm.local_ranks)):
            out = self._buf(lane, i, "sigma", x.shape[0], 0, torch.float32, o.device)
            if x.shape[0]:
                with torch.cuda.device(o.device):
                    check(lib.gnr_density_list(o._handle, s_._handle, _ptr(rays_all[i]), _ptr(tmin_all[i]), _ptr(x), x.shape[0],
                                               chunks[i].s, div[0], div[1], rank, _ptr(out), _stream()), "gnr_density_list")
            sig.append(out)
        tm.mark("density at owners")
        back = self.comm.all_to_all_known(sig, matrix.T, [self._buf(lane, i, "sigma_back", ch.max_valid, 0, torch.float32, ch.m.device)
                                                          for i, ch in enumerate(chunks)])
        tm.mark("all-to-all sigma")
        yield
        app_sends, app_dests = [], []
        for i, (ch, dest, sg, rank) in enumerate(zip(chunks, dests, back, self.comm.local_ranks)):
            with torch.cuda.device(ch.m.device):
                ch.launch_weights(sg, dest)
                tm.mark("weights")
                send = self._buf(lane, i, "app_send_ids", ch.max_app, 0, torch.int32, ch.m.device)
                dest_a = self._buf(lane, i, "app_dest", ch.max_app, 0, torch.int32, ch.m.device)
                ch.launch_route_ids(1, div, rank * cap, send, dest_a, cnts[i])
                tm.mark("route appearance")
                app_sends.append(send)
                app_dests.append(dest_a)
        amatrix = self.comm.gather_counts(cnts)
        for ch in chunks:
            with torch.cuda.device(ch.m.device):
                ch.checked_status()
        tm.mark("counts of the appearance lists")
        self.samples["valid"] += sum(ch.num_valid for ch in chunks)
        self.samples["app"] += sum(ch.num_app for ch in chunks)
        yield
        n_in = [int(amatrix[:, r].sum()) for r in self.comm.local_ranks]
        arecv = self.comm.all_to_all_known(app_sends, amatrix, [self._buf(lane, i, "app_recv_ids", n, 0, torch.int32, o.device)
                                                                for i, (o, n) in enumerate(zip(self.owners, n_in))])
        tm.mark("all-to-all appearance ids")
        rgb_o = []
        for i, (o, s_, x, rank) in enumerate(zip(self.owners, self.samplers, arecv, self.comm.local_ranks)):
            out = self._buf(lane, i, "rgb_owner", x.shape[0], 3, torch.float32, o.device)[: x.shape[0]]
            if x.shape[0]:
                keep, sc, nbytes = _scratch(o, x.shape[0], lane)
                with torch.cuda.device(o.device):
                    check(lib.gnr_appearance_list(o._handle, s_._handle, _ptr(rays_all[i]), _ptr(tmin_all[i]), _ptr(x), x.shape[0],
                                                  chunks[i].s, div[0], div[1], rank, sc, nbytes, _ptr(out), _stream()),
                          "gnr_appearance_list")
            rgb_o.append(out)
        tm.mark("appearance at owners")
        rgb_back = self.comm.all_to_all_known(rgb_o, amatrix.T, [self._buf(lane, i, "rgb_back", ch.max_app, 3, torch.float32, ch.m.device)
                                                                 for i, ch in enumerate(chunks)])
        tm.mark("all-to-all rgb")
        for i, (ch, dest_a, rb) in enumerate(zip(chunks, app_dests, rgb_back)):
            with torch.cuda.device(ch.m.device):
                rgb_s = self._buf(lane, i, "rgb_list", ch.num_app, 3, torch.float32, ch.m.device)[: ch.num_app]
                if ch.num_app:
                    torch.index_select(rb, 0, dest_a[: ch.num_app], out=rgb_s)
                result.append(ch.composite(rgb_s, white_bg))
        tm.mark("composite")

    def _chunk_steps(self, rays, n_samples, white_bg, lane, result, cap):
        if cap:
            return self._steps_ids(rays, n_samples, white_bg, lane, result, cap)
        return self._steps(rays, n_samples, white_bg, lane, result)

    def _steps(self, rays: Sequence[torch.Tensor], n_samples: int, white_bg: bool, lane: int, result: list):
        """Generator over the four steps of one chunk; ``result`` receives per local rank ``(rgb_map, depth_map)``."""
        tm, div, nb = self.timer, self.division, self.comm.world
        chunks, sends, dests, cnts = [], [], [], []
        # ---- 1: sample globally; block assignment + grouping by owner on the device ---------------------------------
        for i, (s_, r) in enumerate(zip(self.samplers, rays)):
            with torch.cuda.device(s_.device):
                ch = _Chunk(s_, r, n_samples, slot=lane)
                ch.launch_sample()
                tm.mark("sample")
                send = self._buf(lane, i, "send", ch.max_valid, 3, torch.float32, s_.device)
                dest = self._buf(lane, i, "dest", ch.max_valid, 0, torch.int32, s_.device)
                cnt = self._buf(lane, i, "cnt", nb, 0, torch.int32, s_.device)
                ch.launch_route(0, div, send, dest, cnt)
                tm.mark("route valid")
                chunks.append(ch)
                sends.append(send)
                dests.append(dest)
                cnts.append(cnt)
        matrix = self.comm.gather_counts(cnts)
        for ch in chunks:
            with torch.cuda.device(ch.m.device):
                ch.checked_status()
        tm.mark("counts of the valid lists")
        yield
        # ---- 2: points travel to the owners, density there, values travel back --------------------------------------
        n_in = [int(matrix[:, r].sum()) for r in self.comm.local_ranks]
        recv = self.comm.all_to_all_known(sends, matrix, [self._buf(lane, i, "recv", n, 3, torch.float32, o.device)
                                                          for i, (o, n) in enumerate(zip(self.owners, n_in))])
        tm.mark("all-to-all points")
        sig = []
        for i, (o, x) in enumerate(zip(self.owners, recv)):
            out = self._buf(lane, i, "sigma", x.shape[0], 0, torch.float32, o.device)
            if x.shape[0]:
                with torch.cuda.device(o.device):
                    check(lib.gnr_density_points(o._handle, _ptr(x), x.shape[0], None, _ptr(out), _stream()), "gnr_density_points")
            sig.append(out)
        tm.mark("density at owners")
        back = self.comm.all_to_all_known(sig, matrix.T, [self._buf(lane, i, "sigma_back", ch.max_valid, 0, torch.float32, ch.m.device)
                                                          for i, ch in enumerate(chunks)])
        tm.mark("all-to-all sigma")
        yield
        # ---- 3: weights and the appearance list at the ray's rank; route it by owner ----------------------------------
        app_sends, app_dests = [], []
        for i, (ch, dest, sg) in enumerate(zip(chunks, dests, back)):
            with torch.cuda.device(ch.m.device):
                ch.launch_weights(sg, dest)
                tm.mark("weights")
                send = self._buf(lane, i, "app_send", ch.max_app, 6, torch.float32, ch.m.device)
                dest_a = self._buf(lane, i, "app_dest", ch.max_app, 0, torch.int32, ch.m.device)
                ch.launch_route(1, div, send, dest_a, cnts[i])
                tm.mark("route appearance")
                app_sends.append(send)
                app_dests.append(dest_a)
        amatrix = self.comm.gather_counts(cnts)
        for ch in chunks:
            with torch.cuda.device(ch.m.device):
                ch.checked_status()
        tm.mark("counts of the appearance lists")
        self.samples["valid"] += sum(ch.num_valid for ch in chunks)
        self.samples["app"] += sum(ch.num_app for ch in chunks)
        yield
        # ---- 4: (point, view) rows travel to the owners, colour there, values travel back, composite -----------------
        n_in = [int(amatrix[:, r].sum()) for r in self.comm.local_ranks]
        arecv = self.comm.all_to_all_known(app_sends, amatrix, [self._buf(lane, i, "app_recv", n, 6, torch.float32, o.device)
                                                                for i, (o, n) in enumerate(zip(self.owners, n_in))])
        tm.mark("all-to-all appearance points")
        rgb_o = []
        for i, (o, x) in enumerate(zip(self.owners, arecv)):
            out = self._buf(lane, i, "rgb_owner", x.shape[0], 3, torch.float32, o.device)[: x.shape[0]]
            if x.shape[0]:
                keep, sc, nbytes = _scratch(o, x.shape[0], lane)
                with torch.cuda.device(o.device):
                    check(lib.gnr_appearance_rows(o._handle, _ptr(x), x.shape[0], sc, nbytes, _ptr(out), _stream()),
                          "gnr_appearance_rows")
            rgb_o.append(out)
        tm.mark("appearance at owners")
        rgb_back = self.comm.all_to_all_known(rgb_o, amatrix.T, [self._buf(lane, i, "rgb_back", ch.max_app, 3, torch.float32, ch.m.device)
                                                                 for i, ch in enumerate(chunks)])
        tm.mark("all-to-all rgb")
        for i, (ch, dest_a, rb) in enumerate(zip(chunks, app_dests, rgb_back)):
            with torch.cuda.device(ch.m.device):
                rgb_s = self._buf(lane, i, "rgb_list", ch.num_app, 3, torch.float32, ch.m.device)[: ch.num_app]
                if ch.num_app:
                    torch.index_select(rb, 0, dest_a[: ch.num_app], out=rgb_s)
                result.append(ch.composite(rgb_s, white_bg))
        tm.mark("composite")

    @torch.no_grad()
    def render_chunk(self, rays: Sequence[torch.Tensor], n_samples: int = -1, white_bg: bool = True):
        """``rays[i]``: the chunk of rays local rank i is responsible for (they differ per rank).
        Returns per local rank ``(rgb_map, depth_map)`` of its own rays."""
        cap = self._agree_ray_capacity(max(r.shape[0] for r in rays)) if self.ship_ids else 0
        self.timer.start()
        out: list = []
        for _ in self._chunk_steps(rays, n_samples, white_bg, 0, out, cap):
            pass
        return out

    @torch.no_grad()
    def render_frame(self, chunk_list: Sequence[Sequence[torch.Tensor]], n_samples: int = -1, white_bg: bool = True,
                     lanes: int = 2):
        """``chunk_list[c][i]``: chunk c of local rank i (every rank of the group passes the same number of
        chunks).  Two chunks are in flight, each on its own stream; returns per chunk what ``render_chunk``
        returns.  Only the single-process-per-rank form overlaps; with several local ranks (loopback) the
        lanes still alternate but share the current device's streams."""
        self.samples = {"valid": 0, "app": 0}
        cap = 0
        if self.ship_ids and len(chunk_list):
            cap = self._agree_ray_capacity(max(r.shape[0] for c in chunk_list for r in c))
        self.timer.start()
        return _run_lanes(lambda c, lane, out: self._chunk_steps(chunk_list[c], n_samples, white_bg, lane, out, cap),
                          len(chunk_list), lanes, self.samplers[0].device, self._streams, 2)
