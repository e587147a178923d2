"""Tile-row workload division across GPUs ("final" mode of the reference).

Mirrors gaussian_renderer/workload_division.py of the reference for the live path:
``division_pos_heuristic`` (:75-94), ``DivisionStrategyFinal`` (:684-778),
``DivisionStrategyHistoryFinal`` (:781-824), ``start_strategy_final`` (:827-916) and
``finish_strategy_final`` (:919-973).  The split unit is a tile row (a 16-pixel-high strip across the full image
width); the rows of the whole camera batch, concatenated, are cut into ``world_size`` contiguous ranges by a
running-time heuristic, so a GPU gets (part of) one or several cameras.

Differences from the reference, none of which change a result:
  * the reference reads rank, world size, tile grid and flags from process-wide globals; here they come from an
    explicit :class:`DivisionContext` (``configure`` installs a default one, so the reference's call signatures
    keep working);
  * the heuristic vectors are a few hundred floats and live on the CPU, so cutting the batch costs no GPU
    synchronisation (the reference runs cumsum/searchsorted on the GPU and reads the result back);
  * per-camera times are gathered with a flat ``all_gather_into_tensor`` (works on NCCL and gloo).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

BLOCK_X, BLOCK_Y = 16, 16


@dataclass
class DivisionContext:
    image_height: int
    image_width: int
    rank: int = 0
    world_size: int = 1
    bsz: int = 1
    group: object = None                  # torch.distributed process group (None = default group)
    device: object = None                 # device of compute_locally / tile-bound tensors
    local_sampling: bool = False
    border_divpos_coeff: float = 1.0      # reference default (arguments/__init__.py)
    heuristic_decay: float = 0.0
    no_heuristics_update: bool = False
    adjust_strategy_warmp_iterations: int = -1
    iteration: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def tile_x(self):
        return (self.image_width + BLOCK_X - 1) // BLOCK_X

    @property
    def tile_y(self):
        return (self.image_height + BLOCK_Y - 1) // BLOCK_Y


_default_ctx: DivisionContext | None = None


def configure(ctx: DivisionContext):
    global _default_ctx
    _default_ctx = ctx
    return ctx


def _ctx(ctx):
    c = ctx or _default_ctx
    if c is None:
        raise RuntimeError("workload_division: call configure(DivisionContext(...)) first or pass ctx=")
    return c


def division_pos_heuristic(heuristic, tile_num, world_size, right=False):
    """Cut ``tile_num`` rows into ``world_size`` contiguous parts of (nearly) equal accumulated heuristic."""
    assert heuristic.shape[0] == tile_num, "the length of heuristics should be the same as the number of tiles."
    heuristic = heuristic.detach().to("cpu", torch.float32)
    heuristic_prefix_sum = torch.cumsum(heuristic, dim=0)
    heuristic_sum = heuristic_prefix_sum[-1]
    heuristic_per_worker = heuristic_sum / world_size
    thresholds = torch.arange(1, world_size) * heuristic_per_worker
    division_indices = torch.searchsorted(heuristic_prefix_sum, thresholds, right=right)
    return [0] + division_indices.tolist() + [tile_num]


_TILE_BOUNDS = {}
_LOCAL_MASKS = {}


class DivisionStrategyFinal:
    """Which GPUs render which tile rows of one camera."""

    def __init__(self, camera, world_size, gpu_ids, division_pos, gpu_for_this_camera_tilelr, ctx=None):
        ctx = _ctx(ctx)
        cuts = [int(c) for c in division_pos]
        bands = list(zip(cuts[:-1], cuts[1:]))
        problems = []
        if world_size <= 0 or len(gpu_ids) != world_size:
            problems.append(f"{len(gpu_ids)} gpu ids for world_size {world_size}")
        if len(cuts) != world_size + 1 or cuts[:1] != [0] or cuts[-1:] != [ctx.tile_y]:
            problems.append(f"cuts {cuts} do not run from 0 to {ctx.tile_y} in {world_size} bands")
        if any(hi <= lo for lo, hi in bands):
            problems.append(f"cuts {cuts} are not strictly ascending")
        if [tuple(map(int, lr)) for lr in gpu_for_this_camera_tilelr] != bands:
            problems.append(f"row ranges {list(gpu_for_this_camera_tilelr)} do not match cuts {cuts}")
        assert not problems, "invalid division of a camera: " + "; ".join(problems)
        self.ctx = ctx
        self.camera = camera
        self.world_size = world_size
        self.gpu_ids = gpu_ids
        self.rank = gpu_ids.index(ctx.rank) if ctx.rank in gpu_ids else -1
        self.division_pos = division_pos

    def tile_bounds(self, device=None):
        """int32 (world_size+1) linear tile ids of the band boundaries (division_pos * TILE_X)."""
        dev = torch.device(device or self.ctx.device or "cpu")
        key = (tuple(self.division_pos), self.ctx.tile_x, dev)
        t = _TILE_BOUNDS.get(key)
        if t is None:                       # cuts rarely move: keep the device copies instead of one upload per call
            if len(_TILE_BOUNDS) > 4096:
                _TILE_BOUNDS.clear()
            t = (torch.tensor(self.division_pos, dtype=torch.int32) * self.ctx.tile_x).to(dev)
            _TILE_BOUNDS[key] = t
        return t

    def get_local2j_ids(self, means2D, radii, raster_settings, cuda_args):
        """(list of index tensors per destination, (P, world_size) bool mask), as the reference returns them.
        The fused exchange (cgx.exchange) does not go through this method; it is kept for callers that do."""
        import diff_gaussian_rasterization

        mask = diff_gaussian_rasterization._C.get_local2j_ids_bool(
            raster_settings.image_height, raster_settings.image_width, self.rank, self.world_size, means2D, radii,
            self.tile_bounds(means2D.device), cuda_args)
        return [mask[:, rk].nonzero() for rk in range(self.world_size)], mask

    def get_compute_locally(self):
        if self.ctx.rank not in self.gpu_ids:
            return None
        rank = self.gpu_ids.index(self.ctx.rank)
        tx, ty = self.ctx.tile_x, self.ctx.tile_y
        dev = torch.device(self.ctx.device or "cpu")
        key = (self.division_pos[rank], self.division_pos[rank + 1], tx, ty, dev)
        m = _LOCAL_MASKS.get(key)
        if m is None:                       # read-only downstream, so one tensor per distinct band is shared
            if len(_LOCAL_MASKS) > 4096:
                _LOCAL_MASKS.clear()
            m = torch.zeros(ty * tx, dtype=torch.bool, device=dev)
            m[self.division_pos[rank] * tx: self.division_pos[rank + 1] * tx] = True
            m = _LOCAL_MASKS[key] = m.view(ty, tx)
        return m

    def get_compute_locally_all(self):
        if self.ctx.rank not in self.gpu_ids:
            return None
        return torch.ones(self.ctx.tile_y, self.ctx.tile_x, dtype=torch.bool, device=self.ctx.device or "cpu")

    def get_extended_compute_locally(self):
        return None


class DivisionStrategyHistoryFinal:
    """Per-camera running-time heuristic (one value per tile row) and the log of past divisions."""

    def __init__(self, dataset, world_size, rank, ctx=None):
        ctx = _ctx(ctx)
        self.ctx = ctx
        self.world_size = world_size
        self.rank = rank
        self.accum_heuristic = {}
        cameras = dataset.cameras if hasattr(dataset, "cameras") else dataset
        for camera in cameras:
            self.accum_heuristic[camera.uid] = torch.ones((ctx.tile_y,), dtype=torch.float32)
        self.history = []

    def store_stats(self, batched_cameras, gpu_camera_running_time, batched_strategies):
        """Append one log entry: per camera who rendered which rows in how many ms, per rank and per camera totals."""
        per_rank = [0.0] * self.world_size
        per_camera, info = [], []
        for k, (camera, strategy) in enumerate(zip(batched_cameras, batched_strategies)):
            ms = [gpu_camera_running_time[rank][k] for rank in strategy.gpu_ids]
            for rank, t in zip(strategy.gpu_ids, ms):
                per_rank[rank] += t
            per_camera.append(sum(ms))
            info.append({"camera_id": camera.uid, "gpu_ids": strategy.gpu_ids, "division_pos": strategy.division_pos,
                         "each_gpu_running_time": ms})
        self.history.append({"iteration": self.ctx.iteration, "all_gpu_running_time": per_rank,
                             "all_camera_running_time": per_camera, "batched_camera_info": info})

    def to_json(self):
        return self.history


def start_strategy_final(batched_cameras, strategy_history, ctx=None):
    """Division of this batch.  Returns (one DivisionStrategyFinal per camera, gpuid -> [(camera idx, row_l, row_r)])."""
    ctx = _ctx(ctx)
    ws = ctx.world_size
    n_tiles_per_image = ctx.tile_y
    total_tiles = n_tiles_per_image * len(batched_cameras)
    batched_strategies = []
    gpuid2tasks = [[] for _ in range(ws)]

    if ctx.local_sampling:
        bsz_per_gpu = ctx.bsz // ws
        for idx, camera in enumerate(batched_cameras):
            gpu_id = idx // bsz_per_gpu
            gpuid2tasks[gpu_id].append((idx, 0, n_tiles_per_image))
            batched_strategies.append(DivisionStrategyFinal(camera, 1, [gpu_id], [0, n_tiles_per_image],
                                                            [(0, n_tiles_per_image)], ctx=ctx))
        return batched_strategies, gpuid2tasks

    rows = n_tiles_per_image
    cost = torch.cat([strategy_history.accum_heuristic[camera.uid] for camera in batched_cameras], dim=0)
    cuts = division_pos_heuristic(cost, total_tiles, ws, right=True)
    # a cut closer than border_divpos_coeff rows to an image border moves onto the border
    margin = ctx.border_divpos_coeff
    for i in range(1, ws):
        image, row = divmod(cuts[i], rows)
        if row + margin >= rows:
            cuts[i] = (image + 1) * rows
        elif row <= margin:
            cuts[i] = image * rows
    too_thin = [i for i in range(ws) if cuts[i + 1] - cuts[i] <= margin]
    assert not too_thin, f"ranks {too_thin} would get {margin} tile rows or fewer: cuts {cuts}"

    for idx, camera in enumerate(batched_cameras):
        first = idx * rows                                    # this camera's rows in the concatenated batch
        ranks, bands = [], []
        for rank in range(ws):
            lo, hi = max(cuts[rank], first) - first, min(cuts[rank + 1], first + rows) - first
            if hi <= lo:
                continue                                      # rank's range does not reach into this camera
            ranks.append(rank)
            bands.append((lo, hi))
            gpuid2tasks[rank].append((idx, lo, hi))
        batched_strategies.append(DivisionStrategyFinal(camera, len(ranks), ranks, [0] + [hi for _, hi in bands],
                                                        bands, ctx=ctx))
    return batched_strategies, gpuid2tasks


def allgather_float_list(values, ctx):
    """(world_size, len(values)) nested list of every rank's values."""
    import torch.distributed as dist

    if ctx.world_size == 1 or not dist.is_available() or not dist.is_initialized():
        return [list(map(float, values))]
    backend = dist.get_backend(ctx.group)
    dev = ctx.device if backend == "nccl" else "cpu"
    local = torch.tensor(list(map(float, values)), dtype=torch.float32, device=dev)
    out = torch.empty(ctx.world_size * local.numel(), dtype=torch.float32, device=dev)
    dist.all_gather_into_tensor(out, local, group=ctx.group)
    return out.view(ctx.world_size, -1).cpu().tolist()


def local_running_times(batched_strategies, batched_statistic_collector, ctx=None):
    """This rank's render time per camera of the batch (forward + backward + twice the loss forward, the
    reference's cost model, utils/workload_division.py finish_strategy_final); -1 for cameras it did not render."""
    ctx = _ctx(ctx)
    times = []
    for idx, strategy in enumerate(batched_strategies):
        if ctx.rank not in strategy.gpu_ids:
            times.append(-1.0)
            continue
        st = batched_statistic_collector[idx]
        times.append(float(st["forward_render_time"]) + float(st["backward_render_time"])
                     + float(st.get("forward_loss_time", 0.0)) * 2)
    return times


def finish_strategy_final(batched_cameras, strategy_history, batched_strategies, batched_statistic_collector,
                          ctx=None, gathered_times=None):
    """Feed the measured per-camera times back into the per-row heuristics.  ``gathered_times`` ([rank][camera],
    every rank's `local_running_times`) skips the all-gather when the caller already exchanged them."""
    ctx = _ctx(ctx)
    if gathered_times is None:
        gathered_times = allgather_float_list(
            local_running_times(batched_strategies, batched_statistic_collector, ctx), ctx)
    gpu_camera_running_time = gathered_times
    strategy_history.store_stats(batched_cameras, gpu_camera_running_time, batched_strategies)

    if ((ctx.iteration <= ctx.adjust_strategy_warmp_iterations) or (ctx.world_size == 1) or ctx.no_heuristics_update
            or (ctx.bsz >= ctx.world_size and (ctx.image_height <= 1080 or ctx.image_width <= 1920))
            or (ctx.image_height <= 600 or ctx.image_width <= 1000)):
        return

    keep = ctx.heuristic_decay
    for k, (camera, strategy) in enumerate(zip(batched_cameras, batched_strategies)):
        # every row of a band costs the band's time divided by its height
        per_row = torch.zeros((ctx.tile_y,), dtype=torch.float32)
        for rank, lo, hi in zip(strategy.gpu_ids, strategy.division_pos[:-1], strategy.division_pos[1:]):
            per_row[lo:hi] = gpu_camera_running_time[rank][k] / (hi - lo)
        old = strategy_history.accum_heuristic[camera.uid]
        strategy_history.accum_heuristic[camera.uid] = per_row if keep == 0 else old * keep + per_row * (1 - keep)
