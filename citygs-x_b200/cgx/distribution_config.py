"""Mapping from the reference's ``image_distribution_mode`` strings to (loss mode, division mode, flags).

Mirrors gaussian_renderer/distribution_config.py of the reference.  That table is dead code upstream: the
default mode is "final" (arguments/__init__.py:248) and ``init_image_distribution_config`` is imported but
never called; it is kept here, table-driven, so that configs written for the reference still resolve.
Only the "final" tile-row division (cgx.workload_division) is implemented behind it.
"""
from collections import namedtuple

ImageDistributionConfig = namedtuple(
    "ImageDistributionConfig",
    ["loss_distribution_mode", "workloads_division_mode", "avoid_pixels_all2all", "local_running_time_mode"])

_BWD = ["backward_render_time"]
_FULL = ["backward_render_time", "forward_render_time", "forward_loss_time", "forward_loss_time"]

_TABLE = {
    "0": ("replicated_loss_computation", "DivisionStrategyUniform", False, _BWD),
    "1": ("general_distributed_loss_computation", "DivisionStrategyUniform", False, _BWD),
    "2": ("general_distributed_loss_computation", "DivisionStrategyDynamicAdjustment", False, _BWD),
    "3": ("avoid_pixel_all2all_loss_computation", "DivisionStrategyDynamicAdjustment", True, _FULL),
    "4": ("avoid_pixel_all2all_loss_computation_adjust_mode6", "DivisionStrategyAsGrid", True, _FULL),
}


def init_image_distribution_config(args):
    mode = args.image_distribution_mode
    if mode not in _TABLE:
        raise ValueError(f"Unknown image_distribution_mode: {mode}")
    loss, division, avoid, times = _TABLE[mode]
    args.image_distribution_config = ImageDistributionConfig(loss, division, avoid, list(times))
    return args.image_distribution_config
