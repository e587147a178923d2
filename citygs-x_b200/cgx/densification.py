"""Densification statistics fed by the hot path (the consumer side of the contract, not the densifier itself).

Two forms.  `DensificationStats` is the plain per-Gaussian form (the shape of the reference's commented-out
``add_densification_stats``, densification.py:63-76): per local Gaussian and per camera of the batch the norm of the
screen-space position gradient of the Gaussians that were visible (`radii > 0` from the LOCAL preprocess,
`means2D.grad` as it comes back through the reverse exchange), a visit counter and, optionally, the running maximum
of the screen radius.  It is what the benchmark's capacity sweep updates every step.  `AnchorStatistics` is the form
the reference's trainer actually calls for its anchor model (scene/gaussian_model.py:1181-1205 ``training_statis``).

The reference indexes with boolean masks (a host synchronisation per mask); here every update is a dense masked
expression, so nothing blocks the host.  Values are identical: rows outside the mask receive +0.
"""
from __future__ import annotations

import torch


class DensificationStats:
    def __init__(self, n_gaussians: int, device, track_max_radii: bool = True):
        self.grad_accum = torch.zeros(n_gaussians, 1, device=device)
        self.denom = torch.zeros(n_gaussians, 1, device=device)
        self.max_radii2D = torch.zeros(n_gaussians, dtype=torch.int32, device=device) if track_max_radii else None

    @torch.no_grad()
    def update(self, radii: torch.Tensor, means2D: torch.Tensor):
        """radii: int32 (P) of one camera from the local preprocess; means2D: the (P,2) leaf of that camera whose
        ``.grad`` the backward pass has filled (a camera that received no gradient contributes nothing)."""
        g = means2D.grad
        if g is None:
            return
        visible = (radii > 0).unsqueeze(1)
        self.grad_accum += torch.linalg.vector_norm(g[:, :2], dim=-1, keepdim=True) * visible
        self.denom += visible
        if self.max_radii2D is not None:
            torch.maximum(self.max_radii2D, radii.to(torch.int32), out=self.max_radii2D)

    def update_batch(self, per_camera):
        """per_camera: iterable of (radii, means2D), e.g. ``TrainingStep.last``."""
        for radii, means2D in per_camera:
            self.update(radii, means2D)

    def mean_gradient(self):
        """Average gradient norm over the visits, NaN-free (0 where never visible): what the densifier thresholds."""
        return self.grad_accum / self.denom.clamp_min(1.0)


class AnchorStatistics:
    """The statistics the reference's densifier reads for its anchor / neural-Gaussian model
    (scene/gaussian_model.py:1181-1205 ``training_statis``): per anchor the accumulated opacity of its visible
    neural Gaussians and a visit count, per (anchor, offset) slot the accumulated screen-space gradient norm and a
    visit count, routed through the three nested masks of the model (anchor visible -> offset selected -> Gaussian
    on screen).

    The reference writes through chained boolean indexing (`x[mask] += y`, one host synchronisation per mask).
    Here every update is a ``masked_scatter`` of a dense source, so nothing blocks the host; the values are the same.
    """

    def __init__(self, n_anchors: int, n_offsets: int, device):
        self.n_offsets = n_offsets
        self.opacity_accum = torch.zeros(n_anchors, 1, device=device)
        self.anchor_demon = torch.zeros(n_anchors, 1, device=device)
        self.offset_gradient_accum = torch.zeros(n_anchors * n_offsets, 1, device=device)
        self.offset_denom = torch.zeros(n_anchors * n_offsets, 1, device=device)

    @torch.no_grad()
    def training_statis(self, viewspace_point_grad, opacity, update_filter, offset_selection_mask, anchor_visible_mask):
        """viewspace_point_grad: (G, >=2) gradient of the screen-space positions of the G neural Gaussians that were
        rasterised; opacity: (V * n_offsets, 1) raw opacities of the V visible anchors' slots; update_filter: (G,)
        bool, Gaussian was on screen (radii > 0); offset_selection_mask: (V * n_offsets,) bool, slot produced a
        Gaussian (G = its number of True entries); anchor_visible_mask: (N,) bool with V True entries."""
        n_off = self.n_offsets
        avm = anchor_visible_mask.view(-1, 1)
        per_anchor = opacity.detach().reshape(-1).clamp_min(0).view(-1, n_off).sum(dim=1, keepdim=True)
        self.opacity_accum += torch.zeros_like(self.opacity_accum).masked_scatter(avm, per_anchor)
        self.anchor_demon += avm
        slots = avm.expand(-1, n_off).reshape(-1, 1)                                       # slot of a visible anchor
        selected = torch.zeros_like(slots).masked_scatter(slots, offset_selection_mask.view(-1, 1))
        on_screen = update_filter.view(-1, 1)
        norm = torch.linalg.vector_norm(viewspace_point_grad[:, :2], dim=-1, keepdim=True) * on_screen
        self.offset_gradient_accum += torch.zeros_like(self.offset_gradient_accum).masked_scatter(selected, norm)
        self.offset_denom += torch.zeros_like(self.offset_denom).masked_scatter(selected, on_screen.to(norm.dtype))
