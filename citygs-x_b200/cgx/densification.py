"""Densification statistics fed by the hot path (the consumer side of the contract, not the densifier itself):
the reference accumulates, per local Gaussian and per camera of the batch, the norm of the screen-space position
gradient of the Gaussians that were visible (`radii > 0` from the LOCAL preprocess, `means2D.grad` as it comes back
through the reverse exchange), together with a visit counter (scene/gaussian_model.py:1181-1205, driven by
densification.py:63-76); the running maximum of the screen radius is commented out there and optional here.

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
