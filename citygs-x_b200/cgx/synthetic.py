"""Seeded synthetic scenes and cameras with the shapes of the reference's aerial-city workloads.

They stand in for the MatrixCity / Mill-19 / UrbanScene3D scenes the reference
trains on (those datasets are not redistributed here).  Camera matrices follow the
reference's conventions exactly: ``viewmatrix = getWorld2View2(R, T).T`` and
``projmatrix = viewmatrix @ getProjectionMatrix(znear=.01, zfar=100).T``
(scene/cameras.py:118-140, utils/graphics_utils.py:42-76), i.e. row-vector
matrices with the translation in elements 12..14.

Everything is generated in fp32 on the CPU from ``torch.Generator().manual_seed(20250 + cfg)``
and moved to the device by the caller.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

ZNEAR, ZFAR = 0.01, 100.0

SH_C0 = 0.28209479177387814
SH_C1 = 0.4886025119029199
SH_C2 = (1.0925484305920792, -1.0925484305920792, 0.31539156525252005, -1.0925484305920792, 0.5462742152960396)
SH_C3 = (-0.5900435899266435, 2.890611442640554, -0.4570457994644658, 0.3731763325901154, -0.4570457994644658,
         1.445305721320277, -0.5900435899266435)


@dataclass
class Camera:
    uid: int
    W: int
    H: int
    FoVx: float
    FoVy: float
    tanfovx: float
    tanfovy: float
    viewmatrix: torch.Tensor   # (4,4) world_view_transform (already transposed, row-vector convention)
    projmatrix: torch.Tensor   # (4,4) full_proj_transform
    campos: torch.Tensor       # (3,)

    def to(self, device):
        return Camera(self.uid, self.W, self.H, self.FoVx, self.FoVy, self.tanfovx, self.tanfovy,
                      self.viewmatrix.to(device), self.projmatrix.to(device), self.campos.to(device))


def look_at_camera(uid: int, eye, target, W: int, H: int, fov_x_deg: float = 60.0, world_up=(0.0, 0.0, 1.0)) -> Camera:
    """Pinhole camera at ``eye`` looking at ``target``; camera axes x right, y down, z forward."""
    eye = torch.tensor(eye, dtype=torch.float64)
    target = torch.tensor(target, dtype=torch.float64)
    up = torch.tensor(world_up, dtype=torch.float64)
    fwd = target - eye
    fwd = fwd / fwd.norm()
    if abs(float(fwd @ up)) > 0.999:            # nadir view: pick another up hint
        up = torch.tensor((0.0, 1.0, 0.0), dtype=torch.float64)
    right = torch.linalg.cross(fwd, up)
    right = right / right.norm()
    down = torch.linalg.cross(fwd, right)
    R = torch.stack([right, down, fwd], dim=1)   # camera-to-world rotation (columns = camera axes)
    T = -(R.T @ eye)                             # world-to-camera translation
    Rt = torch.eye(4, dtype=torch.float64)
    Rt[:3, :3] = R.T
    Rt[:3, 3] = T
    view = Rt.to(torch.float32).T.contiguous()   # getWorld2View2(R, T).transpose(0, 1)

    FoVx = math.radians(fov_x_deg)
    FoVy = 2.0 * math.atan(math.tan(FoVx * 0.5) * H / W)
    tanx, tany = math.tan(FoVx * 0.5), math.tan(FoVy * 0.5)
    top, right_ = tany * ZNEAR, tanx * ZNEAR
    Pm = torch.zeros(4, 4)
    Pm[0, 0] = 2.0 * ZNEAR / (2 * right_)
    Pm[1, 1] = 2.0 * ZNEAR / (2 * top)
    Pm[3, 2] = 1.0
    Pm[2, 2] = ZFAR / (ZFAR - ZNEAR)
    Pm[2, 3] = -(ZFAR * ZNEAR) / (ZFAR - ZNEAR)
    proj = (view.unsqueeze(0).bmm(Pm.T.contiguous().unsqueeze(0))).squeeze(0).contiguous()
    campos = view.inverse()[3, :3].contiguous()
    return Camera(uid, W, H, FoVx, FoVy, tanx, tany, view, proj, campos)


def eval_sh(deg: int, sh: torch.Tensor, dirs: torch.Tensor) -> torch.Tensor:
    """sh: (P, 16, 3); dirs: (P, 3) unit vectors -> (P, 3) (before the +0.5 shift)."""
    x, y, z = dirs[:, 0:1], dirs[:, 1:2], dirs[:, 2:3]
    res = SH_C0 * sh[:, 0]
    if deg > 0:
        res = res - SH_C1 * y * sh[:, 1] + SH_C1 * z * sh[:, 2] - SH_C1 * x * sh[:, 3]
    if deg > 1:
        xx, yy, zz, xy, yz, xz = x * x, y * y, z * z, x * y, y * z, x * z
        res = (res + SH_C2[0] * xy * sh[:, 4] + SH_C2[1] * yz * sh[:, 5] + SH_C2[2] * (2.0 * zz - xx - yy) * sh[:, 6]
               + SH_C2[3] * xz * sh[:, 7] + SH_C2[4] * (xx - yy) * sh[:, 8])
    if deg > 2:
        res = (res + SH_C3[0] * y * (3 * xx - yy) * sh[:, 9] + SH_C3[1] * xy * z * sh[:, 10]
               + SH_C3[2] * y * (4 * zz - xx - yy) * sh[:, 11] + SH_C3[3] * z * (2 * zz - 3 * xx - 3 * yy) * sh[:, 12]
               + SH_C3[4] * x * (4 * zz - xx - yy) * sh[:, 13] + SH_C3[5] * z * (xx - yy) * sh[:, 14]
               + SH_C3[6] * x * (xx - 3 * yy) * sh[:, 15])
    return res


def quaternion_to_matrix(q: torch.Tensor) -> torch.Tensor:
    """Real-first quaternions (P,4) -> rotation matrices (P,3,3)."""
    r, i, j, k = q.unbind(-1)
    two_s = 2.0 / (q * q).sum(-1)
    o = torch.stack((1 - two_s * (j * j + k * k), two_s * (i * j - k * r), two_s * (i * k + j * r),
                     two_s * (i * j + k * r), 1 - two_s * (i * i + k * k), two_s * (j * k - i * r),
                     two_s * (i * k - j * r), two_s * (j * k + i * r), 1 - two_s * (i * i + j * j)), -1)
    return o.reshape(q.shape[:-1] + (3, 3))


def build_all_map(means3D, scales, rotations, cam: Camera) -> torch.Tensor:
    """PGSR per-Gaussian 5-vector [normal_cam(3), 1, plane distance] as the reference's caller builds it
    (gaussian_renderer/__init__.py:1501-1518).  Works on any device."""
    Rm = quaternion_to_matrix(torch.nn.functional.normalize(rotations, p=2, dim=-1))
    idx = scales.min(dim=-1)[1][..., None, None].expand(-1, 3, -1)
    normal = Rm.gather(2, idx).squeeze(2)
    to_cam = cam.campos.to(means3D.device) - means3D
    neg = (normal * to_cam).sum(-1) < 0.0
    normal = torch.where(neg[:, None], -normal, normal)
    V = cam.viewmatrix.to(means3D.device)
    local_normal = normal @ V[:3, :3]
    pts = means3D @ V[:3, :3] + V[3, :3]
    out = torch.zeros(means3D.shape[0], 5, device=means3D.device, dtype=torch.float32)
    out[:, :3] = local_normal
    out[:, 3] = 1.0
    out[:, 4] = (local_normal * pts).sum(-1).abs()
    return out


def make_gaussians(P: int, box, gen: torch.Generator, clustered: bool = False):
    """box = (xy_half_extent, z_max).  Returns dict of fp32 CPU tensors (activated parameters)."""
    half, zmax = box
    if not clustered:
        u = torch.rand(P, 3, generator=gen)
        means = torch.stack([(u[:, 0] * 2 - 1) * half, (u[:, 1] * 2 - 1) * half, u[:, 2] * zmax], 1)
    else:
        nb = 512
        centres = (torch.rand(nb, 2, generator=gen) * 2 - 1) * half
        sigma = 5.0 + 20.0 * torch.rand(nb, generator=gen)
        heights = 80.0 * torch.rand(nb, generator=gen)
        w = 1.0 / torch.arange(1, nb + 1, dtype=torch.float64) ** 1.2
        n_blob = int(P * 0.8)
        counts = torch.floor(w / w.sum() * n_blob).to(torch.int64)
        counts[0] += n_blob - int(counts.sum())
        bid = torch.repeat_interleave(torch.arange(nb), counts)
        xy = centres[bid] + torch.randn(n_blob, 2, generator=gen) * sigma[bid, None]
        z = torch.rand(n_blob, generator=gen) * heights[bid]
        n_g = P - n_blob
        gxy = (torch.rand(n_g, 2, generator=gen) * 2 - 1) * half
        gz = torch.rand(n_g, generator=gen)
        means = torch.cat([torch.cat([xy, z[:, None]], 1), torch.cat([gxy, gz[:, None]], 1)], 0)
        means = means[torch.randperm(P, generator=gen)]
    scales = torch.exp(torch.randn(P, 3, generator=gen) * 0.5 - 3.0)
    rot = torch.nn.functional.normalize(torch.randn(P, 4, generator=gen), dim=-1)
    opac = torch.sigmoid(torch.randn(P, 1, generator=gen))
    sh = torch.cat([torch.randn(P, 1, 3, generator=gen) * 0.5, torch.randn(P, 15, 3, generator=gen) * 0.05], 1)
    return dict(means3D=means.float().contiguous(), scales=scales.contiguous(), rotations=rot.contiguous(),
                opacities=opac.contiguous(), sh=sh.contiguous())


def colours_for(g, cam: Camera) -> torch.Tensor:
    d = g["means3D"] - cam.campos.to(g["means3D"].device)
    d = d / d.norm(dim=1, keepdim=True)
    return torch.clamp_min(eval_sh(3, g["sh"], d) + 0.5, 0.0).contiguous()


# ----------------------------------------------------------------------------- the five benchmark configurations
def ring_cameras(n, radius, height, W, H, uid0=0):
    return [look_at_camera(uid0 + k, (radius * math.cos(2 * math.pi * k / n), radius * math.sin(2 * math.pi * k / n),
                                       height), (0.0, 0.0, 0.0), W, H) for k in range(n)]


def config(cfg: int, n_gaussians: int | None = None, n_cameras: int | None = None, res: tuple | None = None):
    """Return (gaussians dict, [Camera...]) for benchmark configuration ``cfg`` (0..4).  The optional
    overrides shrink a configuration for tests while keeping its distribution."""
    gen = torch.Generator().manual_seed(20250 + cfg)
    if cfg == 0:
        P, (W, H) = n_gaussians or 50_000, res or (256, 144)
        g = make_gaussians(P, (50.0, 20.0), gen)
        cams = ring_cameras(n_cameras or 2, 60.0, 40.0, W, H)
    elif cfg == 1:
        P, (W, H) = n_gaussians or 1_000_000, res or (1920, 1080)
        g = make_gaussians(P, (100.0, 30.0), gen)
        cams = [look_at_camera(0, (0.0, -60.0, 60.0), (0.0, 0.0, 0.0), W, H)]
    elif cfg in (2, 4):
        P, (W, H) = n_gaussians or 6_000_000, res or (1600, 1200)
        g = make_gaussians(P, (300.0, 40.0), gen)
        cams = ring_cameras(n_cameras or 8, 200.0, 120.0, W, H)
    elif cfg == 3:
        P, (W, H) = n_gaussians or 20_000_000, res or (3840, 2160)
        g = make_gaussians(P, (600.0, 1.0), gen, clustered=True)
        n = n_cameras or 16
        cams = []
        for k in range(n):
            gx, gy = k % 4, k // 4
            eye = ((gx - 1.5) * 300.0, (gy - 1.5) * 300.0, 300.0)
            # pitch 80 degrees below the horizon: look slightly ahead (+y) of the nadir point
            tgt = (eye[0], eye[1] + 300.0 / math.tan(math.radians(80.0)), 0.0)
            cams.append(look_at_camera(k, eye, tgt, W, H))
    else:
        raise ValueError(f"unknown config {cfg}")
    return g, cams
