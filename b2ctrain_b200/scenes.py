"""Seeded synthetic scenes, cameras and targets for the parity tests and the benchmark.

No dataset is involved: the benchmark configurations are themselves synthetic (distributions stated per config
below). Everything is numpy on the host, in the host-side layout of the reference's SplatCloud (src/ply.h:12-22):
pos_op [n][4] = (x, y, z, opacity logit), quat [n][4] = (w, x, y, z) unnormalised, lscale [n][4] = (log sx, log sy,
log sz, floor f), sh [n][K][3] coefficient-major.
"""
import math

import numpy as np


def camera_gpu(R, t, fx, fy, cx, cy, W, H):
    """The CameraGPU record (src/gpu/render.h:10-24): pose, intrinsics and the EWA Jacobian clamp limits, all fp32."""
    R = np.asarray(R, np.float32).reshape(3, 3)
    t = np.asarray(t, np.float32)
    pos = -(R.T @ t)
    f = np.float32
    fx, fy, cx, cy = f(fx), f(fy), f(cx), f(cy)
    return dict(R=R.reshape(9).copy(), t=t.copy(), pos=pos.astype(np.float32), fx=fx, fy=fy, cx=cx, cy=cy, W=int(W), H=int(H),
                lim_pos_x=(f(1.15) * f(W) - cx) / fx, lim_pos_y=(f(1.15) * f(H) - cy) / fy,
                lim_neg_x=(f(-0.15) * f(W) - cx) / fx, lim_neg_y=(f(-0.15) * f(H) - cy) / fy)


def look_at_camera(eye, W, H, fx, fy=None, target=(0.0, 0.0, 0.0)):
    """Pinhole camera at `eye` looking at `target`, OpenCV axes (+X right, +Y down, +Z forward), world up = +Y up."""
    eye = np.asarray(eye, np.float64)
    fwd = np.asarray(target, np.float64) - eye
    fwd /= np.linalg.norm(fwd)
    up = np.array([0.0, 1.0, 0.0])
    if abs(fwd @ up) > 0.999:
        up = np.array([0.0, 0.0, 1.0])
    right = np.cross(fwd, up); right /= np.linalg.norm(right)
    down = np.cross(fwd, right)
    R = np.stack([right, down, fwd])          # world -> camera rows
    t = -R @ eye
    return camera_gpu(R, t, fx, fx if fy is None else fy, W / 2.0, H / 2.0, W, H)


def orbit_eye(radius, azimuth_deg, elevation_deg):
    a, e = math.radians(azimuth_deg), math.radians(elevation_deg)
    return (radius * math.cos(e) * math.sin(a), radius * math.sin(e), radius * math.cos(e) * math.cos(a))


def make_splats(n, degree, seed, log_scale=(-4.0, 0.5), opacity=(0.0, 1.0), heavy_tail=False, bimodal_opacity=False):
    """Means uniform in the unit ball; log-scales, opacity logits normal; unit quaternions from normalised N(0,1)^4;
    SH DC ~ N(0.5, 0.2), higher bands ~ N(0, 0.2)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    K = (degree + 1) ** 2
    d = rng.standard_normal((n, 3)); d /= np.linalg.norm(d, axis=1, keepdims=True)
    pos = d * np.cbrt(rng.random((n, 1)))
    if heavy_tail:   # 90% small, 10% large splats that cover hundreds of tiles
        big = rng.random(n) < 0.1
        ls = np.where(big[:, None], rng.normal(-1.0, 0.5, (n, 3)), rng.normal(-5.0, 0.5, (n, 3)))
    else:
        ls = rng.normal(log_scale[0], log_scale[1], (n, 3))
    q = rng.standard_normal((n, 4)); q /= np.linalg.norm(q, axis=1, keepdims=True)
    if bimodal_opacity:
        hi = rng.random(n) < 0.5
        op = np.where(hi, rng.normal(4.0, 0.5, n), rng.normal(-4.0, 0.5, n))
    else:
        op = rng.normal(opacity[0], opacity[1], n)
    sh = rng.normal(0.0, 0.2, (n, K, 3)); sh[:, 0, :] = rng.normal(0.5, 0.2, (n, 3))
    f32 = np.float32
    return dict(n=n, degree=degree, pos_op=np.concatenate([pos, op[:, None]], 1).astype(f32), quat=q.astype(f32),
                lscale=np.concatenate([ls, np.zeros((n, 1))], 1).astype(f32), sh=np.ascontiguousarray(sh.astype(f32)))


def perturbed(scene, sigma, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    out = dict(scene)
    for k in ("pos_op", "quat", "sh"):
        out[k] = (scene[k] + rng.normal(0, sigma, scene[k].shape)).astype(np.float32)
    ls = scene["lscale"].copy(); ls[:, :3] += rng.normal(0, sigma, (scene["n"], 3)).astype(np.float32)
    out["lscale"] = ls
    return out


def floor_for_cameras(scene, cams):
    """3D-filter floor f = sqrt(0.1) * min over cameras of distance / focal (src/gpu/refine.cu:27-38), fp32."""
    p = scene["pos_op"][:, :3].astype(np.float32)
    best = np.full(scene["n"], np.inf, np.float32)
    for c in cams:
        d = np.sqrt(((p - c["pos"][None, :]) ** 2).sum(1, dtype=np.float32)).astype(np.float32)
        best = np.minimum(best, d / max(np.float32(0.5) * (c["fx"] + c["fy"]), np.float32(1e-6)))
    out = dict(scene); ls = scene["lscale"].copy(); ls[:, 3] = np.float32(math.sqrt(0.1)) * best; out["lscale"] = ls
    return out


def pack_rgba8(img, alpha=None):
    """Quantise a float RGBA image [P][4] to packed RGBA8 the way the reference packs rendered targets
    (src/train/teacher.cu:11-17): round half up, colour clamped to alpha. `alpha` overrides the alpha byte."""
    q = np.clip(np.floor(np.asarray(img, np.float64) * 255.0 + 0.5), 0, 255).astype(np.uint32)
    a = q[:, 3] if alpha is None else np.asarray(alpha, np.uint32)
    r, g, b = np.minimum(q[:, 0], a), np.minimum(q[:, 1], a), np.minimum(q[:, 2], a)
    return (r | (g << 8) | (b << 16) | (a << 24)).astype(np.uint32)


def ellipse_mask(W, H, coverage=0.4):
    """Binary centred ellipse covering `coverage` of the frame, as an alpha byte plane."""
    y, x = np.mgrid[0:H, 0:W]
    s = math.sqrt(coverage / math.pi)   # semi-axes s*W, s*H  ->  area pi s^2 W H
    inside = ((x + 0.5 - W / 2) / (s * W)) ** 2 + ((y + 0.5 - H / 2) / (s * H)) ** 2 <= 1.0
    return np.where(inside, 255, 0).astype(np.uint32).reshape(-1)


def gradcheck_scene(seed, n=24, W=48, H=40, degree=2):
    """A small scene in the mould of the reference's gradient check (tests/tests.cpp:32-59): n splats in front of an
    identity camera, random RGBA target, random normal-free weights."""
    rng = np.random.Generator(np.random.PCG64(seed))
    K = (degree + 1) ** 2
    u = lambda *s: rng.random(s)
    un = lambda *s: rng.random(s) * 2 - 1
    pos = np.stack([un(n) * 0.6, un(n) * 0.5, 2.0 + un(n) * 0.5], 1)
    ls = np.log(0.05 + 0.08 * u(n, 3))
    q = np.stack([1.0 + un(n) * 0.5, un(n) * 0.5, un(n) * 0.5, un(n) * 0.5], 1)
    op = un(n) * 2.0
    sh = un(n, K, 3) * 0.3; sh[:, 0, :] = un(n, 3) * 1.5
    f32 = np.float32
    scene = dict(n=n, degree=degree, pos_op=np.concatenate([pos, op[:, None]], 1).astype(f32), quat=q.astype(f32),
                 lscale=np.concatenate([ls, np.zeros((n, 1))], 1).astype(f32), sh=np.ascontiguousarray(sh.astype(f32)))
    cam = camera_gpu(np.eye(3), np.zeros(3), 40.0, 40.0, W / 2.0, H / 2.0, W, H)
    rgba = (u(W * H, 4) * 255).astype(np.uint32)
    gt = rgba[:, 0] | (rgba[:, 1] << 8) | (rgba[:, 2] << 16) | (rgba[:, 3] << 24)
    wts = (64 + u(W * H) * 191).astype(np.uint8)
    return scene, cam, gt.astype(np.uint32), wts


# ---- the benchmark configurations ----

def config_cameras(cfg):
    if cfg == 0:
        return [look_at_camera((0.0, 0.0, 3.0), 64, 64, 64.0)]
    if cfg == 1:
        return [look_at_camera(orbit_eye(4.0, 30.0, 15.0), 1920, 1080, 1080.0)]
    if cfg == 2:
        rng = np.random.Generator(np.random.PCG64(2002))
        return [look_at_camera(orbit_eye(4.0, 360.0 * v / 64, rng.uniform(-30.0, 60.0)), 1920, 1080, 1080.0) for v in range(64)]
    if cfg == 3:
        return [look_at_camera(orbit_eye(4.0, 720.0 * v / 256, -20.0 + 60.0 * v / 255), 3840, 2160, 2160.0) for v in range(256)]
    if cfg == 4:
        return [look_at_camera(orbit_eye(4.0, 20.0, 10.0), 1024, 1024, 1024.0)]
    raise ValueError(cfg)


CONFIG_SPLATS = {0: (2000, 1), 1: (500_000, 3), 2: (3_000_000, 3), 3: (6_000_000, 4), 4: (1_000_000, 3)}


def config_scene(cfg, n=None, gt_set=False):
    """The splat set of benchmark configuration `cfg` (seed 1000 + cfg; the seed-distinct ground-truth set adds 7777).
    `n` overrides the count (tests use reduced counts)."""
    n0, deg = CONFIG_SPLATS[cfg]
    n = n0 if n is None else n
    seed = 1000 + cfg + (7777 if gt_set else 0)
    if cfg == 3:
        s = make_splats(n, deg, seed, opacity=(1.0, 1.0))
    elif cfg == 4:
        s = make_splats(n, deg, seed, heavy_tail=True, bimodal_opacity=True)
    else:
        s = make_splats(n, deg, seed)
    return floor_for_cameras(s, config_cameras(cfg))
