"""Generates tests/golden/*.npz: inputs plus the outputs of the reference's own CPU check on them.

Run in a container that has the reference tree (it is built into oracle/_ref/libref.so by `make -C oracle`):
    python tests/golden/make_golden.py
The fixtures hold (1) `reference_loss` of tests/reference.cpp on small seeded scenes in the three loss modes the
reference's gradient test uses (tests/tests.cpp:398-441: transparent + alpha lane, masked with scale 1.7, plain), and
(2) central differences of that function at three step sizes for a sample of parameters, which pin the analytic
backward. The GPU box has no reference tree; its tests read these files.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from b2ctrain_b200 import scenes  # noqa: E402
from oracle import orc  # noqa: E402

F = np.float32
EPS = [1e-5, 1e-4, 4e-4]


def loss_params(mode):
    masked = mode == 1
    return dict(l1_w=F(0.8), ssim_w=F(-0.2), bg=(F(0.2), F(0.1), F(0.3)), composite=int(mode == 0), mask=int(masked),
                alpha_lane=int(mode == 0), match_alpha_weight=F(0.3), scale=F(1.7) if masked else F(1.0))


def param_ref(scene, i, p):
    if p < 3: return scene["pos_op"], (i, p)
    if p == 3: return scene["pos_op"], (i, 3)
    if p < 8: return scene["quat"], (i, p - 4)
    if p < 11: return scene["lscale"], (i, p - 8)
    return scene["sh"], (i, (p - 11) // 3, (p - 11) % 3)


def gradcheck_fixture(mode):
    scene, cam, gt, wts = scenes.gradcheck_scene(1234 + mode)
    lp = loss_params(mode)
    bg = np.array(lp["bg"], np.float64)
    ref = orc.reference_loss(scene, cam, bg, gt, wts, lp)
    K = (scene["degree"] + 1) ** 2
    per = 11 + 3 * K
    idx, fds = [], []
    for i in range(0, scene["n"], 2):
        for p in range(per):
            if p >= 11 and (p - 11) % 5:
                continue
            arr, at = param_ref(scene, i, p)
            orig = arr[at]
            row = []
            for e in EPS:
                arr[at] = orig + F(e); hi = float(arr[at]); lp_ = orc.reference_loss(scene, cam, bg, gt, wts, lp)
                arr[at] = orig - F(e); lo = float(arr[at]); lm_ = orc.reference_loss(scene, cam, bg, gt, wts, lp)
                arr[at] = orig
                row.append((lp_ - lm_) / (hi - lo))
            idx.append((i, p)); fds.append(row)
    out = dict(ref_loss=ref, fd_index=np.array(idx, np.int32), fd=np.array(fds, np.float64), fd_eps=np.array(EPS), gt=gt, wts=wts)
    out.update({f"scene_{k}": scene[k] for k in ("pos_op", "quat", "lscale", "sh")})
    out.update({f"cam_{k}": np.asarray(v) for k, v in cam.items()})
    out.update({f"lp_{k}": np.asarray(v) for k, v in lp.items()})
    out["degree"] = scene["degree"]
    return out


def config0_fixture():
    """BASELINE config 0 (2,000 splats, SH degree 1, 64x64) without the floor (the reference's CPU check has none)."""
    scene = scenes.make_splats(2000, 1, 1000)
    cam = scenes.config_cameras(0)[0]
    target = scenes.perturbed(scene, 0.01, 1000 + 7777)
    lp = dict(l1_w=F(0.8), ssim_w=F(-0.2), bg=(F(0), F(0), F(0)), composite=0, mask=0, alpha_lane=0, match_alpha_weight=F(0.1), scale=F(1.0))
    bg = np.zeros(3)
    img = orc.step(target, cam, bg, None, None, lp, backward=False, want_image=True)["rgba"]
    gt = scenes.pack_rgba8(img, alpha=np.full(64 * 64, 255))
    ref = orc.reference_loss(scene, cam, bg, gt, None, lp)
    return dict(ref_loss=ref, gt=gt)


def normals_fixture():
    """The reference's normal lane (tests/reference.cpp:67-75,132-140; gradient-test mode `normals`, tests/tests.cpp:399):
    its loss with the photometric weights at zero is a function of the composited pseudo-normal image alone."""
    scene, cam, gt, wts = scenes.gradcheck_scene(1234 + 2)
    rng = np.random.Generator(np.random.PCG64(99))
    P = cam["W"] * cam["H"]
    gtn = rng.integers(0, 2 ** 32, P, dtype=np.uint64).astype(np.uint32)   # about half of the pixels carry alpha > 127
    bg = np.array([0.2, 0.1, 0.3])
    scale = 0.05 / 100.0
    out = dict(gtn=gtn, wts=wts, normal_scale=scale,
               ref_normal_loss=orc.reference_loss_normals(scene, cam, bg, gt, gtn, None, scale),
               ref_normal_loss_weighted=orc.reference_loss_normals(scene, cam, bg, gt, gtn, wts, scale))
    return out


if __name__ == "__main__":
    assert orc.ref_lib() is not None, "oracle/_ref/libref.so is missing: run `make -C oracle` where the reference tree exists"
    here = os.path.dirname(os.path.abspath(__file__))
    only = sys.argv[1:]   # e.g. `make_golden.py normals` regenerates one fixture
    for mode in range(3):
        if not only or f"gradcheck{mode}" in only:
            np.savez_compressed(os.path.join(here, f"gradcheck_mode{mode}.npz"), **gradcheck_fixture(mode))
            print("wrote gradcheck mode", mode)
    if not only or "config0" in only:
        np.savez_compressed(os.path.join(here, "config0.npz"), **config0_fixture())
        print("wrote config0")
    if not only or "normals" in only:
        np.savez_compressed(os.path.join(here, "normals.npz"), **normals_fixture())
        print("wrote normals")
