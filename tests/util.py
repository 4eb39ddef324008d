"""Shared helpers of the test suite: golden fixtures and the GPU harness (the mould of the reference's test Harness,
tests/tests.cpp:61-102)."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Stated tolerances of the parity tests.
TOL_RECORD_REL = 2e-5      # projected records vs the double oracle (relative, with an absolute floor per field)
TOL_IMAGE_ABS = 2e-4       # rendered image, max abs
TOL_LOSS_REL = 1e-5        # loss value
TOL_GRAD_REL_L2 = 1e-4     # parameter gradients, relative L2 against the analytic double oracle
TOL_ADAM_REL = 1e-5        # Adam state after one step


def load_gradcheck(mode):
    z = np.load(os.path.join(GOLDEN, f"gradcheck_mode{mode}.npz"))
    deg = int(z["degree"])
    scene = dict(n=z["scene_pos_op"].shape[0], degree=deg, **{k: z[f"scene_{k}"].copy() for k in ("pos_op", "quat", "lscale", "sh")})
    cam = {k[4:]: z[k] for k in z.files if k.startswith("cam_")}
    cam = {k: (v if v.ndim else v.item()) for k, v in cam.items()}
    lp = {k[3:]: z[k] for k in z.files if k.startswith("lp_")}
    lp = {k: (tuple(v.tolist()) if v.ndim else v.item()) for k, v in lp.items()}
    return scene, cam, z["gt"], z["wts"], lp, z


def fd_rule_ok(analytic, fd):
    """The reference's acceptance rule (tests/tests.cpp:431-435): fail when rel > 2% AND abs > 1e-5."""
    denom = max(abs(fd), abs(analytic))
    rel = abs(fd - analytic) / denom if denom > 1e-7 else 0.0
    return not (rel > 0.02 and abs(fd - analytic) > 1e-5)


def check_against_fd(grad, z):
    """grad [n][per] vs the stored central differences of the reference's loss. A parameter passes when the analytic
    value meets the reference's rule at ANY of the stored step sizes (kinks of L1 / clamps inside one stencil do not
    then count against it); returns (fails, total, fails at the reference's own step 1e-4)."""
    fails = fails_1e4 = 0
    for (i, p), row in zip(z["fd_index"], z["fd"]):
        a = float(grad[i, p])
        ok = [fd_rule_ok(a, float(f)) for f in row]
        fails += not any(ok)
        fails_1e4 += not ok[1]
    return fails, len(z["fd_index"]), fails_1e4


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


class Harness:
    """Device model + context + view for one scene; methods return host arrays."""

    def __init__(self, scene, cam, gt=None, wts=None, lp=None, bg=None, device="cuda:0", want_depth=False, isect_cap=None):
        import torch
        from b2ctrain_b200 import api
        self.api, self.torch = api, torch
        self.scene, self.cam_d = scene, cam
        self.model = api.Model(device).upload(scene)
        self.ctx = api.RenderCtx(device)
        self.ctx.want_depth = want_depth
        self.ctx.setup(cam["W"], cam["H"], self.model.cap, isect_cap=isect_cap)
        lp = dict(lp or {})
        self.bg = tuple(float(x) for x in (bg if bg is not None else lp.get("bg", (0, 0, 0))))
        self.rp = api.RenderParams(cam, bg=self.bg, sh_degree=scene.get("active_degree", scene["degree"]), bwd_info=True)
        self.view = None
        if gt is not None:
            t_gt = torch.from_numpy(np.ascontiguousarray(gt).view(np.int32)).to(device)
            t_w = None if wts is None else torch.from_numpy(np.ascontiguousarray(wts, dtype=np.uint8)).to(device)
            self.view = api.ViewGPU(t_gt, t_w, cam["W"], cam["H"])
            lp.setdefault("bg", self.bg)
            lp["bg"] = tuple(float(x) for x in lp["bg"])
            for k in ("composite", "mask", "alpha_lane"):
                lp[k] = bool(lp.get(k, 0))
            self.lp = api.LossParams(**{k: (float(v) if isinstance(v, (np.floating, float)) else v) for k, v in lp.items()})

    def u32(self, t, n=None):
        a = t.cpu().numpy().view(np.uint32)
        return a if n is None else a[:n]

    def forward(self):
        self.api.render_forward(self.ctx, self.model, self.rp)
        return self

    def loss(self):
        self.forward()
        self.ctx.loss_accum.zero_()
        self.api.photometric_loss(self.ctx, self.view, self.lp)
        return float(self.ctx.loss_accum[0].item())

    def analytic(self):
        """Parameter gradients through the reference's debug lane OptimParams::grad_out (tests/tests.cpp:89-101)."""
        api, torch = self.api, self.torch
        K = self.model.K()
        grads = torch.zeros((self.model.n, 11 + 3 * K), dtype=torch.float32, device=self.model.device)
        val = self.loss()
        api.rasterize_backward(self.ctx, self.model, self.rp)
        op = api.OptimParams(self.cam_d, active_sh_degree=self.rp.sh_degree, grad_out=grads)
        api.optimizer_step(self.ctx, self.model, op)
        torch.cuda.synchronize()
        return val, grads.cpu().numpy()
