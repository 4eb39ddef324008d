"""ctypes bindings of the CPU oracle (liboracle.so) and of the reference's own CPU check (_ref/libref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's CPU-baseline leg, never by
the package. Build with `make -C oracle`.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORC_REC = 16
MX, MY, C00, C01, C11, OPAC, Z, POWER, R, G, B, EX, EY, OK, MAXSCREEN = range(15)


class OrcCamera(C.Structure):
    _fields_ = [("R", C.c_float * 9), ("t", C.c_float * 3), ("pos", C.c_float * 3), ("fx", C.c_float), ("fy", C.c_float),
                ("cx", C.c_float), ("cy", C.c_float), ("W", C.c_int32), ("H", C.c_int32), ("lim_pos_x", C.c_float),
                ("lim_pos_y", C.c_float), ("lim_neg_x", C.c_float), ("lim_neg_y", C.c_float)]


class OrcLoss(C.Structure):
    _fields_ = [("l1_w", C.c_float), ("ssim_w", C.c_float), ("bg", C.c_float * 3), ("composite", C.c_int32),
                ("mask", C.c_int32), ("alpha_lane", C.c_int32), ("match_alpha_weight", C.c_float), ("scale", C.c_float),
                ("grad_scale", C.c_float)]


class OrcAdam(C.Structure):
    _fields_ = [("t", C.c_int32), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float), ("lr_mean", C.c_float),
                ("lr_rot", C.c_float), ("lr_scale", C.c_float), ("lr_opac", C.c_float), ("lr_dc", C.c_float),
                ("lr_sh_rest", C.c_float), ("sparse", C.c_int32)]


_lib = None
_ref = None


def reference_tree():
    """Where the reference checkout lies, or None: the B2C_REFERENCE environment variable, else a `reference` folder
    beside the repository."""
    for cand in (os.environ.get("B2C_REFERENCE"), os.path.join(_HERE, "..", "..", "reference")):
        if cand and os.path.isfile(os.path.join(cand, "tests", "reference.cpp")):
            return os.path.abspath(cand)
    return None


def build():
    import subprocess
    ref = reference_tree()
    subprocess.run(["make", "-C", _HERE] + ([f"REF={ref}"] if ref else []), check=True, capture_output=True)


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _lib = C.CDLL(path)
        _lib.orc_loss.restype = C.c_double
        _lib.orc_step.restype = C.c_double
        _lib.orc_bin.restype = C.c_int64
    return _lib


def ref_lib():
    """The reference's unmodified CPU check, or None when it was never built here."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libref.so")
        if not os.path.exists(path):
            return None
        _ref = C.CDLL(path)
        _ref.ref_reference_loss.restype = C.c_double
    return _ref


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _f64(a):
    return np.ascontiguousarray(a, dtype=np.float64)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def camera_struct(cam):
    """cam: dict with R[9], t[3], pos[3], fx, fy, cx, cy, W, H and the four Jacobian clamp limits."""
    s = OrcCamera()
    for i in range(9):
        s.R[i] = float(cam["R"][i])
    for i in range(3):
        s.t[i] = float(cam["t"][i])
        s.pos[i] = float(cam["pos"][i])
    for k in ("fx", "fy", "cx", "cy", "lim_pos_x", "lim_pos_y", "lim_neg_x", "lim_neg_y"):
        setattr(s, k, float(cam[k]))
    s.W, s.H = int(cam["W"]), int(cam["H"])
    return s


def loss_struct(lp):
    s = OrcLoss()
    s.l1_w, s.ssim_w = lp.get("l1_w", 0.8), lp.get("ssim_w", -0.2)
    for i in range(3):
        s.bg[i] = float(lp.get("bg", (0, 0, 0))[i])
    s.composite, s.mask, s.alpha_lane = int(lp.get("composite", 0)), int(lp.get("mask", 0)), int(lp.get("alpha_lane", 0))
    s.match_alpha_weight, s.scale, s.grad_scale = lp.get("match_alpha_weight", 0.1), lp.get("scale", 1.0), lp.get("grad_scale", 1.0)
    return s


def adam_struct(op):
    s = OrcAdam()
    s.t = int(op.get("t", 1))
    s.beta1, s.beta2, s.eps = op.get("beta1", 0.9), op.get("beta2", 0.999), op.get("eps", 1e-15)
    s.lr_mean, s.lr_rot, s.lr_scale = op.get("lr_mean", 0.0), op.get("lr_rot", 2e-3), op.get("lr_scale", 5e-3)
    s.lr_opac, s.lr_dc, s.lr_sh_rest = op.get("lr_opac", 0.012), op.get("lr_dc", 2e-3), op.get("lr_sh_rest", 2e-4)
    s.sparse = int(op.get("sparse", 0))
    return s


def project(scene, cam, active_degree=None):
    n, deg = scene["n"], scene["degree"]
    act = deg if active_degree is None else active_degree
    rec = np.zeros((n, ORC_REC), np.float64)
    cs = camera_struct(cam)
    lib().orc_project(n, deg, act, _p(_f32(scene["pos_op"])), _p(_f32(scene["quat"])), _p(_f32(scene["lscale"])),
                      _p(_f32(scene["sh"])), C.byref(cs), _p(rec))
    return rec


def records_to_proj(rec):
    """Double records -> the fp32 (proj0, proj1) pair the binning stage consumes; power = -1 marks 'no record'."""
    ok = rec[:, OK] != 0
    p0 = rec[:, [MX, MY, C00, C01]].astype(np.float32)
    p1 = rec[:, [C11, OPAC, Z, POWER]].astype(np.float32)
    p1[~ok, 3] = -1.0
    return np.ascontiguousarray(p0), np.ascontiguousarray(p1)


def tiles_of_record(r, W, H, max_tiles=4096):
    tiles = np.zeros(max_tiles, np.uint32)
    f = C.c_float
    k = lib().orc_tiles_of_record(f(r[0]), f(r[1]), f(r[2]), f(r[3]), f(r[4]), f(r[5]), W, H, _p(tiles), max_tiles)
    return tiles[:min(k, max_tiles)], k


def bin_sort(p0, p1, W, H):
    n = p0.shape[0]
    n_tiles = ((W + 7) // 8) * ((H + 7) // 8)
    p0, p1 = _f32(p0), _f32(p1)
    tile_count = np.zeros(n, np.uint32)
    ranges = np.zeros((n_tiles, 2), np.uint32)
    total = lib().orc_bin(n, _p(p0), _p(p1), W, H, _p(tile_count), None, None, C.c_int64(0), _p(ranges))
    vals = np.zeros(max(total, 1), np.uint32)
    keys = np.zeros(max(total, 1), np.uint32)
    lib().orc_bin(n, _p(p0), _p(p1), W, H, _p(tile_count), _p(vals), _p(keys), C.c_int64(total), _p(ranges))
    return tile_count, vals[:total], keys[:total], ranges


def raster_fwd(W, H, geo, col, vals, ranges, bg, bwd_info=True, want_depth=False):
    P = W * H
    geo, col = _f64(geo), _f64(col)
    ranges = np.array(ranges, dtype=np.uint32, copy=True)
    rgba = np.zeros((P, 4)); T = np.zeros(P); last = np.zeros(P, np.uint32)
    depth = np.zeros(P) if want_depth else None
    bgd = _f64(bg)
    vals = _u32(vals) if len(vals) else np.zeros(1, np.uint32)
    lib().orc_raster_fwd(W, H, _p(geo), _p(col), _p(vals), _p(ranges), _p(bgd), int(bwd_info), _p(rgba), _p(T), _p(last), _p(depth))
    return rgba, T, last, ranges, depth


def features(scene, cam, mode, feat_buffer=None):
    """Per-splat feature lanes [n][3]: mode 1 pseudo-normals, mode 2 the caller's buffer (clamped)."""
    n = scene["n"]
    out = np.zeros((n, 3), np.float64)
    cs = camera_struct(cam)
    fb = None if feat_buffer is None else _f32(feat_buffer)
    lib().orc_features(n, int(mode), _p(_f32(scene["pos_op"])), _p(_f32(scene["quat"])), _p(_f32(scene["lscale"])), _p(fb), C.byref(cs), _p(out))
    return out


def raster_feat(W, H, geo, feat, vals, ranges):
    """Composited feature image [P][3] over the lists of bin_sort (same walk as raster_fwd)."""
    out = np.zeros((W * H, 3), np.float64)
    vals = _u32(vals) if len(vals) else np.zeros(1, np.uint32)
    rng = np.ascontiguousarray(ranges, dtype=np.uint32)
    lib().orc_raster_feat(W, H, _p(_f64(geo)), _p(_f64(feat)), _p(vals), _p(rng), _p(out))
    return out


def normal_loss_of(feat_img, gtn, weights, normal_scale):
    """The reference's normal loss (src/gpu/loss.cu normal_loss_kernel; tests/reference.cpp:132-140) of a composited
    feature image, in numpy: L1 + (1 - cosine) on the pixels whose packed target has alpha > 127."""
    g = np.asarray(gtn, np.uint32)
    on = ((g >> 24) & 0xFF) > 127
    gx = (g & 0xFF) * (2.0 / 255.0) - 1.0
    gy = 1.0 - ((g >> 8) & 0xFF) * (2.0 / 255.0)
    gz = 1.0 - ((g >> 16) & 0xFF) * (2.0 / 255.0)
    wp = np.ones(len(g)) if weights is None else np.asarray(weights, np.float64) / 255.0
    px, py, pz = feat_img[:, 0], feat_img[:, 1], feat_img[:, 2]
    pl = np.maximum(np.sqrt(px * px + py * py + pz * pz), 1e-6)
    gl = np.maximum(np.sqrt(gx * gx + gy * gy + gz * gz), 1e-6)
    per = normal_scale * wp * (np.abs(px - gx) + np.abs(py - gy) + np.abs(pz - gz) + 1.0 - (px * gx + py * gy + pz * gz) / (pl * gl))
    return float(per[on].sum())


def reference_loss_normals(scene, cam, bg, gt, gtn, weights, normal_scale, l1_w=0.0, ssim_w=0.0, scale=1.0):
    """The reference's `reference_loss` with its normal lane on (pseudo-normal features)."""
    r = ref_lib()
    if r is None or not hasattr(r, "ref_reference_loss_normals"):
        return None
    n, deg = scene["n"], scene["degree"]
    assert deg <= 3 and not np.any(scene["lscale"][:, 3] != 0)
    pos = _f32(scene["pos_op"][:, :3]); opac = _f32(scene["pos_op"][:, 3]); ls = _f32(scene["lscale"][:, :3])
    intr = np.array([cam["fx"], cam["fy"], cam["cx"], cam["cy"]], np.float32)
    w = None if weights is None else np.ascontiguousarray(weights, dtype=np.uint8)
    d = C.c_double
    r.ref_reference_loss_normals.restype = C.c_double
    return r.ref_reference_loss_normals(n, deg, _p(pos), _p(ls), _p(_f32(scene["quat"])), _p(opac), _p(_f32(scene["sh"])), int(cam["W"]), int(cam["H"]),
                                        _p(intr), _p(_f32(cam["R"])), _p(_f32(cam["t"])), _p(_f32(cam["pos"])), _p(_f64(bg)), d(l1_w), d(ssim_w),
                                        d(scale), _p(_u32(gt)), _p(_u32(gtn)), d(normal_scale), _p(w))


def loss(W, H, pred, gt, weights, lp, want_grad=True):
    pred = _f64(pred)
    v_out = np.zeros((W * H, 4)) if want_grad else None
    ls = loss_struct(lp)
    w = None if weights is None else np.ascontiguousarray(weights, dtype=np.uint8)
    val = lib().orc_loss(W, H, _p(pred), _p(_u32(gt)), _p(w), C.byref(ls), _p(v_out))
    return val, v_out


def eval_metrics(W, H, pred, gt, mask_weighted=False):
    """eval_kernel (src/gpu/loss.cu:241-293) in double: the prediction is clamped and quantised to 8 bits (in fp32, as
    the device decides the rounding), the target is taken on black, SSIM uses the 11-tap sigma-1.5 window with zero
    padding, variances clamped at zero, SSIM clamped to [-1, 1]; with mask_weighted the per-pixel error and SSIM are
    multiplied by the target's alpha. Returns (sum of squared errors, sum of SSIM) over pixels and channels."""
    from scipy.ndimage import correlate1d
    p32 = np.clip(np.asarray(pred, np.float32).reshape(H, W, 4)[:, :, :3], np.float32(0), np.float32(1)) * np.float32(255)
    q = np.rint(p32).astype(np.float64) / 255.0
    g = np.asarray(gt, np.uint32).reshape(H, W)
    t = np.stack([((g >> (8 * c)) & 0xFF).astype(np.float64) / 255.0 for c in range(3)], -1)
    m = ((g >> 24) & 0xFF).astype(np.float64) / 255.0 if mask_weighted else np.ones((H, W))
    x = np.arange(11) - 5.0
    w = np.exp(-x * x / (2 * 1.5 * 1.5)); w /= w.sum()
    blur = lambda a: correlate1d(correlate1d(a, w, axis=0, mode="constant"), w, axis=1, mode="constant")
    C1, C2 = 0.01 ** 2, 0.03 ** 2
    se = ssim_sum = 0.0
    for c in range(3):
        a, b = q[:, :, c], t[:, :, c]
        mu1, mu2 = blur(a), blur(b)
        s1, s2, s12 = np.maximum(blur(a * a) - mu1 * mu1, 0), np.maximum(blur(b * b) - mu2 * mu2, 0), blur(a * b) - mu1 * mu2
        ssim = np.clip(((2 * mu1 * mu2 + C1) * (2 * s12 + C2)) / ((mu1 * mu1 + mu2 * mu2 + C1) * (s1 + s2 + C2)), -1, 1)
        se += float(((np.abs(a - b) * m) ** 2).sum())
        ssim_sum += float((ssim * m).sum())
    return se, ssim_sum


def raster_bwd(n, W, H, geo, col, vals, ranges, bg, rgba, T, last, v_out):
    v_splat = np.zeros((n, 13)); vis = np.zeros(n, np.uint32); visw = np.zeros(n)
    vals = _u32(vals) if len(vals) else np.zeros(1, np.uint32)
    lib().orc_raster_bwd(n, W, H, _p(_f64(geo)), _p(_f64(col)), _p(vals), _p(_u32(ranges)), _p(_f64(bg)), _p(_f64(rgba)),
                         _p(_f64(T)), _p(_u32(last)), _p(_f64(v_out)), _p(v_splat), _p(vis), _p(visw))
    return v_splat, vis, visw


def proj_bwd(scene, cam, v_splat, vis, tile_count, active_degree=None):
    n, deg = scene["n"], scene["degree"]
    act = deg if active_degree is None else active_degree
    K = (deg + 1) ** 2
    grad = np.zeros((n, 11 + 3 * K))
    cs = camera_struct(cam)
    lib().orc_proj_bwd(n, deg, act, _p(_f32(scene["pos_op"])), _p(_f32(scene["quat"])), _p(_f32(scene["lscale"])),
                       _p(_f32(scene["sh"])), C.byref(cs), _p(_f64(v_splat)), _p(_u32(vis)), _p(_u32(tile_count)), _p(grad))
    return grad


def adam(state, grad, active, op, degree):
    """state: dict of fp32 arrays pos_op, quat, lscale, sh[n][K][3], m_pos, v_pos, m_q, v_q, m_ls, v_ls, m_sh, v_sh and
    uint32 last_step; updated in place (arrays must be C-contiguous and of the right dtype)."""
    n = state["pos_op"].shape[0]
    s = adam_struct(op)
    act = np.ascontiguousarray(active, dtype=np.uint8)
    keys = ["pos_op", "quat", "lscale", "sh", "m_pos", "v_pos", "m_q", "v_q", "m_ls", "v_ls", "m_sh", "v_sh"]
    for k in keys:
        assert state[k].dtype == np.float32 and state[k].flags["C_CONTIGUOUS"], k
    assert state["last_step"].dtype == np.uint32
    lib().orc_adam(n, degree, *[_p(state[k]) for k in keys], _p(state["last_step"]), _p(_f64(grad)), _p(act), C.byref(s))


def min_scale(pos_op, lscale, cam_pos, cam_focal):
    ls = np.array(lscale, dtype=np.float32, copy=True)
    cp, cf = _f32(cam_pos), _f32(cam_focal)
    lib().orc_min_scale(pos_op.shape[0], _p(_f32(pos_op)), _p(ls), _p(cp), _p(cf), len(cf))
    return ls


def step(scene, cam, bg, gt, weights, lp, backward=True, want_image=False):
    """Pure double chain: forward + loss (+ analytic backward). Returns dict(loss, grad, rgba, counters)."""
    n, deg = scene["n"], scene["degree"]
    K = (deg + 1) ** 2
    W, H = cam["W"], cam["H"]
    rgba = np.zeros((W * H, 4)) if want_image else None
    grad = np.zeros((n, 11 + 3 * K)) if backward else None
    counters = np.zeros(4, np.int64)
    cs, ls = camera_struct(cam), loss_struct(lp)
    w = None if weights is None else np.ascontiguousarray(weights, dtype=np.uint8)
    g = None if gt is None else _u32(gt)
    val = lib().orc_step(n, deg, scene.get("active_degree", deg), _p(_f32(scene["pos_op"])), _p(_f32(scene["quat"])),
                         _p(_f32(scene["lscale"])), _p(_f32(scene["sh"])), C.byref(cs), _p(_f64(bg)), _p(g), _p(w),
                         C.byref(ls), int(backward), _p(rgba), _p(grad), _p(counters))
    return dict(loss=val, grad=grad, rgba=rgba, V=int(counters[0]), I=int(counters[1]), I_b=int(counters[2]))


def reference_loss(scene, cam, bg, gt, weights, lp):
    """The reference's own `reference_loss` (no floor, SH degree <= 3)."""
    r = ref_lib()
    if r is None:
        return None
    n, deg = scene["n"], scene["degree"]
    assert deg <= 3 and not np.any(scene["lscale"][:, 3] != 0), "reference_loss has no floor and stops at SH degree 3"
    pos = _f32(scene["pos_op"][:, :3]); opac = _f32(scene["pos_op"][:, 3]); ls = _f32(scene["lscale"][:, :3])
    intr = np.array([cam["fx"], cam["fy"], cam["cx"], cam["cy"]], np.float32)
    w = None if weights is None else np.ascontiguousarray(weights, dtype=np.uint8)
    d = C.c_double
    return r.ref_reference_loss(n, deg, _p(pos), _p(ls), _p(_f32(scene["quat"])), _p(opac), _p(_f32(scene["sh"])),
                                int(cam["W"]), int(cam["H"]), _p(intr), _p(_f32(cam["R"])), _p(_f32(cam["t"])),
                                _p(_f32(cam["pos"])), _p(_f64(bg)), int(lp.get("composite", 0)), int(lp.get("mask", 0)),
                                int(lp.get("alpha_lane", 0)), d(lp.get("l1_w", 0.8)), d(lp.get("ssim_w", -0.2)),
                                d(lp.get("match_alpha_weight", 0.1)), d(lp.get("scale", 1.0)), _p(_u32(gt)), _p(w))


def num_threads():
    return int(lib().orc_num_threads())


def set_num_threads(n):
    """OpenMP threads of the oracle's loops (a launcher may have exported OMP_NUM_THREADS=1 to this process)."""
    lib().orc_set_num_threads(int(n))


# ---- the reference's own CUDA kernels (oracle/_ref/librefcuda.so), second oracle and speed incumbent ----

_refcu = None


def refcuda_lib():
    """The reference's unmodified CUDA implementation built for sm_100a, or None when it was never built here."""
    global _refcu
    if _refcu is None:
        path = os.path.join(_HERE, "_ref", "librefcuda.so")
        if not os.path.exists(path):
            return None
        _refcu = C.CDLL(path)
        _refcu.refcu_create.restype = C.c_void_p
        _refcu.refcu_error.restype = C.c_char_p
        _refcu.refcu_num_isect.restype = C.c_uint32
        _refcu.refcu_time_steps.restype = C.c_float
    return _refcu


class RefCuda:
    """One scene + view on the reference's CUDA path. Methods mirror the reference's test Harness (tests/tests.cpp:61-102)."""

    def __init__(self, scene, cam):
        self.l = refcuda_lib()
        assert self.l is not None, "oracle/_ref/librefcuda.so is missing"
        self.scene, self.cam = scene, cam
        n, self.W, self.H = scene["n"], int(cam["W"]), int(cam["H"])
        self.K = (scene["degree"] + 1) ** 2
        floor = _f32(scene["lscale"][:, 3])
        self.h = C.c_void_p(self.l.refcu_create(n, scene["degree"], _p(_f32(scene["pos_op"][:, :3])), _p(_f32(scene["lscale"][:, :3])), _p(_f32(scene["quat"])),
                                                _p(_f32(scene["pos_op"][:, 3])), _p(_f32(scene["sh"])), _p(floor) if np.any(floor != 0) else None, self.W, self.H))
        self._check(0)
        self.intr = np.array([cam["fx"], cam["fy"], cam["cx"], cam["cy"]], np.float32)
        self.R, self.t = _f32(cam["R"]), _f32(cam["t"])

    def _check(self, rc):
        err = self.l.refcu_error(self.h).decode()
        if rc != 0 or err:
            raise RuntimeError(f"reference CUDA path: {err}")

    def close(self):
        if self.h:
            self.l.refcu_destroy(self.h)
            self.h = None

    def set_view(self, gt, weights=None):
        w = None if weights is None else np.ascontiguousarray(weights, dtype=np.uint8)
        self._check(self.l.refcu_set_view(self.h, _p(_u32(gt)), _p(w)))

    def forward(self, bg=(0, 0, 0), bwd_info=True):
        self.bg = _f32(bg)
        self._check(self.l.refcu_forward(self.h, _p(self.intr), _p(self.R), _p(self.t), _p(self.bg), int(bwd_info)))

    def loss(self, lp):
        p = np.array([lp.get("l1_w", 0.8), lp.get("ssim_w", -0.2), *lp.get("bg", (0, 0, 0)), lp.get("match_alpha_weight", 0.1), lp.get("scale", 1.0),
                      lp.get("grad_scale", 1.0)], np.float32)
        f = np.array([int(lp.get("composite", 0)), int(lp.get("mask", 0)), int(lp.get("alpha_lane", 0))], np.int32)
        out = C.c_float(0)
        self._check(self.l.refcu_loss(self.h, _p(p), _p(f), C.byref(out)))
        return float(out.value)

    def backward(self, tensor_core=False, grad_scale=1.0):
        self._check(self.l.refcu_backward(self.h, _p(self.intr), _p(self.R), _p(self.t), _p(self.bg), int(tensor_core), C.c_float(grad_scale)))

    def grads(self):
        out = np.zeros((self.scene["n"], 11 + 3 * self.K), np.float32)
        self._check(self.l.refcu_grads(self.h, _p(self.intr), _p(self.R), _p(self.t), _p(out)))
        return out

    def optim(self, t=1, sparse=True, lr_mean=1.6e-4, lr_rot=2e-3, lr_scale=5e-3, lr_opac=0.012, lr_dc=2e-3, lr_sh_rest=2e-4, noise_weight=0.0,
              noise_clamp=0.0, seed=42, step=0):
        """optimizer_step (src/gpu/optim.h:50) on the lanes the context holds, with the camera of the last forward."""
        f = np.array([lr_mean, lr_rot, lr_scale, lr_opac, lr_dc, lr_sh_rest, noise_weight, noise_clamp], np.float32)
        u = np.array([t, int(sparse), seed, step], np.uint32)
        self._check(self.l.refcu_optim_full(self.h, _p(self.intr), _p(self.R), _p(self.t), _p(f), _p(u)))

    def set_lanes(self, v_splat, vis_flag):
        self._check(self.l.refcu_set_lanes(self.h, _p(_f32(v_splat)), _p(_u32(vis_flag))))

    def set_image(self, rgba):
        self._check(self.l.refcu_set_image(self.h, _p(_f32(rgba))))

    def eval_metrics(self, mask_weighted=False):
        out = np.zeros(2, np.float32)
        self._check(self.l.refcu_eval(self.h, int(mask_weighted), _p(out)))
        return float(out[0]), float(out[1])

    def v_out(self):
        out = np.zeros((self.W * self.H, 4), np.float32)
        self._check(self.l.refcu_v_out(self.h, _p(out)))
        return out

    def cap(self):
        return int(self.l.refcu_cap(self.h))

    def model_state(self):
        """Parameters and Adam state as host arrays in the layout of Model.download / the oracle's state dict."""
        n, K, cap = self.scene["n"], self.K, self.cap()
        d4 = lambda k: self.download(k, (n, 4), np.float32)

        def planar(dc, hi):
            a = self.download(dc, (3, cap), np.float32)
            b = self.download(hi, (3 * (K - 1), cap), np.float32) if K > 1 else np.zeros((0, cap), np.float32)
            return np.ascontiguousarray(np.concatenate([a, b], 0)[:, :n].T.reshape(n, K, 3))
        return dict(pos_op=d4("pos_op"), quat=d4("quat"), lscale=d4("lscale"), sh=planar("sh_dc", "sh_hi32"), m_pos=d4("m_pos_op"), v_pos=d4("v_pos_op"),
                    m_q=d4("m_quat"), v_q=d4("v_quat"), m_ls=d4("m_lscale"), v_ls=d4("v_lscale"), m_sh=planar("m_sh_dc", "m_sh_hi32"),
                    v_sh=self.download("v_sh", (n,), np.float32), last_step=self.download("last_step", (n,), np.uint32),
                    vis_count=self.download("vis_count", (n,), np.float32), refine_norm=self.download("refine_norm", (n,), np.float32))

    def refine(self, stats, cam_pos, cam_focal, iter=1000, total=30000, growth_allowed=True, max_splats=10_000_000, growth_grad_threshold=0.0025,
               growth_select_fraction=0.25, split_at_screen_size=0.5, opac_decay=0.004, seed=42, no_new=False, cull_weight=0.0):
        """RefineState::run (src/gpu/refine.h) on the handle's model; stats [4][n] = refine_norm, max_screen, vis_count, vis_weight.
        Returns dict(n, pruned, relocated, grown, split_oversized, culled); the model's n changes with it."""
        fp = np.array([growth_grad_threshold, growth_select_fraction, split_at_screen_size, opac_decay, cull_weight], np.float32)
        up = np.array([iter, total, int(growth_allowed), max_splats, seed, int(no_new)], np.uint32)
        out = np.zeros(6, np.int32)
        self._check(self.l.refcu_refine(self.h, _p(_f32(stats)), _p(_f32(cam_pos)), _p(_f32(cam_focal)), len(cam_focal), _p(fp), _p(up), _p(out)))
        self.scene = dict(self.scene, n=int(out[0]))
        return dict(zip(("n", "pruned", "relocated", "grown", "split_oversized", "culled"), (int(x) for x in out)))

    def evidence(self, cams, labels=None, masked=False, has_alpha=False):
        """compute_evidence (src/train/evidence.h) over the cameras, all against the view set with set_view; returns
        (evidence [n][7], labels [n][2] or None)."""
        rows = np.concatenate([np.concatenate([[c["fx"], c["fy"], c["cx"], c["cy"]], _f32(c["R"]), _f32(c["t"])]) for c in cams]).astype(np.float32)
        n = self.scene["n"]
        ev = np.zeros((n, 7), np.float32)
        lab = None if labels is None else np.zeros((n, 2), np.float32)
        lb = None if labels is None else np.ascontiguousarray(labels, dtype=np.uint8)
        self._check(self.l.refcu_evidence(self.h, len(cams), _p(rows), _p(lb), int(masked), int(has_alpha), _p(ev), _p(lab)))
        return ev, lab

    def download(self, what, shape, dtype):
        sel = dict(proj0=0, proj1=1, proj2=2, tile_count=3, vals_sorted=4, keys_sorted=5, tile_ranges=6, out_rgba=7, last_idx=8, v_splat=9, pos_op=10, quat=11,
                   lscale=12, sh_dc=13, sh_hi32=14, m_pos_op=15, v_pos_op=16, m_quat=17, v_quat=18, m_lscale=19, v_lscale=20, m_sh_dc=21, m_sh_hi32=22,
                   v_sh=23, last_step=24, vis_count=25, refine_norm=26, out_feat=27)[what]
        out = np.zeros(shape, dtype)
        self._check(self.l.refcu_download(self.h, sel, _p(out), C.c_size_t(out.nbytes)))
        return out

    def num_isect(self):
        return int(self.l.refcu_num_isect(self.h))

    def time_steps(self, bg=(0, 0, 0), tensor_core=True, warm=3, iters=10, lr_mean=1e-5):
        ms = self.l.refcu_time_steps(self.h, _p(self.intr), _p(self.R), _p(self.t), _p(_f32(bg)), int(tensor_core), warm, iters, C.c_float(lr_mean))
        self._check(0 if ms >= 0 else 1)
        return float(ms)
