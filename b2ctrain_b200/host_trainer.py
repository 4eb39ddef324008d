"""ctypes binding of the C++ host library (libb2chost.so): the reference's step loop (src/train/trainer.cpp:452-529)
with views in flight and view-level data parallelism, run entirely in C++ (b2ctrain_b200/host/trainer.cpp). Python only
hands over the scene, the views and a CUDA stream; no step logic, collective or kernel launch happens on this side.
"""
import ctypes as C
import os

import numpy as np

from . import api

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb2chost.so")


class B2chConfig(C.Structure):
    _fields_ = [("views_in_flight", C.c_int32), ("render_chunks", C.c_int32), ("isect_cap", C.c_uint64), ("ssim_weight", C.c_float),
                ("mask", C.c_int32), ("alpha_lane", C.c_int32), ("composite", C.c_int32), ("match_alpha_weight", C.c_float), ("loss_scale", C.c_float),
                ("bg", C.c_float * 3), ("lr_mean", C.c_float), ("lr_rot", C.c_float), ("lr_scale", C.c_float), ("lr_opac", C.c_float), ("lr_dc", C.c_float),
                ("lr_sh_rest", C.c_float), ("sparse", C.c_int32), ("noise_weight", C.c_float), ("noise_clamp", C.c_float), ("seed", C.c_uint32),
                ("shard_update", C.c_int32)]


_P = C.c_void_p
SIGNATURES = {
    "b2ch_last_error": (C.c_char_p, []),
    "b2ch_trainer_create": (C.c_void_p, [C.c_int32, C.c_int32, _P, _P, _P, _P, C.c_int32, C.c_int32, _P, C.c_int32, C.c_int32, _P]),
    "b2ch_trainer_destroy": (None, [_P]),
    "b2ch_trainer_add_view": (C.c_int, [_P, _P, _P]),
    "b2ch_trainer_step": (C.c_int, [_P, _P, C.c_int32, _P, C.c_int32]),
    "b2ch_trainer_read_loss": (C.c_int, [_P, _P, _P]),
    "b2ch_trainer_set_profile": (C.c_int, [_P, C.c_int32]),
    "b2ch_trainer_info": (C.c_int, [_P, _P]),
    "b2ch_trainer_download": (C.c_int, [_P, _P, _P, _P, _P]),
    "b2ch_trainer_reduce_statistics": (C.c_int, [_P, _P]),
    "b2ch_trainer_checksum": (C.c_uint64, [_P, _P]),
    "b2ch_trainer_refine": (C.c_int, [_P, _P, _P, C.c_int32, _P, _P, _P, _P]),
    "b2ch_refine_once": (C.c_int, [C.c_int32, C.c_int32, _P, _P, _P, _P, _P, _P, _P, C.c_int32, _P, _P, C.c_int32, C.c_int32, _P, C.c_int32, _P, _P, _P, _P, _P]),
    "b2ch_renderer_create": (_P, [C.c_int32, C.c_int32, _P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_uint64]),
    "b2ch_renderer_destroy": (None, [_P]),
    "b2ch_renderer_render": (C.c_int, [_P, _P, _P, C.c_int32, _P, _P, _P]),
    "b2ch_renderer_finish": (C.c_int, [_P]),
    "b2ch_renderer_info": (C.c_int, [_P, _P]),
    "b2ch_render_headless": (C.c_int, [C.c_char_p, C.c_char_p, C.c_char_p, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P]),
    "b2ch_ply_read": (C.c_int, [C.c_char_p, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "b2ch_ply_write": (C.c_int, [C.c_char_p, C.c_int32, C.c_int32, _P, _P, _P, _P, _P, _P, _P, C.c_char_p]),
}

_lib = None


def lib():
    """Loads libb2chost.so (and libb2k.so, which it links); raises when it has not been built."""
    global _lib
    if _lib is None:
        api.lib()
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `make -C b2ctrain_b200/host`")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            f = getattr(l, name)
            f.restype, f.argtypes = res, args
        _lib = l
    return _lib


def _check(status, what):
    if status != 0:
        raise RuntimeError(f"{what}: {lib().b2ch_last_error().decode()}")


def make_dp_id():
    """The 128-byte rendezvous id rank 0 creates (b2k_dp_unique_id) and sends to the other ranks."""
    buf = (C.c_uint8 * 128)()
    api._check(api.lib().b2k_dp_unique_id(buf), "b2k_dp_unique_id")
    return bytes(buf)


def dp_slice(n, rank, world):
    """(first, count) of the splats whose update `rank` owns in the sharded data-parallel step (b2k_dp_slice)."""
    a, b = C.c_int32(0), C.c_int32(0)
    api._check(api.lib().b2k_dp_slice(int(n), int(rank), int(world), C.byref(a), C.byref(b)), "b2k_dp_slice")
    return a.value, b.value


class HostTrainer:
    """b2c::StepTrainer behind the C entry points. `scene` is the host dict of b2ctrain_b200.scenes."""

    def __init__(self, scene, W, H, rank=0, world=1, dp_id=None, views_in_flight=4, render_chunks=1, isect_cap=0, ssim_weight=0.2, mask=False,
                 alpha_lane=False, composite=False, match_alpha_weight=0.1, loss_scale=1.0, bg=(0.0, 0.0, 0.0), lr_mean=0.0, lr_rot=2e-3, lr_scale=5e-3,
                 lr_opac=0.012, lr_dc=2e-3, lr_sh_rest=2e-4, sparse=True, noise_weight=0.0, noise_clamp=0.0, seed=42, shard_update=True):
        cfg = B2chConfig()
        cfg.views_in_flight, cfg.render_chunks, cfg.isect_cap, cfg.ssim_weight = int(views_in_flight), int(render_chunks), int(isect_cap or 0), ssim_weight
        cfg.mask, cfg.alpha_lane, cfg.composite = int(mask), int(alpha_lane), int(composite)
        cfg.match_alpha_weight, cfg.loss_scale = match_alpha_weight, loss_scale
        for i in range(3):
            cfg.bg[i] = float(bg[i])
        cfg.lr_mean, cfg.lr_rot, cfg.lr_scale, cfg.lr_opac, cfg.lr_dc, cfg.lr_sh_rest = lr_mean, lr_rot, lr_scale, lr_opac, lr_dc, lr_sh_rest
        cfg.sparse, cfg.noise_weight, cfg.noise_clamp, cfg.seed, cfg.shard_update = int(sparse), noise_weight, noise_clamp, int(seed), int(shard_update)
        f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
        self.n, self.degree, self.W, self.H = int(scene["n"]), int(scene["degree"]), int(W), int(H)
        arrays = [f32(scene[k]) for k in ("pos_op", "quat", "lscale", "sh")]
        idbuf = None if dp_id is None else (C.c_uint8 * 128).from_buffer_copy(dp_id)
        self.h = lib().b2ch_trainer_create(self.n, self.degree, *[a.ctypes.data_as(_P) for a in arrays], self.W, self.H, C.byref(cfg), int(rank), int(world), idbuf)
        if not self.h:
            raise RuntimeError(f"b2ch_trainer_create: {lib().b2ch_last_error().decode()}")
        self.h = C.c_void_p(self.h)

    def close(self):
        if self.h:
            lib().b2ch_trainer_destroy(self.h)
            self.h = None

    def add_view(self, cam, rgba):
        """cam: camera dict of b2ctrain_b200.scenes; rgba: packed RGBA8 target as a numpy array (or anything exposing a
        buffer of W * H 32-bit words). Returns the view's index."""
        c = api.camera_from(cam)
        ptr = None
        if rgba is not None:   # None: a view another rank renders (only its camera is known here)
            t = np.ascontiguousarray(np.asarray(rgba).view(np.uint32))
            assert t.size == self.W * self.H
            ptr = t.ctypes.data_as(_P)
        idx = lib().b2ch_trainer_add_view(self.h, C.byref(c), ptr)
        if idx < 0:
            raise RuntimeError(f"b2ch_trainer_add_view: {lib().b2ch_last_error().decode()}")
        return idx

    def step(self, views, stream, from_host=False):
        """One optimisation step over the views (indices), enqueued on the CUDA stream given as an integer handle."""
        arr = (C.c_int32 * len(views))(*views)
        _check(lib().b2ch_trainer_step(self.h, arr, len(views), C.c_void_p(int(stream)), int(from_host)), "b2ch_trainer_step")

    def read_loss(self, stream):
        out = (C.c_float * 16)()
        _check(lib().b2ch_trainer_read_loss(self.h, out, C.c_void_p(int(stream))), "b2ch_trainer_read_loss")
        return np.array(out[:], np.float32)

    def set_profile(self, on):
        lib().b2ch_trainer_set_profile(self.h, int(on))

    def info(self):
        out = (C.c_uint64 * 11)()
        _check(lib().b2ch_trainer_info(self.h, out), "b2ch_trainer_info")
        ms = np.frombuffer(bytes(out)[64:88], np.float32)
        return dict(isect_cap=int(out[0]), overflow_redos=int(out[1]), h2d_bytes=int(out[2]), n=int(out[3]), adam_t=int(out[4]), lanes=int(out[5]),
                    views=int(out[6]), tile_bits=int(out[7]), phase_ms=dict(views=float(ms[0]), update=float(ms[1]), step=float(ms[2]), update_wait=float(ms[3]), update_kernel=float(ms[4]),
                                  update_barrier=float(ms[5])))

    def download(self):
        K = (self.degree + 1) ** 2
        a = [np.zeros((self.n, 4), np.float32) for _ in range(3)] + [np.zeros((self.n, K, 3), np.float32)]
        _check(lib().b2ch_trainer_download(self.h, *[x.ctypes.data_as(_P) for x in a]), "b2ch_trainer_download")
        return dict(n=self.n, degree=self.degree, pos_op=a[0], quat=a[1], lscale=a[2], sh=a[3])

    def refine(self, stream, cam_pos, cam_focal, iter=1000, total=30000, growth_allowed=True, max_splats=10_000_000, growth_grad_threshold=0.0025,
               growth_select_fraction=0.25, split_at_screen_size=0.5, opac_decay=0.004, seed=42, no_new=False, cull_weight=0.0):
        """StepTrainer::refine (collective over the ranks). Returns the counts; the model's size follows."""
        f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
        fp = np.array([growth_grad_threshold, growth_select_fraction, split_at_screen_size, opac_decay, cull_weight], np.float32)
        up = np.array([iter, total, int(growth_allowed), max_splats, seed, int(no_new)], np.uint32)
        cp, cf, out = f32(cam_pos), f32(cam_focal), np.zeros(6, np.int32)
        p = lambda a: a.ctypes.data_as(_P)
        _check(lib().b2ch_trainer_refine(self.h, p(cp), p(cf), len(cf), p(fp), p(up), C.c_void_p(int(stream)), p(out)), "b2ch_trainer_refine")
        self.n = int(out[0])
        return dict(zip(("n", "pruned", "relocated", "grown", "split_oversized", "culled"), (int(x) for x in out)))

    def reduce_statistics(self, stream):
        _check(lib().b2ch_trainer_reduce_statistics(self.h, C.c_void_p(int(stream))), "b2ch_trainer_reduce_statistics")

    def checksum(self, stream):
        return int(lib().b2ch_trainer_checksum(self.h, C.c_void_p(int(stream))))


# ---- files: splat PLY (src/ply.cpp:80-226) and the headless render front end (src/render/renderer.cpp:199-368) ----

def read_ply(path):
    """Host cloud dict of the reference's SplatCloud fields: n, degree, pos [n][3], log_scale [n][3], quat [n][4], opacity
    [n], sh [n][K][3], plus evidence [n][7] / labels [n][2] when the file carries them, and has_scales."""
    n, deg, flags = C.c_int32(0), C.c_int32(0), C.c_int32(0)
    p = path.encode()
    _check(lib().b2ch_ply_read(p, C.byref(n), C.byref(deg), None, None, None, None, None, None, None, C.byref(flags)), "read_ply")
    n, K = n.value, (deg.value + 1) ** 2
    out = dict(n=n, degree=deg.value, pos=np.zeros((n, 3), np.float32), log_scale=np.zeros((n, 3), np.float32), quat=np.zeros((n, 4), np.float32),
               opacity=np.zeros(n, np.float32), sh=np.zeros((n, K, 3), np.float32), has_scales=bool(flags.value & 1))
    if flags.value & 2:
        out["evidence"] = np.zeros((n, 7), np.float32)
    if flags.value & 4:
        out["labels"] = np.zeros((n, 2), np.float32)
    ptr = lambda k: out[k].ctypes.data_as(_P) if k in out else None
    _check(lib().b2ch_ply_read(p, C.byref(C.c_int32()), C.byref(C.c_int32()), ptr("pos"), ptr("log_scale"), ptr("quat"), ptr("opacity"), ptr("sh"),
                               ptr("evidence"), ptr("labels"), None), "read_ply")
    return out


def write_ply(path, cloud, comment=""):
    f32 = lambda k: None if cloud.get(k) is None else np.ascontiguousarray(cloud[k], dtype=np.float32)
    arrs = {k: f32(k) for k in ("pos", "log_scale", "quat", "opacity", "sh", "evidence", "labels")}
    ptr = lambda k: None if arrs[k] is None else arrs[k].ctypes.data_as(_P)
    _check(lib().b2ch_ply_write(path.encode(), int(cloud["n"]), int(cloud["degree"]), ptr("pos"), ptr("log_scale"), ptr("quat"), ptr("opacity"), ptr("sh"),
                                ptr("evidence"), ptr("labels"), comment.encode()), "write_ply")


def cloud_from_scene(scene):
    """The SplatCloud-style dict of a scene dict of b2ctrain_b200.scenes (the floor lane is not part of the file format)."""
    return dict(n=scene["n"], degree=scene["degree"], pos=scene["pos_op"][:, :3], log_scale=scene["lscale"][:, :3], quat=scene["quat"],
                opacity=scene["pos_op"][:, 3], sh=scene["sh"])


class HostRenderer:
    """b2c::StreamRenderer: many cameras of one model, `lanes` of them in flight on separate streams; the 8-bit image and
    the depth map of a camera are copied to (pinned) host arrays on a copy stream while later cameras render."""

    def __init__(self, scene, W, H, depth=True, render_chunks=1, lanes=1, isect_cap=0):
        f = lambda a: np.ascontiguousarray(a, np.float32)
        self._keep = [f(scene["pos_op"]), f(scene["quat"]), f(scene["lscale"]), f(scene["sh"])]
        p = [a.ctypes.data_as(C.c_void_p) for a in self._keep]
        self.W, self.H = W, H
        self.h = lib().b2ch_renderer_create(int(scene["n"]), int(scene["degree"]), p[0], p[1], p[2], p[3], int(W), int(H), int(depth), int(render_chunks), int(lanes), int(isect_cap))
        if not self.h:
            raise RuntimeError("b2ch_renderer_create: " + lib().b2ch_last_error().decode())
        self.h = C.c_void_p(self.h)

    def close(self):
        if self.h:
            lib().b2ch_renderer_destroy(self.h)
            self.h = None

    def render(self, cam, stream, background=None, sh_degree=-1, host_rgba8=None, host_depth=None):
        """host_rgba8 / host_depth: data pointers (ints) of pinned host buffers of W * H words, or None."""
        from .api import camera_from
        cs = cam if not isinstance(cam, dict) else camera_from(cam)
        bg = (C.c_float * 3)(*background) if background is not None else None
        _check(lib().b2ch_renderer_render(self.h, C.byref(cs), bg, int(sh_degree), C.c_void_p(host_rgba8) if host_rgba8 else None,
                                          C.c_void_p(host_depth) if host_depth else None, C.c_void_p(int(stream))), "b2ch_renderer_render")

    def finish(self):
        _check(lib().b2ch_renderer_finish(self.h), "b2ch_renderer_finish")

    def info(self):
        out = (C.c_uint64 * 5)()
        _check(lib().b2ch_renderer_info(self.h, out), "b2ch_renderer_info")
        return dict(num_isect=int(out[0]), isect_cap=int(out[1]), d2h_bytes=int(out[2]), tile_bits=int(out[3]), redone=int(out[4]))


def render_headless(splat, cameras, output_dir, background=(0.0, 0.0, 0.0), sh_degree=-1, depth=False, render_chunks=1, rank=0, world=1):
    bg = (C.c_float * 3)(*background)
    done = C.c_int32(0)
    _check(lib().b2ch_render_headless(splat.encode(), cameras.encode(), output_dir.encode(), bg, int(sh_degree), int(depth), int(render_chunks), int(rank),
                                      int(world), C.byref(done)), "render_headless")
    return done.value


def refine_once(scene, stats, cam_pos, cam_focal, W=64, H=64, iter=1000, total=30000, growth_allowed=True, max_splats=10_000_000, growth_grad_threshold=0.0025,
                growth_select_fraction=0.25, split_at_screen_size=0.5, opac_decay=0.004, seed=42, no_new=False, cull_weight=0.0):
    """One RefineState::run of the C++ host (src/gpu/refine.cu:244-342) on a scene dict with statistics [4][n] = refine_norm,
    max_screen, vis_count, vis_weight. Returns (refined scene dict, counts dict, pairs [2][k] parent -> child slot)."""
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    n, deg = int(scene["n"]), int(scene["degree"])
    K, capn = (deg + 1) ** 2, 2 * n + 16
    fp = np.array([growth_grad_threshold, growth_select_fraction, split_at_screen_size, opac_decay, cull_weight], np.float32)
    up = np.array([iter, total, int(growth_allowed), max_splats, seed, int(no_new)], np.uint32)
    ins = [f32(scene[k]) for k in ("pos_op", "quat", "lscale", "sh")] + [f32(stats), f32(cam_pos), f32(cam_focal)]
    outs = [np.zeros((capn, 4), np.float32) for _ in range(3)] + [np.zeros((capn, K, 3), np.float32)]
    pairs, out = np.zeros((2, capn), np.uint32), np.zeros(7, np.int32)
    p = lambda a: a.ctypes.data_as(_P)
    _check(lib().b2ch_refine_once(n, deg, *[p(a) for a in ins[:6]], p(ins[6]), len(ins[6]), p(fp), p(up), int(W), int(H), p(out), capn, *[p(a) for a in outs],
                                  p(pairs)), "refine_once")
    m, k = int(out[0]), int(out[6])
    counts = dict(zip(("n", "pruned", "relocated", "grown", "split_oversized", "culled"), (int(x) for x in out[:6])))
    refined = dict(n=m, degree=deg, pos_op=outs[0][:m], quat=outs[1][:m], lscale=outs[2][:m], sh=outs[3][:m])
    return refined, counts, np.ascontiguousarray(pairs.reshape(-1)[: 2 * k].reshape(2, k))
