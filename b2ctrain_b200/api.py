"""Host-side mirror of the reference's operator API for the splat hot path, over the C ABI of libb2k.so.

Names, argument meaning and error behaviour follow the reference's C++ interface: Model (src/model.h:14-40),
RenderCtx / RenderParams / CameraGPU (src/gpu/render.h:10-95), ViewGPU / LossParams (src/gpu/loss.h:7-30),
OptimParams (src/gpu/optim.h:6-45) and the free functions render_forward, project_splats, bin_and_sort,
rasterize_forward, rasterize_backward, photometric_loss, accumulate_loss, eval_metrics, optimizer_step. Errors raise
RuntimeError, as the reference's CUDA_CHECK / fail() do (src/gpu/util.cuh:13-15).

torch is used only to own device memory and streams; every computation is a kernel of libb2k.so. There is no CPU
path: importing works without a GPU (so the symbol table can be checked), computing without the library or without a
GPU raises.
"""
import ctypes as C
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb2k.so")

B2K_OK, B2K_ERR_ARG, B2K_ERR_CAPACITY, B2K_ERR_UNSUPPORTED, B2K_ERR_CUDA, B2K_ERR_OVERFLOW = range(6)
GRAD_LANES = 13


class B2kCamera(C.Structure):
    _fields_ = [("R", C.c_float * 9), ("t", C.c_float * 3), ("pos", C.c_float * 3), ("fx", C.c_float), ("fy", C.c_float),
                ("cx", C.c_float), ("cy", C.c_float), ("W", C.c_int32), ("H", C.c_int32), ("lim_pos_x", C.c_float),
                ("lim_pos_y", C.c_float), ("lim_neg_x", C.c_float), ("lim_neg_y", C.c_float)]


_MODEL_PTRS = ["pos_op", "quat", "lscale", "sh_dc", "sh_hi", "m_pos_op", "v_pos_op", "m_quat", "v_quat", "m_lscale", "v_lscale",
               "m_sh_dc", "m_sh_hi", "v_sh", "refine_norm", "max_screen", "vis_count", "vis_weight", "last_step"]


class B2kModel(C.Structure):
    _fields_ = [("n", C.c_int32), ("cap", C.c_int32), ("degree", C.c_int32)] + [(k, C.c_void_p) for k in _MODEL_PTRS]


class B2kCtx(C.Structure):
    _fields_ = [("W", C.c_int32), ("H", C.c_int32), ("tiles_x", C.c_int32), ("tiles_y", C.c_int32), ("n_tiles", C.c_int32),
                ("tile_bits", C.c_int32), ("n_cap", C.c_int32),
                ("proj0", C.c_void_p), ("proj1", C.c_void_p), ("proj2", C.c_void_p), ("tile_count", C.c_void_p), ("hit_info", C.c_void_p),
                ("depth_keys", C.c_void_p), ("depth_keys_sorted", C.c_void_p), ("order_in", C.c_void_p), ("order", C.c_void_p),
                ("tile_off", C.c_void_p), ("keys", C.c_void_p), ("vals", C.c_void_p), ("keys_sorted", C.c_void_p),
                ("vals_sorted", C.c_void_p), ("isect_cap", C.c_uint64), ("num_isect", C.c_void_p), ("sort_tmp", C.c_void_p),
                ("sort_tmp_bytes", C.c_uint64), ("tile_ranges", C.c_void_p), ("out_rgba", C.c_void_p), ("out_feat", C.c_void_p),
                ("out_depth", C.c_void_p), ("last_idx", C.c_void_p), ("v_splat", C.c_void_p), ("vis_flag", C.c_void_p), ("vis_list", C.c_void_p),
                ("v_out", C.c_void_p), ("loss_accum", C.c_void_p), ("n_chunks", C.c_int32), ("proj3", C.c_void_p), ("chunk_words", C.c_void_p),
                ("bwd_scratch", C.c_void_p), ("bwd_scratch_bytes", C.c_uint64)]


class B2kRenderOpts(C.Structure):
    _fields_ = [("bg", C.c_float * 3), ("sh_degree", C.c_int32), ("bwd_info", C.c_int32), ("pos_override", C.c_void_p),
                ("quat_override", C.c_void_p), ("lscale_override", C.c_void_p), ("feat_mode", C.c_int32), ("feat_buffer", C.c_void_p)]


class B2kLoss(C.Structure):
    _fields_ = [("rgba", C.c_void_p), ("weights", C.c_void_p), ("l1_w", C.c_float), ("ssim_w", C.c_float), ("bg", C.c_float * 3),
                ("composite", C.c_int32), ("mask", C.c_int32), ("alpha_lane", C.c_int32), ("match_alpha_weight", C.c_float),
                ("scale", C.c_float), ("grad_scale", C.c_float)]


class B2kOptim(C.Structure):
    _fields_ = [("active_sh_degree", C.c_int32), ("t", C.c_int32), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("lr_mean", C.c_float), ("lr_rot", C.c_float), ("lr_scale", C.c_float), ("lr_opac", C.c_float), ("lr_dc", C.c_float),
                ("lr_sh_rest", C.c_float), ("noise_weight", C.c_float), ("noise_clamp", C.c_float), ("seed", C.c_uint32),
                ("step", C.c_uint32), ("sparse", C.c_int32), ("pos_override", C.c_void_p), ("quat_override", C.c_void_p),
                ("lscale_override", C.c_void_p), ("grad_out", C.c_void_p), ("touched_out", C.c_void_p)]


# Every entry point include/b2k.h declares, with its argument types (the symbol-table test walks this list).
_P, _S = C.c_void_p, C.c_void_p
SIGNATURES = {
    "b2k_project": (C.c_int, [_P, _P, _P, _P, _S]),
    "b2k_count_tiles": (C.c_int, [_P, C.c_int32, _S]),
    "b2k_bin_sort": (C.c_int, [_P, C.c_int32, _S]),
    "b2k_read_num_isect": (C.c_int, [_P, _S, _P]),
    "b2k_bin_sort_static": (C.c_int, [_P, C.c_int32, _S]),
    "b2k_bin_sort_profile": (C.c_int, [_P, C.c_int32, _S, _P]),
    "b2k_static_max_splats": (C.c_uint32, []),
    "b2k_raster_fwd": (C.c_int, [_P, _P, _S]),
    "b2k_render_chunked": (C.c_int, [_P, _P, _P, _P, _S]),
    "b2k_sort_tmp_bytes": (C.c_uint64, [C.c_int32, C.c_uint64]),
    "b2k_sort_passes": (C.c_int32, [C.c_int32]),
    "b2k_loss_photometric": (C.c_int, [_P, _P, _S]),
    "b2k_loss_accumulate": (C.c_int, [_P, _S]),
    "b2k_loss_zero": (C.c_int, [_P, C.c_int32, C.c_int32, _S]),
    "b2k_loss_fold": (C.c_int, [_P, _P, _S]),
    "b2k_step_begin": (C.c_int, [_P, _S]),
    "b2k_eval_metrics": (C.c_int, [_P, _P, C.c_int32, _S]),
    "b2k_bwd_scratch_bytes": (C.c_uint64, [C.c_int32, C.c_int32, C.c_int32, C.c_uint64]),
    "b2k_raster_bwd": (C.c_int, [_P, _P, _P, _S]),
    "b2k_raster_bwd_scaled": (C.c_int, [_P, _P, _P, C.c_float, _S]),
    "b2k_optim_fused": (C.c_int, [_P, _P, _P, _P, _S]),
    "b2k_proj_bwd": (C.c_int, [_P, _P, _P, _P, _P, _S]),
    "b2k_adam": (C.c_int, [_P, _P, _P, _S]),
    "b2k_adam_range": (C.c_int, [_P, _P, _P, C.c_int32, C.c_int32, _S]),
    "b2k_sort_pairs_tmp_bytes": (C.c_uint64, []),
    "b2k_sort_pairs_u32": (C.c_int, [_P, _P, _P, _P, C.c_uint32, _P, C.c_uint64, _S]),
    "b2k_refine_flags": (C.c_int, [_P, _P, C.c_float, C.c_float, _P, _P, _P, _S]),
    "b2k_refine_sample_keys": (C.c_int, [_P, _P, _P, C.c_int32, C.c_float, C.c_uint32, _P, _P, _P, _S]),
    "b2k_refine_oversized": (C.c_int, [_P, _P, _P, C.c_float, _P, _S]),
    "b2k_refine_mark": (C.c_int, [_P, C.c_int32, _P, _S]),
    "b2k_refine_split": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_int32, C.c_float, _P, _S]),
    "b2k_refine_kill": (C.c_int, [_P, _P, C.c_int32, _S]),
    "b2k_refine_opacity_decay": (C.c_int, [_P, C.c_float, _S]),
    "b2k_refine_bake_floor": (C.c_int, [_P, _S]),
    "b2k_refine_axis_keys": (C.c_int, [_P, C.c_int32, _P, _P, _S]),
    "b2k_key_to_float": (C.c_float, [C.c_uint32]),
    "b2k_evidence_view": (C.c_int, [_P, _P, _P, _P, C.c_int32, C.c_float, _P, _S]),
    "b2k_evidence_fold": (C.c_int, [_P, _P, _P, _P, _S]),
    "b2k_label_vote": (C.c_int, [_P, _P, _P, _P, C.c_int32, _P, _S]),
    "b2k_label_bins": (C.c_int32, []),
    "b2k_dp_unique_id": (C.c_int, [_P]),
    "b2k_dp_init": (C.c_int, [_P, _P, C.c_int32, C.c_int32]),
    "b2k_dp_destroy": (C.c_int, [_P]),
    "b2k_dp_allreduce_grads": (C.c_int, [_P, _P, C.c_uint64, _S]),
    "b2k_dp_allreduce_stat": (C.c_int, [_P, _P, C.c_uint64, C.c_int32, _S]),
    "b2k_dp_barrier": (C.c_int, [_P, _S]),
    "b2k_dp_share": (C.c_int, [_P, _P, _P, _S]),
    "b2k_dp_release_shares": (C.c_int, [_P, _S]),
    "b2k_dp_gather_slices": (C.c_int, [_P, _P, C.c_uint64, C.c_int32, C.c_uint64, C.c_int32, _S]),
    "b2k_dp_slice": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, _P, _P]),
    "b2k_dp_adam_shard": (C.c_int, [_P, _P, _P, _P, _S]),
    "b2k_min_scale": (C.c_int, [_P, _P, _P, C.c_int32, _S]),
    "b2k_select_tmp_words": (C.c_uint64, [C.c_int32]),
    "b2k_select_flagged": (C.c_int, [_P, C.c_int32, _P, _P, _P, _S]),
    "b2k_gather_lanes": (C.c_int, [_P, _P, _P, C.c_int32, C.c_int32, C.c_uint64, C.c_int32, _S]),
    "b2k_pack_rgba8": (C.c_int, [_P, _P, C.c_int32, C.c_int32, _S]),
    "b2k_quantize_rgba8": (C.c_int, [_P, _P, C.c_int32, _S]),
    "b2k_error_string": (C.c_char_p, [C.c_int]),
    "b2k_last_cuda_error": (C.c_int, []),
    "b2k_version": (C.c_char_p, []),
}

_lib = None


def lib():
    """Loads libb2k.so; raises when it has not been built (there is no fallback path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m b2ctrain_b200.build` (no CPU fallback exists)")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            f = getattr(l, name)
            f.restype, f.argtypes = res, args
        _lib = l
    return _lib


def _check(status, what):
    if status != B2K_OK:
        l = lib()
        msg = l.b2k_error_string(status).decode()
        if status == B2K_ERR_CUDA:
            msg += f" (cudaError {l.b2k_last_cuda_error()})"
        raise RuntimeError(f"{what}: {msg}")


def _stream(stream):
    if stream is None:
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if isinstance(stream, torch.cuda.Stream):
        return C.c_void_p(stream.cuda_stream)
    return C.c_void_p(int(stream))


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def camera_from(cam):
    """CameraGPU record from a camera dict of b2ctrain_b200.scenes (CameraGPU::from, src/gpu/render.h:15-24)."""
    s = B2kCamera()
    for i in range(9):
        s.R[i] = float(cam["R"][i])
    for i in range(3):
        s.t[i] = float(cam["t"][i])
        s.pos[i] = float(cam["pos"][i])
    for k in ("fx", "fy", "cx", "cy", "lim_pos_x", "lim_pos_y", "lim_neg_x", "lim_neg_y"):
        setattr(s, k, float(cam[k]))
    s.W, s.H = int(cam["W"]), int(cam["H"])
    return s


def _capacity_for(n):
    cap = 1024
    while cap < n:
        cap *= 2
    return cap


class Model:
    """Device splat model: parameters, Adam moments and refine statistics (src/model.h:14-40). Capacity doubles from
    1024 (src/model.cu:10-11); SH is planar with stride `cap`."""

    def __init__(self, device="cuda:0"):
        self.device = torch.device(device)
        self.n = self.cap = 0
        self.degree = 3
        self.adam_t = 0
        self.sh_fp16 = False

    def K(self):
        return (self.degree + 1) ** 2

    def upload(self, cloud):
        """cloud: host dict(n, degree, pos_op [n][4], quat [n][4], lscale [n][4], sh [n][K][3]) (Model::upload,
        src/model.cu:46-83; unlike the reference the floor lane lscale[:, 3] is taken from the cloud)."""
        if self.sh_fp16:
            raise RuntimeError("Model.upload: fp16 SH storage is not implemented (unsupported lane)")
        self.n, self.degree = int(cloud["n"]), int(cloud["degree"])
        self.cap = _capacity_for(self.n)
        K, cap, dev = self.K(), self.cap, self.device
        f32 = dict(dtype=torch.float32, device=dev)

        def up4(a):
            t = torch.zeros((cap, 4), **f32)
            t[: self.n] = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev)
            return t

        self.pos_op, self.quat, self.lscale = up4(cloud["pos_op"]), up4(cloud["quat"]), up4(cloud["lscale"])
        sh = torch.from_numpy(np.ascontiguousarray(cloud["sh"], dtype=np.float32)).to(dev).reshape(self.n, K * 3)
        planar = torch.zeros((K * 3, cap), **f32)
        planar[:, : self.n] = sh.t()
        self.sh_dc = planar[:3].contiguous()
        self.sh_hi = planar[3:].contiguous() if K > 1 else torch.zeros((0, cap), **f32)
        self.zero_optimizer()
        self.zero_stats()
        return self

    def zero_optimizer(self):
        z = lambda *s: torch.zeros(s, dtype=torch.float32, device=self.device)
        cap, K = self.cap, self.K()
        self.m_pos_op, self.v_pos_op, self.m_quat, self.v_quat, self.m_lscale, self.v_lscale = (z(cap, 4) for _ in range(6))
        self.m_sh_dc, self.m_sh_hi, self.v_sh = z(3, cap), z(3 * (K - 1), cap), z(cap)
        self.last_step = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self.adam_t = 0

    def zero_stats(self):
        z = lambda: torch.zeros(self.cap, dtype=torch.float32, device=self.device)
        self.refine_norm, self.max_screen, self.vis_count, self.vis_weight = z(), z(), z(), z()

    def download(self):
        n, K = self.n, self.K()
        planar = torch.cat([self.sh_dc, self.sh_hi], 0)[:, :n]
        return dict(n=n, degree=self.degree, pos_op=self.pos_op[:n].cpu().numpy(), quat=self.quat[:n].cpu().numpy(),
                    lscale=self.lscale[:n].cpu().numpy(), sh=planar.t().reshape(n, K, 3).contiguous().cpu().numpy())

    def compact(self, keep, extras=(), stream=None):
        """Model::compact (src/model.cu:120-155): keeps the splats whose flag in `keep` (device int32 [n]) is non-zero,
        in their order, across parameters, moments, statistics and the caller's extra per-splat float tensors (each
        [cap], replaced in the returned list). Returns (new n, extras). Synchronises for the count, like the reference."""
        if self.n == 0:
            return 0, list(extras)
        n, cap, dev = self.n, self.cap, self.device
        idx = torch.zeros(n, dtype=torch.int32, device=dev)
        cnt = torch.zeros(1, dtype=torch.int32, device=dev)
        tmp = torch.zeros(int(lib().b2k_select_tmp_words(n)), dtype=torch.int32, device=dev)
        _check(lib().b2k_select_flagged(_ptr(keep), n, _ptr(idx), _ptr(cnt), _ptr(tmp), _stream(stream)), "Model.compact")
        kept = int(cnt.item())
        if kept == n:
            return n, list(extras)

        def gather(t, lanes, elem_bytes):
            if t is None or t.numel() == 0 or lanes == 0:
                return t
            fresh = torch.zeros_like(t)   # an in-place gather would race
            _check(lib().b2k_gather_lanes(_ptr(t), _ptr(fresh), _ptr(idx), kept, lanes, cap, elem_bytes, _stream(stream)), "Model.compact")
            return fresh

        hi_lanes = 3 * (self.K() - 1)
        for k in ("pos_op", "quat", "lscale", "m_pos_op", "v_pos_op", "m_quat", "v_quat", "m_lscale", "v_lscale"):
            setattr(self, k, gather(getattr(self, k), 1, 16))
        for k, lanes in (("sh_dc", 3), ("sh_hi", hi_lanes), ("m_sh_dc", 3), ("m_sh_hi", hi_lanes), ("v_sh", 1), ("refine_norm", 1),
                         ("max_screen", 1), ("vis_count", 1), ("vis_weight", 1), ("last_step", 1)):
            setattr(self, k, gather(getattr(self, k), lanes, 4))
        out = [gather(e, 1, 4) for e in extras]
        self.n = kept
        return kept, out

    def sh_planar_to_host(self, dc, hi):
        n, K = self.n, self.K()
        return torch.cat([dc, hi], 0)[:, :n].t().reshape(n, K, 3).contiguous().cpu().numpy()

    def struct(self):
        s = B2kModel()
        s.n, s.cap, s.degree = self.n, self.cap, self.degree
        for k in _MODEL_PTRS:
            t = getattr(self, k, None)
            setattr(s, k, None if t is None or t.numel() == 0 else t.data_ptr())
        return s


class RenderCtx:
    """Per-view scratch (src/gpu/render.h:66-95); member names follow the reference. `setup` sizes everything; the
    intersection buffers start at 2^22 entries (src/gpu/render.cu:20) and double on overflow."""

    def __init__(self, device="cuda:0"):
        self.device = torch.device(device)
        self.W = self.H = self.tiles_x = self.tiles_y = self.n_tiles = self.tile_bits = 0
        self.n_cap = 0
        self.isect_cap = 0
        self.num_isect = 0
        self.want_depth = False
        self.n_chunks = 1          # > 1: render_forward composites the view front to back in this many depth chunks
        self.chunk_words = None

    def setup(self, W, H, n_splats, stream=None, isect_cap=None, n_chunks=None):
        if n_chunks is not None:
            self.n_chunks = max(1, int(n_chunks))
        dev = self.device
        self.W, self.H = int(W), int(H)
        self.tiles_x, self.tiles_y = (self.W + 7) // 8, (self.H + 7) // 8
        self.n_tiles = self.tiles_x * self.tiles_y
        self.tile_bits = 1
        while (1 << self.tile_bits) < self.n_tiles + 1:
            self.tile_bits += 1
        n = max(int(n_splats), 1)
        u32 = lambda *s: torch.zeros(s, dtype=torch.int32, device=dev)
        f32 = lambda *s: torch.zeros(s, dtype=torch.float32, device=dev)
        if n > self.n_cap:
            self.proj0, self.proj1, self.proj2 = f32(n, 4), f32(n, 4), f32(n, 4)
            self.proj3 = f32(n, 2)
            self.tile_count, self.tile_off = u32(n), u32(n)
            self.hit_info = u32(n, 4)
            self.depth_keys, self.depth_keys_sorted, self.order_in, self.order = u32(n), u32(n), u32(n), u32(n)
            self.v_splat, self.vis_flag = f32(n, GRAD_LANES), u32(n)
            self.vis_list = u32(n)
            self.n_cap = n
        P = self.W * self.H
        self.tile_ranges = u32(self.n_chunks * self.n_tiles, 2)
        self.chunk_words = u32(32 + self.n_tiles + (self.tiles_x + 1) * (self.tiles_y + 1)) if self.n_chunks > 1 else None
        self.out_rgba, self.out_feat, self.v_out = f32(P, 4), f32(P, 4), f32(P, 4)
        self.out_depth = f32(P) if self.want_depth else None
        self.last_idx = u32(P)
        self.loss_accum = f32(16)
        self.d_num_isect = u32(4)
        if self.isect_cap == 0 or (isect_cap and isect_cap > self.isect_cap):
            self._alloc_isect(isect_cap or (1 << 22))
        else:
            self._alloc_isect(self.isect_cap)   # the backward scratch depends on the image size and the chunk count
        nbytes = int(lib().b2k_sort_tmp_bytes(self.n_cap, self.isect_cap))
        self.sort_tmp = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        return self

    def _alloc_isect(self, cap):
        u32 = lambda: torch.zeros(cap, dtype=torch.int32, device=self.device)
        self.keys, self.vals, self.keys_sorted, self.vals_sorted = u32(), u32(), u32(), u32()
        self.isect_cap = int(cap)
        # checkpoints and work list of the segmented backward: sized from the intersection capacity
        self.bwd_scratch = torch.zeros(int(lib().b2k_bwd_scratch_bytes(self.W, self.H, self.n_chunks, self.isect_cap)), dtype=torch.uint8,
                                       device=self.device)

    def struct(self):
        s = B2kCtx()
        for k in ("W", "H", "tiles_x", "tiles_y", "n_tiles", "tile_bits", "n_cap"):
            setattr(s, k, getattr(self, k))
        for k in ("proj0", "proj1", "proj2", "tile_count", "hit_info", "depth_keys", "depth_keys_sorted", "order_in", "order", "tile_off", "keys",
                  "vals", "keys_sorted", "vals_sorted", "sort_tmp", "tile_ranges", "out_rgba", "out_feat", "out_depth", "last_idx",
                  "v_splat", "vis_flag", "vis_list", "v_out", "loss_accum", "chunk_words", "proj3", "bwd_scratch"):
            t = getattr(self, k, None)
            setattr(s, k, None if t is None else t.data_ptr())
        s.num_isect = self.d_num_isect.data_ptr()
        s.isect_cap = self.isect_cap
        s.sort_tmp_bytes = self.sort_tmp.numel()
        s.bwd_scratch_bytes = self.bwd_scratch.numel()
        s.n_chunks = self.n_chunks
        return s


class RenderParams:
    """RenderParams (src/gpu/render.h:29-63). Lanes this library does not implement raise when set. feat: "None",
    "Normals" or "Buffer" (FeatureMode, render.h:27; forward only); feat_buffer: [n][3] device tensor for "Buffer"."""
    _UNSUPPORTED = ("warp", "sh_frame", "app", "col_base", "hollow_z")
    _FEAT = {"None": 0, "Normals": 1, "Buffer": 2}

    def __init__(self, cam, bg=(0.0, 0.0, 0.0), sh_degree=3, bwd_info=True):
        self.cam, self.bg, self.sh_degree, self.bwd_info = cam, tuple(bg), sh_degree, bwd_info
        self.feat = "None"
        self.feat_buffer = None
        self.mip = False
        self.pos_override = self.quat_override = self.lscale_override = None
        for k in self._UNSUPPORTED:
            setattr(self, k, None)

    def struct(self):
        if self.mip or any(getattr(self, k) is not None for k in self._UNSUPPORTED):
            raise RuntimeError("RenderParams: mip / warp / sh_frame / app / hollow lanes are not implemented (unsupported lane)")
        if self.feat not in self._FEAT or (self.feat == "Buffer") != (self.feat_buffer is not None):
            raise RuntimeError("RenderParams: feat is None, Normals or Buffer, and feat_buffer goes with Buffer")
        s = B2kRenderOpts()
        s.feat_mode, s.feat_buffer = self._FEAT[self.feat], _ptr(self.feat_buffer)
        for i in range(3):
            s.bg[i] = float(self.bg[i])
        s.sh_degree, s.bwd_info = int(self.sh_degree), int(bool(self.bwd_info))
        s.pos_override, s.quat_override, s.lscale_override = _ptr(self.pos_override), _ptr(self.quat_override), _ptr(self.lscale_override)
        return s

    def camera(self):
        return self.cam if isinstance(self.cam, B2kCamera) else camera_from(self.cam)


class ViewGPU:
    """A training view resident on the GPU (src/gpu/loss.h:7-18): packed RGBA8 target and optional u8 weights."""

    def __init__(self, rgba, weights=None, W=0, H=0):
        self.rgba, self.weights, self.W, self.H = rgba, weights, W, H
        self.normals = None


class LossParams:
    """LossParams (src/gpu/loss.h:20-30)."""

    def __init__(self, **kw):
        self.l1_w, self.ssim_w = 0.8, -0.2
        self.bg = (0.0, 0.0, 0.0)
        self.composite = self.mask = self.alpha_lane = False
        self.match_alpha_weight, self.scale, self.normal_scale, self.grad_scale = 0.1, 1.0, 0.0, 1.0
        for k, v in kw.items():
            if not hasattr(self, k):
                raise TypeError(k)
            setattr(self, k, v)

    def struct(self, view):
        if self.normal_scale != 0.0:
            raise RuntimeError("LossParams: the normal-supervision lane is not implemented (unsupported lane)")
        s = B2kLoss()
        s.rgba, s.weights = _ptr(view.rgba), _ptr(view.weights)
        s.l1_w, s.ssim_w = self.l1_w, self.ssim_w
        for i in range(3):
            s.bg[i] = float(self.bg[i])
        s.composite, s.mask, s.alpha_lane = int(self.composite), int(self.mask), int(self.alpha_lane)
        s.match_alpha_weight, s.scale, s.grad_scale = self.match_alpha_weight, self.scale, self.grad_scale
        return s


class OptimParams:
    """OptimParams (src/gpu/optim.h:6-45), defaults included."""
    _UNSUPPORTED = ("g_pos_out", "sh_frame", "update_mask", "canon_rot", "spa_z", "stretch_w", "g_app_out")

    def __init__(self, cam, **kw):
        self.cam = cam
        self.mip = False
        self.active_sh_degree = 3
        self.t = 1
        self.beta1, self.beta2, self.eps = 0.9, 0.999, 1e-15
        self.lr_mean = 0.0
        self.lr_rot, self.lr_scale, self.lr_opac, self.lr_dc, self.lr_sh_rest = 2e-3, 5e-3, 0.012, 2e-3, 2e-4
        self.noise_weight = self.noise_clamp = 0.0
        self.seed, self.step = 42, 0
        self.pos_override = self.quat_override = self.lscale_override = None
        self.frozen = False
        self.sparse = False
        self.grad_out = None
        self.touched_out = None   # bitmap of (n + 31) // 32 words: projection_backward marks the splats it adds a row for
        for k in self._UNSUPPORTED:
            setattr(self, k, None)
        for k, v in kw.items():
            if not hasattr(self, k):
                raise TypeError(k)
            setattr(self, k, v)

    def struct(self):
        if self.mip or self.frozen or any(getattr(self, k) is not None for k in self._UNSUPPORTED):
            raise RuntimeError("OptimParams: cage / deformation / sparsification lanes are not implemented (unsupported lane)")
        s = B2kOptim()
        for k in ("active_sh_degree", "t", "beta1", "beta2", "eps", "lr_mean", "lr_rot", "lr_scale", "lr_opac", "lr_dc", "lr_sh_rest",
                  "noise_weight", "noise_clamp", "seed", "step"):
            setattr(s, k, getattr(self, k))
        s.sparse = int(bool(self.sparse))
        s.pos_override, s.quat_override, s.lscale_override = _ptr(self.pos_override), _ptr(self.quat_override), _ptr(self.lscale_override)
        s.grad_out = _ptr(self.grad_out)
        s.touched_out = _ptr(self.touched_out)
        return s

    def camera(self):
        return self.cam if isinstance(self.cam, B2kCamera) else camera_from(self.cam)


# ---- operators (src/gpu/render.h:97-109, src/gpu/loss.h:32-41, src/gpu/optim.h:50) ----

def project_splats(ctx, m, p, stream=None):
    ms, cs, os_, cam = m.struct(), ctx.struct(), p.struct(), p.camera()
    _check(lib().b2k_project(C.byref(ms), C.byref(cam), C.byref(os_), C.byref(cs), _stream(stream)), "project_splats")


def count_tiles(ctx, m, stream=None):
    """Tile counts, hit masks and depth keys from the records already in ctx.proj0 / ctx.proj1."""
    cs = ctx.struct()
    _check(lib().b2k_count_tiles(C.byref(cs), m.n, _stream(stream)), "count_tiles")


def bin_and_sort(ctx, m, stream=None, sync=True):
    """With sync=True behaves like the reference (binning.cu:125-133): reads the intersection total back, and when it
    exceeds the buffers grows them by doubling and redoes the binning. sync=False leaves the total on the device."""
    cs = ctx.struct()
    _check(lib().b2k_bin_sort(C.byref(cs), m.n, _stream(stream)), "bin_and_sort")
    if not sync:
        return
    total = C.c_uint32(0)
    st = lib().b2k_read_num_isect(C.byref(cs), _stream(stream), C.byref(total))
    if st == B2K_ERR_OVERFLOW:
        cap = ctx.isect_cap
        while cap < total.value:
            cap *= 2
        ctx._alloc_isect(cap)
        cs = ctx.struct()
        _check(lib().b2k_bin_sort(C.byref(cs), m.n, _stream(stream)), "bin_and_sort")
        st = lib().b2k_read_num_isect(C.byref(cs), _stream(stream), C.byref(total))
    _check(st, "bin_and_sort")
    ctx.num_isect = int(total.value)


def bin_and_sort_profile(ctx, m, stream=None):
    """bin_and_sort timed phase by phase with CUDA events inside the library; returns the ten durations in ms (see
    b2k_bin_sort_profile in include/b2k.h). Synchronises."""
    cs = ctx.struct()
    ms = (C.c_float * 10)()
    _check(lib().b2k_bin_sort_profile(C.byref(cs), m.n, _stream(stream), ms), "bin_and_sort_profile")
    return list(ms)


def rasterize_forward(ctx, p, stream=None):
    cs, os_ = ctx.struct(), p.struct()
    _check(lib().b2k_raster_fwd(C.byref(cs), C.byref(os_), _stream(stream)), "rasterize_forward")


def render_forward(ctx, m, p, stream=None, sync=True):
    """render_forward (src/gpu/render.h:97). A context set up with n_chunks > 1 renders front to back in depth chunks
    (b2k_render_chunked: same image and gradients, intersections behind saturated pixels never sorted)."""
    if ctx.n_chunks > 1:
        return render_chunked(ctx, m, p, stream, sync=sync)
    project_splats(ctx, m, p, stream)
    bin_and_sort(ctx, m, stream, sync=sync)
    rasterize_forward(ctx, p, stream)


def render_chunked(ctx, m, p, stream=None, sync=True):
    """b2k_render_chunked; with sync the slot count is read back and the view redone with larger buffers on overflow."""
    while True:
        cs, ms, os_, cam = ctx.struct(), m.struct(), p.struct(), p.camera()
        _check(lib().b2k_render_chunked(C.byref(ms), C.byref(cam), C.byref(os_), C.byref(cs), _stream(stream)), "render_chunked")
        if not sync:
            return None
        total = C.c_uint32(0)
        st = lib().b2k_read_num_isect(C.byref(cs), _stream(stream), C.byref(total))
        ctx.num_isect = int(total.value)
        if st == B2K_ERR_OVERFLOW:
            cap = ctx.isect_cap
            while cap < ctx.num_isect + 32 * ctx.n_chunks:
                cap *= 2
            ctx._alloc_isect(cap)
            continue
        _check(st, "render_chunked")
        return ctx.num_isect


def photometric_loss(ctx, view, lp, stream=None):
    cs, ls = ctx.struct(), lp.struct(view)
    _check(lib().b2k_loss_photometric(C.byref(cs), C.byref(ls), _stream(stream)), "photometric_loss")


def accumulate_loss(ctx, stream=None):
    cs = ctx.struct()
    _check(lib().b2k_loss_accumulate(C.byref(cs), _stream(stream)), "accumulate_loss")


def zero_loss(ctx, first=0, count=16, stream=None):
    """loss_accum[first : first + count] = 0 on the stream."""
    cs = ctx.struct()
    _check(lib().b2k_loss_zero(C.byref(cs), int(first), int(count), _stream(stream)), "zero_loss")


def step_begin(ctx, stream=None):
    """Clears the context's loss accumulator and its running intersection maximum (start of a training step)."""
    cs = ctx.struct()
    _check(lib().b2k_step_begin(C.byref(cs), _stream(stream)), "step_begin")


def fold_loss(dst_ctx, src_ctx, stream=None):
    """Adds the running loss sum and view count of src_ctx into dst_ctx's."""
    a, b = dst_ctx.struct(), src_ctx.struct()
    _check(lib().b2k_loss_fold(C.byref(a), C.byref(b), _stream(stream)), "fold_loss")


def eval_metrics(ctx, view, mask_weighted=False, stream=None):
    cs = ctx.struct()
    _check(lib().b2k_eval_metrics(C.byref(cs), _ptr(view.rgba), int(mask_weighted), _stream(stream)), "eval_metrics")


def rasterize_backward(ctx, m, p, stream=None):
    cs, ms, os_ = ctx.struct(), m.struct(), p.struct()
    _check(lib().b2k_raster_bwd(C.byref(cs), C.byref(ms), C.byref(os_), _stream(stream)), "rasterize_backward")


def rasterize_backward_tc(ctx, m, p, grad_scale, stream=None):
    """rasterize_backward_tc (src/gpu/render.h:107-109): v_out carries grad_scale, the per-splat lanes leave divided by it."""
    cs, ms, os_ = ctx.struct(), m.struct(), p.struct()
    _check(lib().b2k_raster_bwd_scaled(C.byref(cs), C.byref(ms), C.byref(os_), C.c_float(grad_scale), _stream(stream)), "rasterize_backward_tc")


def optimizer_step(ctx, m, op, stream=None):
    cs, ms, os_, cam = ctx.struct(), m.struct(), op.struct(), op.camera()
    _check(lib().b2k_optim_fused(C.byref(cs), C.byref(ms), C.byref(cam), C.byref(os_), _stream(stream)), "optimizer_step")


# ---- data-parallel split of optimizer_step ----

def projection_backward(ctx, m, op, grad, stream=None):
    cs, ms, os_, cam = ctx.struct(), m.struct(), op.struct(), op.camera()
    _check(lib().b2k_proj_bwd(C.byref(cs), C.byref(ms), C.byref(cam), C.byref(os_), _ptr(grad), _stream(stream)), "projection_backward")


def adam_step(m, op, grad, stream=None, first=0, count=None):
    """The update half of the data-parallel split from the accumulator grad[n][11+3K]; first/count restrict it to a
    slice of splats (first a multiple of 4)."""
    ms, os_ = m.struct(), op.struct()
    if first == 0 and count is None:
        _check(lib().b2k_adam(C.byref(ms), C.byref(os_), _ptr(grad), _stream(stream)), "adam_step")
    else:
        count = m.n - first if count is None else count
        _check(lib().b2k_adam_range(C.byref(ms), C.byref(os_), _ptr(grad), int(first), int(count), _stream(stream)), "adam_step")


def update_min_scale(m, cam_pos, cam_focal, stream=None):
    """RefineState::update_min_scale (src/gpu/refine.cu:166-170): cam_pos [c][3], cam_focal [c] device tensors."""
    ms = m.struct()
    _check(lib().b2k_min_scale(C.byref(ms), _ptr(cam_pos), _ptr(cam_focal), int(cam_focal.numel()), _stream(stream)), "update_min_scale")


def pack_rgba8(rgba, out, alpha_override=-1, stream=None):
    _check(lib().b2k_pack_rgba8(_ptr(rgba), _ptr(out), int(out.numel()), int(alpha_override), _stream(stream)), "pack_rgba8")
