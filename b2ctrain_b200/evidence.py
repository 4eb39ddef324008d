"""compute_evidence / download_evidence / download_labels (src/train/evidence.h) over the C ABI: per-splat multi-view
evidence [n][7] = (w_in, w_all, err, effective views, direction xyz) and the label vote [n][2] = (winning class, its
share). Views shard over ranks like training views; the accumulators are summed over ranks before the download."""
import ctypes as C

import numpy as np
import torch

from . import api


class Evidence:
    def __init__(self, model, device="cuda:0"):
        self.m, self.device = model, torch.device(device)
        self.bins = int(api.lib().b2k_label_bins())
        self.acc = torch.zeros((model.n, 8), dtype=torch.float32, device=self.device)     # the exported seven + sum of w_in^2 (evidence.cu:21)
        self.view_acc = torch.zeros((model.n, 3), dtype=torch.float32, device=self.device)
        self.votes = None

    def add_view(self, ctx, cam, view, masked=False, has_alpha=False, labels=None, normal_weight=0.0, stream=None):
        """One view of compute_evidence's loop (evidence.cu:212-239): render with bwd_info, replay, fold."""
        m = self.m
        rp = api.RenderParams(cam, sh_degree=m.degree, bwd_info=True)
        use_normals = normal_weight > 0.0 and view.normals is not None
        if use_normals:
            rp.feat = "Normals"
        api.render_forward(ctx, m, rp, stream, sync=True)
        self.view_acc.zero_()
        cs, ms = ctx.struct(), m.struct()
        masked_alpha = int(bool(masked and has_alpha))
        api._check(api.lib().b2k_evidence_view(C.byref(cs), api._ptr(view.rgba), api._ptr(view.normals) if use_normals else None, api._ptr(view.weights),
                                               masked_alpha, C.c_float(normal_weight), api._ptr(self.view_acc), api._stream(stream)), "evidence_view")
        if labels is not None:
            if self.votes is None:
                self.votes = torch.zeros((m.n, self.bins), dtype=torch.float32, device=self.device)
            api._check(api.lib().b2k_label_vote(C.byref(cs), api._ptr(view.rgba), api._ptr(labels), api._ptr(view.weights), masked_alpha, api._ptr(self.votes),
                                                api._stream(stream)), "label_vote")
        pos = (C.c_float * 3)(*[float(x) for x in cam["pos"]])
        api._check(api.lib().b2k_evidence_fold(C.byref(ms), api._ptr(self.view_acc), pos, api._ptr(self.acc), api._stream(stream)), "evidence_fold")

    def reduce(self, world):
        """Sum of the accumulators over ranks that each added their share of the views ([n][8], and [n][bins])."""
        if world > 1:
            torch.distributed.all_reduce(self.acc)
            if self.votes is not None:
                torch.distributed.all_reduce(self.votes)

    def download_evidence(self):
        a = self.acc.cpu().numpy().astype(np.float32)
        out = np.zeros((a.shape[0], 7), np.float32)
        out[:, :3] = a[:, :3]
        with np.errstate(divide="ignore", invalid="ignore"):
            out[:, 3] = np.where(a[:, 7] > 0, (a[:, 0] * a[:, 0]) / a[:, 7], 0.0)   # participation ratio: effective number of views
        out[:, 4:7] = a[:, 4:7]
        return out

    def download_labels(self):
        out = np.zeros((self.m.n, 2), np.float32)
        if self.votes is None:
            return out
        v = self.votes.cpu().numpy()
        total, win = v.sum(1, dtype=np.float32), v.argmax(1)
        best = v[np.arange(len(v)), win]
        ok = total > 0
        out[ok, 0], out[ok, 1] = win[ok], best[ok] / total[ok]
        return out
