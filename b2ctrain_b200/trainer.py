"""The per-step sequence of the reference's trainer and renderer over the operator API, with view-level data
parallelism.

`Trainer.step` follows one iteration of train_phase (src/train/trainer.cpp:452-529): per view render_forward,
photometric_loss, accumulate_loss, rasterize_backward, then the parameter update. The reference's step is one view on
one GPU; here a step may hold several views and several ranks:

  * every rank holds a full model replica and renders the views `rank, rank + world, ...` of the step;
  * each view's projection backward ADDS into a dense per-splat gradient accumulator [n][11+3K] (the layout of the
    reference's OptimParams::grad_out lane, src/gpu/optim.cu:292-297);
  * an all-reduce (sum) of that accumulator over NCCL, then the identical Adam update on every rank, so replicas stay
    bit-identical. The accumulator is reduced in a few slices of splats and the update of a slice runs while the next
    slice is still on the wire. The step loss is the sum of the per-view losses (its gradient is the all-reduced sum).

A single-view, single-rank step uses the fused projection-backward + Adam kernel exactly like the reference.
`Renderer.render` follows render_main's per-camera loop (src/render/renderer.cpp:345-363) up to the device image.
"""
import numpy as np
import torch

from . import api


def partition_views(n_views, rank, world):
    """Views of a step taken by `rank`: round-robin, so every rank gets the same count (+-1) whatever the step size."""
    return list(range(rank, n_views, world))


def slice_bounds(n, slices, align=128):
    """Splits the splats [0, n) into up to `slices` contiguous ranges whose starts are multiples of `align` (the update
    kernel's block), returned as (first, count) pairs that cover [0, n) exactly."""
    if n <= 0:
        return []
    per = -(-n // max(1, slices))
    per = -(-per // align) * align
    return [(a, min(per, n - a)) for a in range(0, n, per)]


def reduce_gradients(grad, world):
    """Sum of the per-rank gradient accumulators over all ranks (NCCL on GPUs, gloo in the CPU tests)."""
    if world > 1:
        torch.distributed.all_reduce(grad, op=torch.distributed.ReduceOp.SUM)
    return grad


# How each refinement statistic combines over ranks that saw different views: refine_norm and max_screen are running
# maxima (optim.cu:122-124, project.cu:82-83), vis_count and vis_weight running sums (optim.cu:122, raster_bwd.cu:134).
STATISTIC_REDUCTIONS = {"refine_norm": "max", "max_screen": "max", "vis_count": "sum", "vis_weight": "sum"}


def reduce_statistics(stats, world):
    """All-reduces the per-splat refinement statistics in place so that every rank holds what a single process that
    rendered all views would hold. `stats` maps the names of STATISTIC_REDUCTIONS to tensors [n]. Call it once before
    the statistics are read (the refinement pass) and clear them afterwards on every rank: reducing twice without a
    clear would count the sums twice."""
    if world > 1:
        ops = {"max": torch.distributed.ReduceOp.MAX, "sum": torch.distributed.ReduceOp.SUM}
        for name, how in STATISTIC_REDUCTIONS.items():
            if name in stats and stats[name] is not None:
                torch.distributed.all_reduce(stats[name], op=ops[how])
    return stats


class Trainer:
    def __init__(self, cloud, W, H, device="cuda:0", rank=0, world=1, lr_mean=1.6e-4, sparse=True, noise_weight=0.0,
                 noise_clamp=0.0, ssim_weight=0.2, isect_cap=None, views_in_flight=1, reduce_slices=4, render_chunks=1):
        self.device = torch.device(device)
        self.rank, self.world = rank, world
        self.model = api.Model(device).upload(cloud)
        # One context and stream per view in flight: views of a step are independent until the update, so the
        # latency-bound raster kernels of one view overlap the throughput-bound binning of another. All of them add
        # into one gradient accumulator (the projection backward accumulates with reductions at the L2).
        self.lanes = max(1, int(views_in_flight))
        self.reduce_slices = int(reduce_slices)
        self.ctxs = [api.RenderCtx(device) for _ in range(self.lanes)]
        for c in self.ctxs:
            c.setup(W, H, self.model.cap, isect_cap=isect_cap, n_chunks=render_chunks)   # > 1: front-to-back depth chunks
        self.ctx = self.ctxs[0]
        self.streams = [torch.cuda.Stream(device=self.device) for _ in range(self.lanes)] if self.lanes > 1 else [None]
        self.W, self.H = W, H
        self.lr_mean, self.sparse = lr_mean, sparse
        self.noise_weight, self.noise_clamp = noise_weight, noise_clamp
        self.lp = api.LossParams(l1_w=1.0 - ssim_weight, ssim_w=-ssim_weight)
        K = self.model.K()
        self.grad = torch.zeros((self.model.n, 11 + 3 * K), dtype=torch.float32, device=self.device)
        self.step_no = 0
        P = W * H
        # device staging for targets that arrive from host memory (double-buffered on a copy stream)
        self._stage = [torch.zeros(P, dtype=torch.int32, device=self.device) for _ in range(2 * self.lanes)]
        self._copy_stream = torch.cuda.Stream(device=self.device)
        self._staged_evt = [torch.cuda.Event() for _ in range(2 * self.lanes)]
        self._free_evt = [torch.cuda.Event() for _ in range(2 * self.lanes)]
        self.h2d_bytes = 0
        self.overflow_redos = 0  # steps whose views were redone with larger intersection buffers
        self.profile = False     # when set, step() records an event after each phase (read with phase_ms())
        self._marks = []

    def _mark(self, name):
        if self.profile:
            e = torch.cuda.Event(enable_timing=True)
            e.record(torch.cuda.current_stream(self.device))
            self._marks.append((name, e))

    def phase_ms(self):
        """Device time of each phase of the last profiled step: 'views', then 'all_reduce' and 'adam' or, when
        the two are pipelined by slices, 'all_reduce+adam'."""
        torch.cuda.synchronize(self.device)
        out = {}
        for (_, a), (name, b) in zip(self._marks[:-1], self._marks[1:]):
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out

    def my_views(self, n_views):
        return partition_views(n_views, self.rank, self.world)

    def _target(self, t, slot):
        """A device int32 tensor of packed RGBA8. Host (pinned) tensors are copied on the copy stream."""
        if t.is_cuda:
            return t
        dst = self._stage[slot]
        cur = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(self._free_evt[slot])
            dst.copy_(t, non_blocking=True)
            self._staged_evt[slot].record(self._copy_stream)
        cur.wait_event(self._staged_evt[slot])
        self.h2d_bytes += t.numel() * 4
        return dst

    def view_pass(self, cam, target, bg=(0.0, 0.0, 0.0), weights=None, slot=0, fused_op=None, lane=0):
        """forward + loss + backward of one view; then either the fused optimizer (fused_op given) or the gradient
        accumulation into the lane's accumulator. Runs on the current stream with the lane's context."""
        m, ctx = self.model, self.ctxs[lane]
        rp = api.RenderParams(cam, bg=bg, sh_degree=m.degree, bwd_info=True)
        api.render_forward(ctx, m, rp, sync=False)
        tgt = self._target(target, slot)
        view = api.ViewGPU(tgt, weights, self.W, self.H)
        api.photometric_loss(ctx, view, self.lp)
        if not target.is_cuda:
            self._free_evt[slot].record(torch.cuda.current_stream(self.device))
        api.accumulate_loss(ctx)
        api.rasterize_backward(ctx, m, rp)
        if fused_op is not None:
            api.optimizer_step(ctx, m, fused_op)
        else:
            api.projection_backward(ctx, m, self._op(cam), self.grad)

    def _op(self, cam):
        return api.OptimParams(cam, active_sh_degree=self.model.degree, t=self.model.adam_t, lr_mean=self.lr_mean, sparse=self.sparse,
                               noise_weight=self.noise_weight, noise_clamp=self.noise_clamp, step=self.step_no)

    def step(self, cams, targets, bg=(0.0, 0.0, 0.0)):
        """One optimisation step over `cams` / `targets` (the whole step's views; this rank takes its share).
        Returns the device tensor loss_accum (index 0: loss of the last view, 2: running sum, 3: count).

        The intersection totals stay on the device while the views run; once per step the largest total of every lane
        is read back (4 bytes per lane), and when a view did not fit, the buffers grow and the rank's views are redone
        (the reference grows inside every bin_and_sort, src/gpu/binning.cu:125-133). Nothing is lost by the late
        check: a view that overflowed adds nothing to the accumulator or the model (b2k_proj_bwd / b2k_optim_fused)."""
        m = self.model
        m.adam_t += 1
        self.step_no += 1
        mine = self.my_views(len(cams))
        self._marks = []
        self._mark("start")
        fused = self.world == 1 and len(cams) == 1
        while True:
            self._views(cams, targets, bg, mine, fused)
            if not self.check_overflow()[1]:
                break
            self.overflow_redos += 1
            if not fused:
                self.grad.zero_()
        if fused:
            return self.ctx.loss_accum
        self._mark("views")
        op = self._op(cams[0])
        if self.world == 1 or self.reduce_slices <= 1:
            reduce_gradients(self.grad, self.world)
            self._mark("all_reduce")
            api.adam_step(m, op, self.grad)
            self._mark("adam")
        else:
            # NCCL runs the slices in issue order on its own stream; the update of slice k waits for reduction k only.
            bounds = slice_bounds(m.n, self.reduce_slices)
            works = [torch.distributed.all_reduce(self.grad[a:a + c], op=torch.distributed.ReduceOp.SUM, async_op=True) for a, c in bounds]
            for (a, c), w in zip(bounds, works):
                w.wait()
                api.adam_step(m, op, self.grad, first=a, count=c)
            self._mark("all_reduce+adam")
        return self.ctx.loss_accum

    def _views(self, cams, targets, bg, mine, fused):
        """Forward, loss and backward of this rank's views, `lanes` of them in flight; every lane's running loss ends
        up in lane 0's accumulator."""
        for c in self.ctxs:
            api.step_begin(c)            # every lane, also the ones that get no view this step
        if fused:
            self.view_pass(cams[0], targets[0], bg, fused_op=self._op(cams[0]))
        elif self.lanes == 1:
            for j, v in enumerate(mine):
                api.zero_loss(self.ctx, 0, 2)
                self.view_pass(cams[v], targets[v], bg, slot=j & 1)
        else:
            main = torch.cuda.current_stream(self.device)
            start = torch.cuda.Event(); start.record(main)
            for j, v in enumerate(mine):
                lane = j % self.lanes
                with torch.cuda.stream(self.streams[lane]):
                    if j < self.lanes:
                        self.streams[lane].wait_event(start)
                    api.zero_loss(self.ctxs[lane], 0, 2)
                    self.view_pass(cams[v], targets[v], bg, slot=2 * lane + ((j // self.lanes) & 1), lane=lane)
            used = min(self.lanes, len(mine))
            for lane in range(used):
                done = torch.cuda.Event(); done.record(self.streams[lane]); main.wait_event(done)
            for lane in range(1, used):       # fold the lanes' running losses into lane 0
                api.fold_loss(self.ctx, self.ctxs[lane])

    def reduce_statistics(self):
        """Makes the refinement statistics of the model global over the ranks (see reduce_statistics above)."""
        m = self.model
        reduce_statistics({k: getattr(m, k)[:m.n] for k in STATISTIC_REDUCTIONS}, self.world)

    def check_overflow(self):
        """Reads every lane's largest intersection total of the step back; grows the buffers of a lane that did not
        hold it (the reference does this inside every bin_and_sort, src/gpu/binning.cu:125-133). Returns
        (largest total, whether any lane grew)."""
        total, over = 0, False
        torch.cuda.synchronize(self.device)
        for ctx in self.ctxs:
            t = int(ctx.d_num_isect[2].item()) & 0xFFFFFFFF
            total = max(total, t)
            if t > ctx.isect_cap:
                cap = ctx.isect_cap
                while cap < t + 32 * max(1, ctx.n_chunks):
                    cap *= 2
                ctx._alloc_isect(cap)
                over = True
        return total, over


class Renderer:
    """Forward-only rendering of cameras split round-robin over ranks; outputs stay on the producing GPU."""

    def __init__(self, cloud, W, H, device="cuda:0", rank=0, world=1, want_depth=True, isect_cap=None, render_chunks=1):
        self.device = torch.device(device)
        self.rank, self.world = rank, world
        self.model = api.Model(device).upload(cloud)
        self.ctx = api.RenderCtx(device)
        self.ctx.want_depth = want_depth
        self.ctx.setup(W, H, self.model.cap, isect_cap=isect_cap, n_chunks=render_chunks)

    def render(self, cam, bg=(0.0, 0.0, 0.0), sync=False):
        rp = api.RenderParams(cam, bg=bg, sh_degree=self.model.degree, bwd_info=False)
        api.render_forward(self.ctx, self.model, rp, sync=sync)
        return self.ctx.out_rgba, self.ctx.out_depth


def render_targets(cloud, cams, device="cuda:0", noise_sigma=0.0, seed=0, alpha=255, isect_cap=None):
    """Targets for the synthetic benchmark: renders of a ground-truth splat set on black, optional N(0, sigma) pixel
    noise, clamped and quantised to packed RGBA8 like the reference's rendered targets (src/train/teacher.cu:11-17).
    Returns a list of host (pinned) int32 tensors."""
    W, H = cams[0]["W"], cams[0]["H"]
    r = Renderer(cloud, W, H, device, want_depth=False, isect_cap=isect_cap)
    gen = torch.Generator(device=device); gen.manual_seed(seed)
    out = []
    for cam in cams:
        while True:
            img, _ = r.render(cam, sync=False)
            total = int(r.ctx.d_num_isect[0].item()) & 0xFFFFFFFF
            if total <= r.ctx.isect_cap:
                break
            cap = r.ctx.isect_cap
            while cap < total:
                cap *= 2
            r.ctx._alloc_isect(cap)
        img = img.clone()
        if noise_sigma > 0:
            img[:, :3] += torch.randn((W * H, 3), generator=gen, device=device) * noise_sigma
        packed = torch.zeros(W * H, dtype=torch.int32, device=device)
        api.pack_rgba8(img.clamp_(0.0, 1.0), packed, alpha_override=alpha)
        host = torch.empty(W * H, dtype=torch.int32).pin_memory()
        host.copy_(packed)
        out.append(host)
    torch.cuda.synchronize()
    return out, r.ctx.isect_cap
