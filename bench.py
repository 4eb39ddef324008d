"""Benchmark of the splat render-and-backprop hot path.

    python bench.py --gpus N --steps K --warmup W            (N > 1: under torchrun, one rank per GPU)
    python bench.py --impl reference ...                     (the CPU restatement of the reference path, host cores)

Workload (N = 1 and up): BASELINE config 2 -- 3M splats, SH degree 3, 64 views of 1920x1080 per step on a radius-4
sphere, targets = renders of a seed-distinct 3M-splat ground-truth set on black. One step = forward + L1/SSIM loss +
backward + projection backward for all 64 views (sharded over the ranks), one all-reduce of the 59-float per-splat
gradients when N > 1, then sparse Adam. Metric: train views/s, whole job. Inputs are seeded synthetic data.
`--workload stress` is BASELINE config 4 (1M heavy-tailed splats, 1024x1024, masked loss + alpha lane, one step);
`--workload render` measures BASELINE config 3 (6M splats, SH degree 4, 3840x2160 cameras, RGB + alpha + depth) in
Mpix/s instead; `--workload step1` BASELINE config 1 (500k splats, one 1080p view per step, fused optimizer).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def pick_chunks(n_splats):
    """Depth chunks of the front-to-back renderer by scene size, from measurements on one B200: 500k splats at 1080p 1.40 ms
    per step with 2 chunks (1.51 whole-view, 1.48 / 1.61 with 3 / 4); 3M splats at 1080p 604 / 623 / 618 views/s with 3 / 4 /
    5; 6M splats at 4K 2,012 / 2,406 / 2,485 Mpix/s with 3 / 4 / 5."""
    if n_splats >= 4_000_000:
        return 5
    if n_splats >= 1_000_000:
        return 4
    return 2 if n_splats >= 250_000 else 1


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b2k", choices=["b2k", "reference"])
    ap.add_argument("--workload", default="train", choices=["train", "render", "step1", "stress"])
    ap.add_argument("--splats", type=int, default=None, help="override the splat count (testing only; the line says so)")
    ap.add_argument("--views", type=int, default=None, help="override views per step / cameras (testing only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-incumbent", action="store_true", help="skip timing the reference CUDA kernels beside the product")
    ap.add_argument("--no-render", action="store_true", help="train workload: skip the render sub-object (config 3 sample)")
    ap.add_argument("--render-splats", type=int, default=None, help="override config 3's splat count in the render sub-object (testing only)")
    ap.add_argument("--views-in-flight", type=int, default=8, help="views of a step processed concurrently on separate streams")
    ap.add_argument("--allreduce", action="store_true", help="N > 1: ncclAllReduce of the dense gradient + replicated Adam instead of the sharded "
                    "peer-memory update")
    ap.add_argument("--chunks", type=int, default=0, help="depth chunks of the front-to-back renderer (1 = bin the whole view first, as the reference "
                    "does; 0 = choose: 4 for scenes of a million splats and more, where most intersections lie behind saturated pixels, else 1)")
    ap.add_argument("--render-lanes", type=int, default=4, help="render workload: cameras in flight on separate streams")
    ap.add_argument("--stage-views", type=int, default=4, help="views timed stage by stage for the roofline object")
    return ap.parse_args()


WORKLOADS = {"train": 2, "step1": 1, "render": 3, "stress": 4}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index):
        self.rows, self.proc, self.idx, self.t_mark = [], None, gpu_index, None

    def start(self):
        """Starts sampling (nvidia-smi needs about half a second before its first line: call this before the warm-up)."""
        if self.proc is not None:
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def mark(self):
        """The timed region starts now: stop() reports the samples taken from here on."""
        self.t_mark = time.monotonic()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        self.proc = None
        good = [(t, r) for t, r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        rows = [r for t, r in good if self.t_mark is None or t >= self.t_mark]
        window = "timed region"
        if not rows and good:   # a timed region shorter than the sampling period: the warm-up ran the same load just before it
            rows, window = [r for _, r in good[-4:]], "warm-up and timed region"
        if not rows:            # the whole run was shorter than nvidia-smi's start-up: one query right after it
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=10).stdout.strip().splitlines()
                rows = [[c.strip() for c in l.split(",")] for l in out if l.strip()]
                rows = [r for r in rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
                window = "one query right after the timed region"
            except (OSError, subprocess.SubprocessError):
                rows = []
        sm = [float(r[0]) for r in rows]
        mx = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [nm for k, nm in enumerate(names) if any(r[3 + k].lower().startswith("active") for r in rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm),
                "window": window}


def cpu_reference_arm(args, cfg):
    """The reference path on the host cores: the oracle port (forward + loss + analytic backward + Adam), all OpenMP
    threads, one view of the workload per step."""
    from b2ctrain_b200 import scenes
    from oracle import orc
    orc.set_num_threads(os.cpu_count() or 1)   # all host cores, also under a launcher that exported OMP_NUM_THREADS=1
    n0, deg = scenes.CONFIG_SPLATS[cfg]
    n = args.splats or n0
    scene = scenes.config_scene(cfg, n=n)
    cams = scenes.config_cameras(cfg)
    W, H = cams[0]["W"], cams[0]["H"]
    gt = np.full(W * H, 0xFF000000, np.uint32)
    lp = dict(l1_w=np.float32(0.8), ssim_w=np.float32(-0.2))
    K = (deg + 1) ** 2
    state = None
    times = []
    for s in range(args.warmup + args.steps):
        cam = cams[s % len(cams)]
        t0 = time.perf_counter()
        if args.workload == "render":
            orc.step(scene, cam, np.zeros(3), None, None, lp, backward=False, want_image=True)
        else:
            out = orc.step(scene, cam, np.zeros(3), gt, None, lp, backward=True)
            if state is None:
                z4 = lambda: np.zeros((n, 4), np.float32)
                state = dict(pos_op=scene["pos_op"], quat=scene["quat"], lscale=scene["lscale"], sh=scene["sh"], m_pos=z4(), v_pos=z4(), m_q=z4(),
                             v_q=z4(), m_ls=z4(), v_ls=z4(), m_sh=np.zeros((n, K, 3), np.float32), v_sh=np.zeros(n, np.float32),
                             last_step=np.zeros(n, np.uint32))
            orc.adam(state, out["grad"], np.any(out["grad"] != 0, axis=1), dict(t=s + 1, lr_mean=1.6e-4, sparse=1), deg)
        dt = time.perf_counter() - t0
        if s >= args.warmup:
            times.append(dt)
        if s == 0 and dt > 60:   # keep the arm within minutes
            times.append(dt)
            break
    sec = float(np.mean(times))
    if args.workload == "render":
        value, unit, metric = W * H / sec / 1e6, "Mpix/s", "render Mpix/s"
    else:
        value, unit, metric = 1.0 / sec, "views/s", "train views/s"
    return dict(value=value, unit=unit, metric=metric, cores=orc.num_threads(), sec_per_unit=sec, n=n, W=W, H=H,
                sample=f"{len(times)} x one view of the workload ({n} splats, {W}x{H}), forward+loss+backward+Adam" if args.workload != "render"
                else f"{len(times)} x one camera of the workload ({n} splats, {W}x{H}), forward only")


def main():
    # Stdout carries exactly one JSON line: anything a library prints there meanwhile (NCCL's version banner, for one) goes
    # to stderr instead.
    out_fd = os.dup(1)
    os.dup2(2, 1)
    emit = lambda obj: os.write(out_fd, (json.dumps(obj) + "\n").encode())
    args = parse()
    cfg = WORKLOADS[args.workload]
    if args.chunks <= 0:
        from b2ctrain_b200 import scenes as _scenes
        n_splats = args.splats or _scenes.CONFIG_SPLATS[cfg][0]
        args.chunks = pick_chunks(n_splats)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return
        # torchrun exports OMP_NUM_THREADS=1 to its ranks: the CPU arm uses every host core whatever launched it.
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
        r = cpu_reference_arm(args, cfg)
        line = {"metric": r["metric"], "value": r["value"], "unit": r["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": r["sec_per_unit"] * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
                "data": "synthetic", "impl": "reference",
                "config": {"workload": workload_name(args, cfg, r["n"]), "views_per_step": 1, "l2_policy": "inputs larger than L2"},
                "cpu_baseline": {"value": r["value"], "unit": r["unit"], "cores": r["cores"], "kind": "port", "sample": r["sample"], "dtype": "f64",
                                 "views_per_step": 1},
                "e2e": {"value": r["value"], "unit": r["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
        emit(line)
        return

    import torch
    import torch.distributed as dist
    from b2ctrain_b200 import api, scenes
    from b2ctrain_b200.trainer import Renderer, Trainer, render_targets

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    device = f"cuda:{local_rank}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(device))
    api.lib()

    n0, deg = scenes.CONFIG_SPLATS[cfg]
    n = args.splats or n0
    cams = scenes.config_cameras(cfg)
    if args.views:
        cams = cams[: args.views]
    W, H = cams[0]["W"], cams[0]["H"]
    scene = scenes.config_scene(cfg, n=n)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    if args.workload == "render":
        result = bench_render(args, scene, cams, device, rank, world, barrier, max_over_ranks, sampler)
    else:
        result = bench_train(args, cfg, scene, cams, device, rank, world, barrier, max_over_ranks, sampler)
        if args.workload == "train" and not args.no_render:
            # The second half of the metric: render Mpix/s on config 3 (6M splats SH4, 3840x2160, RGB + alpha + depth),
            # cameras split over the ranks, a bounded sample of the 256-camera orbit (16 cameras per rank).
            del scene
            torch.cuda.empty_cache()
            n3 = args.render_splats or scenes.CONFIG_SPLATS[3][0]
            cams3 = scenes.config_cameras(3)[:: max(1, 256 // (16 * world))][: 16 * world]
            rargs = argparse.Namespace(**{**vars(args), "steps": 1, "warmup": 3, "chunks": pick_chunks(n3)})
            r = bench_render(rargs, scenes.config_scene(3, n=n3), cams3, device, rank, world, barrier, max_over_ranks, ClockSampler(local_rank))
            if rank == 0:
                r["config"]["workload"] = workload_name(argparse.Namespace(splats=args.render_splats, views=None), 3, n3) + f" [sample: {len(cams3)} of its 256 cameras]"
                result["render"] = r
    if rank == 0:
        result.update({"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None, "data": "synthetic",
                       "dtype": "f32"})
        result["config"]["workload"] = workload_name(args, cfg, n)
        if not args.no_cpu_baseline and world == 1:
            r = cpu_reference_arm(argparse.Namespace(**{**vars(args), "steps": 1, "warmup": 0}), cfg)
            result["cpu_baseline"] = {"value": r["value"], "unit": r["unit"], "cores": r["cores"], "kind": "port", "sample": r["sample"], "dtype": "f64",
                                      "views_per_step": 1}
        emit(result)
    if world > 1:
        dist.destroy_process_group()


def workload_name(args, cfg, n):
    base = {1: "config1: 500k splats SH3, one 1920x1080 view per step, fused projection-backward + sparse Adam",
            2: "config2: 3M splats SH3, 64 views of 1920x1080 per step sharded by view, all-reduce of 59 floats per splat, sparse Adam",
            3: "config3: 6M splats SH4, 256 cameras of 3840x2160, RGB + alpha + depth, forward only",
            4: "config4: 1M heavy-tailed splats SH3, one 1024x1024 view per step, masked loss (ellipse, 40%) + alpha lane, scale 1/0.4, fused optimizer"}[cfg]
    if args.splats or args.views:
        base += f" [REDUCED for testing: splats={n}, views={args.views}]"
    return base


def presize(tr_or_r, cams, mine, targets, is_train):
    """Runs each of this rank's views once to size the intersection buffers (the reference grows them inside
    bin_and_sort; here the count stays on the device during the timed steps)."""
    import torch
    from b2ctrain_b200 import api
    ctx, m = tr_or_r.ctx, tr_or_r.model
    stats = []
    for v in mine:
        while True:
            rp = api.RenderParams(cams[v], sh_degree=m.degree, bwd_info=is_train)
            api.render_forward(ctx, m, rp, sync=False)
            total = int(ctx.d_num_isect[0].item()) & 0xFFFFFFFF
            if total <= ctx.isect_cap:
                break
            cap = ctx.isect_cap
            while cap < total:
                cap *= 2
            ctx._alloc_isect(cap)
        ranges = ctx.tile_ranges.view(-1, 2).clone()
        if ctx.n_chunks > 1:   # the chunked renderer leaves box areas in tile_count: count the exact intersections with the whole-view projection
            api.project_splats(ctx, m, rp)
        tc = ctx.tile_count[: m.n]
        stats.append(dict(V=int((tc != 0).sum().item()), I=int(tc.to(torch.int64).sum().item()), I_sorted=total,
                          I_b=int((ranges[:, 1].to(torch.int64) - ranges[:, 0]).clamp_(min=0).sum().item())))
    torch.cuda.synchronize()
    return stats


def bench_train(args, cfg, scene, cams, device, rank, world, barrier, max_over_ranks, sampler):
    import torch
    import torch.distributed as dist
    from b2ctrain_b200 import api, scenes
    from b2ctrain_b200.trainer import Trainer, render_targets
    n, deg = scene["n"], scene["degree"]
    W, H = cams[0]["W"], cams[0]["H"]
    P = W * H
    n_views = len(cams)
    gt_scene = scenes.config_scene(cfg, n=n, gt_set=True)
    mine = list(range(rank, n_views, world))
    noise = 0.05 if cfg == 1 else 0.0
    host_targets_mine, cap = render_targets(gt_scene, [cams[v] for v in mine], device, noise_sigma=noise, seed=1234 + rank)
    del gt_scene
    torch.cuda.empty_cache()
    host_targets = [None] * n_views
    for j, v in enumerate(mine):
        host_targets[v] = host_targets_mine[j]
    if args.chunks > 1:   # the chunked renderer sorts a fraction of what the whole-view target renders needed; the trainer regrows if it must
        cap = min(cap, 1 << 24)
    median_scale = float(np.median(np.exp(scene["lscale"][:, :3])))
    # The timed step runs in the C++ host (b2ctrain_b200/host/trainer.cpp behind libb2chost.so): views in flight, the
    # data-parallel split and every collective are C++ over the C ABI; this script only hands over scene, views and a stream.
    # MCMC noise on, as the reference's trainer applies it every step (src/train/trainer.cpp:524): lr_mean * mean_noise_weight
    # (default 50), clamp = median scale.
    from b2ctrain_b200 import host_trainer as ht
    lr_mean = 2e-5 * median_scale
    loss_kw = dict(mask=True, alpha_lane=True, loss_scale=1.0 / 0.4) if cfg == 4 else {}
    ident = [None]
    if world > 1:
        ident = [ht.make_dp_id() if rank == 0 else None]
        dist.broadcast_object_list(ident, src=0)
    lanes = 1 if n_views == 1 else args.views_in_flight
    tr = ht.HostTrainer(scene, W, H, rank=rank, world=world, dp_id=ident[0], views_in_flight=lanes, render_chunks=args.chunks, isect_cap=cap,
                        lr_mean=lr_mean, sparse=True, noise_weight=lr_mean * 50.0, noise_clamp=median_scale, shard_update=not args.allreduce, **loss_kw)
    if cfg == 4:   # per-pixel binary mask in the alpha byte, alpha-match lane, --normalize-masked-loss
        mask = torch.from_numpy(scenes.ellipse_mask(W, H, 0.4).astype(np.int64))
        for v in mine:
            t = host_targets[v].to(torch.int64) & 0xFFFFFFFF
            t = torch.where(mask > 0, (t & 0x00FFFFFF) | (255 << 24), torch.zeros_like(t))
            t = torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
            host_targets[v].copy_(t)
    for v in range(n_views):   # every rank knows every camera; targets only for the views it renders
        tr.add_view(cams[v], host_targets[v].numpy() if host_targets[v] is not None else None)
    all_views = list(range(n_views))
    stream = torch.cuda.current_stream().cuda_stream

    def timed(from_host, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        loss = None
        for _ in range(steps):
            tr.step(all_views, stream, from_host=from_host)
            loss = tr.read_loss(stream) if from_host else None   # the step's result read back (16 floats)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)), loss

    sampler.start()
    timed(False, args.warmup)       # also grows the intersection buffers to what the views need
    redos_warm = tr.info()["overflow_redos"]
    sampler.mark()
    ms, _ = timed(False, args.steps)
    clocks = sampler.stop()
    timed(True, 1)
    tr.info()                       # resets the byte counter
    ms_e2e, loss = timed(True, args.steps)
    info = tr.info()
    h2d = info["h2d_bytes"] / args.steps
    if world > 1:   # whole-job totals
        t = torch.tensor([h2d], dtype=torch.float64, device=device)
        dist.all_reduce(t)
        h2d = float(t.item())
    assert info["overflow_redos"] == redos_warm, "intersection buffers overflowed inside the timed region"
    phases = None
    if n_views > 1:   # one more step with an event after each phase; every phase reported as the max over ranks
        barrier()
        tr.set_profile(True)
        tr.step(all_views, stream)
        tr.set_profile(False)
        mine_ms = tr.info()["phase_ms"]
        phases = {k: max_over_ranks(v) for k, v in sorted(mine_ms.items())}
        phases["views_fastest_rank"] = -max_over_ranks(-mine_ms["views"])
        phases["update_form"] = ("Adam from the accumulator (one rank)" if world == 1 else "all-reduce + replicated Adam" if args.allreduce
                                 else "sharded: peer-memory reduce + Adam + parameter broadcast in one kernel")
    tile_bits = info["tile_bits"]
    cap = info["isect_cap"]
    tr.close()
    del tr
    torch.cuda.empty_cache()
    # Stage timing, counts and the roofline object: the same operators one stage at a time through the Python mirror (rank 0).
    py = stats = None
    if rank == 0:
        py = Trainer(scene, W, H, device, 0, 1, lr_mean=lr_mean, sparse=True, noise_weight=lr_mean * 50.0, noise_clamp=median_scale, isect_cap=cap,
                     views_in_flight=1, render_chunks=args.chunks)
        if cfg == 4:
            py.lp.mask, py.lp.alpha_lane, py.lp.scale = True, True, 1.0 / 0.4
        dev_targets = {v: host_targets[v].to(device) for v in mine[: max(1, args.stage_views)]}
        stats = presize(py, cams, mine[: max(1, args.stage_views)], dev_targets, True)

    views_per_step = n_views
    value = views_per_step * args.steps / (ms / 1e3)
    e2e_value = views_per_step * args.steps / (ms_e2e / 1e3)
    from b2ctrain_b200 import api as _api
    passes = int(_api.lib().b2k_sort_passes(int(tile_bits)))
    launches_view = 1 + (1 + 12 + 2 + 3 * passes + 1) + 1 + 1 + 1 + 1 + 1
    if args.chunks > 1:   # projection 2, depth sort 13, chunk words 1, per chunk 6 (+1 after the first) + the tile-sort passes, then loss .. projection backward
        launches_view = 2 + 13 + 1 + sum(6 + (2 if ch else 0) + 3 * passes for ch in range(args.chunks)) + 5
    launches = args.steps * (n_views * launches_view + (0 if (world == 1 and n_views == 1) else world))   # all ranks
    res = {"metric": "train views/s", "value": value, "unit": "views/s", "ms_per_step": ms / args.steps, "scaling": "strong",
           "config": {"views_per_step": views_per_step, "render": ("front to back in %d depth chunks, saturated tiles stop emitting" % args.chunks) if args.chunks > 1 else "whole view binned before compositing", "splats": n, "sh_degree": deg, "resolution": f"{W}x{H}", "parallelism": f"dp{world} by view",
                      "l2_policy": "inputs larger than L2 (per view > 126 MB of records, lists and images; 64 distinct views per step)",
                      "scene_counts_view0": stats[0] if stats else None},
           "e2e": {"value": e2e_value, "unit": "views/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 64, "ms_per_step": ms_e2e / args.steps},
           "gpu_launches": launches, "clocks": clocks, "loss_last_view": float(loss[0]) if loss is not None else None}
    if phases:
        res["step_phases_ms_max_over_ranks"] = phases
    res["config"]["host"] = "C++ (libb2chost.so): step loop, streams and collectives; Python passes scene, views and a stream"
    if rank == 0:
        res["roofline"], res["stages"] = stage_roofline(args, py, cams, dev_targets, mine, stats, clocks)
        if world == 1 and not args.no_incumbent:
            res["reference_cuda"] = incumbent(scene, cams[mine[0]], host_targets[mine[0]], cfg == 4)
    return res


def incumbent(scene, cam, host_target, masked):
    """The reference's own CUDA kernels (built unmodified for sm_100a, oracle/_ref/librefcuda.so) timed on one view of the
    same workload in the same run: its full single-view step (forward, loss, backward, fused optimizer), both backward
    variants. A reported comparison; the checker library is never part of the product path."""
    from oracle import orc
    if orc.refcuda_lib() is None:
        return {"unavailable": "oracle/_ref/librefcuda.so was not built (no reference tree at build time)"}
    try:
        ref = orc.RefCuda(scene, cam)
        ref.set_view(host_target.numpy().view(np.uint32))
        out = {}
        for name, tc in (("tc", True), ("warp", False)):
            ms = ref.time_steps(tensor_core=tc, warm=2, iters=5, lr_mean=0.0)
            out[name] = {"ms_per_view": ms, "views_per_s": 1e3 / ms}
        ref.close()
        out["what"] = "reference b2ctrain CUDA kernels, -O3 --use_fast_math, sm_100a, same B200, one view per step, 5 timed steps, learning rates 0 so the scene stays fixed"
        return out
    except Exception as e:   # the incumbent is informative only
        return {"unavailable": str(e)[:200]}


def stage_roofline(args, tr, cams, targets, mine, stats, clocks=None):
    """Times the stages of a view one at a time with CUDA events (on the launching stream) over a few views, in the
    form the timed steps ran (chunked or whole-view rendering), and derives the roofline object for the stage that takes
    longest. Algorithmic bytes / flops per stage: the `alg` / `flop` tables below, from the counts of the view measured
    on the device (n splats, V visible, I_sorted pairs sorted, I_b fragments inside the shrunk ranges, touched splats, P
    pixels, F fragment-pixel evaluations)."""
    import torch
    from b2ctrain_b200 import api
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"
    m, ctx = tr.model, tr.ctx
    K, chunks = m.K(), ctx.n_chunks
    views = mine[: max(1, args.stage_views)]
    names = (["render_chunked"] if chunks > 1 else ["project", "bin_sort", "raster_fwd"]) + ["loss", "raster_bwd", "proj_bwd"]
    acc = {k: 0.0 for k in names}
    touched = F = 0
    for v in views:
        rp = api.RenderParams(cams[v], sh_degree=m.degree, bwd_info=True)
        view = api.ViewGPU(targets[v], None, ctx.W, ctx.H)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
        torch.cuda.synchronize()
        ev[0].record()
        if chunks > 1:
            api.render_forward(ctx, m, rp, sync=False)
            k = 1
        else:
            api.project_splats(ctx, m, rp); ev[1].record()
            api.bin_and_sort(ctx, m, sync=False); ev[2].record()
            api.rasterize_forward(ctx, rp)
            k = 3
        ev[k].record(); api.photometric_loss(ctx, view, tr.lp)
        ev[k + 1].record(); api.rasterize_backward(ctx, m, rp)
        ev[k + 2].record(); api.projection_backward(ctx, m, tr._op(cams[v]), tr.grad)
        ev[k + 3].record()
        torch.cuda.synchronize()
        for j, nm in enumerate(names):
            acc[nm] += ev[j].elapsed_time(ev[j + 1])
        touched = int(ctx.d_num_isect[1].item()) & 0xFFFFFFFF     # splats the backward touched: the list the projection backward walks
        assert (int(ctx.d_num_isect[0].item()) & 0xFFFFFFFF) <= ctx.isect_cap, "a stage-timing view overflowed the intersection buffers"
        # F: fragments every pixel walked = sum over the tile's ranges of min(last, range end) - range start.
        last = (ctx.last_idx.to(torch.int64) & 0x7FFFFFFF)
        tx = (torch.arange(ctx.W, device=last.device) // 8).repeat(ctx.H)
        ty = (torch.arange(ctx.H, device=last.device) // 8).repeat_interleave(ctx.W)
        rg = ctx.tile_ranges.view(max(chunks, 1), ctx.n_tiles, 2).to(torch.int64)[:, ty * ctx.tiles_x + tx]
        F = int((torch.minimum(last[None, :], rg[:, :, 1]) - rg[:, :, 0]).clamp_(min=0).sum().item())
    tr.grad.zero_()
    nv = len(views)
    st = stats[0]
    V, I, Is, Ib, n, P, tiles = st["V"], st["I"], st["I_sorted"], st["I_b"], m.n, ctx.W * ctx.H, ctx.n_tiles
    passes = int(api.lib().b2k_sort_passes(int(ctx.tile_bits)))
    alg = {"project": 48 * n + 12 * K * V + 48 * V + 28 * n,
           "bin_sort": 16 * n * 4 + 24 * n + 8 * I + 16 * I * passes + 4 * I + 8 * tiles,
           "raster_fwd": 52 * Ib + 36 * P,
           # chunked renderer: records + colours of every splat, the depth sort, per chunk the rank / box words, then emit, tile
           # sort and ranges on the pairs that survive, and the compositing of what the ranges hold
           "render_chunked": (48 * n + 12 * K * V + 64 * n) + 16 * n * 4 + 20 * n + (8 + 16 * passes + 4) * Is + 8 * tiles * max(chunks, 1) + 52 * Ib + 36 * P,
           "loss": 20 * P + 16 * P, "raster_bwd": 28 * P + 52 * Ib + 52 * touched,
           "proj_bwd": (52 + 48 + 12 * K) * touched + 2 * 4 * (11 + 3 * K) * touched + 8 * n}   # flags of all splats, records of the touched ones
    # Loss: per pixel and channel 64/54 x (5 + 5 + 3) + 3 eleven-tap blurs (the strip's horizontal halo) = 203 FMA, plus the
    # moment products and the SSIM expression (~60 flop).
    flop = {"raster_fwd": 24 * F, "render_chunked": 24 * F, "raster_bwd": 90 * F, "loss": 3 * P * (2 * 203 + 60)}
    stages = {nm: {"ms": acc[nm] / nv, "algorithmic_bytes": int(alg[nm]), "achieved_gbs": alg[nm] / (acc[nm] / nv * 1e-3) / 1e9} for nm in names}
    if chunks <= 1:   # kernel-level split of the binning stage (events inside the library)
        ph = np.zeros(10)
        for v in views:
            api.project_splats(ctx, m, api.RenderParams(cams[v], sh_degree=m.degree, bwd_info=True))
            ph += np.array(api.bin_and_sort_profile(ctx, m))
        ph /= nv
        stages["bin_sort"]["phases_ms"] = {"depth_sort": ph[0], "scan_emit": ph[1], "tile_count": [ph[2 + 2 * p] for p in range(min(passes, 3))],
                                           "tile_scatter": [ph[3 + 2 * p] for p in range(min(passes, 3))], "tile_ranges": ph[8], "total": ph[9]}
    props = torch.cuda.get_device_properties(ctx.last_idx.device)
    sm_mhz = float((clocks or {}).get("sm_mhz") or 1965.0)   # median SM clock sampled during the timed region
    fp32_peak = 2 * 128 * props.multi_processor_count * sm_mhz * 1e6
    # Step roofline of the path that was timed: every stage at the larger of its HBM time and its FP32 time, never more than it took.
    t_roof = {nm: max(alg[nm] / (hbm * 1e9), flop.get(nm, 0) / fp32_peak) * 1e3 for nm in names}
    t_roof = {nm: min(t_roof[nm], stages[nm]["ms"]) for nm in names}
    measured = sum(stages[nm]["ms"] for nm in names)
    stages["step_roofline"] = {"t_roof_ms_per_view": sum(t_roof.values()), "t_measured_ms_per_view": measured, "frac": sum(t_roof.values()) / measured,
                               "per_stage_frac": {nm: t_roof[nm] / stages[nm]["ms"] for nm in names}, "fragment_pixel_evaluations": F,
                               "fp32_peak_tflops": fp32_peak / 1e12, "sm_mhz": sm_mhz, "touched_splats": touched,
                               "note": "stages of the timed form (" + ("chunked" if chunks > 1 else "whole-view") + " rendering) back to back on one stream; the "
                                       "optimizer update (once per step) is not included"}
    # The roofline object: the single-kernel stage with the largest time per view (the chunked renderer is ~70 launches, not one kernel).
    kernel_of = {"project": "project_kernel", "raster_fwd": "raster_fwd_kernel", "loss": "photometric_strip_kernel", "raster_bwd": "raster_bwd_kernel", "proj_bwd": "proj_bwd_kernel"}
    kernel_ms = {kernel_of[nm]: stages[nm]["ms"] for nm in names if nm in kernel_of}
    if chunks <= 1:
        kernel_ms["radix_scatter_kernel"] = float(np.mean(stages["bin_sort"]["phases_ms"]["tile_scatter"]))
    top = max(kernel_ms, key=kernel_ms.get)
    per_launch_ms = kernel_ms[top]
    if top == "radix_scatter_kernel":
        stage, bytes_launch, traffic = "bin_sort", 16 * I, int(16.7 * I)   # dram read + write per launch: ncu capture at half the splat count, scaled by pairs
        note = f"{passes} launches per view on I = {I} pairs; 16 B per pair per launch"
    else:
        stage = [k for k, v in kernel_of.items() if v == top][0]
        bytes_launch, traffic, note = alg[stage], None, "one launch per view"
        if top == "raster_bwd_kernel":
            traffic = int(80.7 * Ib)   # dram read + write per launch from an ncu capture at half the splat count (100.3 MB at I_b = 1,243,915), scaled by fragments
        elif top == "photometric_strip_kernel":
            traffic = int(22.7 * P)    # ncu capture of one 1920x1080 view: 43.1 MB read + 4.0 MB written (the gradient image stays in L2)
    a = bytes_launch / (per_launch_ms * 1e-3) / 1e9
    hbm_view = {"achieved": a, "peak": hbm, "unit": "GB/s", "frac": a / hbm, "traffic": traffic, "peak_source": peak_src, "algorithmic_bytes_per_launch": int(bytes_launch)}
    if stage in flop:   # the compositing kernels are bound by FP32 issue: that roof is the headline, the HBM figure rides beside it
        f = flop[stage] / (per_launch_ms * 1e-3)
        roof = {"bound": "fp32", "kernel": top, "achieved": f / 1e12, "peak": fp32_peak / 1e12, "unit": "TFLOP/s", "frac": f / fp32_peak, "traffic": traffic,
                "peak_source": "2 x 128 lanes x SMs x the SM clock sampled in the timed region (no tensor pipe on this path)",
                "flop_per_launch": flop[stage], "hbm": hbm_view}
        if stage != "loss":
            roof["fragment_pixel_evaluations"] = F
    else:
        roof = {"bound": "hbm", "kernel": top, **hbm_view}
    roof.update({"ms_per_launch": per_launch_ms, "note": note, "kernel_ms_per_view": {k: float(v) for k, v in kernel_ms.items()}})
    return roof, stages


def bench_render(args, scene, cams, device, rank, world, barrier, max_over_ranks, sampler):
    import torch
    from b2ctrain_b200.trainer import Renderer
    W, H = cams[0]["W"], cams[0]["H"]
    mine = list(range(rank, len(cams), world))
    from b2ctrain_b200 import host_trainer as ht
    r = Renderer(scene, W, H, device, rank, world, want_depth=True, render_chunks=args.chunks)
    stats = presize(r, cams, mine, None, False)   # counts of the first camera through the Python mirror, outside any timed region
    tile_bits, r_cap = r.ctx.tile_bits, r.ctx.isect_cap
    del r
    torch.cuda.empty_cache()
    # The timed loops run in the C++ host (b2c::StreamRenderer). e2e: every camera's RGBA8 image and depth map land in pinned
    # host memory, copied on a second stream while the next camera renders; the last copy is inside the timed region.
    lanes = max(1, args.render_lanes)
    hr = ht.HostRenderer(scene, W, H, depth=True, render_chunks=args.chunks, lanes=lanes, isect_cap=r_cap)
    slots = lanes + 1
    host_rgba = [torch.empty(W * H, dtype=torch.int32).pin_memory() for _ in range(slots)]
    host_depth = [torch.empty(W * H, dtype=torch.float32).pin_memory() for _ in range(slots)]
    stream = torch.cuda.current_stream().cuda_stream

    def timed(steps, e2e):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            for j, v in enumerate(mine):
                if e2e:
                    hr.render(cams[v], stream, host_rgba8=host_rgba[j % slots].data_ptr(), host_depth=host_depth[j % slots].data_ptr())
                else:
                    hr.render(cams[v], stream)
        hr.finish()   # every camera rendered (and, end to end, read back)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    sampler.start()
    timed(max(1, args.warmup // 3), False)
    sampler.mark()
    ms = timed(args.steps, False)
    clocks = sampler.stop()
    ms_e2e = timed(args.steps, True)
    hr.close()
    mpix = len(cams) * W * H * args.steps / 1e6
    from b2ctrain_b200 import api as _api
    passes = int(_api.lib().b2k_sort_passes(int(tile_bits)))
    launches_view = 1 + (1 + 12 + 2 + 3 * passes + 1) + 1
    if args.chunks > 1:
        launches_view = 2 + 13 + 1 + sum(6 + (2 if ch else 0) + 3 * passes for ch in range(args.chunks))
    return {"metric": "render Mpix/s", "value": mpix / (ms / 1e3), "unit": "Mpix/s", "ms_per_step": ms / args.steps, "scaling": "strong",
            "config": {"cameras": len(cams), "render": ("front to back in %d depth chunks, saturated tiles stop emitting" % args.chunks) if args.chunks > 1 else "whole view binned before compositing", "splats": scene["n"], "sh_degree": scene["degree"], "resolution": f"{W}x{H}", "parallelism": f"cameras over {world} GPUs", "cameras_in_flight": lanes,
                       "l2_policy": "inputs larger than L2", "scene_counts_view0": stats[0] if stats else None},
            "e2e": {"value": mpix / (ms_e2e / 1e3), "unit": "Mpix/s", "h2d_bytes_per_step": 100 * len(cams), "d2h_bytes_per_step": 8 * W * H * len(mine),
                    "what": "RGBA8 image (quantised on the device) + fp32 depth map of every camera into pinned host memory, copies overlapped with the next render"},
            "gpu_launches": args.steps * len(mine) * launches_view, "clocks": clocks}


if __name__ == "__main__":
    main()
