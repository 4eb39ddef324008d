"""Pins on the reference's OWN CUDA kernels (oracle/_ref/librefcuda.so, built unmodified for sm_100a) for the parts of
the path its CPU check never exercises: the Adam / Adam-mini / lazy catch-up / MCMC-noise update of optimizer_step,
the evaluation metrics, and one full-size view of each benchmark configuration (image, loss, parameter gradients),
together with the full-size identity of the chunked renderer and the whole-view binning."""
import numpy as np
import pytest

from b2ctrain_b200 import scenes
from oracle import orc
from tests.util import Harness, rel_l2

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(orc.refcuda_lib() is None, reason="oracle/_ref/librefcuda.so was not built (no reference tree at build time)")]

# Stated tolerances. Both sides are fp32 kernels; the reference side is compiled with --use_fast_math.
TOL_STEP_UPDATE = 1e-4       # a parameter's update (new - old) after a plain Adam step, relative to the update + the group's step scale
TOL_STEP_UPDATE_GAP = 2e-3   # ... at the third step, a lazy catch-up over skipped steps (fp32 1 - 0.999^t cancels, and the two
                             # sides have run on their own states since the first step; observed 9e-4)
TOL_STEP_VALUE = 4e-7        # plus this much of (|value| + 1): fp32 rounding of the stored parameter
TOL_STEP_MOMENT = 2e-5       # Adam moments, relative L2
TOL_FULL_IMAGE = 1e-3        # full-size image, abs, for all but TOL_FULL_IMAGE_OFF of the pixels
TOL_FULL_IMAGE_OFF = 1e-5    # fraction of pixels that may sit on a discrete decision (alpha cut, transmittance stop)
TOL_FULL_IMAGE_ONE_FRAGMENT = 5e-3   # and what such a pixel may differ by (observed: 1.3e-3 .. 2.0e-3)
TOL_FULL_LOSS = 2e-4         # full-size loss, relative (observed 2e-6 .. 1e-4)
TOL_FULL_GRAD = 2e-4         # full-size parameter gradients (grad_out), relative L2 (observed 1.2e-5 .. 7.6e-5)


def optimizer_scene(degree):
    scene = scenes.make_splats(3000, degree, 31 + degree, log_scale=(-3.2, 0.5))
    rng = np.random.Generator(np.random.PCG64(5))
    faint = rng.random(scene["n"]) < 0.35            # near-transparent splats: the only ones the MCMC noise moves, (1 - o)^150
    scene["pos_op"][faint, 3] = rng.uniform(-5.3, -3.5, int(faint.sum())).astype(np.float32)
    cam = scenes.look_at_camera(scenes.orbit_eye(3.0, 25.0, 10.0), 160, 120, 120.0)
    return scenes.floor_for_cameras(scene, [cam]), cam


def product_state(h):
    m, n = h.model, h.model.n
    d = m.download()
    f = lambda t: t[:n].cpu().numpy()
    d.update(m_pos=f(m.m_pos_op), v_pos=f(m.v_pos_op), m_q=f(m.m_quat), v_q=f(m.v_quat), m_ls=f(m.m_lscale), v_ls=f(m.v_lscale),
             m_sh=m.sh_planar_to_host(m.m_sh_dc, m.m_sh_hi), v_sh=f(m.v_sh), last_step=h.u32(m.last_step, n), vis_count=f(m.vis_count),
             refine_norm=f(m.refine_norm))
    return d


@pytest.mark.parametrize("variant", ["fused", "split", "fused_dense"])
def test_optimizer_step_matches_the_reference_kernel(variant):
    """One real optimizer step at t = 1, 2 and, after a gap, 5 (lazy catch-up), MCMC noise on with a fixed seed, from
    identical screen-space lanes: parameters, moments, Adam-mini second moment, last_step and the statistics against
    the reference's optim_kernel (src/gpu/optim.cu:100-378). `split` is b2k_proj_bwd + b2k_adam."""
    degree = 3 if variant != "split" else 2
    scene, cam = optimizer_scene(degree)
    n, K = scene["n"], (degree + 1) ** 2
    sparse = variant != "fused_dense"
    rng = np.random.Generator(np.random.PCG64(77))
    ref = orc.RefCuda(scene, cam)
    h = Harness(scene, cam)
    kw = dict(lr_mean=1.6e-4, noise_weight=5e-3, noise_clamp=2e-3, seed=1234)
    moved_by_noise = 0
    # Adam normalises every component by its own second moment, so a gradient component that is zero up to rounding
    # (1e-6 of its group's largest) takes a full +-lr step whose sign is the sign of the rounding error: such
    # components are excluded from the parameter comparison of the element-wise groups (they must stay rare).
    sure = {k: np.ones((n, 4), bool) for k in ("pos_op", "quat", "lscale")}
    # A splat whose opacity sits on the 1/255 cull threshold has a gradient on one side of the comparison and none on
    # the other (the two projections differ in the last bits, and the opacity itself moves by about a percent per step):
    # splats within 8 % of the threshold are left out.
    s2, f2 = np.exp(2.0 * scene["lscale"][:, :3].astype(np.float64)), scene["lscale"][:, 3:4].astype(np.float64) ** 2
    opac = np.sqrt(np.prod(s2 / (s2 + f2), axis=1)) / (1.0 + np.exp(-scene["pos_op"][:, 3].astype(np.float64)))
    rows = np.abs(opac * 255.0 - 1.0) > 0.08
    assert rows.mean() > 0.95

    def set_product_lanes():
        h.ctx.v_splat[:n].copy_(h.torch.from_numpy(v_splat)); h.ctx.vis_flag[:n].copy_(h.torch.from_numpy(vis.view(np.int32)))

    for t in (1, 2, 5):
        ref.forward(); h.forward()                      # tile counts of the current parameters on both sides
        v_splat = (rng.standard_normal((n, 13)) * 1e-2).astype(np.float32); v_splat[:, 9] = np.abs(v_splat[:, 9]); v_splat[:, 10:] = 0
        vis = (rng.random(n) < 0.6).astype(np.uint32)
        v_splat[vis == 0] = 0
        ref.set_lanes(v_splat, vis)
        set_product_lanes()
        G = h.torch.zeros((n, 11 + 3 * K), dtype=h.torch.float32, device="cuda:0")
        h.api.optimizer_step(h.ctx, h.model, h.api.OptimParams(cam, active_sh_degree=degree, grad_out=G))   # consumes the lanes
        g = np.abs(G.cpu().numpy())
        for k, lo, hi in (("pos_op", 0, 4), ("quat", 4, 8), ("lscale", 8, 11)):
            grp = g[:, lo:hi]
            sure[k][:, : hi - lo] &= (grp >= 1e-6 * grp.max(1, keepdims=True)) | (grp.max(1, keepdims=True) == 0)
        # the gradient pass above also counted the visibility statistic: put it back, the step below counts it once
        h.model.vis_count[:n].copy_(h.torch.from_numpy(ref.download("vis_count", (n,), np.float32)))
        set_product_lanes()
        start = product_state(h)
        before = start["pos_op"][:, :3].copy()
        ref.optim(t=t, sparse=sparse, step=t, **kw)
        op = h.api.OptimParams(cam, active_sh_degree=degree, t=t, sparse=sparse, step=t, **kw)
        if variant == "split":
            g = h.torch.zeros((n, 11 + 3 * K), dtype=h.torch.float32, device="cuda:0")
            h.api.projection_backward(h.ctx, h.model, op, g)
            h.api.adam_step(h.model, op, g)
        else:
            h.api.optimizer_step(h.ctx, h.model, op)
        h.torch.cuda.synchronize()
        want, got = ref.model_state(), product_state(h)
        # A parameter is held through its UPDATE: the two steps may differ by TOL_STEP_UPDATE of the step taken (fp32
        # bias corrections 1 - beta^t cancel, and the reference evaluates powf under fast-math), plus the rounding of the
        # value itself. The same bound relative to the value would be meaningless for a logit that lands next to zero.
        tol = TOL_STEP_UPDATE if t <= 2 else TOL_STEP_UPDATE_GAP
        for k in ("pos_op", "quat", "lscale", "sh"):
            # the step scale of the group: its learning rate (Adam's normalised step), for the means also the noise clamp
            scale = {"pos_op": np.array([kw["lr_mean"] + kw["noise_clamp"]] * 3 + [0.012]), "quat": 2e-3, "lscale": 5e-3, "sh": 2e-3}[k]
            bound = tol * (np.abs(want[k] - start[k]) + scale) + TOL_STEP_VALUE * (np.abs(want[k]) + 1.0)
            excess = (np.abs(got[k] - want[k]) / bound)[rows]
            if k in sure:
                assert sure[k].mean() > 0.995, (k, sure[k].mean())
                excess = excess[sure[k][rows]]
            assert float(excess.max()) <= 1.0, (variant, t, k, float(excess.max()))
        for k in ("m_pos", "v_pos", "m_q", "v_q", "m_ls", "v_ls", "m_sh", "v_sh"):
            assert rel_l2(got[k][rows], want[k][rows]) <= TOL_STEP_MOMENT, (variant, t, k, rel_l2(got[k][rows], want[k][rows]))
        assert np.array_equal(got["last_step"][rows], want["last_step"][rows]), (variant, t)
        assert np.array_equal(got["vis_count"], want["vis_count"]) and rel_l2(got["refine_norm"], want["refine_norm"]) <= 1e-6
        # the Adam step of a mean is at most lr_mean; anything larger is the noise draw
        moved_by_noise += int((np.abs(got["pos_op"][:, :3] - before).max(1) > 4 * kw["lr_mean"]).sum())
    ref.close()
    assert moved_by_noise > 200, moved_by_noise        # the noise lane was really exercised


@pytest.mark.parametrize("mask_weighted", [False, True])
def test_eval_metrics_match_oracle_and_reference_kernel(mask_weighted):
    """b2k_eval_metrics (eval_kernel, src/gpu/loss.cu:241-293): squared-error and SSIM sums of the 8-bit-quantised
    prediction, plain and alpha-weighted, on a ragged image, against the double oracle and the reference's kernel."""
    W, H = 83, 61
    rng = np.random.Generator(np.random.PCG64(17 + int(mask_weighted)))
    scene = scenes.make_splats(16, 0, 3)
    cam = scenes.look_at_camera(scenes.orbit_eye(3.0, 25.0, 10.0), W, H, float(H))
    gt = rng.integers(0, 2 ** 32, W * H, dtype=np.uint64).astype(np.uint32)
    pred = (rng.random((W * H, 4)) * 1.2 - 0.1).astype(np.float32)      # some values outside [0, 1]: the clamp is exercised
    pred[: W * 16, :3] = ((gt[: W * 16, None] >> np.array([0, 8, 16], np.uint32)) & 0xFF).astype(np.float32) / 255.0   # a band equal to the target
    h = Harness(scene, cam, gt, None, dict(l1_w=0.8, ssim_w=-0.2))
    h.ctx.out_rgba.copy_(h.torch.from_numpy(pred))
    h.api.zero_loss(h.ctx)
    h.api.eval_metrics(h.ctx, h.view, mask_weighted)
    acc = h.ctx.loss_accum.cpu().numpy()
    want = orc.eval_metrics(W, H, pred, gt, mask_weighted)
    assert abs(acc[4] - want[0]) <= 1e-5 * want[0] and abs(acc[5] - want[1]) <= 1e-5 * abs(want[1]), (acc[4:6], want)
    assert np.all(acc[:4] == 0) and np.all(acc[6:] == 0)
    h.api.eval_metrics(h.ctx, h.view, mask_weighted)                    # the sums accumulate across calls
    assert abs(float(h.ctx.loss_accum[4]) - 2 * want[0]) <= 2e-5 * want[0]
    ref = orc.RefCuda(scene, cam)
    ref.set_view(gt); ref.set_image(pred)
    theirs = ref.eval_metrics(mask_weighted)
    ref.close()
    assert abs(acc[4] - theirs[0]) <= 2e-5 * theirs[0] and abs(acc[5] - theirs[1]) <= 2e-5 * abs(theirs[1]), (acc[4:6], theirs)


def full_size_case(cfg):
    """One view of benchmark configuration cfg at its full size: scene, camera, packed target (a render of the
    seed-distinct ground-truth set, quantised), loss parameters."""
    import torch
    from b2ctrain_b200.trainer import render_targets
    cam = scenes.config_cameras(cfg)[0]
    scene = scenes.config_scene(cfg)
    targets, _ = render_targets(scenes.config_scene(cfg, gt_set=True), [cam], "cuda:0", noise_sigma=0.05 if cfg == 1 else 0.0, seed=99)
    gt = targets[0].numpy().view(np.uint32).copy()
    lp = dict(l1_w=0.8, ssim_w=-0.2)
    if cfg == 4:   # binary ellipse mask in the alpha byte, masked loss + alpha lane, scale 1 / coverage
        mask = scenes.ellipse_mask(cam["W"], cam["H"], 0.4)
        gt = np.where(mask > 0, (gt & np.uint32(0x00FFFFFF)) | np.uint32(0xFF000000), np.uint32(0)).astype(np.uint32)
        lp.update(mask=1, alpha_lane=1, scale=1.0 / 0.4, match_alpha_weight=0.1)
    torch.cuda.empty_cache()
    return scene, cam, gt, lp


@pytest.mark.parametrize("cfg", [1, 2, 4])
def test_full_size_view_chunked_equals_whole_and_matches_reference_kernels(cfg):
    """Benchmark configurations 1, 2 and 4 at full size, one view: (i) the chunked renderer (4 depth chunks, what the
    benchmark runs) against the whole-view binning: image, transmittance and depth bit-identical, per-splat gradient
    lanes equal to summation order; (ii) the product against the reference's CUDA kernels: image, loss, grad_out."""
    import torch
    from b2ctrain_b200 import api
    scene, cam, gt, lp = full_size_case(cfg)
    n, W, H = scene["n"], cam["W"], cam["H"]
    h = Harness(scene, cam, gt, None, lp, want_depth=True, isect_cap=1 << 24)
    loss, grad = h.analytic()
    whole = dict(rgba=h.ctx.out_rgba.clone(), T=h.ctx.out_feat[:, 3].clone(), depth=h.ctx.out_depth.clone())
    # (i) chunked vs whole
    ctx = api.RenderCtx("cuda:0"); ctx.want_depth = True
    ctx.setup(W, H, h.model.cap, isect_cap=1 << 24, n_chunks=4)
    api.render_forward(ctx, h.model, h.rp, sync=True)
    assert torch.equal(ctx.out_rgba, whole["rgba"]) and torch.equal(ctx.out_feat[:, 3], whole["T"]) and torch.equal(ctx.out_depth, whole["depth"])
    api.zero_loss(ctx)
    api.photometric_loss(ctx, h.view, h.lp)
    api.rasterize_backward(ctx, h.model, h.rp)
    h.forward(); api.zero_loss(h.ctx); api.photometric_loss(h.ctx, h.view, h.lp); api.rasterize_backward(h.ctx, h.model, h.rp)
    v_whole, v_chunk = h.ctx.v_splat[:n].cpu().numpy(), ctx.v_splat[:n].cpu().numpy()
    assert torch.equal(h.ctx.vis_flag[:n], ctx.vis_flag[:n])
    # Same fragments, same per-pixel arithmetic; the two forms cut a tile's list into replay segments at different places
    # (every 128 fragments, and additionally where a depth chunk hands over), and a segment's colour-behind term starts from
    # final sum - checkpoint, so the sums differ in rounding. Observed 4e-6 .. 1.2e-5 over configs 1, 2, 4 and runs.
    assert rel_l2(v_chunk, v_whole) <= 2e-5, rel_l2(v_chunk, v_whole)
    assert ctx.num_isect < h.ctx.num_isect
    del ctx
    img = whole["rgba"].cpu().numpy()
    del whole
    torch.cuda.empty_cache()
    # (ii) the reference's kernels on the same inputs
    ref = orc.RefCuda(scene, cam)
    ref.set_view(gt)
    ref.forward()
    ref_loss = ref.loss(lp)
    ref_img = ref.download("out_rgba", (W * H, 4), np.float32)
    ref.backward(tensor_core=False)
    ref_grad = ref.grads()
    ref.close()
    d = np.abs(img - ref_img)
    err_img, err_mean, off = float(d.max()), float(d.mean()), float(np.mean(d.max(1) > TOL_FULL_IMAGE))
    err_loss, err_grad = abs(loss - ref_loss) / abs(ref_loss), rel_l2(grad, ref_grad)
    print(f"config {cfg}: image max abs {err_img:.2e}, mean abs {err_mean:.2e}, pixels off by more than {TOL_FULL_IMAGE:g}: {off:.2e} of the image; "
          f"loss rel {err_loss:.2e}, grad_out rel L2 {err_grad:.2e}")
    # A pixel differs by more than rounding only where a discrete decision fell the other way under the reference's
    # fast-math (a fragment at the 1/255 alpha cut or the transmittance stop): such a pixel moves by at most one
    # fragment's contribution, and there are a handful of them among millions.
    assert err_img <= TOL_FULL_IMAGE_ONE_FRAGMENT and off <= TOL_FULL_IMAGE_OFF and err_mean <= 1e-6
    assert err_loss <= TOL_FULL_LOSS and err_grad <= TOL_FULL_GRAD


def test_loss_value_and_gradient_image_match_reference_kernel_in_the_masked_alpha_combination():
    """The loss combination of benchmark configuration 4 (mask + alpha lane + scale 1 / 0.4 on a binary alpha) on a
    random prediction: value and gradient image against the reference's photometric_kernel."""
    W, H = 83, 61
    rng = np.random.Generator(np.random.PCG64(4))
    scene = scenes.make_splats(16, 0, 3)
    cam = scenes.look_at_camera(scenes.orbit_eye(3.0, 25.0, 10.0), W, H, float(H))
    gt = rng.integers(0, 2 ** 24, W * H, dtype=np.uint64).astype(np.uint32) | (scenes.ellipse_mask(W, H, 0.4) << np.uint32(24)).astype(np.uint32)
    gt[(gt >> 24) == 0] = 0
    pred = rng.random((W * H, 4)).astype(np.float32)
    lp = dict(l1_w=0.8, ssim_w=-0.2, mask=1, alpha_lane=1, scale=2.5, match_alpha_weight=0.1)
    h = Harness(scene, cam, gt, None, lp)
    h.ctx.out_rgba.copy_(h.torch.from_numpy(pred))
    h.api.zero_loss(h.ctx)
    h.api.photometric_loss(h.ctx, h.view, h.lp)
    ref = orc.RefCuda(scene, cam)
    ref.set_view(gt); ref.set_image(pred)
    want = ref.loss(lp)
    v_ref = ref.v_out()
    ref.close()
    got = float(h.ctx.loss_accum[0])
    assert abs(got - want) <= 2e-5 * abs(want), (got, want)
    v = h.ctx.v_out.cpu().numpy()
    assert rel_l2(v, v_ref) <= 2e-4 and np.max(np.abs(v - v_ref)) <= 2e-3 * np.max(np.abs(v_ref))


@pytest.mark.parametrize("masked", [False, True])
def test_evidence_and_label_vote_match_the_reference_kernels(masked):
    """compute_evidence over three views (src/train/evidence.cu:48-196): per-splat in-mask weight, total weight, error,
    effective view count and direction, and the winning class with its share, against the reference's kernels."""
    import torch
    from b2ctrain_b200 import api
    from b2ctrain_b200.evidence import Evidence
    W, H = 160, 120
    scene = scenes.make_splats(5000, 2, 61, log_scale=(-3.0, 0.5))
    cams = [scenes.look_at_camera(scenes.orbit_eye(3.0, a, 10.0), W, H, 120.0) for a in (0.0, 50.0, 140.0)]
    scene = scenes.floor_for_cameras(scene, cams)
    rng = np.random.Generator(np.random.PCG64(9))
    gt = rng.integers(0, 2 ** 32, W * H, dtype=np.uint64).astype(np.uint32)
    wts = rng.integers(0, 256, W * H).astype(np.uint8)
    labels = (np.arange(W * H) // (W * 8) % 7).astype(np.uint8)        # bands of classes; one band beyond the bin count
    labels[: W * 4] = 40
    ref = orc.RefCuda(scene, cams[0])
    ref.set_view(gt, wts)
    want_ev, want_lab = ref.evidence(cams, labels, masked=masked, has_alpha=True)
    ref.close()
    m = api.Model("cuda:0").upload(scene)
    ctx = api.RenderCtx("cuda:0"); ctx.setup(W, H, m.cap)
    view = api.ViewGPU(torch.from_numpy(gt.view(np.int32)).cuda(), torch.from_numpy(wts).cuda(), W, H)
    ev = Evidence(m)
    lab_t = torch.from_numpy(labels).cuda()
    for cam in cams:
        ev.add_view(ctx, cam, view, masked=masked, has_alpha=True, labels=lab_t)
    got_ev, got_lab = ev.download_evidence(), ev.download_labels()
    assert np.abs(want_ev[:, 1]).max() > 1.0
    for k, name in enumerate(("w_in", "w_all", "err")):
        assert rel_l2(got_ev[:, k], want_ev[:, k]) <= 2e-5, name
    assert rel_l2(got_ev[:, 4:7], want_ev[:, 4:7]) <= 2e-5
    seen = want_ev[:, 0] > 1e-3                                          # the ratio of two tiny sums is ill-conditioned
    assert np.max(np.abs(got_ev[seen, 3] - want_ev[seen, 3])) <= 1e-3 and np.all(got_ev[:, 3] <= 3.0 + 1e-4)
    sure = want_lab[:, 1] > 0.55                                         # a clear winner: the class must agree
    assert sure.sum() > 500 and np.array_equal(got_lab[sure, 0], want_lab[sure, 0])
    assert np.max(np.abs(got_lab[sure, 1] - want_lab[sure, 1])) <= 1e-4
    assert np.array_equal(got_lab[:, 1] > 0, want_lab[:, 1] > 0)


@pytest.mark.parametrize("case", ["grow", "relocate_and_cull", "no_new"])
def test_refinement_pass_matches_the_reference(case):
    """RefineState::run (src/gpu/refine.cu:244-342) of the C++ host against the reference's, from the same model,
    statistics, cameras and seeds: the same counts, the same parents chosen in the same order, the same refined splats."""
    from b2ctrain_b200 import host_trainer as ht
    n, deg = 20000, 2
    scene = scenes.make_splats(n, deg, 71, log_scale=(-3.5, 0.6))
    cams = [scenes.look_at_camera(scenes.orbit_eye(3.0, a, 10.0), 64, 64, 64.0) for a in (0.0, 120.0, 240.0)]
    scene = scenes.floor_for_cameras(scene, cams)
    rng = np.random.Generator(np.random.PCG64(3))
    dead = rng.random(n) < (0.001 if case == "grow" else 0.08)
    scene["pos_op"][dead, 3] = -9.0                                     # transparent: pruned
    scene["pos_op"][5, 0] = np.nan; scene["lscale"][7, 1] = 12.0        # non-finite, absurdly large
    stats = np.stack([np.abs(rng.normal(0.002, 0.002, n)), np.abs(rng.normal(0.2, 0.2, n)), (rng.random(n) < 0.8) * rng.integers(1, 9, n), rng.random(n) * 5.0]).astype(np.float32)
    kw = dict(iter=3000, total=30000, seed=11, cull_weight=0.3 if case == "relocate_and_cull" else 0.0, no_new=case == "no_new",
              max_splats=n + 2500 if case == "grow" else 10_000_000)
    cam_pos, cam_focal = np.stack([c["pos"] for c in cams]).astype(np.float32), np.full(3, 64.0, np.float32)
    ref = orc.RefCuda(scene, cams[0])
    want_counts = ref.refine(stats, cam_pos, cam_focal, **kw)
    want = ref.model_state()
    ref.close()
    got, counts, pairs = ht.refine_once(scene, stats, cam_pos, cam_focal, **kw)
    print(case, counts)
    assert counts == want_counts
    if case == "no_new":
        assert counts["relocated"] == counts["grown"] == counts["split_oversized"] == 0 and counts["n"] == n and counts["pruned"] > 1000
    elif case == "grow":
        assert counts["grown"] > 100 and counts["split_oversized"] > 100 and counts["n"] > n
    else:
        assert counts["relocated"] > 1000 and counts["culled"] > 1000
    assert pairs.shape[1] == counts["relocated"] + counts["grown"] + counts["split_oversized"]
    fin = np.isfinite(want["pos_op"]).all(1) & np.isfinite(got["pos_op"]).all(1)
    assert fin.mean() > 0.999
    for k in ("pos_op", "quat", "lscale", "sh"):
        a, b = got[k][fin].reshape(fin.sum(), -1), want[k][fin].reshape(fin.sum(), -1)
        close = (np.abs(a - b) <= 2e-4 * (np.abs(b) + 1e-2)).all(1)
        assert close.mean() >= 0.999, (k, close.mean())                # a draw decided in the last bits of a key may swap two parents
