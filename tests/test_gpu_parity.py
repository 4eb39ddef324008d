"""GPU parity tests: every CUDA stage, called through the C ABI, against the CPU oracle on the same seeded inputs,
and the whole chain against the golden outputs of the reference's own CPU check."""
import numpy as np
import pytest

from b2ctrain_b200 import scenes
from oracle import orc
from tests.util import (TOL_ADAM_REL, TOL_GRAD_REL_L2, TOL_IMAGE_ABS, TOL_LOSS_REL, TOL_RECORD_REL, Harness, check_against_fd,
                        load_gradcheck, rel_l2)

pytestmark = pytest.mark.gpu


def small_scene(n=4000, degree=3, seed=21, W=160, H=120, floor=True):
    scene = scenes.make_splats(n, degree, seed, log_scale=(-3.2, 0.5))
    cam = scenes.look_at_camera(scenes.orbit_eye(3.0, 25.0, 10.0), W, H, float(H))
    if floor:
        scene = scenes.floor_for_cameras(scene, [cam])
    return scene, cam


def gpu_records(h):
    n = h.model.n
    return h.ctx.proj0[:n].cpu().numpy(), h.ctx.proj1[:n].cpu().numpy(), h.ctx.proj2[:n].cpu().numpy(), h.u32(h.ctx.tile_count, n)


@pytest.mark.parametrize("degree", [0, 1, 2, 3, 4])
def test_projection_records(degree):
    scene, cam = small_scene(degree=degree)
    h = Harness(scene, cam)
    h.api.project_splats(h.ctx, h.model, h.rp)
    p0, p1, p2, tc = gpu_records(h)
    rec = orc.project(scene, cam)
    ok_o = rec[:, orc.OK] != 0
    ok_g = p1[:, 3] > -0.5
    # Cull decisions may only differ where the oracle itself sits on a threshold.
    differ = np.nonzero(ok_o != ok_g)[0]
    assert len(differ) <= 2 and all(abs(rec[i, orc.OPAC] - 1 / 255) < 1e-6 or not ok_o[i] for i in differ)
    both = ok_o & ok_g
    assert both.sum() > 0.5 * scene["n"]
    want = np.concatenate([rec[both][:, [orc.MX, orc.MY, orc.C00, orc.C01]], rec[both][:, [orc.C11, orc.OPAC, orc.Z, orc.POWER]]], 1)
    got = np.concatenate([p0[both], p1[both]], 1).astype(np.float64)
    # Conic entries lose relative precision with the conditioning of the 2x2 inverse: scale their tolerance by the
    # largest conic entry of the splat.
    cmax = np.abs(want[:, [2, 3, 4]]).max(1, keepdims=True)
    scale = np.abs(want) + np.array([1.0, 1.0, 0, 0, 0, 0, 0, 1.0])[None, :]
    scale[:, [2, 3, 4]] = cmax
    assert np.max(np.abs(got - want) / scale) <= TOL_RECORD_REL
    vis = both & (tc > 0)
    assert np.max(np.abs(p2[vis][:, :3] - rec[vis][:, orc.R:orc.B + 1])) <= 5e-6


def test_binning_bit_exact():
    """Tile sets, tile counts, sorted fragment order and tile ranges are bit-exact functions of the fp32 records."""
    scene, cam = small_scene(n=6000)
    h = Harness(scene, cam)
    h.api.project_splats(h.ctx, h.model, h.rp)
    h.api.bin_and_sort(h.ctx, h.model)
    p0, p1, _, tc = gpu_records(h)
    tc_o, vals_o, keys_o, ranges_o = orc.bin_sort(p0, p1, cam["W"], cam["H"])
    assert np.array_equal(tc, tc_o)
    assert h.ctx.num_isect == len(vals_o) and len(vals_o) > 10000
    assert np.array_equal(h.u32(h.ctx.vals_sorted, len(vals_o)), vals_o)
    assert np.array_equal(h.u32(h.ctx.keys_sorted, len(vals_o)), keys_o)
    assert np.array_equal(h.u32(h.ctx.tile_ranges).reshape(-1, 2), ranges_o)
    order = h.u32(h.ctx.order, scene["n"])
    zb = np.where(tc > 0, p1[:, 2].view(np.uint32), 0xFFFFFFFF).astype(np.uint64)
    want_order = np.argsort(zb * np.uint64(1 << 32) + np.arange(scene["n"], dtype=np.uint64), kind="stable")
    assert np.array_equal(order, want_order.astype(np.uint32))


def test_binning_bit_exact_at_4k_where_the_tile_sort_uses_nine_bit_digits():
    """A 3840x2160 image has 129,600 tiles, 17 bits of tile id: the tile sort runs two passes of nine-bit digits instead of
    three of eight. Same contract as above, plus the chunked renderer on the same view."""
    import torch
    scene, cam = small_scene(n=1200, W=3840, H=2160)
    h = Harness(scene, cam)
    assert h.ctx.tile_bits == 17 and h.api.lib().b2k_sort_passes(17) == 2 and h.api.lib().b2k_sort_passes(15) == 2 and h.api.lib().b2k_sort_passes(32) == 4
    h.api.project_splats(h.ctx, h.model, h.rp)
    h.api.bin_and_sort(h.ctx, h.model)
    p0, p1, _, tc = gpu_records(h)
    tc_o, vals_o, keys_o, ranges_o = orc.bin_sort(p0, p1, cam["W"], cam["H"])
    assert np.array_equal(tc, tc_o)
    assert h.ctx.num_isect == len(vals_o) and len(vals_o) > 200000 and int(keys_o.max()) >= 1 << 16
    assert np.array_equal(h.u32(h.ctx.vals_sorted, len(vals_o)), vals_o)
    assert np.array_equal(h.u32(h.ctx.keys_sorted, len(vals_o)), keys_o)
    assert np.array_equal(h.u32(h.ctx.tile_ranges).reshape(-1, 2), ranges_o)
    h.api.rasterize_forward(h.ctx, h.rp)
    chunked = h.api.RenderCtx("cuda:0"); chunked.setup(cam["W"], cam["H"], h.model.cap, n_chunks=3)
    h.api.render_forward(chunked, h.model, h.rp, sync=True)
    assert torch.equal(chunked.out_rgba, h.ctx.out_rgba)


def test_binning_depth_ties_and_big_splats():
    scene, cam = small_scene(n=3000, degree=0)
    scene["lscale"][:40, :3] = -1.0                       # splats spanning hundreds of tiles
    scene["pos_op"][100:200, :3] = scene["pos_op"][100, :3]   # identical depth: the index breaks the tie
    h = Harness(scene, cam)
    h.api.project_splats(h.ctx, h.model, h.rp)
    h.api.bin_and_sort(h.ctx, h.model)
    p0, p1, _, tc = gpu_records(h)
    tc_o, vals_o, keys_o, ranges_o = orc.bin_sort(p0, p1, cam["W"], cam["H"])
    assert tc.max() > 100
    assert np.array_equal(tc, tc_o)
    assert np.array_equal(h.u32(h.ctx.vals_sorted, len(vals_o)), vals_o)
    assert np.array_equal(h.u32(h.ctx.tile_ranges).reshape(-1, 2), ranges_o)


def test_binning_overflow_grows_and_matches():
    scene, cam = small_scene(n=6000)
    h = Harness(scene, cam, isect_cap=1024)   # far too small: the wrapper must grow it like binning.cu:129-133
    h.forward()
    p0, p1, _, tc = gpu_records(h)
    _, vals_o, _, _ = orc.bin_sort(p0, p1, cam["W"], cam["H"])
    assert h.ctx.isect_cap >= len(vals_o) > 1024
    assert np.array_equal(h.u32(h.ctx.vals_sorted, len(vals_o)), vals_o)


def oracle_forward_from_gpu_records(h, scene, cam):
    p0, p1, p2, tc = gpu_records(h)
    geo = np.concatenate([p0, p1], 1).astype(np.float64)[:, [0, 1, 2, 3, 4, 5, 6, 7]]
    vals = h.u32(h.ctx.vals_sorted, h.ctx.num_isect)
    return geo, p2[:, :3].astype(np.float64), vals


def test_forward_image_stagewise():
    scene, cam = small_scene()
    bg = (0.2, 0.1, 0.3)
    h = Harness(scene, cam, bg=bg, want_depth=True)
    h.api.project_splats(h.ctx, h.model, h.rp)
    h.api.bin_and_sort(h.ctx, h.model)
    ranges_before = h.u32(h.ctx.tile_ranges).reshape(-1, 2).copy()
    h.api.rasterize_forward(h.ctx, h.rp)
    geo, col, vals = oracle_forward_from_gpu_records(h, scene, cam)
    rgba, T, last, ranges, depth = orc.raster_fwd(cam["W"], cam["H"], geo, col, vals, ranges_before, np.array(bg), True, want_depth=True)
    got = h.ctx.out_rgba.cpu().numpy()
    assert np.max(np.abs(got - rgba)) <= TOL_IMAGE_ABS
    assert np.max(np.abs(h.ctx.out_feat.cpu().numpy()[:, 3] - T)) <= TOL_IMAGE_ABS
    # last_idx / shrunk ranges are discrete: they may differ only at pixels sitting on a cut-off.
    last_g = h.u32(h.ctx.last_idx)
    assert np.mean(last_g != last) < 2e-3
    assert np.mean(h.u32(h.ctx.tile_ranges).reshape(-1, 2)[:, 1] != ranges[:, 1]) < 1e-2
    alpha = rgba[:, 3]
    want_depth = np.where(alpha > 0.05, depth / np.maximum(alpha, 1e-30), np.inf)
    got_depth = h.ctx.out_depth.cpu().numpy()
    sure = np.abs(alpha - 0.05) > 1e-3
    fin = sure & np.isfinite(want_depth)
    assert np.array_equal(np.isfinite(got_depth[sure]), np.isfinite(want_depth[sure]))
    assert np.max(np.abs(got_depth[fin] - want_depth[fin])) <= 2e-3


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
def test_loss_kernel_stagewise(mode):
    """The fused loss kernel on a random prediction, value and gradient, against the oracle in double. Modes 0-2 are
    the reference's gradient-check combinations (tests/tests.cpp:398-441); mode 3 is benchmark configuration 4's:
    mask and alpha lane together on a binary alpha, scale 1 / 0.4."""
    rng = np.random.Generator(np.random.PCG64(40 + mode))
    W, H = 83, 61                                          # ragged: not a multiple of the 16-pixel tile
    scene, cam = small_scene(n=16, W=W, H=H)
    gt = rng.integers(0, 2 ** 32, W * H, dtype=np.uint64).astype(np.uint32)
    wts = rng.integers(64, 256, W * H).astype(np.uint8) if mode in (0, 1) else None
    lp = dict(l1_w=0.8, ssim_w=-0.2, bg=(0.2, 0.1, 0.3), composite=mode == 0, mask=mode in (1, 3), alpha_lane=mode in (0, 3),
              match_alpha_weight=0.3, scale={1: 1.7, 3: 2.5}.get(mode, 1.0), grad_scale=1.0)
    if mode == 3:
        gt = (gt & np.uint32(0x00FFFFFF)) | (scenes.ellipse_mask(W, H, 0.4) << np.uint32(24)).astype(np.uint32)
        gt[(gt >> np.uint32(24)) == 0] = 0
        lp["bg"] = (0.0, 0.0, 0.0)
    h = Harness(scene, cam, gt, wts, lp)
    pred = rng.random((W * H, 4)).astype(np.float32)
    pred[: W * 20] = 0.0                                   # a flat region
    gt[: W * 20] = 0xFF000000 if mode in (1, 2) else 0     # equal to the prediction there (mode 3: alpha 0 too, as outside its ellipse)
    h = Harness(scene, cam, gt, wts, lp)
    h.ctx.out_rgba.copy_(h.torch.from_numpy(pred))
    h.ctx.loss_accum.zero_()
    h.api.photometric_loss(h.ctx, h.view, h.lp)
    f32 = {k: (np.float32(v) if isinstance(v, float) else v) for k, v in lp.items()}
    f32["bg"] = tuple(np.float32(x) for x in lp["bg"])
    want, v_out = orc.loss(W, H, pred, gt, wts, f32)
    got = float(h.ctx.loss_accum[0].item())
    assert abs(got - want) <= 2e-5 * abs(want)
    v = h.ctx.v_out.cpu().numpy()
    assert rel_l2(v, v_out) <= 2e-4
    assert np.max(np.abs(v - v_out)) <= 2e-3 * np.max(np.abs(v_out))


def test_backward_stagewise():
    """Reverse replay on the GPU's own forward state against the oracle's replay of the same state."""
    scene, cam = small_scene()
    rng = np.random.Generator(np.random.PCG64(9))
    bg = (0.2, 0.1, 0.3)
    h = Harness(scene, cam, bg=bg)
    h.forward()
    P = cam["W"] * cam["H"]
    v_out = (rng.standard_normal((P, 4)) * 1e-3).astype(np.float32)
    h.ctx.v_out.copy_(h.torch.from_numpy(v_out))
    h.api.rasterize_backward(h.ctx, h.model, h.rp)
    geo, col, vals = oracle_forward_from_gpu_records(h, scene, cam)
    ranges = h.u32(h.ctx.tile_ranges).reshape(-1, 2)
    want, vis, visw = orc.raster_bwd(scene["n"], cam["W"], cam["H"], geo, col, vals, ranges, np.array(bg), h.ctx.out_rgba.cpu().numpy(),
                                     h.ctx.out_feat.cpu().numpy()[:, 3], h.u32(h.ctx.last_idx), v_out)
    got = h.ctx.v_splat[: scene["n"]].cpu().numpy()
    assert np.array_equal(h.u32(h.ctx.vis_flag, scene["n"]) != 0, vis != 0)
    for lane in range(10):
        assert rel_l2(got[:, lane], want[:, lane]) <= 5e-5, lane
    assert np.all(got[:, 10:] == 0)
    assert rel_l2(h.model.vis_weight[: scene["n"]].cpu().numpy(), visw) <= 1e-5


@pytest.mark.parametrize("degree", [1, 3, 4])
def test_projection_backward_stagewise(degree):
    scene, cam = small_scene(n=3000, degree=degree)
    rng = np.random.Generator(np.random.PCG64(12))
    h = Harness(scene, cam)
    h.api.project_splats(h.ctx, h.model, h.rp)
    n = scene["n"]
    tc = h.u32(h.ctx.tile_count, n)
    v_splat = rng.standard_normal((n, 13)).astype(np.float32)
    v_splat[:, 10:] = 0
    vis = (rng.random(n) < 0.7).astype(np.uint32)
    h.ctx.v_splat[:n].copy_(h.torch.from_numpy(v_splat))
    h.ctx.vis_flag[:n].copy_(h.torch.from_numpy(vis.view(np.int32)))
    K = (degree + 1) ** 2
    grads = h.torch.zeros((n, 11 + 3 * K), dtype=h.torch.float32, device="cuda:0")
    h.api.optimizer_step(h.ctx, h.model, h.api.OptimParams(cam, active_sh_degree=degree, grad_out=grads))
    want = orc.proj_bwd(scene, cam, v_splat, vis, tc)
    got = grads.cpu().numpy()
    for lo, hi in ((0, 3), (3, 4), (4, 8), (8, 11), (11, 11 + 3 * K)):
        assert rel_l2(got[:, lo:hi], want[:, lo:hi]) <= 2e-5, (lo, hi)
    # the optimizer consumed and cleared the lanes
    assert float(h.ctx.v_splat[:n][h.torch.from_numpy(vis != 0).cuda()].abs().max()) == 0.0
    assert int(h.ctx.vis_flag[:n].abs().max()) == 0


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_full_chain_against_reference_golden(mode):
    """Forward + loss + backward + projection backward on the reference's gradient-check scenes: loss within
    tolerance of `reference_loss`, gradients within the reference's finite-difference rule and within 1e-4 relative
    L2 of the analytic double oracle."""
    scene, cam, gt, wts, lp, z = load_gradcheck(mode)
    h = Harness(scene, cam, gt, wts, lp)
    loss, grad = h.analytic()
    assert abs(loss - float(z["ref_loss"])) <= TOL_LOSS_REL * abs(float(z["ref_loss"]))
    fails, total, fails_1e4 = check_against_fd(grad, z)
    assert fails == 0 and fails_1e4 <= 0.05 * total
    want = orc.step(scene, cam, np.array(lp["bg"], np.float64), gt, wts, lp, backward=True)["grad"]
    assert rel_l2(grad, want) <= TOL_GRAD_REL_L2


def test_config0_full_chain():
    """BASELINE config 0: 2,000 splats, SH degree 1, 64x64, target = perturbed scene rendered."""
    z = np.load("tests/golden/config0.npz")
    scene = scenes.make_splats(2000, 1, 1000)
    cam = scenes.config_cameras(0)[0]
    lp = dict(l1_w=np.float32(0.8), ssim_w=np.float32(-0.2))
    h = Harness(scene, cam, z["gt"], None, lp)
    loss, grad = h.analytic()
    assert abs(loss - float(z["ref_loss"])) <= TOL_LOSS_REL * abs(float(z["ref_loss"]))
    out = orc.step(scene, cam, np.zeros(3), z["gt"], None, lp, backward=True, want_image=True)
    assert np.max(np.abs(h.ctx.out_rgba.cpu().numpy() - out["rgba"])) <= TOL_IMAGE_ABS
    assert rel_l2(grad, out["grad"]) <= TOL_GRAD_REL_L2


def test_adam_fused_and_split_match_oracle():
    scene, cam = small_scene(n=3000, degree=2)
    rng = np.random.Generator(np.random.PCG64(31))
    n, K = scene["n"], 9
    for split in (False, True):
        h = Harness(scene, cam)
        h.api.project_splats(h.ctx, h.model, h.rp)
        tc = h.u32(h.ctx.tile_count, n)
        state = None
        for t in (1, 2, 5):   # t = 5 after 2 exercises the lazy catch-up of splats that skipped steps
            v_splat = (rng.standard_normal((n, 13)) * 1e-2).astype(np.float32); v_splat[:, 10:] = 0
            vis = (rng.random(n) < 0.6).astype(np.uint32)
            h.ctx.v_splat[:n].copy_(h.torch.from_numpy(v_splat))
            h.ctx.vis_flag[:n].copy_(h.torch.from_numpy(vis.view(np.int32)))
            cur = h.model.download()
            if state is None:
                z4 = lambda: np.zeros((n, 4), np.float32)
                state = dict(m_pos=z4(), v_pos=z4(), m_q=z4(), v_q=z4(), m_ls=z4(), v_ls=z4(), m_sh=np.zeros((n, K, 3), np.float32),
                             v_sh=np.zeros(n, np.float32), last_step=np.zeros(n, np.uint32))
            state.update(pos_op=cur["pos_op"].copy(), quat=cur["quat"].copy(), lscale=cur["lscale"].copy(), sh=cur["sh"].copy())
            grad = orc.proj_bwd(cur, cam, v_splat, vis, tc)
            active = np.any(grad != 0, axis=1)
            opd = dict(t=t, lr_mean=1.6e-4, sparse=1)
            orc.adam(state, grad, active, opd, 2)
            op = h.api.OptimParams(cam, active_sh_degree=2, t=t, lr_mean=1.6e-4, sparse=True)
            if split:
                g = h.torch.zeros((n, 11 + 3 * K), dtype=h.torch.float32, device="cuda:0")
                op.touched_out = h.torch.zeros(((n + 31) // 32,), dtype=h.torch.int32, device="cuda:0")
                h.api.projection_backward(h.ctx, h.model, op, g)
                # the bitmap the sharded data-parallel update reads: every row that holds something is marked, nothing else
                # but splats whose gradient came out as exact zeros
                rows = (g != 0).any(dim=1).cpu().numpy()
                bits = np.unpackbits(op.touched_out.cpu().numpy().view(np.uint8), bitorder="little")[:n].astype(bool)
                assert np.all(bits[rows]) and bits.sum() <= rows.sum() + 8 and bits.sum() > 0
                h.api.adam_step(h.model, op, g)
                assert float(g.abs().max()) == 0.0
            else:
                h.api.optimizer_step(h.ctx, h.model, op)
            got = h.model.download()
            # fp32 bias corrections 1 - beta^t cancel (1 - 0.999^5 keeps ~1e-5 relative precision), and the catch-up
            # multiplies that into a several-step drift: parameters are held to 2e-5 on plain steps, 1e-4 after a gap.
            tol = 2e-5 if t <= 2 else 1e-4
            for k in ("pos_op", "quat", "lscale", "sh"):
                assert np.max(np.abs(got[k] - state[k]) / (np.abs(state[k]) + 1e-3)) <= tol, (split, t, k)
            assert rel_l2(h.model.m_pos_op[:n].cpu().numpy(), state["m_pos"]) <= TOL_ADAM_REL
            assert rel_l2(h.model.v_quat[:n].cpu().numpy(), state["v_q"]) <= TOL_ADAM_REL
            assert rel_l2(h.model.v_sh[:n].cpu().numpy(), state["v_sh"]) <= TOL_ADAM_REL
            assert rel_l2(h.model.sh_planar_to_host(h.model.m_sh_dc, h.model.m_sh_hi), state["m_sh"]) <= TOL_ADAM_REL
            assert np.array_equal(h.u32(h.model.last_step, n), state["last_step"])
            # keep the two sides in lock step: the next step starts from the GPU's parameters on both
            state.update(m_pos=h.model.m_pos_op[:n].cpu().numpy().copy(), v_pos=h.model.v_pos_op[:n].cpu().numpy().copy(),
                         m_q=h.model.m_quat[:n].cpu().numpy().copy(), v_q=h.model.v_quat[:n].cpu().numpy().copy(),
                         m_ls=h.model.m_lscale[:n].cpu().numpy().copy(), v_ls=h.model.v_lscale[:n].cpu().numpy().copy(),
                         m_sh=h.model.sh_planar_to_host(h.model.m_sh_dc, h.model.m_sh_hi).copy(), v_sh=h.model.v_sh[:n].cpu().numpy().copy())


def test_empty_scene_and_all_culled():
    cam = scenes.look_at_camera((0.0, 0.0, 3.0), 40, 24, 40.0)
    scene = scenes.make_splats(16, 0, 3)
    scene["pos_op"][:, 2] += 10.0
    h = Harness(scene, cam, bg=(0.1, 0.2, 0.3))
    h.forward()
    assert h.ctx.num_isect == 0
    img = h.ctx.out_rgba.cpu().numpy()
    assert np.allclose(img[:, :3], [0.1, 0.2, 0.3]) and np.all(img[:, 3] == 0)


def test_determinism_of_integer_outputs():
    scene, cam = small_scene(n=5000)
    outs = []
    for _ in range(2):
        h = Harness(scene, cam)
        h.forward()
        outs.append((h.u32(h.ctx.vals_sorted, h.ctx.num_isect).copy(), h.u32(h.ctx.tile_ranges).copy(), h.u32(h.ctx.last_idx).copy(),
                     h.ctx.out_rgba.cpu().numpy().copy()))
    for a, b in zip(outs[0], outs[1]):
        assert np.array_equal(a, b)


def test_min_scale_and_pack():
    scene, cam = small_scene(n=500, floor=False)
    h = Harness(scene, cam)
    cams = [scenes.look_at_camera(scenes.orbit_eye(4, a, 10), 64, 64, 64.0) for a in (0, 90, 200)]
    cp = h.torch.tensor(np.stack([c["pos"] for c in cams]), dtype=h.torch.float32, device="cuda:0")
    cf = h.torch.tensor([64.0] * 3, dtype=h.torch.float32, device="cuda:0")
    h.api.update_min_scale(h.model, cp, cf)
    want = orc.min_scale(scene["pos_op"], scene["lscale"], cp.cpu().numpy(), cf.cpu().numpy())[:, 3]
    assert np.allclose(h.model.lscale[:500, 3].cpu().numpy(), want, rtol=1e-5)
    img = np.random.Generator(np.random.PCG64(1)).random((1000, 4)).astype(np.float32)
    out = h.torch.zeros(1000, dtype=h.torch.int32, device="cuda:0")
    h.api.pack_rgba8(h.torch.from_numpy(img).cuda(), out)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), scenes.pack_rgba8(img))


def test_multi_view_accumulation_equals_sum_of_view_gradients():
    """Data-parallel semantics: the accumulator after several views == the sum of the per-view grad_out gradients, and
    the split Adam consumes (and clears) it."""
    from b2ctrain_b200.trainer import Trainer
    scene, cam0 = small_scene(n=3000, degree=2)
    cams = [scenes.look_at_camera(scenes.orbit_eye(3.0, a, 10.0), 160, 120, 120.0) for a in (10.0, 60.0, 130.0)]
    rng = np.random.Generator(np.random.PCG64(77))
    gts = [rng.integers(0, 2 ** 32, 160 * 120, dtype=np.uint64).astype(np.uint32) | np.uint32(0xFF000000) for _ in cams]
    lp = dict(l1_w=0.8, ssim_w=-0.2)
    total = 0
    for cam, gt in zip(cams, gts):
        _, g = Harness(scene, cam, gt, None, lp).analytic()
        total = total + g.astype(np.float64)
    import torch
    tr = Trainer(scene, 160, 120, "cuda:0", 0, 1, lr_mean=1e-4, sparse=True)
    targets = [torch.from_numpy(g.view(np.int32)).cuda() for g in gts]
    tr.model.adam_t += 1
    for cam, t in zip(cams, targets):
        tr.view_pass(cam, t)
    got = tr.grad.cpu().numpy()
    assert rel_l2(got, total) <= 1e-5
    before = tr.model.download()
    tr.api = None
    from b2ctrain_b200 import api
    api.adam_step(tr.model, tr._op(cams[0]), tr.grad)
    after = tr.model.download()
    assert float(tr.grad.abs().max()) == 0.0
    moved = np.any(before["pos_op"] != after["pos_op"], axis=1)
    assert np.array_equal(moved, np.any(got[:, :4] != 0, axis=1) | moved) and moved.sum() > 100


def test_full_chain_ragged_image_size():
    """Image sizes that are multiples of neither the 8-pixel raster tile nor the 16-pixel loss tile."""
    scene = scenes.make_splats(1500, 2, 33, log_scale=(-2.8, 0.5))
    cam = scenes.look_at_camera(scenes.orbit_eye(3.0, -40.0, 20.0), 150, 97, 110.0)
    scene = scenes.floor_for_cameras(scene, [cam])
    rng = np.random.Generator(np.random.PCG64(3))
    gt = rng.integers(0, 2 ** 32, 150 * 97, dtype=np.uint64).astype(np.uint32)
    wts = rng.integers(0, 256, 150 * 97).astype(np.uint8)
    lp = dict(l1_w=np.float32(0.8), ssim_w=np.float32(-0.2), bg=(np.float32(0.3), np.float32(0.2), np.float32(0.1)), composite=1, alpha_lane=1,
              match_alpha_weight=np.float32(0.25))
    h = Harness(scene, cam, gt, wts, lp)
    loss, grad = h.analytic()
    want = orc.step(scene, cam, np.array(lp["bg"], np.float64), gt, wts, lp, backward=True, want_image=True)
    assert np.max(np.abs(h.ctx.out_rgba.cpu().numpy() - want["rgba"])) <= TOL_IMAGE_ABS
    assert abs(loss - want["loss"]) <= TOL_LOSS_REL * abs(want["loss"])
    assert rel_l2(grad, want["grad"]) <= TOL_GRAD_REL_L2


def test_full_chain_masked_loss_with_alpha_lane():
    """Benchmark configuration 4's loss combination through the whole chain: binary ellipse alpha, mask and alpha lane
    on, scale 1 / 0.4; image, loss and gradients against the double oracle."""
    scene, cam = small_scene(n=3000, degree=2, seed=44)
    W, H = cam["W"], cam["H"]
    rng = np.random.Generator(np.random.PCG64(14))
    gt = rng.integers(0, 2 ** 24, W * H, dtype=np.uint64).astype(np.uint32) | (scenes.ellipse_mask(W, H, 0.4) << np.uint32(24)).astype(np.uint32)
    gt[(gt >> np.uint32(24)) == 0] = 0
    lp = dict(l1_w=np.float32(0.8), ssim_w=np.float32(-0.2), mask=1, alpha_lane=1, scale=np.float32(2.5), match_alpha_weight=np.float32(0.1))
    h = Harness(scene, cam, gt, None, lp)
    loss, grad = h.analytic()
    want = orc.step(scene, cam, np.zeros(3), gt, None, lp, backward=True, want_image=True)
    assert np.max(np.abs(h.ctx.out_rgba.cpu().numpy() - want["rgba"])) <= TOL_IMAGE_ABS
    assert abs(loss - want["loss"]) <= TOL_LOSS_REL * abs(want["loss"])
    assert rel_l2(grad, want["grad"]) <= TOL_GRAD_REL_L2


def test_adam_by_slices_equals_adam_over_the_whole_model():
    """The sliced update (pipelined with the all-reduce on several GPUs) is bit-identical to the whole-model call."""
    import torch
    from b2ctrain_b200 import api
    from b2ctrain_b200.trainer import slice_bounds
    n, deg = 1000, 3
    scene = scenes.make_splats(n, deg, 77)
    cam = scenes.look_at_camera(scenes.orbit_eye(3.0, 10.0, 10.0), 64, 48, 50.0)
    K = (deg + 1) ** 2
    gen = torch.Generator(device="cuda:0"); gen.manual_seed(5)
    results = []
    for sliced in (False, True):
        m = api.Model("cuda:0").upload(scene)
        for t in (1, 2):
            g = torch.randn((n, 11 + 3 * K), generator=torch.Generator(device="cuda:0").manual_seed(t), device="cuda:0") * 1e-3
            g[::3] = 0   # untouched splats are skipped in sparse mode
            op = api.OptimParams(cam, active_sh_degree=deg, t=t, lr_mean=1e-4, sparse=True, noise_weight=1e-3, noise_clamp=1e-2, step=t)
            if sliced:
                for a, c in slice_bounds(n, 3):
                    api.adam_step(m, op, g, first=a, count=c)
            else:
                api.adam_step(m, op, g)
            assert float(g.abs().max()) == 0.0
        d = m.download()
        results.append((d, m.v_sh[:n].cpu().numpy().copy(), m.last_step[:n].cpu().numpy().copy()))
    for k in ("pos_op", "quat", "lscale", "sh"):
        assert np.array_equal(results[0][0][k], results[1][0][k]), k
    assert np.array_equal(results[0][1], results[1][1]) and np.array_equal(results[0][2], results[1][2])
    assert np.count_nonzero(results[0][2]) == n - len(range(0, n, 3))


@pytest.mark.parametrize("n_chunks", [2, 3, 5])
def test_chunked_front_to_back_render_matches_whole_view_binning(n_chunks):
    """b2k_render_chunked composites the same fragments in the same order as project + bin_sort + raster_fwd, so the
    image, transmittance, depth and (after the loss) the per-splat gradient lanes agree; dense, opaque splats make
    tiles saturate early, so later chunks skip them and fewer intersections are sorted. Big-box splats are present."""
    import torch
    from b2ctrain_b200 import api
    W, H, n = 200, 136, 30000
    scene = scenes.make_splats(n, 2, 91, log_scale=(-3.0, 0.7), opacity=(2.0, 1.0))
    scene["lscale"][::20, :3] = -1.5   # every 20th splat covers more than 64 tiles (the warp-per-splat paths)
    cam = scenes.look_at_camera(scenes.orbit_eye(3.0, 40.0, 15.0), W, H, float(H) * 1.4)
    scene = scenes.floor_for_cameras(scene, [cam])
    rng = np.random.Generator(np.random.PCG64(4))
    gt = torch.from_numpy(rng.integers(0, 2 ** 31, W * H, dtype=np.int64).astype(np.int32)).cuda()
    m = api.Model("cuda:0").upload(scene)
    out = []
    for chunks in (1, n_chunks):
        ctx = api.RenderCtx("cuda:0"); ctx.want_depth = True
        ctx.setup(W, H, m.cap, n_chunks=chunks)
        rp = api.RenderParams(cam, bg=(0.2, 0.1, 0.3), sh_degree=2, bwd_info=True)
        api.render_forward(ctx, m, rp, sync=True)
        used = ctx.num_isect
        api.photometric_loss(ctx, api.ViewGPU(gt, None, W, H), api.LossParams())
        api.rasterize_backward(ctx, m, rp)
        torch.cuda.synchronize()
        big = int((ctx.hit_info[:n].cpu().numpy().view(np.uint32).reshape(-1, 4)[:, 2] == 0xFFFFFFFF).sum())
        out.append(dict(rgba=ctx.out_rgba.cpu().numpy(), T=ctx.out_feat[:, 3].cpu().numpy(), depth=ctx.out_depth.cpu().numpy(),
                        v=ctx.v_splat[:n].cpu().numpy(), vis=ctx.vis_flag[:n].cpu().numpy(), loss=float(ctx.loss_accum[0]), used=used, big=big,
                        ranges=ctx.tile_ranges.cpu().numpy().view(np.uint32).reshape(chunks, -1, 2), last=ctx.last_idx.cpu().numpy().view(np.uint32)))
    a, b = out
    assert a["big"] > 50
    assert np.array_equal(a["rgba"], b["rgba"]) and np.array_equal(a["T"], b["T"]) and np.array_equal(a["depth"], b["depth"])
    assert abs(a["loss"] - b["loss"]) <= 1e-6 * abs(a["loss"])   # the same image; the loss sums its tiles with atomics
    assert np.array_equal(a["vis"], b["vis"])
    assert rel_l2(b["v"], a["v"]) <= 1e-5
    assert b["used"] < 0.7 * a["used"], (a["used"], b["used"])          # saturated tiles stopped emitting
    # the ranges the backward walks are never longer than in the whole-view binning (a chunk's unused tail is dropped)
    walked = int((b["ranges"][:, :, 1].astype(np.int64) - b["ranges"][:, :, 0]).clip(min=0).sum())
    assert 0 < walked <= int((a["ranges"][0, :, 1].astype(np.int64) - a["ranges"][0, :, 0]).sum())


@pytest.mark.parametrize("mode", ["Normals", "Buffer"])
def test_forward_feature_lanes_match_oracle(mode):
    """FeatureMode::Normals / Buffer in the forward (project.cu:62-77, raster_fwd.cu:52,62): out_feat.xyz against the
    oracle's feature compositing (itself pinned on the reference's normal lane), colour image unchanged."""
    import torch
    from b2ctrain_b200 import api
    scene, cam = small_scene(n=3000, degree=2, seed=33)
    n, W, H = scene["n"], cam["W"], cam["H"]
    m = api.Model("cuda:0").upload(scene)
    ctx = api.RenderCtx("cuda:0"); ctx.setup(W, H, m.cap)
    rng = np.random.Generator(np.random.PCG64(8))
    buf = rng.normal(0, 60, (n, 3)).astype(np.float32); buf[5, 1] = np.inf
    rp = api.RenderParams(cam, bg=(0.1, 0.2, 0.3), sh_degree=2, bwd_info=True)
    api.render_forward(ctx, m, rp, sync=True)
    plain = ctx.out_rgba.cpu().numpy().copy()
    assert float(ctx.out_feat[:, :3].abs().max()) == 0.0
    rp.feat = mode
    if mode == "Buffer":
        rp.feat_buffer = torch.from_numpy(buf).cuda()
    api.render_forward(ctx, m, rp, sync=True)
    assert np.array_equal(ctx.out_rgba.cpu().numpy(), plain)
    got = ctx.out_feat[:, :3].cpu().numpy()
    rec = orc.project(scene, cam)
    p0, p1 = orc.records_to_proj(rec)
    tc, vals, keys, ranges = orc.bin_sort(p0, p1, W, H)
    feat = orc.features(scene, cam, 1 if mode == "Normals" else 2, buf)
    want = orc.raster_feat(W, H, np.ascontiguousarray(rec[:, :8]), feat, vals, ranges)
    tol = TOL_IMAGE_ABS * (1.0 if mode == "Normals" else 100.0)   # buffer values reach +-100
    assert np.max(np.abs(got - want)) <= tol
    assert np.abs(want).max() > 0.5
    # the chunked renderer composites the same lanes (forward only: its backward reads colour sums where they would go)
    whole_feat, whole_depth_T = ctx.out_feat.clone(), ctx.out_rgba.clone()
    for chunks in (2, 4):
        ctx2 = api.RenderCtx("cuda:0"); ctx2.setup(W, H, m.cap, n_chunks=chunks)
        with pytest.raises(RuntimeError, match="unsupported lane"):
            api.render_forward(ctx2, m, rp, sync=True)        # bwd_info is still set
        rp.bwd_info = False
        api.render_forward(ctx2, m, rp, sync=True)
        assert torch.equal(ctx2.out_feat, whole_feat) and torch.equal(ctx2.out_rgba, whole_depth_T), chunks
        rp.bwd_info = True


def test_model_compact_keeps_flagged_splats_in_order():
    """Model::compact (src/model.cu:120-155): every per-splat array, planar SH lanes included, is gathered by the stable
    list of kept indices."""
    import torch
    from b2ctrain_b200 import api
    n, deg = 5000, 2
    scene = scenes.make_splats(n, deg, 55)
    m = api.Model("cuda:0").upload(scene)
    g = torch.Generator(device="cuda:0"); g.manual_seed(3)
    for k in ("m_pos_op", "v_quat", "m_sh_dc", "m_sh_hi", "v_sh", "refine_norm", "vis_count"):
        getattr(m, k).copy_(torch.rand(getattr(m, k).shape, generator=g, device="cuda:0"))
    m.last_step[:n] = torch.arange(n, dtype=torch.int32, device="cuda:0")
    extra = torch.rand(m.cap, generator=g, device="cuda:0")
    before = {k: getattr(m, k).clone() for k in api._MODEL_PTRS}
    keep = (torch.rand(n, generator=g, device="cuda:0") < 0.37).to(torch.int32)
    keep[0], keep[n - 1] = 1, 1
    idx = torch.nonzero(keep).flatten()
    kept, (extra2,) = m.compact(keep, [extra])
    assert kept == len(idx) == m.n
    for k in ("pos_op", "quat", "lscale", "m_pos_op", "v_quat"):
        assert torch.equal(getattr(m, k)[:kept], before[k][idx]), k
    for k in ("sh_dc", "sh_hi", "m_sh_dc", "m_sh_hi"):
        assert torch.equal(getattr(m, k)[:, :kept], before[k][:, idx]), k
    for k in ("v_sh", "refine_norm", "vis_count", "last_step"):
        assert torch.equal(getattr(m, k)[:kept], before[k][idx]), k
    assert torch.equal(extra2[:kept], extra[idx])
    assert m.compact(torch.ones(kept, dtype=torch.int32, device="cuda:0"))[0] == kept   # nothing to drop: untouched
    d = m.download()
    assert np.array_equal(d["sh"], scene["sh"][idx.cpu().numpy()])


def test_chunked_render_edge_cases():
    """The chunked renderer on inputs with nothing to do: no splats, splats that are all culled (behind the camera), an
    image smaller than a tile, and more chunks than visible splats. Output = the whole-view path's."""
    import torch
    from b2ctrain_b200 import api
    cases = []
    base = scenes.make_splats(40, 1, 5, log_scale=(-2.5, 0.3))
    cam = scenes.look_at_camera(scenes.orbit_eye(3.0, 10.0, 5.0), 37, 21, 30.0)
    cases.append(("few splats, five chunks", base, cam))
    behind = {k: (v.copy() if hasattr(v, "copy") else v) for k, v in base.items()}
    behind["pos_op"][:, :3] = np.asarray(cam["pos"], np.float32) * 3.0          # on the far side of the camera: every splat is culled
    cases.append(("all culled", behind, cam))
    tiny = scenes.look_at_camera(scenes.orbit_eye(3.0, 0.0, 0.0), 5, 3, 6.0)
    cases.append(("image smaller than a tile", base, tiny))
    for name, scene, c in cases:
        m = api.Model("cuda:0").upload(scene)
        imgs = []
        for chunks in (1, 5):
            ctx = api.RenderCtx("cuda:0"); ctx.want_depth = True
            ctx.setup(c["W"], c["H"], m.cap, n_chunks=chunks)
            rp = api.RenderParams(c, bg=(0.3, 0.2, 0.1), sh_degree=1, bwd_info=True)
            api.render_forward(ctx, m, rp, sync=True)
            gt = torch.zeros(c["W"] * c["H"], dtype=torch.int32, device="cuda:0")
            api.photometric_loss(ctx, api.ViewGPU(gt, None, c["W"], c["H"]), api.LossParams())
            api.rasterize_backward(ctx, m, rp)
            torch.cuda.synchronize()
            imgs.append((ctx.out_rgba.cpu().numpy(), ctx.out_depth.cpu().numpy(), ctx.v_splat[:m.n].cpu().numpy()))
        assert np.array_equal(imgs[0][0], imgs[1][0]), name
        assert np.array_equal(imgs[0][1], imgs[1][1]), name
        assert rel_l2(imgs[1][2], imgs[0][2]) <= 1e-5 or float(np.abs(imgs[0][2]).max()) == 0.0, name
    # an empty model
    m = api.Model("cuda:0").upload(scenes.make_splats(0, 1, 1))
    ctx = api.RenderCtx("cuda:0"); ctx.setup(16, 16, 1, n_chunks=3)
    api.render_forward(ctx, m, api.RenderParams(cam | dict(W=16, H=16), bg=(0.5, 0.25, 0.125), sh_degree=1, bwd_info=True), sync=True)
    img = ctx.out_rgba.cpu().numpy()
    assert np.allclose(img[:, :3], [0.5, 0.25, 0.125]) and np.all(img[:, 3] == 0.0)


def trainer_case(n_views=6):
    import torch
    scene, _ = small_scene(n=6000, degree=2)
    cams = [scenes.look_at_camera(scenes.orbit_eye(3.0, 360.0 * v / n_views, 10.0 + 5.0 * v), 160, 120, 120.0) for v in range(n_views)]
    rng = np.random.Generator(np.random.PCG64(123))
    targets = [torch.from_numpy((rng.integers(0, 2 ** 32, 160 * 120, dtype=np.uint64).astype(np.uint32) | np.uint32(0xFF000000)).view(np.int32)).cuda()
               for _ in cams]
    return scene, cams, targets


def test_trainer_step_with_too_small_intersection_buffers_grows_and_matches():
    """A step whose views overflow the intersection buffers is redone with larger ones before anything is applied
    (the reference grows inside every bin_and_sort, src/gpu/binning.cu:125-133): the updated model equals a run that
    started with large buffers, for the multi-view step and for the fused single-view step."""
    import torch
    from b2ctrain_b200.trainer import Trainer
    scene, cams, targets = trainer_case()
    for views in (len(cams), 1):
        out = []
        for cap in (1 << 22, 2048):
            tr = Trainer(scene, 160, 120, "cuda:0", 0, 1, lr_mean=1e-4, sparse=True, isect_cap=cap, views_in_flight=1)
            for _ in range(2):
                acc = tr.step(cams[:views], targets[:views])
            torch.cuda.synchronize()
            out.append((tr.model.download(), acc.cpu().numpy().copy(), tr.overflow_redos, tr.ctx.isect_cap))
        (big, acc_big, redo_big, _), (small, acc_small, redo_small, cap_small) = out
        assert redo_big == 0 and redo_small >= 1 and cap_small > 2048
        for k in ("pos_op", "quat", "lscale", "sh"):
            # one view per lane in issue order: the accumulator sums are the same sums, up to the order of the atomics
            assert np.max(np.abs(big[k] - small[k]) / (np.abs(big[k]) + 1e-3)) <= 2e-5, (views, k)
        assert abs(acc_big[2] - acc_small[2]) <= 1e-5 * abs(acc_big[2]) and acc_big[3] == acc_small[3] == views


def test_trainer_views_in_flight_match_single_lane():
    """Four views in flight on four streams (the benchmark's default) accumulate the same gradient and the same running
    loss as one view at a time, up to summation order; lanes that get no view in a step add nothing stale."""
    import torch
    from b2ctrain_b200.trainer import Trainer
    scene, cams, targets = trainer_case()
    res = []
    for lanes in (1, 4):
        tr = Trainer(scene, 160, 120, "cuda:0", 0, 1, lr_mean=0.0, sparse=True, views_in_flight=lanes)
        acc6 = tr.step(cams, targets).cpu().numpy().copy()         # six views: lanes 0 and 1 take two each
        tr.model.adam_t += 1
        tr._views(cams[:2], targets[:2], (0.0, 0.0, 0.0), [0, 1], False)   # then two views: lanes 2 and 3 stay idle
        torch.cuda.synchronize()
        res.append((acc6, tr.ctx.loss_accum.cpu().numpy().copy(), tr.grad.cpu().numpy().copy()))
    (a6, a2, g1), (b6, b2, g4) = res
    assert a6[3] == b6[3] == 6 and abs(a6[2] - b6[2]) <= 1e-5 * abs(a6[2])
    assert a2[3] == b2[3] == 2 and abs(a2[2] - b2[2]) <= 1e-5 * abs(a2[2])
    assert rel_l2(g4, g1) <= 1e-5 and np.abs(g1).max() > 0
