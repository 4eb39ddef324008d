"""Files of the headless front end (b2ctrain_b200/host/ply.cpp, render_io.cpp): splat PLY in the layout the reference
reads and writes (src/ply.cpp:80-226), cameras.json (src/render/renderer.cpp:185-197, 207-212), and the per-camera render
loop to raw buffers."""
import json
import os
import struct

import numpy as np
import pytest

from b2ctrain_b200 import host_trainer as ht
from b2ctrain_b200 import scenes


def cloud(n=257, degree=2, seed=3):
    s = scenes.make_splats(n, degree, seed)
    return ht.cloud_from_scene(s), s


def test_ply_round_trip_binary(tmp_path):
    c, _ = cloud()
    rng = np.random.Generator(np.random.PCG64(1))
    c["evidence"] = rng.random((c["n"], 7)).astype(np.float32)
    c["labels"] = np.stack([rng.integers(0, 5, c["n"]).astype(np.float32), rng.random(c["n"]).astype(np.float32)], 1)
    path = str(tmp_path / "a.ply")
    ht.write_ply(path, c, comment="SH degree: 2")
    back = ht.read_ply(path)
    assert back["n"] == c["n"] and back["degree"] == 2 and back["has_scales"]
    for k in ("pos", "log_scale", "opacity", "sh", "evidence", "labels"):
        assert np.array_equal(back[k], np.asarray(c[k], np.float32)), k
    q = c["quat"] / np.linalg.norm(c["quat"], axis=1, keepdims=True)          # the writer normalises rotations
    assert np.allclose(back["quat"], q, atol=1e-6)
    head = open(path, "rb").read(400).decode("latin1")
    assert head.startswith("ply\nformat binary_little_endian 1.0\ncomment SH degree: 2\nelement vertex 257\nproperty float x\n")
    # f_rest is channel-major in the file: column 14 is coefficient 1 of the red channel, column 14 + (K - 1) of green
    body = open(path, "rb").read().split(b"end_header\n", 1)[1]
    row0 = np.frombuffer(body[: 4 * (14 + 24 + 9)], np.float32)
    assert row0[14] == c["sh"][0, 1, 0] and row0[14 + 8] == c["sh"][0, 1, 1] and row0[11] == c["sh"][0, 0, 0]


def test_ply_ascii_mixed_types_and_rgb_fallback(tmp_path):
    path = str(tmp_path / "pts.ply")
    with open(path, "w") as f:
        f.write("ply\nformat ascii 1.0\ncomment made by a test\nelement vertex 2\nproperty double x\nproperty float y\nproperty float z\n"
                "property uchar red\nproperty uchar green\nproperty uchar blue\nend_header\n0.5 1 -2 255 0 128\n1e-1 2 3 0 255 64\n")
    c = ht.read_ply(path)
    assert c["n"] == 2 and c["degree"] == 0 and not c["has_scales"]
    assert np.allclose(c["pos"], [[0.5, 1, -2], [0.1, 2, 3]])
    C0 = 0.28209479177387814
    assert np.allclose(c["sh"][:, 0, :], (np.array([[255, 0, 128], [0, 255, 64]]) / 255.0 - 0.5) / C0, atol=1e-6)
    assert np.array_equal(c["quat"], [[1, 0, 0, 0], [1, 0, 0, 0]])            # identity where the file has none


def test_ply_errors(tmp_path):
    bad = str(tmp_path / "bad.ply")
    open(bad, "w").write("ply\nformat binary_little_endian 1.0\nelement vertex 3\nproperty float x\nproperty float y\nproperty float z\nend_header\n")
    with pytest.raises(RuntimeError, match="truncated"):
        ht.read_ply(bad)
    open(bad, "w").write("ply\nformat binary_big_endian 1.0\nelement vertex 0\nproperty float x\nend_header\n")
    with pytest.raises(RuntimeError, match="big-endian"):
        ht.read_ply(bad)
    open(bad, "w").write("ply\nformat ascii 1.0\nelement vertex 1\nproperty float x\nproperty float y\nproperty float z\nproperty float f_rest_0\nend_header\n0 0 0 0\n")
    with pytest.raises(RuntimeError, match="not a valid SH layout"):
        ht.read_ply(bad)
    with pytest.raises(RuntimeError, match="failed to open"):
        ht.read_ply(str(tmp_path / "missing.ply"))


def gl_camera_entry(name, cam):
    """A cameras.json entry (OpenGL camera-to-world rotation, position) of a camera dict of b2ctrain_b200.scenes."""
    R = np.asarray(cam["R"], np.float64).reshape(3, 3)
    c2w = R.T * np.array([1.0, -1.0, -1.0])[None, :]
    return dict(name=name, fx=float(cam["fx"]), fy=float(cam["fy"]), cx=float(cam["cx"]), cy=float(cam["cy"]), position=[float(x) for x in cam["pos"]],
                rotation=c2w.tolist())


@pytest.mark.gpu
def test_headless_render_writes_what_the_operators_render(tmp_path):
    """PLY + cameras.json in, raw RGBA8 / depth buffers out: the same bytes as quantising the image render_forward leaves
    for the same splats and cameras (cameras split over two 'ranks' to cover the round-robin share)."""
    import torch
    from b2ctrain_b200 import api
    c, scene = cloud(n=4000, degree=2, seed=8)
    W, H = 96, 64
    cams = [scenes.look_at_camera(scenes.orbit_eye(3.0, a, 15.0), W, H, 80.0) for a in (0.0, 70.0, 200.0)]
    ply, cj = str(tmp_path / "s.ply"), str(tmp_path / "cameras.json")
    ht.write_ply(ply, c)
    json.dump(dict(width=W, height=H, cameras=[gl_camera_entry(f"view{i}.png", cam) for i, cam in enumerate(cams)]), open(cj, "w"))
    assert ht.render_headless(ply, cj, str(tmp_path), background=(0.1, 0.2, 0.3), depth=True, rank=0, world=2) == 2
    assert ht.render_headless(ply, cj, str(tmp_path), background=(0.1, 0.2, 0.3), depth=True, rank=1, world=2) == 1
    flat = dict(scene); flat["lscale"] = scene["lscale"].copy(); flat["lscale"][:, 3] = 0                      # the file format has no floor lane
    flat["quat"] = ht.read_ply(ply)["quat"]                                                                    # as written: the writer normalises in fp32
    m = api.Model("cuda:0").upload(flat)
    ctx = api.RenderCtx("cuda:0"); ctx.want_depth = True
    ctx.setup(W, H, m.cap)
    for i, cam in enumerate(cams):
        api.render_forward(ctx, m, api.RenderParams(cam, bg=(0.1, 0.2, 0.3), sh_degree=2, bwd_info=False))
        scaled = (np.clip(ctx.out_rgba.cpu().numpy(), 0, 1) * np.float32(255)).astype(np.float64)   # the product in fp32, as the front end forms it
        want = np.floor(scaled + 0.5).astype(np.uint8)                                                # lround: halves away from zero
        got = np.fromfile(str(tmp_path / f"view{i}.rgba8"), np.uint8).reshape(-1, 4)
        diff = np.abs(got.astype(int) - want.astype(int))
        print(f"view {i}: differing {np.mean(diff > 0):.2e}, max {diff.max()}, per channel {np.mean(diff > 0, axis=0)}")
        # The front end composes the camera from the JSON entry in fp32 (translation = -R * position, as the reference's
        # camera_from_json does); the operator call above takes the float64 camera of the scene generator. The images agree
        # to an ulp, which can move a value that sits on a rounding boundary by one step.
        assert diff.max() <= 1 and np.mean(diff > 0) <= 1e-3
        depth = np.fromfile(str(tmp_path / f"view{i}.depth.f32"), np.float32)
        ref = ctx.out_depth.cpu().numpy()
        fin = np.isfinite(ref)
        assert np.array_equal(np.isfinite(depth), fin)
        off = np.abs(depth[fin] - ref[fin]) > 2e-4 * np.abs(ref[fin])   # a ratio of two sums under the same ulp-level camera difference;
        assert off.mean() <= 1e-3                                      # a pixel where a fragment sits on the 1/255 cut may move further


@pytest.mark.gpu
def test_stream_renderer_reads_back_quantised_images_and_depth():
    """b2c::StreamRenderer (device-side quantisation, read-back overlapped with the next camera) against render_forward of
    the operator mirror quantised with numpy: the same bytes up to the ulp-level camera difference described above, for a
    run of cameras that reuses the two staging slots, whole-view and chunked."""
    import torch
    from b2ctrain_b200 import api
    scene = scenes.make_splats(5000, 2, 21)
    W, H = 112, 80
    cams = [scenes.look_at_camera(scenes.orbit_eye(3.0, a, 10.0), W, H, 70.0) for a in (0.0, 45.0, 130.0, 220.0, 300.0)]
    m = api.Model("cuda:0").upload(scene)
    ctx = api.RenderCtx("cuda:0"); ctx.want_depth = True
    ctx.setup(W, H, m.cap)
    stream = torch.cuda.current_stream().cuda_stream
    for chunks, lanes, cap in ((1, 1, 0), (3, 1, 0), (3, 3, 0), (1, 2, 4096), (3, 2, 4096)):
        hr = ht.HostRenderer(scene, W, H, depth=True, render_chunks=chunks, lanes=lanes, isect_cap=cap)
        rgba = [torch.zeros(W * H, dtype=torch.int32).pin_memory() for _ in cams]
        depth = [torch.zeros(W * H, dtype=torch.float32).pin_memory() for _ in cams]
        for i, cam in enumerate(cams):
            hr.render(cam, stream, background=(0.2, 0.1, 0.3), host_rgba8=rgba[i].data_ptr(), host_depth=depth[i].data_ptr())
        hr.finish()
        info = hr.info()
        assert info["d2h_bytes"] == (len(cams) + info["redone"]) * W * H * 8
        assert (info["redone"] > 0) == (cap != 0)          # buffers that start too small: those cameras are rendered again
        hr.close()
        for i, cam in enumerate(cams):
            api.render_forward(ctx, m, api.RenderParams(cam, bg=(0.2, 0.1, 0.3), sh_degree=2, bwd_info=False))
            scaled = (np.clip(ctx.out_rgba.cpu().numpy(), 0, 1) * np.float32(255)).astype(np.float64)
            want = np.floor(scaled + 0.5).astype(np.uint8)
            got = rgba[i].numpy().view(np.uint8).reshape(-1, 4)
            diff = np.abs(got.astype(int) - want.astype(int))
            assert diff.max() <= 1 and np.mean(diff > 0) <= 1e-3, (chunks, i, diff.max(), np.mean(diff > 0))
            ref = ctx.out_depth.cpu().numpy()
            fin = np.isfinite(ref)
            d = depth[i].numpy()
            assert np.array_equal(np.isfinite(d), fin)
            assert (np.abs(d[fin] - ref[fin]) > 2e-4 * np.abs(ref[fin])).mean() <= 1e-3


@pytest.mark.gpu
def test_quantize_rgba8_rounds_like_lround():
    """b2k_quantize_rgba8 against lround(clamp(x, 0, 1) * 255) with the product formed in fp32, on values that sit on and
    next to the rounding boundaries, outside [0, 1], and on random ones."""
    import ctypes as C
    import torch
    from b2ctrain_b200 import api
    rng = np.random.Generator(np.random.PCG64(7))
    k = np.arange(256, dtype=np.float64)
    edge = np.concatenate([(k + 0.5) / 255.0, np.nextafter(((k + 0.5) / 255.0).astype(np.float32), np.float32(0)), np.nextafter(((k + 0.5) / 255.0).astype(np.float32), np.float32(2)),
                           [-1.0, -0.0, 0.0, 1.0, 1.5, 0.49999997 / 255.0]])
    vals = np.concatenate([edge.astype(np.float32), rng.random(4096 * 4 - edge.size).astype(np.float32)]).reshape(-1, 4)
    x = torch.from_numpy(vals).cuda()
    out = torch.zeros(vals.shape[0], dtype=torch.int32, device="cuda:0")
    st = api.lib().b2k_quantize_rgba8(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), C.c_int32(vals.shape[0]), None)
    assert st == 0
    torch.cuda.synchronize()
    p = (np.clip(vals, np.float32(0), np.float32(1)) * np.float32(255)).astype(np.float64)   # the fp32 product, exactly
    want = np.floor(p + 0.5).astype(np.uint8)
    got = out.cpu().numpy().view(np.uint8).reshape(-1, 4)
    assert np.array_equal(got, want)
