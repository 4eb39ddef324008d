"""The C++ step trainer (b2ctrain_b200/host/trainer.cpp behind libb2chost.so) against the Python mirror of the same step
sequence, and its data-parallel forms on two GPUs where the box has them."""
import os
import subprocess
import sys

import numpy as np
import pytest

from b2ctrain_b200 import scenes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def case(n_views=6, n=6000):
    scene = scenes.make_splats(n, 2, 21, log_scale=(-3.2, 0.5))
    cams = [scenes.look_at_camera(scenes.orbit_eye(3.0, 360.0 * v / n_views, 10.0 + 5.0 * v), 160, 120, 120.0) for v in range(n_views)]
    scene = scenes.floor_for_cameras(scene, cams)
    rng = np.random.Generator(np.random.PCG64(123))
    targets = [(rng.integers(0, 2 ** 32, 160 * 120, dtype=np.uint64).astype(np.uint32) | np.uint32(0xFF000000)) for _ in cams]
    return scene, cams, targets


def test_slices_of_the_sharded_update_partition_the_splats():
    """b2k_dp_slice: contiguous, block-aligned slices that cover [0, n) exactly, for ragged sizes and more ranks than blocks."""
    from b2ctrain_b200 import host_trainer as ht
    for n in (0, 1, 127, 128, 129, 1000, 3_000_000, 3_000_001):
        for world in (1, 2, 3, 4, 8, 16):
            at = 0
            for r in range(world):
                first, count = ht.dp_slice(n, r, world)
                assert first == at and count >= 0 and (first % 128 == 0 or count == 0)
                at += count
            assert at == n


def test_host_library_exports_every_entry_point_of_its_header():
    import re
    from b2ctrain_b200 import host_trainer as ht
    hdr = open(os.path.join(ROOT, "b2ctrain_b200", "host", "host_c.h")).read()
    declared = set(re.findall(r"\b(b2ch_\w+)\s*\(", hdr))
    assert declared == set(ht.SIGNATURES), declared ^ set(ht.SIGNATURES)
    l = ht.lib()
    for name in declared:
        assert hasattr(l, name), name


@pytest.mark.gpu
@pytest.mark.parametrize("views,lanes,cap", [(6, 4, 0), (6, 1, 2048), (1, 1, 0), (1, 1, 2048)])
def test_cpp_step_matches_python_step(views, lanes, cap):
    """Two steps of the C++ trainer and of the Python mirror from the same scene, views and settings: the same model up
    to the order of the accumulating atomics, the same running loss; with buffers that start too small, after regrowing."""
    import torch
    from b2ctrain_b200 import host_trainer as ht
    from b2ctrain_b200.trainer import Trainer
    scene, cams, targets = case()
    kw = dict(lr_mean=1e-4, sparse=True, noise_weight=5e-3, noise_clamp=2e-3)
    py = Trainer(scene, 160, 120, "cuda:0", 0, 1, views_in_flight=lanes, isect_cap=cap or None, **kw)
    dev_targets = [torch.from_numpy(t.view(np.int32)).cuda() for t in targets]
    cpp = ht.HostTrainer(scene, 160, 120, views_in_flight=lanes, isect_cap=cap, **kw)
    for cam, t in zip(cams, targets):
        cpp.add_view(cam, t)
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        acc = py.step(cams[:views], dev_targets[:views])
        cpp.step(list(range(views)), stream)
    torch.cuda.synchronize()
    a, b = py.model.download(), cpp.download()
    for k in ("pos_op", "quat", "lscale", "sh"):
        # Same kernels, same inputs; the two runs differ in the order of the accumulating atomics, which Adam turns into
        # a few percent of one learning-rate step (2e-3 for rotations) where a gradient component is close to zero.
        assert np.max(np.abs(a[k] - b[k]) / (np.abs(a[k]) + 1e-3)) <= 1e-4, k
    la, lb = acc.cpu().numpy(), cpp.read_loss(stream)
    assert la[3] == lb[3] == views and abs(la[2] - lb[2]) <= 1e-5 * abs(la[2])
    info = cpp.info()
    assert info["adam_t"] == 2 and (info["overflow_redos"] >= 1) == (cap == 2048)
    # streaming the targets in from pinned host memory gives the same step
    cpp.step(list(range(views)), stream, from_host=True)
    py.step(cams[:views], dev_targets[:views])
    torch.cuda.synchronize()
    a, b = py.model.download(), cpp.download()
    assert np.max(np.abs(a["pos_op"] - b["pos_op"]) / (np.abs(a["pos_op"]) + 1e-3)) <= 5e-5
    assert cpp.info()["h2d_bytes"] == min(views, 6) * 160 * 120 * 4
    cpp.close()


@pytest.mark.gpu
@pytest.mark.parametrize("shard", [1, 0])
def test_two_rank_data_parallel_step_matches_one_rank(shard):
    """Two ranks on two GPUs (child processes, NCCL without NVLS): three steps of six views sharded by view, with the
    sharded peer-memory update and with all-reduce + replicated Adam. Replicas end bit-identical (checksums agree) and
    equal the one-rank result up to summation order."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B2K_DP_SHARD=str(shard))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29541",
                          os.path.join(ROOT, "tests", "dp_worker.py")], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "dp worker ok" in out.stdout
