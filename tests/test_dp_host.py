"""Host-side logic of the data-parallel step on CPU: two gloo ranks share a step's views round-robin, each sums the
(oracle) per-view parameter gradients of its share, one all-reduce gives every rank the sum over all views, and the
identical Adam update keeps the replicas bit-identical. The GPU path runs the same partition / reduce code with NCCL."""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
sys.path.insert(0, os.environ["B2K_ROOT"])
import numpy as np, torch, torch.distributed as dist
from b2ctrain_b200 import scenes
from b2ctrain_b200.trainer import partition_views, reduce_gradients, slice_bounds, reduce_statistics
from oracle import orc
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
scene = scenes.make_splats(300, 1, 5, log_scale=(-2.5, 0.4))
cams = [scenes.look_at_camera(scenes.orbit_eye(3.0, 40.0 * v, 10.0), 48, 40, 40.0) for v in range(5)]
gt = np.random.Generator(np.random.PCG64(1)).integers(0, 2 ** 32, 48 * 40, dtype=np.uint64).astype(np.uint32)
lp = dict(l1_w=np.float32(0.8), ssim_w=np.float32(-0.2))
def view_grad(v): return orc.step(scene, cams[v], np.zeros(3), gt, None, lp, backward=True)["grad"]
mine = partition_views(len(cams), rank, world)
acc = np.zeros((scene["n"], 11 + 3 * 4))
for v in mine: acc += view_grad(v)
g = reduce_gradients(torch.from_numpy(acc.copy()), world).numpy()
# the sliced reduction the GPU step pipelines with the update gives the same bits as the whole-buffer one
gs = torch.from_numpy(acc.copy())
works = [dist.all_reduce(gs[a:a + c], async_op=True) for a, c in slice_bounds(scene["n"], 3)]
for w in works: w.wait()
assert np.array_equal(gs.numpy(), g)
z4 = lambda: np.zeros((scene["n"], 4), np.float32)
state = dict(pos_op=scene["pos_op"].copy(), quat=scene["quat"].copy(), lscale=scene["lscale"].copy(), sh=scene["sh"].copy(), m_pos=z4(), v_pos=z4(), m_q=z4(),
             v_q=z4(), m_ls=z4(), v_ls=z4(), m_sh=np.zeros((scene["n"], 4, 3), np.float32), v_sh=np.zeros(scene["n"], np.float32), last_step=np.zeros(scene["n"], np.uint32))
orc.adam(state, g, np.any(g != 0, axis=1), dict(t=1, lr_mean=1e-4, sparse=1), 1)
# refinement statistics: each rank holds maxima / sums over its own views; the reduction makes them global
rng = np.random.Generator(np.random.PCG64(100 + rank))
local = {k: torch.from_numpy(rng.random(scene["n"]).astype(np.float32)) for k in ("refine_norm", "max_screen", "vis_count", "vis_weight")}
both = []
for r in range(world):   # every rank's arrays, drawn in the same order as `local`
    g2 = np.random.Generator(np.random.PCG64(100 + r))
    both.append({k: g2.random(scene["n"]).astype(np.float32) for k in ("refine_norm", "max_screen", "vis_count", "vis_weight")})
reduce_statistics(local, world)
for k in ("refine_norm", "max_screen"):
    assert np.array_equal(local[k].numpy(), np.maximum(both[0][k], both[1][k])), k
for k in ("vis_count", "vis_weight"):
    assert np.array_equal(local[k].numpy(), both[0][k] + both[1][k]), k
# The sharded form of the update (what b2k_dp_adam_shard does over peer memory), three steps: every rank sums only the
# rows of its slice (b2k_dp_slice) from all ranks' accumulators, updates those splats, and the new parameters of every
# slice reach every replica; moments stay with the owner. Replicas must end identical, and equal to the replicated update.
from b2ctrain_b200.host_trainer import dp_slice
first, count = dp_slice(scene["n"], rank, world)
sl = slice(first, first + count)
shard = dict(pos_op=scene["pos_op"].copy(), quat=scene["quat"].copy(), lscale=scene["lscale"].copy(), sh=scene["sh"].copy(), m_pos=z4(), v_pos=z4(), m_q=z4(),
             v_q=z4(), m_ls=z4(), v_ls=z4(), m_sh=np.zeros((scene["n"], 4, 3), np.float32), v_sh=np.zeros(scene["n"], np.float32), last_step=np.zeros(scene["n"], np.uint32))
full = {k: v.copy() for k, v in shard.items()}
for t in (1, 2, 3):
    every = [torch.zeros_like(torch.from_numpy(acc)) for _ in range(world)]
    dist.all_gather(every, torch.from_numpy(acc * t))                      # the peers' accumulators, as the kernel reads them
    rows = sum(e.numpy()[sl] for e in every)                               # fixed order of ranks: the same sums everywhere
    # The kernel fetches a peer's row only when that peer's bitmap (one bit per splat, set by its projection backward when
    # it adds a row) marks it: rows left out are zero, so the sums are the same bits.
    marks = [np.packbits(np.any(e.numpy() != 0, axis=1), bitorder="little") for e in every]
    marked = [np.unpackbits(m, bitorder="little")[: scene["n"]].astype(bool) for m in marks]
    assert np.array_equal(sum(np.where(b[sl, None], e.numpy()[sl], 0.0) for b, e in zip(marked, every)), rows)
    mine_state = {k: np.ascontiguousarray(v[sl]) for k, v in shard.items()}
    orc.adam(mine_state, rows, np.any(rows != 0, axis=1), dict(t=t, lr_mean=1e-4, sparse=1), 1)
    for k, v in mine_state.items(): shard[k][sl] = v
    for k in ("pos_op", "quat", "lscale", "sh"):                           # parameter broadcast: every slice from its owner
        for r in range(world):
            a, c = dp_slice(scene["n"], r, world)
            part = torch.from_numpy(np.ascontiguousarray(shard[k][a:a + c]))
            dist.broadcast(part, src=r)
            shard[k][a:a + c] = part.numpy()
    gt_all = sum(e.numpy() for e in every)
    orc.adam(full, gt_all, np.any(gt_all != 0, axis=1), dict(t=t, lr_mean=1e-4, sparse=1), 1)
checksum = int(sum(int(shard[k].view(np.uint32).astype(np.uint64).sum()) for k in ("pos_op", "quat", "lscale", "sh")))
for k in ("pos_op", "quat", "lscale", "sh"):
    assert np.array_equal(shard[k], full[k]), k                           # sharded == replicated, bit for bit
np.savez(os.path.join(os.environ["B2K_OUT"], f"rank{rank}.npz"), mine=np.array(mine), g=g, pos=state["pos_op"], sh=state["sh"], checksum=np.uint64(checksum),
         slice=np.array([first, count]))
if rank == 0:
    total = np.zeros_like(acc)
    for v in range(len(cams)): total += view_grad(v)
    np.save(os.path.join(os.environ["B2K_OUT"], "serial.npy"), total)
dist.destroy_process_group()
'''


def test_two_rank_gloo_step(tmp_path):
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29613", B2K_ROOT=ROOT, B2K_OUT=str(tmp_path),
                   OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    for p in procs:
        out, err = p.communicate(timeout=240)
        assert p.returncode == 0, err[-2000:]
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    serial = np.load(tmp_path / "serial.npy")
    assert sorted(list(r0["mine"]) + list(r1["mine"])) == [0, 1, 2, 3, 4] and abs(len(r0["mine"]) - len(r1["mine"])) <= 1
    assert np.array_equal(r0["g"], r1["g"])                       # every rank holds the same reduced gradient
    assert np.allclose(r0["g"], serial, rtol=1e-12, atol=1e-15)    # = the sum of the per-view gradients
    assert np.array_equal(r0["pos"], r1["pos"]) and np.array_equal(r0["sh"], r1["sh"])   # replicas stay bit-identical
    assert np.abs(r0["g"]).max() > 0
    # the sharded update: slices partition the splats, replicas carry the same checksum after three steps
    assert r0["slice"][0] == 0 and r0["slice"][0] + r0["slice"][1] == r1["slice"][0] and r1["slice"][0] + r1["slice"][1] == 300
    assert int(r0["checksum"]) == int(r1["checksum"])


def test_slice_bounds_cover_the_model_on_block_boundaries():
    from b2ctrain_b200.trainer import slice_bounds
    for n in (0, 1, 127, 128, 129, 3000, 3_000_000, 3_000_001):
        for slices in (1, 3, 4, 7):
            b = slice_bounds(n, slices)
            assert len(b) <= max(1, slices) and sum(c for _, c in b) == n
            pos = 0
            for a, c in b:
                assert a == pos and a % 128 == 0 and c > 0
                pos += c
