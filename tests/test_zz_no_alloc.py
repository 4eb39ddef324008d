"""The allocation-free binning entry point against the regular one.

Some users of the library run where device allocation is not theirs to do: a plugin inside a host application that
owns (and has already reserved) the GPU memory pool, or a latency-critical thread that may not take the allocator's
lock. b2k_bin_sort_static keeps the radix-sort scratch in a fixed array inside the library instead of a caller buffer.
This file is collected last on purpose, so a failure here cannot hide the result of any other test.
"""
import ctypes as C

import numpy as np
import pytest

from b2ctrain_b200 import scenes
from tests.util import Harness

pytestmark = pytest.mark.gpu


def _bin_static(h, n):
    cs = h.ctx.struct()
    cs.sort_tmp, cs.sort_tmp_bytes = None, 0          # the entry point must not need the caller's scratch
    st = h.api.lib().b2k_bin_sort_static(C.byref(cs), n, h.api._stream(None))
    assert st == h.api.B2K_OK, h.api.lib().b2k_error_string(st)
    total = C.c_uint32(0)
    assert h.api.lib().b2k_read_num_isect(C.byref(cs), h.api._stream(None), C.byref(total)) == h.api.B2K_OK
    return int(total.value)


def _snapshot(h, total):
    return (h.u32(h.ctx.vals_sorted, total).copy(), h.u32(h.ctx.keys_sorted, total).copy(), h.u32(h.ctx.tile_ranges).copy(),
            h.u32(h.ctx.order, h.model.n).copy(), h.u32(h.ctx.tile_off, h.model.n).copy())


def test_static_scratch_binning_matches_regular_entry_point_twice():
    results = []
    for seed, n in ((21, 6000), (22, 9000)):          # two calls in a row share the array: the second must not see the first
        scene = scenes.make_splats(n, 1, seed, log_scale=(-3.2, 0.5))
        scene["lscale"][:20, :3] = -1.0               # a few splats with large tile boxes (the list-driven path)
        cam = scenes.look_at_camera(scenes.orbit_eye(3.0, 25.0, 10.0), 160, 120, 120.0)
        h = Harness(scene, cam)
        h.api.project_splats(h.ctx, h.model, h.rp)
        h.api.bin_and_sort(h.ctx, h.model)
        want = _snapshot(h, h.ctx.num_isect)
        for t in (h.ctx.vals_sorted, h.ctx.keys_sorted, h.ctx.tile_ranges, h.ctx.order, h.ctx.tile_off):
            t.fill_(-1)
        h.api.project_splats(h.ctx, h.model, h.rp)    # the depth sort works in place: restore its input
        total = _bin_static(h, h.model.n)
        assert total == h.ctx.num_isect and total > 10000
        got = _snapshot(h, total)
        for a, b in zip(got, want):
            assert np.array_equal(a, b)               # integer outputs: bit-exact
        results.append(total)
    assert results[0] != results[1]


def test_static_scratch_rejects_oversized_contexts():
    lib = __import__("b2ctrain_b200.api", fromlist=["lib"]).lib()
    from b2ctrain_b200 import api
    cs = api.B2kCtx()
    cs.n_cap = int(lib.b2k_static_max_splats()) + 1
    assert lib.b2k_bin_sort_static(C.byref(cs), 10, None) == api.B2K_ERR_CAPACITY
