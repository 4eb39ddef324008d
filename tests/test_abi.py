"""CPU tests of the drop-in boundary: the C-ABI library loads and exports every symbol include/b2k.h declares, and
argument validation answers with a status instead of touching a device."""
import ctypes as C
import os
import re

import pytest

from b2ctrain_b200 import api, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return api.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b2k.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2k_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_table_agree():
    assert declared_symbols() == sorted(api.SIGNATURES)


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_status_strings(lib):
    assert lib.b2k_error_string(api.B2K_OK) == b"ok"
    assert b"overflow" in lib.b2k_error_string(api.B2K_ERR_OVERFLOW)
    assert lib.b2k_version().startswith(b"b2k")


def test_null_arguments_are_rejected_without_a_device(lib):
    assert lib.b2k_project(None, None, None, None, None) == api.B2K_ERR_ARG
    assert lib.b2k_bin_sort(None, 0, None) == api.B2K_ERR_ARG
    assert lib.b2k_raster_fwd(None, None, None) == api.B2K_ERR_ARG
    assert lib.b2k_loss_photometric(None, None, None) == api.B2K_ERR_ARG
    assert lib.b2k_raster_bwd(None, None, None, None) == api.B2K_ERR_ARG
    assert lib.b2k_optim_fused(None, None, None, None, None) == api.B2K_ERR_ARG
    assert lib.b2k_adam(None, None, None, None) == api.B2K_ERR_ARG
    assert lib.b2k_adam_range(None, None, None, 0, 0, None) == api.B2K_ERR_ARG
    assert lib.b2k_render_chunked(None, None, None, None, None) == api.B2K_ERR_ARG
    one_chunk = api.B2kCtx(); one_chunk.n_chunks = 1   # the chunked renderer wants 2 to 5 chunks
    assert lib.b2k_render_chunked(C.byref(api.B2kModel()), C.byref(api.B2kCamera()), C.byref(api.B2kRenderOpts()), C.byref(one_chunk), None) == api.B2K_ERR_ARG
    m = api.B2kModel(); m.n, m.cap, m.degree = 4, 2, 1   # cap < n
    assert lib.b2k_project(C.byref(m), C.byref(api.B2kCamera()), C.byref(api.B2kRenderOpts()), C.byref(api.B2kCtx()), None) == api.B2K_ERR_ARG
    assert lib.b2k_sort_tmp_bytes(1000, 1 << 22) > 0


def test_unsupported_lanes_raise():
    rp = api.RenderParams(dict(), sh_degree=1)
    rp.hollow_z = object()
    with pytest.raises(RuntimeError, match="unsupported lane"):
        rp.struct()
    with pytest.raises(RuntimeError, match="unsupported lane"):
        api.OptimParams(dict(), frozen=True).struct()
    with pytest.raises(RuntimeError, match="unsupported lane"):
        api.LossParams(normal_scale=0.5).struct(api.ViewGPU(None))
