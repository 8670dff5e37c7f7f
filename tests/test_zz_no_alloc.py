"""The allocation-free decode entry point against the regular one.

``aq_linear_decode_static`` is for hosts that can pass inputs and outputs to this library
but cannot give it a workspace (fixed-signature operator plug-ins, runtimes that stop
allocating device memory after start-up).  It must return what ``aq_linear`` returns for
the same layer, call after call, although all its calls share one built-in scratch array.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from oracle import alignquant_oracle as oc
from tests import helpers

pytestmark = pytest.mark.gpu

REL, ABS = 1e-3, 1e-2  # the tolerance every fp32-output comparison in this suite uses


def _static_call(lib, xq, a_s, weights, mode, out, u_meta=None):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.aq_linear_decode_static(
        ctypes.c_void_p(xq.data_ptr()), ctypes.c_void_p(a_s.data_ptr()), mode, xq.size(0),
        ctypes.c_void_p(weights.image.data_ptr()), weights.n_j, weights.n_k,
        None if u_meta is None else ctypes.c_void_p(u_meta.data_ptr()), 2,
        ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream),
    )


@pytest.mark.parametrize("n,k,m", [(640, 4096, 1), (640, 4096, 16), (3072, 3072, 1), (3072, 3072, 9)])
def test_static_scratch_entry_point_matches_regular_entry_point(n, k, m):
    from alignquant_b200 import _lib
    from alignquant_b200.kernels.cuda import extension as ext

    ext.load_extension()
    lib = _lib.load()
    n_j, n_k = n // 64, k // 64
    packed, _, tiles, scales = oc.synthetic_layer(n, k, seed=n + k + m)
    weights, _ = helpers.prepare_layer(packed, n_k)
    xt = helpers.torch_activation(oc.synthetic_activation(m, k, seed=m), torch.float16)
    xq, a_s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode="token")
    ext.set_decode_kernel(stream_k=True)  # the regular entry point with the kernel the static one runs
    try:
        want = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token")
        same_kernel = ext.linear_plan(m, n_j, n_k)["kernel"] == 2
    finally:
        ext.set_decode_kernel()
    assert same_kernel
    for call in range(2):  # two calls in a row share the built-in scratch
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        status = _static_call(lib, xq, a_s, weights, _lib.AQ_SCALE_TOKEN, out)
        assert status == 0, _lib.last_error()
        ext.device_status()
        if same_kernel:  # the regular entry point ran the very same kernel: identical bits
            assert torch.equal(out, want), f"call {call}"
        assert np.allclose(out.cpu().numpy(), want.cpu().numpy(), rtol=REL, atol=ABS), f"call {call}"
    # and through the Python wrapper, against the CPU oracle
    out = ext.alignquant_linear_decode_static(xq, a_s, weights, None, scale_mode="token")
    ext.device_status()
    a_mk = oc.expand_act_scales(a_s.cpu().numpy(), m, n_k, "token")
    y64 = oc.dequant_matmul_fp64(xq.cpu().numpy(), a_mk, tiles, scales)
    assert np.allclose(out.cpu().numpy(), y64, rtol=REL, atol=ABS)


def test_static_scratch_entry_point_rejects_what_it_cannot_hold():
    from alignquant_b200 import _lib
    from alignquant_b200.kernels.cuda import extension as ext

    ext.load_extension()
    lib = _lib.load()
    packed, *_ = oc.synthetic_layer(64, 64, seed=1)
    weights, _ = helpers.prepare_layer(packed, 1)
    xq = torch.zeros((17, 64), dtype=torch.int8, device="cuda")
    a_s = torch.ones((17,), dtype=torch.float32, device="cuda")
    out = torch.empty((17, 64), dtype=torch.float32, device="cuda")
    assert _static_call(lib, xq, a_s, weights, _lib.AQ_SCALE_TOKEN, out) == -1
    assert "1 to 16 rows" in _lib.last_error()
    # A layer whose stream-K scratch need exceeds the built-in array: refused before anything is
    # queued or read, so small stand-in buffers are enough (more than 1024 x 148 tiles = more than
    # 256 CTA ranges of 16 rows).
    weights.n_j, weights.n_k = 4096, 64
    assert _static_call(lib, xq[:16], a_s[:16], weights, _lib.AQ_SCALE_TOKEN, out) == -3
    assert "built-in scratch holds" in _lib.last_error()
    weights.n_j, weights.n_k = 16385, 1  # more tile rows than the counter region has counters
    assert _static_call(lib, xq[:1], a_s[:1], weights, _lib.AQ_SCALE_TOKEN, out) == -1
    torch.cuda.synchronize()


def test_static_scratch_entry_point_with_output_transform_and_tile_scales():
    """Non-identity inverse output transform and 16 x 64 activation-tile scales: the same bits as
    ``aq_linear`` where that runs the same kernel."""
    from alignquant_b200 import _lib
    from alignquant_b200.kernels.cuda import extension as ext

    ext.load_extension()
    lib = _lib.load()
    n, k, m = 640, 1024, 11
    n_j, n_k = n // 64, k // 64
    packed, _, tiles, scales = oc.synthetic_layer(n, k, seed=23)
    weights, _ = helpers.prepare_layer(packed, n_k)
    from alignquant_b200.quantization.exact import metadata_stack

    u_meta = metadata_stack([3, -1, 0, 7, 2, -1, 5, 1, 4, 6], torch.device("cuda"))
    xt = helpers.torch_activation(oc.synthetic_activation(m, k, seed=2), torch.float16)
    xq, a_s = ext.alignquant_activation_quantize_cuda(xt, None)
    ext.set_decode_kernel(stream_k=True)  # the regular entry point with the kernel the static one runs
    try:
        want = ext.alignquant_linear_prepared(xq, a_s, weights, u_meta)
        assert ext.linear_plan(m, n_j, n_k)["kernel"] == 2
    finally:
        ext.set_decode_kernel()
    for call in range(2):
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        assert _static_call(lib, xq, a_s, weights, _lib.AQ_SCALE_TILE, out, u_meta) == 0, _lib.last_error()
        ext.device_status()
        assert torch.equal(out, want), f"call {call}"
    a_mk = np.repeat(a_s.cpu().numpy().reshape(-1, n_k), 16, axis=0)[:m]
    y64 = oc.dequant_matmul_fp64(xq.cpu().numpy(), a_mk, tiles, scales, u_meta.cpu().numpy())
    assert np.allclose(want.cpu().numpy(), y64, rtol=REL, atol=ABS)
