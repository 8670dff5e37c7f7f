"""The tensor-parallel sums on ONE GPU, with the peer played by the test.

Both kernels (``aq_allreduce_f32`` and the fused ``aq_linear_allreduce``) exchange values through
buffers that every rank can address; a value travels with the number of the call in one 8-byte
unit, and a rank polls its own receive area until the tags match.  Here rank 1's exchange buffer
is a second buffer on the same GPU and rank 1 itself never runs:
  * nothing ever writes rank 1's values: the bounded poll runs out, the kernel ends by itself and
    ``aq_device_status`` reports the rank that did not arrive (the wait gives up and returns;
    nothing faults or hangs);
  * the test writes rank 1's tagged values into rank 0's receive area BEFORE the launch: the call
    finds them, and its result must be rank 0's values plus those, bit for bit.
No kernel waits for another kernel in either case.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from oracle import alignquant_oracle as oc
from tests import helpers

pytestmark = pytest.mark.gpu

HEADER_BYTES = 1024  # call counter, CTA counter, padding
WORLD = 2


@pytest.fixture()
def peers():
    from alignquant_b200 import _lib
    from alignquant_b200.kernels.cuda import extension as ext

    ext.load_extension()
    lib = _lib.load()
    max_count = 16 * 3072
    size = int(lib.aq_allreduce_buffer_bytes(WORLD, max_count))
    assert size == HEADER_BYTES + 2 * WORLD * max_count * 8
    buffers = [torch.zeros(size, dtype=torch.uint8, device="cuda") for _ in range(WORLD)]
    array = (ctypes.c_void_p * WORLD)(*[b.data_ptr() for b in buffers])
    yield lib, ext, buffers, array, max_count
    ext.set_peer_poll_limit(None)
    torch.cuda.synchronize()


def _units(buffer: torch.Tensor, max_count: int) -> torch.Tensor:
    """The receive areas of an exchange buffer as int32 [parity][rank][position][value bits, call number]."""
    return buffer[HEADER_BYTES:].view(torch.int32).view(2, WORLD, max_count, 2)


def _play_peer(buffer: torch.Tensor, max_count: int, call: int, rank: int, values: torch.Tensor) -> None:
    units = _units(buffer, max_count)
    units[call & 1, rank, : values.numel(), 0] = values.reshape(-1).view(torch.int32)
    units[call & 1, rank, : values.numel(), 1] = call


def _allreduce(lib, partial, out, array, max_count):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.aq_allreduce_f32(ctypes.c_void_p(partial.data_ptr()), ctypes.c_void_p(out.data_ptr()), partial.numel(), 0, WORLD,
                                ctypes.cast(array, ctypes.c_void_p), max_count, ctypes.c_void_p(stream))


def test_peer_sum_gives_up_when_the_peer_never_arrives_and_recovers(peers):
    from alignquant_b200 import _lib

    lib, ext, buffers, array, max_count = peers
    gen = torch.Generator(device="cuda").manual_seed(3)
    partial = torch.randn(4096, generator=gen, device="cuda")
    out = torch.zeros_like(partial)
    ext.set_peer_poll_limit(4096)
    assert int(lib.aq_get_option(_lib.AQ_OPT_PEER_POLL_LIMIT)) == 4096
    assert _allreduce(lib, partial, out, array, max_count) == 0, _lib.last_error()
    status = lib.aq_device_status(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))  # returns: the kernel ended by itself
    assert status == -4 and "rank 1" in _lib.last_error()
    assert lib.aq_device_status(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0  # reported once
    # rank 0 pushed its values, tagged with call number 1, into rank 1's receive area all the same
    sent = _units(buffers[1], max_count)[1, 0, : partial.numel()]
    assert torch.equal(sent[:, 0].view(torch.float32), partial) and bool((sent[:, 1] == 1).all())

    # the buffers are zeroed again, the peer's values are in place before the launch: a normal call
    ext.set_peer_poll_limit(None)
    for call in (1, 2, 3):
        if call == 1:
            for b in buffers:
                b.zero_()
        peer = torch.randn(4096, generator=gen, device="cuda")
        _play_peer(buffers[0], max_count, call, 1, peer)
        assert _allreduce(lib, partial, out, array, max_count) == 0, _lib.last_error()
        ext.device_status()
        assert torch.equal(out, partial + peer), f"call {call}"  # rank order: own value first


@pytest.fixture(params=["small-CTA kernel", "ring kernel"])
def decode_kernel(request):
    """Both decode kernels carry the fused epilogue; the ring kernel is forced through the option."""
    from alignquant_b200.kernels.cuda import extension as ext

    ext.load_extension()
    ext.set_decode_kernel(cluster_only=request.param == "ring kernel")
    yield request.param
    ext.set_decode_kernel()


@pytest.mark.parametrize("m", [1, 7, 16, 24])
def test_fused_projection_and_rank_sum_with_a_played_peer(peers, decode_kernel, m):
    from alignquant_b200 import _lib

    lib, ext, buffers, array, max_count = peers
    n, k = 2048, 512  # a row-parallel shard; both decode kernels take it
    n_j, n_k = n // 64, k // 64
    plan = ext.linear_plan(m, n_j, n_k)
    assert plan["kernel"] == 3 and (plan["splits"] > 1) == (decode_kernel == "ring kernel")
    packed, _, tiles, scales = oc.synthetic_layer(n, k, seed=5)
    weights, _ = helpers.prepare_layer(packed, n_k)
    xt = helpers.torch_activation(oc.synthetic_activation(m, k, seed=m), torch.float16)
    xq, a_s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode="token")
    own = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token")
    gen = torch.Generator(device="cuda").manual_seed(m)
    stream = torch.cuda.current_stream().cuda_stream

    def fused(out):
        return lib.aq_linear_allreduce(
            ctypes.c_void_p(xq.data_ptr()), ctypes.c_void_p(a_s.data_ptr()), _lib.AQ_SCALE_TOKEN, m,
            ctypes.c_void_p(weights.image.data_ptr()), n_j, n_k, None, _lib.AQ_F32, ctypes.c_void_p(out.data_ptr()),
            0, WORLD, ctypes.cast(array, ctypes.c_void_p), max_count, None, 0, ctypes.c_void_p(stream))

    for call in (1, 2):
        peer = torch.randn((m, n), generator=gen, device="cuda")
        _play_peer(buffers[0], max_count, call, 1, peer)
        out = torch.full((m, n), float("nan"), device="cuda")
        assert fused(out) == 0, _lib.last_error()
        ext.device_status()
        assert torch.equal(out, own + peer), f"call {call}"
        sent = _units(buffers[1], max_count)[call & 1, 0, : m * n]
        assert torch.equal(sent[:, 0].view(torch.float32).view(m, n), own) and bool((sent[:, 1] == call).all())

    # call 3 finds no peer values: the poll runs out, the kernel ends, the status names the wait
    ext.set_peer_poll_limit(2048)
    out = torch.zeros((m, n), device="cuda")
    assert fused(out) == 0, _lib.last_error()
    assert lib.aq_device_status(ctypes.c_void_p(stream)) == -4 and "timed out" in _lib.last_error()


@pytest.mark.parametrize("m", [1, 4, 7])
def test_quantizer_projection_and_rank_sum_in_one_call_with_a_played_peer(peers, m):
    """aq_quant_linear with exchange buffers: quantizer, projection and the sum over the ranks; one
    launch for one row where the small-CTA kernel applies, two otherwise; same bits."""
    from alignquant_b200 import _lib

    lib, ext, buffers, array, max_count = peers
    n, k = 3072, 1536  # a row-parallel shard: the small-CTA decode kernel carries epilogue and quantizer
    n_j, n_k = n // 64, k // 64
    assert ext.linear_plan(m, n_j, n_k)["kernel"] == 3 and ext.quant_linear_is_fused(m, n_j, n_k) == (m == 1)
    packed, *_ = oc.synthetic_layer(n, k, seed=6)
    weights, _ = helpers.prepare_layer(packed, n_k)
    xt = helpers.torch_activation(oc.synthetic_activation(m, k, seed=m), torch.float16)
    ref_q, ref_s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode="token")
    own = ext.alignquant_linear_prepared(ref_q, ref_s, weights, None, scale_mode="token")
    gen = torch.Generator(device="cuda").manual_seed(m)
    stream = torch.cuda.current_stream().cuda_stream
    q = torch.zeros((m, k), dtype=torch.int8, device="cuda")
    s = torch.zeros((m,), device="cuda")
    for call in (1, 2):
        peer = torch.randn((m, n), generator=gen, device="cuda")
        _play_peer(buffers[0], max_count, call, 1, peer)
        out = torch.full((m, n), float("nan"), device="cuda")
        status = lib.aq_quant_linear(
            ctypes.c_void_p(xt.data_ptr()), _lib.AQ_F16, m, ctypes.c_void_p(weights.image.data_ptr()), n_j, n_k, None,
            _lib.AQ_F32, ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(s.data_ptr()),
            None, 0, 0, WORLD, ctypes.cast(array, ctypes.c_void_p), max_count, None, 0, ctypes.c_void_p(stream))
        assert status == 0, _lib.last_error()
        ext.device_status()
        assert torch.equal(out, own + peer), f"call {call}"
        assert torch.equal(q, ref_q) and torch.equal(s, ref_s)
