"""GPU parity of the tensor-memory (tcgen05) GEMM against the CPU oracle."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import alignquant_oracle as oc
from tests import helpers

pytestmark = pytest.mark.gpu

REL, ABS = 1e-3, 1e-2


@pytest.fixture(scope="module")
def ext():
    from alignquant_b200.kernels.cuda import extension

    extension.load_extension()
    return extension


@pytest.fixture()
def options(ext):
    """Library options are process-wide: put the defaults back after the test."""
    yield ext
    ext.set_gemm_tile("auto")
    ext.set_gemm_split(0)
    ext.set_gemm_rounding(False)


def _case(ext, m, n, k, scale_mode, seed, fraction=0.6, act_dtype=torch.bfloat16):
    n_j, n_k = n // 64, k // 64
    packed, states, tiles, scales = oc.synthetic_layer(n, k, seed=seed, w4_fraction=fraction)
    weights, _ = helpers.prepare_layer(packed, n_k)
    x = oc.synthetic_activation(m, k, seed=seed + 1, dtype="bfloat16" if act_dtype == torch.bfloat16 else np.float16)
    xt = helpers.torch_activation(x, act_dtype)
    xq, a_s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode=scale_mode)
    if scale_mode == "token":
        a_mk = oc.expand_act_scales(a_s.cpu().numpy(), m, n_k, "token")
    else:
        a_mk = np.repeat(a_s.cpu().numpy().reshape(-1, n_k), 16, axis=0)[:m]
    return weights, tiles, scales, xq, a_s, a_mk


@pytest.mark.parametrize("scale_mode", ["tile", "token"])
@pytest.mark.parametrize("m", [2, 64, 128, 130, 300])
@pytest.mark.parametrize("n,k", [(64, 64), (192, 192), (256, 1024), (320, 128)])
def test_gemm_matches_oracle(ext, n, k, m, scale_mode):
    n_j, n_k = n // 64, k // 64
    weights, tiles, scales, xq, a_s, a_mk = _case(ext, m, n, k, scale_mode, seed=n + k + m)
    dump = torch.full((m, n_j, n_k, 64), -7, dtype=torch.int32, device="cuda")
    out = ext.alignquant_linear_prepared(xq, a_s, weights, None, schedule="forced_prefill_m64",
                                         scale_mode=scale_mode, acc_dump=dump)
    ext.device_status()
    xq_np = xq.cpu().numpy()
    assert np.array_equal(dump.cpu().numpy(), oc.tile_accumulators_c(xq_np, tiles)), "int32 tile accumulators differ"
    got = out.cpu().numpy()
    want = helpers.planned_fp32(ext, xq_np, a_mk, tiles, scales, m, n_j, n_k, schedule="forced_prefill_m64")
    assert np.array_equal(got, want), "fp32 not in the planned operation order"
    assert np.allclose(got, oc.dequant_matmul_fp64(xq_np, a_mk, tiles, scales), rtol=REL, atol=ABS)


@pytest.mark.parametrize("tile", ["paired", "narrow", "wide"])
@pytest.mark.parametrize("m,n,k", [(130, 192, 192), (300, 320, 1024)])
def test_gemm_separate_rounding_is_the_reference_order(options, tile, m, n, k):
    """AQ_GEMM_ROUNDING_SEPARATE: multiply and add rounded separately, K tiles in increasing order."""
    ext = options
    ext.set_gemm_rounding(True)
    ext.set_gemm_tile(tile)
    n_j, n_k = n // 64, k // 64
    weights, tiles, scales, xq, a_s, a_mk = _case(ext, m, n, k, "tile", seed=n + k + m)
    out = ext.alignquant_linear_prepared(xq, a_s, weights, None, schedule="forced_prefill_m64")
    ext.device_status()
    splits = ext.linear_plan(m, n_j, n_k, schedule="forced_prefill_m64")["splits"]
    want = oc.linear_fp32_c(xq.cpu().numpy(), a_mk, tiles, scales, splits)
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("fraction", [0.0, 1.0])
def test_gemm_uniform_precision_layers(ext, fraction):
    m, n, k = 256, 256, 256
    weights, tiles, scales, xq, a_s, a_mk = _case(ext, m, n, k, "token", seed=3, fraction=fraction)
    out = ext.alignquant_linear_prepared(xq, a_s, weights, None, schedule="forced_prefill_m64", scale_mode="token")
    ext.device_status()
    want = helpers.planned_fp32(ext, xq.cpu().numpy(), a_mk, tiles, scales, m, n // 64, k // 64, schedule="forced_prefill_m64")
    assert np.array_equal(out.cpu().numpy(), want)


def test_gemm_auto_schedule_bf16_output_and_bounds(ext):
    m, n, k = 200, 384, 512
    weights, tiles, scales, xq, a_s, a_mk = _case(ext, m, n, k, "token", seed=21)
    canvas = torch.full((m + 2, n), 77.0, dtype=torch.bfloat16, device="cuda")
    out = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token",
                                         output_dtype=torch.bfloat16, out=canvas[1 : m + 1])
    ext.device_status()
    assert bool((canvas[0] == 77.0).all()) and bool((canvas[m + 1] == 77.0).all())
    want = torch.from_numpy(helpers.planned_fp32(ext, xq.cpu().numpy(), a_mk, tiles, scales, m, n // 64, k // 64)).to(torch.bfloat16)
    assert torch.equal(out.cpu(), want)


def test_gemm_reference_fixture_with_output_transform(ext, golden_dir):
    g = dict(np.load(golden_dir / "linear_transformed.npz"))
    m, k = g["x"].shape
    n_j, n_k = g["states"].shape
    packed = {key[len("packed_"):]: v for key, v in g.items() if key.startswith("packed_")}
    weights, _ = helpers.prepare_layer(packed, n_k)
    xq = torch.from_numpy(g["xq"]).cuda()
    a_s = torch.from_numpy(np.ascontiguousarray(g["act_scales"])).cuda()
    u_meta = torch.from_numpy(g["u_metadata"]).cuda()
    dump = torch.zeros((m, n_j, n_k, 64), dtype=torch.int32, device="cuda")
    out = ext.alignquant_linear_prepared(xq, a_s, weights, u_meta, schedule="forced_prefill_m64", acc_dump=dump)
    ext.device_status()
    assert np.array_equal(dump.cpu().numpy(), g["acc"])
    assert np.allclose(out.cpu().numpy(), g["y"], rtol=REL, atol=ABS)


def test_gemm_agrees_with_streaming_kernel_bit_for_bit(options):
    ext = options
    ext.set_gemm_rounding(True)  # the streaming kernel rounds multiply and add separately
    m, n, k = 96, 256, 384
    weights, tiles, scales, xq, a_s, a_mk = _case(ext, m, n, k, "tile", seed=8)
    splits = ext.linear_plan(m, n // 64, k // 64, schedule="forced_prefill_m64")["splits"]
    a = ext.alignquant_linear_prepared(xq, a_s, weights, None, schedule="forced_prefill_m64")
    b = ext.alignquant_linear_prepared(xq, a_s, weights, None, schedule="forced_prefill",
                                       decode_splits=splits if splits in (1, 2, 4, 8) else 1)
    if splits not in (1, 2, 4, 8):
        pytest.skip(f"the GEMM chose {splits} K ranges, which the streaming kernel cannot be forced to")
    ext.device_status()
    assert torch.equal(a, b)


@pytest.mark.parametrize("tile", ["paired", "narrow", "wide"])
def test_gemm_all_cta_tiles(options, tile):
    """The three CTA tiles give the same bits (K long enough to wrap the stage ring)."""
    ext = options
    ext.set_gemm_tile(tile)
    m, n, k = 260, 448, 1280
    weights, tiles, scales, xq, a_s, a_mk = _case(ext, m, n, k, "tile", seed=31)
    dump = torch.zeros((m, n // 64, k // 64, 64), dtype=torch.int32, device="cuda")
    out = ext.alignquant_linear_prepared(xq, a_s, weights, None, schedule="forced_prefill_m64", acc_dump=dump)
    plain = ext.alignquant_linear_prepared(xq, a_s, weights, None, schedule="forced_prefill_m64")
    ext.device_status()
    xq_np = xq.cpu().numpy()
    assert np.array_equal(dump.cpu().numpy(), oc.tile_accumulators_c(xq_np, tiles))
    want = helpers.planned_fp32(ext, xq_np, a_mk, tiles, scales, m, n // 64, k // 64, schedule="forced_prefill_m64")
    assert np.array_equal(out.cpu().numpy(), want)
    assert np.array_equal(plain.cpu().numpy(), want)


@pytest.mark.parametrize("split", ["2", "3", "8"])
@pytest.mark.parametrize("m", [40, 128, 200])
def test_gemm_split_k_clusters(options, m, split):
    """K ranges over a thread-block cluster: integer sums exact, FP32 in split order, output transform applied."""
    ext = options
    ext.set_gemm_split(int(split))
    n, k = 320, 2048
    weights, tiles, scales, xq, a_s, a_mk = _case(ext, m, n, k, "tile", seed=77 + m)
    n_j, n_k = n // 64, k // 64
    plan = ext.linear_plan(m, n_j, n_k, schedule="forced_prefill_m64")
    assert plan["kernel"] == 1 and plan["splits"] == int(split)
    dump = torch.zeros((m, n_j, n_k, 64), dtype=torch.int32, device="cuda")
    out = ext.alignquant_linear_prepared(xq, a_s, weights, None, schedule="forced_prefill_m64", acc_dump=dump)
    ext.device_status()
    xq_np = xq.cpu().numpy()
    assert np.array_equal(dump.cpu().numpy(), oc.tile_accumulators_c(xq_np, tiles))
    assert np.array_equal(out.cpu().numpy(), oc.linear_fp32_c(xq_np, a_mk, tiles, scales, int(split), fused=True))
