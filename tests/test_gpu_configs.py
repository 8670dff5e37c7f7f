"""GPU parity at the benchmark configurations' own shapes.

Every case builds a seeded 60 % W4 layer of a configuration's shape on the GPU with the package's
packer, decodes the packed artifact tensors independently with the CPU oracle, and compares the
library with the oracle on the same int8 activations:
  * every per-(row, N64 tile, K64 tile) int32 sum bit for bit (through ``acc_dump``) wherever the
    dump stays below about 1 GB;
  * the FP32 result bit for bit in the summation order ``aq_linear_plan`` reports;
  * the result against the FP64 dequantize-and-matmul within rel 1e-3 / abs 1e-2 (for the largest
    products on a subset of rows that contains the first and last row of several CTA tiles).
Configurations: a single M16 x K3072 x N8192 linear; the Llama-3.2-3B projection groups at
M in {1, 4, 8, 16} (fp16) and M in {512, 2048, 8192} (bf16); the Qwen3-4B groups at M = 8; the
Qwen3-14B groups at M = 32 and their shards under 8-way tensor parallelism.
"""

from __future__ import annotations

import functools

import numpy as np
import pytest
import torch

from oracle import alignquant_oracle as oc

pytestmark = pytest.mark.gpu

REL, ABS = 1e-3, 1e-2  # contract tolerance of fp outputs against the FP64 dequantize-and-matmul
DUMP_LIMIT_BYTES = 1 << 30

LLAMA = {"qkv": (5120, 3072), "o": (3072, 3072), "gate_up": (16384, 3072), "down": (3072, 8192)}
QWEN3_4B = {"qkv": (6144, 2560), "o": (2560, 4096), "gate_up": (19456, 2560), "down": (2560, 9728)}
QWEN3_14B = {"qkv": (7168, 5120), "o": (5120, 5120), "gate_up": (34816, 5120), "down": (5120, 17408)}
# per-rank shards under 8-way tensor parallelism: columns of qkv / gate_up, K of o / down
QWEN3_14B_TP8 = {"qkv": (896, 5120), "o": (5120, 640), "gate_up": (4352, 5120), "down": (5120, 2176)}


@pytest.fixture(scope="module")
def ext():
    from alignquant_b200.kernels.cuda import extension

    extension.load_extension()
    return extension


@functools.lru_cache(maxsize=2)
def _layer(n: int, k: int):
    """(prepared weights, logical int8 tiles, tile scales) of a seeded layer of this shape."""
    from alignquant_b200.kernels.cuda import extension as ext
    from alignquant_b200.synthetic import synthetic_module_tensors

    tensors = synthetic_module_tensors(n, k, seed=n * 7 + k, device="cuda")
    weights = ext.prepare_weights(
        tensors["state_bits"], tensors["w4_payload"], tensors["w4_scales"], tensors["w8_payload"], tensors["w8_scales"],
        tensors["w4_row_offsets"], tensors["w8_row_offsets"], n_k=k // 64,
    )
    host = {name: t.cpu().numpy() for name, t in tensors.items()}
    del tensors
    states, tiles, scales = oc.unpack_module_arrays(host, n // 64, k // 64)
    assert abs(float((states == oc.P4).mean()) - 0.6) < 0.01
    return weights, tiles, scales


def _edge_rows(m: int) -> np.ndarray:
    """First and last rows of the first, a middle and the last 128-row CTA tile (and of a 16-row group)."""
    blocks = sorted({0, (m // 128) // 2, (m - 1) // 128})
    rows = set()
    for b in blocks:
        lo, hi = b * 128, min(m, (b + 1) * 128) - 1
        rows.update((lo, min(lo + 15, hi), min(lo + 16, hi), hi))
    return np.asarray(sorted(rows), dtype=np.int64)


def _check(ext, n: int, k: int, m: int, act_dtype: torch.dtype, out_dtype: torch.dtype = torch.float32) -> None:
    from alignquant_b200.synthetic import synthetic_activation

    n_j, n_k = n // 64, k // 64
    weights, tiles, scales = _layer(n, k)
    x = synthetic_activation(m, k, seed=m * 31 + n_k, dtype=act_dtype, device="cuda")
    xq, a_s = ext.alignquant_activation_quantize_cuda(x, None, scale_mode="token")
    q_ref, s_ref = oc.a8_token_quantize(x.float().cpu().numpy())
    xq_np = xq.cpu().numpy()
    assert np.array_equal(xq_np, q_ref) and np.array_equal(a_s.cpu().numpy(), s_ref), "quantizer differs from the oracle"
    a_mk = oc.expand_act_scales(s_ref, m, n_k, "token")

    dump_bytes = m * n_j * n_k * 64 * 4
    dump = torch.full((m, n_j, n_k, 64), -7, dtype=torch.int32, device="cuda") if dump_bytes <= DUMP_LIMIT_BYTES else None
    out = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token", acc_dump=dump)
    ext.device_status()
    if dump is not None:
        got_acc = dump.cpu().numpy()
        del dump
        assert np.array_equal(got_acc, oc.tile_accumulators_c(xq_np, tiles)), "int32 tile sums differ"
        del got_acc
        # the run without the dump takes the production instantiation of the kernel
        plain = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token")
        ext.device_status()
        assert torch.equal(plain, out)

    plan = ext.linear_plan(m, n_j, n_k)
    if plan["kernel"] in (2, 3):  # the look-ahead only asks the L2 to fetch: same bits with it
        ahead = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token", prefetch=weights)
        ext.device_status()
        assert torch.equal(ahead, out)
    got = out.cpu().numpy()
    if plan["kernel"] == 2:
        want = oc.linear_fp32_ranges_c(xq_np, a_mk, tiles, scales, plan["splits"], plan["workers"])
    else:
        fused = plan["kernel"] == 1 and not ext.gemm_rounding_is_separate()
        want = oc.linear_fp32_c(xq_np, a_mk, tiles, scales, plan["splits"], plan["workers"], fused=fused)
    assert np.array_equal(got, want), f"fp32 result differs from the planned summation order {plan}"

    rows = np.arange(m) if m <= 64 else _edge_rows(m)
    y64 = oc.linear_fp64_c(xq_np[rows], a_mk[rows], tiles, scales)
    assert np.allclose(got[rows], y64, rtol=REL, atol=ABS)
    if out_dtype != torch.float32:
        low = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token", output_dtype=out_dtype)
        ext.device_status()
        assert torch.equal(low.cpu(), torch.from_numpy(want).to(out_dtype)), "low-precision result is not the rounded fp32 result"
        # fp16 keeps the rel 1e-3 / abs 1e-2 contract; bf16 has 8 bits of mantissa (2^-9 per rounding)
        rel = REL if out_dtype == torch.float16 else 1e-2
        assert np.allclose(low[torch.from_numpy(rows).cuda()].float().cpu().numpy(), y64, rtol=rel, atol=ABS)


def test_config0_single_linear_m16_k3072_n8192(ext):
    _check(ext, 8192, 3072, 16, torch.float16, out_dtype=torch.float16)


@pytest.mark.parametrize("m", [1, 4, 8, 16])
@pytest.mark.parametrize("group", list(LLAMA))
def test_config1_llama_decode_sweep(ext, group, m):
    n, k = LLAMA[group]
    _check(ext, n, k, m, torch.float16, out_dtype=torch.float16)


@pytest.mark.parametrize("m", [512, 2048])
@pytest.mark.parametrize("group", list(LLAMA))
def test_config2_llama_prefill(ext, group, m):
    n, k = LLAMA[group]
    _check(ext, n, k, m, torch.bfloat16, out_dtype=torch.bfloat16)


def test_config2_llama_prefill_m8192(ext):
    n, k = LLAMA["o"]
    _check(ext, n, k, 8192, torch.bfloat16)


@pytest.mark.parametrize("group", list(QWEN3_4B))
def test_config3_qwen3_4b_decode_batch8(ext, group):
    n, k = QWEN3_4B[group]
    _check(ext, n, k, 8, torch.bfloat16, out_dtype=torch.bfloat16)


@pytest.mark.parametrize("group", list(QWEN3_14B))
def test_config4_qwen3_14b_decode_batch32(ext, group):
    n, k = QWEN3_14B[group]
    _check(ext, n, k, 32, torch.bfloat16)


@pytest.mark.parametrize("group", list(QWEN3_14B_TP8))
def test_config4_qwen3_14b_tp8_shards(ext, group):
    n, k = QWEN3_14B_TP8[group]
    _check(ext, n, k, 32, torch.bfloat16)


@pytest.mark.parametrize("m", [1, 16])
def test_ring_kernel_with_more_than_256_tiles_per_cta(ext, m):
    """150 tile rows (no K split: one CTA per row) of 257 tiles: a warp of the ring kernel takes 33
    tiles, one more than the 32 whose records its lanes hold at a time."""
    plan = ext.linear_plan(m, 150, 257)
    assert plan["kernel"] == 3 and plan["splits"] == 1
    _check(ext, 9600, 16448, m, torch.float16)
