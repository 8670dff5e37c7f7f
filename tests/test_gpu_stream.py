"""GPU parity of the quantizer, the weight re-layout and the streaming (small-M) kernel
against the CPU oracle, through the Python operator API and the C ABI behind it."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import alignquant_oracle as oc
from tests import helpers

pytestmark = pytest.mark.gpu

REL, ABS = 1e-3, 1e-2  # contract tolerance of fp outputs against the FP64 dequantize-and-matmul


@pytest.fixture(scope="module")
def ext():
    from alignquant_b200.kernels.cuda import extension

    extension.load_extension()
    return extension


@pytest.mark.parametrize("fraction", [0.6, 0.0, 1.0])
@pytest.mark.parametrize("n,k", [(64, 64), (128, 192), (192, 320)])
def test_repack_image_is_exact(ext, n, k, fraction):
    packed, states, tiles, scales = helpers.forced_layer(n, k, seed=n + k, fraction=fraction)
    weights, _ = helpers.prepare_layer(packed, k // 64)
    image = weights.image.cpu().numpy()
    word, rec_scale, payload = helpers.expected_image(states, tiles, scales)
    n_tiles = states.size
    rec = image[: n_tiles * 8].view(np.uint32).reshape(n_tiles, 2)
    assert np.array_equal(rec[:, 0], word)
    assert np.array_equal(rec[:, 1].view(np.float32), rec_scale)
    start = -(-n_tiles * 8 // 2048) * 2048
    assert np.array_equal(image[start : start + payload.size], payload)
    assert image.size == start + payload.size


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,k", [(1, 64), (5, 192), (16, 3072), (130, 256)])
def test_token_quantizer_bit_exact(ext, m, k, dtype):
    x = oc.synthetic_activation(m, k, seed=m * 7 + k, dtype="bfloat16" if dtype == torch.bfloat16 else np.float16)
    x = x.astype(np.float32)
    if m > 2:
        x[2] = 0.0  # all-zero row takes the scale floor
    xt = helpers.torch_activation(x, dtype)
    q, s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode="token")
    q_ref, s_ref = oc.a8_token_quantize(xt.float().cpu().numpy())
    assert np.array_equal(s.cpu().numpy(), s_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)


@pytest.mark.parametrize("k", [4096, 8192, 16384])
def test_token_quantizer_rounding_boundaries(ext, k):
    """Quotients on and next to .5 boundaries, long rows (register path and re-read path)."""
    rng = np.random.default_rng(k)
    rows = []
    for amax in (127.0, 100.0, 3.1415927, 0.017, 65504.0):
        scale = np.float32(amax) / np.float32(127.0)
        targets = (rng.integers(-127, 127, size=k).astype(np.float32) + np.float32(0.5))
        x = (targets * scale).astype(np.float32)
        x += rng.choice(np.array([0.0, 1.0, -1.0, 2.0, -2.0], dtype=np.float32), size=k) * np.spacing(x)
        x[0] = amax
        rows.append(np.clip(x, -amax, amax))
    x = np.stack(rows).astype(np.float32)
    xt = torch.from_numpy(x).cuda()
    q, s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode="token")
    q_ref, s_ref = oc.a8_token_quantize(x)
    assert np.array_equal(s.cpu().numpy(), s_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,k", [(1, 64), (5, 2560), (8, 5120), (32, 3072), (3, 8192), (2, 16384)])
def test_rmsnorm_quantizer_bit_exact(ext, m, k, dtype):
    """Fused RMSNorm + per-token quantizer against the oracle's restatement of the decoder's norm
    module followed by the token quantizer: int8 codes, scales and the normalised values."""
    name = "bfloat16" if dtype == torch.bfloat16 else (np.float16 if dtype == torch.float16 else np.float32)
    rng = np.random.default_rng(m * 13 + k)
    x = oc.round_to_dtype(oc.synthetic_activation(m, k, seed=m + k, dtype=np.float32) * np.float32(0.37), name)
    w = oc.round_to_dtype(1.0 + 0.1 * rng.standard_normal(k, dtype=np.float32), name)
    if m > 2:
        x[2] = 0.0  # all-zero row: the norm returns zeros and the scale takes its floor
    eps = 1e-6
    xt, wt = torch.from_numpy(x).cuda().to(dtype), torch.from_numpy(w).cuda().to(dtype)
    normed = torch.empty_like(xt)
    q, s = ext.alignquant_rmsnorm_quantize_cuda(xt, wt, eps, normed=normed)
    q_ref, s_ref, y_ref = oc.rmsnorm_token_quantize(x, w, eps, name)
    assert np.array_equal(normed.float().cpu().numpy(), y_ref)
    assert np.array_equal(s.cpu().numpy(), s_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)
    # the same codes as the two-step path on the module's output
    q2, s2 = ext.alignquant_activation_quantize_cuda(normed, None, scale_mode="token")
    assert torch.equal(q2, q) and torch.equal(s2, s)
    if dtype != torch.float32:  # and the module arithmetic is torch's own
        xf = xt.float()
        n = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dtype)
        assert float((wt * n - normed).abs().max()) <= float(normed.abs().max()) * 2.0 ** -7


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,k", [(1, 64), (4, 192), (16, 3072), (17, 128), (130, 256)])
def test_tile_quantizer_bit_exact_identity(ext, m, k, dtype):
    x = oc.synthetic_activation(m, k, seed=m * 11 + k, dtype="bfloat16" if dtype == torch.bfloat16 else np.float16)
    xt = helpers.torch_activation(x, dtype)
    meta = torch.from_numpy(oc.identity_metadata(k // 64)).cuda()
    q, s = ext.alignquant_activation_quantize_cuda(xt, meta)
    rows = 1 if m == 1 else 16 * ((m + 15) // 16)
    xp = np.zeros((rows, k), dtype=np.float64)
    xp[:m] = xt.float().cpu().numpy()
    q_ref, s_ref = oc.a8_tile_quantize(xp)
    assert np.array_equal(s.cpu().numpy().reshape(s_ref.shape), s_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref[:m])


def test_tile_quantizer_matches_reference_fixture_with_transform(ext, golden_dir):
    g = dict(np.load(golden_dir / "act_quant_mixed.npz"))
    xt = torch.from_numpy(g["x"]).cuda()
    meta = torch.from_numpy(g["v_metadata"]).cuda()
    q, s = ext.alignquant_activation_quantize_cuda(xt, meta)
    # The kernel evaluates the 64-point butterfly in FP64, the reference's CPU path one
    # FP64 matmul: values agree to rounding noise, so scales agree to float32 rounding
    # and int8 codes may differ by one step on a vanishing fraction of elements.
    assert np.allclose(s.cpu().numpy(), g["scales"], rtol=1e-6, atol=0)
    diff = np.abs(q.cpu().numpy().astype(np.int32) - g["q"].astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3


def _run_linear(ext, xq, a_s, weights, u_meta, m, n_j, n_k, **kw):
    dump = torch.full((m, n_j, n_k, 64), -7, dtype=torch.int32, device="cuda")
    out = ext.alignquant_linear_prepared(xq, a_s, weights, u_meta, acc_dump=dump, **kw)
    ext.device_status()
    return out, dump


@pytest.mark.parametrize("scale_mode", ["tile", "token"])
@pytest.mark.parametrize("m", [1, 4, 16, 17, 32, 33, 64, 128])
@pytest.mark.parametrize("n,k", [(64, 64), (128, 192), (192, 512)])
def test_stream_linear_matches_oracle(ext, n, k, m, scale_mode):
    n_j, n_k = n // 64, k // 64
    packed, states, tiles, scales = oc.synthetic_layer(n, k, seed=n * 3 + k)
    weights, _ = helpers.prepare_layer(packed, n_k)
    x = oc.synthetic_activation(m, k, seed=m + n + k)
    xt = helpers.torch_activation(x, torch.float16)
    xq, a_s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode=scale_mode)
    xq_np = xq.cpu().numpy()
    if scale_mode == "token":
        a_mk = oc.expand_act_scales(a_s.cpu().numpy(), m, n_k, "token")
    else:
        a_mk = np.repeat(a_s.cpu().numpy().reshape(-1, n_k), 16, axis=0)[:m]
    acc_ref = oc.tile_accumulators_c(xq_np, tiles)
    y64 = oc.dequant_matmul_fp64(xq_np, a_mk, tiles, scales)
    schedule = "forced_decode" if m == 1 else "forced_prefill"
    for split in (1, 2, 0):
        if split > n_k:
            continue
        out, dump = _run_linear(ext, xq, a_s, weights, None, m, n_j, n_k,
                                schedule=schedule, decode_splits=split, scale_mode=scale_mode)
        assert np.array_equal(dump.cpu().numpy(), acc_ref), f"int32 tile accumulators differ (split {split})"
        got = out.cpu().numpy()
        if split:
            want = oc.linear_fp32_c(xq_np, a_mk, tiles, scales, split)
            assert np.array_equal(got, want), f"fp32 result not in reference operation order (split {split})"
        elif m <= 32:  # automatic schedule: decode kernels, sums grouped as the library's plan says
            want = helpers.planned_fp32(ext, xq_np, a_mk, tiles, scales, m, n_j, n_k, schedule=schedule)
            assert np.array_equal(got, want), "fp32 result differs from the planned summation order"
        assert np.allclose(got, y64, rtol=REL, atol=ABS)


@pytest.fixture
def decode_kernel(request, ext):
    """Runs the test under a forced decode kernel and restores the automatic choice."""
    ext.set_decode_kernel(cluster_only=request.param == "cluster", stream_k=request.param == "streamk")
    yield request.param
    ext.set_decode_kernel()


@pytest.mark.parametrize("decode_kernel", ["auto", "cluster", "streamk"], indirect=True)
@pytest.mark.parametrize("m", [1, 7, 8, 16, 24, 32])
@pytest.mark.parametrize("n,k", [(3072, 3072), (1024, 8192), (5120, 256), (16384, 1024), (640, 4096)])
def test_decode_kernel_many_ranges(ext, n, k, m, decode_kernel):
    """Layers with more tiles than SMs through every decode kernel: the automatic choice, the ring
    kernel alone, and the persistent stream-K kernel (up to 16 rows), whose ranges start and end
    inside tile rows and reuse the workspace across calls."""
    n_j, n_k = n // 64, k // 64
    wanted = {"cluster": (3,), "streamk": (2,) if m <= 16 else (3,), "auto": (2, 3)}[decode_kernel]
    assert ext.linear_plan(m, n_j, n_k)["kernel"] in wanted
    packed, states, tiles, scales = oc.synthetic_layer(n, k, seed=n + k)
    weights, _ = helpers.prepare_layer(packed, n_k)
    xt = helpers.torch_activation(oc.synthetic_activation(m, k, seed=m), torch.float16)
    for scale_mode in ("token", "tile"):
        xq, a_s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode=scale_mode)
        xq_np = xq.cpu().numpy()
        if scale_mode == "token":
            a_mk = oc.expand_act_scales(a_s.cpu().numpy(), m, n_k, "token")
        else:
            a_mk = np.repeat(a_s.cpu().numpy().reshape(-1, n_k), 16, axis=0)[:m]
        want = helpers.planned_fp32(ext, xq_np, a_mk, tiles, scales, m, n_j, n_k)
        for _ in range(3):
            out = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode=scale_mode)
            ext.device_status()
            assert np.array_equal(out.cpu().numpy(), want)
    dump = torch.zeros((m, n_j, n_k, 64), dtype=torch.int32, device="cuda")
    ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="tile", acc_dump=dump)
    ext.device_status()
    assert np.array_equal(dump.cpu().numpy(), oc.tile_accumulators_c(xq_np, tiles))


@pytest.mark.parametrize("fraction", [0.0, 1.0])
def test_stream_linear_uniform_precision_layers(ext, fraction):
    n, k, m = 128, 256, 8
    packed, states, tiles, scales = helpers.forced_layer(n, k, seed=5, fraction=fraction)
    weights, _ = helpers.prepare_layer(packed, k // 64)
    xt = helpers.torch_activation(oc.synthetic_activation(m, k, seed=9), torch.float16)
    xq, a_s = ext.alignquant_activation_quantize_cuda(xt, None)
    out, dump = _run_linear(ext, xq, a_s, weights, None, m, n // 64, k // 64, decode_splits=1)
    xq_np = xq.cpu().numpy()
    a_mk = np.repeat(a_s.cpu().numpy().reshape(-1, k // 64), 16, axis=0)[:m]
    assert np.array_equal(dump.cpu().numpy(), oc.tile_accumulators_c(xq_np, tiles))
    assert np.array_equal(out.cpu().numpy(), oc.linear_fp32_c(xq_np, a_mk, tiles, scales, 1))


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_stream_linear_half_outputs_and_bounds(ext, out_dtype):
    n, k, m = 192, 320, 13
    n_j, n_k = n // 64, k // 64
    packed, states, tiles, scales = oc.synthetic_layer(n, k, seed=77)
    weights, _ = helpers.prepare_layer(packed, n_k)
    xt = helpers.torch_activation(oc.synthetic_activation(m, k, seed=1), torch.float16)
    xq, a_s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode="token")
    canvas = torch.full((m + 2, n), 123.0, dtype=out_dtype, device="cuda")  # canary rows around the output
    out = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token",
                                         output_dtype=out_dtype, out=canvas[1 : m + 1])
    ext.device_status()
    assert bool((canvas[0] == 123.0).all()) and bool((canvas[m + 1] == 123.0).all())
    a_mk = oc.expand_act_scales(a_s.cpu().numpy(), m, n_k, "token")
    y64 = oc.dequant_matmul_fp64(xq.cpu().numpy(), a_mk, tiles, scales)
    assert np.allclose(out.float().cpu().numpy(), y64, rtol=1e-2 if out_dtype == torch.bfloat16 else REL, atol=ABS)


@pytest.mark.parametrize("name", ["linear_identity", "linear_m1", "linear_transformed"])
def test_reference_fixture_end_to_end(ext, golden_dir, name):
    """Raw artifact tensors from the reference's packer -> quantize -> linear -> y of the
    reference's CPU dequantize-and-matmul, through the reference-signature call."""
    g = dict(np.load(golden_dir / f"{name}.npz"))
    m, k = g["x"].shape
    n_j, n_k = g["states"].shape
    t = helpers.to_cuda({key[len("packed_"):]: v for key, v in g.items() if key.startswith("packed_")})
    xt = torch.from_numpy(g["x"]).cuda()
    v_meta = torch.from_numpy(g["v_metadata"]).cuda()
    u_meta = torch.from_numpy(g["u_metadata"]).cuda()
    xq, a_s = ext.alignquant_activation_quantize_cuda(xt, v_meta)
    if name != "linear_transformed":
        assert np.array_equal(xq.cpu().numpy(), g["xq"])
        assert np.array_equal(a_s.cpu().numpy().reshape(-1, n_k), g["act_scales"][: (m + 15) // 16])
    out = ext.alignquant_linear_cuda(
        xq, a_s, t["state_bits"], t["w4_payload"], t["w4_scales"], t["w8_payload"], t["w8_scales"],
        t["w4_row_offsets"], t["w8_row_offsets"], u_meta,
    )
    ext.device_status()
    assert tuple(out.shape) == (m, n_j * 64) and out.dtype == torch.float32
    assert np.allclose(out.cpu().numpy(), g["y"], rtol=REL, atol=ABS)
    # with the fixture's own int8 activations the integer tile sums are exact
    xq_fix = torch.from_numpy(g["xq"]).cuda()
    a_fix = torch.from_numpy(np.ascontiguousarray(g["act_scales"][: (m + 15) // 16])).cuda()
    weights, _ = helpers.prepare_layer({key[len("packed_"):]: v for key, v in g.items() if key.startswith("packed_")}, n_k)
    out2, dump = _run_linear(ext, xq_fix, a_fix, weights, u_meta, m, n_j, n_k)
    assert np.array_equal(dump.cpu().numpy(), g["acc"])
    assert np.allclose(out2.cpu().numpy(), g["y"], rtol=REL, atol=ABS)


@pytest.mark.parametrize("kernel", ["auto", "cluster", "streamk"])
@pytest.mark.parametrize("m", [1, 9, 24, 40, 200])
def test_output_transform_through_every_kernel(ext, kernel, m):
    """Non-identity output (U) transforms on most tile rows, identity on the others, through the
    small-CTA kernel (cluster exchange of its column groups), the ring kernel (also its 17-32-row
    variant), the stream-K kernel and the GEMM: against the FP64 dequantize-and-matmul with the
    inverse transform, and the same bits from every call."""
    from alignquant_b200.quantization.exact import metadata_stack

    if kernel == "streamk" and m > 16:
        pytest.skip("the stream-K kernel takes at most 16 rows")
    n, k = 3072, 512
    n_j, n_k = n // 64, k // 64
    packed, _, tiles, scales = oc.synthetic_layer(n, k, seed=91)
    weights, _ = helpers.prepare_layer(packed, n_k)
    seeds = [(j * 7) % 11 - 1 for j in range(n_j)]  # -1 (identity) on every eleventh row
    u_meta = metadata_stack(seeds, torch.device("cuda"))
    xt = helpers.torch_activation(oc.synthetic_activation(m, k, seed=m), torch.float16)
    ext.set_decode_kernel(cluster_only=kernel == "cluster", stream_k=kernel == "streamk")
    try:
        for scale_mode in ("token", "tile"):
            xq, a_s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode=scale_mode)
            outs = [ext.alignquant_linear_prepared(xq, a_s, weights, u_meta, scale_mode=scale_mode) for _ in range(2)]
            ext.device_status()
            assert torch.equal(outs[0], outs[1])
            if scale_mode == "token":
                a_mk = oc.expand_act_scales(a_s.cpu().numpy(), m, n_k, "token")
            else:
                a_mk = np.repeat(a_s.cpu().numpy().reshape(-1, n_k), 16, axis=0)[:m]
            y64 = oc.dequant_matmul_fp64(xq.cpu().numpy(), a_mk, tiles, scales, u_meta.cpu().numpy())
            assert np.allclose(outs[0].cpu().numpy(), y64, rtol=REL, atol=ABS), scale_mode
            # and the transform really acts: without it the result is a different one
            plain = oc.dequant_matmul_fp64(xq.cpu().numpy(), a_mk, tiles, scales)
            assert not np.allclose(outs[0].cpu().numpy(), plain, rtol=REL, atol=ABS)
    finally:
        ext.set_decode_kernel()


@pytest.mark.parametrize("m,k", [(16, 3072), (5, 8192), (40, 2560)])
def test_tile_quantizer_with_input_transform_at_layer_sizes(ext, m, k):
    """The V-transform quantizer on rows as long as the benchmark layers' K (48, 128 and 40 tiles, every
    seventh an identity): scales to float32 rounding of the oracle's FP64 matmul, codes equal except for
    at most one step on less than one in a thousand (the kernel's butterfly and the matmul differ in the
    last bits of FP64)."""
    from alignquant_b200.quantization.exact import metadata_stack

    n_k = k // 64
    seeds = [(t * 5) % 7 - 1 for t in range(n_k)]
    meta = metadata_stack(seeds, torch.device("cuda"))
    x = oc.synthetic_activation(m, k, seed=k + m)
    xt = helpers.torch_activation(x, torch.float16)
    q, s = ext.alignquant_activation_quantize_cuda(xt, meta)
    pad = np.zeros((16 * ((m + 15) // 16), k))
    pad[:m] = xt.float().cpu().numpy()
    q_ref, s_ref = oc.a8_tile_quantize(oc.transform_activation(pad, meta.cpu().numpy()))
    assert np.allclose(s.cpu().numpy().reshape(-1, n_k), s_ref, rtol=1e-6, atol=0)
    diff = np.abs(q.cpu().numpy().astype(np.int32) - q_ref[:m].astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3


@pytest.fixture
def always_one_launch(ext):
    """aq_quant_linear as one launch wherever the kernel can do it, whatever the layer's size."""
    ext.set_quant_fusion_tiles(1 << 40)
    yield
    ext.set_quant_fusion_tiles()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,k,m", [(3072, 3072, 1), (5120, 3072, 1), (640, 3072, 1), (3072, 384, 1), (3072, 3072, 2),
                                   (16384, 1024, 1), (3072, 8192, 4), (256, 512, 1), (5120, 3072, 40)])
def test_quantizer_and_projection_in_one_call(ext, always_one_launch, n, k, m, dtype):
    """alignquant_quant_linear: the bits of quantizer + projection, whether it runs as one launch (the
    small-CTA decode kernel quantizing its own row: one fp16 / bf16 row) or as two."""
    n_j, n_k = n // 64, k // 64
    packed, _, tiles, scales = oc.synthetic_layer(n, k, seed=n + k)
    weights, _ = helpers.prepare_layer(packed, n_k)
    xt = helpers.torch_activation(oc.synthetic_activation(m, k, seed=m + n), dtype)
    fused = ext.quant_linear_is_fused(m, n_j, n_k)
    assert fused == (m == 1 and (n, k) in ((3072, 3072), (5120, 3072), (640, 3072), (3072, 384)))
    ref_q, ref_s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode="token")
    for out_dtype in (torch.float32, torch.float16):
        want = ext.alignquant_linear_prepared(ref_q, ref_s, weights, None, scale_mode="token", output_dtype=out_dtype)
        q = torch.full((m, k), 99, dtype=torch.int8, device="cuda")
        s = torch.full((m,), float("nan"), device="cuda")
        for _ in range(2):
            got = ext.alignquant_quant_linear(xt, weights, None, output_dtype=out_dtype, quantized=(q, s), prefetch=weights)
            ext.device_status()
            assert torch.equal(got, want)
            assert torch.equal(q, ref_q) and torch.equal(s, ref_s)
    # the quantized rows against the oracle, the result against the FP64 reference
    q_ref, s_ref = oc.a8_token_quantize(xt.float().cpu().numpy())
    assert np.array_equal(ref_q.cpu().numpy(), q_ref) and np.array_equal(ref_s.cpu().numpy(), s_ref)
    if m <= 8:
        a_mk = oc.expand_act_scales(s_ref, m, n_k, "token")
        y64 = oc.dequant_matmul_fp64(q_ref, a_mk, tiles, scales)
        got = ext.alignquant_quant_linear(xt, weights, None)
        assert np.allclose(got.cpu().numpy(), y64, rtol=REL, atol=ABS)


def test_one_launch_only_for_layers_up_to_the_tile_limit(ext):
    assert ext.quant_linear_is_fused(1, 48, 24) and ext.quant_linear_is_fused(1, 48, 48)  # 1152 and 2304 tiles
    assert not ext.quant_linear_is_fused(1, 80, 48) and not ext.quant_linear_is_fused(2, 48, 24)  # 3840 tiles; two rows
    ext.set_quant_fusion_tiles(0)
    try:
        assert not ext.quant_linear_is_fused(1, 48, 24)
    finally:
        ext.set_quant_fusion_tiles()


def test_quantizer_and_projection_in_one_call_with_output_transform(ext):
    from alignquant_b200.quantization.exact import metadata_stack

    n, k, m = 3072, 3072, 1
    n_j, n_k = n // 64, k // 64
    packed, *_ = oc.synthetic_layer(n, k, seed=77)
    weights, _ = helpers.prepare_layer(packed, n_k)
    u_meta = metadata_stack([(j * 5) % 9 - 1 for j in range(n_j)], torch.device("cuda"))  # identity and non-identity rows
    xt = helpers.torch_activation(oc.synthetic_activation(m, k, seed=9), torch.bfloat16)
    assert ext.quant_linear_is_fused(m, n_j, n_k)
    q, s = ext.alignquant_activation_quantize_cuda(xt, None, scale_mode="token")
    want = ext.alignquant_linear_prepared(q, s, weights, u_meta, scale_mode="token")
    got = ext.alignquant_quant_linear(xt, weights, u_meta)
    ext.device_status()
    assert torch.equal(got, want)


def test_reference_signature_caches_the_image_of_long_lived_tensors(ext, golden_dir, monkeypatch):
    """The reference-signature call re-lays-out the weights once for tensors that stay alive, also
    when one of them is not contiguous; a new tensor object is a new layer."""
    g = dict(np.load(golden_dir / "linear_identity.npz"))
    t = helpers.to_cuda({key[len("packed_"):]: v for key, v in g.items() if key.startswith("packed_")})
    wide = torch.zeros(tuple(t["w8_payload"].shape[:-1]) + (128,), dtype=torch.int8, device="cuda")
    wide[..., :64] = t["w8_payload"]
    strided = wide[..., :64]  # same values, not contiguous, alive for the whole test
    assert not strided.is_contiguous() or strided.numel() == 0
    xq = torch.from_numpy(g["xq"]).cuda()
    a_s = torch.from_numpy(np.ascontiguousarray(g["act_scales"][: (xq.shape[0] + 15) // 16])).cuda()
    u_meta = torch.from_numpy(g["u_metadata"]).cuda()
    builds = []
    real = ext.prepare_weights
    monkeypatch.setattr(ext, "prepare_weights", lambda *a, **k: (builds.append(1), real(*a, **k))[1])
    outs = [ext.alignquant_linear_cuda(xq, a_s, t["state_bits"], t["w4_payload"], t["w4_scales"], strided, t["w8_scales"],
                                       t["w4_row_offsets"], t["w8_row_offsets"], u_meta) for _ in range(3)]
    ext.device_status()
    assert len(builds) == 1 and torch.equal(outs[0], outs[2])
    assert np.allclose(outs[0].cpu().numpy(), g["y"], rtol=REL, atol=ABS)
    ext.alignquant_linear_cuda(xq, a_s, t["state_bits"], t["w4_payload"], t["w4_scales"], t["w8_payload"], t["w8_scales"],
                               t["w4_row_offsets"], t["w8_row_offsets"], u_meta)
    assert len(builds) == 2


def test_argument_errors_raise(ext):
    packed, *_ = oc.synthetic_layer(64, 64, seed=1)
    weights, t = helpers.prepare_layer(packed, 1)
    xq = torch.zeros((2, 64), dtype=torch.int8, device="cuda")
    s = torch.ones((1,), dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError):
        ext.alignquant_linear_prepared(xq, s, weights, None, schedule="fastest")
    with pytest.raises(RuntimeError, match="forced decode schedule requires exactly one row"):
        ext.alignquant_linear_prepared(xq, s, weights, None, schedule="forced_decode")
    with pytest.raises(RuntimeError, match="decode_splits may not exceed"):
        ext.alignquant_linear_prepared(xq, s, weights, None, decode_splits=2)
    with pytest.raises(RuntimeError, match="one scalar per M16x64 tile"):
        ext.alignquant_linear_prepared(xq, torch.ones(3, device="cuda"), weights, None)
    with pytest.raises(RuntimeError, match="K must be a multiple of 64"):
        ext.alignquant_activation_quantize_cuda(torch.zeros((2, 65), device="cuda", dtype=torch.float16), None)
    with pytest.raises(RuntimeError, match="selected payload count mismatch"):
        ext.prepare_weights(t["state_bits"], t["w4_payload"], t["w4_scales"], t["w8_payload"], t["w8_scales"],
                            t["w4_row_offsets"], t["w8_row_offsets"], n_k=2)
