"""install_alignquant on a tiny decoder with the real kernels (GPU)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import alignquant_oracle as oc
from tests.test_model_glue import FULL_SHAPES, _artifact, _Tiny

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("scale_mode", ["tile", "token"])
@pytest.mark.parametrize("rows", [1, 5, 40, 200])
def test_installed_model_matches_oracle(scale_mode, rows):
    from alignquant_b200.kernels.cuda import extension as ext
    from alignquant_b200.quantization.model import AlignQuantLinear, install_alignquant, reset_alignquant_state

    ext.load_extension()
    artifact, dense = _artifact()
    model = _Tiny().cuda().to(torch.bfloat16)
    installed, meta = install_alignquant(model, artifact, "cuda", scale_mode=scale_mode)
    assert len(installed) == 7 and all(isinstance(m, AlignQuantLinear) for m in installed)
    layer = model.model.layers[0]
    reset_alignquant_state(model)

    def expected(x_bf16, name):
        x = x_bf16.float().cpu().numpy()
        n, k = FULL_SHAPES[name]
        if scale_mode == "token":
            xq, s = oc.a8_token_quantize(x)
            xd = xq.astype(np.float64) * s[:, None]
        else:
            pad = np.zeros((16 * ((x.shape[0] + 15) // 16), k))
            pad[: x.shape[0]] = x
            xq, s = oc.a8_tile_quantize(pad)
            xd = (xq.astype(np.float64).reshape(pad.shape[0], k // 64, 64)
                  * np.repeat(s, 16, axis=0)[:, :, None].astype(np.float64)).reshape(pad.shape)[: x.shape[0]]
        return xd @ dense[name].T

    gen = torch.Generator(device="cuda").manual_seed(rows)
    hidden = torch.randn((2, rows // 2, 128) if rows % 2 == 0 else (rows, 128), generator=gen, device="cuda").to(torch.bfloat16)
    wide = torch.randn((rows, 256), generator=gen, device="cuda").to(torch.bfloat16)
    outs = {
        "self_attn.q_proj": layer.self_attn.q_proj(hidden), "self_attn.k_proj": layer.self_attn.k_proj(hidden),
        "self_attn.v_proj": layer.self_attn.v_proj(hidden), "self_attn.o_proj": layer.self_attn.o_proj(wide),
        "mlp.gate_proj": layer.mlp.gate_proj(hidden), "mlp.up_proj": layer.mlp.up_proj(hidden),
        "mlp.down_proj": layer.mlp.down_proj(wide),
    }
    ext.device_status()
    for short, got in outs.items():
        name = f"model.layers.0.{short}"
        src = wide if short.endswith(("o_proj", "down_proj")) else hidden
        want = expected(src.reshape(-1, src.shape[-1]), name)
        if short == "self_attn.v_proj":
            want = want + layer.self_attn.v_proj.bias.float().cpu().numpy()
        assert got.dtype == torch.bfloat16 and got.shape[:-1] == src.shape[:-1]
        # bf16 output: 8 bits of mantissa on top of the rel 1e-3 / abs 1e-2 contract
        assert np.allclose(got.float().cpu().numpy().reshape(want.shape), want, rtol=1e-2, atol=2e-2), short


def test_reference_built_artifact_installs_and_matches_reference_outputs(golden_dir):
    """tests/golden/artifact_tiny (written by the reference's build_artifact, non-identity V/U seeds and
    bitmaps cut from its Llama-3.2-3B preset, one all-W4 and one all-W8 module) through load_artifact,
    install_alignquant and the kernels, against the reference's FP64 outputs for the same inputs."""
    from alignquant_b200.kernels.cuda import extension as ext
    from alignquant_b200.quantization.artifact import load_artifact
    from alignquant_b200.quantization.model import install_alignquant, reset_alignquant_state

    ext.load_extension()
    io = dict(np.load(golden_dir / "artifact_tiny_io.npz"))
    artifact = load_artifact(golden_dir / "artifact_tiny")
    model = _Tiny(layers=2).cuda().to(torch.float16)
    installed, meta = install_alignquant(model, artifact, "cuda")  # reference scale mode: 16 x 64 tiles
    assert len(installed) == 14 and meta["projection_group_count"] == 8
    inputs = {k: torch.from_numpy(io[f"x{k}"]).cuda() for k in (128, 256)}
    for index, layer in enumerate(model.model.layers):
        reset_alignquant_state(model)
        for short in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                      "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"):
            module = layer.get_submodule(short)
            got = module(inputs[module.in_features])
            ext.device_status()
            want = io[f"model.layers.{index}.{short}/y"]
            if module.bias is not None:
                want = want + module.bias.float().cpu().numpy()
            assert got.dtype == torch.float16
            # fp16 result (2^-11 relative) on top of the rel 1e-3 / abs 1e-2 contract
            assert np.allclose(got.float().cpu().numpy(), want, rtol=2e-3, atol=1e-2), (index, short)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 8, 40])
def test_fused_norm_feeds_the_projection_group(rows, dtype):
    """AlignQuantRMSNorm: the normalised tensor is the stock module's (to one rounding step of the
    dtype, the sum of squares being taken in FP64), the int8 rows it leaves are exactly the
    quantizer's for that tensor, and the projections give the same bits whether they take them or
    quantize the tensor themselves."""
    from alignquant_b200.kernels.cuda import extension as ext
    from alignquant_b200.quantization.model import AlignQuantRMSNorm, install_alignquant, reset_alignquant_state

    ext.load_extension()
    artifact, _ = _artifact()
    model = _Tiny(norms=True).cuda().to(dtype)
    _, meta = install_alignquant(model, artifact, "cuda", scale_mode="token", fuse_norms=True)
    assert meta["fused_norm_count"] == 2
    layer = model.model.layers[0]
    assert isinstance(layer.input_layernorm, AlignQuantRMSNorm)
    gen = torch.Generator(device="cuda").manual_seed(rows)
    x = (torch.randn((rows, 128), generator=gen, device="cuda") * 3).to(dtype)
    for norm, members in ((layer.input_layernorm, (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj)),
                          (layer.post_attention_layernorm, (layer.mlp.gate_proj, layer.mlp.up_proj))):
        reset_alignquant_state(model)
        y = norm(x)
        want = norm.original(x)
        step = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7  # one unit in the last place, relative
        assert torch.allclose(y.float(), want.float(), rtol=2 * step, atol=1e-6)
        xq, scales = y._alignquant_quantized
        ref_q, ref_s = ext.alignquant_activation_quantize_cuda(y, None, scale_mode="token")
        assert torch.equal(xq, ref_q) and torch.equal(scales, ref_s)
        fused = [m(y) for m in members]
        ext.device_status()
        fresh_input = y.clone()  # no int8 rows attached: the group launches its own quantizer
        fresh = [m(fresh_input) for m in members]
        ext.device_status()
        for a, b in zip(fused, fresh):
            assert torch.equal(a, b)
