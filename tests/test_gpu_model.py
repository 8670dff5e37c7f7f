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
