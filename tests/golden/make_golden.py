"""Generate the golden fixtures in this directory from the reference's own code.

Run where the reference checkout is available (it is not available on the GPU
machines, which is why the outputs are committed):

    python tests/golden/make_golden.py /path/to/AlignQuant

Every array below is produced by functions of the reference package
(``alignquant.quantization.exact`` and ``alignquant.quantization.artifact``);
nothing from this repository is imported, so the fixtures are independent of
the code they check.  The linear cases follow the recipe of the reference's CPU
dequantize-and-matmul (alignquant/quantization/calibration.py:552-572) with the
per-tile selected W4/W8 payload.  ``artifact_tiny/`` is a whole artifact directory
written by the reference's ``build_artifact`` (alignquant/quantization/artifact.py:271-389)
for a two-layer toy decoder, the way ``alignquant/build.py:62-100`` feeds it, with
precision bitmaps and V/U seeds cut from the reference's Llama-3.2-3B preset;
``artifact_tiny_io.npz`` holds inputs and the reference's FP64 outputs per module.
"""

from __future__ import annotations

import json
import shutil
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch


def main(reference_root: str) -> None:
    sys.dont_write_bytecode = True
    sys.path.insert(0, reference_root)
    from alignquant.quantization import artifact as ra
    from alignquant.quantization import exact as rx

    out_dir = Path(__file__).resolve().parent
    gen = torch.Generator().manual_seed(20250601)

    # ---- transform metadata and matrices (exact.py:16-71) -------------------
    seeds = [-1, 0, 1, 2, 7, 123]
    meta = torch.stack([rx.structured_transform_metadata(s) for s in seeds])
    mats = torch.stack([rx.structured_transform_matrix(s) for s in seeds])
    np.savez_compressed(
        out_dir / "transforms.npz",
        seeds=np.asarray(seeds, np.int64),
        metadata=meta.numpy(),
        matrices=mats.numpy(),
    )

    # ---- format: pack_w4w8_replacement_module (artifact.py:131-199) ---------
    n_j, n_k = 3, 5
    states = torch.where(torch.rand((n_j, n_k), generator=gen) < 0.6, ra.P4, ra.P8).to(torch.uint8)
    states[0, 0] = ra.P8
    states[0, 1] = ra.P4
    q4 = torch.randint(-8, 8, (n_j, n_k, 64, 64), generator=gen, dtype=torch.int8)
    q8 = torch.randint(-128, 128, (n_j, n_k, 64, 64), generator=gen, dtype=torch.int8)
    s4 = torch.rand((n_j, n_k), generator=gen) * 0.01 + 1e-4
    s8 = torch.rand((n_j, n_k), generator=gen) * 0.001 + 1e-5
    packed = ra.pack_w4w8_replacement_module(states=states, qweight4=q4, weight_scale4=s4, qweight8=q8, weight_scale8=s8)
    ra.validate_w4w8_replacement_module(packed, n_j=n_j, n_k=n_k)
    np.savez_compressed(
        out_dir / "format.npz",
        states=states.numpy(), q4=q4.numpy(), q8=q8.numpy(),
        s4=s4.to(torch.float32).numpy(), s8=s8.to(torch.float32).numpy(),
        layout_b_offsets=ra.layout_b_offsets().numpy(),
        **{f"packed_{k}": v.numpy() for k, v in packed.items()},
    )

    # ---- weight quantization (exact.py:165-241) ------------------------------
    w = (torch.randn((2, 3, 64, 64), generator=gen, dtype=torch.float64) * 0.02)
    w[1, 2] = 0.0  # all-zero tile takes the scale floor
    out = {"tiles": w.numpy()}
    for bits in (4, 8):
        scales = rx.mse_scales(w, bits=bits)
        out[f"mse_scales{bits}"] = scales.numpy()
        out[f"q{bits}"] = rx.quantize_tiles(w, scales, bits=bits).numpy()
    np.savez_compressed(out_dir / "weight_quant.npz", **out)

    # ---- activation quantization (exact.py:120-135, 244-274) ------------------
    m, k = 32, 192
    x = torch.randn((m, k), generator=gen, dtype=torch.float32)
    x[:, 5] *= 20.0
    x[3, :64] = 0.0
    x = x.to(torch.float16)
    for name, v_seeds in (("identity", [-1, -1, -1]), ("mixed", [0, 3, -1])):
        tiles = x.reshape(m, k // 64, 64).permute(1, 0, 2)  # [K, M, 64]
        transformed = rx.transform_activation_tiles(tiles, v_seeds=v_seeds)
        grouped = transformed.reshape(k // 64, m // 16, 16, 64)
        q, scales = rx.a8_endpoint_quantize_tiles(grouped)
        np.savez_compressed(
            out_dir / f"act_quant_{name}.npz",
            x=x.numpy(), v_seeds=np.asarray(v_seeds),
            v_metadata=torch.stack([rx.structured_transform_metadata(s) for s in v_seeds]).numpy(),
            transformed=transformed.permute(1, 0, 2).reshape(m, k).numpy(),
            q=q.reshape(k // 64, m, 64).permute(1, 0, 2).reshape(m, k).numpy(),
            scales=scales.permute(1, 0).contiguous().numpy(),  # [M/16, K/64] FP64
        )

    # ---- full mixed linear (calibration.py:552-572 recipe) --------------------
    cases = (
        ("linear_identity", 16, 128, 128, None, None),
        ("linear_m1", 1, 192, 64, None, None),
        ("linear_transformed", 32, 192, 128, [0, 5, -1], [2, -1]),
    )
    for name, m, k, n, v_seeds, u_seeds in cases:
        n_j, n_k = n // 64, k // 64
        v_seeds = v_seeds or [-1] * n_k
        u_seeds = u_seeds or [-1] * n_j
        weight = (torch.randn((n, k), generator=gen, dtype=torch.float32) * 0.02).to(torch.float16)
        wt = rx.transform_weight_tiles(rx.split_weight_tiles(weight), v_seeds=v_seeds, u_seeds=u_seeds)
        q4, s4 = rx.mse_quantize_tiles(wt, bits=4)
        q8, s8 = rx.mse_quantize_tiles(wt, bits=8)
        states = torch.where(torch.rand((n_j, n_k), generator=gen) < 0.6, ra.P4, ra.P8).to(torch.uint8)
        states.view(-1)[0] = ra.P4
        states.view(-1)[-1] = ra.P8
        packed = ra.pack_w4w8_replacement_module(states=states, qweight4=q4, weight_scale4=s4, qweight8=q8, weight_scale8=s8)
        sel_q = torch.where((states == ra.P4)[:, :, None, None], q4, q8)
        sel_s = torch.where(states == ra.P4, s4.to(torch.float32), s8.to(torch.float32))

        x = torch.randn((m, k), generator=gen, dtype=torch.float32)
        x[:, 7] *= 20.0
        x = x.to(torch.float16)
        rows = 16 * ((m + 15) // 16)
        xp = torch.zeros((rows, k), dtype=x.dtype)
        xp[:m] = x
        tiles = xp.reshape(rows, n_k, 64).permute(1, 0, 2)
        transformed = rx.transform_activation_tiles(tiles, v_seeds=v_seeds)
        aq, a_s = rx.a8_endpoint_quantize_tiles(transformed.reshape(n_k, rows // 16, 16, 64))
        a_s32 = a_s.to(torch.float32)
        a8 = rx.reconstruct_tiles(aq, a_s32, dtype=torch.float64).reshape(n_k, rows, 64).permute(1, 0, 2)[:m]
        wd = rx.reconstruct_tiles(sel_q, sel_s, dtype=torch.float64)
        y_t = torch.einsum("mki,jkoi->mjo", a8, wd)
        y = rx.inverse_output_tiles(y_t.permute(1, 0, 2), u_seeds=u_seeds).permute(1, 0, 2).reshape(m, n)
        aq_rows = aq.reshape(n_k, rows, 64).permute(1, 0, 2).reshape(rows, k)[:m]
        acc = torch.einsum("mki,jkoi->mjko", aq_rows.reshape(m, n_k, 64).to(torch.int32), sel_q.to(torch.int32))
        np.savez_compressed(
            out_dir / f"{name}.npz",
            x=x.numpy(), v_seeds=np.asarray(v_seeds), u_seeds=np.asarray(u_seeds),
            v_metadata=torch.stack([rx.structured_transform_metadata(s) for s in v_seeds]).numpy(),
            u_metadata=torch.stack([rx.structured_transform_metadata(s) for s in u_seeds]).numpy(),
            states=states.numpy(), tiles=sel_q.numpy(), tile_scales=sel_s.numpy(),
            xq=aq_rows.numpy(),
            act_scales=a_s32.permute(1, 0).contiguous().numpy(),  # [rows/16, n_k] float32
            acc=acc.numpy().astype(np.int32),
            y_before_u=y_t.reshape(m, n).numpy(),
            y=y.numpy(),
            **{f"packed_{key}": value.numpy() for key, value in packed.items()},
        )
    # ---- a whole artifact directory through build_artifact (artifact.py:271-389) ----------
    preset = json.loads((Path(reference_root) / "alignquant" / "data" / "llama-3.2-3b-instruct.json").read_text())
    preset_rows = {row["name"]: row for row in preset["modules"]}
    toy_shapes = {
        "self_attn.q_proj": (256, 128), "self_attn.k_proj": (128, 128), "self_attn.v_proj": (128, 128),
        "self_attn.o_proj": (128, 256), "mlp.gate_proj": (256, 128), "mlp.up_proj": (256, 128),
        "mlp.down_proj": (128, 256),
    }
    shares_v_with = {"self_attn.k_proj": "self_attn.q_proj", "self_attn.v_proj": "self_attn.q_proj",
                     "mlp.up_proj": "mlp.gate_proj"}  # members of a fused group share the V seeds
    m = 5
    inputs = {128: None, 256: None}
    for k in inputs:
        x = torch.randn((m, k), generator=gen, dtype=torch.float32)
        x[:, 3] *= 20.0
        inputs[k] = x.to(torch.float16)
    modules, io = [], {f"x{k}": v.numpy() for k, v in inputs.items()}
    for layer in (0, 1):
        for short, (n, k) in toy_shapes.items():
            name = f"model.layers.{layer}.{short}"
            n_j, n_k = n // 64, k // 64
            row = preset_rows[name]
            # the first n_j * n_k bits of the preset's bitmap and the first seeds of its lists
            bitmap = bytes.fromhex(row["w4_state_bits_lsb_hex"])[: (n_j * n_k + 7) // 8]
            states = ra.unpack_w4w8_state_bits(torch.tensor(list(bitmap), dtype=torch.uint8), n_j=n_j, n_k=n_k)
            if name == "model.layers.1.mlp.down_proj":
                states = torch.full_like(states, ra.P4)  # an all-W4 module
            if name == "model.layers.1.self_attn.o_proj":
                states = torch.full_like(states, ra.P8)  # an all-W8 module
            v_row = preset_rows[f"model.layers.{layer}.{shares_v_with.get(short, short)}"]
            v_seeds = [int(v) for v in v_row["r5"]["v_seeds"][:n_k]]
            u_seeds = [int(v) for v in row["r5"]["u_seeds"][:n_j]]
            weight = (torch.randn((n, k), generator=gen, dtype=torch.float32) * 0.02).to(torch.float16)
            wt = rx.transform_weight_tiles(rx.split_weight_tiles(weight.to(torch.float64)), v_seeds=v_seeds, u_seeds=u_seeds)
            q4, s4 = rx.mse_quantize_tiles(wt, bits=4)
            q8, s8 = rx.mse_quantize_tiles(wt, bits=8)
            plan = SimpleNamespace(variant="R5", t_seed=-1, v_seeds=v_seeds, u_seeds=u_seeds)
            modules.append(SimpleNamespace(
                layer_name=name, weight_state_map=states, qweight4=q4.to(torch.int8), weight_scale4=s4.to(torch.float32),
                qweight8=q8.to(torch.int8), weight_scale8=s8.to(torch.float32), n_j=n_j, n_k=n_k, in_features=k,
                out_features=n, p4_codebook=None, plan=SimpleNamespace(normalized=lambda *, n_k, n_j, _p=plan: _p),
            ))
            # the module's output for the toy input (calibration.py:552-572 recipe, selected payload)
            sel_q = torch.where((states == ra.P4)[:, :, None, None], q4, q8)
            sel_s = torch.where(states == ra.P4, s4.to(torch.float32), s8.to(torch.float32))
            xp = torch.zeros((16, k), dtype=torch.float16)
            xp[:m] = inputs[k]
            transformed = rx.transform_activation_tiles(xp.reshape(16, n_k, 64).permute(1, 0, 2), v_seeds=v_seeds)
            aq, a_s = rx.a8_endpoint_quantize_tiles(transformed.reshape(n_k, 1, 16, 64))
            a8 = rx.reconstruct_tiles(aq, a_s.to(torch.float32), dtype=torch.float64).reshape(n_k, 16, 64).permute(1, 0, 2)[:m]
            wd = rx.reconstruct_tiles(sel_q, sel_s, dtype=torch.float64)
            y_t = torch.einsum("mki,jkoi->mjo", a8, wd)
            y = rx.inverse_output_tiles(y_t.permute(1, 0, 2), u_seeds=u_seeds).permute(1, 0, 2).reshape(m, n)
            io[f"{name}/y"] = y.numpy()
            io[f"{name}/v_seeds"] = np.asarray(v_seeds)
            io[f"{name}/u_seeds"] = np.asarray(u_seeds)
            io[f"{name}/states"] = states.numpy()
    artifact_dir = out_dir / "artifact_tiny"
    if artifact_dir.exists():
        shutil.rmtree(artifact_dir)
    ra.build_artifact(artifact_dir, modules=modules, model_identity={"id": "toy-decoder", "revision": "none", "loader": "none"})
    ra.load_artifact(artifact_dir)  # the reference's own loader accepts what it wrote
    np.savez_compressed(out_dir / "artifact_tiny_io.npz", **io)
    print("wrote", sorted(p.name for p in out_dir.glob("*.npz")), "and", artifact_dir.name)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
