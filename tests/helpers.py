"""Helpers shared by the GPU parity tests: synthetic layers on the device and the
numpy model of the prepared weight image."""

from __future__ import annotations

import numpy as np
import torch

from oracle import alignquant_oracle as oc


def expected_image(states: np.ndarray, tiles: np.ndarray, scales: np.ndarray):
    """(records uint32/float32 pairs, payload bytes) the re-layout must produce."""
    n_j, n_k = states.shape
    offsets, flags, rec_scales, chunks = [], [], [], []
    units = 0
    for j in range(n_j):
        for k in range(n_k):
            t = tiles[j, k]  # [n, kk]
            if states[j, k] == oc.P4:
                v = t.reshape(64, 2, 2, 16).astype(np.uint8)  # [n][h][half][i]
                byte = (v[:, :, 0, :] & 15) | ((v[:, :, 1, :] & 15) << 4)
                chunks.append(np.ascontiguousarray(byte).reshape(-1))
                offsets.append(units)
                flags.append(1)
                rec_scales.append(np.float32(scales[j, k]) * np.float32(0.0625))
                units += 1
            else:
                v = t.reshape(64, 4, 16)  # [n][c][i]
                out = np.empty_like(v)
                n = np.arange(64)
                for c in range(4):
                    out[n, c ^ ((n >> 1) & 3)] = v[n, c]
                chunks.append(out.reshape(-1).view(np.uint8))
                offsets.append(units)
                flags.append(0)
                rec_scales.append(np.float32(scales[j, k]))
                units += 2
    word = np.asarray(offsets, dtype=np.uint32) | (np.asarray(flags, dtype=np.uint32) << 31)
    return word, np.asarray(rec_scales, dtype=np.float32), np.concatenate(chunks)


def to_cuda(packed: dict, device="cuda") -> dict:
    return {k: torch.from_numpy(np.ascontiguousarray(v)).to(device) for k, v in packed.items()}


def prepare_layer(packed: dict, n_k: int, device="cuda"):
    from alignquant_b200.kernels.cuda.extension import prepare_weights

    t = to_cuda(packed, device)
    weights = prepare_weights(
        t["state_bits"], t["w4_payload"], t["w4_scales"], t["w8_payload"], t["w8_scales"],
        t["w4_row_offsets"], t["w8_row_offsets"], n_k=n_k,
    )
    return weights, t


def torch_activation(x: np.ndarray, dtype: torch.dtype, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x.astype(np.float32))).to(device=device, dtype=dtype)


def forced_layer(n: int, k: int, seed: int, fraction: float):
    """synthetic_layer with an exact all-W4 (1.0) / all-W8 (0.0) / mixed map."""
    return oc.synthetic_layer(n, k, seed, w4_fraction=fraction)


def planned_fp32(ext, xq_np, a_mk, tiles, scales, m, n_j, n_k, **plan_args):
    """FP32 result in the summation order the library reports for this problem."""
    plan = ext.linear_plan(m, n_j, n_k, **plan_args)
    if plan["kernel"] == 2:
        return oc.linear_fp32_ranges_c(xq_np, a_mk, tiles, scales, plan["splits"], plan["workers"])
    # the GEMM adds a tile with one fused multiply-add unless the library is told otherwise
    fused = plan["kernel"] == 1 and not ext.gemm_rounding_is_separate()
    return oc.linear_fp32_c(xq_np, a_mk, tiles, scales, plan["splits"], plan["workers"], fused=fused)
