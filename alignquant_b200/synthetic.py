"""Seeded synthetic layers and activations of the benchmark configurations.

Weights are fp16 N(0, 0.02) cut into 64x64 tiles; a seeded random 60 % of the tiles
are W4 (symmetric, scale = tile absmax / 7) and the rest W8 (absmax / 127), scales
rounded to fp16 and stored as float32; rounding is half-to-even with clamping, the
rule of the reference's ``quantize_tiles`` (alignquant/quantization/exact.py:220-234).
Activations are N(0, 1) with a seeded 0.5 % of the channels scaled by 20.  Everything
runs in torch on the chosen device so that whole models can be built on the GPU.
"""

from __future__ import annotations

import torch

from alignquant_b200.quantization.artifact import P4, P8, pack_w4w8_replacement_module


def synthetic_module_tensors(
    n: int, k: int, seed: int, *, device: torch.device | str = "cuda", w4_fraction: float = 0.6,
    weight_std: float = 0.02,
) -> dict[str, torch.Tensor]:
    """The seven packed artifact tensors of one seeded random ``[n, k]`` layer."""
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(int(seed))
    n_j, n_k = n // 64, k // 64
    weight = (torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * weight_std).half()
    tiles = weight.float().view(n_j, 64, n_k, 64).permute(0, 2, 1, 3)
    total = n_j * n_k
    order = torch.randperm(total, generator=gen, device=device)
    states = torch.full((total,), P8, dtype=torch.uint8, device=device)
    states[order[: int(round(w4_fraction * total))]] = P4
    states = states.view(n_j, n_k)
    absmax = tiles.abs().amax(dim=(-2, -1)).double()
    floor = 2.0 ** -24
    s4 = (absmax / 7.0).half().float().clamp_min(floor)
    s8 = (absmax / 127.0).half().float().clamp_min(floor)
    q4 = torch.round(tiles.double() / s4.double()[..., None, None]).clamp(-8, 7).to(torch.int8)
    q8 = torch.round(tiles.double() / s8.double()[..., None, None]).clamp(-128, 127).to(torch.int8)
    return pack_w4w8_replacement_module(
        states=states, qweight4=q4, weight_scale4=s4, qweight8=q8, weight_scale8=s8
    )


def synthetic_activation(
    m: int, k: int, seed: int, *, dtype: torch.dtype = torch.float16, device: torch.device | str = "cuda",
    outlier_fraction: float = 0.005,
) -> torch.Tensor:
    """N(0,1) activations ``[m, k]`` with a seeded 0.5 % of channels scaled x20."""
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(int(seed))
    x = torch.randn((m, k), generator=gen, device=device, dtype=torch.float32)
    count = max(1, int(round(outlier_fraction * k)))
    columns = torch.randperm(k, generator=gen, device=device)[:count]
    x[:, columns] *= 20.0
    return x.to(dtype)


def algorithmic_weight_bytes(tensors: dict[str, torch.Tensor]) -> int:
    """Bytes of a layer in the artifact format: payloads, scales, bitmap and offsets."""
    return sum(int(t.numel()) * int(t.element_size()) for t in tensors.values())
