"""Structured-transform metadata of the runtime (the only numerics the hot path needs).

Everything else of the reference's ``alignquant/quantization/exact.py`` (MSE scale
search, calibration helpers) is offline tooling and stays with the reference.
"""

from __future__ import annotations

import torch

TILE = 64
IDENTITY_SEED = -1


def structured_transform_metadata(seed: int, *, device: torch.device | str | None = None) -> torch.Tensor:
    """``[4, 64]`` int32 rows (mode, permutation, left sign, right sign) of one transform seed.

    Seed -1 is the identity (mode 0), seed 0 the plain 64-point Hadamard transform, a
    positive seed draws the permutation and the two sign vectors from a CPU
    ``torch.Generator`` seeded with ``0x52464451 + seed`` -- the draw order (randperm,
    then two randint(0, 2) vectors mapped to -1/+1) fixes the artifact semantics and
    follows alignquant/quantization/exact.py:16-38 of the reference.
    """
    value = int(seed)
    if value < IDENTITY_SEED:
        raise ValueError(f"Transform seed must be >= {IDENTITY_SEED}, got {value}.")
    rows = torch.ones((4, TILE), dtype=torch.int32)
    rows[0] = 0 if value == IDENTITY_SEED else 1
    rows[1] = torch.arange(TILE, dtype=torch.int32)
    if value > 0:
        generator = torch.Generator(device="cpu").manual_seed(0x52464451 + value)
        rows[1] = torch.randperm(TILE, generator=generator).to(torch.int32)
        for index in (2, 3):
            bits = torch.randint(0, 2, (TILE,), generator=generator, dtype=torch.int64)
            rows[index] = (2 * bits - 1).to(torch.int32)
    return rows.to(device=device) if device is not None else rows


def metadata_stack(seeds, device: torch.device | str | None = None) -> torch.Tensor:
    """``[len(seeds), 4, 64]`` int32 stack of :func:`structured_transform_metadata`."""
    stack = torch.stack([structured_transform_metadata(int(seed)) for seed in seeds], dim=0).contiguous()
    return stack.to(device=device) if device is not None else stack


__all__ = ["IDENTITY_SEED", "TILE", "metadata_stack", "structured_transform_metadata"]
