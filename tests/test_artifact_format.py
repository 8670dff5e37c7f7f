"""The package's own packer/unpacker against the reference-generated fixture (CPU)."""

from __future__ import annotations

import numpy as np
import torch

from alignquant_b200.quantization import artifact as fmt
from oracle import alignquant_oracle as oc


def test_packer_matches_reference_fixture(golden_dir):
    g = dict(np.load(golden_dir / "format.npz"))
    assert np.array_equal(fmt.layout_b_offsets().numpy(), g["layout_b_offsets"])
    packed = fmt.pack_w4w8_replacement_module(
        states=torch.from_numpy(g["states"]), qweight4=torch.from_numpy(g["q4"]),
        weight_scale4=torch.from_numpy(g["s4"]), qweight8=torch.from_numpy(g["q8"]),
        weight_scale8=torch.from_numpy(g["s8"]),
    )
    for name in fmt.REPLACEMENT_TENSOR_NAMES:
        assert packed[name].dtype == torch.from_numpy(g[f"packed_{name}"]).dtype, name
        assert np.array_equal(packed[name].numpy(), g[f"packed_{name}"]), name
    n_j, n_k = g["states"].shape
    states = fmt.validate_w4w8_replacement_module(packed, n_j=n_j, n_k=n_k)
    assert np.array_equal(states.numpy(), g["states"])


def test_state_bits_and_int4_roundtrip():
    gen = torch.Generator().manual_seed(0)
    for n_j, n_k in ((1, 1), (2, 5), (7, 9)):
        states = torch.where(torch.rand((n_j, n_k), generator=gen) < 0.5, fmt.P4, fmt.P8).to(torch.uint8)
        bits = fmt.pack_w4w8_state_bits(states)
        assert np.array_equal(bits.numpy(), oc.pack_state_bits(states.numpy()))
        assert torch.equal(fmt.unpack_w4w8_state_bits(bits, n_j=n_j, n_k=n_k), states)
    packed = torch.randint(0, 256, (3, 64, 32), generator=gen, dtype=torch.uint8)
    assert np.array_equal(fmt.unpack_signed_int4(packed).numpy(), oc.unpack_signed_int4(packed.numpy()))


def test_synthetic_module_is_valid_and_sixty_percent_w4():
    from alignquant_b200.synthetic import synthetic_module_tensors

    tensors = synthetic_module_tensors(192, 320, seed=4, device="cpu")
    states = fmt.validate_w4w8_replacement_module(tensors, n_j=3, n_k=5)
    assert int((states == fmt.P4).sum()) == 9
    _, tiles, scales = oc.unpack_module({k: v.numpy() for k, v in tensors.items()}, 3, 5)
    assert np.abs(tiles[states.numpy() == fmt.P4]).max() <= 8
    assert scales.min() > 0
