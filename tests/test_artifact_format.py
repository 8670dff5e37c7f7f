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


# ---- a whole artifact directory written by the reference's build_artifact ---------------------


def test_load_artifact_accepts_the_reference_built_directory(golden_dir):
    """Manifest, shard and tensor digests, shapes, offsets and totals of tests/golden/artifact_tiny."""
    loaded = fmt.load_artifact(golden_dir / "artifact_tiny")
    io = dict(np.load(golden_dir / "artifact_tiny_io.npz"))
    manifest = loaded["manifest"]
    assert manifest["schema"] == fmt.REPLACEMENT_ARTIFACT_SCHEMA and len(manifest["modules"]) == 14
    fractions = {}
    for row in manifest["modules"]:
        name, n_j, n_k = row["layer_name"], int(row["n_j"]), int(row["n_k"])
        tensors = loaded["modules"][name]
        states = fmt.validate_w4w8_replacement_module(tensors, n_j=n_j, n_k=n_k)
        assert np.array_equal(states.numpy(), io[f"{name}/states"])
        assert row["r5"]["v_seeds"] == io[f"{name}/v_seeds"].tolist() and row["r5"]["u_seeds"] == io[f"{name}/u_seeds"].tolist()
        fractions[name] = float((states == fmt.P4).float().mean())
        # the oracle's unpacker reads the same tiles the package's validator accepted
        o_states, _, o_scales = oc.unpack_module({k: v.numpy() for k, v in tensors.items()}, n_j, n_k)
        assert np.array_equal(o_states, states.numpy()) and o_scales.min() > 0
    assert fractions["model.layers.1.mlp.down_proj"] == 1.0 and fractions["model.layers.1.self_attn.o_proj"] == 0.0
    seeds = [s for row in manifest["modules"] for s in row["r5"]["v_seeds"] + row["r5"]["u_seeds"]]
    assert sum(s != -1 for s in seeds) / len(seeds) > 0.9  # the preset's transforms are almost all non-identity


def test_load_artifact_fails_closed_on_a_flipped_byte(golden_dir, tmp_path):
    import shutil

    import pytest

    source = golden_dir / "artifact_tiny"
    # one byte of a shard's payload
    shard_copy = tmp_path / "shard"
    shutil.copytree(source, shard_copy)
    shard = sorted(shard_copy.glob("*.safetensors"))[3]
    data = bytearray(shard.read_bytes())
    data[-100] ^= 0x01
    shard.write_bytes(bytes(data))
    with pytest.raises(RuntimeError, match="shard digest mismatch"):
        fmt.load_artifact(shard_copy)
    # one byte of the manifest
    manifest_copy = tmp_path / "manifest"
    shutil.copytree(source, manifest_copy)
    text = (manifest_copy / "manifest.json").read_text()
    (manifest_copy / "manifest.json").write_text(text.replace('"n_j": 4', '"n_j": 5', 1))
    with pytest.raises(RuntimeError, match="manifest digest mismatch"):
        fmt.load_artifact(manifest_copy)
    # a shard whose file digest was "repaired" in the manifest still fails on the tensor digest
    tensor_copy = tmp_path / "tensor"
    shutil.copytree(source, tensor_copy)
    shard = sorted(tensor_copy.glob("*.safetensors"))[0]
    data = bytearray(shard.read_bytes())
    data[-1] ^= 0x80
    shard.write_bytes(bytes(data))
    import hashlib
    import json

    manifest = json.loads((tensor_copy / "manifest.json").read_text())
    manifest["modules"][0]["file_sha256"] = hashlib.sha256(bytes(data)).hexdigest()
    text = json.dumps(manifest, indent=2, sort_keys=True) + "\n"
    (tensor_copy / "manifest.json").write_text(text)
    (tensor_copy / "manifest.sha256").write_text(f"{hashlib.sha256(text.encode()).hexdigest()}  manifest.json\n")
    with pytest.raises((RuntimeError, ValueError)):
        fmt.load_artifact(tensor_copy)
