"""The packed W4/W8 replacement-artifact format (byte-for-byte the reference's).

On-disk contract (reference: alignquant/quantization/artifact.py:19-31, 62-128,
131-234, 392-439): one safetensors shard per module with seven tensors --
``state_bits`` (LSB-first bitmap over flattened (j, k), 1 = W4), ``w4_payload``
``[T4, 64, 32]`` uint8 (Layout-B order, two values per byte, low nibble first),
``w4_scales`` ``[T4]`` float32, ``w8_payload`` ``[T8, 64, 64]`` int8 (Layout-B),
``w8_scales`` ``[T8]`` float32 and two ``[n_j + 1]`` int32 row-offset prefixes --
plus ``manifest.json`` / ``manifest.sha256`` with per-file and per-tensor digests.

The packer here is vectorised torch code that runs on any device; it is used to
build synthetic layers on the GPU and by the tests.  Building artifacts from a
calibrated model stays with the reference's offline tools.
"""

from __future__ import annotations

import hashlib
import json
import math
from collections.abc import Mapping
from functools import lru_cache
from pathlib import Path
from typing import Any

import torch

P4 = 4
P8 = 8
REPLACEMENT_ARTIFACT_SCHEMA = "alignquant_w4w8_a8_v3"
REPLACEMENT_ARTIFACT_VERSION = 3
REPLACEMENT_TENSOR_NAMES = (
    "state_bits",
    "w4_payload",
    "w4_scales",
    "w8_payload",
    "w8_scales",
    "w4_row_offsets",
    "w8_row_offsets",
)


@lru_cache(maxsize=None)
def _layout_b_offsets_cpu() -> torch.Tensor:
    k = torch.arange(64, dtype=torch.int64).view(64, 1)
    n = torch.arange(64, dtype=torch.int64).view(1, 64)
    k16, quad = k // 16, n // 4
    t = (k16 % 2) + 2 * (n % 4)
    vector = 8 * (k16 // 2) + 4 * (t // 4) + ((t % 4) ^ (quad % 4))
    return (256 * quad + 16 * vector + k % 16).contiguous()


def layout_b_offsets(*, device: torch.device | str | None = None) -> torch.Tensor:
    """Physical byte offset of logical element [k, n] of a 64x64 tile (artifact.py:62-73).

    Every aligned 16-byte vector holds 16 consecutive k of one output column; a
    256-byte block holds four columns; the XOR is the shared-memory bank swizzle of
    the SM80 tensor-core operand layout the format was designed for.
    """
    offsets = _layout_b_offsets_cpu()
    return offsets.to(device) if device is not None else offsets.clone()


def _to_physical(logical_kn: torch.Tensor) -> torch.Tensor:
    offsets = layout_b_offsets(device=logical_kn.device).reshape(-1)
    gather = torch.empty_like(offsets)
    gather[offsets] = torch.arange(4096, device=offsets.device)
    flat = logical_kn.reshape(*logical_kn.shape[:-2], 4096)
    return flat[..., gather].reshape(logical_kn.shape)


def unpack_signed_int4(packed: torch.Tensor) -> torch.Tensor:
    """Low-nibble-first signed INT4 -> INT8 (artifact.py:85-100)."""
    if packed.dtype != torch.uint8:
        raise TypeError(f"Packed W4 payload must be uint8, got {packed.dtype}.")
    wide = packed.to(torch.int16)
    pair = torch.stack((wide & 0xF, (wide >> 4) & 0xF), dim=-1)
    pair = torch.where(pair >= 8, pair - 16, pair)
    return pair.reshape(*packed.shape[:-1], packed.shape[-1] * 2).to(torch.int8).contiguous()


def pack_w4w8_state_bits(states: torch.Tensor) -> torch.Tensor:
    """[n_j, n_k] map of P4/P8 -> LSB-first bitmap with 1 = W4 (artifact.py:103-116)."""
    flat = torch.as_tensor(states, dtype=torch.uint8).reshape(-1)
    if not bool(torch.all((flat == P4) | (flat == P8))):
        raise ValueError("Weight states may contain only P4 and P8.")
    total = int(flat.numel())
    padded = torch.zeros(math.ceil(total / 8) * 8, dtype=torch.int32, device=flat.device)
    padded[:total] = (flat == P4).to(torch.int32)
    weights = (1 << torch.arange(8, dtype=torch.int32, device=flat.device))
    return (padded.view(-1, 8) * weights).sum(dim=1).to(torch.uint8).contiguous()


def unpack_w4w8_state_bits(state_bits: torch.Tensor, *, n_j: int, n_k: int) -> torch.Tensor:
    """Inverse of :func:`pack_w4w8_state_bits` (artifact.py:119-128)."""
    total = int(n_j) * int(n_k)
    packed = torch.as_tensor(state_bits, dtype=torch.uint8).reshape(-1)
    if int(packed.numel()) != math.ceil(total / 8):
        raise ValueError(f"Expected {math.ceil(total / 8)} state bytes.")
    shifts = torch.arange(8, dtype=torch.int32, device=packed.device)
    bits = ((packed.to(torch.int32)[:, None] >> shifts) & 1).reshape(-1)[:total]
    return torch.where(bits.bool(), P4, P8).to(torch.uint8).view(int(n_j), int(n_k))


def pack_w4w8_replacement_module(
    *,
    states: torch.Tensor,
    qweight4: torch.Tensor,
    weight_scale4: torch.Tensor,
    qweight8: torch.Tensor,
    weight_scale8: torch.Tensor,
) -> dict[str, torch.Tensor]:
    """Keep one packed payload and one scale per tile (artifact.py:131-199).

    ``qweight4`` / ``qweight8`` are the candidate tiles ``[n_j, n_k, 64(out), 64(in)]``,
    ``weight_scale4`` / ``weight_scale8`` their ``[n_j, n_k]`` scales.  Tiles of one row
    are contiguous in k order inside each arena, rows follow each other, so the arena
    order is simply the row-major order of the selected tiles.
    """
    device = qweight4.device
    state_map = torch.as_tensor(states, dtype=torch.uint8).to(device)
    if state_map.ndim != 2:
        raise ValueError(f"states must be [n_j,n_k], got {tuple(state_map.shape)}.")
    n_j, n_k = map(int, state_map.shape)
    expected = (n_j, n_k, 64, 64)
    q4 = qweight4.detach().to(torch.int8)
    q8 = qweight8.detach().to(device=device, dtype=torch.int8)
    s4 = weight_scale4.detach().to(device=device, dtype=torch.float32)
    s8 = weight_scale8.detach().to(device=device, dtype=torch.float32)
    if tuple(q4.shape) != expected or tuple(q8.shape) != expected:
        raise ValueError(f"Candidate weights must be {expected}.")
    if tuple(s4.shape) != (n_j, n_k) or tuple(s8.shape) != (n_j, n_k):
        raise ValueError("Candidate scales must be [n_j,n_k].")
    if bool((q4 < -8).any()) or bool((q4 > 7).any()):
        raise ValueError("W4 values must be signed INT4 in [-8,7].")
    if not bool(torch.isfinite(s4).all() and torch.isfinite(s8).all()):
        raise ValueError("Weight scales must be finite.")
    if bool((s4 <= 0).any() or (s8 <= 0).any()):
        raise ValueError("Weight scales must be positive.")

    mask4 = (state_map == P4).reshape(-1)
    mask8 = ~mask4
    physical4 = _to_physical(q4.reshape(-1, 64, 64)[mask4].transpose(1, 2))
    physical8 = _to_physical(q8.reshape(-1, 64, 64)[mask8].transpose(1, 2))
    nibbles = physical4.to(torch.int16) & 0xF
    w4_payload = (nibbles[..., 0::2] | (nibbles[..., 1::2] << 4)).to(torch.uint8)
    zero = torch.zeros(1, dtype=torch.int64, device=device)
    per_row4 = (state_map == P4).sum(dim=1)
    per_row8 = (state_map == P8).sum(dim=1)
    return {
        "state_bits": pack_w4w8_state_bits(state_map),
        "w4_payload": w4_payload.reshape(-1, 64, 32).contiguous(),
        "w4_scales": s4.reshape(-1)[mask4].contiguous(),
        "w8_payload": physical8.reshape(-1, 64, 64).contiguous(),
        "w8_scales": s8.reshape(-1)[mask8].contiguous(),
        "w4_row_offsets": torch.cat((zero, per_row4.cumsum(0))).to(torch.int32),
        "w8_row_offsets": torch.cat((zero, per_row8.cumsum(0))).to(torch.int32),
    }


def validate_w4w8_replacement_module(
    tensors: Mapping[str, torch.Tensor], *, n_j: int, n_k: int
) -> torch.Tensor:
    """Validate one selected-payload shard; returns its state map (artifact.py:202-234)."""
    if set(tensors) != set(REPLACEMENT_TENSOR_NAMES):
        raise RuntimeError("Unexpected replacement tensors.")
    states = unpack_w4w8_state_bits(tensors["state_bits"].cpu(), n_j=n_j, n_k=n_k)
    count4 = int((states == P4).sum())
    count8 = int((states == P8).sum())
    expected = {
        "w4_payload": ((count4, 64, 32), torch.uint8),
        "w4_scales": ((count4,), torch.float32),
        "w8_payload": ((count8, 64, 64), torch.int8),
        "w8_scales": ((count8,), torch.float32),
        "w4_row_offsets": ((int(n_j) + 1,), torch.int32),
        "w8_row_offsets": ((int(n_j) + 1,), torch.int32),
    }
    for name, (shape, dtype) in expected.items():
        tensor = tensors[name]
        if tuple(tensor.shape) != shape or tensor.dtype != dtype:
            raise RuntimeError(f"Invalid {name}: {tuple(tensor.shape)} {tensor.dtype}.")
    zero = torch.zeros(1, dtype=torch.int64)
    for precision, name in ((P4, "w4_row_offsets"), (P8, "w8_row_offsets")):
        want = torch.cat((zero, (states == precision).sum(1).cumsum(0)))
        if not torch.equal(tensors[name].detach().cpu().to(torch.int64), want):
            raise RuntimeError(f"Invalid {name}.")
    for name in ("w4_scales", "w8_scales"):
        scales = tensors[name]
        if not bool(torch.isfinite(scales).all()) or bool((scales <= 0).any()):
            raise RuntimeError(f"Invalid {name}.")
    return states


def shard_w4w8_replacement_module(
    tensors: Mapping[str, torch.Tensor],
    *,
    n_j: int,
    n_k: int,
    rows: tuple[int, int] | None = None,
    cols: tuple[int, int] | None = None,
) -> dict[str, torch.Tensor]:
    """The seven tensors of the sub-layer made of tile rows ``rows`` and tile columns ``cols``.

    Tensor-parallel sharding happens on tile boundaries: a column-parallel projection keeps
    a range of tile rows (output features), a row-parallel one a range of tile columns
    (input features).  Precision bits, payloads and scales are per tile, so the shard is an
    exact sub-selection -- nothing is re-quantized.  Arena order stays (j, k) row-major.
    """
    j0, j1 = rows if rows is not None else (0, int(n_j))
    k0, k1 = cols if cols is not None else (0, int(n_k))
    if not (0 <= j0 < j1 <= n_j and 0 <= k0 < k1 <= n_k):
        raise ValueError(f"Invalid shard rows={rows} cols={cols} for a {n_j}x{n_k} tile grid.")
    states = unpack_w4w8_state_bits(tensors["state_bits"].cpu(), n_j=n_j, n_k=n_k)
    is4 = (states == P4).reshape(-1)
    # arena index of every tile inside its own precision's arena
    index4 = torch.cumsum(is4.to(torch.int64), 0) - 1
    index8 = torch.cumsum((~is4).to(torch.int64), 0) - 1
    keep = torch.zeros((n_j, n_k), dtype=torch.bool)
    keep[j0:j1, k0:k1] = True
    keep = keep.reshape(-1)
    take4 = index4[keep & is4]
    take8 = index8[keep & ~is4]
    sub_states = states[j0:j1, k0:k1].contiguous()
    zero = torch.zeros(1, dtype=torch.int64)
    device = tensors["w4_payload"].device
    return {
        "state_bits": pack_w4w8_state_bits(sub_states).to(tensors["state_bits"].device),
        "w4_payload": tensors["w4_payload"][take4.to(device)].contiguous(),
        "w4_scales": tensors["w4_scales"][take4.to(device)].contiguous(),
        "w8_payload": tensors["w8_payload"][take8.to(device)].contiguous(),
        "w8_scales": tensors["w8_scales"][take8.to(device)].contiguous(),
        "w4_row_offsets": torch.cat((zero, (sub_states == P4).sum(1).cumsum(0))).to(torch.int32).to(device),
        "w8_row_offsets": torch.cat((zero, (sub_states == P8).sum(1).cumsum(0))).to(torch.int32).to(device),
    }


def _sha256_bytes(value: bytes) -> str:
    return hashlib.sha256(value).hexdigest()


def _file_sha256(path: Path) -> str:
    digest = hashlib.sha256()
    with path.open("rb") as handle:
        while chunk := handle.read(8 * 1024 * 1024):
            digest.update(chunk)
    return digest.hexdigest()


def _tensor_sha256(tensor: torch.Tensor) -> str:
    return _sha256_bytes(tensor.detach().cpu().contiguous().numpy().tobytes())


def load_artifact(root: str | Path, *, device: str | torch.device = "cpu") -> dict[str, Any]:
    """Load and fully validate one replacement artifact directory (artifact.py:392-439).

    Checks the manifest digest, schema and version, every shard's file digest, every
    tensor's shape, dtype, offsets, scales and digest, the per-module tile counts and
    the artifact totals.  Returns ``{"root", "manifest", "modules"}``.
    """
    from safetensors.torch import load_file

    target = Path(root).expanduser().resolve()
    manifest_text = (target / "manifest.json").read_text(encoding="utf-8")
    recorded = (target / "manifest.sha256").read_text(encoding="utf-8").split()[0]
    if _sha256_bytes(manifest_text.encode()) != recorded:
        raise RuntimeError("Replacement manifest digest mismatch.")
    manifest = json.loads(manifest_text)
    if (
        manifest.get("schema") != REPLACEMENT_ARTIFACT_SCHEMA
        or manifest.get("version") != REPLACEMENT_ARTIFACT_VERSION
    ):
        raise ValueError("Unsupported W4/W8 replacement artifact.")
    modules: dict[str, dict[str, torch.Tensor]] = {}
    totals = {"w4": 0, "w8": 0, "tiles": 0, "tensor_bytes": 0, "file_bytes": 0}
    for row in manifest["modules"]:
        shard = target / row["file"]
        if _file_sha256(shard) != row["file_sha256"]:
            raise RuntimeError(f"Replacement shard digest mismatch: {row['file']}.")
        tensors = load_file(shard, device=str(device))
        validate_w4w8_replacement_module(tensors, n_j=int(row["n_j"]), n_k=int(row["n_k"]))
        for name in REPLACEMENT_TENSOR_NAMES:
            if _tensor_sha256(tensors[name]) != row["tensor_sha256"][name]:
                raise RuntimeError(f"Tensor digest mismatch for {row['layer_name']}/{name}.")
        count4 = int(tensors["w4_scales"].numel())
        count8 = int(tensors["w8_scales"].numel())
        if row["tile_counts"] != {"w4": count4, "w8": count8, "total": count4 + count8}:
            raise RuntimeError(f"Tile count mismatch for {row['layer_name']}.")
        modules[str(row["layer_name"])] = tensors
        totals["w4"] += count4
        totals["w8"] += count8
        totals["tiles"] += count4 + count8
        totals["tensor_bytes"] += sum(int(t.numel()) * int(t.element_size()) for t in tensors.values())
        totals["file_bytes"] += int(shard.stat().st_size)
    for name, value in totals.items():
        if int(manifest["totals"][name]) != value:
            raise RuntimeError(f"Artifact total mismatch: {name}.")
    return {"root": target, "manifest": manifest, "modules": modules}


__all__ = [
    "P4",
    "P8",
    "REPLACEMENT_ARTIFACT_SCHEMA",
    "REPLACEMENT_ARTIFACT_VERSION",
    "REPLACEMENT_TENSOR_NAMES",
    "layout_b_offsets",
    "load_artifact",
    "pack_w4w8_replacement_module",
    "pack_w4w8_state_bits",
    "shard_w4w8_replacement_module",
    "unpack_signed_int4",
    "unpack_w4w8_state_bits",
    "validate_w4w8_replacement_module",
]
