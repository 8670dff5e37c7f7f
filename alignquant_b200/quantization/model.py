"""Install and execute a W4/W8-A8 replacement artifact on the B200 kernels.

Same public surface as the reference's ``alignquant/quantization/model.py``
(``install_alignquant``, ``AlignQuantLinear``, ``reset_alignquant_state``,
``projection_groups``): q/k/v and gate/up projections of a decoder layer are fused into
one launch over their concatenated output tiles (members in alphabetical order, as in
the reference, model.py:27-46), the group output is computed once per activation and
handed out as column slices.

Differences, all behind keyword arguments with reference-compatible defaults:
  * the concatenated arenas are re-laid-out once into the prepared image the kernels
    stream (``prepare_weights``) and the raw arenas are dropped;
  * rows are never padded -- the kernels accept any row count;
  * ``scale_mode="token"`` selects per-row activation scales (only for identity V);
  * ``tp_rank`` / ``tp_size`` / ``process_group`` install a tile-aligned tensor-parallel
    shard: q/k/v/gate/up keep a range of tile rows per member (column parallel), o/down a
    range of tile columns (row parallel) followed by an all-reduce of the partial output;
  * every group knows the group that runs after it in a decoder layer (qkv -> o -> gate_up ->
    down -> next layer's qkv) and hands that group's weight image to the decode kernels as a
    look-ahead, so that the L2 cache fetches it while the current projection runs.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from pathlib import Path
from typing import Any

import torch
from torch import nn

from alignquant_b200.kernels.cuda import extension as _ext
from alignquant_b200.models.decoder import iter_target_linears
from alignquant_b200.quantization.artifact import (
    REPLACEMENT_TENSOR_NAMES,
    load_artifact,
    pack_w4w8_state_bits,
    shard_w4w8_replacement_module,
    unpack_w4w8_state_bits,
)
from alignquant_b200.quantization.exact import metadata_stack

COLUMN_PARALLEL_SUFFIXES = (".q_proj", ".k_proj", ".v_proj", ".gate_proj", ".up_proj")
ROW_PARALLEL_SUFFIXES = (".o_proj", ".down_proj")


def projection_groups(module_names: Sequence[str]) -> dict[str, tuple[str, ...]]:
    """Group q/k/v into ``<attn>.qkv`` and gate/up into ``<mlp>.gate_up``; others stay single."""
    groups: dict[str, list[str]] = {}
    for name in sorted({str(value) for value in module_names}):
        parent, _, leaf = name.rpartition(".")
        if parent.endswith(".self_attn") and leaf in ("q_proj", "k_proj", "v_proj"):
            key = parent + ".qkv"
        elif parent.endswith(".mlp") and leaf in ("gate_proj", "up_proj"):
            key = parent + ".gate_up"
        else:
            key = name
        groups.setdefault(key, []).append(name)
    result = {key: tuple(values) for key, values in sorted(groups.items())}
    for key, members in result.items():
        expected = 3 if key.endswith(".qkv") else 2 if key.endswith(".gate_up") else 1
        if len(members) != expected:
            raise ValueError(f"Incomplete projection group {key}: {members}.")
    return result


def _cuda_device(value: torch.device | str) -> torch.device:
    device = torch.device(value)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if device.type != "cuda":
        raise ValueError(f"Native W4/W8A8 runtime requires a CUDA device, got {device}.")
    return device


def _seed_list(raw: Any, *, count: int, name: str) -> tuple[int, ...]:
    if not isinstance(raw, (list, tuple)) or len(raw) != int(count):
        raise ValueError(f"R5 {name} must contain exactly {count} seeds.")
    seeds = tuple(int(item) for item in raw)
    if any(item < -1 for item in seeds):
        raise ValueError(f"R5 {name} contains an invalid seed.")
    return seeds


def _validated_seeds(row: Mapping[str, Any], *, n_j: int, n_k: int) -> tuple[tuple[int, ...], tuple[int, ...]]:
    """(V seeds, U seeds) of one manifest row; rejects anything but the frozen R5 runtime form."""
    decision = row.get("r5")
    if not isinstance(decision, Mapping) or str(decision.get("variant", "")) != "R5":
        raise ValueError(f"{row.get('layer_name', '<unknown>')} is not a frozen R5 module.")
    if int(decision.get("t_seed", -1)) != -1:
        raise ValueError("Native W4/W8A8 R5 runtime rejects a non-identity T transform.")
    if set(decision) != {"variant", "t_seed", "v_seeds", "u_seeds"}:
        raise ValueError(
            f"R5 artifact for {row.get('layer_name', '<unknown>')} contains unsupported "
            "diagonal/factor payload or unknown fields."
        )
    return (
        _seed_list(decision["v_seeds"], count=n_k, name="V"),
        _seed_list(decision["u_seeds"], count=n_j, name="U"),
    )


def tensor_parallel_range(total: int, rank: int, size: int, what: str) -> tuple[int, int]:
    """Tile range of shard ``rank`` of ``size`` over ``total`` tiles (must divide evenly)."""
    if size < 1 or not 0 <= rank < size:
        raise ValueError(f"Invalid tensor-parallel rank {rank} of {size}.")
    if total % size:
        raise ValueError(f"{what}: {total} tiles cannot be split evenly over {size} ranks.")
    step = total // size
    return rank * step, (rank + 1) * step


class _PreparedGroupOutput:
    __slots__ = ("key", "original_shape", "rows", "combined", "consumed_members")

    def __init__(self, key, original_shape, rows, combined):
        self.key = key
        self.original_shape = original_shape
        self.rows = rows
        self.combined = combined
        self.consumed_members: set[str] = set()


class _ProjectionGroupRuntime:
    """Owns and executes one fused QKV, gate/up or single projection group."""

    def __init__(
        self,
        group_id: str,
        members: Sequence[str],
        rows: Mapping[str, Mapping[str, Any]],
        tensors: Mapping[str, Mapping[str, torch.Tensor]],
        device: torch.device,
        *,
        reuse_activation: bool = True,
        scale_mode: str = "tile",
        tp_rank: int = 0,
        tp_size: int = 1,
    ) -> None:
        self.group_id = str(group_id)
        self.members = tuple(str(item) for item in members)
        if not self.members or len(set(self.members)) != len(self.members):
            raise ValueError(f"Projection group {self.group_id} has empty or duplicate members.")
        if set(rows) != set(self.members) or set(tensors) != set(self.members):
            raise ValueError(f"Projection group {self.group_id} has incomplete member artifacts.")
        self.device = torch.device(device)
        self.reuse_activation = bool(reuse_activation)
        self.scale_mode = str(scale_mode)
        self.member_slices: dict[str, tuple[int, int]] = {}
        self.row_parallel = tp_size > 1 and self.members[0].endswith(ROW_PARALLEL_SUFFIXES)

        state_rows, u_seeds = [], []
        arenas = {"w4_payload": [], "w4_scales": [], "w8_payload": [], "w8_scales": []}
        offsets = {"w4": [0], "w8": [0]}
        v_seeds: tuple[int, ...] | None = None
        n_k: int | None = None
        column = 0
        for member in self.members:
            row, member_tensors = rows[member], dict(tensors[member])
            if set(member_tensors) != set(REPLACEMENT_TENSOR_NAMES):
                raise ValueError(f"Unexpected replacement tensors for {member}.")
            m_nj, m_nk = int(row["n_j"]), int(row["n_k"])
            if m_nj <= 0 or m_nk <= 0:
                raise ValueError(f"Invalid tile geometry for {member}.")
            m_v, m_u = _validated_seeds(row, n_j=m_nj, n_k=m_nk)
            if tp_size > 1:
                if member.endswith(COLUMN_PARALLEL_SUFFIXES):
                    j0, j1 = tensor_parallel_range(m_nj, tp_rank, tp_size, member)
                    member_tensors = shard_w4w8_replacement_module(member_tensors, n_j=m_nj, n_k=m_nk, rows=(j0, j1))
                    m_u, m_nj = m_u[j0:j1], j1 - j0
                elif member.endswith(ROW_PARALLEL_SUFFIXES):
                    k0, k1 = tensor_parallel_range(m_nk, tp_rank, tp_size, member)
                    member_tensors = shard_w4w8_replacement_module(member_tensors, n_j=m_nj, n_k=m_nk, cols=(k0, k1))
                    m_v, m_nk = m_v[k0:k1], k1 - k0
                else:
                    raise ValueError(f"{member} has no tensor-parallel sharding rule.")
            if n_k is None:
                n_k, v_seeds = m_nk, m_v
            elif m_nk != n_k or m_v != v_seeds:
                raise ValueError(f"Projection group {self.group_id} does not share K geometry and V seeds.")
            state_rows.append(unpack_w4w8_state_bits(member_tensors["state_bits"].cpu(), n_j=m_nj, n_k=m_nk))
            for prefix in ("w4", "w8"):
                payload = member_tensors[f"{prefix}_payload"].detach()
                scale = member_tensors[f"{prefix}_scales"].detach()
                prefix_offsets = member_tensors[f"{prefix}_row_offsets"].detach().cpu().to(torch.int64).view(-1)
                if (
                    int(prefix_offsets.numel()) != m_nj + 1
                    or int(prefix_offsets[0]) != 0
                    or bool((prefix_offsets[1:] < prefix_offsets[:-1]).any())
                    or int(prefix_offsets[-1]) != int(payload.shape[0])
                    or int(scale.numel()) != int(payload.shape[0])
                ):
                    raise ValueError(f"Malformed {prefix.upper()} arena or offsets for {member}.")
                base = offsets[prefix][-1]
                offsets[prefix].extend(base + int(value) for value in prefix_offsets[1:])
                arenas[f"{prefix}_payload"].append(payload)
                arenas[f"{prefix}_scales"].append(scale)
            u_seeds.extend(m_u)
            self.member_slices[member] = (column, column + m_nj * 64)
            column += m_nj * 64

        assert n_k is not None and v_seeds is not None
        self.n_k = n_k
        self.v_seeds = v_seeds
        self.out_features = column
        if self.scale_mode == "token" and any(seed != -1 for seed in v_seeds):
            raise ValueError(f"{self.group_id}: per-token activation scales need identity V transforms.")
        to_device = lambda t: t.to(device=self.device).contiguous()  # noqa: E731
        raw = {
            "state_bits": to_device(pack_w4w8_state_bits(torch.cat(state_rows, dim=0))),
            "w4_payload": to_device(torch.cat(arenas["w4_payload"], dim=0)),
            "w4_scales": to_device(torch.cat(arenas["w4_scales"], dim=0)),
            "w8_payload": to_device(torch.cat(arenas["w8_payload"], dim=0)),
            "w8_scales": to_device(torch.cat(arenas["w8_scales"], dim=0)),
            "w4_row_offsets": to_device(torch.tensor(offsets["w4"], dtype=torch.int32)),
            "w8_row_offsets": to_device(torch.tensor(offsets["w8"], dtype=torch.int32)),
        }
        # one-time re-layout; the raw arenas are not kept
        self.weights = _ext.prepare_weights(*(raw[name] for name in REPLACEMENT_TENSOR_NAMES), n_k=n_k)
        del raw
        identity_v = all(seed == -1 for seed in v_seeds)
        self.v_metadata = None if identity_v else metadata_stack(v_seeds, self.device)
        self.u_metadata = None if all(seed == -1 for seed in u_seeds) else metadata_stack(u_seeds, self.device)
        self._prepared: _PreparedGroupOutput | None = None
        self.has_bias = False  # set at install: a biased member keeps the kernel output in FP32
        self.next_weights = None  # weights of the group that runs next (look-ahead), set at install

    @staticmethod
    def _activation_key(activation: torch.Tensor) -> tuple[Any, ...]:
        return (
            activation.device.type, activation.device.index, activation.data_ptr(),
            int(activation.storage_offset()), tuple(int(v) for v in activation.shape),
            tuple(int(v) for v in activation.stride()), str(activation.dtype),
        )

    def project_member(self, activation: torch.Tensor, *, member: str) -> tuple[torch.Tensor, tuple[int, ...]]:
        """Slice of the group's output that belongs to ``member``, computing the group once."""
        name = str(member)
        if name not in self.members:
            raise ValueError(f"{name} is not a member of projection group {self.group_id}.")
        key = self._activation_key(activation)
        if not self.reuse_activation:
            self._prepared = None
        if self._prepared is not None:
            if self._prepared.key != key:
                missing = sorted(set(self.members) - self._prepared.consumed_members)
                raise RuntimeError(
                    f"Projection group {self.group_id} received a new activation before "
                    f"members {missing} consumed the prior combined output."
                )
            if name in self._prepared.consumed_members:
                raise RuntimeError(
                    f"Projection group {self.group_id} member {name} was called twice for the same activation."
                )
            prepared = self._prepared
        else:
            if activation.device != self.device:
                raise ValueError(f"Projection group {self.group_id} is on {self.device}, got {activation.device}.")
            if activation.dim() < 1:
                raise ValueError(f"Native W4/W8A8 linear expects [...,K], got {tuple(activation.shape)}.")
            original_shape = tuple(int(v) for v in activation.shape)
            width = original_shape[-1]
            if width != self.n_k * 64:
                raise ValueError(f"Activation K mismatch for {self.group_id}: {width} vs {self.n_k * 64}.")
            rows = int(activation.numel()) // width
            if rows <= 0:
                raise ValueError("Activation must contain at least one row.")
            flat = activation.reshape(rows, width)
            ready = getattr(activation, "_alignquant_quantized", None)  # left by AlignQuantRMSNorm
            if not (ready is not None and self.scale_mode == "token" and self.v_metadata is None
                    and tuple(ready[0].shape) == (rows, width)):
                ready = None
            # Low-precision kernel output only for bias-free groups, as in the reference
            # (model.py:343-349): with a bias the FP32 result is kept through the bias add and
            # rounded once at the end.  Row-parallel partials stay FP32 for the sum over ranks.
            low_precision = activation.dtype in (torch.bfloat16, torch.float16) and not self.row_parallel and not self.has_bias
            out_dtype = activation.dtype if low_precision else torch.float32
            combined = None
            self.sum_fused = False
            reducer = getattr(self, "peer_allreduce", None)
            one_call = ready is None and self.scale_mode == "token" and self.v_metadata is None
            if one_call:
                # quantizer and projection (and, at decode sizes, the sum over the ranks) as one call:
                # one launch where the decode kernel quantizes its own rows, two otherwise
                if self.row_parallel and reducer is not None:
                    combined = _ext.alignquant_quant_linear(flat, self.weights, self.u_metadata, output_dtype=out_dtype,
                                                            reducer=reducer, prefetch=self.next_weights)
                    self.sum_fused = combined is not None
                if combined is None:
                    combined = _ext.alignquant_quant_linear(flat, self.weights, self.u_metadata, output_dtype=out_dtype,
                                                            prefetch=self.next_weights)
            else:
                if ready is not None:
                    qx, scales = ready
                else:
                    qx, scales = _ext.alignquant_activation_quantize_cuda(flat, self.v_metadata, scale_mode=self.scale_mode)
                if self.row_parallel and reducer is not None:
                    # decode sizes: projection and the sum over the ranks in one kernel
                    combined = _ext.alignquant_linear_allreduce(
                        qx, scales, self.weights, self.u_metadata, reducer, scale_mode=self.scale_mode, output_dtype=out_dtype,
                        prefetch=self.next_weights,
                    )
                    self.sum_fused = combined is not None
                if combined is None:
                    combined = _ext.alignquant_linear_prepared(
                        qx, scales, self.weights, self.u_metadata, scale_mode=self.scale_mode, output_dtype=out_dtype,
                        prefetch=self.next_weights,
                    )
            if tuple(combined.shape) != (rows, self.out_features):
                raise RuntimeError(
                    f"Projection group {self.group_id} returned {tuple(combined.shape)}, "
                    f"expected {(rows, self.out_features)}."
                )
            prepared = _PreparedGroupOutput(key, original_shape, rows, combined)
            self._prepared = prepared
        start, stop = self.member_slices[name]
        result = prepared.combined[:, start:stop]
        prepared.consumed_members.add(name)
        if not self.reuse_activation or prepared.consumed_members == set(self.members):
            self._prepared = None
        return result, prepared.original_shape

    def reset_pending(self) -> None:
        """Discard an incomplete shared projection after an aborted forward."""
        self._prepared = None


class AlignQuantLinear(nn.Module):
    """A frozen artifact-backed linear running on the native W4/W8A8 kernels."""

    def __init__(self, linear: nn.Linear, *, layer_name: str, runtime: _ProjectionGroupRuntime,
                 process_group: Any = None, peer_allreduce: Any = None) -> None:
        super().__init__()
        self.layer_name = str(layer_name)
        object.__setattr__(self, "runtime", runtime)
        object.__setattr__(self, "process_group", process_group)
        object.__setattr__(self, "peer_allreduce", peer_allreduce)
        self.in_features = int(linear.in_features)
        self.out_features = int(linear.out_features)
        start, stop = runtime.member_slices[self.layer_name]
        if self.in_features != runtime.n_k * 64 or self.out_features != stop - start:
            raise ValueError(f"Linear geometry disagrees with projection group for {self.layer_name}.")
        bias = None if linear.bias is None else linear.bias.detach().to(device=runtime.device).contiguous()
        self.register_buffer("bias", bias, persistent=False)

    def forward(self, activation: torch.Tensor) -> torch.Tensor:
        result, original_shape = self.runtime.project_member(activation, member=self.layer_name)
        if self.runtime.row_parallel and not getattr(self.runtime, "sum_fused", False):
            import torch.distributed as dist

            result = result.contiguous()
            reducer = self.peer_allreduce
            if (reducer is not None and result.dtype == torch.float32 and result.numel() % 4 == 0
                    and result.numel() <= reducer.max_count):
                reducer(result)  # decode-sized partials: one kernel over peer memory
            else:
                dist.all_reduce(result, group=self.process_group)  # sum of the K-shard partials
        if self.bias is not None:
            result = result.float() + self.bias.float()  # FP32 through the bias add, one rounding below
        result = result.reshape(*original_shape[:-1], self.out_features)
        return result.to(dtype=activation.dtype)


class AlignQuantRMSNorm(nn.Module):
    """The RMSNorm in front of a projection group, with the group's activation quantizer in the
    same kernel (``aq_rmsnorm_quantize``).

    Returns the normalised tensor as the module it replaces does, and leaves the int8 rows and
    their scales on it, where the projection group picks them up instead of launching its own
    quantizer (the reference runs the model's norm module and then the quantizer:
    alignquant/quantization/model.py:329-331).  The sum of squares is taken in FP64 where the stock
    module uses FP32; every rounding step of the result is the module's.  Inputs the kernel does
    not take (other dtypes, CPU tensors) go through the original module.
    """

    def __init__(self, norm: nn.Module) -> None:
        super().__init__()
        self.original = norm
        self.eps = float(getattr(norm, "variance_epsilon", getattr(norm, "eps", 1e-6)))

    @property
    def weight(self) -> torch.Tensor:
        return self.original.weight

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        weight = self.original.weight
        width = int(hidden.shape[-1]) if hidden.dim() else 0
        if (not hidden.is_cuda or hidden.dtype not in (torch.float16, torch.bfloat16) or weight.dtype != hidden.dtype
                or width % 64 or hidden.numel() == 0 or tuple(weight.shape) != (width,)):
            return self.original(hidden)
        flat = hidden.reshape(-1, width)
        normed = torch.empty_like(flat)
        quantized = _ext.alignquant_rmsnorm_quantize_cuda(flat, weight, self.eps, normed=normed)
        result = normed.reshape(hidden.shape)
        result._alignquant_quantized = quantized
        return result


def _fuse_norms(model: nn.Module, runtimes: Mapping[str, "_ProjectionGroupRuntime"]) -> int:
    """Replace the RMSNorm in front of every token-mode, identity-V projection group that follows one."""
    preceding = {"self_attn": "input_layernorm", "mlp": "post_attention_layernorm"}
    replaced = 0
    for runtime in runtimes.values():
        if runtime.scale_mode != "token" or runtime.v_metadata is not None or runtime.row_parallel:
            continue
        parts = runtime.members[0].split(".")  # ... layers.N.self_attn.q_proj
        if len(parts) < 3 or parts[-2] not in preceding or parts[-1] not in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"):
            continue
        try:
            layer = model.get_submodule(".".join(parts[:-2]))
        except AttributeError:
            continue
        norm = getattr(layer, preceding[parts[-2]], None)
        weight = getattr(norm, "weight", None)
        if (norm is None or isinstance(norm, AlignQuantRMSNorm) or weight is None or weight.dim() != 1
                or int(weight.numel()) != runtime.n_k * 64 or "rmsnorm" not in type(norm).__name__.lower()):
            continue
        setattr(layer, preceding[parts[-2]], AlignQuantRMSNorm(norm))
        replaced += 1
    return replaced


def install_alignquant(
    model: nn.Module,
    artifact: Mapping[str, Any] | str | Path,
    device: torch.device | str | None,
    *,
    reuse_activation: bool = True,
    scale_mode: str = "tile",
    tp_rank: int = 0,
    tp_size: int = 1,
    process_group: Any = None,
    peer_allreduce: Any = None,
    fuse_norms: bool = False,
) -> tuple[list[AlignQuantLinear], dict[str, Any]]:
    """Replace exactly the artifact-covered decoder projections of ``model``.

    With ``tp_size > 1`` the model's linears must already have the per-rank shapes
    (output features / tp for q, k, v, gate, up; input features / tp for o, down) while the
    artifact holds the full layers; each rank keeps its tile-aligned shard.  ``peer_allreduce``
    (a ``kernels.cuda.allreduce.PeerAllReduce``) takes over the sum of the row-parallel
    partials for FP32 results that fit its buffer; larger ones go through ``dist.all_reduce``.
    ``fuse_norms`` also replaces the RMSNorm in front of the q/k/v and gate/up groups by
    ``AlignQuantRMSNorm`` (token scale mode, identity V only).
    Returns the installed modules and a metadata dict, like the reference
    (alignquant/quantization/model.py:419-539).
    """
    target_device = None if device is None else _cuda_device(device)
    loaded = artifact if isinstance(artifact, Mapping) else load_artifact(artifact, device="cpu")
    if set(loaded) != {"root", "manifest", "modules"}:
        raise ValueError("Replacement artifact must contain root, manifest, and modules.")
    manifest, module_tensors = loaded["manifest"], loaded["modules"]
    if not isinstance(manifest, Mapping) or not isinstance(module_tensors, Mapping):
        raise TypeError("Replacement artifact manifest and modules must be mappings.")
    manifest_rows = list(manifest.get("modules", ()))
    if not manifest_rows:
        raise ValueError("Replacement artifact must contain at least one module.")
    row_map: dict[str, Mapping[str, Any]] = {}
    for row in manifest_rows:
        name = str(row.get("layer_name", ""))
        if not name or name in row_map:
            raise ValueError(f"Duplicate or empty artifact module name: {name!r}.")
        row_map[name] = row
    targets = iter_target_linears(model)
    if not targets:
        raise ValueError("Model has no target linear projections.")
    target_names = {name for _, _, name, _ in targets}
    if len(target_names) != len(targets) or target_names != set(row_map):
        raise ValueError(
            "Artifact/model target coverage mismatch: "
            f"model={len(targets)} artifact={len(row_map)} "
            f"missing={sorted(target_names - set(row_map))[:3]} "
            f"extra={sorted(set(row_map) - target_names)[:3]}"
        )
    if set(module_tensors) != set(row_map):
        raise ValueError("Loaded replacement tensor coverage differs from manifest coverage.")

    records: dict[str, tuple[nn.Module, str, torch.device]] = {}
    for parent, attr, name, linear in targets:
        full = tuple(int(v) for v in row_map[name].get("shape", ()))
        local = (int(linear.out_features), int(linear.in_features))
        expected = full
        if tp_size > 1 and len(full) == 2:
            expected = (full[0] // tp_size, full[1]) if name.endswith(COLUMN_PARALLEL_SUFFIXES) else (full[0], full[1] // tp_size)
        if local != expected:
            raise ValueError(f"Artifact shape mismatch for {name}: {list(full)} (tp {tp_size}) vs {local}.")
        if int(row_map[name]["n_j"]) != full[0] // 64 or int(row_map[name]["n_k"]) != full[1] // 64:
            raise ValueError(f"Artifact tile geometry mismatch for {name}.")
        records[name] = (parent, attr, target_device if target_device is not None else _cuda_device(linear.weight.device))
    del targets

    groups = projection_groups(tuple(sorted(records)))
    runtimes: dict[str, _ProjectionGroupRuntime] = {}
    installed: list[AlignQuantLinear] = []
    for group_id, members in groups.items():
        devices = {records[m][2] for m in members}
        if len(devices) != 1:
            raise ValueError(f"Projection group {group_id} spans CUDA devices: {devices}.")
        runtime = _ProjectionGroupRuntime(
            group_id, members, {m: row_map[m] for m in members}, {m: module_tensors[m] for m in members},
            next(iter(devices)), reuse_activation=reuse_activation, scale_mode=scale_mode,
            tp_rank=tp_rank, tp_size=tp_size,
        )
        runtimes[group_id] = runtime
        for name in members:
            parent, attr, _ = records.pop(name)
            runtime.peer_allreduce = peer_allreduce
            runtime.has_bias = runtime.has_bias or getattr(parent, attr).bias is not None
            module = AlignQuantLinear(getattr(parent, attr), layer_name=name, runtime=runtime, process_group=process_group,
                                      peer_allreduce=peer_allreduce)
            setattr(parent, attr, module)
            installed.append(module)
    model._alignquant_projection_groups = tuple(runtimes.values())
    chain = execution_order(runtimes)
    for position, group_id in enumerate(chain):
        successor = runtimes[chain[(position + 1) % len(chain)]]
        if successor.device == runtimes[group_id].device and len(chain) > 1:
            runtimes[group_id].next_weights = successor.weights
    fused_norms = _fuse_norms(model, runtimes) if fuse_norms else 0
    metadata = {
        "fused_norm_count": fused_norms,
        "module_count": len(installed),
        "projection_group_count": len(runtimes),
        "groups": {group: list(members) for group, members in groups.items()},
        "reuse_activation": bool(reuse_activation),
        "scale_mode": str(scale_mode),
        "tensor_parallel": {"rank": int(tp_rank), "size": int(tp_size)},
    }
    return installed, metadata


def execution_order(group_ids: Sequence[str]) -> list[str]:
    """Group ids in the order a decoder runs them: by layer index, then qkv, o, gate_up, down."""
    rank = {"qkv": 0, "q_proj": 0, "k_proj": 0, "v_proj": 0, "o_proj": 1, "gate_up": 2, "gate_proj": 2, "up_proj": 2, "down_proj": 3}

    def key(group_id: str):
        parts = group_id.split(".")
        layer = next((int(parts[i + 1]) for i, part in enumerate(parts[:-1]) if part == "layers" and parts[i + 1].isdigit()), -1)
        return (layer, rank.get(parts[-1], 4), group_id)

    return sorted((str(g) for g in group_ids), key=key)


def reset_alignquant_state(model: nn.Module) -> None:
    """Reset transient shared-projection state between independent forwards."""
    for runtime in getattr(model, "_alignquant_projection_groups", ()):
        runtime.reset_pending()


__all__ = ["AlignQuantLinear", "install_alignquant", "projection_groups", "reset_alignquant_state"]
