"""Python operator API of the native W4/W8-A8 path.

Same callables as the reference's ``alignquant/kernels/cuda/extension.py:254-319``
(``load_extension``, ``alignquant_activation_quantize_cuda``,
``alignquant_linear_cuda``), backed by ``libalignquant_b200.so`` through ctypes.
Tensors are passed to the C ABI as raw device pointers together with the current
CUDA stream; outputs are allocated here with torch's caching allocator.

Additions over the reference API: ``scale_mode`` ("tile" = the reference's
16x64-tile scales, the default; "token" = one scale per row), fp16 output, row
counts that are not multiples of 16, and ``prepare_weights`` /
``alignquant_linear_prepared`` for callers that keep the re-laid-out weight image.
"""

from __future__ import annotations

import weakref
from dataclasses import dataclass

import torch

from alignquant_b200 import _lib

_DTYPE_CODES = {torch.float16: _lib.AQ_F16, torch.bfloat16: _lib.AQ_BF16, torch.float32: _lib.AQ_F32}
_SCALE_MODES = {"tile": _lib.AQ_SCALE_TILE, "token": _lib.AQ_SCALE_TOKEN}


def load_extension() -> None:
    """Load the native library before a timed region (extension.py:254-257 of the reference)."""
    if not torch.cuda.is_available():
        raise RuntimeError("The W4/W8A8 extension requires a visible CUDA device.")
    capability = torch.cuda.get_device_capability()
    if capability[0] != 10:
        raise RuntimeError(f"The W4/W8A8 extension requires SM100 (B200), got {capability}.")
    _lib.load()


def _stream(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def _ptr(tensor: torch.Tensor | None) -> int | None:
    if tensor is None or tensor.numel() == 0:
        return None
    return int(tensor.data_ptr())


def _require_cuda(tensor: torch.Tensor, name: str) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(f"{name} must be CUDA")


def _scale_mode_code(scale_mode: str) -> int:
    try:
        return _SCALE_MODES[str(scale_mode)]
    except KeyError as error:
        raise ValueError(f"Unknown scale_mode {scale_mode!r}; expected {tuple(_SCALE_MODES)}.") from error


def alignquant_activation_quantize_cuda(
    activation: torch.Tensor,
    v_metadata: torch.Tensor | None,
    *,
    tile_major: bool = False,
    scale_mode: str = "tile",
    out: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantize ``[M, K]`` activations to int8; returns ``(int8, float32 scales)``.

    ``scale_mode="tile"``: scales are ``[ceil(M/16), K/64]`` (``[K/64]`` when M <= 16,
    as in the reference, linear.cu:1539-1542) after the structured V transform.
    ``scale_mode="token"``: scales are ``[M]``; ``v_metadata`` must be None or identity.
    ``tile_major=True`` returns the reference's ``[M/16, K/64, 16, 64]`` arrangement; it
    exists for API compatibility only (the kernels here read row-major activations).
    ``out=(int8, scales)`` reuses caller-owned contiguous buffers of the right size.
    """
    mode = _scale_mode_code(scale_mode)
    _require_cuda(activation, "x")
    if activation.dtype not in _DTYPE_CODES:
        raise RuntimeError("x must be bf16, fp16, or fp32")
    if activation.dim() != 2 or activation.size(0) < 1:
        raise RuntimeError("x must be [M,K] with positive M")
    x = activation.contiguous()
    m, k = int(x.size(0)), int(x.size(1))
    if k % 64:
        raise RuntimeError("K must be a multiple of 64")
    n_k = k // 64
    if tile_major and (m < 128 or m % 16):
        raise RuntimeError("tile-major A8 output requires at least 128 rows (a multiple of 16)")
    meta = None
    if v_metadata is not None:
        _require_cuda(v_metadata, "v_metadata")
        if v_metadata.dtype != torch.int32:
            raise RuntimeError("v_metadata must be int32")
        if tuple(v_metadata.shape) != (n_k, 4, 64):
            raise RuntimeError("v_metadata must be [K/64,4,64]")
        if v_metadata.device != x.device:
            raise RuntimeError("x and v_metadata must share one device")
        meta = v_metadata.contiguous()
        if mode == _lib.AQ_SCALE_TOKEN:
            if bool((meta[:, 0, 0] != 0).any()):
                raise RuntimeError("per-token scales do not support a non-identity V transform")
            meta = None
    n_m = (m + 15) // 16
    scale_shape = (m,) if mode == _lib.AQ_SCALE_TOKEN else ((n_k,) if n_m == 1 else (n_m, n_k))
    with torch.cuda.device(x.device):
        if out is not None:
            q, scales = out
            if (q.dtype != torch.int8 or tuple(q.shape) != (m, k) or not q.is_contiguous()
                    or scales.dtype != torch.float32 or tuple(scales.shape) != scale_shape
                    or not scales.is_contiguous() or q.device != x.device or scales.device != x.device):
                raise RuntimeError("out must be (contiguous int8 [M,K], contiguous float32 scales) on x's device")
            if tile_major:
                raise RuntimeError("out= is not available with tile_major=True")
        else:
            q = torch.empty((m, k), dtype=torch.int8, device=x.device)
            scales = torch.empty(scale_shape, dtype=torch.float32, device=x.device)
        _lib.check(
            _lib.load().aq_quantize_act(
                _ptr(x), _DTYPE_CODES[x.dtype], m, k, _ptr(meta), mode, _ptr(q), _ptr(scales), _stream(x.device)
            )
        )
    if tile_major:
        q = q.view(m // 16, 16, n_k, 64).permute(0, 2, 1, 3).contiguous()
    return q, scales


def alignquant_rmsnorm_quantize_cuda(
    activation: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    *,
    out: tuple[torch.Tensor, torch.Tensor] | None = None,
    normed: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """RMSNorm (Llama / Qwen3 module arithmetic) + per-token int8 quantizer in one kernel.

    ``activation`` [M, K] and ``weight`` [K] share one dtype (fp16 / bf16 / fp32).  Returns
    ``(int8 [M, K], float32 scales [M])``, what ``alignquant_activation_quantize_cuda(norm(x),
    None, scale_mode="token")`` returns; ``normed`` (same dtype, [M, K]) optionally receives the
    normalised activations as well.
    """
    _require_cuda(activation, "x")
    if activation.dtype not in _DTYPE_CODES or weight.dtype != activation.dtype:
        raise RuntimeError("x and weight must share one dtype: bf16, fp16, or fp32")
    if activation.dim() != 2 or activation.size(0) < 1:
        raise RuntimeError("x must be [M,K] with positive M")
    x, w = activation.contiguous(), weight.contiguous()
    m, k = int(x.size(0)), int(x.size(1))
    if k % 64 or tuple(w.shape) != (k,) or w.device != x.device:
        raise RuntimeError("K must be a multiple of 64 and weight must be [K] on x's device")
    with torch.cuda.device(x.device):
        if out is not None:
            q, scales = out
            if (q.dtype != torch.int8 or tuple(q.shape) != (m, k) or not q.is_contiguous() or scales.dtype != torch.float32
                    or tuple(scales.shape) != (m,) or not scales.is_contiguous()):
                raise RuntimeError("out must be (contiguous int8 [M,K], contiguous float32 [M])")
        else:
            q = torch.empty((m, k), dtype=torch.int8, device=x.device)
            scales = torch.empty((m,), dtype=torch.float32, device=x.device)
        if normed is not None and (normed.dtype != x.dtype or tuple(normed.shape) != (m, k) or not normed.is_contiguous()):
            raise RuntimeError("normed must be a contiguous [M,K] tensor of x's dtype")
        _lib.check(
            _lib.load().aq_rmsnorm_quantize(
                _ptr(x), _DTYPE_CODES[x.dtype], m, k, _ptr(w), float(eps), _ptr(q), _ptr(scales), _ptr(normed), _stream(x.device)
            )
        )
    return q, scales


@dataclass
class PreparedWeights:
    """A layer's weights re-laid-out once for the B200 kernels (see ``aq_repack``)."""

    image: torch.Tensor
    n_j: int
    n_k: int
    t4: int
    t8: int

    @property
    def device(self) -> torch.device:
        return self.image.device

    def payload_bytes(self) -> int:
        return self.t4 * 2048 + self.t8 * 4096

    def algorithmic_bytes(self) -> int:
        """Weight-side bytes a kernel must read: tiles plus one 8-byte record per tile."""
        return self.payload_bytes() + 8 * (self.t4 + self.t8)


def prepare_weights(
    state_bits: torch.Tensor,
    w4_payload: torch.Tensor,
    w4_scales: torch.Tensor,
    w8_payload: torch.Tensor,
    w8_scales: torch.Tensor,
    w4_row_offsets: torch.Tensor,
    w8_row_offsets: torch.Tensor,
    *,
    n_k: int,
) -> PreparedWeights:
    """Validate the seven artifact tensors of a layer and build its prepared image.

    The checks are those of the reference's host function (linear.cu:1594-1639).
    """
    tensors = {
        "state_bits": (state_bits, torch.uint8),
        "w4_payload": (w4_payload, torch.uint8),
        "w4_scales": (w4_scales, torch.float32),
        "w8_payload": (w8_payload, torch.int8),
        "w8_scales": (w8_scales, torch.float32),
        "w4_row_offsets": (w4_row_offsets, torch.int32),
        "w8_row_offsets": (w8_row_offsets, torch.int32),
    }
    device = state_bits.device
    for name, (tensor, dtype) in tensors.items():
        _require_cuda(tensor, name)
        if tensor.dtype != dtype:
            raise RuntimeError(f"{name} must be {str(dtype).replace('torch.', '')}")
        if tensor.device != device:
            raise RuntimeError("all inputs must share one CUDA device")
    if w4_payload.dim() != 3 or tuple(w4_payload.shape[1:]) != (64, 32):
        raise RuntimeError("w4_payload must be [tiles,64,32]")
    if w8_payload.dim() != 3 or tuple(w8_payload.shape[1:]) != (64, 64):
        raise RuntimeError("w8_payload must be [tiles,64,64]")
    t4, t8 = int(w4_payload.size(0)), int(w8_payload.size(0))
    if t4 != w4_scales.numel():
        raise RuntimeError("W4 payload/scale count mismatch")
    if t8 != w8_scales.numel():
        raise RuntimeError("W8 payload/scale count mismatch")
    if w4_row_offsets.dim() != 1 or w8_row_offsets.dim() != 1:
        raise RuntimeError("row offsets must be rank 1")
    if w4_row_offsets.numel() != w8_row_offsets.numel():
        raise RuntimeError("row offset sizes differ")
    n_j = int(w4_row_offsets.numel()) - 1
    if n_j <= 0:
        raise RuntimeError("N must contain at least one 64-column tile")
    if state_bits.numel() != (n_j * n_k + 7) // 8:
        raise RuntimeError("state_bits byte count mismatch")
    if t4 + t8 != n_j * n_k:
        raise RuntimeError("selected payload count mismatch")
    lib = _lib.load()
    size = int(lib.aq_prepared_bytes(n_j, n_k, t4, t8))
    if size < 0:
        _lib.check(size)
    with torch.cuda.device(device):
        image = torch.empty((size,), dtype=torch.uint8, device=device)
        keep = [t.contiguous() for t, _ in tensors.values()]
        _lib.check(
            lib.aq_repack(
                _ptr(keep[0]), _ptr(keep[1]), _ptr(keep[2]), _ptr(keep[3]), _ptr(keep[4]), _ptr(keep[5]),
                _ptr(keep[6]), n_j, n_k, t4, t8, _ptr(image), size, _stream(device),
            )
        )
    return PreparedWeights(image=image, n_j=n_j, n_k=n_k, t4=t4, t8=t8)


def alignquant_linear_prepared(
    activation: torch.Tensor,
    activation_scales: torch.Tensor,
    weights: PreparedWeights,
    u_metadata: torch.Tensor | None,
    *,
    schedule: str = "auto",
    decode_splits: int = 0,
    output_dtype: torch.dtype = torch.float32,
    scale_mode: str = "tile",
    acc_dump: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    prefetch: PreparedWeights | None = None,
) -> torch.Tensor:
    """Run one packed projection on a prepared weight image; returns ``[M, N]``.

    ``prefetch``: the weights of the projection that runs next.  The decode kernels ask the L2
    cache to fetch that image while this projection runs (``aq_linear_ahead``); other kernels
    ignore it.
    """
    try:
        schedule_code = _lib.SCHEDULE_CODES[str(schedule)]
    except KeyError as error:
        raise ValueError(
            f"Unknown W4/W8A8 schedule {schedule!r}; expected {tuple(_lib.SCHEDULE_CODES)}."
        ) from error
    if output_dtype not in _DTYPE_CODES:
        raise ValueError("Projection output_dtype must be torch.float32, torch.bfloat16 or torch.float16.")
    mode = _scale_mode_code(scale_mode)
    _require_cuda(activation, "x_int8")
    _require_cuda(activation_scales, "activation_scales")
    if activation.dtype != torch.int8:
        raise RuntimeError("x_int8 must be int8")
    if activation_scales.dtype != torch.float32:
        raise RuntimeError("activation_scales must be float32")
    n_j, n_k = weights.n_j, weights.n_k
    x = activation
    if x.dim() == 4:  # the reference's tile-major arrangement [M/16, K/64, 16, 64]
        if x.size(2) != 16 or x.size(3) != 64:
            raise RuntimeError("tile-major x_int8 must be [M/16,K/64,16,64] with M>=128")
        x = x.permute(0, 2, 1, 3).reshape(x.size(0) * 16, x.size(1) * 64)
    if x.dim() != 2:
        raise RuntimeError("x_int8 must be [M,K] or tile-major [M/16,K/64,16,64]")
    x = x.contiguous()
    m = int(x.size(0))
    if int(x.size(1)) != n_k * 64:
        raise RuntimeError(f"K mismatch: activation has {int(x.size(1))}, weights have {n_k * 64}")
    scales = activation_scales.contiguous()
    expected = m if mode == _lib.AQ_SCALE_TOKEN else ((m + 15) // 16) * n_k
    if scales.numel() != expected:
        raise RuntimeError(
            "activation_scales must contain one scalar per M16x64 tile"
            if mode == _lib.AQ_SCALE_TILE
            else "activation_scales must contain one scalar per row"
        )
    device = x.device
    if scales.device != device or weights.device != device:
        raise RuntimeError("all inputs must share one CUDA device")
    meta = None
    if u_metadata is not None:
        _require_cuda(u_metadata, "u_metadata")
        if u_metadata.dtype != torch.int32:
            raise RuntimeError("u_metadata must be int32")
        if tuple(u_metadata.shape) != (n_j, 4, 64):
            raise RuntimeError("u_metadata must be [N/64,4,64]")
        if u_metadata.device != device:
            raise RuntimeError("all inputs must share one CUDA device")
        meta = u_metadata.contiguous()
    if acc_dump is not None:
        if acc_dump.dtype != torch.int32 or tuple(acc_dump.shape) != (m, n_j, n_k, 64) or not acc_dump.is_contiguous():
            raise RuntimeError("acc_dump must be a contiguous int32 [M,N/64,K/64,64] tensor")
    lib = _lib.load()
    with torch.cuda.device(device):
        if out is None:
            out = torch.empty((m, n_j * 64), dtype=output_dtype, device=device)
        elif out.dtype != output_dtype or tuple(out.shape) != (m, n_j * 64) or not out.is_contiguous():
            raise RuntimeError("out must be a contiguous [M,N] tensor of output_dtype")
        ws_bytes = int(lib.aq_linear_workspace_bytes(m, n_j, n_k, schedule_code, int(decode_splits)))
        if ws_bytes < 0:
            _lib.check(ws_bytes)
        workspace = _workspace(device, ws_bytes) if ws_bytes else None
        if prefetch is not None and prefetch.device != device:
            raise RuntimeError("prefetch must name weights on the device of this call")
        _lib.check(
            lib.aq_linear_ahead(
                _ptr(x), _ptr(scales), mode, m, _ptr(weights.image), n_j, n_k, _ptr(meta), schedule_code,
                int(decode_splits), _DTYPE_CODES[output_dtype], _ptr(out), _ptr(workspace), ws_bytes,
                _ptr(acc_dump), None if prefetch is None else _ptr(prefetch.image),
                0 if prefetch is None else int(prefetch.image.numel()), _stream(device),
            )
        )
    return out


def alignquant_linear_allreduce(
    activation: torch.Tensor,
    activation_scales: torch.Tensor,
    weights: PreparedWeights,
    u_metadata: torch.Tensor | None,
    reducer,
    *,
    output_dtype: torch.dtype = torch.float32,
    scale_mode: str = "tile",
    out: torch.Tensor | None = None,
    prefetch: PreparedWeights | None = None,
) -> torch.Tensor | None:
    """Row-parallel projection and the sum over the tensor-parallel ranks in ONE kernel.

    ``reducer`` is a ``kernels.cuda.allreduce.PeerAllReduce``.  Returns the summed ``[M, N]``
    result, or ``None`` when the problem does not take the decode kernel that carries the fused
    epilogue (more than 32 rows, very few tile rows, result larger than the exchange buffers);
    the caller then runs ``alignquant_linear_prepared`` followed by ``reducer(...)``.
    Every rank must take the same branch: the decision depends only on the shapes.
    """
    mode = _scale_mode_code(scale_mode)
    n_j, n_k = weights.n_j, weights.n_k
    x = activation.contiguous()
    if x.dim() != 2 or x.dtype != torch.int8 or int(x.size(1)) != n_k * 64:
        raise RuntimeError("x_int8 must be int8 [M,K] matching the weights")
    m = int(x.size(0))
    if m * n_j * 64 > reducer.max_count or linear_plan(m, n_j, n_k)["kernel"] != 3:
        return None
    scales = activation_scales.contiguous()
    device = x.device
    meta = None if u_metadata is None else u_metadata.contiguous()
    lib = _lib.load()
    with torch.cuda.device(device):
        if out is None:
            out = torch.empty((m, n_j * 64), dtype=output_dtype, device=device)
        _lib.check(
            lib.aq_linear_allreduce(
                _ptr(x), _ptr(scales), mode, m, _ptr(weights.image), n_j, n_k, _ptr(meta), _DTYPE_CODES[output_dtype],
                _ptr(out), reducer.rank, reducer.world, reducer.peer_array_pointer(), reducer.max_count,
                None if prefetch is None else _ptr(prefetch.image),
                0 if prefetch is None else int(prefetch.image.numel()), _stream(device),
            )
        )
    return out


def quant_linear_is_fused(m: int, n_j: int, n_k: int) -> bool:
    """Whether ``alignquant_quant_linear`` runs this problem (fp16 / bf16 rows) as one launch."""
    return bool(_lib.load().aq_quant_linear_fused(int(m), int(n_j), int(n_k)))


def alignquant_quant_linear(
    activation: torch.Tensor,
    weights: PreparedWeights,
    u_metadata: torch.Tensor | None,
    *,
    output_dtype: torch.dtype = torch.float32,
    out: torch.Tensor | None = None,
    quantized: tuple[torch.Tensor, torch.Tensor] | None = None,
    reducer=None,
    prefetch: PreparedWeights | None = None,
) -> torch.Tensor | None:
    """Per-token activation quantizer and projection in one call (``aq_quant_linear``).

    ``activation`` is ``[M, K]`` in fp16 / bf16 / fp32 (no input transform).  Same bits as
    ``alignquant_activation_quantize_cuda(x, None, scale_mode="token")`` followed by
    ``alignquant_linear_prepared`` (or ``alignquant_linear_allreduce`` when ``reducer`` is
    given); one launch instead of two where ``quant_linear_is_fused`` says so.  ``quantized``
    (int8 ``[M, K]``, float32 ``[M]``) receives the quantized activations; allocated when not
    passed.  With ``reducer``: returns ``None`` where the fused sum does not apply, exactly as
    ``alignquant_linear_allreduce`` does, and nothing has been enqueued then.
    """
    if output_dtype not in _DTYPE_CODES:
        raise ValueError("Projection output_dtype must be torch.float32, torch.bfloat16 or torch.float16.")
    _require_cuda(activation, "x")
    if activation.dtype not in _DTYPE_CODES:
        raise RuntimeError("x must be bf16, fp16, or fp32")
    n_j, n_k = weights.n_j, weights.n_k
    if activation.dim() != 2 or int(activation.size(0)) < 1 or int(activation.size(1)) != n_k * 64:
        raise RuntimeError("x must be [M,K] with positive M and the weights' K")
    x = activation.contiguous()
    m, k = int(x.size(0)), int(x.size(1))
    device = x.device
    if weights.device != device:
        raise RuntimeError("all inputs must share one CUDA device")
    if reducer is not None and (m * n_j * 64 > reducer.max_count or linear_plan(m, n_j, n_k)["kernel"] != 3):
        return None
    meta = None
    if u_metadata is not None:
        _require_cuda(u_metadata, "u_metadata")
        if u_metadata.dtype != torch.int32 or tuple(u_metadata.shape) != (n_j, 4, 64) or u_metadata.device != device:
            raise RuntimeError("u_metadata must be int32 [N/64,4,64] on x's device")
        meta = u_metadata.contiguous()
    lib = _lib.load()
    with torch.cuda.device(device):
        if quantized is not None:
            q, scales = quantized
            if (q.dtype != torch.int8 or tuple(q.shape) != (m, k) or not q.is_contiguous() or scales.dtype != torch.float32
                    or tuple(scales.shape) != (m,) or not scales.is_contiguous() or q.device != device or scales.device != device):
                raise RuntimeError("quantized must be (contiguous int8 [M,K], contiguous float32 [M]) on x's device")
        else:
            q = torch.empty((m, k), dtype=torch.int8, device=device)
            scales = torch.empty((m,), dtype=torch.float32, device=device)
        if out is None:
            out = torch.empty((m, n_j * 64), dtype=output_dtype, device=device)
        elif out.dtype != output_dtype or tuple(out.shape) != (m, n_j * 64) or not out.is_contiguous():
            raise RuntimeError("out must be a contiguous [M,N] tensor of output_dtype")
        ws_bytes, workspace = 0, None
        if reducer is None:
            ws_bytes = int(lib.aq_linear_workspace_bytes(m, n_j, n_k, _lib.SCHEDULE_CODES["auto"], 0))
            if ws_bytes < 0:
                _lib.check(ws_bytes)
            workspace = _workspace(device, ws_bytes) if ws_bytes else None
        if prefetch is not None and prefetch.device != device:
            raise RuntimeError("prefetch must name weights on the device of this call")
        _lib.check(
            lib.aq_quant_linear(
                _ptr(x), _DTYPE_CODES[x.dtype], m, _ptr(weights.image), n_j, n_k, _ptr(meta), _DTYPE_CODES[output_dtype],
                _ptr(out), _ptr(q), _ptr(scales), _ptr(workspace), ws_bytes,
                0 if reducer is None else reducer.rank, 1 if reducer is None else reducer.world,
                None if reducer is None else reducer.peer_array_pointer(), 0 if reducer is None else reducer.max_count,
                None if prefetch is None else _ptr(prefetch.image),
                0 if prefetch is None else int(prefetch.image.numel()), _stream(device),
            )
        )
    return out


_WORKSPACES: dict[tuple, torch.Tensor] = {}


def _workspace(device: torch.device, size: int) -> torch.Tensor:
    """Zeroed scratch for split-K partials, one per (device, stream).

    The kernels leave the workspace zeroed, and calls on one stream run in order, so a
    single buffer per stream is reused by every call; it only grows.
    """
    key = (device.index, _stream(device))
    buffer = _WORKSPACES.get(key)
    if buffer is None or buffer.numel() < size:
        buffer = torch.zeros((max(size, 1 << 21),), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buffer
    return buffer


_PREPARED_CACHE: dict[tuple, PreparedWeights] = {}


def _cached_prepared(tensors: tuple[torch.Tensor, ...], n_k: int) -> PreparedWeights:
    """Prepared image of the caller's seven arena tensors, cached while those tensors live.

    Key and lifetime follow the caller's own tensor objects (storage address, offset, shape,
    strides, version counter), not contiguous temporaries made from them, so a caller that passes
    long-lived tensors pays the re-layout once whatever their memory format.  Tensors that are
    themselves per-call temporaries (a fresh view or slice object on every call) cannot be
    cached across calls: their image is rebuilt each time, which costs a pass over the weights.
    """
    key = tuple(
        (int(t.untyped_storage().data_ptr()), int(t.storage_offset()), tuple(t.shape), tuple(t.stride()), int(t._version))
        for t in tensors
    ) + (n_k, str(tensors[0].device))
    hit = _PREPARED_CACHE.get(key)
    if hit is None:
        hit = prepare_weights(*(t.contiguous() for t in tensors), n_k=n_k)
        _PREPARED_CACHE[key] = hit
        for tensor in tensors:  # the image is only valid while the source tensors are alive
            weakref.finalize(tensor, _PREPARED_CACHE.pop, key, None)
    return hit


def alignquant_linear_cuda(
    activation: torch.Tensor,
    activation_scales: torch.Tensor,
    state_bits: torch.Tensor,
    w4_payload: torch.Tensor,
    w4_scales: torch.Tensor,
    w8_payload: torch.Tensor,
    w8_scales: torch.Tensor,
    w4_row_offsets: torch.Tensor,
    w8_row_offsets: torch.Tensor,
    u_metadata: torch.Tensor,
    *,
    schedule: str = "auto",
    decode_splits: int = 0,
    output_dtype: torch.dtype = torch.float32,
    scale_mode: str = "tile",
) -> torch.Tensor:
    """Run one packed projection from the raw artifact tensors (reference signature).

    The weight arenas are re-laid-out on first use and the image is cached for as long
    as the seven tensor objects passed here stay alive (per-call temporaries are re-laid-out
    on every call); callers that own the weights should call ``prepare_weights`` once and
    ``alignquant_linear_prepared`` per step instead.
    """
    if activation.dim() == 4:
        n_k = int(activation.size(1))
    else:
        n_k = int(activation.size(-1)) // 64
    tensors = (state_bits, w4_payload, w4_scales, w8_payload, w8_scales, w4_row_offsets, w8_row_offsets)
    weights = _cached_prepared(tensors, n_k)
    return alignquant_linear_prepared(
        activation, activation_scales, weights, u_metadata,
        schedule=schedule, decode_splits=decode_splits, output_dtype=output_dtype, scale_mode=scale_mode,
    )


def device_status(device: torch.device | str | None = None) -> None:
    """Synchronise the current stream and raise if a kernel gave up a device-side wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        status = _lib.load().aq_device_status(_stream(dev))
        if status != _lib.AQ_OK:
            _WORKSPACES.clear()  # arrival counters may be left non-zero by an aborted kernel
        _lib.check(status)


def alignquant_linear_decode_static(
    activation: torch.Tensor,
    activation_scales: torch.Tensor,
    weights: PreparedWeights,
    u_metadata: torch.Tensor | None,
    *,
    output_dtype: torch.dtype = torch.float32,
    scale_mode: str = "tile",
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Decode projection (at most 16 rows) that needs no workspace from the caller.

    For hosts that may only hand over inputs and outputs -- fixed-signature operator
    plug-ins, runtimes that forbid device allocation once they are up -- the library
    runs its stream-K decode kernel on a 2 MiB scratch array of its own
    (``aq_linear_decode_static``).  Layers that need more scratch raise ``RuntimeError``.
    All calls on a device share that array: calls whose kernels could overlap (different
    streams) must be serialised by the caller.  The very first call on a device looks up
    the array's address and should be made outside of a stream capture.  Only ``out`` is
    allocated here (by torch) when the caller does not pass it.
    """
    if output_dtype not in _DTYPE_CODES:
        raise ValueError("Projection output_dtype must be torch.float32, torch.bfloat16 or torch.float16.")
    mode = _scale_mode_code(scale_mode)
    x = activation.contiguous()
    if x.dtype != torch.int8 or x.dim() != 2 or not x.is_cuda:
        raise RuntimeError("x_int8 must be a CUDA int8 [M,K] tensor")
    m = int(x.size(0))
    n_j, n_k = weights.n_j, weights.n_k
    if int(x.size(1)) != n_k * 64:
        raise RuntimeError(f"K mismatch: activation has {int(x.size(1))}, weights have {n_k * 64}")
    scales = activation_scales.contiguous()
    if scales.dtype != torch.float32 or scales.numel() != (m if mode == _lib.AQ_SCALE_TOKEN else ((m + 15) // 16) * n_k):
        raise RuntimeError("activation_scales has the wrong dtype or size for this scale_mode")
    device = x.device
    meta = None if u_metadata is None else u_metadata.contiguous()
    with torch.cuda.device(device):
        if out is None:
            out = torch.empty((m, n_j * 64), dtype=output_dtype, device=device)
        _lib.check(
            _lib.load().aq_linear_decode_static(
                _ptr(x), _ptr(scales), mode, m, _ptr(weights.image), n_j, n_k, _ptr(meta),
                _DTYPE_CODES[output_dtype], _ptr(out), _stream(device),
            )
        )
    return out


def set_peer_poll_limit(polls: int | None) -> None:
    """How often a tensor-parallel sum polls for a peer before giving up (None: the default)."""
    _lib.check(_lib.load().aq_set_option(_lib.AQ_OPT_PEER_POLL_LIMIT, (1 << 22) if polls is None else int(polls)))


def set_gemm_rounding(separate: bool) -> None:
    """GEMM FP32 accumulation: one fused multiply-add per tile (default) or the reference
    kernels' separately rounded multiply and add (``AQ_OPT_GEMM_ROUNDING``)."""
    _lib.check(_lib.load().aq_set_option(
        _lib.AQ_OPT_GEMM_ROUNDING, _lib.AQ_GEMM_ROUNDING_SEPARATE if separate else _lib.AQ_GEMM_ROUNDING_FUSED))


def gemm_rounding_is_separate() -> bool:
    return int(_lib.load().aq_get_option(_lib.AQ_OPT_GEMM_ROUNDING)) == _lib.AQ_GEMM_ROUNDING_SEPARATE


def set_gemm_tile(name: str = "auto") -> None:
    """Force a CTA tile of the GEMM: "auto", "paired", "narrow" or "wide" (``AQ_OPT_GEMM_TILE``)."""
    _lib.check(_lib.load().aq_set_option(_lib.AQ_OPT_GEMM_TILE, _lib.GEMM_TILES[str(name)]))


def set_decode_kernel(cluster_only: bool = False, stream_k: bool = False) -> None:
    """``cluster_only``: never use the decode kernel of many small CTAs; ``stream_k``: the persistent
    stream-K kernel for everything of at most 16 rows (``AQ_OPT_DECODE_KERNEL``); neither: automatic."""
    value = _lib.AQ_DECODE_KERNEL_STREAMK if stream_k else _lib.AQ_DECODE_KERNEL_CLUSTER if cluster_only else _lib.AQ_DECODE_KERNEL_AUTO
    _lib.check(_lib.load().aq_set_option(_lib.AQ_OPT_DECODE_KERNEL, value))


def set_quant_fusion_tiles(tiles: int = 2400) -> None:
    """Largest layer (in 64 x 64 tiles) for which ``alignquant_quant_linear`` runs as one launch; 0: never
    (``AQ_OPT_QUANT_FUSION_TILES``)."""
    _lib.check(_lib.load().aq_set_option(_lib.AQ_OPT_QUANT_FUSION_TILES, int(tiles)))


def set_gemm_split(split: int = 0) -> None:
    """Force the number of K ranges of the GEMM, 0 = automatic (``AQ_OPT_GEMM_SPLIT``)."""
    _lib.check(_lib.load().aq_set_option(_lib.AQ_OPT_GEMM_SPLIT, int(split)))


def measure_int8_peak(pairs: int = 4096, device: torch.device | str | None = None) -> float:
    """Integer TOPS of back-to-back ``tcgen05.mma kind::i8`` on all SMs (``aq_measure_int8_peak``)."""
    import ctypes

    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    tops = ctypes.c_double()
    with torch.cuda.device(dev):
        _lib.check(_lib.load().aq_measure_int8_peak(int(pairs), ctypes.addressof(tops), _stream(dev)))
    return float(tops.value)


def linear_plan(m: int, n_j: int, n_k: int, *, schedule: str = "auto", decode_splits: int = 0) -> dict[str, int]:
    """Kernel family, split count and accumulator count ``aq_linear`` will use.

    ``kernel``: 0 cluster kernel (tiles of a split added in increasing k), 1 GEMM,
    2 persistent stream-K kernel, 3 warp-per-tile cluster kernel; see ``aq_linear_plan``
    in ``include/alignquant_b200.h`` for how ``splits`` and ``workers`` fix the FP32
    summation order.
    """
    import ctypes

    kernel, splits, workers = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    _lib.check(
        _lib.load().aq_linear_plan(
            int(m), int(n_j), int(n_k), _lib.SCHEDULE_CODES[str(schedule)], int(decode_splits),
            ctypes.addressof(kernel), ctypes.addressof(splits), ctypes.addressof(workers),
        )
    )
    return {"kernel": kernel.value, "splits": splits.value, "workers": workers.value}


__all__ = [
    "load_extension",
    "alignquant_activation_quantize_cuda",
    "alignquant_rmsnorm_quantize_cuda",
    "alignquant_linear_cuda",
    "alignquant_linear_prepared",
    "alignquant_linear_decode_static",
    "prepare_weights",
    "PreparedWeights",
    "device_status",
    "linear_plan",
    "set_peer_poll_limit",
    "set_gemm_rounding",
    "gemm_rounding_is_separate",
    "set_gemm_tile",
    "measure_int8_peak",
    "set_gemm_split",
    "set_decode_kernel",
]
