"""Locate the decoder projections a W4/W8 replacement artifact covers."""

from __future__ import annotations

from torch import nn

TARGET_PATH_SUFFIXES = (
    ".self_attn.q_proj",
    ".self_attn.k_proj",
    ".self_attn.v_proj",
    ".self_attn.o_proj",
    ".mlp.up_proj",
    ".mlp.down_proj",
    ".mlp.gate_proj",
)
_LAYER_PREFIXES = ("model.language_model.layers.", "model.layers.")


def decoder_layer_prefix(model: nn.Module) -> str:
    """The one decoder layer tree of ``model`` (alignquant/models/decoder.py:19-37)."""
    model_type = str(getattr(getattr(model, "config", None), "model_type", ""))
    if model_type.startswith("qwen3_5"):
        raise ValueError(
            "Qwen3.5 hybrid linear-attention coverage is not implemented; "
            "the optional model must not be partially quantized"
        )
    names = [name for name, _ in model.named_modules()]
    present = [prefix for prefix in _LAYER_PREFIXES if any(name.startswith(prefix) for name in names)]
    if len(present) != 1:
        raise ValueError(
            "Expected exactly one supported decoder layer tree at "
            "model.layers or model.language_model.layers"
        )
    return present[0]


def iter_target_linears(model: nn.Module) -> list[tuple[nn.Module, str, str, nn.Linear]]:
    """(parent, attribute, full name, linear) of every decoder q/k/v/o/gate/up/down projection,
    in model order; vision towers and projectors stay untouched
    (alignquant/models/decoder.py:40-70)."""
    modules = dict(model.named_modules())
    prefix = decoder_layer_prefix(model)
    found = []
    for name, module in modules.items():
        if isinstance(module, nn.Linear) and name.startswith(prefix) and name.endswith(TARGET_PATH_SUFFIXES):
            parent_name, _, attr = name.rpartition(".")
            found.append((modules[parent_name] if parent_name else model, attr, name, module))
    return found
