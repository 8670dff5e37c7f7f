"""Host-side logic of the model glue on CPU: grouping, metadata, tile-aligned sharding.

The kernels are replaced by the CPU oracle here (test-only monkeypatching of the three
extension calls the runtime makes), so that grouping, slicing, caching and the
tensor-parallel algebra -- column shards concatenate, row-shard partial sums add up -- are
checked without a GPU; the all-reduce runs over two gloo ranks.
"""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from alignquant_b200.quantization import artifact as fmt
from alignquant_b200.quantization import exact
from alignquant_b200.quantization import model as glue
from oracle import alignquant_oracle as oc


def test_transform_metadata_matches_reference_fixture(golden_dir):
    g = dict(np.load(golden_dir / "transforms.npz"))
    for seed, meta in zip(g["seeds"], g["metadata"]):
        assert np.array_equal(exact.structured_transform_metadata(int(seed)).numpy(), meta)
    with pytest.raises(ValueError):
        exact.structured_transform_metadata(-2)


def test_projection_groups_follow_reference_rules():
    names = [f"model.layers.0.self_attn.{p}_proj" for p in "qkvo"] + [f"model.layers.0.mlp.{p}_proj" for p in ("gate", "up", "down")]
    groups = glue.projection_groups(names)
    assert groups["model.layers.0.self_attn.qkv"] == tuple(f"model.layers.0.self_attn.{p}_proj" for p in "kqv")
    assert groups["model.layers.0.mlp.gate_up"] == ("model.layers.0.mlp.gate_proj", "model.layers.0.mlp.up_proj")
    assert groups["model.layers.0.self_attn.o_proj"] == ("model.layers.0.self_attn.o_proj",)
    with pytest.raises(ValueError, match="Incomplete projection group"):
        glue.projection_groups(names[:2])


@pytest.mark.parametrize("rows,cols", [((1, 3), None), (None, (2, 5)), ((0, 1), (0, 1))])
def test_shard_is_an_exact_sub_selection(rows, cols):
    packed, states, tiles, scales = oc.synthetic_layer(256, 320, seed=11)
    t = {k: torch.from_numpy(v) for k, v in packed.items()}
    shard = fmt.shard_w4w8_replacement_module(t, n_j=4, n_k=5, rows=rows, cols=cols)
    j0, j1 = rows or (0, 4)
    k0, k1 = cols or (0, 5)
    fmt.validate_w4w8_replacement_module(shard, n_j=j1 - j0, n_k=k1 - k0)
    s_states, s_tiles, s_scales = oc.unpack_module({k: v.numpy() for k, v in shard.items()}, j1 - j0, k1 - k0)
    assert np.array_equal(s_states, states[j0:j1, k0:k1])
    assert np.array_equal(s_tiles, tiles[j0:j1, k0:k1])
    assert np.array_equal(s_scales, scales[j0:j1, k0:k1])


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_tensor_parallel_ranges_of_the_qwen3_14b_shape(tp):
    """Head groups and MLP width of the 14B shape split on tile borders at every rank count the
    multi-GPU configuration names: the ranks' ranges are disjoint, in order and cover everything."""
    hidden, inter, heads, kv_heads, head_dim = 5120, 17408, 40, 8, 128
    totals = {"q_proj rows": heads * head_dim // 64, "k_proj rows": kv_heads * head_dim // 64,
              "gate_proj rows": inter // 64, "o_proj k": heads * head_dim // 64, "down_proj k": inter // 64}
    for what, total in totals.items():
        ranges = [glue.tensor_parallel_range(total, rank, tp, what) for rank in range(tp)]
        assert ranges[0][0] == 0 and ranges[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        assert {hi - lo for lo, hi in ranges} == {total // tp}
    if tp == 8:  # 5 query heads, 1 KV head, 2176 MLP columns per rank
        assert glue.tensor_parallel_range(totals["q_proj rows"], 3, 8, "q") == (30, 40)
        assert glue.tensor_parallel_range(totals["k_proj rows"], 3, 8, "k") == (6, 8)
        assert glue.tensor_parallel_range(totals["down_proj k"], 7, 8, "down") == (238, 272)
    assert hidden % 64 == 0


def test_tensor_parallel_range_rejects_uneven_and_invalid_ranks():
    with pytest.raises(ValueError, match="cannot be split evenly"):
        glue.tensor_parallel_range(272, 0, 3, "down_proj k")
    with pytest.raises(ValueError, match="Invalid tensor-parallel rank"):
        glue.tensor_parallel_range(272, 8, 8, "down_proj k")


# ---- a tiny decoder and a CPU stand-in for the three extension calls -------------------------


class _Attn(nn.Module):
    def __init__(self, hidden, q_out, kv_out, o_in):
        super().__init__()
        self.q_proj = nn.Linear(hidden, q_out, bias=False)
        self.k_proj = nn.Linear(hidden, kv_out, bias=False)
        self.v_proj = nn.Linear(hidden, kv_out, bias=True)
        self.o_proj = nn.Linear(o_in, hidden, bias=False)


class _Mlp(nn.Module):
    def __init__(self, hidden, inter_out, inter_in):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter_out, bias=False)
        self.up_proj = nn.Linear(hidden, inter_out, bias=False)
        self.down_proj = nn.Linear(inter_in, hidden, bias=False)


class TinyRMSNorm(nn.Module):
    """The arithmetic of the Llama / Qwen3 RMSNorm module."""

    def __init__(self, hidden, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.linspace(0.5, 1.5, hidden))
        self.variance_epsilon = eps

    def forward(self, hidden_states):
        dtype = hidden_states.dtype
        x = hidden_states.to(torch.float32)
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.variance_epsilon)
        return self.weight * x.to(dtype)


class _Layer(nn.Module):
    def __init__(self, hidden, q, kv, inter, tp, norms=False):
        super().__init__()
        self.self_attn = _Attn(hidden, q // tp, kv // tp, q // tp)
        self.mlp = _Mlp(hidden, inter // tp, inter // tp)
        if norms:
            self.input_layernorm = TinyRMSNorm(hidden)
            self.post_attention_layernorm = TinyRMSNorm(hidden)


class _Tiny(nn.Module):
    def __init__(self, tp=1, hidden=128, q=256, kv=128, inter=256, layers=1, norms=False):
        super().__init__()
        self.config = type("C", (), {"model_type": "llama"})()
        self.model = nn.Module()
        self.model.layers = nn.ModuleList([_Layer(hidden, q, kv, inter, tp, norms) for _ in range(layers)])


FULL_SHAPES = {
    "model.layers.0.self_attn.q_proj": (256, 128), "model.layers.0.self_attn.k_proj": (128, 128),
    "model.layers.0.self_attn.v_proj": (128, 128), "model.layers.0.self_attn.o_proj": (128, 256),
    "model.layers.0.mlp.gate_proj": (256, 128), "model.layers.0.mlp.up_proj": (256, 128),
    "model.layers.0.mlp.down_proj": (128, 256),
}


def _artifact():
    rows, modules, dense = [], {}, {}
    for index, (name, (n, k)) in enumerate(FULL_SHAPES.items()):
        packed, states, tiles, scales = oc.synthetic_layer(n, k, seed=40 + index)
        modules[name] = {key: torch.from_numpy(value) for key, value in packed.items()}
        rows.append({"layer_name": name, "shape": [n, k], "n_j": n // 64, "n_k": k // 64,
                     "r5": {"variant": "R5", "t_seed": -1, "v_seeds": [-1] * (k // 64), "u_seeds": [-1] * (n // 64)}})
        w = tiles.astype(np.float64) * scales.astype(np.float64)[:, :, None, None]
        dense[name] = w.transpose(0, 2, 1, 3).reshape(n, k)
    return {"root": None, "manifest": {"modules": rows}, "modules": modules}, dense


class _CpuWeights:
    def __init__(self, tensors, n_k):
        raw = {k: v.cpu().numpy() for k, v in tensors.items()}
        self.n_j, self.n_k = raw["w4_row_offsets"].size - 1, n_k
        _, self.tiles, self.scales = oc.unpack_module(raw, self.n_j, n_k)


def _patch(monkeypatch):
    def prepare(*tensors, n_k):
        return _CpuWeights(dict(zip(fmt.REPLACEMENT_TENSOR_NAMES, tensors)), n_k)

    def quantize(x, v_metadata, *, scale_mode="tile", **_):
        q, s = oc.a8_token_quantize(x.float().numpy())
        return torch.from_numpy(q), torch.from_numpy(s)

    def linear(xq, scales, weights, u_metadata, *, scale_mode="tile", output_dtype=torch.float32, **_):
        a = oc.expand_act_scales(scales.numpy(), xq.shape[0], weights.n_k, "token")
        return torch.from_numpy(oc.dequant_matmul_fp64(xq.numpy(), a, weights.tiles, weights.scales)).to(output_dtype)

    def quant_linear(x, weights, u_metadata, *, output_dtype=torch.float32, reducer=None, **_):
        if reducer is not None:
            return None  # no peer-memory kernels on the CPU: the glue falls back to dist.all_reduce
        return linear(*quantize(x, None), weights, u_metadata, output_dtype=output_dtype)

    monkeypatch.setattr(glue._ext, "alignquant_quant_linear", quant_linear)
    monkeypatch.setattr(glue._ext, "prepare_weights", prepare)
    monkeypatch.setattr(glue._ext, "alignquant_activation_quantize_cuda", quantize)
    monkeypatch.setattr(glue._ext, "alignquant_linear_prepared", linear)
    monkeypatch.setattr(glue, "_cuda_device", lambda value: torch.device("cpu"))


def test_install_groups_caches_and_slices(monkeypatch):
    _patch(monkeypatch)
    artifact, dense = _artifact()
    model = _Tiny()
    installed, meta = glue.install_alignquant(model, artifact, "cpu", scale_mode="token")
    assert meta["module_count"] == 7 and meta["projection_group_count"] == 4
    attn = model.model.layers[0].self_attn
    x = torch.from_numpy(oc.synthetic_activation(5, 128, seed=3).astype(np.float32))
    q, k, v = attn.q_proj(x), attn.k_proj(x), attn.v_proj(x)
    xq, s = oc.a8_token_quantize(x.numpy())
    xd = xq.astype(np.float64) * s[:, None]
    for got, name in ((q, "q_proj"), (k, "k_proj")):
        assert np.allclose(got.numpy(), xd @ dense[f"model.layers.0.self_attn.{name}"].T, rtol=1e-5, atol=1e-5)
    want_v = xd @ dense["model.layers.0.self_attn.v_proj"].T + attn.v_proj.bias.numpy()
    assert np.allclose(v.numpy(), want_v, rtol=1e-5, atol=1e-5)
    # protocol errors of the shared projection, as in the reference
    attn.q_proj(x)
    with pytest.raises(RuntimeError, match="called twice"):
        attn.q_proj(x)
    glue.reset_alignquant_state(model)
    attn.q_proj(x)
    with pytest.raises(RuntimeError, match="received a new activation"):
        attn.k_proj(x + 1)
    glue.reset_alignquant_state(model)
    with pytest.raises(ValueError, match="coverage mismatch"):
        bad = dict(artifact, manifest={"modules": artifact["manifest"]["modules"][:-1]})
        glue.install_alignquant(_Tiny(), bad, "cpu")


def test_fuse_norms_replaces_only_the_norms_in_front_of_projection_groups(monkeypatch):
    _patch(monkeypatch)
    artifact, _ = _artifact()
    model = _Tiny(norms=True)
    _, meta = glue.install_alignquant(model, artifact, "cpu", scale_mode="token", fuse_norms=True)
    layer = model.model.layers[0]
    assert meta["fused_norm_count"] == 2
    assert isinstance(layer.input_layernorm, glue.AlignQuantRMSNorm)
    assert isinstance(layer.post_attention_layernorm, glue.AlignQuantRMSNorm)
    assert layer.input_layernorm.eps == 1e-5 and layer.input_layernorm.weight is layer.input_layernorm.original.weight
    # a CPU tensor goes through the original module, and nothing is left on the result
    x = torch.randn(3, 128)
    y = layer.input_layernorm(x)
    assert torch.equal(y, layer.input_layernorm.original(x)) and not hasattr(y, "_alignquant_quantized")
    # tile scale mode (the reference's) keeps the stock norms
    plain = _Tiny(norms=True)
    _, meta = glue.install_alignquant(plain, artifact, "cpu", fuse_norms=True)
    assert meta["fused_norm_count"] == 0 and isinstance(plain.model.layers[0].input_layernorm, TinyRMSNorm)


def _tp_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import pytest as _pytest

        mp_patch = _pytest.MonkeyPatch()
        _patch(mp_patch)
        artifact, dense = _artifact()
        model = _Tiny(tp=world)
        glue.install_alignquant(model, artifact, "cpu", scale_mode="token", tp_rank=rank, tp_size=world)
        layer = model.model.layers[0]
        x = torch.from_numpy(oc.synthetic_activation(3, 128, seed=5).astype(np.float32))
        q = layer.self_attn.q_proj(x)
        layer.self_attn.k_proj(x), layer.self_attn.v_proj(x)
        gathered = [torch.empty_like(q) for _ in range(world)]
        dist.all_gather(gathered, q)
        # row parallel: every rank feeds its slice of the full intermediate activation
        full = torch.from_numpy(oc.synthetic_activation(3, 256, seed=6).astype(np.float32))
        # per-token scales are shard-local, so quantize per shard for the expected value too
        part = full[:, rank * 128 : (rank + 1) * 128].contiguous()
        down = layer.mlp.down_proj(part)
        if rank == 0:
            results["q"] = torch.cat(gathered, dim=1).numpy()
            results["down"] = down.numpy()
        mp_patch.undo()
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_shards_recombine_over_gloo():
    world, port = 2, 29511 + os.getpid() % 200
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_tp_worker, args=(world, port, results), nprocs=world, join=True)
    _, dense = _artifact()
    x = oc.synthetic_activation(3, 128, seed=5).astype(np.float32)
    xq, s = oc.a8_token_quantize(x)
    want_q = (xq.astype(np.float64) * s[:, None]) @ dense["model.layers.0.self_attn.q_proj"].T
    assert np.allclose(results["q"], want_q, rtol=1e-5, atol=1e-5)  # column shards concatenate
    full = oc.synthetic_activation(3, 256, seed=6).astype(np.float32)
    want_down = 0
    for r in range(world):
        pq, ps = oc.a8_token_quantize(np.ascontiguousarray(full[:, r * 128 : (r + 1) * 128]))
        want_down = want_down + (pq.astype(np.float64) * ps[:, None]) @ dense["model.layers.0.mlp.down_proj"][:, r * 128 : (r + 1) * 128].T
    assert np.allclose(results["down"], want_down, rtol=1e-5, atol=1e-5)  # row-shard partials add up
