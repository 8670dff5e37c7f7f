"""End-to-end generation runs with random-init decoder models and synthetic artifacts.

    python -m alignquant_b200.runner --model qwen3-4b --batch 8 --prompt-len 2048 --new-tokens 128
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m alignquant_b200.runner --model qwen3-14b --batch 32 --prompt-len 1024 --new-tokens 256

The model is built from a Hugging Face config with the named shape (no checkpoint, no
tokenizer: random weights, random token ids), every decoder projection is replaced by
the packed W4/W8-A8 format with a seeded 60 % W4 map, and greedy decoding is timed with
CUDA events: prefill tokens/s over the prompt pass, decode tokens/s over the generated
tokens (KV cache of fixed size, the decode step captured once into a CUDA graph and
replayed).  Under ``torch.distributed.run`` the decoder is built per rank with 1/tp of the
heads and of the MLP width (tile-aligned tensor parallelism, all-reduce after o_proj and
down_proj); embeddings, norms and the LM head are replicated.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

SHAPES = {
    # name: hidden, intermediate, layers, q heads, kv heads, head dim, vocab, family
    "llama-3.2-3b": (3072, 8192, 28, 24, 8, 128, 128256, "llama"),
    "qwen3-4b": (2560, 9728, 36, 32, 8, 128, 151936, "qwen3"),
    "qwen3-14b": (5120, 17408, 40, 40, 8, 128, 151936, "qwen3"),
    "tiny": (256, 512, 2, 4, 2, 64, 1024, "qwen3"),
}


def _register_grouped_decode_attention() -> str:
    """Attention for the decode step that reads each KV head once.

    With a fixed-size KV cache the stock SDPA path needs a mask and therefore materialises K and V
    once per query head of a group (``repeat_kv``), which dominated the decode step.  Here the
    query heads of one KV group are stacked as rows of one batched matmul against the cached K
    and V; prompts (more than one query position) go through the stock SDPA function.  This is
    runner plumbing around the quantized projections, not part of them.
    """
    from transformers import AttentionInterface
    from transformers.integrations.sdpa_attention import sdpa_attention_forward
    from transformers.masking_utils import AttentionMaskInterface, sdpa_mask

    def grouped_decode_attention(module, query, key, value, attention_mask, dropout=0.0, scaling=None,
                                 is_causal=None, **kwargs):
        batch, q_heads, q_len, head_dim = query.shape
        kv_heads = key.shape[1]
        if q_len != 1 or q_heads % kv_heads != 0:
            return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout,
                                          scaling=scaling, is_causal=is_causal, **kwargs)
        scale = head_dim ** -0.5 if scaling is None else scaling
        q = query.reshape(batch, kv_heads, q_heads // kv_heads, head_dim)
        scores = torch.matmul(q, key.transpose(-1, -2)).float() * scale  # [B, kv heads, group, cache length]
        if attention_mask is not None:
            mask = attention_mask[:, :, :, : key.shape[2]]
            if mask.dtype == torch.bool:  # True = attend
                scores = scores.masked_fill(~mask, float("-inf"))
            else:
                scores = scores + mask.float()
        probs = torch.softmax(scores, dim=-1).to(query.dtype)
        out = torch.matmul(probs, value)  # [B, kv heads, group, head_dim]
        return out.reshape(batch, q_heads, 1, head_dim).transpose(1, 2).contiguous(), None

    AttentionInterface.register("grouped_decode", grouped_decode_attention)
    AttentionMaskInterface.register("grouped_decode", sdpa_mask)  # same masks as the stock SDPA path
    return "grouped_decode"


def build_model(name: str, tp: int, device: torch.device, layers: int | None = None):
    """Random-init decoder of the named shape with 1/tp of the heads and MLP width."""
    import transformers

    hidden, inter, n_layers, heads, kv_heads, head_dim, vocab, family = SHAPES[name]
    if heads % tp or kv_heads % tp or (inter // 64) % tp:
        raise ValueError(f"{name} cannot be split over {tp} ranks on tile boundaries")
    common = dict(
        hidden_size=hidden, intermediate_size=inter // tp, num_hidden_layers=layers or n_layers,
        num_attention_heads=heads // tp, num_key_value_heads=kv_heads // tp, head_dim=head_dim,
        vocab_size=vocab, max_position_embeddings=8192, tie_word_embeddings=False,
    )
    config = (transformers.LlamaConfig if family == "llama" else transformers.Qwen3Config)(**common)
    config._attn_implementation = _register_grouped_decode_attention()
    torch.manual_seed(1234)  # same embeddings / norms / head on every rank
    with torch.device(device):
        model = transformers.AutoModelForCausalLM.from_config(config, dtype=torch.bfloat16)
    return model.eval()


def synthetic_artifact(model, name: str, tp: int, seed: int, device: torch.device) -> dict:
    """Artifact mapping (manifest rows + packed tensors) with the FULL layer shapes."""
    from alignquant_b200.models.decoder import iter_target_linears
    from alignquant_b200.quantization.model import COLUMN_PARALLEL_SUFFIXES
    from alignquant_b200.synthetic import synthetic_module_tensors

    rows, modules = [], {}
    for index, (_, _, full_name, linear) in enumerate(iter_target_linears(model)):
        n, k = int(linear.out_features), int(linear.in_features)
        if full_name.endswith(COLUMN_PARALLEL_SUFFIXES):
            n *= tp
        else:
            k *= tp
        modules[full_name] = synthetic_module_tensors(n, k, seed=seed * 100003 + index, device=device)
        rows.append({
            "layer_name": full_name, "shape": [n, k], "n_j": n // 64, "n_k": k // 64,
            "r5": {"variant": "R5", "t_seed": -1, "v_seeds": [-1] * (k // 64), "u_seeds": [-1] * (n // 64)},
        })
    return {"root": None, "manifest": {"modules": rows}, "modules": modules}


def run(args) -> dict:
    import torch.distributed as dist

    from alignquant_b200.kernels.cuda import extension as ext
    from alignquant_b200.quantization.model import install_alignquant, reset_alignquant_state

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=device)
    ext.load_extension()
    model = build_model(args.model, world, device, layers=args.layers)
    artifact = synthetic_artifact(model, args.model, world, seed=7, device=device)
    reducer = None
    if world > 1 and os.environ.get("ALIGNQUANT_B200_ALLREDUCE", "peer") == "peer":
        from alignquant_b200.kernels.cuda.allreduce import PeerAllReduce

        reducer = PeerAllReduce(64 * SHAPES[args.model][0], device)  # up to 64 rows of hidden-size partials
    installed, install_meta = install_alignquant(model, artifact, device, scale_mode=args.scale_mode, tp_rank=rank,
                                                 tp_size=world, peer_allreduce=reducer,
                                                 fuse_norms=not getattr(args, "stock_norms", False))
    del artifact
    torch.cuda.empty_cache()

    gen = torch.Generator(device=device).manual_seed(99)
    vocab = SHAPES[args.model][6]
    prompt = torch.randint(0, vocab, (args.batch, args.prompt_len), generator=gen, device=device)

    def generate():
        """Greedy decoding on a static KV cache; the decode step is replayed from a CUDA graph."""
        from transformers import StaticCache

        reset_alignquant_state(model)
        cache = StaticCache(config=model.config, max_cache_len=args.prompt_len + args.new_tokens)
        events = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        token = torch.empty((args.batch, 1), dtype=torch.long, device=device)
        position = torch.empty((1,), dtype=torch.long, device=device)

        def step():
            out = model(input_ids=token, past_key_values=cache, cache_position=position, use_cache=True)
            token.copy_(out.logits[:, -1].argmax(dim=-1, keepdim=True))
            position.add_(1)

        mode = "eager"
        with torch.inference_mode():
            events[0].record()
            out = model(input_ids=prompt, past_key_values=cache,
                        cache_position=torch.arange(args.prompt_len, device=device), use_cache=True)
            token.copy_(out.logits[:, -1].argmax(dim=-1, keepdim=True))
            position.fill_(args.prompt_len)
            events[1].record()
            steps = args.new_tokens - 1
            eager_steps = min(2, steps) if args.decode_graph else steps
            for _ in range(eager_steps):
                step()
            graph = None
            if steps > eager_steps:
                try:
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        step()
                    mode = "cuda graph replay"
                except Exception as error:  # an op of the model that cannot be captured
                    if rank == 0:
                        print(f"[runner] decode step not captured ({type(error).__name__}: {error}); eager", flush=True)
                    graph = None
                    torch.cuda.synchronize()
            events[2].record()
            for _ in range(steps - eager_steps):
                if graph is not None:
                    graph.replay()
                else:
                    step()
            events[3].record()
        torch.cuda.synchronize()
        timed_steps = steps - eager_steps if steps > eager_steps else steps
        decode_seconds = (events[2].elapsed_time(events[3]) if steps > eager_steps else events[1].elapsed_time(events[2])) / 1e3
        return events[0].elapsed_time(events[1]) / 1e3, decode_seconds, timed_steps, mode

    if args.warmup:
        generate()
    prefill_s, decode_s, decode_steps, decode_mode = generate()
    ext.device_status(device)
    if world > 1:
        t = torch.tensor([prefill_s, decode_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        prefill_s, decode_s = (float(v) for v in t)
    return {
        "model": args.model, "layers": args.layers or SHAPES[args.model][2], "tp": world, "batch": args.batch,
        "prompt_len": args.prompt_len, "new_tokens": args.new_tokens, "scale_mode": args.scale_mode,
        "quantized_modules": len(installed), "fused_norms": install_meta["fused_norm_count"],
        "prefill_tokens_per_s": args.batch * args.prompt_len / prefill_s,
        "decode_tokens_per_s": args.batch * decode_steps / decode_s, "decode_steps_timed": decode_steps,
        "decode_launch": decode_mode, "decode_ms_per_step": decode_s * 1e3 / max(decode_steps, 1),
        "prefill_s": prefill_s, "decode_s": decode_s, "rank": rank, "world": world,
    }


def generation_record(model: str, batch: int, prompt_len: int, new_tokens: int, *, layers: int | None = None,
                      scale_mode: str = "token", warmup: int = 1) -> dict:
    """One generation run as a dict (what ``main`` prints); callable from another script.

    Reads RANK / LOCAL_RANK / WORLD_SIZE from the environment and uses the default process
    group if one is initialised already.
    """
    args = argparse.Namespace(model=model, batch=batch, prompt_len=prompt_len, new_tokens=new_tokens, layers=layers,
                              scale_mode=scale_mode, warmup=warmup, decode_graph=True)
    return run(args)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", choices=sorted(SHAPES), default="qwen3-4b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--layers", type=int, default=None, help="override the number of decoder layers")
    ap.add_argument("--scale-mode", choices=("tile", "token"), default="token")
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--stock-norms", action="store_true",
                    help="keep the model's RMSNorm modules (default: norm + activation quantizer as one kernel)")
    ap.add_argument("--no-decode-graph", dest="decode_graph", action="store_false",
                    help="run every decode step eagerly instead of replaying a CUDA graph")
    result = run(ap.parse_args())
    if result["rank"] == 0:
        print(json.dumps(result), flush=True)
    if result["world"] > 1:
        # communicators whose collectives live in captured graphs are not torn down (that was
        # seen to block); every rank has synchronised and leaves
        import sys

        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
