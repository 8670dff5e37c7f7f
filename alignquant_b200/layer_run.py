"""Run one packed W4/W8-A8 projection on synthetic weights and report its time.

    python -m alignquant_b200.layer_run --n 5120 --k 3072 --rows 2048 --repeat 20
    python -m alignquant_b200.layer_run --n 3072 --k 8192 --rows 1 --scale-mode token --flush-l2
    python -m alignquant_b200.layer_run --n 5120 --k 3072 --rows 1,4,8,16 --layers 28 --with-quantizer

A seeded 60 % W4 layer of the given shape is packed into the artifact format, prepared
once, and the quantize -> linear pair is launched ``--repeat`` times; CUDA events around the
linear calls give the mean kernel time, from which the line reports integer TOPS
(2*M*N*K) and the weight stream in GB/s.  The same command is the small case used for
profiler captures of a single kernel.

With ``--layers L`` (L > 1) the line describes the projection as a decoder runs it: L layers of
the shape with distinct weights (so the weights of a pass exceed the L2 when L x layer bytes does),
launched back to back from one CUDA graph, optionally each preceded by its activation quantizer
(``--with-quantizer``); ``--rows`` may then list several row counts, one JSON line each.
"""

from __future__ import annotations

import argparse
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--n", type=int, required=True, help="output features (multiple of 64)")
    ap.add_argument("--k", type=int, required=True, help="input features (multiple of 64)")
    ap.add_argument("--rows", default="1", help="row count, or a comma-separated list with --layers")
    ap.add_argument("--layers", type=int, default=1, help="distinct layers launched back to back from a CUDA graph")
    ap.add_argument("--with-quantizer", action="store_true", help="with --layers: quantizer before every projection")
    ap.add_argument("--repeat", type=int, default=20)
    ap.add_argument("--w4-fraction", type=float, default=0.6)
    ap.add_argument("--scale-mode", choices=("tile", "token"), default="token")
    ap.add_argument("--out-dtype", choices=("float32", "bfloat16", "float16"), default="bfloat16")
    ap.add_argument("--schedule", default="auto")
    ap.add_argument("--flush-l2", action="store_true", help="overwrite a 512 MB buffer before every launch")
    ap.add_argument("--gemm-tile", choices=("auto", "paired", "narrow", "wide"), default="auto", help="CTA tile of the GEMM")
    ap.add_argument("--gemm-split", type=int, default=0, help="K ranges of the GEMM (1..8), 0 = automatic")
    ap.add_argument("--gemm-separate-rounding", action="store_true",
                    help="GEMM adds a tile with a separately rounded multiply and add (the reference kernels' order)")
    ap.add_argument("--cluster-decode", action="store_true", help="keep the register-staged decode kernel off")
    ap.add_argument("--one-call", action="store_true",
                    help="with --layers: quantizer and projection through alignquant_quant_linear (one launch where it applies)")
    ap.add_argument("--quant-fusion-tiles", type=int, default=None,
                    help="largest layer in tiles for which --one-call runs as one launch (AQ_OPT_QUANT_FUSION_TILES)")
    ap.add_argument("--lookahead", action="store_true",
                    help="with --layers: every projection names the next layer's weights as its L2 look-ahead")
    args = ap.parse_args()

    from alignquant_b200.kernels.cuda import extension as ext
    from alignquant_b200.synthetic import algorithmic_weight_bytes, synthetic_activation, synthetic_module_tensors

    ext.load_extension()
    ext.set_gemm_tile(args.gemm_tile)
    ext.set_gemm_rounding(args.gemm_separate_rounding)
    ext.set_gemm_split(args.gemm_split)
    ext.set_decode_kernel(cluster_only=args.cluster_decode)
    if args.quant_fusion_tiles is not None:
        ext.set_quant_fusion_tiles(args.quant_fusion_tiles)
    device = torch.device("cuda", 0)
    row_counts = [int(v) for v in str(args.rows).split(",")]
    if args.layers > 1:
        chain(args, ext, device, row_counts, synthetic_module_tensors, synthetic_activation, algorithmic_weight_bytes)
        return
    if len(row_counts) != 1:
        raise SystemExit("--rows takes a list only together with --layers")
    args.rows = row_counts[0]
    tensors = synthetic_module_tensors(args.n, args.k, seed=1, w4_fraction=args.w4_fraction, device=device)
    weight_bytes = algorithmic_weight_bytes(tensors)
    weights = ext.prepare_weights(
        tensors["state_bits"], tensors["w4_payload"], tensors["w4_scales"], tensors["w8_payload"], tensors["w8_scales"],
        tensors["w4_row_offsets"], tensors["w8_row_offsets"], n_k=args.k // 64,
    )
    x = synthetic_activation(args.rows, args.k, seed=2, device=device)
    out_dtype = getattr(torch, args.out_dtype)
    out = torch.empty((args.rows, args.n), dtype=out_dtype, device=device)
    junk = torch.empty(512 << 20, dtype=torch.uint8, device=device) if args.flush_l2 else None
    xq, scales = ext.alignquant_activation_quantize_cuda(x, None, scale_mode=args.scale_mode)
    plan = ext.linear_plan(args.rows, args.n // 64, args.k // 64, schedule=args.schedule)
    total_ms = 0.0
    for index in range(args.repeat + 2):
        if junk is not None:
            junk.fill_(index & 0xFF)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        ext.alignquant_linear_prepared(xq, scales, weights, None, schedule=args.schedule, scale_mode=args.scale_mode,
                                       output_dtype=out_dtype, out=out)
        end.record()
        torch.cuda.synchronize()
        if index >= 2:
            total_ms += begin.elapsed_time(end)
    ext.device_status(device)
    seconds = total_ms / 1e3 / args.repeat
    print(json.dumps({
        "n": args.n, "k": args.k, "rows": args.rows, "plan": plan,
        "us": seconds * 1e6, "tops": 2.0 * args.rows * args.n * args.k / seconds / 1e12,
        "weight_gbs": weight_bytes / seconds / 1e9, "scale_mode": args.scale_mode, "out_dtype": args.out_dtype,
        "gemm_tile": args.gemm_tile, "gemm_rounding": "separate" if args.gemm_separate_rounding else "fused",
    }))


def chain(args, ext, device, row_counts, synthetic_module_tensors, synthetic_activation, algorithmic_weight_bytes) -> None:
    """L distinct layers of one shape back to back from a CUDA graph; one JSON line per row count."""
    layers, weight_bytes = [], 0
    for index in range(args.layers):
        tensors = synthetic_module_tensors(args.n, args.k, seed=1 + index, w4_fraction=args.w4_fraction, device=device)
        weight_bytes += algorithmic_weight_bytes(tensors)
        layers.append(ext.prepare_weights(
            tensors["state_bits"], tensors["w4_payload"], tensors["w4_scales"], tensors["w8_payload"], tensors["w8_scales"],
            tensors["w4_row_offsets"], tensors["w8_row_offsets"], n_k=args.k // 64,
        ))
        del tensors
    out_dtype = getattr(torch, args.out_dtype)
    for rows in row_counts:
        x = synthetic_activation(rows, args.k, seed=2 + rows, device=device)
        xq, scales = ext.alignquant_activation_quantize_cuda(x, None, scale_mode=args.scale_mode)
        out = torch.empty((rows, args.n), dtype=out_dtype, device=device)

        def sweep() -> None:
            for index, weights in enumerate(layers):
                ahead = layers[(index + 1) % len(layers)] if args.lookahead else None
                if args.one_call:
                    ext.alignquant_quant_linear(x, weights, None, output_dtype=out_dtype, out=out, quantized=(xq, scales), prefetch=ahead)
                    continue
                if args.with_quantizer:
                    ext.alignquant_activation_quantize_cuda(x, None, scale_mode=args.scale_mode, out=(xq, scales))
                ext.alignquant_linear_prepared(xq, scales, weights, None, schedule=args.schedule, scale_mode=args.scale_mode,
                                               output_dtype=out_dtype, out=out, prefetch=ahead)

        sweep()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            sweep()
        for _ in range(3):
            graph.replay()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        for _ in range(args.repeat):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        ext.device_status(device)
        seconds = begin.elapsed_time(end) / 1e3 / args.repeat / args.layers
        print(json.dumps({
            "n": args.n, "k": args.k, "rows": rows, "layers": args.layers, "with_quantizer": bool(args.with_quantizer),
            "plan": ext.linear_plan(rows, args.n // 64, args.k // 64, schedule=args.schedule),
            "us_per_layer": seconds * 1e6, "weight_gbs": weight_bytes / args.layers / seconds / 1e9,
            "scale_mode": args.scale_mode, "out_dtype": args.out_dtype, "lookahead": bool(args.lookahead),
            "one_call": bool(args.one_call), "one_launch": bool(args.one_call and ext.quant_linear_is_fused(rows, args.n // 64, args.k // 64)),
        }), flush=True)


if __name__ == "__main__":
    main()
