"""Benchmark of the mixed W4/W8-A8 linear hot path on B200.

Workload (one "step"): the decode sweep over every quantized linear of a random-init
Llama-3.2-3B-shaped decoder -- 28 layers x {qkv 3072->5120, o 3072->3072,
gate_up 3072->16384, down 8192->3072}, row counts M in {1, 4, 8, 16}, 60 % W4 tiles,
per-token INT8 activations -- i.e. 448 (activation quantizer -> packed GEMV) pairs
over ~2 GB of distinct weights (larger than L2, so no flush is needed between steps).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

With N > 1 (launched under torch.distributed.run) every layer is sharded
tensor-parallel: column shards of qkv/gate_up, row shards of o/down whose [M, 3072]
partials are summed over the ranks through peer memory inside the GEMV kernel (with
ALIGNQUANT_B200_ALLREDUCE=nccl: by an NCCL all-reduce); total work is fixed ("strong" scaling).

Rank 0 prints one JSON line.  `value` is algorithmic bytes per second with every
input resident in HBM (CUDA-graph replay, CUDA-event timing, max over ranks); `e2e`
is the same sweep through the public Python API from pinned host buffers, host<->device
copies included; `roofline` times the packed-GEMV kernel alone; `cpu_baseline` times
the CPU oracle (the reference's dequantize-and-matmul recipe) on a bounded sample.
`--impl reference` runs only that CPU arm.

Every quantizer + projection pair is one call of `aq_quant_linear` (one launch where the
quantizer runs inside the GEMV kernel, two otherwise).  With `--lookahead` every projection also
names the weights of the projection that runs after it (`next_prepared`), as the quantized
modules of an installed model do; between back-to-back projections that measured slower, so
it is off here.

The line also carries the other two legs of the metric (`--legs` selects them):
`prefill` -- the same four Llama-3.2-3B shapes at M = 2048 with bf16 activations through the
tensor-memory GEMM, in integer TOPS against the nominal 4.5 POPS and against this GPU's own
back-to-back `tcgen05.mma kind::i8` rate (`aq_measure_int8_peak`); `generation` -- prompt and
generated tokens per second of a random-init Qwen3-4B-shaped model on one GPU, or of the
tensor-parallel Qwen3-14B-shaped model on N > 1 GPUs, with a shortened, stated token count.
With N > 1 the fused projection + rank sum is first checked against the two-step path
(`tp_check`); a mismatch ends the run with a non-zero exit code.  `tp_one_call_bits` says whether the
one-call form gave the bits of quantizer + fused projection.  A multi-GPU run without a result
after `--watchdog` seconds ends itself with a line that names the stage it was in.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

HIDDEN, INTER, LAYERS = 3072, 8192, 28
ROW_COUNTS = (1, 4, 8, 16)
# name -> (N, K, tensor-parallel split axis)
GROUPS = {
    "qkv": (5120, HIDDEN, "n"),
    "o": (HIDDEN, HIDDEN, "k"),
    "gate_up": (2 * INTER, HIDDEN, "n"),
    "down": (HIDDEN, INTER, "k"),
}
WORKLOAD = "llama-3.2-3b decode sweep: 28 layers x (qkv, o, gate_up, down), M in {1,4,8,16}, 60% W4, per-token A8"
FALLBACK_HBM_GBS = 6650.0
NOMINAL_INT8_TOPS = 4500.0
PREFILL_ROWS = 2048
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the packed-GEMV kernel per projection
# group at M = 1, one GPU, from an ncu capture of this sweep's four shapes with the L2 flushed before
# every launch (the sweep's own condition: its 2 GB of weights per step never stay in the L2).
# None until captured; N > 1 is not captured.
NCU_DRAM_BYTES_PER_LAUNCH = {"qkv": 11092736, "o": 6677248, "gate_up": 35363584, "down": 17704192}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("native", "reference"), default="native")
    ap.add_argument("--legs", default="decode,prefill,generation",
                    help="comma-separated legs besides the decode sweep: prefill, generation")
    ap.add_argument("--gen-tokens", type=int, default=32, help="generated tokens of the generation leg")
    ap.add_argument("--watchdog", type=int, default=300,
                    help="multi-GPU runs only: seconds after which a run without a result ends itself with a diagnostic "
                         "line (0: never)")
    ap.add_argument("--lookahead", action="store_true",
                    help="every projection of the sweep names the next one's weights as its L2 look-ahead (off by default: "
                         "between back-to-back projections it was measured to cost about 2 %%)")
    ap.add_argument("--cluster-decode", action="store_true",
                    help="keep the register-staged decode kernel off (AQ_DECODE_KERNEL_CLUSTER), for comparison")
    return ap.parse_args()


def hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = (
        "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return False
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, max_clocks, reasons = [], [], set()
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clocks.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(self.NAMES, parts[2:]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if clocks:
            self.result = {
                "sm_mhz": statistics.median(clocks), "sm_max_mhz": max(max_clocks),
                "reasons": sorted(reasons), "samples": len(clocks),
            }
        return False


# ---------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's dequantize-and-matmul
# ---------------------------------------------------------------------------


def artifact_bytes(n_j: int, n_k: int, w4_tiles: int) -> int:
    """Weight-side algorithmic bytes of a layer in the artifact format."""
    tiles = n_j * n_k
    return w4_tiles * 2048 + (tiles - w4_tiles) * 4096 + 4 * tiles + (tiles + 7) // 8 + 8 * (n_j + 1)


def call_bytes(m: int, n: int, k: int, weight_bytes: int, out_bytes: int = 2) -> int:
    """Algorithmic bytes of one quantize -> linear pair (fp16 in, per-token scales, fp16 out unless stated)."""
    quantizer = m * k * 2 + m * k + 4 * m
    linear = weight_bytes + m * k + 4 * m + m * n * out_bytes
    return quantizer + linear


class CpuSample:
    """One decoder layer's four projection groups at M in {1,4,8,16} on the host cores."""

    description = "1 of 28 layers: (qkv, o, gate_up, down) x M in {1,4,8,16}, FP64 dequantize-and-matmul (numpy/BLAS)"

    def __init__(self):
        import numpy as np

        from oracle import alignquant_oracle as oc

        self.oc, self.np = oc, np
        self.cases = []
        self.bytes = 0
        for index, (name, (n, k, _)) in enumerate(GROUPS.items()):
            _, states, tiles, scales = oc.synthetic_layer(n, k, seed=100 + index, pack=False)
            w_bytes = artifact_bytes(n // 64, k // 64, int((states == oc.P4).sum()))
            for m in ROW_COUNTS:
                x = oc.synthetic_activation(m, k, seed=7 * m + index)
                self.cases.append((x, tiles, scales, k // 64))
                self.bytes += call_bytes(m, n, k, w_bytes)

    def run(self) -> float:
        oc = self.oc
        start = time.perf_counter()
        for x, tiles, scales, n_k in self.cases:
            xq, a_s = oc.a8_token_quantize(x)
            a_mk = oc.expand_act_scales(a_s, x.shape[0], n_k, "token")
            oc.dequant_matmul_fp64(xq, a_mk, tiles, scales)
        return time.perf_counter() - start


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    sample = CpuSample()
    for _ in range(min(args.warmup, 1)):
        sample.run()
    times = [sample.run()]
    budget_steps = max(1, int(120.0 / max(times[0], 1e-3)))  # keep the whole arm within a few minutes
    while len(times) < min(max(1, args.steps), budget_steps):
        times.append(sample.run())
    per_step = sum(times) / len(times)
    value = sample.bytes / per_step / 1e9
    line = {
        "metric": "decode_gemv_hbm_gbs", "value": value, "unit": "GB/s", "impl": "reference",
        "n_gpus": args.gpus, "steps": len(times), "warmup": min(args.warmup, 1), "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": {"workload": WORKLOAD, "step": CpuSample.description},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": CpuSample.description},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------


def prefill_leg(ext, device, steps: int) -> dict:
    """The four Llama-3.2-3B shapes at M = 2048, bf16 activations, through the tensor-memory GEMM."""
    import torch

    from alignquant_b200.synthetic import synthetic_activation, synthetic_module_tensors

    shapes = {}
    total_ops, total_seconds = 0.0, 0.0
    for index, (name, (n, k, _)) in enumerate(GROUPS.items()):
        tensors = synthetic_module_tensors(n, k, seed=900 + index, device=device)
        weights = ext.prepare_weights(
            tensors["state_bits"], tensors["w4_payload"], tensors["w4_scales"], tensors["w8_payload"], tensors["w8_scales"],
            tensors["w4_row_offsets"], tensors["w8_row_offsets"], n_k=k // 64,
        )
        del tensors
        x = synthetic_activation(PREFILL_ROWS, k, seed=950 + index, dtype=torch.bfloat16, device=device)
        xq, a_s = ext.alignquant_activation_quantize_cuda(x, None, scale_mode="token")
        out = torch.empty((PREFILL_ROWS, n), dtype=torch.bfloat16, device=device)

        def call():
            ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token", output_dtype=torch.bfloat16, out=out)

        for _ in range(3):
            call()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        for _ in range(steps):
            call()
        end.record()
        torch.cuda.synchronize()
        seconds = begin.elapsed_time(end) / 1e3 / steps
        ops = 2.0 * PREFILL_ROWS * n * k
        plan = ext.linear_plan(PREFILL_ROWS, n // 64, k // 64)
        shapes[name] = {"n": n, "k": k, "us": seconds * 1e6, "tops": ops / seconds / 1e12, "kernel": plan["kernel"]}
        total_ops += ops
        total_seconds += seconds
        del weights, out, xq, a_s, x
    ext.device_status(device)
    # The activation quantizer at prefill sizes is a plain streaming kernel: bf16 rows in, int8 rows and a
    # scale per row out.  Eight distinct inputs of 134 MB each (more than the L2) are walked round robin.
    q_rows, q_k, q_buffers = 8192, 8192, 8
    xs = [synthetic_activation(q_rows, q_k, seed=970 + i, dtype=torch.bfloat16, device=device) for i in range(q_buffers)]
    q_out = (torch.empty((q_rows, q_k), dtype=torch.int8, device=device), torch.empty((q_rows,), dtype=torch.float32, device=device))
    for i in range(3):
        ext.alignquant_activation_quantize_cuda(xs[i % q_buffers], None, scale_mode="token", out=q_out)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for i in range(2 * q_buffers):
        ext.alignquant_activation_quantize_cuda(xs[i % q_buffers], None, scale_mode="token", out=q_out)
    end.record()
    torch.cuda.synchronize()
    q_seconds = begin.elapsed_time(end) / 1e3 / (2 * q_buffers)
    q_bytes = q_rows * q_k * 2 + q_rows * q_k + 4 * q_rows
    peak, peak_source = hbm_peak()
    quantizer = {"rows": q_rows, "k": q_k, "us": q_seconds * 1e6, "gbs": q_bytes / q_seconds / 1e9,
                 "frac_of_hbm_peak": q_bytes / q_seconds / 1e9 / peak, "hbm_peak_gbs": peak, "peak_source": peak_source,
                 "bytes": q_bytes, "kernel": "quantize_token_kernel<bf16> (per-token scales)"}
    del xs, q_out
    measured_peak = ext.measure_int8_peak(4096, device)
    tops = total_ops / total_seconds / 1e12
    return {
        "quantizer": quantizer,
        "workload": f"llama-3.2-3b prefill: (qkv, o, gate_up, down) at M = {PREFILL_ROWS}, bf16 activations, bf16 results, 60% W4",
        "metric": "prefill_gemm_int8_tops", "value": tops, "unit": "TOPS", "shapes": shapes,
        "frac_of_nominal_peak": tops / NOMINAL_INT8_TOPS, "nominal_peak_tops": NOMINAL_INT8_TOPS,
        "frac_of_measured_peak": tops / measured_peak, "measured_peak_tops": measured_peak,
        "measured_peak_how": "aq_measure_int8_peak: back-to-back tcgen05.mma kind::i8 M128 N256 K32 on every SM, no operand traffic, no drain",
        "drain": "fused multiply-add per K64 tile (AQ_GEMM_ROUNDING_FUSED)",
        "inputs": "weights (35 MB at most) stay in the 126 MB L2 between repeats; the kernel is bound by the tensor pipe and the CUDA-core drain, not by HBM",
    }


def generation_leg(world: int, tokens: int) -> dict:
    """Prompt and generated tokens per second of a random-init model with synthetic artifacts."""
    from alignquant_b200.runner import generation_record

    if world == 1:
        model, batch, prompt_len, full_tokens = "qwen3-4b", 8, 2048, 128
    else:
        model, batch, prompt_len, full_tokens = "qwen3-14b", 32, 1024, 256
    record = generation_record(model, batch, prompt_len, tokens, warmup=1)
    keep = ("model", "layers", "tp", "batch", "prompt_len", "new_tokens", "prefill_tokens_per_s", "decode_tokens_per_s",
            "decode_ms_per_step", "decode_launch", "decode_steps_timed", "quantized_modules", "fused_norms")
    result = {key: record[key] for key in keep}
    result["note"] = (f"{tokens} generated tokens instead of the configuration's {full_tokens} (the decode step does not "
                      "depend on the count beyond the KV-cache length); random-init weights, random token ids")
    return result


class Watchdog:
    """Ends a multi-GPU run that has produced no result in time, naming the stage every rank was in.

    Every device-side wait of the library is bounded, so the GPUs stay usable whatever happens; what
    this guards against is a host-side stall (a collective that one rank never joins, a rendezvous
    that never completes) holding a whole node until an outer limit kills the job without a word.
    """

    def __init__(self, seconds: int, rank: int, world: int):
        import threading

        self.stage, self.rank, self.world, self.seconds = "start", rank, world, seconds
        self.timer = None
        if seconds > 0 and world > 1:
            self.timer = threading.Timer(seconds, self.fire)
            self.timer.daemon = True
            self.timer.start()

    def fire(self) -> None:
        print(f"[bench] rank {self.rank}: no result after {self.seconds} s, stage '{self.stage}'", file=sys.stderr, flush=True)
        if self.rank == 0:
            print(json.dumps({"metric": "decode_gemv_hbm_gbs", "n_gpus": self.world,
                              "error": f"no result after {self.seconds} s; rank 0 was in stage '{self.stage}'"}), flush=True)
        os._exit(5)

    def cancel(self) -> None:
        if self.timer is not None:
            self.timer.cancel()


def run_native(args) -> None:
    import torch
    import torch.distributed as dist

    from alignquant_b200.kernels.cuda import extension as ext
    from alignquant_b200.synthetic import algorithmic_weight_bytes, synthetic_activation, synthetic_module_tensors

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")
    legs = {leg.strip() for leg in args.legs.split(",") if leg.strip()}
    watchdog = Watchdog(args.watchdog, rank, world)
    watchdog.stage = "process group"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ext.load_extension()
    watchdog.stage = "exchange buffers"
    ext.set_decode_kernel(cluster_only=args.cluster_decode)
    reducer = None
    if world > 1 and os.environ.get("ALIGNQUANT_B200_ALLREDUCE", "peer") == "peer":
        from alignquant_b200.kernels.cuda.allreduce import PeerAllReduce

        reducer = PeerAllReduce(max(ROW_COUNTS) * max(n for n, _, axis in GROUPS.values() if axis == "k"), device)

    def all_reduce(tensor) -> None:
        if reducer is not None:
            reducer(tensor)
        else:
            dist.all_reduce(tensor)

    watchdog.stage = "weights"
    # ---- build the sharded model: prepared weight images only (raw arenas are freed)
    layers = []
    weight_bytes = {}
    for layer in range(LAYERS):
        entry = {}
        for index, (name, (n, k, axis)) in enumerate(GROUPS.items()):
            n_local = n // world if axis == "n" else n
            k_local = k // world if axis == "k" else k
            tensors = synthetic_module_tensors(n_local, k_local, seed=((layer * 8 + index) * 64 + rank), device=device)
            weight_bytes[(layer, name)] = algorithmic_weight_bytes(tensors)
            entry[name] = ext.prepare_weights(
                tensors["state_bits"], tensors["w4_payload"], tensors["w4_scales"], tensors["w8_payload"],
                tensors["w8_scales"], tensors["w4_row_offsets"], tensors["w8_row_offsets"], n_k=k_local // 64,
            )
            del tensors
        layers.append(entry)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()

    local_shape = {
        name: (n // world if axis == "n" else n, k // world if axis == "k" else k) for name, (n, k, axis) in GROUPS.items()
    }
    acts = {(m, name): synthetic_activation(m, local_shape[name][1], seed=m * 16 + i, device=device)
            for m in ROW_COUNTS for i, name in enumerate(GROUPS)}
    qbuf = {key: (torch.empty(x.shape, dtype=torch.int8, device=device), torch.empty((x.shape[0],), dtype=torch.float32, device=device))
            for key, x in acts.items()}
    # fp16 results, as the quantized module returns them; the partial results of row-parallel
    # layers under tensor parallelism stay fp32 for the sum over the ranks
    out_dtype = {name: torch.float32 if world > 1 and axis == "k" else torch.float16 for name, (_, _, axis) in GROUPS.items()}
    out_bytes = {name: 4 if dtype == torch.float32 else 2 for name, dtype in out_dtype.items()}
    outs = {(m, name): torch.empty((m, local_shape[name][0]), dtype=out_dtype[name], device=device)
            for m in ROW_COUNTS for name in GROUPS}

    # The step as a flat list of calls; every call names the weights of the call after it (the
    # first call of the next step after the last one) as its look-ahead.
    calls = [(m, li, name) for m in ROW_COUNTS for li in range(LAYERS) for name in GROUPS]
    lookahead = args.lookahead

    def next_weights(position: int):
        if not lookahead:
            return None
        _, li, name = calls[(position + 1) % len(calls)]
        return layers[li][name]

    step_bytes = 0
    linear_bytes = 0
    for m, li, name in calls:
        n, k = local_shape[name]
        step_bytes += call_bytes(m, n, k, weight_bytes[(li, name)], out_bytes[name])
        linear_bytes += weight_bytes[(li, name)] + m * k + 4 * m + m * n * out_bytes[name]
    pairs_per_step = len(calls)
    # pairs that run as ONE launch (the decode kernel quantizes its own rows)
    one_launch_pairs = sum(1 for m, _, name in calls
                           if ext.quant_linear_is_fused(m, local_shape[name][0] // 64, local_shape[name][1] // 64))
    allreduces_per_step = sum(1 for _, _, name in calls if GROUPS[name][2] == "k")

    separate_sums = [0]  # all-reduce kernels of our own launched by the last sweep (not fused ones, not NCCL's)

    def sweep(with_quantizer: bool, with_allreduce: bool) -> None:
        separate_sums[0] = 0
        for position, (m, li, name) in enumerate(calls):
            axis = GROUPS[name][2]
            weights, ahead = layers[li][name], next_weights(position)
            if with_quantizer:
                # quantizer + projection (+ sum over the ranks) through the one-call entry point: one launch
                # where the decode kernel quantizes its own rows, the quantizer kernel and the projection otherwise
                fused_sum = with_allreduce and reducer is not None and axis == "k"
                y = ext.alignquant_quant_linear(acts[(m, name)], weights, None, output_dtype=out_dtype[name], out=outs[(m, name)],
                                                quantized=qbuf[(m, name)], reducer=reducer if fused_sum else None, prefetch=ahead)
                if y is None:  # the fused sum does not take this shape
                    ext.alignquant_quant_linear(acts[(m, name)], weights, None, output_dtype=out_dtype[name],
                                                out=outs[(m, name)], quantized=qbuf[(m, name)], prefetch=ahead)
                    if with_allreduce and world > 1 and axis == "k":
                        all_reduce(outs[(m, name)])
                        separate_sums[0] += 1 if reducer is not None else 0
                elif with_allreduce and world > 1 and axis == "k" and not fused_sum:
                    all_reduce(outs[(m, name)])
                continue
            xq, a_s = qbuf[(m, name)]
            if with_allreduce and reducer is not None and axis == "k" and ext.alignquant_linear_allreduce(
                    xq, a_s, weights, None, reducer, scale_mode="token", output_dtype=out_dtype[name], out=outs[(m, name)],
                    prefetch=ahead) is not None:
                continue  # projection and the sum over the ranks ran as one kernel
            ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token", output_dtype=out_dtype[name],
                                           out=outs[(m, name)], prefetch=ahead)
            if with_allreduce and world > 1 and axis == "k":
                all_reduce(outs[(m, name)])
                separate_sums[0] += 1 if reducer is not None else 0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps: int, warmup: int) -> float:
        """Seconds per step: CUDA events around `steps` calls, max over ranks."""
        for _ in range(warmup):
            fn()
        barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            fn()
        end.record()
        barrier()
        seconds = begin.elapsed_time(end) / 1e3 / steps
        if world > 1:
            t = torch.tensor([seconds], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            seconds = float(t.item())
        return seconds

    # ---- N > 1: the fused projection + rank sum against projection, then NCCL all-reduce
    watchdog.stage = "tp_check"
    tp_check = None
    if world > 1:
        worst = 0.0
        ok = same_bits = True
        for m in ROW_COUNTS:
            for name, (_, _, axis) in GROUPS.items():
                if axis != "k":
                    continue
                ext.alignquant_activation_quantize_cuda(acts[(m, name)], None, scale_mode="token", out=qbuf[(m, name)])
                xq, a_s = qbuf[(m, name)]
                weights = layers[0][name]
                want = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token", output_dtype=torch.float32)
                dist.all_reduce(want)
                got = None
                if reducer is not None:
                    got = ext.alignquant_linear_allreduce(xq, a_s, weights, None, reducer, scale_mode="token",
                                                          output_dtype=torch.float32)
                if got is None:  # shape without the fused epilogue: projection, then the peer-memory (or NCCL) sum
                    got = ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token", output_dtype=torch.float32)
                    all_reduce(got)
                # the one-call form the timed sweep uses (quantizer inside the kernel at one row): same bits
                one_call = None
                if reducer is not None:
                    one_call = ext.alignquant_quant_linear(acts[(m, name)], weights, None, output_dtype=torch.float32,
                                                           reducer=reducer)
                torch.cuda.synchronize()
                if one_call is not None:
                    ok = ok and bool(torch.isclose(one_call, want, rtol=1e-5, atol=1e-5).all())
                    same_bits = same_bits and torch.equal(one_call, got)
                # NCCL's summation order differs from the rank order of the fused sum
                close = torch.isclose(got, want, rtol=1e-5, atol=1e-5)
                ok = ok and bool(close.all())
                worst = max(worst, float((got - want).abs().max()))
        try:
            ext.device_status(device)
        except RuntimeError as error:  # a bounded device-side wait ran out: every rank still reaches the common result
            ok = False
            print(f"[bench] rank {rank}: {error}", file=sys.stderr)
        failed = torch.tensor([0 if ok else 1, 0 if same_bits else 1], device=device, dtype=torch.int32)
        dist.all_reduce(failed, op=dist.ReduceOp.MAX)
        failed = failed.tolist()
        tp_check = "ok" if failed[0] == 0 else "mismatch"
        one_call_bits = None if reducer is None else ("same" if failed[1] == 0 else "differ")
        if tp_check != "ok":
            if rank == 0:
                print(json.dumps({"metric": "decode_gemv_hbm_gbs", "n_gpus": world, "tp_check": tp_check,
                                  "max_abs_difference": worst}), flush=True)
            barrier()
            sys.stdout.flush()
            os._exit(3)

    # ---- device-resident step: one CUDA graph per rank (kernels and, for N > 1, the all-reduces)
    watchdog.stage = "first sweep (eager)"
    sweep(True, True)
    own_sum_launches = separate_sums[0]
    barrier()
    launch_mode = "cuda graph replay"
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            sweep(True, True)
        step = graph.replay
    except Exception as error:  # a collective that cannot be captured: run the step eagerly
        if world == 1:
            raise
        print(f"[bench] graph capture of the tensor-parallel step failed ({error}); running eagerly", file=sys.stderr)
        launch_mode = "eager"
        torch.cuda.synchronize()
        step = lambda: sweep(True, True)  # noqa: E731
    watchdog.stage = "timed sweep"
    with ClockSampler(local_rank) as clocks:
        seconds = timed(step, args.steps, max(args.warmup, 3))
        # keep the same step running until nvidia-smi (100 ms period) has had time to sample it
        sampling_deadline = time.perf_counter() + 1.0
        while time.perf_counter() < sampling_deadline:
            step()
            torch.cuda.synchronize()
    ext.device_status(device)

    watchdog.stage = "GEMV-only sweep"
    # ---- the packed-GEMV kernel alone (roofline of the dominant kernel)
    kernel_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(kernel_graph):
        sweep(False, False)
    kernel_seconds = timed(kernel_graph.replay, args.steps, 3) / pairs_per_step
    peak, peak_source = hbm_peak()
    achieved = linear_bytes / pairs_per_step / kernel_seconds / 1e9

    watchdog.stage = "end-to-end sweep"
    # ---- end to end through the public API from pinned host buffers
    host_x = {key: x.cpu().pin_memory() for key, x in acts.items()}
    host_out = {key: torch.empty(o.shape, dtype=o.dtype).pin_memory() for key, o in outs.items()}
    h2d = sum(host_x[(m, name)].numel() * 2 for m in ROW_COUNTS for name in GROUPS) * LAYERS
    d2h = sum(host_out[(m, name)].numel() * out_bytes[name] for m in ROW_COUNTS for name in GROUPS) * LAYERS

    def project(position: int, x):
        """quantize -> linear (-> sum over ranks) of call `position` through the public API."""
        m, li, name = calls[position]
        axis = GROUPS[name][2]
        weights, ahead = layers[li][name], next_weights(position)
        y = None
        if reducer is not None and axis == "k":
            y = ext.alignquant_quant_linear(x, weights, None, output_dtype=out_dtype[name], reducer=reducer, prefetch=ahead)
        if y is None:
            y = ext.alignquant_quant_linear(x, weights, None, output_dtype=out_dtype[name], prefetch=ahead)
            if world > 1 and axis == "k":
                all_reduce(y)
        return y

    def e2e_step() -> None:
        for position, (m, li, name) in enumerate(calls):
            y = project(position, host_x[(m, name)].to(device, non_blocking=True))
            host_out[(m, name)].copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    # The same calls captured once into a CUDA graph (the library's entry points are plain
    # asynchronous launches): input copies on one stream, quantize + linear on a second, result
    # copies on a third, so that PCIe traffic overlaps the kernels.  Every replay performs all
    # host->device and device->host copies again.
    e2e_mode = "eager API calls"
    e2e_run = e2e_step
    try:
        copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        x_dev = {(li, m, name): torch.empty_like(acts[(m, name)]) for li in range(LAYERS) for m in ROW_COUNTS for name in GROUPS}
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph):
            main = torch.cuda.current_stream(device)
            copy_in.wait_stream(main)
            copy_out.wait_stream(main)
            # Inputs of one row count are staged (one host->device copy per call) while the calls of
            # the previous row count run: the kernels wait for copies once per row count instead of
            # once per call, which keeps the programmatic dependent launch between consecutive
            # kernels of the main stream.  Results leave once per decoder layer (one copy per call).
            staged = {}
            with torch.cuda.stream(copy_in):
                for m in ROW_COUNTS:
                    for li in range(LAYERS):
                        for name in GROUPS:
                            x_dev[(li, m, name)].copy_(host_x[(m, name)], non_blocking=True)
                    staged[m] = torch.cuda.Event()
                    staged[m].record(copy_in)
            position = 0
            for m in ROW_COUNTS:
                main.wait_event(staged[m])
                for li in range(LAYERS):
                    results = []
                    for name in GROUPS:
                        assert calls[position] == (m, li, name)
                        results.append((name, project(position, x_dev[(li, m, name)])))
                        position += 1
                    computed = torch.cuda.Event()
                    computed.record(main)
                    with torch.cuda.stream(copy_out):
                        copy_out.wait_event(computed)
                        for done_name, done_y in results:
                            host_out[(m, done_name)].copy_(done_y, non_blocking=True)
            main.wait_stream(copy_in)
            main.wait_stream(copy_out)

        def e2e_run() -> None:  # noqa: F811
            e2e_graph.replay()
            torch.cuda.synchronize()

        e2e_run()
        e2e_mode = "one CUDA graph per step (copies on side streams: inputs staged per row count, results read back per layer)"
    except Exception as error:  # capture of pinned copies unsupported: run the calls eagerly
        print(f"[bench] graph capture of the end-to-end step failed ({error}); running eagerly", file=sys.stderr)
        torch.cuda.synchronize()
        e2e_run = e2e_step

    e2e_seconds = timed(e2e_run, max(1, min(args.steps, 5)), 1)

    traffic = None
    if world == 1 and not lookahead and all(v is not None for v in NCU_DRAM_BYTES_PER_LAUNCH.values()):
        traffic = sum(NCU_DRAM_BYTES_PER_LAUNCH.values()) / len(NCU_DRAM_BYTES_PER_LAUNCH)
    total_bytes = step_bytes * world  # every rank streams its own shard
    line = {
        "metric": "decode_gemv_hbm_gbs",
        "value": total_bytes / seconds / 1e9,
        "unit": "GB/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": seconds * 1e3,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "int8",
        "data": "synthetic",
        "config": {
            "workload": WORKLOAD,
            "l2": "2 GB of distinct weights per step exceed the 126 MB L2; no flush between steps",
            "lookahead": ("every projection asks the L2 to fetch the next projection's image while it runs (aq_linear_ahead)"
                          if lookahead else "off"),
            "parallelism": f"tp{world}",
            "pairs": (f"each quantizer + projection pair is one call of aq_quant_linear; {one_launch_pairs} of {pairs_per_step} "
                      "pairs per step run as one launch (the decode kernel quantizes its own rows), the others as two"),
            "launch": launch_mode + ("" if world == 1 else
                                     f" + sum over ranks fused into the GEMV epilogue (peer memory; {own_sum_launches} of "
                                     f"{allreduces_per_step} sums per step as a separate peer-memory kernel)"
                                     if reducer is not None else " + NCCL all-reduce"),
        },
        "clocks": clocks.result,
        "e2e": {"value": total_bytes / e2e_seconds / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "launch": e2e_mode},
        "gpu_launches": (2 * pairs_per_step - one_launch_pairs + own_sum_launches) * args.steps,
        "roofline": {
            "kernel": ("cluster_decode_kernel" if args.cluster_decode else "direct_decode_kernel + cluster_decode_kernel") +
                      " (packed W4/W8 GEMV, M<=16; mean over the sweep's launches)",
            "bound": "hbm",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "peak_source": f"{peak_source} HBM copy bandwidth", "traffic": traffic,
            "traffic_how": ("dram__bytes_read.sum + dram__bytes_write.sum per launch, ncu capture of the four shapes at one "
                            "row with the L2 flushed before each launch, mean over the shapes" if traffic is not None else None),
            "bytes_per_launch": linear_bytes / pairs_per_step, "us_per_launch": kernel_seconds * 1e6,
        },
    }
    if tp_check is not None:
        line["tp_check"] = tp_check
        line["tp_one_call_bits"] = one_call_bits  # one-call form against quantizer + fused projection, bit for bit
    if rank == 0 and world == 1:
        sample = CpuSample()
        sample.run()
        cpu_seconds = min(sample.run() for _ in range(2))
        line["cpu_baseline"] = {
            "value": sample.bytes / cpu_seconds / 1e9, "unit": "GB/s", "cores": os.cpu_count() or 1,
            "kind": "port", "sample": CpuSample.description,
        }

    # ---- the other legs of the metric; the sweep's buffers are released first
    del layers, graph, kernel_graph, step
    try:
        del e2e_graph, x_dev
    except NameError:
        pass
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    if "generation" in legs:
        watchdog.stage = "generation leg"
        try:
            line["generation"] = generation_leg(world, args.gen_tokens)
        except Exception as error:
            line["generation"] = {"error": f"{type(error).__name__}: {error}"}
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    if "prefill" in legs and world == 1:
        try:
            line["prefill"] = prefill_leg(ext, device, max(3, min(args.steps, 10)))
        except Exception as error:  # the headline line is still reported
            line["prefill"] = {"error": f"{type(error).__name__}: {error}"}
    watchdog.cancel()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # Tearing down a communicator whose collectives live in captured graphs was seen to
        # block for ever; the step is finished and reported, so every rank synchronises and
        # leaves without running finalizers.
        barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
