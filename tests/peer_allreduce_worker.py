"""Worker of the multi-GPU all-reduce test: run as N processes, one per GPU (torch.distributed.run)."""

from __future__ import annotations

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist


def main() -> int:
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    from alignquant_b200.kernels.cuda import extension as ext
    from alignquant_b200.kernels.cuda.allreduce import PeerAllReduce

    ext.load_extension()
    reducer = PeerAllReduce(16 * 3072, device)
    ok = True
    gen = torch.Generator(device="cpu").manual_seed(5)
    for round_index, count in enumerate([3072, 4, 16 * 3072, 4 * 3072, 1024, 3072, 3072]):
        parts = torch.randn((world, count), generator=gen, dtype=torch.float32)
        want = parts[0].clone()
        for r in range(1, world):
            want += parts[r]  # rank order, FP32
        mine = parts[rank].to(device)
        out = torch.empty_like(mine)
        reducer(mine, out)
        in_place = mine.clone()
        reducer(in_place)
        torch.cuda.synchronize()
        if not (torch.equal(out.cpu(), want) and torch.equal(in_place.cpu(), want)):
            ok = False
            print(f"rank {rank}: mismatch in round {round_index} (count {count})", file=sys.stderr)
    # replayed from a CUDA graph: the call counter lives on the device
    x = torch.full((8 * 3072,), float(rank + 1), device=device)
    y = torch.empty_like(x)
    reducer(x, y)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        reducer(x, y)
        reducer(y, y)
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    expect = float(sum(range(1, world + 1)) * world)
    if not bool((y == expect).all()):
        ok = False
        print(f"rank {rank}: graph replay gave {y[:4].tolist()} instead of {expect}", file=sys.stderr)
    # projection + sum over the ranks in one kernel against projection, then all-reduce kernel
    from alignquant_b200.synthetic import synthetic_activation, synthetic_module_tensors

    n, k = 2048, 512  # this rank's K shard of a row-parallel layer (enough tile rows for the cluster decode kernel)
    t = synthetic_module_tensors(n, k, seed=100 + rank, device=device)
    weights = ext.prepare_weights(t["state_bits"], t["w4_payload"], t["w4_scales"], t["w8_payload"], t["w8_scales"],
                                  t["w4_row_offsets"], t["w8_row_offsets"], n_k=k // 64)
    for m in (1, 7, 16, 24):
        xq, a_s = ext.alignquant_activation_quantize_cuda(synthetic_activation(m, k, seed=200 + rank + m, device=device),
                                                          None, scale_mode="token")
        separate = reducer(ext.alignquant_linear_prepared(xq, a_s, weights, None, scale_mode="token"))
        fused = ext.alignquant_linear_allreduce(xq, a_s, weights, None, reducer, scale_mode="token")
        torch.cuda.synchronize()
        if fused is None:
            ok = False
            print(f"rank {rank}: the fused path did not apply (m = {m}, plan {ext.linear_plan(m, n // 64, k // 64)})", file=sys.stderr)
        elif not torch.equal(fused, separate):
            ok = False
            print(f"rank {rank}: fused projection + sum differs from the two-kernel path (m = {m})", file=sys.stderr)
    for m in (1, 4, 9):  # quantizer + projection + sum in one call (one launch at one row)
        raw = synthetic_activation(m, k, seed=300 + rank + m, device=device)
        raw_q, raw_s = ext.alignquant_activation_quantize_cuda(raw, None, scale_mode="token")
        separate = reducer(ext.alignquant_linear_prepared(raw_q, raw_s, weights, None, scale_mode="token"))
        one_call = ext.alignquant_quant_linear(raw, weights, None, reducer=reducer)
        torch.cuda.synchronize()
        if one_call is None or not torch.equal(one_call, separate):
            ok = False
            print(f"rank {rank}: quantizer + projection + sum in one call differs (m = {m})", file=sys.stderr)
    out = torch.empty((16, n), dtype=torch.float32, device=device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ext.alignquant_linear_allreduce(xq[:16].contiguous(), a_s[:16].contiguous(), weights, None, reducer,
                                        scale_mode="token", out=out)
    for _ in range(4):
        graph.replay()
    torch.cuda.synchronize()
    want = reducer(ext.alignquant_linear_prepared(xq[:16].contiguous(), a_s[:16].contiguous(), weights, None, scale_mode="token"))
    torch.cuda.synchronize()
    if not torch.equal(out, want):
        ok = False
        print(f"rank {rank}: replayed fused projection + sum differs", file=sys.stderr)
    ext.device_status(device)
    flag = torch.tensor([1 if ok else 0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    if rank == 0:
        print("PEER_ALLREDUCE_OK" if int(flag.item()) == 1 else "PEER_ALLREDUCE_FAILED", flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
