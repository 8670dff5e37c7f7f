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
