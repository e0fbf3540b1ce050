"""One rank of the peer-memory reduction test: run under ``python -m torch.distributed.run`` with one process a GPU.
Every reduction is done twice, by ``tp.PeerReducer`` and by ``tp.ordered_all_reduce`` (NCCL collectives and a sum kernel),
and must give the same bits on every rank; rank 0 prints one JSON line with the verdict and the two timings."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tensorfold_b200 import _lib  # noqa: E402
from tensorfold_b200.cuda import tp  # noqa: E402


def timed(fn, iters):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) * 1e3 / iters], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def graph_timed(fn, iters=20):
    """Microseconds a call when ``iters`` of them replay from one CUDA graph (no launch cost of the host between them)."""

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(iters):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) * 1e3 / (5 * iters)], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    del graph
    return float(t.item())


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    _lib.check(_lib.lib().tf_init(torch.cuda.current_device()), "init")
    shapes = [(1, 6144), (16, 6144), (16, 5120), (256, 6144), (2048, 6144)]
    red = tp.PeerReducer(2048 * 6144, device="cuda")
    equal, times = True, {}
    for shape in shapes:
        for dtype in (torch.bfloat16, torch.float32):
            g = torch.Generator().manual_seed(1000 * rank + shape[0])
            part = (torch.randn(shape, generator=g) * 2).to(dtype).cuda()
            want = tp.ordered_all_reduce(part)
            small = part.numel() * part.element_size() <= red.flagged_up_to
            forms = [red.ALL, red.SHARES] + ([red.FLAGGED] if small else [])
            if small and world >= 4 and part.numel() % (8 * world) == 0:
                forms.append(red.HOPS)
            for form in forms + forms:                          # repeated calls reuse the buffers and keep the flags counting
                red.force = form
                home = red.partial(shape, dtype)
                home.copy_(part)
                got = red.reduce(home)
                equal &= bool(torch.equal(got, want))
            red.force = None
            key = f"{shape[0]}x{shape[1]}_{'bf16' if dtype == torch.bfloat16 else 'f32'}"
            home = red.partial(shape, dtype)
            times[key] = {"peer_us": round(timed(lambda: red.reduce(home), 50), 2),
                          "collective_us": round(timed(lambda: tp.ordered_all_reduce(part), 50), 2),
                          "peer_graph_us": round(graph_timed(lambda: red.reduce(home)), 2),
                          "collective_graph_us": round(graph_timed(lambda: tp.ordered_all_reduce(part)), 2)}
    errors = _lib.device_error(part)
    flag = torch.tensor([int(equal), errors], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    worst = torch.tensor([errors], device="cuda")
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    red.close()
    if rank == 0:
        print(json.dumps({"world": world, "equal": bool(flag[0].item()), "errors": int(worst.item()), "us": times}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
