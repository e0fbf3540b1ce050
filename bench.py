"""Headline benchmark: affine 4-bit / group-64 quantized matmul weight GB/s on the dense-27B projections.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--rows M] [--impl b200|reference]

A step is one pass of the hot path over one decoder layer's seven projections (q, k, v, o, gate, up, down; 191.6 MB of
packed weights) at M rows (default 16: the speculative-verify shape).  Steps cycle through a ring of distinct layer
weights larger than L2, so every pass streams its weights from HBM.  One JSON line is printed by rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

BITS, GS = 4, 64
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 2 ** 20
# DRAM bytes per launch of the dominant kernel over its algorithmic bytes, from one ncu capture of a gate/up set launch
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch; traffic grows with the weight bytes, so a step's
# launches scale by it): 100.48 MB read + 3.95 MB written for 101.55 MB of weights, rows and outputs.
TRAFFIC_RATIO = 1.028
SETS = (("q_proj", "k_proj", "v_proj"), ("o_proj",), ("gate_proj", "up_proj"), ("down_proj",))   # launches of a step


def weight_bytes(n: int, k: int, bits: int = BITS, gs: int = GS) -> int:
    return n * k * bits // 8 + 4 * n * k // gs


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak() -> float:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["bf16_tflops"])
        except Exception:
            pass
    return 1590.0


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 100 ms while the measurement runs (read-only)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self) -> dict:
        sm, mx, reasons = [], 0.0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def layer_shapes():
    from tensorfold_b200 import synthetic

    return list(synthetic.DENSE_27B.items())


# ----------------------------------------------------------------------------------------------------------------------
# the reference arm and the CPU baseline: the oracle's restatement of the reference's CPU path, on the host cores
# ----------------------------------------------------------------------------------------------------------------------

def host_threads() -> int:
    """Threads the CPU arm uses: every core this process may run on, whatever OMP_NUM_THREADS a launcher exported."""

    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_pass(inputs, rows: int) -> None:
    """One pass of the CPU restatement (dequantise to float32 then x.float() @ w.T, all host threads) over the layer."""

    from oracle import native

    for words, s_bits, b_bits, x_bits in inputs:
        native.qmm_f32(x_bits[:rows], words, s_bits, b_bits, GS, BITS)


def cpu_inputs(rows: int):
    """The seven projections of one layer, as the B200 arm runs them."""

    from tensorfold_b200 import synthetic

    out = []
    for name, (n, k) in synthetic.DENSE_27B.items():
        words, scales, biases = synthetic.affine_weight(n, k, BITS, GS, seed=len(out))
        x = synthetic.activations(rows, k, len(out))
        out.append((words.numpy(), synthetic.bf16_bits(scales), synthetic.bf16_bits(biases), synthetic.bf16_bits(x)))
    return out


def layer_bytes_total() -> int:
    from tensorfold_b200 import synthetic

    return sum(weight_bytes(n, k) for n, k in synthetic.DENSE_27B.values())


def reference_torch_baseline(rows: int) -> dict:
    """The reference's own CPU-runnable code for this op, where its checkout can be imported (the directory TENSORFOLD_REFERENCE
    names): ``dequantize`` (families/qwen3_5/cuda/qmm.py:132-149) then ``x.float() @ w.T``, timed
    both ways on one projection (q_proj), all host threads.  Also records whether MLX (the reference's named CPU
    baseline, ``mx.quantized_matmul`` on mx.cpu) can be imported on this box."""

    import importlib

    out = {}
    try:
        importlib.import_module("mlx.core")
        out["mlx"] = "importable"
    except Exception as exc:                                 # noqa: BLE001
        out["mlx"] = f"MLX unavailable on this box ({type(exc).__name__})"
    root = os.environ.get("TENSORFOLD_REFERENCE", "")
    if not root:
        out["reference_torch"] = "reference checkout not present on this box"
        return out
    try:
        import torch

        sys.path.insert(0, os.path.join(root, "src"))
        ref = importlib.import_module("tensorfold.families.qwen3_5.cuda.qmm")
        from tensorfold_b200 import synthetic

        torch.set_num_threads(host_threads())
        n, k = synthetic.DENSE_27B["q_proj"]
        words, scales, biases = synthetic.affine_weight(n, k, BITS, GS, seed=0)
        x = synthetic.activations(rows, k, 0)
        t0 = time.perf_counter()
        w = ref.dequantize(words, scales, biases, GS, BITS)
        t1 = time.perf_counter()
        y = x.float() @ w.float().T
        t2 = time.perf_counter()
        del y
        out["reference_torch"] = {"projection": "q_proj", "dequantize_plus_matmul_gb_s": weight_bytes(n, k) / (t2 - t0) / 1e9,
                                  "matmul_on_dequantised_gb_s": weight_bytes(n, k) / (t2 - t1) / 1e9, "threads": host_threads()}
    except Exception as exc:                                 # noqa: BLE001
        out["reference_torch"] = f"reference import failed: {type(exc).__name__}: {exc}"[:200]
    return out


def cpu_baseline(rows: int, budget_s: float = 15.0) -> dict:
    from oracle import native

    native.set_threads(host_threads())
    inputs = cpu_inputs(rows)
    cpu_pass(inputs, rows)                               # warm the pages
    t0, reps = time.perf_counter(), 0
    while reps < 2 or (time.perf_counter() - t0 < budget_s and reps < 50):
        cpu_pass(inputs, rows)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    total = layer_bytes_total()
    out = {"value": total / dt / 1e9, "unit": "GB/s", "cores": native.threads(), "kind": "port",
           "sample": f"all seven projections of one dense-27B layer at M={rows} ({total / 1e6:.1f} MB of packed "
                     f"weights), {reps} passes of oracle/affine_ref.c (dequantise to float32, float32 dot, OpenMP)"}
    out.update(reference_torch_baseline(rows))
    return out


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import native

    native.set_threads(host_threads())                   # not the one thread a torchrun launcher exports
    inputs = cpu_inputs(args.rows)
    for _ in range(min(args.warmup, 2)):
        cpu_pass(inputs, args.rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(inputs, args.rows)
    dt = time.perf_counter() - t0
    total = layer_bytes_total()
    value = total * args.steps / dt / 1e9
    sample = (f"each step = the seven projections of one dense-27B layer at M={args.rows} "
              f"({total / 1e6:.1f} MB packed weights) on the host cores")
    from tensorfold_b200 import synthetic

    baseline = {"value": value, "unit": "GB/s", "cores": native.threads(), "kind": "port", "sample": sample}
    baseline.update(reference_torch_baseline(args.rows))
    print(json.dumps({
        "impl": "reference", "metric": "affine_4bit_g64_qmm_weight_gbps", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"dense27b_layer_projections_4bit_g64_M{args.rows}", "rows": args.rows, "bits": BITS, "group": GS,
                   "projections": {name: list(shape) for name, shape in synthetic.DENSE_27B.items()},
                   "weight_bytes_per_step": total, "sample": sample},
        "cpu_baseline": baseline,
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------------------------------------------------
# the B200 arm
# ----------------------------------------------------------------------------------------------------------------------

_side_stream = []


def side_stream():
    """The one stream the side figures capture on (each stream that runs the decode kernel holds a scratch area)."""

    import torch

    if not _side_stream:
        _side_stream.append(torch.cuda.Stream())
    return _side_stream[0]


def graph_time(fn, steps: int, stream, reps: int = 5):
    """Capture `steps` calls of fn(i) in one CUDA graph on `stream`; returns (graph, [ms per replay])."""

    import torch

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for i in range(steps):
                fn(i)
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            graph.replay()
            b.record(stream)
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
    return graph, times


def rolled_experts(e: int, n: int, k: int, seed: int):
    """E distinct expert weights from one seeded draw (rows rolled per expert): cheap to make, same distributions."""

    import torch

    from tensorfold_b200 import synthetic

    w = synthetic.affine_weight(n, k, BITS, GS, seed=seed)
    return tuple(torch.stack([torch.roll(t, 7 * i + 1, 0) for i in range(e)]) for t in w)


def moe_layer_bench(dev, rows_list=(16, 2048)) -> dict:
    """The routed-MoE layer: hidden 2688, 128 experts of width 1856, top 6, one shared expert of width 3712."""

    import torch

    from tensorfold_b200 import synthetic
    from tensorfold_b200.cuda import experts, moe
    from tensorfold_b200.cuda.kernels import qmm

    d, e, ni, sni, top_k = 2688, 128, 1856, 3712, 6
    g = torch.Generator().manual_seed(11)
    todev = lambda m: tuple(t.to(dev) for t in m)
    ex = experts.make([todev(rolled_experts(e, ni, d, 1)), todev(rolled_experts(e, ni, d, 2))], todev(rolled_experts(e, d, ni, 3)), GS)
    shared = moe.SharedExpert(qmm.pack_pair(todev(synthetic.affine_weight(sni, d, BITS, GS, seed=4)),
                                            todev(synthetic.affine_weight(sni, d, BITS, GS, seed=5)), GS),
                              qmm.pack(*todev(synthetic.affine_weight(d, sni, BITS, GS, seed=6)), GS))
    wr = (torch.randn((e + 1, d), generator=g) * 0.05).to(torch.bfloat16).to(dev)
    layer = moe.Routed(wr, ex, top_k, shared)
    out = {}
    stream = side_stream()
    per_expert = 3 * weight_bytes(ni, d)
    for rows in rows_list:
        xs = [synthetic.activations(rows, d, 40 + i).to(dev) for i in range(4)]       # different routings in turn
        prefill = rows > 128
        for x in xs:
            moe.run(x, layer, prefill=prefill)
        torch.cuda.synchronize()
        steps = 8
        _, times = graph_time(lambda i: moe.run(xs[i % 4], layer, prefill=prefill), steps, stream)
        us = sorted(times)[len(times) // 2] * 1e3 / steps
        buf = next(b for k, b in moe._scratch.items() if k[0] >= rows and k[5] == prefill)
        moe.run(xs[0], layer, prefill=prefill)
        distinct = int(torch.unique(buf.pick[:rows, :top_k]).numel())
        algo = distinct * per_expert + 3 * weight_bytes(sni, d) + 2 * (e + 1) * d + 2 * rows * d * 2
        flops = 2 * rows * (top_k * 3 * ni * d + 3 * sni * d + (e + 1) * d)
        out[f"M{rows}"] = {"us": us, "distinct_experts": distinct, "algorithmic_gb_s": algo / us / 1e3,
                           "tflops": flops / us / 1e6}
    return out


def layer_sets(xs, layer, ys, splits, pdl: bool) -> None:
    """One layer as the four launches of its dataflow: q/k/v in one persistent launch, o_proj, gate/up in one, down_proj."""

    from tensorfold_b200.cuda.kernels import qmm

    for names in SETS:
        qmm.matmul_set(xs[names[0]], [layer[n] for n in names], sks=[splits[n] for n in names], outs=[ys[n] for n in names], pdl=pdl)


def dense_rows_bench(dev, layers, shapes, ring, splits) -> dict:
    """The same layer at other row counts: weight GB/s at M = 1, 4, 8, 16 (four set launches a layer) and TFLOP/s at
    M = 2048 (through ``matmul``: the row-exact decode arithmetic) and through the tcgen05 prefill kernel."""

    import torch

    from tensorfold_b200 import synthetic
    from tensorfold_b200.cuda.kernels import qmm

    layer_bytes = sum(weight_bytes(n, k) for _, (n, k) in shapes)
    peak, _ = measured_peaks()
    stream = side_stream()
    out = {}
    for rows in (1, 4, 8, 16, 2048):
        xs = {name: synthetic.activations(rows, k, 3).to(dev) for name, (n, k) in shapes}
        ys = {name: torch.empty((rows, n), dtype=torch.bfloat16, device=dev) for name, (n, k) in shapes}

        def fn(i):
            if rows <= 16:
                layer_sets(xs, layers[i % ring], ys, splits, True)
            else:
                for name, _ in shapes:
                    qmm.matmul(xs[name], layers[i % ring][name], out=ys[name], pdl=True, sk=splits[name])

        with torch.cuda.stream(stream):
            for i in range(2):
                fn(i)
        torch.cuda.synchronize()
        steps = 2 * ring if rows <= 16 else 2
        _, times = graph_time(fn, steps, stream)
        us = sorted(times)[len(times) // 2] * 1e3 / steps
        entry = {"us_per_layer": us, "weight_gb_s": layer_bytes / us / 1e3, "of_measured_hbm": layer_bytes / us / 1e3 / peak}
        if rows >= 256:
            flops = 2 * rows * sum(n * k for _, (n, k) in shapes)
            entry["tflops"] = flops / us / 1e6                               # the row-exact decode arithmetic at M rows

            def pf(i):
                for name, _ in shapes:
                    qmm.prefill_matmul(xs[name], layers[i % ring][name], out=ys[name])

            pf(0)
            torch.cuda.synchronize()
            _, ptimes = graph_time(pf, 2 * ring, stream)
            pus = sorted(ptimes)[len(ptimes) // 2] * 1e3 / (2 * ring)
            entry["prefill"] = {"us_per_layer": pus, "tflops": flops / pus / 1e6,
                                "of_measured_bf16_peak": flops / pus / 1e6 / measured_tensor_peak()}
        out[f"M{rows}"] = entry
    return out


def single_matmul_bench(dev, n: int, k: int, bits: int, gs: int, rows_list, seed: int = 0) -> dict:
    """One projection at the given row counts over a ring of weight copies larger than L2: microseconds a call, packed
    weight GB/s and the fraction of the measured HBM peak."""

    import torch

    from tensorfold_b200 import synthetic
    from tensorfold_b200.cuda.kernels import qmm

    peak, _ = measured_peaks()
    nbytes = weight_bytes(n, k, bits, gs)
    ring = max(3, -(-3 * L2_BYTES // nbytes))
    w = synthetic.affine_weight(n, k, bits, gs, seed=seed)
    base = qmm.pack(w[0].to(dev), w[1].to(dev), w[2].to(dev), gs, bits=bits)
    copies = [base] + [qmm.Q4(base.weight.clone(), None, None, n, k, gs, bits) for _ in range(ring - 1)]
    stream = side_stream()
    out = {}
    for rows in rows_list:
        x = synthetic.activations(rows, k, 3).to(dev)
        y = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)
        fn = lambda i: qmm.matmul(x, copies[i % ring], out=y, pdl=True)
        with torch.cuda.stream(stream):
            fn(0), fn(1)
        torch.cuda.synchronize()
        _, times = graph_time(fn, 4 * ring, stream)
        us = sorted(times)[len(times) // 2] * 1e3 / (4 * ring)
        out[f"M{rows}"] = {"us": us, "weight_gb_s": nbytes / us / 1e3, "of_measured_hbm": nbytes / us / 1e3 / peak}
    del copies
    torch.cuda.empty_cache()
    return out


def cfg0_bench(dev) -> dict:
    """The CPU-runnable reference configuration: one 4096 x 4096 affine 4-bit / group-64 matmul at M = 4 (seed 0)."""

    return single_matmul_bench(dev, 4096, 4096, BITS, GS, (4,), seed=0)


def cfg3_bench(dev) -> dict:
    """The mixed-width sweep on a 4096 -> 14336 projection: 2, 3, 5, 6 and 8 bits x groups of 32, 64, 128 at M = 1, 16."""

    out = {}
    for bits in (2, 3, 5, 6, 8):
        for gs in (32, 64, 128):
            out[f"b{bits}_g{gs}"] = single_matmul_bench(dev, 14336, 4096, bits, gs, (1, 16), seed=bits * 10 + gs)
    return out


def lm_head_bench(dev) -> dict:
    """The 248,320-row head of the dense 27B model as one matmul (715 MB of packed weights: larger than L2 by itself)."""

    import torch

    from tensorfold_b200 import synthetic
    from tensorfold_b200.cuda.kernels import qmm

    peak, _ = measured_peaks()
    n, k, block = 248320, 5120, 8192
    w = synthetic.affine_weight(block, k, BITS, GS, seed=91)
    part = qmm.pack(w[0].to(dev), w[1].to(dev), w[2].to(dev), GS)
    reps = -(-n // block)
    weight = part.weight.repeat(reps, 1, 1)[: -(-n // 128)].contiguous()      # distinct memory for every super-block
    head = qmm.Q4(weight, None, None, n, k, GS, BITS)
    nbytes = weight_bytes(n, k)
    stream = side_stream()
    out = {}
    for rows in (1, 16):
        x = synthetic.activations(rows, k, 3).to(dev)
        y = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)
        fn = lambda i: qmm.matmul(x, head, out=y, pdl=True)
        with torch.cuda.stream(stream):
            fn(0)
        torch.cuda.synchronize()
        _, times = graph_time(fn, 4, stream)
        us = sorted(times)[len(times) // 2] * 1e3 / 4
        out[f"M{rows}"] = {"us": us, "weight_gb_s": nbytes / us / 1e3, "of_measured_hbm": nbytes / us / 1e3 / peak}
    return out


def moe_block_tp_bench(dev, rank: int, world: int, rows_list=(16, 2048)) -> dict:
    """Tensor-parallel MoE decoder block: hidden 6144, 160 experts top 8 of width 1536 split by expert across the ranks,
    attention o_proj 8192 -> 6144 row-parallel; both bf16 partials [M, 6144] are reduced in rank order over NVLink, by
    the one-launch peer-memory reduction (``us``) and by the NCCL collectives plus a sum kernel (``us_collectives``).
    ``phases_us``: each of the block's steps replayed alone from a CUDA graph (max over ranks), with the peer reduction."""

    import torch
    import torch.distributed as dist

    from tensorfold_b200 import _lib, synthetic
    from tensorfold_b200.cuda import experts, moe, tp
    from tensorfold_b200.cuda.kernels import qmm

    d, e, ni, top_k, ko = 6144, 160, 1536, 8, 8192
    local_e = e // world
    g = torch.Generator().manual_seed(21)
    todev = lambda m: tuple(t.to(dev) for t in m)

    def local_experts(n, k, seed):
        w = synthetic.affine_weight(n, k, BITS, GS, seed=seed)
        return tuple(torch.stack([torch.roll(t, 7 * (rank * local_e + i) + 1, 0) for i in range(local_e)]) for t in w)

    ex = experts.make([todev(local_experts(ni, d, 1)), todev(local_experts(ni, d, 2))], todev(local_experts(d, ni, 3)), GS)
    wr = (torch.randn((e, d), generator=g) * 0.05).to(torch.bfloat16).to(dev)
    layer = tp.ExpertParallelMoE(wr, ex, top_k, rank * local_e, e)
    wo = synthetic.affine_weight(d, ko // world, BITS, GS, seed=30 + rank)
    o_proj = qmm.pack(*todev(wo), GS)
    red, red_note = None, None
    if world > 1:
        try:                                                 # peer mappings can be refused by a box's set-up: every rank must
            red = tp.PeerReducer(max(rows_list) * d, device=dev)         # agree, or all fall back to the collectives
            made = 1
        except Exception as exc:                             # noqa: BLE001
            made, red_note = 0, f"peer buffers unavailable ({type(exc).__name__}: {exc})"[:200]
        agree = torch.tensor([made], device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if not int(agree.item()):
            red, red_note = None, red_note or "peer buffers unavailable on another rank"

    def biggest(us: float) -> float:
        t = torch.tensor([us], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, iters=20) -> float:
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return biggest(a.elapsed_time(b) * 1e3 / iters)

    def graph_timed(fn, blocks=10, replays=5) -> float:
        side = side_stream()
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(blocks):
                fn()
        graph.replay()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(replays):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        us = biggest(a.elapsed_time(b) * 1e3 / (blocks * replays))
        del graph
        return us

    out = {}
    for rows in rows_list:
        prefill = rows > 128
        buf = layer.buffers(rows, dev, prefill=prefill)
        attn = synthetic.activations(rows, ko // world, 50 + rank).to(dev)
        project = qmm.prefill_matmul if prefill else qmm.matmul

        def block(reducer):
            if reducer is None:
                return layer.run(tp.ordered_all_reduce(project(attn, o_proj)), buf)
            part = reducer.partial((rows, d))
            project(attn, o_proj, out=part)
            return layer.run(reducer.reduce(part), buf, reducer=reducer)

        entry = {"us": graph_timed(lambda: block(red)), "us_eager": timed(lambda: block(red)),
                 "timing": "us: ten blocks replayed from one CUDA graph; us_eager: eager launches; CUDA events, max over ranks",
                 "reduce": "peer memory, one launch" if red is not None else (red_note or "none (one rank)") if world == 1 or red_note
                 else "collectives"}
        if red is not None:
            entry["us_collectives"] = graph_timed(lambda: block(None))
            entry["us_collectives_eager"] = timed(lambda: block(None))
            code = torch.tensor([_lib.device_error(attn)], device=dev)
            dist.all_reduce(code, op=dist.ReduceOp.MAX)
            if int(code.item()):                             # a wait on a peer ran out: the peer figure is not a result
                entry["peer_error"] = int(code.item())
                entry["us"], entry["us_eager"] = entry["us_collectives"], entry["us_collectives_eager"]
                entry["reduce"] = "collectives (a wait on a peer ran out)"
                red = None

        # the same block step by step: each step replayed alone from a CUDA graph of ten (no host launch cost between
        # them; a step that waits for the other ranks, the reductions, still does)
        state = {"h": torch.zeros((rows, d), dtype=torch.bfloat16, device=dev)}
        part_of = (lambda: red.partial((rows, d))) if red is not None else (lambda: state.setdefault(
            "own", torch.empty((rows, d), dtype=torch.bfloat16, device=dev)))
        reduce_of = (lambda p: red.reduce(p)) if red is not None else (lambda p: p)
        width = layer.experts.width

        def route():
            moe.router(state["h"], layer.router[:e], buf.logits[:rows, :e], prefill=prefill)
            moe.select_local_rows(buf.logits[:rows], buf, top_k, e, layer.first, layer.experts.count)
            experts.route(buf.pick[:rows], buf.plan)

        steps = [("o_proj", lambda: state.__setitem__("p", project(attn, o_proj, out=part_of()))),
                 ("reduce_attention", lambda: state.__setitem__("h", reduce_of(state["p"]))),
                 ("route", route),
                 ("gate_up", lambda: experts.gate_up(state["h"], layer.experts, buf.plan, buf.act.view(-1, width), rows)),
                 ("down", lambda: experts.down(buf.act.view(-1, width), layer.experts, buf.plan, buf.y.view(-1, d), rows)),
                 ("combine", lambda: state.__setitem__("p", moe.combine(buf.y[:rows], buf.wts[:rows], part_of()))),
                 ("reduce_experts", lambda: reduce_of(state["p"]))]
        entry["phases_us"] = {}
        for name, fn in steps:                                   # in order: each step leaves the next one's inputs
            if red is None and name.startswith("reduce"):        # one rank: nothing to reduce (and nothing to capture)
                fn()
                continue
            entry["phases_us"][name] = round(graph_timed(fn), 1)
        out[f"M{rows}"] = entry
    if red is not None:
        red.close()
    return out


def glue_bench(dev) -> dict:
    """The row-wise glue that feeds the matmuls, at decode and prompt row counts: microseconds and bytes moved per
    second (reads of the inputs, writes of the outputs and of the group sums) against the measured HBM peak.  A ring of
    buffer sets larger than L2 keeps the figures honest."""

    import torch

    from tensorfold_b200 import synthetic
    from tensorfold_b200.families.qwen3_5.cuda import glue

    peak, _ = measured_peaks()
    stream = side_stream()
    d, n = 5120, 17408
    out = {"add_rmsnorm": {}, "swiglu": {}}
    for rows in (16, 2048):
        ring = max(2, -(-3 * L2_BYTES // (8 * rows * d)))
        ring = min(ring, 64)
        xs = [synthetic.activations(rows, d, 3).to(dev) for _ in range(min(ring, 4))]
        w = torch.ones((d,), dtype=torch.bfloat16, device=dev)
        sets = [(xs[i % len(xs)].clone(), xs[(i + 1) % len(xs)].clone()) for i in range(ring)]
        with torch.cuda.stream(stream):
            glue.add_rmsnorm(sets[0][0], sets[0][1], w, 1e-6)
            torch.cuda.synchronize()
        _, times = graph_time(lambda i: glue.add_rmsnorm(sets[i % ring][0], sets[i % ring][1], w, 1e-6), 4 * ring, stream)
        us = sorted(times)[len(times) // 2] * 1e3 / (4 * ring)
        moved = 8 * rows * d + 4 * rows * (d // 64)
        out["add_rmsnorm"][f"M{rows}"] = {"us": us, "gb_s": moved / us / 1e3, "of_measured_hbm": moved / us / 1e3 / peak}
        del sets
        ring = max(2, min(32, -(-3 * L2_BYTES // (6 * rows * n))))
        gu = [(synthetic.activations(rows, n, 5 + i).to(dev), synthetic.activations(rows, n, 9 + i).to(dev)) for i in range(min(ring, 3))]
        sets = [(gu[i % len(gu)][0].clone(), gu[i % len(gu)][1].clone()) for i in range(ring)]
        with torch.cuda.stream(stream):
            glue.swiglu(*sets[0])
            torch.cuda.synchronize()
        _, times = graph_time(lambda i: glue.swiglu(*sets[i % ring]), 4 * ring, stream)
        us = sorted(times)[len(times) // 2] * 1e3 / (4 * ring)
        moved = 6 * rows * n + 4 * rows * (n // 64)
        out["swiglu"][f"M{rows}"] = {"us": us, "gb_s": moved / us / 1e3, "of_measured_hbm": moved / us / 1e3 / peak}
        del sets, gu
        torch.cuda.empty_cache()
    return out


def load_path_bench(dev, pack: bool = True) -> dict:
    """Checkpoint -> device: one gate_proj-sized projection (4 copies, about 200 MB) written as a safetensors file in
    the temporary directory, then read by byte range, uploaded and tiled.  GB/s of file bytes, whole and for the shard
    rank 1 of 4 owns; whether reads went around the page cache depends on the box's file system."""

    import tempfile
    import time as _time

    import torch

    from tensorfold_b200 import synthetic
    from tensorfold_b200.cuda import checkpoint
    from tensorfold_b200.cuda.kernels import qmm

    n, k = synthetic.DENSE_27B["gate_proj"]
    w, sc, bi = synthetic.affine_weight(2048, k, BITS, GS, seed=77)
    reps = -(-n // 2048)
    tensors = {"weight": w.repeat(reps, 1)[:n].contiguous(), "scales": sc.repeat(reps, 1)[:n].contiguous(),
               "biases": bi.repeat(reps, 1)[:n].contiguous()}
    names = {torch.int32: "I32", torch.bfloat16: "BF16"}
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "layer.safetensors")
        header, at = {}, 0
        for i in range(4):
            for key, t in tensors.items():
                size = t.numel() * t.element_size()
                header[f"l{i}.gate_proj.{key}"] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + size]}
                at += size
        text = json.dumps(header).encode()
        with open(path, "wb") as f:
            f.write(len(text).to_bytes(8, "little"))
            f.write(text)
            for i in range(4):
                for t in tensors.values():
                    f.write(t.view(torch.uint8).numpy().tobytes())
        for label, kw in (("whole", {}), ("rank1_of_4_column", {"rank": 1, "world": 4, "parallel": "column"})):
            spans = checkpoint.Spans()
            ckpt = checkpoint.Checkpoint([path], spans)
            on_gpu = torch.device(dev).type == "cuda"
            if on_gpu:
                torch.cuda.synchronize()
            t0 = _time.perf_counter()
            for i in range(4):
                q = ckpt.linear(f"l{i}.gate_proj", device=dev, **kw)
                if pack:
                    q = qmm.pack(q.weight, q.scales, q.biases, GS)
            if on_gpu:
                torch.cuda.synchronize()
            dt = _time.perf_counter() - t0
            out[label] = {"file_mb": spans.bytes_read / 1e6, "ms": dt * 1e3, "gb_s": spans.bytes_read / dt / 1e9,
                          "around_page_cache": bool(spans.direct)}
            ckpt.close()
    return out


def run_b200(args) -> None:
    import torch
    import torch.distributed as dist

    from tensorfold_b200 import _lib, synthetic
    from tensorfold_b200.cuda import tp
    from tensorfold_b200.cuda.kernels import qmm
    from tensorfold_b200.families.qwen3_5.cuda import distributed
    from tensorfold_b200.families.qwen3_5.cuda.weights import QLinear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the hot path has no CPU implementation")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        from datetime import timedelta

        dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=180))

    rows = args.rows
    shapes = layer_shapes()
    layer_bytes = sum(weight_bytes(n, k) for _, (n, k) in shapes)
    ring = max(2, -(-4 * L2_BYTES * world // layer_bytes))   # distinct layers: each rank's ring holds > 4x L2 of weights
    column = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")          # output rows split across ranks
    layers = []
    for li in range(ring):
        packed = {}
        for pi, (name, (n, k)) in enumerate(shapes):
            w = synthetic.affine_weight(n, k, BITS, GS, seed=1000 * li + pi)
            q = QLinear(w[0].to(dev), w[1].to(dev), w[2].to(dev), gs=GS, bits=BITS)
            if world > 1:
                q = distributed.split_output(q, rank, world) if name in column else distributed.split_input(q, rank, world)
            packed[name] = qmm.pack(q.weight, q.scales, q.biases, GS)
            del q
        layers.append(packed)
    kin = {name: (k if name in column or world == 1 else k // world) for name, (n, k) in shapes}
    nout = {name: (n // world if name in column and world > 1 else n) for name, (n, k) in shapes}
    # One pinned slab for the step's inputs and one for its outputs (and the same on the device): the end-to-end arm
    # then moves a step's rows with one copy each way instead of one per projection.
    def slab(sizes, pinned):
        total = sum(sizes.values())
        buf = torch.empty((total,), dtype=torch.bfloat16).pin_memory() if pinned else torch.empty((total,), dtype=torch.bfloat16, device=dev)
        views, at = {}, 0
        for name, size in sizes.items():
            views[name] = buf[at:at + size]
            at += size
        return buf, views

    x_sizes = {name: rows * kin[name] for name, _ in shapes}
    y_sizes = {name: rows * nout[name] for name, _ in shapes}
    host_x_slab, host_xv = slab(x_sizes, True)
    host_y_slab, host_yv = slab(y_sizes, True)
    dev_x_slab, dev_xv = slab(x_sizes, False)
    dev_y_slab, dev_yv = slab(y_sizes, False)
    host_x = {name: host_xv[name].view(rows, kin[name]) for name, _ in shapes}
    host_y = {name: host_yv[name].view(rows, nout[name]) for name, _ in shapes}
    dev_x = {name: dev_xv[name].view(rows, kin[name]) for name, _ in shapes}
    dev_y = {name: dev_yv[name].view(rows, nout[name]) for name, _ in shapes}
    for i, (name, _) in enumerate(shapes):
        host_x[name].copy_(synthetic.activations(rows, kin[name], 31 + i))
    dev_x_slab.copy_(host_x_slab)
    torch.cuda.synchronize()

    if args.lanes:
        _lib.check(_lib.lib().tf_tune(b"stream_lanes", args.lanes), "tune")
    splits = {}                                              # a load-time decision per projection: its set fills the lanes once
    for names in SETS:
        counts = qmm.set_splits([(nout[n], kin[n]) for n in names], GS)
        splits.update({n: (qmm.split_k(nout[n], kin[n], GS, args.sk_target) if args.sk_target else c) for n, c in zip(names, counts)})
    row_parallel = ("o_proj", "down_proj") if world > 1 else ()
    peer = args.reduce == "peer" and world > 1               # the one-launch reduction over peer memory, or NCCL + a sum kernel
    reducers = {}
    if peer:
        try:
            reducers = {name: tp.PeerReducer(rows * nout[name], device=dev) for name in row_parallel}
            made = 1
        except Exception:                                    # noqa: BLE001 - a box that refuses peer mappings: collectives
            made = 0
        agree = torch.tensor([made], device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        peer = bool(int(agree.item()))
    partial = {name: (reducers[name].partial((rows, nout[name]), torch.float32) if peer else
                      torch.empty((rows, nout[name]), dtype=torch.float32, device=dev)) for name in row_parallel}
    reduced = {}

    def step(i: int, pdl: bool) -> None:
        """One layer as the launches of its dataflow: q/k/v (one persistent launch), o_proj (attention sits between them
        in a model), gate/up (one launch), down_proj.  With several ranks the sets are column-parallel and o/down
        row-parallel: an fp32 partial, then the rank-ordered reduction with one rounding."""

        layer = layers[i % ring]
        for names in SETS:
            if names[0] in row_parallel:
                qmm.matmul(dev_x[names[0]], layer[names[0]], f32=True, out=partial[names[0]], pdl=pdl, sk=splits[names[0]])
                reduced[names[0]] = (reducers[names[0]].reduce(partial[names[0]]) if peer else
                                     tp.ordered_all_reduce(partial[names[0]]))
            else:
                qmm.matmul_set(dev_x[names[0]], [layer[n] for n in names], sks=[splits[n] for n in names],
                               outs=[dev_y[n] for n in names], pdl=pdl)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):                 # eager warm-up (also the first, configuring, calls)
            step(i, False)
    barrier()
    if peer:
        # a peer that never answers costs a second a wait: find that out in the warm-up, not in the timed graph
        code = torch.tensor([_lib.device_error(dev_y["q_proj"])], device=dev)
        dist.all_reduce(code, op=dist.ReduceOp.MAX)
        if int(code.item()):
            peer = False
            partial = {name: torch.empty((rows, nout[name]), dtype=torch.float32, device=dev) for name in row_parallel}
            with torch.cuda.stream(stream):
                for i in range(3):
                    step(i, False)
            barrier()

    # programmatic dependent launch between this library's kernels; NCCL's kernels in between rule it out
    pdl = not args.no_pdl and (world == 1 or peer)

    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    names = [name for name, _ in shapes]

    def span(sizes, first_name, last_name):                  # [from, to) of consecutive projections in a slab
        at = 0
        for name in names:
            if name == first_name:
                lo = at
            at += sizes[name]
            if name == last_name:
                return lo, at
        raise KeyError(last_name)

    def e2e_step(i: int) -> None:
        """One layer with its copies overlapped: q/k/v's rows go in first, the other inputs while q/k/v run; each
        launch's results leave for the host while the next one computes.  Every byte of the step still crosses in the
        step."""

        layer = layers[i % ring]
        main = torch.cuda.current_stream()

        def after(stream_to, fn):                           # fn on stream_to once everything queued on main is done
            ev = torch.cuda.Event()
            ev.record(main)
            stream_to.wait_event(ev)
            with torch.cuda.stream(stream_to):
                fn()

        lo, hi = span(x_sizes, "q_proj", "v_proj")
        rest = span(x_sizes, "o_proj", "down_proj")
        after(copy_in, lambda: dev_x_slab[rest[0]:rest[1]].copy_(host_x_slab[rest[0]:rest[1]], non_blocking=True))
        staged = torch.cuda.Event()
        staged.record(copy_in)
        dev_x_slab[lo:hi].copy_(host_x_slab[lo:hi], non_blocking=True)
        for si, names in enumerate(SETS):
            if si == 1:
                main.wait_event(staged)
            qmm.matmul_set(dev_x[names[0]], [layer[n] for n in names], sks=[splits[n] for n in names],
                           outs=[dev_y[n] for n in names], pdl=False)
            a, b = span(y_sizes, names[0], names[-1])
            after(copy_out, lambda a=a, b=b: host_y_slab[a:b].copy_(dev_y_slab[a:b], non_blocking=True))
        done = torch.cuda.Event()
        done.record(copy_out)
        main.wait_event(done)

    def capture(first: int, count: int, with_copies: bool, use_pdl: bool):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for i in range(first, first + count):
                    if with_copies and world == 1:
                        e2e_step(i)
                        continue
                    if with_copies:
                        dev_x_slab.copy_(host_x_slab, non_blocking=True)
                    step(i, use_pdl)
                    if with_copies:
                        host_y_slab.copy_(dev_y_slab, non_blocking=True)
        return graph

    try:
        timed = capture(0, args.steps, False, pdl)
    except RuntimeError:
        pdl = False
        torch.cuda.synchronize()
        timed = capture(0, args.steps, False, False)

    clocks = ClockSampler(local)
    with clocks:
        with torch.cuda.stream(stream):
            timed.replay()                                   # untimed replay: graph upload, instruction caches
            torch.cuda.synchronize()
            # keep the GPU under this load while clocks are sampled.  The count is agreed across ranks: every replay
            # holds collectives, so all ranks must issue the same number of them.
            t_load = time.perf_counter()
            timed.replay()
            torch.cuda.synchronize()
            once = torch.tensor([time.perf_counter() - t_load], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(once, op=dist.ReduceOp.MAX)
            for _ in range(max(1, min(2000, int(1.5 / max(once.item(), 1e-5))))):
                timed.replay()
            barrier()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            timed.replay()                                   # EXACTLY args.steps steps
            end.record(stream)
            barrier()
            ms = start.elapsed_time(end)
            trials = []
            for _ in range(9):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record(stream)
                timed.replay()
                e.record(stream)
                torch.cuda.synchronize()
                trials.append(s.elapsed_time(e))

            # end to end: host activations in, host results out, one graph replay (copies included) and a sync per step
            e2e_graphs = [capture(i, 1, True, False) for i in range(ring)]
            for g in e2e_graphs:
                g.replay()
            barrier()
            t0 = time.perf_counter()
            for i in range(args.steps):
                e2e_graphs[i % ring].replay()
                stream.synchronize()                         # the step's result is on the host
            e2e_s = time.perf_counter() - t0
    code = torch.tensor([_lib.device_error(dev_y["q_proj"])], device=dev)
    if world > 1:
        dist.all_reduce(code, op=dist.ReduceOp.MAX)          # every rank learns of it, so every rank leaves together
    if int(code.item()) != 0:
        raise RuntimeError(f"a kernel wait gave up during the benchmark (device error {int(code.item())})")

    times = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = times.tolist()

    extras = {}
    wanted = set() if args.no_extras else set(args.extras.split(","))

    def extra(name: str, fn) -> None:                       # a failing side figure must not cost the headline line
        if "all" not in wanted and name not in wanted:
            return
        try:
            extras[name] = fn()
        except Exception as exc:                             # noqa: BLE001 - reported in the line instead
            extras[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    if world == 1:
        extra("dense_rows", lambda: dense_rows_bench(dev, layers, shapes, ring, splits))
        del layers
        torch.cuda.empty_cache()
        extra("cfg0", lambda: cfg0_bench(dev))
        extra("cfg3", lambda: cfg3_bench(dev))
        extra("lm_head", lambda: lm_head_bench(dev))
        extra("moe_layer", lambda: moe_layer_bench(dev))
        extra("glue", lambda: glue_bench(dev))
        extra("load_path", lambda: load_path_bench(dev))
    if "all" in wanted or "moe_block" in wanted:
        extras["moe_block"] = moe_block_tp_bench(dev, rank, world)      # holds collectives: every rank runs it or none

    per_step = len(SETS)                                     # matmul launches a step
    launches = args.steps * (per_step + len(row_parallel))   # + a reduction each (the peer-memory kernel, or the sum kernel
                                                             #   behind NCCL's collectives)
    io_bytes = sum(2 * rows * (n + k) for _, (n, k) in shapes)
    value = layer_bytes * args.steps / (ms * 1e-3) / 1e9     # the whole layer's weights, all ranks together
    peak, peak_kind = measured_peaks()
    achieved = (layer_bytes / world + io_bytes) * args.steps / (ms * 1e-3) / 1e9      # per GPU
    med = sorted(trials)[len(trials) // 2]
    if rank == 0:
        line = {
            "metric": "affine_4bit_g64_qmm_weight_gbps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"dense27b_layer_projections_4bit_g64_M{rows}", "rows": rows, "bits": BITS,
                       "group": GS, "projections": {name: list(shape) for name, shape in shapes},
                       "weight_bytes_per_step": layer_bytes, "ring_layers": ring,
                       "l2": f"steps cycle a ring of {ring} distinct layers ({ring * layer_bytes / world / 1e6:.0f} MB of weights "
                             "a GPU, larger than the 126 MB L2), so no flush is needed",
                       "launch": "CUDA graph of the timed steps" + (", programmatic dependent launch" if pdl else "")
                                 + "; four persistent launches a layer, in dataflow order: q/k/v, o, gate/up, down",
                       "parallelism": "single GPU" if world == 1 else
                       f"tp{world}: q/k/v/gate/up column-parallel, o/down row-parallel (fp32 partials, rank-ordered sum, one rounding; "
                       + ("one launch a reduction over peer memory)" if peer else "NCCL all-gather and a sum kernel)"),
                       "k_slices": splits, "lanes": args.lanes},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "traffic": TRAFFIC_RATIO * (layer_bytes / world + io_bytes) / per_step,
                         "kernel": "qmm_stream_kernel<4,64,%d,*>" % (1 if rows <= 8 else 2),
                         "bytes_per_launch": (layer_bytes / world + io_bytes) / per_step,
                         "us_per_launch": ms * 1e3 / (args.steps * per_step), "launches_per_step": per_step,
                         "note": "the launches of a step run one after another on one stream, so the step time over "
                                 "their count is the kernel's average duration", "per": "GPU"},
            "median_of_9": {"ms_per_step": med / args.steps, "value": layer_bytes * args.steps / (med * 1e-3) / 1e9},
            "e2e": {"value": layer_bytes * args.steps / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": sum(2 * rows * kin[name] for name, _ in shapes),
                    "d2h_bytes_per_step": sum(2 * rows * nout[name] for name, _ in shapes), "ms_per_step": e2e_ms / args.steps},
            "clocks": clocks.summary(),
        }
        line.update(extras)
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(rows)
        print(json.dumps(line))
    if world > 1:
        # CUDA graphs that hold NCCL nodes keep the communicator busy: tearing the process group down under them can
        # block for ever, so the graphs go first and the process leaves without the (optional) group teardown.
        del timed, e2e_graphs
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


CASE_SETS = {"qkv_set": ("q_proj", "k_proj", "v_proj"), "gate_up_set": ("gate_proj", "up_proj")}


def run_case(args) -> None:
    """A small fixed case for profiler captures: one projection of the layer, three distinct weight copies (larger than
    L2 together), six launches at --rows rows."""

    import torch

    from tensorfold_b200 import synthetic
    from tensorfold_b200.cuda.kernels import qmm

    dev = "cuda"
    if args.case in CASE_SETS:                               # a set of projections of one input in one persistent launch
        names = CASE_SETS[args.case]
        k = synthetic.DENSE_27B[names[0]][1]
        copies = []
        for i in range(3):
            ws = [synthetic.affine_weight(*synthetic.DENSE_27B[name], BITS, GS, seed=10 * i + j) for j, name in enumerate(names)]
            copies.append([qmm.pack(w[0].to(dev), w[1].to(dev), w[2].to(dev), GS) for w in ws])
        x = synthetic.activations(args.rows, k, 0).to(dev)
        for i in range(6):
            y = qmm.matmul_set(x, copies[i % 3])[0]
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "rows": args.rows, "launches": 6, "max_abs": float(y.float().abs().max())}))
        return
    if args.case == "moe_experts":                           # the routed experts of the MoE layer (128 experts, top 6)
        from tensorfold_b200.cuda import experts

        d, e, ni, top_k = 2688, 128, 1856, 6
        one = lambda n, k, s: synthetic.affine_weight(n, k, BITS, GS, seed=s)
        rep = lambda w: tuple(torch.stack([torch.roll(t, 7 * i + 1, 0) for i in range(e)]).to(dev) for t in w)
        ex = experts.make([rep(one(ni, d, 1)), rep(one(ni, d, 2))], rep(one(d, ni, 3)), GS)
        g = torch.Generator().manual_seed(4)
        picks = torch.stack([torch.randperm(e, generator=g)[:top_k] for _ in range(args.rows)]).to(torch.int32).to(dev)
        plan = experts.Plan(args.rows, top_k, e, dev, prefill=args.prefill)
        experts.route(picks, plan)
        x = synthetic.activations(args.rows, d, 0).to(dev)
        act = torch.empty((args.rows * top_k, ni), dtype=torch.bfloat16, device=dev)
        y = torch.empty((args.rows * top_k, d), dtype=torch.bfloat16 if args.prefill else torch.float32, device=dev)
        for _ in range(3):
            experts.gate_up(x, ex, plan, act, args.rows)
            experts.down(act, ex, plan, y, args.rows)
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "rows": args.rows, "prefill": args.prefill, "launches": 6,
                          "items": int(plan.counts[0]), "max_abs": float(y.float().abs().max())}))
        return
    n, k = synthetic.DENSE_27B[args.case]
    qs = []
    for i in range(3):
        w = synthetic.affine_weight(n, k, BITS, GS, seed=i)
        qs.append(qmm.pack(w[0].to(dev), w[1].to(dev), w[2].to(dev), GS))
    x = synthetic.activations(args.rows, k, 0).to(dev)
    for i in range(6):
        y = qmm.prefill_matmul(x, qs[i % 3]) if args.prefill else qmm.matmul(x, qs[i % 3])
    torch.cuda.synchronize()
    print(json.dumps({"case": args.case, "rows": args.rows, "prefill": args.prefill, "launches": 6, "max_abs": float(y.float().abs().max())}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--impl", default="b200", choices=("b200", "reference"))
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--case", default="", help="profiler case: run six launches of one projection (e.g. gate_proj), of a set (qkv_set, gate_up_set) or "
                    "of the routed experts (moe_experts) and exit")
    ap.add_argument("--prefill", action="store_true", help="with --case: the prefill arithmetic (tcgen05 kernel)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--reduce", default="peer", choices=("peer", "collectives"),
                    help="several ranks: the one-launch reduction over peer memory, or NCCL collectives and a sum kernel")
    ap.add_argument("--no-extras", action="store_true", help="skip the MoE layer / row-count sweeps reported beside the headline")
    ap.add_argument("--extras", default="all", help="which side figures to run: all, or a comma list of moe_layer, "
                    "dense_rows, cfg0, cfg3, lm_head, glue, load_path, moe_block")
    ap.add_argument("--lanes", type=int, default=0, help="tuning: super-blocks a thread block streams side by side (0 = default)")
    ap.add_argument("--sk-target", type=int, default=0, help="tuning: occupancy target of the K split (0 = default)")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
