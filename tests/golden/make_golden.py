"""Regenerate ``tests/golden/reference_golden.npz`` by importing the reference's own Python on CPU.

Run once where a checkout of the reference is available:

    python tests/golden/make_golden.py /path/to/reference

It calls only pure-Python/torch-CPU functions of the reference (no GPU, no Triton launch): ``dequantize``, ``split_k``,
``bucket``, ``packed_shape``, ``input_slice``, ``max_items``, ``output_rows`` and ``sum_rank_partials``, and the expected
expert plan ``want_plan`` of the reference's own test (tests/cuda/test_experts.py:107-115), taken out of that file by
name because the module around it needs a GPU to import.  The bodies of the Triton kernels ``_topk_rows`` and
``_combine`` (cuda/moe.py:56-85,130-141) are run as plain Python over a small NumPy stand-in for ``tl`` (the way the
reference's own tests/test_cuda_affine.py:36-78 runs its affine kernels without a GPU): the selection order, the tie
rule, the normalisation, every rounding to bf16 and the shared slot are then the reference's own statements; only
``exp`` is NumPy's instead of the GPU's.  The SwiGLU vectors follow the float64 formula of the reference's test
(tests/cuda/test_experts.py:158-162) computed with torch.  The outputs are
small and committed; the tests compare the CPU oracle (and, on a GPU, the kernels) against them, so nothing at test time
needs the reference.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch


def main(ref: str) -> None:
    sys.path.insert(0, str(Path(ref) / "src"))
    from tensorfold.cuda import experts as r_experts
    from tensorfold.cuda.kernels import affine as r_affine
    from tensorfold.cuda.kernels import qmm as r_qmm
    from tensorfold.families.qwen3_5.cuda import distributed as r_dist
    from tensorfold.families.qwen3_5.cuda import qmm as r_lane

    out: dict[str, np.ndarray] = {}
    g = torch.Generator().manual_seed(20240611)

    # dequantize for every bits x group: 5 rows of 4 groups, raw 32-bit words so every straddle pattern occurs
    for bits in r_affine.BITS:
        for gs in r_affine.GROUPS:
            n, k = 5, gs * 4
            words = torch.randint(-(2 ** 31), 2 ** 31 - 1, (n, k * bits // 32), generator=g, dtype=torch.int64)
            words = words.to(torch.int32)
            scales = (torch.rand((n, 4), generator=g) * 0.02 + 0.001).to(torch.bfloat16)
            biases = (torch.randn((n, 4), generator=g) * 0.05).to(torch.bfloat16)
            deq = r_lane.dequantize(words, scales, biases, bits=bits, gs=gs)
            tag = f"deq_b{bits}_g{gs}"
            out[tag + "_words"] = words.numpy()
            out[tag + "_scales"] = scales.view(torch.int16).numpy().view(np.uint16)
            out[tag + "_biases"] = biases.view(torch.int16).numpy().view(np.uint16)
            out[tag + "_w"] = deq.numpy()
            assert r_affine.packed_shape(words.shape, scales.shape, biases.shape, bits, gs) == (n, k)

    # shape-only planning functions
    shapes = [(4096, 4096), (6144, 5120), (1024, 5120), (5120, 6144), (17408, 5120), (5120, 17408), (14336, 4096),
              (6144, 8192), (48, 5120), (200, 1024), (1536, 2048), (248320, 5120), (2688, 1856), (1856, 2688),
              (10240, 5120), (64, 512), (128, 1024)]
    out["split_k_shapes"] = np.asarray(shapes, dtype=np.int64)
    out["split_k_g64"] = np.asarray([r_qmm.split_k(n, k, 64) for n, k in shapes], dtype=np.int64)
    out["split_k_g32"] = np.asarray([r_qmm.split_k(n, k, 32) for n, k in shapes], dtype=np.int64)
    out["split_k_g64_t296"] = np.asarray([r_qmm.split_k(n, k, 64, 296) for n, k in shapes], dtype=np.int64)
    ms = [1, 2, 7, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 128, 2048]
    out["bucket_m"] = np.asarray(ms, dtype=np.int64)
    out["bucket"] = np.asarray([r_qmm.bucket(m) for m in ms], dtype=np.int64)

    # two-rank input slices for every format (k = 4 groups)
    rows = []
    for bits in r_affine.BITS:
        for gs in r_affine.GROUPS:
            for rank in (0, 1):
                (a, b), (g0, g1) = r_affine.input_slice(gs * 4, bits, gs, rank)
                rows.append([bits, gs, rank, a, b, g0, g1])
    out["input_slice"] = np.asarray(rows, dtype=np.int64)

    # expert plan capacity
    cases = [(96, 129, 16), (112, 129, 16), (12288, 129, 64), (14336, 129, 64), (7, 50, 16), (161, 50, 16), (2100, 50, 64)]
    out["max_items_cases"] = np.asarray(cases, dtype=np.int64)
    out["max_items"] = np.asarray([r_experts.max_items(*c) for c in cases], dtype=np.int64)

    # partition map: plain halves, segments (k, k, v) and head blocks
    out["rows_plain_r0"] = r_dist.output_rows(16, 0).numpy()
    out["rows_plain_r1"] = r_dist.output_rows(16, 1).numpy()
    out["rows_seg_r0"] = r_dist.output_rows(40, 0, segments=(8, 8, 24)).numpy()
    out["rows_seg_r1"] = r_dist.output_rows(40, 1, segments=(8, 8, 24)).numpy()
    out["rows_block_r1"] = r_dist.output_rows(32, 1, block=8).numpy()

    # rank-ordered sum: fp32 add, one rounding
    p0 = torch.randn((7, 33), generator=g) * 3
    p1 = torch.randn((7, 33), generator=g) * 3
    out["rank_p0"], out["rank_p1"] = p0.numpy(), p1.numpy()
    out["rank_sum_bf16"] = r_dist.sum_rank_partials([p0, p1]).view(torch.int16).numpy().view(np.uint16)

    # expert-table unpack nibble rule (cuda/experts.py:52-53): slot s of a block word holds input 2 (s % 4) + s // 4
    out["expert_slot_inputs"] = np.asarray([2 * (s % 4) + s // 4 for s in range(8)], dtype=np.int64)
    out["lane_offsets"] = np.asarray(r_qmm.OFFSETS, dtype=np.int64)

    # the expert plan the reference's test expects (pairs grouped by expert in pair order, items of at most `tile`)
    import ast

    source = (Path(ref) / "tests" / "cuda" / "test_experts.py").read_text()
    fn = next(node for node in ast.parse(source).body if isinstance(node, ast.FunctionDef) and node.name == "want_plan")
    scope: dict = {"torch": torch}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "want_plan", "exec"), scope)      # noqa: S102 - the reference's function
    for tag, (rows, slots, e, tile) in {"a": (23, 7, 50, 16), "b": (300, 7, 50, 64), "c": (40, 9, 12, 16)}.items():
        picks = torch.stack([torch.randperm(e, generator=g)[:slots] for _ in range(rows)]).to(torch.int32)
        picks[:, 0] = 3                                        # one expert with a pair in every row
        items, members, distinct = scope["want_plan"](picks, e, tile)
        out[f"plan_{tag}_case"] = np.asarray([rows, slots, e, tile, distinct], dtype=np.int64)
        out[f"plan_{tag}_picks"] = picks.numpy()
        out[f"plan_{tag}_items"] = np.asarray(items, dtype=np.int64).reshape(-1, 3)
        out[f"plan_{tag}_members"] = np.asarray(members, dtype=np.int64)

    # ---- the Triton bodies of the router's top-k and of the combine, run over NumPy
    def bf16(a):
        u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
        return r.view(np.float32)

    class Arr(np.ndarray):
        def to(self, dtype):
            if dtype == "bf16":
                return bf16(np.asarray(self, dtype=np.float32)).view(Arr)
            return np.asarray(self).astype(dtype).view(Arr)

    arr = lambda v: np.asarray(v).view(Arr)

    class Ptr:
        def __init__(self, values, offsets=0):
            self.values, self.offsets = values.reshape(-1), offsets

        def __add__(self, offsets):
            return Ptr(self.values, self.offsets + offsets)

    class TL:
        int32, float32, bfloat16 = np.int32, np.float32, "bf16"
        program = [0, 0]
        constexpr = None
        static_range = range

        @staticmethod
        def load(pointer, mask=True, other=0):
            offsets, mask = np.broadcast_arrays(pointer.offsets, mask)
            result = np.full(offsets.shape, other, dtype=pointer.values.dtype)
            result[mask] = pointer.values[offsets[mask]]
            return arr(result)

        @staticmethod
        def store(pointer, value, mask=True):
            offsets, value, mask = np.broadcast_arrays(pointer.offsets, value, mask)
            pointer.values[offsets[mask]] = value[mask]

        program_id = classmethod(lambda cls, axis: cls.program[axis])
        arange = staticmethod(lambda a, b: arr(np.arange(a, b)))
        zeros = staticmethod(lambda shape, dtype: arr(np.zeros(shape, dtype=dtype)))
        where = staticmethod(lambda c, a, b: arr(np.where(c, a, b)))
        max = staticmethod(lambda a, axis: np.max(a, axis=axis))
        min = staticmethod(lambda a, axis: np.min(a, axis=axis))
        exp = staticmethod(lambda a: np.exp(np.float32(a), dtype=np.float32) if np.ndim(a) == 0 else arr(np.exp(a, dtype=np.float32)))

    source = (Path(ref) / "src" / "tensorfold" / "cuda" / "moe.py").read_text()
    bodies = [n for n in ast.parse(source).body if isinstance(n, ast.FunctionDef) and n.name in ("_topk_rows", "_combine")]
    for fn in bodies:
        fn.decorator_list = []
        for a in fn.args.args:
            a.annotation = None
    scope = {"tl": TL}
    exec(compile(ast.Module(body=bodies, type_ignores=[]), "moe_kernels_on_numpy", "exec"), scope)      # noqa: S102

    rows, ne, top_k = 24, 128, 6
    logits = (torch.randn((rows, ne + 1), generator=g) * 2).numpy().astype(np.float32)
    logits[0, 7] = logits[0, 3] = logits[0].max() + 1           # the largest logit twice: the lower id comes first
    logits[1, 100:104] = logits[1, :100].max() + 0.5            # four equal logits among the chosen
    logits[2, :] = 0.25                                         # all equal: ids 0 .. top_k - 1
    pick = np.zeros((rows, top_k + 1), dtype=np.int32)
    wts = np.zeros((rows, top_k + 1), dtype=np.float32)
    next_pow2 = lambda v: 1 << (v - 1).bit_length()
    for r in range(rows):
        TL.program = [r, 0]
        scope["_topk_rows"](Ptr(logits), Ptr(pick), Ptr(wts), NE=ne, NL=ne + 1, TOPK=top_k, SLOTS=top_k + 1,
                            BLOCK=next_pow2(ne + 1), SLOTP=next_pow2(top_k + 1))
    out["topk_case"] = np.asarray([rows, ne, top_k], dtype=np.int64)
    out["topk_logits"], out["topk_picks"], out["topk_wts"] = logits, pick, wts

    crow, slots, dims = 5, top_k + 1, 700
    y = (torch.randn((crow, slots, dims), generator=g)).numpy().astype(np.float32)
    w = bf16((torch.rand((crow, slots), generator=g)).numpy())
    cout = np.zeros((crow, dims), dtype=np.float32)
    for r in range(crow):
        for blk in range(-(-dims // 512)):
            TL.program = [r, blk]
            scope["_combine"](Ptr(y), Ptr(w), Ptr(cout), S=slots, D=dims, BLOCK=512)
    out["combine_y"], out["combine_w"], out["combine_out"] = y, w, cout

    # ---- SwiGLU as the reference's test states it in float64 (tests/cuda/test_experts.py:158-162)
    gv = (torch.randn((6, 64), generator=g) * 3).float()
    uv = (torch.randn((6, 64), generator=g) * 3).float()
    for tag, limit in (("", 0.0), ("_limit", 2.5)):
        gg, uu = (t.to(torch.bfloat16).double() for t in (gv, uv))
        if limit:
            gg, uu = gg.clamp(max=limit), uu.clamp(-limit, limit)
        out["swiglu_out" + tag] = ((gg * torch.sigmoid(gg)).to(torch.bfloat16).double() * uu).numpy()
    out["swiglu_g"], out["swiglu_u"] = gv.numpy(), uv.numpy()

    dest = Path(__file__).with_name("reference_golden.npz")
    np.savez_compressed(dest, **out)
    print(f"wrote {dest} ({dest.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("TENSORFOLD_REFERENCE"):
        sys.exit("usage: make_golden.py <reference checkout>   (or set TENSORFOLD_REFERENCE)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["TENSORFOLD_REFERENCE"])
