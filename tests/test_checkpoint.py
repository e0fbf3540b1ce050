"""The checkpoint -> device load path on the CPU: safetensors index, byte-range reads (around and through the page
cache) and the shards a rank reads, which must be bit-for-bit what ``distributed.split_output`` / ``split_input`` cut
from the whole tensors (reference: cuda/direct_read.py, families/glm5_next/cuda/split.py:74-229)."""

import json
import struct

import numpy as np
import pytest
import torch

from tensorfold_b200 import synthetic
from tensorfold_b200.cuda import checkpoint
from tensorfold_b200.families.qwen3_5.cuda import distributed
from tensorfold_b200.families.qwen3_5.cuda.weights import QLinear

NAMES = {torch.bfloat16: "BF16", torch.int32: "I32", torch.uint32: "U32", torch.float32: "F32", torch.float16: "F16",
         torch.uint8: "U8", torch.int64: "I64"}


def write_safetensors(path, tensors: dict, pad: int = 0) -> None:
    """A minimal writer: 8-byte header length, JSON header (padded with spaces), tensor bytes back to back."""

    header, blobs, at = {"__metadata__": {"format": "pt"}}, [], 0
    for name, t in tensors.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header).encode() + b" " * pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)


def projection(n, k, bits, gs, seed):
    w, s, b = synthetic.affine_weight(n, k, bits, gs, seed=seed)
    return {"weight": w.view(torch.uint32), "scales": s, "biases": b}


@pytest.fixture()
def files(tmp_path):
    a, b = tmp_path / "model-00001.safetensors", tmp_path / "model-00002.safetensors"
    first = {f"layers.0.q_proj.{k}": v for k, v in projection(384, 512, 4, 64, 1).items()}
    first["norm.weight"] = torch.arange(512, dtype=torch.float32)
    first["tiny"] = torch.tensor([7], dtype=torch.int64)
    second = {f"layers.0.down_proj.{k}": v for k, v in projection(256, 1024, 4, 64, 2).items()}
    second.update({f"layers.0.odd.{k}": v for k, v in projection(128, 768, 3, 32, 3).items()})
    second["norm.weight"] = torch.arange(512, dtype=torch.float32) + 1          # a later file's name wins
    write_safetensors(a, first, pad=3)
    write_safetensors(b, second, pad=5)
    return [a, b], first, second


@pytest.mark.parametrize("direct", [True, False])
def test_tensors_and_row_ranges_come_back_bit_for_bit(files, direct):
    paths, first, second = files
    ckpt = checkpoint.Checkpoint(paths, checkpoint.Spans(direct=direct))
    assert set(ckpt.keys()) == set(first) | set(second) and "tiny" in ckpt and "nothing" not in ckpt
    for name, t in {**first, **second}.items():
        got = ckpt.tensor(name)
        assert got.dtype == t.dtype and got.shape == t.shape
        assert torch.equal(got.view(torch.uint8), t.contiguous().view(torch.uint8)), name
    w = second["layers.0.down_proj.weight"]
    for lo, hi in ((0, 1), (5, 77), (255, 256), (0, 256), (9, 9)):
        got = ckpt.rows("layers.0.down_proj.weight", lo, hi)
        assert got.shape == (hi - lo, w.shape[1]) and torch.equal(got.view(torch.int32), w[lo:hi].view(torch.int32))
    with pytest.raises(ValueError):
        ckpt.rows("layers.0.down_proj.weight", 3, 257)
    with pytest.raises(KeyError):
        ckpt.tensor("nothing")
    ckpt.close()


def test_byte_ranges_at_any_offset_and_length(tmp_path):
    """Reads that start and end anywhere against the 4096-byte grid, across the piece size, and at the end of the file."""

    path = tmp_path / "blob.bin"
    rng = np.random.default_rng(0)
    data = rng.integers(0, 256, size=3 * 4096 + 1234, dtype=np.uint8)
    path.write_bytes(data.tobytes())
    for direct in (True, False):
        spans = checkpoint.Spans(direct=direct)
        for off, n in ((0, 1), (1, 4095), (4095, 2), (4096, 4096), (5000, 7000), (0, data.size), (data.size - 1, 1), (77, 0)):
            got = spans.read(path, off, n)
            assert got.dtype == torch.uint8 and np.array_equal(got.numpy(), data[off:off + n]), (direct, off, n)
        assert spans.bytes_read == sum(n for _, n in ((0, 1), (1, 4095), (4095, 2), (4096, 4096), (5000, 7000), (0, data.size),
                                                       (data.size - 1, 1), (77, 0)))
        with pytest.raises(IOError):
            spans.read(path, data.size - 3, 4)
        with pytest.raises(ValueError):
            spans.read(path, -1, 4)


def test_small_pieces_cover_a_range(tmp_path, monkeypatch):
    monkeypatch.setattr(checkpoint, "PIECE", 4096)                     # many reads per range
    path = tmp_path / "blob.bin"
    data = np.random.default_rng(1).integers(0, 256, size=50_000, dtype=np.uint8)
    path.write_bytes(data.tobytes())
    for direct in (True, False):
        got = checkpoint.Spans(direct=direct).read(path, 4097, 40_000)
        assert np.array_equal(got.numpy(), data[4097:44_097])


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_a_ranks_projection_is_what_the_shard_map_cuts(files, world):
    paths, first, second = files
    for prefix, src, bits, gs in (("layers.0.q_proj", first, 4, 64), ("layers.0.down_proj", second, 4, 64),
                                  ("layers.0.odd", second, 3, 32)):
        whole = QLinear(src[f"{prefix}.weight"].view(torch.int32), src[f"{prefix}.scales"], src[f"{prefix}.biases"], gs=gs, bits=bits)
        for rank in range(world):
            spans = checkpoint.Spans()
            ckpt = checkpoint.Checkpoint(paths, spans)
            col = ckpt.linear(prefix, bits=bits, gs=gs, rank=rank, world=world, parallel="column")
            want = distributed.split_output(whole, rank, world)
            for a, b in ((col.weight, want.weight), (col.scales, want.scales), (col.biases, want.biases)):
                assert a.shape == b.shape and torch.equal(a.view(torch.uint8), b.view(torch.uint8))
            assert col.bits == bits and col.gs == gs and col.n == whole.n // world and col.k == whole.k
            assert spans.bytes_read == whole.nbytes() // world             # a rank reads its own bytes and no others
            if whole.k % (world * gs) == 0 and (whole.k // world // gs * gs * bits) % 32 == 0:
                row = ckpt.linear(prefix, bits=bits, gs=gs, rank=rank, world=world, parallel="row")
                want = distributed.split_input(whole, rank, world)
                for a, b in ((row.weight, want.weight), (row.scales, want.scales), (row.biases, want.biases)):
                    assert a.shape == b.shape and torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def test_segmented_column_shards_keep_concatenated_projections_apart(files):
    """A fused q|k|v style weight: every rank takes its share of each segment, in segment order."""

    paths, first, _ = files
    whole = QLinear(first["layers.0.q_proj.weight"].view(torch.int32), first["layers.0.q_proj.scales"],
                    first["layers.0.q_proj.biases"], gs=64, bits=4)
    ckpt = checkpoint.Checkpoint(paths)
    for rank in range(2):
        got = ckpt.linear("layers.0.q_proj", rank=rank, world=2, parallel="column", segments=(256, 64, 64), block=8)
        want = distributed.split_output(whole, rank, 2, segments=(256, 64, 64), block=8)
        assert torch.equal(got.weight, want.weight) and torch.equal(got.scales, want.scales) and torch.equal(got.biases, want.biases)
    with pytest.raises(ValueError):
        ckpt.linear("layers.0.q_proj", rank=0, world=2, parallel="column", segments=(256, 64, 60))
    with pytest.raises(ValueError):
        ckpt.linear("layers.0.q_proj", rank=2, world=2, parallel="column")
    with pytest.raises(ValueError):
        ckpt.linear("layers.0.q_proj", bits=8)                         # the words do not hold 8-bit codes of that width
    with pytest.raises(KeyError):
        ckpt.linear("layers.0.k_proj")


def test_broken_files_are_refused(tmp_path):
    short = tmp_path / "short.safetensors"
    short.write_bytes(b"\x05\x00")
    with pytest.raises(IOError):
        checkpoint.read_header(short)
    cut = tmp_path / "cut.safetensors"
    write_safetensors(cut, {"w": torch.zeros((4, 4), dtype=torch.float32)})
    cut.write_bytes(cut.read_bytes()[:-8])                             # the data is shorter than the header says
    with pytest.raises(ValueError):
        checkpoint.Checkpoint([cut])
    odd = tmp_path / "odd.safetensors"
    text = json.dumps({"w": {"dtype": "F4", "shape": [2], "data_offsets": [0, 1]}}).encode()
    odd.write_bytes(struct.pack("<Q", len(text)) + text + b"\x00")
    with pytest.raises(ValueError):
        checkpoint.Checkpoint([odd])


@pytest.mark.parametrize("world", [1, 2, 4])
def test_a_ranks_expert_tables_are_what_shard_experts_cuts(tmp_path, world):
    from tensorfold_b200.cuda import tp

    e, ni, d, gs = 8, 64, 128, 64
    stack = lambda n, k, seed: tuple(torch.stack([synthetic.affine_weight(n, k, 4, gs, seed=seed * 100 + i)[j] for i in range(e)])
                                    for j in range(3))
    gate, up, down = stack(ni, d, 1), stack(ni, d, 2), stack(d, ni, 3)
    tensors = {}
    for proj, table in (("gate_proj", gate), ("up_proj", up), ("down_proj", down)):
        for part, t in zip(("weight", "scales", "biases"), table):
            tensors[f"layers.3.mlp.switch_mlp.{proj}.{part}"] = t.view(torch.uint32) if part == "weight" else t
    path = tmp_path / "moe.safetensors"
    write_safetensors(path, tensors, pad=2)
    for rank in range(world):
        spans = checkpoint.Spans()
        got, first = checkpoint.expert_tables(checkpoint.Checkpoint([path], spans), "layers.3.mlp.switch_mlp", rank=rank, world=world)
        (want_gate, want_up), want_down, want_first = tp.shard_experts([gate, up], down, rank, world)
        assert first == want_first
        for proj, want in (("gate_proj", want_gate), ("up_proj", want_up), ("down_proj", want_down)):
            for a, b in zip(got[proj], want):
                assert a.shape == b.shape and torch.equal(a.view(torch.uint8), b.contiguous().view(torch.uint8))
        assert spans.bytes_read == sum(t.numel() * t.element_size() for t in tensors.values()) // world
    with pytest.raises(ValueError):
        checkpoint.expert_tables(checkpoint.Checkpoint([path]), "layers.3.mlp.switch_mlp", rank=0, world=3)
    with pytest.raises(KeyError):
        checkpoint.expert_tables(checkpoint.Checkpoint([path]), "layers.4.mlp.switch_mlp")
