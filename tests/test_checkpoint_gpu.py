"""The load path end to end on a B200: a rank's shard read from safetensors files straight to the device and tiled must
be the tiles of the shard cut from the whole tensors, and multiply to the same bits."""

import pytest
import torch

from tensorfold_b200 import synthetic
from tensorfold_b200.cuda import checkpoint
from tensorfold_b200.cuda.kernels import qmm
from tensorfold_b200.families.qwen3_5.cuda import distributed
from tensorfold_b200.families.qwen3_5.cuda.weights import QLinear

from gpu_util import DEV
from test_checkpoint import projection, write_safetensors

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("parallel", ["column", "row", None])
def test_loaded_shard_equals_the_cut_and_tiled_whole(tmp_path, parallel):
    n, k, gs = 512, 1024, 64
    src = projection(n, k, 4, gs, 11)
    path = tmp_path / "model.safetensors"
    write_safetensors(path, {f"mlp.up_proj.{key}": v for key, v in src.items()}, pad=1)
    whole = QLinear(src["weight"].view(torch.int32), src["scales"], src["biases"], gs=gs, bits=4)
    ckpt = checkpoint.Checkpoint([path])
    rank, world = 1, 2
    got = checkpoint.load_packed(ckpt, "mlp.up_proj", DEV, rank=rank, world=world, parallel=parallel)
    if parallel == "column":
        cut = distributed.split_output(whole, rank, world)
    elif parallel == "row":
        cut = distributed.split_input(whole, rank, world)
    else:
        cut = whole
    want = qmm.pack(cut.weight.to(DEV), cut.scales.to(DEV), cut.biases.to(DEV), gs)
    assert (got.n, got.k) == (want.n, want.k) and torch.equal(got.weight, want.weight)
    x = synthetic.activations(5, want.k, 3).to(DEV)
    assert torch.equal(qmm.matmul(x, got), qmm.matmul(x, want))
    ckpt.close()
