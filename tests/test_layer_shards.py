"""Host logic that walks a model's layer records (CPU): rank shards of a layer and of a whole model keep every checkpoint
word (the shards of all ranks put back together are the original tensors), narrow projections stack only when their
formats agree, and a rank's head candidates always contain what a single GPU would have chosen from.
Follows families/qwen3_5/cuda/distributed.py:101-165, qmm_fast.py:84-115 and decode_tp.py:72-80 of the reference."""

import pytest
import torch

from tensorfold_b200 import synthetic
from tensorfold_b200.cuda.kernels import affine
from tensorfold_b200.families.qwen3_5.cuda import decode_tp, distributed, qmm_fast
from tensorfold_b200.families.qwen3_5.cuda.weights import GDN, Attention, Config, Layer, QLinear, Weights

CFG = Config(hidden=256, intermediate=512, heads=4, kv_heads=2, head_dim=32, k_heads=2, v_heads=4, dk=32, dv=32, vocab=1024)


def linear(n, k, seed, bits=4, gs=64):
    return QLinear(*synthetic.raw_weight(n, k, bits, gs, seed), gs=gs, bits=bits)


def make_layer(seed=0):
    c = CFG
    attn = Attention(q=linear(c.heads * c.head_dim * 2, c.hidden, seed + 1), k=linear(c.kv_heads * c.head_dim, c.hidden, seed + 2),
                     v=linear(c.kv_heads * c.head_dim, c.hidden, seed + 3), o=linear(c.hidden, c.heads * c.head_dim, seed + 4))
    kd, vd = c.k_heads * c.dk, c.v_heads * c.dv
    gdn = GDN(qkv=linear(2 * kd + vd, c.hidden, seed + 5), z=linear(vd, c.hidden, seed + 6), b=linear(c.v_heads * 16, c.hidden, seed + 7),
              a=linear(c.v_heads * 16, c.hidden, seed + 8), out=linear(c.hidden, vd, seed + 9),
              conv=torch.arange((2 * kd + vd) * 4, dtype=torch.float32).view(-1, 4), A_log=torch.arange(c.v_heads, dtype=torch.float32),
              dt_bias=torch.arange(c.v_heads, dtype=torch.float32) + 100)
    return Layer(linear=True, gdn=gdn, attn=attn, gate=linear(c.intermediate, c.hidden, seed + 10),
                 up=linear(c.intermediate, c.hidden, seed + 11), down=linear(c.hidden, c.intermediate, seed + 12))


@pytest.mark.parametrize("world", [2, 4])
def test_layer_shards_put_back_together_are_the_layer(world):
    layer = make_layer()
    if world == 4:                                             # two kv heads do not split four ways
        with pytest.raises(ValueError):
            distributed.split_layer(layer, CFG, 0, world)
        return
    shards = [distributed.split_layer(layer, CFG, r, world) for r in range(world)]
    assert [s.q_heads for s in shards] == [CFG.heads // world] * world and shards[1].rank == 1

    def rows_back(get, segments=None, block=1):
        whole = get(layer)
        out = torch.empty_like(whole.weight)
        for r, s in enumerate(shards):
            out[distributed.output_rows(whole.n, r, world, segments, block)] = get(s.layer).weight
        assert torch.equal(out, whole.weight)

    rows_back(lambda l: l.attn.q, block=2 * CFG.head_dim)
    rows_back(lambda l: l.attn.k, block=CFG.head_dim)
    rows_back(lambda l: l.gate)
    rows_back(lambda l: l.up)
    kd, vd = CFG.k_heads * CFG.dk, CFG.v_heads * CFG.dv
    rows_back(lambda l: l.gdn.qkv, segments=(kd, kd, vd))
    rows_back(lambda l: l.gdn.z, block=CFG.dv)
    for get in (lambda l: l.attn.o, lambda l: l.down, lambda l: l.gdn.out):      # inputs cut in whole groups and words
        whole = get(layer)
        assert torch.equal(torch.cat([get(s.layer).weight for s in shards], dim=1), whole.weight)
        assert torch.equal(torch.cat([get(s.layer).scales for s in shards], dim=1), whole.scales)
    conv_rows = distributed.output_rows(layer.gdn.qkv.n, 1, world, (kd, kd, vd))
    assert torch.equal(shards[1].layer.gdn.conv, layer.gdn.conv[conv_rows])
    assert torch.equal(torch.cat([s.layer.gdn.A_log for s in shards]), layer.gdn.A_log)
    assert torch.equal(torch.cat([s.layer.gdn.dt_bias for s in shards]), layer.gdn.dt_bias)


def test_model_shards_divide_the_config_and_optionally_the_head():
    w = Weights(CFG, embed=None, layers=[make_layer(0), make_layer(20)], head=linear(CFG.vocab, CFG.hidden, 99))
    half = distributed.split_weights(w, 1, 2)
    assert (half.config.heads, half.config.kv_heads, half.config.intermediate) == (2, 1, 256)
    assert half.head is w.head and len(half.layers) == 2
    split = distributed.split_weights(w, 1, 2, split_head=True)
    assert torch.equal(split.head.weight, w.head.weight[CFG.vocab // 2:])
    with pytest.raises(ValueError):
        distributed.split_weights(w, 2, 2)


def test_narrow_projections_stack_only_in_one_format():
    layer = make_layer()
    qmm_fast.stack_small(layer)
    assert layer.attn.kv.n == 2 * CFG.kv_heads * CFG.head_dim
    assert torch.equal(layer.attn.kv.weight, torch.cat([layer.attn.k.weight, layer.attn.v.weight]))
    assert layer.gdn.zba.n == layer.gdn.z.n + layer.gdn.b.n + layer.gdn.a.n
    other = make_layer()
    other.attn.v = linear(CFG.kv_heads * CFG.head_dim, CFG.hidden, 3, bits=8)       # another width: left alone
    qmm_fast.stack_small(other)
    assert other.attn.kv is None and other.gdn.zba is not None


def test_rank_candidates_contain_the_single_gpu_choice():
    g = torch.Generator().manual_seed(5)
    logits = torch.randn((6, 512), generator=g)
    logits[2, 100] = logits[2, 300] = 9.0                       # a tie across the two halves: the lower id must win
    halves = [logits[:, :256], logits[:, 256:]]
    values, ids = zip(*[decode_tp.split_candidates(h, None, r * 256) for r, h in enumerate(halves)])
    merged_v, merged_i = torch.cat(values, dim=1), torch.cat(ids, dim=1)
    pick = torch.where(merged_v[:, 0] >= merged_v[:, 1], merged_i[:, 0], merged_i[:, 1])       # rank 0 first: first maximum
    assert torch.equal(pick, logits.argmax(dim=-1)) and int(pick[2]) == 100
    s = decode_tp.Sampling(seed=1, temperature=0.7, top_k=20)
    values, ids = zip(*[decode_tp.split_candidates(h, s, r * 256) for r, h in enumerate(halves)])
    assert values[0].shape == (6, 20 + decode_tp.MARGIN) and values[0].dtype == torch.float32
    want = torch.topk(logits, 20, dim=-1).indices
    for r in range(6):
        assert set(want[r].tolist()) <= set(torch.cat(ids, dim=1)[r].tolist())
    every = decode_tp.split_candidates(halves[1], decode_tp.Sampling(top_k=0), 256)
    assert every[0].shape == (6, 256) and int(every[1].min()) == 256


def test_input_slices_follow_the_word_rule():
    for rank in range(4):
        (w0, w1), (g0, g1) = affine.input_slice(4096, 3, 64, rank, 4)
        assert (w1 - w0) * 32 == 1024 * 3 and g1 - g0 == 16
