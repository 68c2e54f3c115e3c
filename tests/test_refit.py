"""Refit planning: executing the plan's strided copies (emulated with tensor indexing, all ranks in one process) must
give every engine rank exactly the weights that loading the HF tensors into its shard gives."""

import pytest
import torch

from rl_b200.models.config import preset
from rl_b200.models.hf_io import iter_hf_tensors, load_hf_tensors
from rl_b200.models.transformer import build_model
from rl_b200.parallel.tensor import TP
from rl_b200.refit.plan import build_refit_plan, serving_param_layout


def _shards(cfg, full_sd, tp):
    out = []
    for r in range(tp):
        m = build_model(cfg, dtype=torch.float32, init=False, tp=TP(None, r, tp))
        with torch.no_grad():
            for p in m.parameters():
                p.zero_()
        load_hf_tensors(m, full_sd.get)
        out.append(m)
    return out


@pytest.mark.parametrize("tp_train,tp_serve,world", [(1, 2, 2), (2, 1, 2), (4, 2, 4), (2, 4, 4), (2, 2, 4)])
@pytest.mark.parametrize("variant", ["llama", "qwen3"])
def test_plan_reproduces_serving_shards(tp_train, tp_serve, world, variant):
    over = dict(num_attention_heads=8, num_key_value_heads=4, head_dim=32, hidden_size=256, vocab_size=512)
    if variant == "qwen3":
        over.update(qk_norm=True, attention_bias=False, tie_word_embeddings=False)
    else:
        over.update(attention_bias=True, tie_word_embeddings=True)
    cfg = preset("tiny-llama-oracle", **over)
    full = build_model(cfg, dtype=torch.float32, seed=4)
    sd = {n: t.detach().clone() for n, t in iter_hf_tensors(full)}
    train = _shards(cfg, sd, tp_train)
    want = _shards(cfg, sd, tp_serve)
    plan = build_refit_plan(cfg, world, tp_train, tp_serve)
    layout, total = serving_param_layout(cfg, tp_serve)
    arenas = [torch.full((total,), float("nan")) for _ in range(world)]
    for op in plan.ops:
        src = dict(train[op.src_rank % tp_train].named_parameters())[op.src_param].detach().reshape(-1)
        dst = arenas[op.dst_rank]
        base = layout[op.dst_param][0] + op.dst_offset
        for r in range(op.rows):
            dst[base + r * op.dst_pitch : base + r * op.dst_pitch + op.row_elems] = src[op.src_offset + r * op.src_pitch : op.src_offset + r * op.src_pitch + op.row_elems]
        # a rank pulls from its own training replica
        assert op.src_rank // tp_train == op.dst_rank // tp_train
    for d in range(world):
        for name, p in want[d % tp_serve].named_parameters():
            off, (r, c) = layout[name]
            assert r * c == p.numel(), name
            assert torch.equal(arenas[d][off : off + p.numel()].view(p.shape), p.detach()), (d, name)
    if tp_train == 1:  # data-parallel training: every engine shard is a local slice, nothing crosses the link
        assert all(plan.bytes_over_link(r) == (0, 0) for r in range(world))
    if tp_train == tp_serve:
        assert all(o.src_rank == o.dst_rank for o in plan.ops)


def test_synchronizer_cpu_twin_builds_serving_model():
    from rl_b200.refit.synchronizer import WeightSynchronizer

    cfg = preset("tiny-llama-oracle")
    train = build_model(cfg, dtype=torch.float32, seed=1)
    ws = WeightSynchronizer(train, cfg, tp_serve=1)
    ws.sync_weights()
    from rl_b200.models.transformer import PackedBatch

    ids = torch.randint(0, cfg.vocab_size, (2, 12))
    b = PackedBatch.from_padded(ids, torch.tensor([12, 7]))
    assert torch.equal(ws.serving_model.logits(b), train.logits(b))
    with torch.no_grad():
        train.norm.mul_(1.5)
    ws.sync_weights()
    assert torch.equal(ws.serving_model.logits(b), train.logits(b))


def test_packed_broadcast_pack_unpack_round_trip():
    """Byte-exact packing of mixed-dtype tensors into one buffer (each padded to 16 bytes) and back."""
    from rl_b200.refit.packed_broadcast import _buckets, pack, unpack

    torch.manual_seed(0)
    ts = [("a", torch.randn(3, 5).to(torch.bfloat16)), ("b", torch.arange(7, dtype=torch.int64)), ("c", torch.randn(2, 2, 2)),
          ("d", torch.zeros(0, dtype=torch.float32)), ("e", torch.randn(1).to(torch.float16))]
    buf = pack([t for _, t in ts], "cpu")
    assert buf.dtype == torch.uint8 and buf.numel() % 16 == 0
    out = dict(unpack(buf, [(n, tuple(t.shape), t.dtype) for n, t in ts]))
    for n, t in ts:
        assert out[n].dtype == t.dtype and out[n].shape == t.shape and torch.equal(out[n].view(torch.uint8), t.contiguous().view(torch.uint8))
    groups = list(_buckets(ts, bucket_bytes=64))
    assert [n for g in groups for n, _ in g] == ["a", "b", "c", "d", "e"] and len(groups) >= 2
