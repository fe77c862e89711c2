"""The step's metadata buffer, field by field, built on the CPU (no kernels run)."""

import numpy as np
import pytest
import torch

from redline_b200.cache import CacheManager, GroupInfo
from redline_b200.engine.batch import BatchBuilder, RowSampling, Segment
from redline_b200.parts.spec import CacheSpec


def setup(window=0):
    groups = [GroupInfo(CacheSpec.keys_values("full", 2, 64), [0])]
    if window:
        groups.append(GroupInfo(CacheSpec.keys_values("window", 2, 64, window), [1]))
    cache = CacheManager(groups, [32] * len(groups), 16, 4)
    return cache, BatchBuilder(cache, max_tokens=128, max_seqs=4, max_rows=16, max_seq_len=128,
                               device=torch.device("cpu"))


def test_mixed_batch_layout():
    cache, b = setup()
    x, y, z = cache.open("x"), cache.open("y"), cache.open("z")
    cache.reserve(x, 40), cache.reserve(y, 21), cache.reserve(z, 70)
    ctx = b.build([
        Segment(x, list(range(100, 140)), 0, want=(39,), sampling=RowSampling(0.8, 5, 0.9, (7 << 32) | 3)),
        Segment(y, [9], 20, want=(0,)),
        Segment(z, list(range(3)), 64, want=(0, 2)),
    ])
    assert (ctx.T, ctx.S, ctx.R, ctx.num_decode, ctx.num_tiles) == (44, 3, 4, 1, 2)
    assert ctx.token_ids.tolist() == list(range(100, 140)) + [9] + [0, 1, 2]
    assert ctx.token_src.tolist() == [-1] * 44
    assert ctx.positions.tolist() == list(range(40)) + [20] + [64, 65, 66]
    assert ctx.seq_of_token.tolist() == [0] * 40 + [1] + [2] * 3
    g = ctx.groups[0]
    assert g.block_table.shape == (3, 8)
    assert g.block_table[0].tolist()[:4] == [1, 2, 3, 0] and g.block_table[1].tolist()[:3] == [4, 5, 0]
    assert g.block_table[2].tolist()[:6] == [6, 7, 8, 9, 10, 0]
    slots = g.slots.tolist()
    assert slots[:40] == [16 + i for i in range(40)]          # pages 1, 2, 3 are consecutive
    assert slots[40] == 5 * 16 + 4 and slots[41:] == [10 * 16, 10 * 16 + 1, 10 * 16 + 2]
    assert ctx.decode_info.tolist()[0] == [40, 1, 21, 0] and ctx.decode_parts == 1
    assert ctx.tile_seq.tolist() == [0, 2] and ctx.tile_tok.tolist() == [0, 41]
    assert ctx.tile_rows.tolist() == [40, 3]
    assert ctx.logit_rows.tolist() == [39, 40, 41, 43]
    assert ctx.sample_pos.tolist() == [40, 21, 65, 67]        # position of the token that would be drawn
    assert ctx.temperature.tolist() == pytest.approx([0.8, 0, 0, 0]) and ctx.top_k.tolist() == [5, 0, 0, 0]
    assert ctx.top_p.tolist() == pytest.approx([0.9, 1, 1, 1])
    assert ctx.seed_lo.tolist()[0] == 3 and ctx.seed_hi.tolist()[0] == 7
    assert ctx.state_slot.tolist() == [x.state_slot, y.state_slot, z.state_slot]
    assert ctx.host.q_start == [0, 40, 41] and ctx.host.q_len == [40, 1, 3]


def test_padding_of_a_decode_batch_and_device_fed_tokens():
    cache, b = setup()
    x, y = cache.open("x"), cache.open("y")
    cache.reserve(x, 300 // 16 * 16 // 4), cache.reserve(y, 6)
    ctx = b.build([Segment(x, [11], 70, want=(0,)), Segment(y, [0], 5, want=(0,), src_row=1)], pad_to=4)
    assert (ctx.T, ctx.S, ctx.R, ctx.num_decode, ctx.num_tiles) == (4, 4, 4, 4, 0) and ctx.has_src
    assert ctx.token_src.tolist() == [-1, 1, -1, -1] and ctx.positions.tolist() == [70, 5, 0, 0]
    assert ctx.groups[0].slots.tolist()[2:] == [0, 0]           # dummy rows write page 0
    assert ctx.groups[0].block_table[2].tolist() == [0] * 8
    assert ctx.decode_info.tolist() == [[0, 0, 71, 0], [1, 1, 6, 0], [2, 2, 1, 0], [3, 3, 1, 0]]
    assert ctx.logit_rows.tolist() == [0, 1, 2, 3]
    assert ctx.decode_parts == ctx.parts_capacity == 1
    with pytest.raises(ValueError, match="single tokens"):
        b.build([Segment(x, [1, 2], 71, want=(1,))], pad_to=4)


def test_same_shape_same_addresses_and_limits():
    cache, b = setup(window=32)
    x = cache.open("x")
    cache.reserve(x, 64)
    c1 = b.build([Segment(x, [1], 10, want=(0,))], pad_to=2)
    c2 = b.build([Segment(x, [2], 11, want=(0,))], pad_to=2)
    for name in ("token_ids", "positions", "logit_rows", "top_p"):
        assert getattr(c1, name).data_ptr() == getattr(c2, name).data_ptr()
    assert c1.groups[1].slots.data_ptr() == c2.groups[1].slots.data_ptr() and len(c1.groups) == 2
    with pytest.raises(ValueError, match="exceeds"):
        b.build([Segment(x, list(range(129)), 0)])
    with pytest.raises(ValueError, match="pages reserved"):
        b.build([Segment(x, [1], 64, want=(0,))])
    with pytest.raises(ValueError, match="max_seq_len"):
        cache.reserve(x, 128)
        b.build([Segment(x, [1, 2], 127)])
    with pytest.raises(ValueError, match="wanted index"):
        b.build([Segment(x, [1, 2], 3, want=(2,))])
