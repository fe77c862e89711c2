"""How the pre-norm block and the model pass a norm that one part has handed over to the next
(parts.base.NormHandover): host logic only, with stand-in parts that record what they are given."""

from types import SimpleNamespace

import torch

from redline_b200.ops import build
from redline_b200.parts.base import NormHandover
from redline_b200.parts.block import PreNormBlock


class FakeNorm:
    def __init__(self, name):
        self.name = name
        self.calls = 0

    def add_norm(self, residual, delta, out, rows_idx=None, rows=None):
        self.calls += 1


class FakePart:
    """A mixer or feed-forward whose fused form is taken (or not) and leaves a hand-over (or not)."""

    def __init__(self, takes=True, leaves=True, leaves_for=None):
        self.takes, self.leaves, self.leaves_for = takes, leaves, leaves_for
        self.seen = []          # (hand_in, next_norm) of every call of the fused form

    def forward_into(self, residual, norm, ctx, cache=None, state=None):
        self.seen.append((ctx.hand_in, ctx.next_norm))
        if not self.takes:
            ctx.hand_out = "left by a part that declined"        # must be ignored
            return False
        if self.leaves and ctx.next_norm is not None:
            ctx.hand_out = NormHandover(self.leaves_for or ctx.next_norm, None, None)
        return True

    def forward(self, x, ctx, cache=None, state=None):
        return x


def fake_rt():
    ws = SimpleNamespace(get=lambda name, shape, dtype: torch.zeros(shape, dtype=dtype))
    return SimpleNamespace(workspace=ws, max_tokens=4, dtype=torch.float32)


def fresh_ctx(**kw):
    base = dict(T=2, next_norm=None, hand_in=None, hand_out=None, block_next_norm=None, block_hand=None)
    base.update(kw)
    return SimpleNamespace(**base)


def block(mixer, ffn):
    return PreNormBlock(FakeNorm("mixer_norm"), mixer, FakeNorm("ffn_norm"), ffn, fake_rt())


def test_a_norm_goes_from_the_mixer_to_the_feed_forward_and_on_to_the_next_block():
    b = block(FakePart(), FakePart())
    after = FakeNorm("next block's first norm")
    ctx = fresh_ctx(block_next_norm=after)
    res = torch.zeros(2, 8)
    assert b.forward(res, None, ctx, None, None) is None
    assert b.mixer.seen == [(None, b.ffn_norm)]
    hand, nxt = b.ffn.seen[0]
    assert isinstance(hand, NormHandover) and hand.norm is b.ffn_norm and nxt is after
    assert ctx.block_hand.norm is after                       # carried on to the block after this one
    assert (ctx.hand_in, ctx.hand_out, ctx.next_norm) == (None, None, None)
    assert b.mixer_norm.calls == 0 and b.ffn_norm.calls == 0  # no norm ran as a kernel of its own
    assert b.first_norm() is b.mixer_norm


def test_a_hand_over_from_the_block_before_reaches_the_mixer_only_if_it_is_for_its_norm():
    b = block(FakePart(), FakePart())
    mine = NormHandover(b.mixer_norm, None, None)
    ctx = fresh_ctx(block_hand=mine)
    b.forward(torch.zeros(2, 8), None, ctx, None, None)
    assert b.mixer.seen[0][0] is mine
    other = NormHandover(FakeNorm("someone else's"), None, None)
    b2 = block(FakePart(), FakePart())
    ctx = fresh_ctx(block_hand=other)
    b2.forward(torch.zeros(2, 8), None, ctx, None, None)
    assert b2.mixer.seen[0][0] is None
    assert ctx.block_hand is None                             # the last block: nothing comes after it


def test_a_part_that_declines_or_leaves_something_for_another_norm_breaks_the_chain():
    # the mixer declines: its norm runs as a kernel, and what it wrote into the context is dropped
    b = block(FakePart(takes=False), FakePart())
    ctx = fresh_ctx(block_next_norm=FakeNorm("after"))
    out = b.forward(torch.zeros(2, 8), None, ctx, None, None)
    assert out is not None and b.mixer_norm.calls == 1 and b.ffn.seen == []      # the unfused feed-forward ran
    assert ctx.block_hand is None and ctx.hand_out is None
    # the mixer leaves a hand-over made for some other norm: the feed-forward does not get it
    b = block(FakePart(leaves_for=FakeNorm("other")), FakePart())
    ctx = fresh_ctx()
    b.forward(torch.zeros(2, 8), None, ctx, None, None)
    assert b.ffn.seen[0][0] is None
    # a delta still pending from the block before: no fused mixer, hence no hand-over taken
    b = block(FakePart(), FakePart())
    ctx = fresh_ctx(block_hand=NormHandover(b.mixer_norm, None, None))
    b.forward(torch.zeros(2, 8), torch.zeros(2, 8), ctx, None, None)
    assert b.mixer.seen == [] and b.mixer_norm.calls == 1


def test_built_files_of_other_source_versions_are_removed(tmp_path):
    keep = tmp_path / "gemm-aaaa.so"
    for name in ("gemm-aaaa.so", "gemm-bbbb.so", "gemm_tc-cccc.so", "notes.txt"):
        (tmp_path / name).write_bytes(b"x")
    build.remove_other_versions([str(keep)])
    assert sorted(p.name for p in tmp_path.iterdir()) == ["gemm-aaaa.so", "gemm_tc-cccc.so", "notes.txt"]
