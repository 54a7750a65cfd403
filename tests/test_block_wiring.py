"""How a block hands the norm of the residual stream to its parts (no GPU: fake parts)."""
import torch

from dlgo_b200.parts.block import norm_of


class FakeNorm:
    def __init__(self):
        self.calls = 0
        self.fused = 0

    def forward(self, residual, rows=None):
        self.calls += 1
        return residual * 2

    def forward_fused(self, residual, parts, rows=None):
        self.fused += 1
        residual += parts.sum(0)
        return residual * 2


class PlainNorm:
    def forward(self, residual, rows=None):
        return residual + 1


class Ctx:
    def __init__(self, pending=None):
        self.pending = pending
        self.settled = 0

    def take_pending(self):
        p, self.pending = self.pending, None
        return p

    def settle(self, residual):
        p = self.take_pending()
        if p is not None:
            residual += p.sum(0)
            self.settled += 1


def test_with_nothing_pending_the_norm_runs_once():
    norm, r = FakeNorm(), torch.ones(3, 4)
    assert torch.equal(norm_of(norm, r, Ctx()), r * 2) and norm.calls == 1 and norm.fused == 0
    assert torch.equal(norm_of(PlainNorm(), r, Ctx()), r + 1)


def test_pending_slices_are_added_first_and_then_the_norm_is_computed():
    norm, r = FakeNorm(), torch.ones(3, 4)
    parts = torch.full((2, 3, 4), 0.5)
    x = norm_of(norm, r, Ctx(parts))
    assert norm.fused == 1 and norm.calls == 0 and torch.equal(r, torch.full((3, 4), 2.0)) and torch.equal(x, r * 2)
    r2, ctx = torch.ones(3, 4), Ctx(parts)
    x2 = norm_of(PlainNorm(), r2, ctx)                              # no fused pass: settled first
    assert ctx.settled == 1 and torch.equal(r2, torch.full((3, 4), 2.0)) and torch.equal(x2, r2 + 1)


def test_a_block_names_its_norms_and_may_have_any_number():
    from dlgo_b200.parts.base import Block
    from dlgo_b200.parts.block import PreNormBlock
    import pytest
    n = {"mixer_norm": FakeNorm(), "ffn_norm": FakeNorm(), "post_mixer_norm": PlainNorm()}
    blk = Block(object(), None, n)
    assert list(blk.parts()) == ["mixer_norm", "ffn_norm", "post_mixer_norm", "mixer"]       # no feed-forward: no role
    pre = PreNormBlock(object(), object(), n)
    assert pre.mixer_norm is n["mixer_norm"] and pre.ffn_norm is n["ffn_norm"]
    with pytest.raises(ValueError, match="ffn_norm"):
        PreNormBlock(object(), object(), {"mixer_norm": FakeNorm()})
