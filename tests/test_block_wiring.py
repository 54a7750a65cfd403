"""How a block hands the norm of the residual stream to its parts (no GPU: fake parts)."""
import torch

from dlgo_b200.parts.base import DeferredNorm
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

    def deferred(self, residual):
        return DeferredNorm(self, residual, "fake", torch.ones(residual.shape[1]), 1e-5, torch.float32)


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


class Reader:
    takes_deferred_norm = True


def test_a_part_that_takes_it_gets_the_norm_uncomputed_and_computes_it_once():
    norm, r = FakeNorm(), torch.ones(3, 4)
    x = norm_of(norm, r, Ctx(), Reader())
    assert isinstance(x, DeferredNorm) and norm.calls == 0
    assert x.shape == r.shape and x.kind == "fake" and x.residual is r
    t = x.tensor()
    assert torch.equal(t, r * 2) and x.tensor() is t and norm.calls == 1


def test_other_parts_and_other_norms_get_a_tensor():
    norm, r = FakeNorm(), torch.ones(3, 4)
    assert torch.equal(norm_of(norm, r, Ctx(), object()), r * 2) and norm.calls == 1
    assert torch.equal(norm_of(norm, r, Ctx()), r * 2)
    assert torch.equal(norm_of(PlainNorm(), r, Ctx(), Reader()), r + 1)      # a norm that offers no promise


def test_pending_slices_are_added_first_and_then_the_norm_is_computed():
    norm, r = FakeNorm(), torch.ones(3, 4)
    parts = torch.full((2, 3, 4), 0.5)
    x = norm_of(norm, r, Ctx(parts), Reader())
    assert torch.is_tensor(x) and norm.fused == 1 and torch.equal(r, torch.full((3, 4), 2.0)) and torch.equal(x, r * 2)
    r2, ctx = torch.ones(3, 4), Ctx(parts)
    x2 = norm_of(PlainNorm(), r2, ctx, Reader())                              # no fused pass: settled first
    assert ctx.settled == 1 and torch.equal(r2, torch.full((3, 4), 2.0)) and torch.equal(x2, r2 + 1)
