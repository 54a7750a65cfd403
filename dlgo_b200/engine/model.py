"""A causal language model put together from an :class:`ArchitectureSpec`.

Nothing here knows an architecture by name.  The model builds every part from
the description, asks the parts which tensors they want, hands them their
tensors, and runs the layers in the order the description lists: embedding,
run entries one after another on one fp32 residual stream, final norm on the
wanted rows only, head (the reference does the same for its single sequence and
computes logits for the last position only, models/llm/forward.go:123-204,
models/llm/forward_batch.go:222-235).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from ..config.spec import ArchitectureSpec, PartSpec
from ..parts import registry as R
from ..parts.base import Block, CacheNeed, ParamSpec, Part, StateNeed


class CausalLM:
    def __init__(self, spec: ArchitectureSpec):
        spec.validate()
        self.spec = spec
        self.embedding: Part = R.EMBEDDINGS.build(spec.embedding)
        self.final_norm = R.NORMS.build(spec.final_norm)
        self.head: Part = R.HEADS.build(spec.head)
        self.positions = {name: R.POSITION_ENCODINGS.build(ps) for name, ps in spec.position_encodings.items()}
        self.blocks: List[Block] = []
        for ls in spec.layers:
            mixer = R.MIXERS.build(ls.mixer) if ls.mixer is not None else None
            ffn = R.FEED_FORWARDS.build(ls.ffn) if ls.ffn is not None else None
            norms = {role: R.NORMS.build(ns) for role, ns in ls.norms.items()}
            self.blocks.append(R.BLOCKS.build(PartSpec(ls.block, {"mixer": mixer, "ffn": ffn, "norms": norms})))
        self.order = list(spec.order)
        for i, e in enumerate(self.order):
            if e.cache_of is not None:
                mine = self._cache_need(e.layer)
                theirs = self._cache_need(self.order[e.cache_of].layer)
                if mine is None or theirs is None or (mine.num_kv_heads, mine.head_dim) != (
                        theirs.num_kv_heads, theirs.head_dim):
                    raise ValueError(f"run entry {i} cannot read the cache of entry {e.cache_of}: their shapes differ")
        self.runtime: Any = None
        self.fused_runs: Dict[int, Any] = {}
        self.prompt_runs: Dict[int, Any] = {}

    # ------------------------------------------------------------ declarations
    def _named_parts(self) -> List[Tuple[str, Part]]:
        out: List[Tuple[str, Part]] = [(self.spec.embedding_prefix, self.embedding)]
        for ls, blk in zip(self.spec.layers, self.blocks):
            for role, part in blk.parts().items():      # whatever the block declares: any number of norms
                out.append((ls.prefix + ls.names[role], part))
        out.append((self.spec.final_norm_prefix, self.final_norm))
        out.append((self.spec.head_prefix, self.head))
        return out

    def expected_tensors(self) -> Dict[str, ParamSpec]:
        """Every tensor the weight file must hold: absolute name -> shape and init rule."""
        table: Dict[str, ParamSpec] = {}
        for prefix, part in self._named_parts():
            for rel, ps in part.param_specs().items():
                name = prefix + rel
                if name in table:
                    raise ValueError(f"two parts want the tensor {name!r}")
                table[name] = ps
        return table

    def _cache_need(self, layer: int) -> Optional[CacheNeed]:
        mixer = self.blocks[layer].mixer
        return mixer.cache_need() if mixer is not None else None

    def cache_needs(self) -> Tuple[List[Optional[CacheNeed]], List[Optional[int]], Dict[int, StateNeed]]:
        """Per run entry: what it keeps per position, whose cache it borrows, its fixed-size state."""
        needs: List[Optional[CacheNeed]] = []
        borrows: List[Optional[int]] = []
        states: Dict[int, StateNeed] = {}
        for i, e in enumerate(self.order):
            mixer = self.blocks[e.layer].mixer
            needs.append(mixer.cache_need() if mixer is not None else None)
            borrows.append(e.cache_of)
            sn = mixer.state_need() if mixer is not None else None
            if sn is not None:
                states[i] = sn
        return needs, borrows, states

    # ------------------------------------------------------------------ weights
    def load_weights(self, source: Any, runtime: Any) -> None:
        """Check the file against the expected table (one error for everything), then load."""
        from ..weights.loader import check_against

        expected = {n: ps.shape for n, ps in self.expected_tensors().items()}
        check_against(expected, source.found())
        self.runtime = runtime
        tied = getattr(self.head, "tied_to", None)
        for prefix, part in self._named_parts():
            if part is self.head and tied:
                part.load(lambda rel: source.get(tied), runtime)
            else:
                part.load(lambda rel, _p=prefix: source.get(_p + rel), runtime)
        for pe in self.positions.values():
            pe.prepare(runtime)
        runtime.forget_copies()
        from . import fused_decode, prompt_run
        self.fused_runs = fused_decode.plan_runs(self, runtime)
        self.prompt_runs = prompt_run.plan_runs(self, runtime)

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: Any, cache: Any, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens; logits [wanted, vocab] fp32 for the packed rows ``want_rows`` (int32)."""
        residual = self.embedding.forward(ctx.token_ids)
        i = 0
        while i < len(self.order):
            run = (self.fused_runs if ctx.decode else self.prompt_runs).get(i)
            if run is not None and run.takes(ctx, cache):
                # a run of like blocks: one persistent kernel on a decode step (where that is switched on), one
                # native loop over the layers' launches on a prompt step
                ctx.settle(residual)
                run.run(self, residual, ctx, cache)
                i += run.n
                continue
            blk = self.blocks[self.order[i].layer]
            if not getattr(blk, "handles_pending", False):
                ctx.settle(residual)
            blk.forward(residual, ctx, cache.view(i), cache.state.view(i), self.positions)
            i += 1
        if want_rows is None or want_rows.numel() == 0:
            ctx.settle(residual)
            return None
        pending = ctx.take_pending()
        if pending is not None and ctx.want_identity and hasattr(self.final_norm, "forward_fused"):
            # every row is wanted exactly once, so no row's slices are added twice
            x = self.final_norm.forward_fused(residual, pending, want_rows)
        else:
            if pending is not None:
                ctx.pending = pending
                ctx.settle(residual)
            x = self.final_norm.forward(residual, want_rows)
        return self.head.forward(x)
