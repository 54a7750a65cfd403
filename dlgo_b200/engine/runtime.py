"""What a run is made of: the device, the precision, and the per-step context the parts read."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r}: bfloat16 or float32") from None


class Runtime:
    """Device and precision of a run.

    ``dtype`` is the type of weights, activations between kernels and the cache:
    ``torch.bfloat16`` (tensor-core contractions, fp32 accumulation) or
    ``torch.float32`` (everything in true 32-bit on the fp32 pipes).  The
    residual stream, norm statistics, softmax, rotations and logits are fp32 in
    both.
    """

    def __init__(self, device="cuda:0", dtype="bfloat16"):
        self.device = torch.device(device)
        self.dtype = parse_dtype(dtype)
        if self.device.type != "cuda":
            raise RuntimeError(
                f"the engine runs on a CUDA device only (asked for {self.device}); there is no CPU path")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; the engine has no CPU path")
        self._compute_copies: Dict[Tuple[int, torch.dtype], Tuple[torch.Tensor, torch.Tensor]] = {}

    def compute_copy(self, t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``t`` in the compute precision; tensors that share storage (tied weights) share the copy."""
        dtype = dtype or self.dtype
        if t.dtype == dtype:
            return t
        # the source is kept alive beside its copy, so its address cannot be handed to another
        # tensor while the entry exists
        key = (t.data_ptr(), dtype)
        hit = self._compute_copies.get(key)
        if hit is None or hit[0].shape != t.shape:
            hit = (t, t.to(dtype))
            self._compute_copies[key] = hit
        return hit[1]

    def forget_copies(self) -> None:
        self._compute_copies.clear()


@dataclass
class StepContext:
    """One step's batch as the parts see it (device tensors are int32).

    Tokens of all sequences are packed one after another; sequence ``i`` brings
    ``seq_ntok[i]`` tokens at positions ``seq_start[i] ...``.
    """

    runtime: Runtime
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor      # [T]
    token_pos: torch.Tensor      # [T] absolute position of each token in its sequence
    token_seq: torch.Tensor      # [T] index of the token's sequence in this batch
    seq_slot: torch.Tensor       # [B] cache slot of each sequence
    seq_slots_host: List[int]
    seq_start_host: List[int]
    seq_ntok_host: List[int]
    decode: bool                 # every sequence brings exactly one token
    max_len: int                 # longest sequence after this step (host; sizes grids)
    captured: bool = False       # inside a CUDA graph: sizes must not depend on lengths
    capacity: int = 0            # longest sequence the cache can hold
    want_identity: bool = False  # the wanted rows are exactly rows 0..T-1, each once
    pending: Optional[torch.Tensor] = None   # fp32 [slices, T, d] still to be added to the residual stream
    _tiles: Dict[Tuple[int, bool], Tuple[torch.Tensor, int, int]] = field(default_factory=dict)
    _scratch: Dict[str, torch.Tensor] = field(default_factory=dict)

    def tiles(self, tokens_per_tile: int, heaviest_first: bool = False) -> Tuple[torch.Tensor, int, int]:
        """Tiles of at most ``tokens_per_tile`` consecutive tokens of one sequence:
        (device tensor [n, 3] of (sequence, first token, count), n, largest count).  In the order of the
        tokens, or with ``heaviest_first`` by the number of keys a tile's last token sees, most first
        (a causal kernel whose blocks start in table order then ends with its short tiles)."""
        hit = self._tiles.get((tokens_per_tile, heaviest_first))
        if hit is not None:
            return hit
        rows: List[Tuple[int, int, int]] = []
        ends: List[int] = []
        off = 0
        biggest = 1
        for i, n in enumerate(self.seq_ntok_host):
            for b in range(0, n, tokens_per_tile):
                c = min(tokens_per_tile, n - b)
                rows.append((i, off + b, c))
                ends.append(self.seq_start_host[i] + b + c)
                biggest = max(biggest, c)
            off += n
        if heaviest_first:
            rows = [rows[j] for j in sorted(range(len(rows)), key=lambda j: -ends[j])]
        t = torch.tensor(rows, dtype=torch.int32).to(self.runtime.device, non_blocking=True)
        self._tiles[(tokens_per_tile, heaviest_first)] = (t, len(rows), biggest)
        return self._tiles[(tokens_per_tile, heaviest_first)]

    def scratch(self, name: str, numel: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """A scratch buffer that lives for the step (shared by the layers, which run one after another)."""
        t = self._scratch.get(name)
        if t is None or t.numel() < numel or t.dtype != dtype:
            t = torch.empty((max(numel, 1),), dtype=dtype, device=self.runtime.device)
            self._scratch[name] = t
        return t


    # A part whose last contraction leaves its K-slices unsummed may hand them over instead of adding
    # them to the residual itself: the next reader of the residual (a norm that can fuse the sum, or
    # `settle`) adds them, in slice order.
    def defer(self, residual: torch.Tensor, parts: torch.Tensor) -> None:
        if self.pending is not None:
            self.settle(residual)
        self.pending = parts

    def take_pending(self) -> Optional[torch.Tensor]:
        p, self.pending = self.pending, None
        return p

    def settle(self, residual: torch.Tensor) -> None:
        """Add what is pending into the residual now."""
        p = self.take_pending()
        if p is not None:
            from ..csrc import kernels as K
            K.add_rmsnorm(residual, p, None, 0.0, None)

    def zeros(self, name: str, numel: int, dtype: torch.dtype = torch.int32) -> torch.Tensor:
        """A buffer that is zero when first handed out; kernels that use it leave it zero."""
        t = self._scratch.get(name)
        if t is None or t.numel() < numel or t.dtype != dtype:
            t = torch.zeros((max(numel, 1),), dtype=dtype, device=self.runtime.device)
            self._scratch[name] = t
        return t


def build_context(runtime: Runtime, tokens: Sequence[Sequence[int]], slots: Sequence[int], starts: Sequence[int],
                  capacity: int) -> StepContext:
    """Pack a batch: ``tokens[i]`` are sequence i's next tokens, at positions ``starts[i] ...``."""
    ids: List[int] = []
    pos: List[int] = []
    seq: List[int] = []
    for i, (tk, st) in enumerate(zip(tokens, starts)):
        n = len(tk)
        ids.extend(int(x) for x in tk)
        pos.extend(range(st, st + n))
        seq.extend([i] * n)
    T = len(ids)
    meta = torch.tensor([ids, pos, seq], dtype=torch.int32)
    if T > 0:
        meta = meta.pin_memory() if T >= 1024 else meta
    meta = meta.to(runtime.device, non_blocking=True)
    slot_t = torch.tensor(list(slots), dtype=torch.int32).to(runtime.device, non_blocking=True)
    ntok = [len(t) for t in tokens]
    return StepContext(
        runtime=runtime, n_tokens=T, n_seqs=len(tokens), token_ids=meta[0], token_pos=meta[1], token_seq=meta[2],
        seq_slot=slot_t, seq_slots_host=list(slots), seq_start_host=list(starts), seq_ntok_host=ntok,
        decode=all(n == 1 for n in ntok), max_len=max((s + n for s, n in zip(starts, ntok)), default=0),
        capacity=capacity)
