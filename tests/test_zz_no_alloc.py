"""The attention entry point that allocates nothing, called through its exported C symbol.

Some users of this library cannot ask for device memory at the time they call it: a C or C++
program that links the kernel library without PyTorch and has handed out its whole memory budget
at start-up, or code inside a callback or another library's hook where cudaMalloc is not allowed.
For them `dlgo_attention_noalloc` keeps the split-KV scratch in a fixed device array inside the
library (8 MiB per GPU, held until the process exits).  This test calls that symbol with raw
pointers, as such a caller would, and checks the result against the ordinary entry point
(`dlgo_attention`, which takes its scratch from the caller), twice in a row with different
inputs: the array is shared by all calls and keeps the last call's contents, so the second call
shows whether stale partial sums can leak into a result.  Both entry points run the same kernel,
so each result is also compared with a plain float32 softmax over the keys of every head, which an
error common to both could not pass.  Needs a GPU.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LIMIT_FLOATS = 2 * 1024 * 1024      # DLGO_ATTENTION_NOALLOC_FLOATS in csrc/attention_noalloc.h


def _case(seed, dtype, lens, hq=8, hkv=2, hd=64):
    """A decode step over `lens` cached positions per sequence, with pages laid out in scrambled order."""
    torch.manual_seed(seed)
    B = len(lens)
    n_pages = sum((n + 63) // 64 for n in lens) + 2
    max_pages = max((n + 63) // 64 for n in lens)
    kp = torch.randn(n_pages, hkv, 64, hd, device=DEV).to(dtype)
    vp = torch.randn(n_pages, hkv, 64, hd, device=DEV).to(dtype)
    perm = torch.randperm(n_pages).tolist()
    pt = torch.full((B, max_pages), -1, dtype=torch.int32)
    for i, n in enumerate(lens):
        for pg in range((n + 63) // 64):
            pt[i, pg] = perm.pop()
    q = torch.randn(B, hq * hd, device=DEV).to(dtype)
    tiles = torch.tensor([[i, i, 1] for i in range(B)], dtype=torch.int32, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    return dict(q=q, kp=kp, vp=vp, pt=pt.to(DEV), tiles=tiles, slots=slots, pos=pos, B=B, hq=hq, hkv=hkv, hd=hd)


def _call_noalloc(lib, c, n_splits, out):
    from dlgo_b200.csrc.kernels import dtype_code
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    i = ctypes.c_int
    return lib.dlgo_attention_noalloc(
        p(c["q"]), i(dtype_code(c["q"].dtype)), i(c["B"]), i(c["q"].stride(0)), p(c["kp"]), p(c["vp"]), p(c["pt"]),
        i(c["pt"].shape[1]), p(c["tiles"]), i(c["B"]), i(1), p(c["slots"]), p(c["pos"]), p(out), i(out.stride(0)),
        i(c["hq"]), i(c["hkv"]), i(c["hd"]), i(64), i(n_splits), i(c["hq"] // c["hkv"]), i(0),
        ctypes.c_float(1.0 / math.sqrt(c["hd"])), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _plain(c):
    """softmax(q . k / sqrt(hd)) v over the keys 0 .. pos of every head, in float32 with tensor operations
    (models/llm/forward.go:258-278); kv head = head // (heads per kv head)."""
    B, hq, hkv, hd = c["B"], c["hq"], c["hkv"], c["hd"]
    out = torch.zeros(B, hq * hd)
    q, kp, vp, pt, pos = (c[k].float().cpu() if c[k].is_floating_point() else c[k].cpu() for k in ("q", "kp", "vp", "pt", "pos"))
    for b in range(B):
        n = int(pos[b]) + 1
        pages = [int(pt[b, pg]) for pg in range((n + 63) // 64)]
        for h in range(hq):
            g = h // (hq // hkv)
            keys = torch.cat([kp[p, g] for p in pages])[:n]
            vals = torch.cat([vp[p, g] for p in pages])[:n]
            s = (keys @ q[b, h * hd:(h + 1) * hd]) / math.sqrt(hd)
            out[b, h * hd:(h + 1) * hd] = torch.softmax(s, dim=0) @ vals
    return out


def _call_ordinary(c, n_splits):
    from dlgo_b200.csrc import kernels as K
    out = torch.full((c["B"], c["hq"] * c["hd"]), float("nan"), dtype=c["q"].dtype, device=DEV)
    scratch = torch.full((K.attention_scratch_floats(c["B"], c["hq"], c["hd"], n_splits) + 1,), float("nan"), device=DEV)
    K.attention(c["q"], c["q"].stride(0), c["B"], c["kp"], c["vp"], c["pt"], c["tiles"], 1, c["slots"], c["pos"], out,
                c["hq"], c["hkv"], c["hd"], 1.0 / math.sqrt(c["hd"]), 0, n_splits, c["hq"] // c["hkv"], scratch)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_entry_point_matches_the_ordinary_one_on_two_calls_in_a_row(dtype):
    from dlgo_b200.csrc import build
    lib = build.load_library("attention")
    lib.dlgo_attention_noalloc_needs.restype = ctypes.c_longlong
    tol = dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=1e-2, rtol=1.6e-2)
    # first call: long sequences, many slices; second call: other data, FEWER slices and shorter
    # sequences, so most of what the first call left in the shared array is still there
    for seed, lens, n_splits in ((1, [700, 64, 333, 129], 6), (2, [90, 5, 200], 3)):
        c = _case(seed, dtype, lens)
        need = lib.dlgo_attention_noalloc_needs(c["B"], c["hq"], c["hd"], n_splits)
        assert 0 < need <= LIMIT_FLOATS
        out = torch.full((c["B"], c["hq"] * c["hd"]), float("nan"), dtype=dtype, device=DEV)
        before = torch.cuda.memory_allocated()
        st = _call_noalloc(lib, c, n_splits, out)
        assert st == 0, f"dlgo_attention_noalloc returned {st}"
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        ref = _call_ordinary(c, n_splits)
        assert torch.isfinite(out.float()).all()
        torch.testing.assert_close(out.float(), ref.float(), **tol)
        plain_tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(out.float().cpu(), _plain(c), **plain_tol)
    # one slice needs no scratch at all and takes the same path
    c = _case(3, dtype, [100, 30])
    out = torch.full((2, c["hq"] * c["hd"]), float("nan"), dtype=dtype, device=DEV)
    assert _call_noalloc(lib, c, 1, out) == 0
    torch.testing.assert_close(out.float(), _call_ordinary(c, 1).float(), **tol)


def test_noalloc_entry_point_refuses_sizes_beyond_its_maximum():
    from dlgo_b200.csrc import build
    lib = build.load_library("attention")
    lib.dlgo_attention_noalloc_needs.restype = ctypes.c_longlong
    c = _case(4, torch.float32, [64] * 4)
    c["B"] = 4000                                   # claimed size only: the call must refuse before it launches
    assert lib.dlgo_attention_noalloc_needs(4000, 8, 64, 16) > LIMIT_FLOATS
    out = torch.zeros(4, 8 * 64, device=DEV)
    assert _call_noalloc(lib, c, 16, out) == -1     # DLGO_ERR_SIZE
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
