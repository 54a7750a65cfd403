"""Each kernel alone against a plain fp32 reference written here, at sizes other than the engine's.
Needs a GPU."""
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def K():
    from dlgo_b200.csrc import kernels
    return kernels


def tol(dtype):
    return dict(atol=2e-6, rtol=2e-6) if dtype == "float32" else dict(atol=1e-2, rtol=1.6e-2)


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    table = torch.randn(37, 50, device=DEV).to(DT[dtype])
    toks = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = K().embed(toks, table)
    assert out.dtype == torch.float32 and torch.equal(out, table.float()[toks.long()])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,eps", [(1, 1e-5), (50, 1e-6), (200, 3e-6), (2048, 1e-5), (5000, 1e-2)])
def test_rmsnorm(dtype, d, eps):
    x = torch.randn(7, d, device=DEV) * 3
    w = 1 + 0.1 * torch.randn(d, device=DEV)
    ref = P.rmsnorm(x.cpu(), w.cpu(), eps)
    out = K().rmsnorm(x, w, eps, DT[dtype])
    assert out.dtype == DT[dtype]
    torch.testing.assert_close(out.float().cpu(), ref, **tol(dtype))
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    torch.testing.assert_close(K().rmsnorm(x, w, eps, DT[dtype], rows).float().cpu(), ref[[6, 0, 3]], **tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("R,d", [(256, 48), (300, 512), (1000, 2048), (257, 3000), (260, 4096)])
def test_rmsnorm_many_rows(dtype, R, d):
    # many rows take the warp-per-row kernel
    torch.manual_seed(R + d)
    x = torch.randn(R, d, device=DEV) * 2
    x[3] *= 50.0                                                 # rows of very different scale
    w = 1 + 0.1 * torch.randn(d, device=DEV)
    ref = P.rmsnorm(x.cpu(), w.cpu(), 1e-5)
    torch.testing.assert_close(K().rmsnorm(x, w, 1e-5, DT[dtype]).float().cpu(), ref, **tol(dtype))
    rows = torch.arange(R - 1, -1, -1, dtype=torch.int32, device=DEV)
    torch.testing.assert_close(K().rmsnorm(x, w, 1e-5, DT[dtype], rows).float().cpu(), ref.flip(0), **tol(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(dtype):
    gu = (torch.randn(5, 2 * 77, device=DEV) * 4).to(DT[dtype])
    ref = P.swiglu(gu.float().cpu()[:, :77], gu.float().cpu()[:, 77:])
    torch.testing.assert_close(K().swiglu(gu).float().cpu(), ref, **tol(dtype))


# ------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K_", [(1, 1, 1), (3, 65, 17), (70, 130, 96), (129, 50, 200), (64, 64, 64), (5, 1000, 33)])
def test_gemm_simt(dtype, M, N, K_):
    k = K()
    x = torch.randn(M, K_, device=DEV).to(DT[dtype])
    w = torch.randn(N, K_, device=DEV).to(DT[dtype])
    ref = (x.double() @ w.double().t()).float()
    t = dict(atol=1e-5 * math.sqrt(K_), rtol=1e-5) if dtype == "float32" else dict(atol=3e-2 * math.sqrt(K_), rtol=1.6e-2)
    torch.testing.assert_close(k.gemm_simt(x, w, k.EPI_STORE).float(), ref, **t)
    f32 = k.gemm_simt(x, w, k.EPI_STORE_F32)
    assert f32.dtype == torch.float32
    torch.testing.assert_close(f32, ref, atol=1e-5 * math.sqrt(K_), rtol=1e-5)
    res = torch.randn(M, N, device=DEV)
    acc = res.clone()
    k.gemm_simt(x, w, k.EPI_ADD_F32, acc)
    torch.testing.assert_close(acc, res + ref, atol=1e-5 * math.sqrt(K_), rtol=1e-5)
    # a strided input (a column block of a wider tensor) is taken by its row stride
    wide = torch.randn(M, K_ + 24, device=DEV).to(DT[dtype])
    torch.testing.assert_close(k.gemm_simt(wide[:, 8:8 + K_], w, k.EPI_STORE_F32),
                               (wide[:, 8:8 + K_].double() @ w.double().t()).float(), atol=1e-5 * math.sqrt(K_), rtol=1e-5)


def test_gemm_rows_do_not_depend_on_the_batch():
    k = K()
    x = torch.randn(90, 200, device=DEV)
    w = torch.randn(77, 200, device=DEV)
    full = k.gemm_simt(x, w, k.EPI_STORE_F32)
    assert torch.equal(k.gemm_simt(x[17:18].contiguous(), w, k.EPI_STORE_F32), full[17:18])


# --------------------------------------------------------------- rope + append
def _paged(n_pages, hkv, hd, dtype, fill=float("nan")):
    return (torch.full((n_pages, hkv, 64, hd), fill, device=DEV, dtype=DT[dtype]),
            torch.full((n_pages, hkv, 64, hd), fill, device=DEV, dtype=DT[dtype]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hq,hkv,hd,rot,inter", [(4, 2, 16, 16, False), (3, 1, 32, 32, True), (5, 5, 48, 24, False),
                                                 (2, 1, 80, 32, True)])
def test_rope_append(dtype, hq, hkv, hd, rot, inter):
    from dlgo_b200.parts.rope import RotaryEmbedding
    pe = RotaryEmbedding(hd, rot, 10000.0, 300, pairing="interleaved" if inter else "split_half")
    cos, sin = pe.tables()
    # two sequences: slot 3 brings positions 62..66 (crosses a page edge), slot 1 brings position 130
    pos = [62, 63, 64, 65, 66, 130]
    seq = [0, 0, 0, 0, 0, 1]
    slots = torch.tensor([3, 1], dtype=torch.int32, device=DEV)
    pt = torch.full((4, 5), -1, dtype=torch.int32, device=DEV)
    pt[3, 0], pt[3, 1], pt[1, 2] = 5, 2, 7
    kp, vp = _paged(8, hkv, hd, dtype)
    ld = (hq + 2 * hkv) * hd
    qkv = torch.randn(6, ld, device=DEV).to(DT[dtype])
    orig = qkv.float().cpu().clone()
    K().rope_append(qkv, cos.to(DEV), sin.to(DEV), torch.tensor(pos, dtype=torch.int32, device=DEV),
                    torch.tensor(seq, dtype=torch.int32, device=DEV), slots, pt, kp, vp, hq, hkv, hd, rot, inter)

    def rotate(vec, p):
        out = vec.clone()
        for i in range(rot // 2):
            i0, i1 = (2 * i, 2 * i + 1) if inter else (i, i + rot // 2)
            c, s = cos[p, i], sin[p, i]
            out[i0] = vec[i0] * c - vec[i1] * s
            out[i1] = vec[i0] * s + vec[i1] * c
        return out

    t = tol(dtype)
    pages = {62: (5, 62), 63: (5, 63), 64: (2, 0), 65: (2, 1), 66: (2, 2), 130: (7, 2)}
    for r, p in enumerate(pos):
        for h in range(hq):
            torch.testing.assert_close(qkv[r, h * hd:(h + 1) * hd].float().cpu(), rotate(orig[r, h * hd:(h + 1) * hd], p), **t)
        pg, off = pages[p]
        for h in range(hkv):
            ko = orig[r, (hq + h) * hd:(hq + h + 1) * hd]
            vo = orig[r, (hq + hkv + h) * hd:(hq + hkv + h + 1) * hd]
            torch.testing.assert_close(kp[pg, h, off].float().cpu(), rotate(ko, p), **t)
            assert torch.equal(vp[pg, h, off].float().cpu(), vo)
    written = (~torch.isnan(kp.float())).sum().item()
    assert written == 6 * hkv * hd, "the append wrote outside its positions"
    # an entry that borrows another's cache rotates its queries and writes nothing
    kp2, vp2 = _paged(8, hkv, hd, dtype)
    q2 = orig.to(DEV).to(DT[dtype]).clone()
    K().rope_append(q2, cos.to(DEV), sin.to(DEV), torch.tensor(pos, dtype=torch.int32, device=DEV),
                    torch.tensor(seq, dtype=torch.int32, device=DEV), slots, pt, kp2, vp2, hq, hkv, hd, rot, inter, False)
    assert torch.isnan(kp2.float()).all() and torch.equal(q2[:, :hq * hd], qkv[:, :hq * hd])


# ------------------------------------------------------------------- attention
def _attention_case(dtype, hq, hkv, hd, seqs, window=0, n_splits=1, decode=False, special=None, dead_pages=False,
                    kernel="general"):
    """seqs: list of (kv length before the step, new tokens).  Builds pages in a scrambled order,
    runs the kernel, returns (out, reference)."""
    k = K()
    torch.manual_seed(hq * 1000 + hd + len(seqs))
    B = len(seqs)
    total = [s + n for s, n in seqs]
    max_pages = max((t + 63) // 64 for t in total) + 1
    n_pages = sum((t + 63) // 64 for t in total) + 3
    perm = torch.randperm(n_pages).tolist()
    kp, vp = _paged(n_pages, hkv, hd, dtype)
    pt = torch.full((B + 2, max_pages), -1, dtype=torch.int32)
    slots = [B + 1 - i for i in range(B)]                       # slots in falling order, not 0..B-1
    Ks, Vs, qs, pos, seq_of = [], [], [], [], []
    for i, (s, n) in enumerate(seqs):
        Kf = torch.randn(total[i], hkv, hd)
        Vf = torch.randn(total[i], hkv, hd)
        if special:
            special(i, Kf, Vf)
        Kf, Vf = Kf.to(DT[dtype]).float(), Vf.to(DT[dtype]).float()
        Ks.append(Kf); Vs.append(Vf)
        first_live = max(0, s - window + 1) // 64 if (window and dead_pages) else 0
        for pg in range((total[i] + 63) // 64):
            if pg < first_live:
                continue                                         # given back: the kernel may not touch it
            page = perm.pop()
            pt[slots[i], pg] = page
            lo, hi = pg * 64, min(total[i], pg * 64 + 64)
            kp[page, :, :hi - lo] = Kf[lo:hi].transpose(0, 1).to(DEV).to(DT[dtype])
            vp[page, :, :hi - lo] = Vf[lo:hi].transpose(0, 1).to(DEV).to(DT[dtype])
        for j in range(n):
            q = torch.randn(hq, hd)
            if special:
                special(i, None, None, q, s + j)
            qs.append(q.to(DT[dtype]).float()); pos.append(s + j); seq_of.append(i)
    T_ = len(qs)
    ld = hq * hd + 16                                            # a row stride wider than the heads
    qbuf = torch.zeros(T_, ld, dtype=DT[dtype], device=DEV)
    qbuf[:, :hq * hd] = torch.stack(qs).reshape(T_, hq * hd).to(DEV).to(DT[dtype])
    qt, gchunk = k.attention_tile_shape(hd, hq // hkv, decode)
    tiles, off = [], 0
    for i, (s, n) in enumerate(seqs):
        for b in range(0, n, qt):
            tiles.append((i, off + b, min(qt, n - b)))
        off += n
    out = torch.full((T_, hq * hd), float("nan"), dtype=DT[dtype], device=DEV)
    scratch = torch.full((max(1, k.attention_scratch_floats(T_, hq, hd, n_splits)),), float("nan"), device=DEV)
    if kernel == "prefill_tc":
        tl, off = [], 0
        for i, (s_, n) in enumerate(seqs):
            for b0 in range(0, n, 128):
                tl.append((i, off + b0, min(128, n - b0)))
            off += n
        k.attention_prefill_tc(qbuf, ld, T_, kp, vp, pt.to(DEV), torch.tensor(tl, dtype=torch.int32, device=DEV),
                               torch.tensor(slots, dtype=torch.int32, device=DEV),
                               torch.tensor(pos, dtype=torch.int32, device=DEV), out, hq, hkv, hd, 1.0 / math.sqrt(hd),
                               window)
        k.check_device_errors()
    elif kernel.startswith("decode_mma"):
        keys = int(kernel.rsplit("_", 1)[1])
        assert all(n == 1 for _, n in seqs) and k.attention_decode_mma_takes(DT[dtype], hd, 64, n_splits)
        for _ in range(2):
            out.fill_(float("nan"))
            k.attention_decode_mma(qbuf, ld, T_, kp, vp, pt.to(DEV), torch.tensor(slots, dtype=torch.int32, device=DEV),
                                   torch.tensor(pos, dtype=torch.int32, device=DEV), out, hq, hkv, hd,
                                   1.0 / math.sqrt(hd), window, n_splits, keys, scratch if n_splits > 8 else None)
    elif kernel == "decode":
        assert all(n == 1 for _, n in seqs) and k.attention_decode_takes(DT[dtype], hd, 64)
        # three ways to combine slices: a cluster (no scratch, up to 8 slices), the last slice (scratch and
        # counters), a second kernel (scratch only)
        cnt = torch.zeros(T_ * hkv * ((hq // hkv + 3) // 4), dtype=torch.int32, device=DEV)
        ways = [(scratch, cnt), (scratch, None)] + ([(None, None)] if n_splits <= 8 else [])
        results = []
        for sc_, cn_ in ways:
            for _ in range(2):      # twice: the counters must be left ready for the next call
                out.fill_(float("nan"))
                k.attention_decode(qbuf, ld, T_, kp, vp, pt.to(DEV), torch.tensor(slots, dtype=torch.int32, device=DEV),
                                   torch.tensor(pos, dtype=torch.int32, device=DEV), out, hq, hkv, hd,
                                   1.0 / math.sqrt(hd), window, n_splits, sc_, cn_)
            results.append(out.clone())
        assert int(cnt.abs().sum()) == 0
        for r_ in results[1:]:
            torch.testing.assert_close(r_.float(), results[0].float(), atol=1e-5 if dtype == "float32" else 1e-2, rtol=1e-2)
    else:
        k.attention(qbuf, ld, T_, kp, vp, pt.to(DEV), torch.tensor(tiles, dtype=torch.int32, device=DEV),
                    max(t[2] for t in tiles), torch.tensor(slots, dtype=torch.int32, device=DEV),
                    torch.tensor(pos, dtype=torch.int32, device=DEV), out, hq, hkv, hd, 1.0 / math.sqrt(hd), window,
                    n_splits, gchunk, scratch)
    ref = torch.zeros(T_, hq * hd)
    G = hq // hkv
    for r in range(T_):
        i, p = seq_of[r], pos[r]
        lo = max(0, p - window + 1) if window else 0
        for h in range(hq):
            sc = (Ks[i][lo:p + 1, h // G] @ qs[r][h]) * (1.0 / math.sqrt(hd))
            ref[r, h * hd:(h + 1) * hd] = P.softmax(sc) @ Vs[i][lo:p + 1, h // G]
    return out.float().cpu(), ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hq,hkv,hd", [(4, 2, 16), (3, 1, 32), (5, 5, 48), (8, 2, 64), (6, 3, 128), (2, 1, 256),
                                       (40, 1, 128)])
def test_attention_prompts_chunks_and_single_tokens_in_one_batch(dtype, hq, hkv, hd):
    out, ref = _attention_case(dtype, hq, hkv, hd, [(0, 70), (129, 1), (60, 9), (0, 1)])
    torch.testing.assert_close(out, ref, **(dict(atol=2e-5, rtol=1e-5) if dtype == "float32" else dict(atol=2e-2, rtol=2e-2)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kernel", ["general", "decode"])
@pytest.mark.parametrize("n_splits", [1, 2, 3, 7, 16])
def test_attention_decode_in_slices(dtype, n_splits, kernel):
    out, ref = _attention_case(dtype, 8, 2, 64, [(299, 1), (0, 1), (64, 1), (63, 1), (127, 1)], n_splits=n_splits,
                               decode=True, kernel=kernel)
    torch.testing.assert_close(out, ref, **(dict(atol=2e-5, rtol=1e-5) if dtype == "float32" else dict(atol=2e-2, rtol=2e-2)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kernel", ["general", "decode"])
@pytest.mark.parametrize("far", [0, 3, 63, 64, 448, 698, 699])
def test_attention_finds_one_far_key_among_hundreds(dtype, far, kernel):
    # one key lines up with the query and outweighs the other 699: the output is that key's value
    def special(i, Kf, Vf, q=None, p=None):
        if Kf is not None:
            Kf.mul_(0.05)
            Kf[far, :, 0] = 12.0
        else:
            q.mul_(0.05)
            q[:, 0] = 12.0
    for n_splits in (1, 5):
        out, ref = _attention_case(dtype, 4, 2, 64, [(699, 1)], n_splits=n_splits, decode=True, special=special,
                                   kernel=kernel)
        torch.testing.assert_close(out, ref, **(dict(atol=2e-5, rtol=1e-5) if dtype == "float32" else dict(atol=2e-2, rtol=2e-2)))
        assert float((out - ref).abs().max()) < 0.05 and float(ref.abs().max()) > 0.5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kernel", ["general", "decode"])
@pytest.mark.parametrize("where", ["first_inside", "last_outside"])
def test_attention_window_edge(dtype, where, kernel):
    # window 100 at position 300 keeps keys 201..300; a dominant key sits on either side of the edge
    edge = 201 if where == "first_inside" else 200

    def special(i, Kf, Vf, q=None, p=None):
        if Kf is not None:
            Kf.mul_(0.05)
            Kf[edge, :, 0] = 12.0
            Vf[edge] = 7.0
        else:
            q.mul_(0.05)
            q[:, 0] = 12.0
    for n_splits, dead in ((1, False), (3, True)):
        out, ref = _attention_case(dtype, 4, 2, 32, [(300, 1)], window=100, n_splits=n_splits, decode=True,
                                   special=special, dead_pages=dead, kernel=kernel)
        torch.testing.assert_close(out, ref, **(dict(atol=2e-5, rtol=1e-5) if dtype == "float32" else dict(atol=3e-2, rtol=2e-2)))
        if where == "first_inside":
            assert float((out - 7.0).abs().max()) < 0.1
        else:
            assert float(out.abs().max()) < 6.0
    # and for a prompt chunk whose queries straddle the window differently
    out, ref = _attention_case(dtype, 4, 2, 32, [(250, 60)], window=100, special=special, dead_pages=True)
    torch.testing.assert_close(out, ref, **(dict(atol=2e-5, rtol=1e-5) if dtype == "float32" else dict(atol=3e-2, rtol=2e-2)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hq,hkv,hd", [(4, 2, 16), (3, 1, 32), (8, 2, 64), (6, 3, 128), (2, 1, 256), (40, 2, 64),
                                       (5, 5, 48)])
def test_attention_decode_kernel_sizes(dtype, hq, hkv, hd):
    k = K()
    if not k.attention_decode_takes(DT[dtype], hd, 64):
        assert (hd, dtype) in ((48, "bfloat16"), (48, "float32"), (256, "float32"))
        return
    for n_splits in (1, 4):
        out, ref = _attention_case(dtype, hq, hkv, hd, [(500, 1), (0, 1), (65, 1)], n_splits=n_splits, decode=True,
                                   kernel="decode")
        torch.testing.assert_close(out, ref, **(dict(atol=2e-5, rtol=1e-5) if dtype == "float32" else dict(atol=2e-2, rtol=2e-2)))


@pytest.mark.parametrize("keys", [16, 32])
@pytest.mark.parametrize("hq,hkv,hd", [(8, 2, 64), (3, 1, 128), (4, 4, 64), (32, 8, 64), (24, 2, 128), (9, 1, 64)])
def test_attention_decode_on_the_tensor_cores(hq, hkv, hd, keys):
    # lengths around page and tile edges, a first token, several slices (clusters), more heads per
    # kv head than one block takes (12 and 9 > 8)
    for n_splits in (1, 2, 5, 8, 11):      # 2..8: a cluster; more: scratch and a second kernel
        out, ref = _attention_case("bfloat16", hq, hkv, hd, [(500, 1), (0, 1), (65, 1), (15, 1), (16, 1), (31, 1), (127, 1)],
                                   n_splits=n_splits, decode=True, kernel=f"decode_mma_{keys}")
        torch.testing.assert_close(out, ref, atol=2e-2, rtol=2e-2)
    assert not K().attention_decode_mma_takes(torch.bfloat16, 96, 64, 1)
    assert not K().attention_decode_mma_takes(torch.float32, 64, 64, 1)
    with pytest.raises(Exception):                               # more than 8 slices need scratch
        K().attention_decode_mma(torch.zeros(1, 64, dtype=torch.bfloat16, device=DEV), 64, 1,
                                 torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16, device=DEV),
                                 torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16, device=DEV),
                                 torch.zeros(1, 1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                                 torch.zeros(1, dtype=torch.int32, device=DEV),
                                 torch.zeros(1, 64, dtype=torch.bfloat16, device=DEV), 1, 1, 64, 0.125, 0, 9, 16, None)


@pytest.mark.parametrize("keys", [16, 32])
@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 500, 638, 639])
def test_attention_decode_mma_finds_one_far_key(far, keys):
    def special(i, Kf, Vf, q=None, p=None):
        if Kf is not None:
            Kf.mul_(0.05)
            Kf[far, :, 0] = 12.0
            Vf[far] = 7.0
        else:
            q.mul_(0.05)
            q[:, 0] = 12.0
    for n_splits in (1, 4):
        out, ref = _attention_case("bfloat16", 8, 2, 64, [(639, 1)], special=special, n_splits=n_splits, decode=True,
                                   kernel=f"decode_mma_{keys}")
        torch.testing.assert_close(out, ref, atol=3e-2, rtol=2e-2)
        assert float((out - 7.0).abs().max()) < 0.1


@pytest.mark.parametrize("where", ["first_inside", "last_outside"])
def test_attention_decode_mma_window_edge_and_dead_pages(where):
    edge = 201 if where == "first_inside" else 200

    def special(i, Kf, Vf, q=None, p=None):
        if Kf is not None:
            Kf.mul_(0.05)
            Kf[edge, :, 0] = 12.0
            Vf[edge] = 7.0
        else:
            q.mul_(0.05)
            q[:, 0] = 12.0
    for n_splits, dead in ((1, False), (3, True)):
        out, ref = _attention_case("bfloat16", 4, 2, 64, [(300, 1)], window=100, n_splits=n_splits, decode=True,
                                   special=special, dead_pages=dead, kernel="decode_mma_16")
        torch.testing.assert_close(out, ref, atol=3e-2, rtol=2e-2)
        if where == "first_inside":
            assert float((out - 7.0).abs().max()) < 0.1
        else:
            assert float(out.abs().max()) < 6.0


@pytest.mark.parametrize("hq,hkv,hd", [(8, 2, 64), (3, 1, 128), (4, 4, 64)])
@pytest.mark.parametrize("seqs", [[(0, 1)], [(0, 70)], [(0, 128)], [(0, 129)], [(0, 300), (0, 5)], [(60, 9), (129, 1), (0, 200)],
                                  [(200, 130)], [(0, 700)]])
def test_attention_prefill_on_the_tensor_cores(hq, hkv, hd, seqs):
    out, ref = _attention_case("bfloat16", hq, hkv, hd, seqs, kernel="prefill_tc")
    torch.testing.assert_close(out, ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("far", [0, 63, 64, 127, 128, 500, 639])
def test_attention_prefill_tc_finds_one_far_key(far):
    def special(i, Kf, Vf, q=None, p=None):
        if Kf is not None:
            Kf.mul_(0.05)
            Kf[far, :, 0] = 12.0
        else:
            q.mul_(0.05)
            q[:, 0] = 12.0
    out, ref = _attention_case("bfloat16", 4, 2, 64, [(0, 700)], special=special, kernel="prefill_tc")
    torch.testing.assert_close(out, ref, atol=3e-2, rtol=2e-2)
    assert float(ref[650].abs().max()) > 0.5


@pytest.mark.parametrize("hd", [64, 128])
def test_attention_prefill_tc_window_and_dead_pages(hd):
    def special(i, Kf, Vf, q=None, p=None):
        if Kf is not None:
            Kf.mul_(0.05)
            Kf[201, :, 0] = 12.0
            Vf[201] = 7.0
        else:
            q.mul_(0.05)
            q[:, 0] = 12.0
    out, ref = _attention_case("bfloat16", 4, 2, hd, [(250, 140)], window=100, special=special, dead_pages=True,
                               kernel="prefill_tc")
    torch.testing.assert_close(out, ref, atol=3e-2, rtol=2e-2)


def test_attention_refuses_sizes_it_does_not_take():
    k = K()
    z = torch.zeros(1, 8, device=DEV)
    i = torch.zeros(1, 3, dtype=torch.int32, device=DEV)
    pages = torch.zeros(1, 1, 64, 6, device=DEV)
    with pytest.raises(k.KernelError, match="size"):
        k.attention(z, 8, 1, pages, pages, i, i, 1, i[0], i[0], torch.zeros(1, 6, device=DEV), 1, 1, 6, 1.0)
    pages = torch.zeros(1, 1, 64, 512, device=DEV)
    with pytest.raises(k.KernelError, match="size"):
        k.attention(torch.zeros(1, 512, device=DEV), 512, 1, pages, pages, i, i, 1, i[0], i[0],
                    torch.zeros(1, 512, device=DEV), 1, 1, 512, 1.0)


# -------------------------------------------------------------------- sampling
@pytest.mark.parametrize("V", [5, 384, 1000, 128256])
def test_argmax_first_maximum_wins(V):
    lg = torch.randn(6, V, device=DEV)
    lg[1, V // 2] = 50.0
    lg[2, [0, V - 1]] = 60.0                    # a tie: the smaller index
    lg[3, V - 1] = 70.0
    lg[4] = -float("inf")
    lg[5] = 3.0
    got = K().argmax(lg).cpu().tolist()
    want = [P.argmax(lg[r].cpu()) if V <= 1000 else int(lg[r].argmax()) for r in range(6)]
    want[2], want[4], want[5] = 0, 0, 0
    assert got == want


def test_uniform_matches_the_plain_philox():
    draws = torch.tensor([0, 1, 2, 500, 0], dtype=torch.int32, device=DEV)
    reqs = torch.tensor([0, 0, 7, 3, 65000], dtype=torch.int32, device=DEV)
    for seed in (0, 7, 2 ** 40 + 5):
        got = K().uniform(seed, draws, reqs).cpu().tolist()
        want = [P.philox_uniform(seed, int(d), int(r)) for d, r in zip(draws.tolist(), reqs.tolist())]
        assert got == want


@pytest.mark.parametrize("V", [7, 384, 5000, 16384, 20000, 128256])
def test_sample_is_the_inverse_cdf_of_the_softmax(V):
    torch.manual_seed(V)
    R = 64
    lg = torch.randn(R, V, device=DEV) * 3
    lg[:, V // 3] = -float("inf")                                # a filtered token can never be drawn
    temps = torch.full((R,), 0.8, device=DEV)
    reqs = torch.arange(R, dtype=torch.int32, device=DEV)
    draws = torch.full((R,), 5, dtype=torch.int32, device=DEV)
    got = K().sample(lg, temps, reqs, draws, 11).cpu().tolist()
    assert got == K().sample(lg, temps, reqs, draws, 11).cpu().tolist()
    p = torch.softmax(lg.double().cpu() / 0.8, dim=1)
    c = torch.cumsum(p, dim=1)
    for r in range(R):
        u = P.philox_uniform(11, 5, r)
        t = got[r]
        assert t != V // 3 and p[r, t] > 0
        lo = float(c[r, t - 1]) if t > 0 else 0.0
        assert lo - 1e-5 <= u <= float(c[r, t]) + 1e-5, f"row {r}: u={u} outside [{lo}, {float(c[r, t])}]"
    one = torch.full((2, V), -float("inf"), device=DEV)
    one[:, V - 1] = 0.0
    assert K().sample(one, temps[:2], reqs[:2], draws[:2], 3).cpu().tolist() == [V - 1, V - 1]


def test_sample_frequencies_follow_the_probabilities():
    probs = torch.tensor([0.5, 0.25, 0.125, 0.125])
    n = 4000
    lg = torch.log(probs).to(DEV).repeat(n, 1)
    got = K().sample(lg, torch.ones(n, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
                     torch.arange(n, dtype=torch.int32, device=DEV), 1)
    freq = torch.bincount(got.cpu().long(), minlength=4).float() / n
    assert float((freq - probs).abs().max()) < 0.03


@pytest.mark.parametrize("V,k,p,mp,pen,temp", [(50, 5, 0.9, 0.0, 1.1, 0.7), (1000, 40, 0.9, 0.0, 1.1, 0.7),
                                               (1000, 999, 0.5, 0.05, 1.0, 1.3), (777, 1, 1.0, 0.0, 2.0, 0.5),
                                               (5000, 300, 0.95, 0.01, 1.5, 1.0), (128256, 40, 0.9, 0.02, 1.1, 0.7),
                                               (4099, 64, 1.0, 0.1, 1.0, 2.0), (301, 300, 0.3, 0.0, 1.2, 0.9),
                                               (1000, 0, 0.8, 0.0, 1.0, 1.0), (5000, 0, 0.5, 0.02, 1.3, 0.7),
                                               (128256, 0, 0.9, 0.0, 1.1, 0.7), (640, 0, 1.0, 0.2, 1.0, 1.5)])
def test_filter_kernel_against_the_plain_filters(V, k, p, mp, pen, temp):
    g = torch.Generator().manual_seed(V + k)
    R = 4
    lg = torch.randn(R, V, generator=g) * 3.0
    lg[1, : min(V, 20)] = 7.5                                   # a block of ties at the top of row 1
    recent = [torch.randint(0, V, (n,), generator=g).tolist() for n in (64, 10, 0, 33)]
    recent[0][5] = recent[0][4]                                 # a repeated token counts once
    width = 64
    rec = torch.tensor([(r + [-1] * width)[:width] for r in recent], dtype=torch.int32, device=DEV)
    pad = torch.full((R, V + 3), 99.0)                          # a row stride that is not the width
    pad[:, :V] = lg
    got = K().filter_logits(pad.to(DEV)[:, :V], temp, k, p, mp, pen, rec).cpu()
    for r in range(R):
        want = P.filter_logits(lg[r], recent[r], pen, temp, k, p, mp)
        kept_w, kept_g = torch.isfinite(want), torch.isfinite(got[r])
        if not torch.equal(kept_w, kept_g):
            # the two may differ only on values that tie with the last kept one (the order among
            # equal probabilities is the sort's, in the reference too) or where the running sum
            # meets p within rounding
            diff = (kept_w != kept_g).nonzero().flatten().tolist()
            edge = want[kept_w].min()
            sm = P.softmax(torch.where(kept_w | kept_g, got[r].nan_to_num(neginf=-1e30), torch.tensor(-1e30)))
            cum_w = float(sm[kept_w].sum())
            for i in diff:
                v = got[r, i] if kept_g[i] else want[i]
                assert abs(float(v - edge)) < 1e-5 or abs(cum_w - p) < 1e-4, (r, i, float(v), float(edge))
        both = kept_w & kept_g
        assert both.any()
        torch.testing.assert_close(got[r][both], want[both], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("V,k,p,mp,pen,temp", [(50, 5, 0.9, 0.0, 1.1, 0.7), (1000, 40, 0.9, 0.0, 1.1, 0.7),
                                               (777, 1, 1.0, 0.0, 2.0, 0.5), (5000, 200, 0.95, 0.01, 1.5, 1.0),
                                               (128256, 40, 0.9, 0.02, 1.1, 0.7), (4099, 64, 1.0, 0.1, 1.0, 2.0),
                                               (128256, 128, 0.5, 0.0, 1.0, 1.3), (20000, 3, 1.0, 0.0, 1.0, 1.0)])
def test_filters_and_draw_from_the_top_k_candidates(V, k, p, mp, pen, temp):
    """The fused path for a small top-k (candidates per chunk of the vocabulary, then one block per row)
    against the plain filters and the plain inverse CDF, and against the two separate kernels."""
    kk = K()
    assert kk.filter_draw_chunks(V, k) == (V + 8191) // 8192
    g = torch.Generator().manual_seed(V + k)
    R = 6
    lg = torch.randn(R, V, generator=g) * 3.0
    lg[1, : min(V, 20)] = 7.5                                   # a block of ties at the top of row 1
    lg[2, V // 2] = -float("inf")
    recent = [torch.randint(0, V, (n,), generator=g).tolist() for n in (64, 10, 0, 33, 64, 1)]
    recent[0][5] = recent[0][4]                                 # a repeated token counts once
    rec = torch.tensor([(r + [-1] * 64)[:64] for r in recent], dtype=torch.int32, device=DEV)
    pad = torch.full((R, V + 3), 99.0)                          # a row stride that is not the width
    pad[:, :V] = lg
    dev_lg = pad.to(DEV)[:, :V]
    reqs = torch.tensor([0, 3, 1, 70000, 5, 2], dtype=torch.int32, device=DEV)
    kept, cdf = [], []
    for r in range(R):
        want = P.filter_logits(lg[r], recent[r], pen, temp, k, p, mp)
        kept.append(torch.isfinite(want))
        cdf.append(torch.cumsum(torch.softmax(want.double(), dim=0), dim=0))
    same = total = 0
    for d in range(12):
        draws = torch.full((R,), d, dtype=torch.int32, device=DEV)
        got = kk.filter_draw(dev_lg, temp, k, p, mp, pen, rec, reqs, draws, 9).cpu().tolist()
        assert got == kk.filter_draw(dev_lg, temp, k, p, mp, pen, rec, reqs, draws, 9).cpu().tolist()
        work = kk.filter_logits(dev_lg, temp, k, p, mp, pen, rec)
        old = kk.sample(work, torch.ones(R, device=DEV), reqs, draws, 9).cpu().tolist()
        for r in range(R):
            t, u = got[r], P.philox_uniform(9, d, int(reqs[r]))
            total += 1
            same += t == old[r]
            if not kept[r][t]:
                # only a value that ties with the last kept one, or a prefix that meets p within rounding
                w = work[r].cpu()
                assert torch.isfinite(w[t]) and abs(float(w[t] - w[torch.isfinite(w)].min())) < 1e-5, (r, d, t)
                continue
            lo = float(cdf[r][t - 1]) if t > 0 else 0.0
            assert lo - 2e-5 <= u <= float(cdf[r][t]) + 2e-5, f"row {r} draw {d}: u={u} outside [{lo}, {float(cdf[r][t])}]"
    assert same >= total - 2, (same, total)                     # (sums in another order: a draw on an edge may differ)


def test_filters_and_draw_fall_back_when_ties_overflow_the_candidate_lists():
    # every logit equal: top-k keeps the whole vocabulary (ties at the cutoff stay), far more than the lists
    # hold; such a row goes through the whole-row filters and draw, the other rows do not notice
    kk = K()
    V, R = 128256, 3
    lg = torch.randn(R, V, device=DEV) * 2.0
    lg[1] = 0.25
    reqs = torch.arange(R, dtype=torch.int32, device=DEV)
    seen = set()
    for d in range(6):
        draws = torch.full((R,), d, dtype=torch.int32, device=DEV)
        got = kk.filter_draw(lg, 0.7, 40, 0.9, 0.0, 1.0, None, reqs, draws, 3).cpu().tolist()
        work = kk.filter_logits(lg, 0.7, 40, 0.9, 0.0, 1.0, None)
        old = kk.sample(work, torch.ones(R, device=DEV), reqs, draws, 3).cpu().tolist()
        assert got[1] == old[1]
        u = P.philox_uniform(3, d, 1)
        assert abs(got[1] - u * V) <= 2                          # uniform over the vocabulary, in index order
        seen.add(got[1])
        assert got[0] == old[0] and got[2] == old[2]
    assert len(seen) == 6
    assert kk.filter_draw_chunks(V, 0) == 0 and kk.filter_draw_chunks(V, 257) == 0 and kk.filter_draw_chunks(300, 300) == 0
    with pytest.raises(kk.KernelError):
        kk.filter_draw(lg, 0.7, 0, 0.9, 0.0, 1.0, None, reqs, reqs, 3)


def test_filtered_sampling_stays_inside_the_kept_set():
    from dlgo_b200.sampling import DeviceSampler, SamplerConfig
    g = torch.Generator().manual_seed(4)
    V, R = 3000, 6
    lg = (torch.randn(R, V, generator=g) * 2.0).to(DEV)
    cfg = SamplerConfig(temperature=0.8, top_k=7, top_p=0.95, min_p=0.0, repetition_penalty=1.3)
    recent = [torch.randint(0, V, (20,), generator=g).tolist() for _ in range(R)]
    s = DeviceSampler(seed=5)
    seen = [set() for _ in range(R)]
    for d in range(40):
        got = s.sample(lg, cfg, list(range(R)), [d] * R, recent).cpu().tolist()
        for r in range(R):
            seen[r].add(got[r])
    for r in range(R):
        want = P.filter_logits(lg[r].cpu(), recent[r], 1.3, 0.8, 7, 0.95, 0.0)
        kept = set(torch.isfinite(want).nonzero().flatten().tolist())
        assert seen[r] <= kept and len(seen[r]) > 1
    # the same (seed, request, draw) gives the same token whatever else is in the batch
    a = s.sample(lg, cfg, list(range(R)), [3] * R, recent).cpu().tolist()
    b = s.sample(lg[2:4], cfg, [2, 3], [3, 3], recent[2:4]).cpu().tolist()
    assert a[2:4] == b


# ------------------------------------------------------- tensor-core contraction
def _tc_ref(a, b):
    return a.double() @ b.double().t()


@pytest.mark.parametrize("Ra,Rb,K_,bn", [(128, 16, 64, 16), (128, 256, 64, 256), (300, 7, 200, 16), (77, 40, 96, 64),
                                         (256, 130, 2048, 128), (1000, 33, 264, 64), (130, 600, 328, 256)])
def test_gemm_tc_all_epilogues_both_orientations(Ra, Rb, K_, bn):
    k = K()
    torch.manual_seed(Ra + Rb)
    a = torch.randn(Ra, K_, device=DEV).to(torch.bfloat16)
    b = torch.randn(Rb, K_, device=DEV).to(torch.bfloat16)
    ref = _tc_ref(a, b).float()
    t = dict(atol=2e-3 * math.sqrt(K_), rtol=1e-2)
    for transposed in (False, True):
        want = ref.t() if transposed else ref
        shape = (Rb, Ra) if transposed else (Ra, Rb)
        o = torch.full(shape, float("nan"), device=DEV)
        k.gemm_tc(a, b, o, transposed, k.TC_STORE_F32, bn)
        torch.testing.assert_close(o, want, atol=1e-4 * math.sqrt(K_), rtol=1e-5)
        ob = torch.full(shape, float("nan"), device=DEV, dtype=torch.bfloat16)
        k.gemm_tc(a, b, ob, transposed, k.TC_STORE, bn)
        torch.testing.assert_close(ob.float(), want, **t)
        res = torch.randn(shape, device=DEV)
        acc = res.clone()
        k.gemm_tc(a, b, acc, transposed, k.TC_ADD_F32, bn)
        torch.testing.assert_close(acc, res + want, atol=1e-4 * math.sqrt(K_), rtol=1e-5)
    k.check_device_errors()


@pytest.mark.parametrize("Ra,Rb,K_,bn,epi", [(2100, 2600, 200, 256, "store"), (1300, 5000, 328, 128, "add"),
                                             (700, 9000, 72, 256, "f32")])
def test_gemm_tc_persistent_over_many_tiles(Ra, Rb, K_, bn, epi):
    # more tiles than SMs: every CTA walks several tiles with its two accumulators in turn
    k = K()
    torch.manual_seed(Ra)
    a = torch.randn(Ra, K_, device=DEV).to(torch.bfloat16)
    b = torch.randn(Rb, K_, device=DEV).to(torch.bfloat16)
    ref = _tc_ref(a, b).float()
    if epi == "store":
        o = torch.full((Ra, Rb), float("nan"), device=DEV, dtype=torch.bfloat16)
        k.gemm_tc(a, b, o, False, k.TC_STORE, bn, static_operand=2)
        torch.testing.assert_close(o.float(), ref, atol=2e-3 * math.sqrt(K_), rtol=1e-2)
    elif epi == "add":
        res = torch.randn(Ra, Rb, device=DEV)
        o = res.clone()
        k.gemm_tc(a, b, o, False, k.TC_ADD_F32, bn)
        torch.testing.assert_close(o, res + ref, atol=1e-4 * math.sqrt(K_), rtol=1e-5)
    else:
        o = torch.full((Ra, Rb), float("nan"), device=DEV)
        k.gemm_tc(a, b, o, False, k.TC_STORE_F32, bn)
        torch.testing.assert_close(o, ref, atol=1e-4 * math.sqrt(K_), rtol=1e-5)
    k.check_device_errors()


@pytest.mark.parametrize("Ra,Rb,K_,tile,epi", [(256, 256, 64, 256, "f32"), (300, 700, 200, 256, "store"),
                                               (2100, 2600, 328, 256, "add"), (1000, 5000, 72, 128, "f32"),
                                               (4000, 4200, 520, 256, "store")])
def test_gemm_tc_cta_pairs(Ra, Rb, K_, tile, epi):
    # 256 x tile tiles computed by pairs of CTAs (cta_group::2), persistent over many tiles
    k = K()
    torch.manual_seed(Ra + tile)
    a = torch.randn(Ra, K_, device=DEV).to(torch.bfloat16)
    b = torch.randn(Rb, K_, device=DEV).to(torch.bfloat16)
    ref = _tc_ref(a, b).float()
    if epi == "store":
        o = torch.full((Ra, Rb), float("nan"), device=DEV, dtype=torch.bfloat16)
        k.gemm_tc(a, b, o, False, k.TC_STORE, 256, pair_tile=tile)
        torch.testing.assert_close(o.float(), ref, atol=2e-3 * math.sqrt(K_), rtol=1e-2)
    elif epi == "add":
        res = torch.randn(Ra, Rb, device=DEV)
        o = res.clone()
        k.gemm_tc(a, b, o, False, k.TC_ADD_F32, 256, pair_tile=tile)
        torch.testing.assert_close(o, res + ref, atol=1e-4 * math.sqrt(K_), rtol=1e-5)
    else:
        o = torch.full((Ra, Rb), float("nan"), device=DEV)
        k.gemm_tc(a, b, o, False, k.TC_STORE_F32, 256, pair_tile=tile)
        torch.testing.assert_close(o, ref, atol=1e-4 * math.sqrt(K_), rtol=1e-5)
    k.check_device_errors()


@pytest.mark.parametrize("N,T_,K_,splits", [(256, 5, 512, 2), (384, 16, 2048, 8), (130, 33, 200, 4), (2048, 64, 8192, 9),
                                            (128, 1, 640, 10)])
def test_gemm_tc_split_k_is_exact_and_repeatable(N, T_, K_, splits):
    k = K()
    torch.manual_seed(N + T_)
    w = torch.randn(N, K_, device=DEV).to(torch.bfloat16)
    x = torch.randn(T_, K_, device=DEV).to(torch.bfloat16)
    bn = 16 if T_ <= 16 else (32 if T_ <= 32 else 64)
    ws = torch.full((k.gemm_tc_workspace_floats(N, T_, bn, splits),), float("nan"), device=DEV)
    cnt = torch.zeros(64, dtype=torch.int32, device=DEV)
    ref = _tc_ref(x, w).float()
    outs = []
    for _ in range(3):
        o = torch.full((T_, N), float("nan"), device=DEV)
        k.gemm_tc(w, x, o, True, k.TC_STORE_F32, bn, splits, ws, cnt)
        outs.append(o)
    torch.testing.assert_close(outs[0], ref, atol=1e-4 * math.sqrt(K_), rtol=1e-5)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    assert int(cnt.abs().sum()) == 0
    res = torch.randn(T_, N, device=DEV)
    acc = res.clone()
    k.gemm_tc(w, x, acc, True, k.TC_ADD_F32, bn, splits, ws, cnt)
    torch.testing.assert_close(acc, res + ref, atol=1e-4 * math.sqrt(K_), rtol=1e-5)
    k.check_device_errors()


@pytest.mark.parametrize("N,T_,K_,splits", [(384, 8, 2048, 8), (130, 13, 200, 3), (2048, 40, 8192, 9), (128, 1, 640, 10)])
def test_gemm_tc_k_slices_add_themselves_into_the_residual(N, T_, K_, splits):
    """Every K-slice adds its tile into the fp32 target with reductions at the memory: the sum of all, in
    an order that is not fixed (so compared with a tolerance of fp32 rounding, not bit for bit)."""
    k = K()
    g = torch.Generator().manual_seed(N + T_)
    w = torch.randn(N, K_, generator=g).to(torch.bfloat16).to(DEV)
    x = torch.randn(T_, K_, generator=g).to(torch.bfloat16).to(DEV)
    bn = 16 if T_ <= 16 else (32 if T_ <= 32 else 64)
    ref = _tc_ref(x, w).float()
    res = torch.randn(T_, N, generator=g).to(DEV)
    acc = res.clone()
    k.gemm_tc(w, x, acc, True, k.TC_RED_F32, bn, splits, static_operand=1)
    torch.testing.assert_close(acc, res + ref, atol=1e-4 * math.sqrt(K_), rtol=1e-5)
    k.check_device_errors()


@pytest.mark.parametrize("T_", [3, 40, 200])
def test_gemm_tc_swiglu_epilogue(T_):
    k = K()
    F_, d = 112, 72
    torch.manual_seed(T_)
    gate = torch.randn(F_, d, device=DEV).to(torch.bfloat16)
    up = torch.randn(F_, d, device=DEV).to(torch.bfloat16)
    x = (torch.randn(T_, d, device=DEV) * 0.3).to(torch.bfloat16)
    inter = torch.stack([gate.view(F_ // 16, 16, d), up.view(F_ // 16, 16, d)], dim=1).reshape(2 * F_, d).contiguous()
    ref = P.swiglu((x.double() @ gate.double().t()).float().cpu(), (x.double() @ up.double().t()).float().cpu())
    h = torch.full((T_, F_), float("nan"), device=DEV, dtype=torch.bfloat16)
    if T_ <= 64:
        bn = 16 if T_ <= 16 else 64
        k.gemm_tc(inter, x, h, True, k.TC_SWIGLU, bn)
    else:
        k.gemm_tc(x, inter, h, False, k.TC_SWIGLU, 256)
    torch.testing.assert_close(h.float().cpu(), ref, atol=3e-2, rtol=2e-2)
    k.check_device_errors()


def test_gemm_tc_refuses_what_it_cannot_take():
    k = K()
    a = torch.zeros(128, 60, device=DEV, dtype=torch.bfloat16)     # K not a multiple of 8
    o = torch.zeros(128, 128, device=DEV)
    with pytest.raises(k.KernelError, match="size"):
        k.gemm_tc(a, a, o, False, k.TC_STORE_F32, 128)
    b = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(k.KernelError, match="size"):
        k.gemm_tc(b, b, o, False, k.TC_STORE_F32, 48)               # not a tile width
    ws, cnt = torch.zeros(1 << 16, device=DEV), torch.zeros(4, dtype=torch.int32, device=DEV)
    with pytest.raises(k.KernelError, match="size"):
        k.gemm_tc(b, b, o, False, k.TC_STORE_F32, 128, 2, ws, cnt)  # more K-slices than K blocks
    with pytest.raises(k.KernelError, match="workspace"):
        k.gemm_tc(b, b, o, False, k.TC_STORE_F32, 128, 2)           # K-slices without their workspace


# ------------------------------------------------ partial sums handed to the next kernel
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("S,d", [(1, 50), (3, 200), (8, 2048), (9, 96), (18, 4096), (5, 1028), (17, 3000), (2, 1024)])
def test_add_rmsnorm_settles_partials_in_order(dtype, S, d):
    k = K()
    torch.manual_seed(S * d)
    x = torch.randn(6, d, device=DEV)
    parts = torch.randn(S, 6, d, device=DEV)
    w = 1 + 0.1 * torch.randn(d, device=DEV)
    want = x.clone()
    for s_ in range(S):
        want = want + parts[s_]
    ref = P.rmsnorm(want.cpu(), w.cpu(), 1e-5)
    x1 = x.clone()
    out = k.add_rmsnorm(x1, parts, w, 1e-5, DT[dtype])
    assert torch.equal(x1, want)                                  # slices added in order: bit for bit
    torch.testing.assert_close(out.float().cpu(), ref, **tol(dtype))
    x2 = x.clone()
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    out2 = k.add_rmsnorm(x2, parts, w, 1e-5, DT[dtype], rows)
    torch.testing.assert_close(out2.float().cpu(), ref[[4, 1]], **tol(dtype))
    assert torch.equal(x2[[4, 1]], want[[4, 1]]) and torch.equal(x2[[0, 2, 3, 5]], x[[0, 2, 3, 5]])
    x3 = x.clone()
    assert k.add_rmsnorm(x3, parts, None, 0.0, None) is None and torch.equal(x3, want)


@pytest.mark.parametrize("N,T_,K_,splits,bn", [(256, 5, 512, 2, 16), (384, 16, 2048, 8, 16), (130, 33, 200, 4, 64),
                                               (128, 1, 640, 1, 16)])
def test_gemm_tc_leaves_partials_for_the_next_kernel(N, T_, K_, splits, bn):
    k = K()
    torch.manual_seed(N + T_)
    w = torch.randn(N, K_, device=DEV).to(torch.bfloat16)
    x = torch.randn(T_, K_, device=DEV).to(torch.bfloat16)
    parts = torch.full((splits, T_, N), float("nan"), device=DEV)
    k.gemm_tc(w, x, parts, True, k.TC_PARTIAL, bn, splits)
    torch.testing.assert_close(parts.sum(0), (x.double() @ w.double().t()).float(), atol=1e-4 * math.sqrt(K_), rtol=1e-5)
    k.check_device_errors()


def test_rope_append_from_partials():
    from dlgo_b200.parts.rope import RotaryEmbedding
    k = K()
    hq, hkv, hd = 4, 2, 32
    pe = RotaryEmbedding(hd, hd, 10000.0, 200)
    cos, sin = (t.to(DEV) for t in pe.tables())
    ld = (hq + 2 * hkv) * hd
    torch.manual_seed(0)
    parts = torch.randn(3, 2, ld, device=DEV)
    whole = (parts[0] + parts[1] + parts[2])
    pos = torch.tensor([5, 70], dtype=torch.int32, device=DEV)
    seq = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    pt = torch.tensor([[0, -1], [1, 2]], dtype=torch.int32, device=DEV)
    res = []
    for use_parts in (False, True):
        kp, vp = _paged(3, hkv, hd, "float32")
        qkv = whole.clone() if not use_parts else torch.full((2, ld), float("nan"), device=DEV)
        k.rope_append(qkv, cos, sin, pos, seq, slots, pt, kp, vp, hq, hkv, hd, hd, False, True, parts if use_parts else None)
        res.append((qkv[:, :hq * hd].clone(), kp.clone(), vp.clone()))
    # (the two paths are different kernels and may contract x0*c - x1*s differently: one ulp)
    torch.testing.assert_close(res[1][0], res[0][0], atol=1e-6, rtol=1e-6)
    for a, b in zip(res[0][1:], res[1][1:]):
        torch.testing.assert_close(torch.nan_to_num(b, nan=-7.0), torch.nan_to_num(a, nan=-7.0), atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("write_cache", [True, False])
def test_rope_append_from_a_sum_that_it_leaves_zero(write_cache):
    """The projection's K-slices may have added themselves into one fp32 sum: the rotation reads it once
    and leaves zeros behind, also where it has nothing to write (an entry that borrows another's cache)."""
    from dlgo_b200.parts.rope import RotaryEmbedding
    k = K()
    hq, hkv, hd = 5, 2, 48
    pe = RotaryEmbedding(hd, 32, 10000.0, 200)
    cos, sin = (t.to(DEV) for t in pe.tables())
    ld = (hq + 2 * hkv) * hd
    torch.manual_seed(1)
    whole = torch.randn(3, ld, device=DEV)
    pos = torch.tensor([5, 70, 127], dtype=torch.int32, device=DEV)
    seq = torch.tensor([0, 1, 1], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    pt = torch.tensor([[0, -1], [1, 2]], dtype=torch.int32, device=DEV)
    kp0, vp0 = _paged(3, hkv, hd, "bfloat16")
    q0 = whole.to(torch.bfloat16)
    k.rope_append(q0, cos, sin, pos, seq, slots, pt, kp0, vp0, hq, hkv, hd, 32, False, write_cache)
    kp1, vp1 = _paged(3, hkv, hd, "bfloat16")
    q1 = torch.full((3, ld), float("nan"), device=DEV, dtype=torch.bfloat16)
    total = whole.clone().view(1, 3, ld)
    k.rope_append(q1, cos, sin, pos, seq, slots, pt, kp1, vp1, hq, hkv, hd, 32, False, write_cache, total, True)
    assert int((total != 0).sum()) == 0, "the sum was not left zero"
    # (the plain path rounds the projection to bfloat16 before it rotates, this one after: one rounding apart)
    torch.testing.assert_close(q1[:, :hq * hd].float(), q0[:, :hq * hd].float(), atol=4e-2, rtol=2e-2)
    for a, b in ((kp0, kp1), (vp0, vp1)):
        assert torch.equal(torch.isnan(a.float()), torch.isnan(b.float()))
        torch.testing.assert_close(torch.nan_to_num(b.float(), nan=-7.0), torch.nan_to_num(a.float(), nan=-7.0),
                                   atol=4e-2, rtol=2e-2)
    with pytest.raises(k.KernelError):      # two slices are not a sum
        k.rope_append(q1, cos, sin, pos, seq, slots, pt, kp1, vp1, hq, hkv, hd, 32, False, True,
                      torch.zeros(2, 3, ld, device=DEV), True)


@pytest.mark.parametrize("hq,hkv,hd,d", [(8, 2, 64, 256), (32, 8, 64, 2048), (3, 1, 128, 384), (24, 8, 128, 512),
                                         (2, 1, 64, 200)])
@pytest.mark.parametrize("pair", [256, 0])
@pytest.mark.parametrize("write_cache", [True, False])
def test_qkv_projection_that_rotates_and_appends_in_its_epilogue(hq, hkv, hd, d, pair, write_cache):
    """Prompt tokens of three sequences (positions across page edges, pages in a scrambled order) through the
    q|k|v projection whose epilogue rotates q and k and appends k and v, against the product in float32 followed
    by the plain rotation; rows of pages that no token of the step owns stay untouched."""
    from dlgo_b200.parts.rope import RotaryEmbedding
    k = K()
    n_cols = (hq + 2 * hkv) * hd
    assert k.gemm_tc_rope_takes(n_cols, d, hq, hkv, hd, 64) and not k.gemm_tc_rope_takes(n_cols, d, hq, hkv, 96, 64)
    assert not k.gemm_tc_rope_takes(n_cols, d, hq, hkv, hd, 32) and not k.gemm_tc_rope_takes(n_cols + hd, d, hq, hkv, hd, 64)
    torch.manual_seed(hq + hd + d)
    cos, sin = (t.to(DEV) for t in RotaryEmbedding(hd, hd, 10000.0, 600, "split_half").tables())
    seqs = [(0, 70), (120, 141), (63, 2)]                          # (positions already held, new tokens)
    T_ = sum(n for _, n in seqs)
    pages_per = [(s + n + 63) // 64 for s, n in seqs]
    n_pages = sum(pages_per) + 2
    perm = torch.randperm(n_pages).tolist()
    pt = torch.full((len(seqs) + 1, max(pages_per)), -1, dtype=torch.int32)
    slots = [2, 0, 3]
    for i, n in enumerate(pages_per):
        for pg in range(n):
            pt[slots[i], pg] = perm.pop()
    pos = torch.tensor([s + j for s, n in seqs for j in range(n)], dtype=torch.int32, device=DEV)
    seq = torch.tensor([i for i, (s, n) in enumerate(seqs) for _ in range(n)], dtype=torch.int32, device=DEV)
    x = (torch.randn(T_, d, device=DEV) * 0.5).to(torch.bfloat16)
    w = (torch.randn(n_cols, d, device=DEV) * d ** -0.5).to(torch.bfloat16)
    kp = torch.full((n_pages, hkv, 64, hd), 55.0, device=DEV, dtype=torch.bfloat16)
    vp = torch.full((n_pages, hkv, 64, hd), 55.0, device=DEV, dtype=torch.bfloat16)
    qkv = torch.full((T_, n_cols), 33.0, device=DEV, dtype=torch.bfloat16)
    rope = k.rope_args(cos, sin, pos, seq, torch.tensor(slots, dtype=torch.int32, device=DEV), pt.to(DEV), kp, vp,
                       hq, hkv, hd, write_cache)
    k.gemm_tc_rope(x, w, qkv, pair, rope)
    k.check_device_errors()
    ref = (x.float().cpu() @ w.float().cpu().t()).view(T_, hq + 2 * hkv, hd)
    freqs = P.rope_frequencies(hd, 10000.0, None)
    rot = torch.stack([torch.stack([P.rope(ref[t, h], int(pos[t]), freqs) for h in range(hq + hkv)]) for t in range(T_)])
    got = qkv.float().cpu().view(T_, hq + 2 * hkv, hd)
    torch.testing.assert_close(got[:, :hq], rot[:, :hq], atol=2e-2, rtol=2e-2)
    assert float((got[:, hq:] - 33.0).abs().max()) == 0.0         # the k and v columns are not written
    written = torch.zeros(n_pages, 64, dtype=torch.bool)
    kc, vc = kp.float().cpu(), vp.float().cpu()
    for t in range(T_):
        i, p_ = int(seq[t]), int(pos[t])
        page = int(pt[slots[i], p_ // 64])
        written[page, p_ % 64] = True
        if write_cache:
            torch.testing.assert_close(kc[page, :, p_ % 64], rot[t, hq:], atol=2e-2, rtol=2e-2)
            torch.testing.assert_close(vc[page, :, p_ % 64], ref[t, hq + hkv:], atol=1e-2, rtol=1e-2)   # (rounded to bfloat16)
    untouched = ~written if write_cache else torch.ones_like(written)
    assert float((kc.transpose(1, 2)[untouched] - 55.0).abs().max()) == 0.0
    assert float((vc.transpose(1, 2)[untouched] - 55.0).abs().max()) == 0.0


@pytest.mark.parametrize("hq,hkv,hd,S", [(8, 2, 64, 3), (32, 8, 64, 6), (3, 1, 128, 8), (8, 1, 64, 11), (12, 4, 128, 1)])
@pytest.mark.parametrize("keys", [16, 32])
def test_tensor_core_decode_attention_with_the_rotation_and_append_inside(hq, hkv, hd, S, keys):
    # the kernel fed with the projection's unsummed slices against rope_append followed by the same
    # kernel fed with the finished q: same outputs, same rows appended to the cache
    from dlgo_b200.parts.rope import RotaryEmbedding
    k = K()
    assert k.attention_decode_mma_fuses_rope(hq, hkv, hd, hd, False)
    assert not k.attention_decode_mma_fuses_rope(hq, hkv, hd, hd // 2, False)
    assert not k.attention_decode_mma_fuses_rope(hq, hkv, hd, hd, True)
    torch.manual_seed(hd + S)
    cos, sin = (t.to(DEV) for t in RotaryEmbedding(hd, hd, 10000.0, 700, "split_half").tables())
    lens = [300, 1, 64, 65, 640]                                  # positions 299, 0, 63 (page end), 64 (page start), 639
    B = len(lens)
    pages_per = [(n + 63) // 64 for n in lens]
    n_pages = sum(pages_per) + 1
    perm = torch.randperm(n_pages).tolist()
    pt = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
    for i, n in enumerate(pages_per):
        for pg in range(n):
            pt[i, pg] = perm.pop()
    pt = pt.to(DEV)
    ld = (hq + 2 * hkv) * hd
    parts = torch.randn(S, B, ld, device=DEV) * 0.6
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    results = {}
    for fused in (False, True):
        for n_splits in (1, 4, 8):
            torch.manual_seed(1)
            kp = torch.randn(n_pages, hkv, 64, hd, device=DEV).to(torch.bfloat16)
            vp = torch.randn(n_pages, hkv, 64, hd, device=DEV).to(torch.bfloat16)
            out = torch.full((B, hq * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
            if not fused:
                qkv = torch.empty(B, ld, device=DEV, dtype=torch.bfloat16)
                k.rope_append(qkv, cos, sin, pos, seq, seq, pt, kp, vp, hq, hkv, hd, hd, False, True, parts)
                k.attention_decode_mma(qkv, ld, B, kp, vp, pt, seq, pos, out, hq, hkv, hd, hd ** -0.5, 0, n_splits, keys)
            else:
                k.attention_decode_mma(None, ld, B, kp, vp, pt, seq, pos, out, hq, hkv, hd, hd ** -0.5, 0, n_splits,
                                       keys, None, parts, cos, sin, True)
            results[(fused, n_splits)] = (out.float().clone(), kp.float().clone(), vp.float().clone())
    for n_splits in (1, 4, 8):
        a, b = results[(False, n_splits)], results[(True, n_splits)]
        torch.testing.assert_close(b[0], a[0], atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(b[1], a[1], atol=1e-2, rtol=8e-3)   # (x0*c - x1*s may contract differently: one ulp)
        assert torch.equal(b[2], a[2])


@pytest.mark.parametrize("hq,hkv,hd", [(32, 8, 64), (24, 8, 128), (8, 1, 64)])
@pytest.mark.parametrize("n_splits", [1, 3, 8])
def test_tensor_core_decode_attention_reads_and_clears_the_projections_sum(hq, hkv, hd, n_splits):
    # the schedule of a decode step: the q|k|v projection's K-slices have added themselves into ONE fp32 sum;
    # the attention kernel rotates, appends, attends, and leaves the sum zero.  Against rope_append (on the
    # sum) followed by the kernel fed with the finished q.
    from dlgo_b200.parts.rope import RotaryEmbedding
    k = K()
    torch.manual_seed(hd + n_splits)
    cos, sin = (t.to(DEV) for t in RotaryEmbedding(hd, hd, 10000.0, 700, "split_half").tables())
    lens = [300, 1, 64, 65, 640, 129]
    B = len(lens)
    pages_per = [(n + 63) // 64 for n in lens]
    n_pages = sum(pages_per) + 1
    perm = torch.randperm(n_pages).tolist()
    pt = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
    for i, n in enumerate(pages_per):
        for pg in range(n):
            pt[i, pg] = perm.pop()
    pt = pt.to(DEV)
    ld = (hq + 2 * hkv) * hd
    total = torch.randn(1, B, ld, device=DEV) * 0.6
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    got = {}
    for fused in (False, True):
        torch.manual_seed(1)
        kp = torch.randn(n_pages, hkv, 64, hd, device=DEV).to(torch.bfloat16)
        vp = torch.randn(n_pages, hkv, 64, hd, device=DEV).to(torch.bfloat16)
        out = torch.full((B, hq * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
        if not fused:
            qkv = torch.empty(B, ld, device=DEV, dtype=torch.bfloat16)
            k.rope_append(qkv, cos, sin, pos, seq, seq, pt, kp, vp, hq, hkv, hd, hd, False, True, total.clone())
            k.attention_decode_mma(qkv, ld, B, kp, vp, pt, seq, pos, out, hq, hkv, hd, hd ** -0.5, 0, n_splits, 32)
        else:
            work = total.clone()
            k.attention_decode_mma(None, ld, B, kp, vp, pt, seq, pos, out, hq, hkv, hd, hd ** -0.5, 0, n_splits, 32,
                                   None, work, cos, sin, True, clear_parts=True)
            assert float(work.abs().max()) == 0.0, "the sum must be zero again for the next step"
        got[fused] = (out.float().clone(), kp.float().clone(), vp.float().clone())
    torch.testing.assert_close(got[True][0], got[False][0], atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(got[True][1], got[False][1], atol=1e-2, rtol=8e-3)
    torch.testing.assert_close(got[True][2], got[False][2], atol=1e-2, rtol=8e-3)
