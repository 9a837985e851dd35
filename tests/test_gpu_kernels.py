"""Each kernel alone against a plain PyTorch float32 reference of the same
operation, at sizes other than the tiny models'.  Inputs are built so that a
fault shows: one far key among hundreds carries the attention, a window's edge
decides the result, pages are scattered over the cache."""
import math

import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
PAGE = 64


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == "float32" else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("wdtype", ["float32", "bfloat16"])
def test_embed(wdtype):
    from picolm_b200 import ops
    table = torch.randn(301, 72).to(DT[wdtype])
    toks = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = ops.embed(toks.to(DEV), table.to(DEV))
    assert out.dtype == torch.float32
    assert torch.equal(out.cpu(), P.embed(toks.tolist(), table.float()))


@pytest.mark.parametrize("wdtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("odtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,eps", [(200, 1e-5), (2048, 1e-6), (7, 0.1)])
def test_rmsnorm(wdtype, odtype, d, eps):
    from picolm_b200 import ops
    torch.manual_seed(d)
    x = torch.randn(9, d) * 3
    x[2] *= 1e-3                                            # a row where eps matters
    w = (1 + 0.1 * torch.randn(d)).to(DT[wdtype])
    delta = torch.randn(9, d)
    ref = P.rmsnorm(x + delta, w.float(), eps)
    xd = x.to(DEV).clone()
    out = ops.rmsnorm(xd, w.to(DEV), eps, DT[odtype], delta=delta.to(DEV))
    assert torch.allclose(out.float().cpu(), ref.to(DT[odtype]).float(), **tol(odtype))
    assert torch.equal(xd.cpu(), x + delta)                 # the sum is written back
    # gathered rows, no delta, stream untouched
    rows = torch.tensor([8, 0, 2], dtype=torch.int32)
    xd = x.to(DEV).clone()
    out = ops.rmsnorm(xd, w.to(DEV), eps, DT[odtype], rows=rows.to(DEV))
    assert torch.allclose(out.float().cpu(), P.rmsnorm(x, w.float(), eps)[rows.long()].to(DT[odtype]).float(), **tol(odtype))
    assert torch.equal(xd.cpu(), x)
    # gathered rows with a delta: the stream stays as it was
    out = ops.rmsnorm(xd, w.to(DEV), eps, DT[odtype], delta=delta.to(DEV), rows=rows.to(DEV))
    assert torch.allclose(out.float().cpu(), ref[rows.long()].to(DT[odtype]).float(), **tol(odtype))
    assert torch.equal(xd.cpu(), x)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(dtype):
    from picolm_b200 import ops
    torch.manual_seed(1)
    gu = (torch.randn(13, 2 * 172) * 4).to(DT[dtype])
    ref = P.swiglu(gu[:, :172].float(), gu[:, 172:].float())
    out = ops.swiglu(gu.to(DEV))
    assert torch.allclose(out.float().cpu(), ref.to(DT[dtype]).float(), **tol(dtype))


@pytest.mark.parametrize("types", [("float32", "float32", "float32"), ("bfloat16", "bfloat16", "bfloat16"),
                                   ("bfloat16", "bfloat16", "float32"), ("bfloat16", "float32", "float32")])
@pytest.mark.parametrize("M,N,K", [(1, 53, 91), (37, 130, 172), (129, 64, 16), (70, 257, 300)])
def test_gemm_simt(types, M, N, K):
    from picolm_b200 import ops
    torch.manual_seed(M * N + K)
    a = torch.randn(M, K).to(DT[types[0]])
    w = torch.randn(N, K).to(DT[types[1]])
    ref = P.linear(a.double(), w.double())
    out = ops.gemm_simt(a.to(DEV), w.to(DEV), DT[types[2]])
    assert out.dtype == DT[types[2]]
    t = dict(atol=1e-4, rtol=1e-5) if types[2] == "float32" else dict(atol=0.1, rtol=1e-2)
    assert torch.allclose(out.double().cpu(), ref, **t)


def _paged(k, v, lens, n_pages, dtype, seed):
    """Scatter per-sequence K/V [len, G, hd] over a paged cache with shuffled page numbers."""
    G, hd = k[0].shape[1:]
    g = torch.Generator().manual_seed(seed)
    free = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    kc = torch.full((n_pages, G, PAGE, hd), float("nan")).to(dtype)
    vc = torch.full((n_pages, G, PAGE, hd), float("nan")).to(dtype)
    max_pages = max((n + PAGE - 1) // PAGE for n in lens) + 1
    table = torch.zeros((len(lens), max_pages), dtype=torch.int32)
    for b, n in enumerate(lens):
        for blk in range((n + PAGE - 1) // PAGE):
            page = free.pop()
            table[b, blk] = page
            m = min(PAGE, n - blk * PAGE)
            kc[page, :, :m] = k[b][blk * PAGE:blk * PAGE + m].transpose(0, 1).to(dtype)
            vc[page, :, :m] = v[b][blk * PAGE:blk * PAGE + m].transpose(0, 1).to(dtype)
    return kc, vc, table


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,hd", [(6, 2, 48), (5, 5, 16), (8, 1, 128), (4, 2, 80)])
def test_attention_rows_finds_a_far_key(dtype, H, G, hd):
    """Sequences of unequal lengths; in each, one chosen far key matches the last
    queries strongly, so the output is essentially that key's value: a kernel
    that skips, misplaces or double-counts keys gives a visibly different row."""
    from picolm_b200 import ops
    torch.manual_seed(H * 100 + hd)
    lens = [300, 1, 65, 130]
    new = [3, 1, 65, 2]                                      # queries: the last `new` positions of each sequence
    ks, vs, qs, pos, seq = [], [], [], [], []
    for b, n in enumerate(lens):
        k, v = torch.randn(n, G, hd) * 0.3, torch.randn(n, G, hd)
        q = torch.randn(new[b], H, hd) * 0.3
        far = n // 7
        k[far] *= 3.0                                        # the far key stands out; the others stay small
        for h in range(H):
            q[-1, h] = k[far, h // (H // G)] * (40.0 / (k[far, h // (H // G)].norm() ** 2)) * math.sqrt(hd)
        ks.append(k), vs.append(v), qs.append(q)
        pos += list(range(n - new[b], n))
        seq += [b] * new[b]
    dt = DT[dtype]
    ks = [k.to(dt).float() for k in ks]
    vs = [v.to(dt).float() for v in vs]
    qs = [q.to(dt).float() for q in qs]
    kc, vc, table = _paged(ks, vs, lens, 16, dt, 5)
    scale = 1.0 / math.sqrt(hd)
    ref = []
    for b, n in enumerate(lens):
        full_q = torch.zeros(n, H, hd)
        full_q[n - new[b]:] = qs[b]
        ref.append(P.attention(full_q, ks[b], vs[b], scale)[n - new[b]:].reshape(new[b], H * hd))
    ref = torch.cat(ref)
    out = ops.attention_rows(torch.cat(qs).to(dt).to(DEV), kc.to(DEV), vc.to(DEV),
                             torch.tensor(pos, dtype=torch.int32, device=DEV),
                             torch.tensor(seq, dtype=torch.int32, device=DEV), table.to(DEV), G, scale)
    assert torch.isfinite(out).all()
    assert torch.allclose(out.float().cpu(), ref, **(dict(atol=2e-5, rtol=1e-5) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)))
    # the last query of sequence 0 sees (almost) only the far key's value
    far_v = vs[0][lens[0] // 7]
    row = out.float().cpu()[new[0] - 1].reshape(H, hd)
    for h in range(H):
        assert torch.allclose(row[h], far_v[h // (H // G)], atol=5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_rows_window_edge(dtype):
    """With a window of W the key at distance W-1 counts and the key at distance
    W does not: both are made dominant in turn."""
    from picolm_b200 import ops
    H = G = 2
    hd, n, W = 32, 200, 70
    dt = DT[dtype]
    torch.manual_seed(9)
    for dist, inside in ((W - 1, True), (W, False)):
        k = (torch.randn(n, G, hd) * 0.1).to(dt).float()
        v = torch.randn(n, G, hd).to(dt).float()
        q = torch.zeros(1, H, hd)
        for h in range(H):
            kk = k[n - 1 - dist, h]
            q[0, h] = kk * (50.0 / kk.norm() ** 2) * math.sqrt(hd)
        q = q.to(dt).float()
        kc, vc, table = _paged([k], [v], [n], 8, dt, 2)
        out = ops.attention_rows(q.to(dt).to(DEV), kc.to(DEV), vc.to(DEV),
                                 torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                                 torch.tensor([0], dtype=torch.int32, device=DEV), table.to(DEV), G,
                                 1.0 / math.sqrt(hd), window=W).float().cpu().reshape(H, hd)
        full_q = torch.zeros(n, H, hd)
        full_q[-1] = q[0]
        ref = P.attention(full_q, k, v, 1.0 / math.sqrt(hd), window=W)[-1]
        assert torch.allclose(out, ref, atol=3e-2 if dtype == "bfloat16" else 2e-5)
        hit = torch.allclose(out, v[n - 1 - dist], atol=5e-2)
        assert hit == inside


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pairing", ["half", "adjacent"])
@pytest.mark.parametrize("H,G,hd,rot", [(3, 1, 32, 32), (4, 2, 48, 16), (2, 2, 16, 16)])
def test_rope_store(dtype, pairing, H, G, hd, rot):
    """Rotation against the plain formula, and every K/V row lands at its own
    (page, kv head, place in page); nothing else in the cache changes."""
    from picolm_b200 import ops
    dt = DT[dtype]
    torch.manual_seed(hd + rot)
    pos = [0, 1, 63, 64, 129, 7]
    seq = [0, 0, 0, 0, 0, 1]
    table = torch.tensor([[5, 2, 9], [3, 0, 0]], dtype=torch.int32)
    T = len(pos)
    qkv = torch.randn(T, (H + 2 * G) * hd).to(dt)
    cos, sin = P.rope_table(200, rot, 10000.0, None)
    cos, sin = cos.float(), sin.float()
    kc = torch.full((10, G, PAGE, hd), 7.0).to(dt)
    vc = torch.full((10, G, PAGE, hd), 7.0).to(dt)
    q_out = torch.empty(T, H, hd, dtype=dt, device=DEV)
    kcd, vcd = kc.to(DEV), vc.to(DEV)
    ops.rope_store(qkv.to(DEV), q_out, kcd, vcd, cos.to(DEV), sin.to(DEV),
                   torch.tensor(pos, dtype=torch.int32, device=DEV), torch.tensor(seq, dtype=torch.int32, device=DEV),
                   table.to(DEV), H, G, hd, rot, pairing)
    x = qkv.float().reshape(T, H + 2 * G, hd)

    def rotate(part):                                       # [T, heads, hd] by each token's own position
        out = part.clone()
        for t, p in enumerate(pos):
            out[t:t + 1, :, :rot] = P.rope(part[t:t + 1, :, :rot], cos[p:p + 1], sin[p:p + 1], pairing)
        return out

    t_ = tol(dtype)
    assert torch.allclose(q_out.float().cpu(), rotate(x[:, :H]).to(dt).float(), **t_)
    k_ref, v_ref = rotate(x[:, H:H + G]).to(dt).float(), x[:, H + G:]
    expect_k, expect_v = kc.float().clone(), vc.float().clone()
    for t, (p, b) in enumerate(zip(pos, seq)):
        page = table[b, p // PAGE].item()
        expect_k[page, :, p % PAGE] = k_ref[t]
        expect_v[page, :, p % PAGE] = v_ref[t]
    assert torch.allclose(kcd.float().cpu(), expect_k, **t_)
    assert torch.equal(vcd.float().cpu(), expect_v)


def test_argmax_first_index_on_ties():
    from picolm_b200 import ops
    x = torch.randn(5, 1000)
    x[0, 700] = x[0, 30] = 9.0
    x[1, 999] = 20.0
    x[2] = 0.0
    x[3, 0] = 50.0
    out = ops.argmax(x.to(DEV)).cpu().tolist()
    assert out == [P.argmax(r) for r in x]
    assert out[0] == 30 and out[2] == 0


@pytest.mark.parametrize("temperature,top_k,top_p,min_p", [
    (0.8, 40, 0.9, 0.05), (1.0, 0, 1.0, 0.0), (0.5, 5, 1.0, 0.0), (1.3, 0, 0.7, 0.0), (0.9, 0, 1.0, 0.2),
    (2.0, 3, 0.5, 0.5)])
def test_sample_against_the_reference_chain(temperature, top_k, top_p, min_p):
    """Same kept set and weights as the reference's chain; the draw walks in
    index order.  Several rows, each with its own xorshift64 stream, several
    draws in a row (the state advances in place)."""
    from picolm_b200 import ops
    from picolm_b200.sampling import stream_seed
    torch.manual_seed(3)
    V = 777
    logits = torch.randn(6, V) * 3
    states = [stream_seed(42, i) for i in range(6)]
    rng = torch.tensor(states, dtype=torch.int64, device=DEV)
    ld = logits.to(DEV)
    for _ in range(4):
        got = ops.sample(ld, rng, temperature, top_k, top_p, min_p).cpu().tolist()
        for r in range(6):
            states[r], want = P.sample_index_order(logits[r], temperature, top_k, top_p, min_p, states[r])
            kept, _ = P.sampling_weights(logits[r], temperature, top_k, top_p, min_p)
            assert got[r] in kept
            assert got[r] == want, f"row {r}: kernel drew {got[r]}, the plain chain {want}"
    back = [s if s >= 0 else s + (1 << 64) for s in rng.cpu().tolist()]
    assert back == states


@pytest.mark.parametrize("V", [7, 4099, 50257, 128256])
def test_sample_vocabulary_sizes(V):
    """Vocabularies from fewer entries than the cluster has CTAs up to the largest in use: rows of very
    different spread, one of them with a far token that carries almost all of the mass."""
    from picolm_b200 import ops
    from picolm_b200.sampling import stream_seed
    torch.manual_seed(V)
    logits = torch.randn(3, V) * torch.tensor([[0.5], [3.0], [8.0]])
    logits[1, V - 1] = 40.0
    states = [stream_seed(7, i) for i in range(3)]
    rng = torch.tensor(states, dtype=torch.int64, device=DEV)
    for params in ((0.8, 40, 0.9, 0.05), (1.1, 0, 0.95, 0.0)):
        got = ops.sample(logits.to(DEV), rng, *params).cpu().tolist()
        for r in range(3):
            states[r], want = P.sample_index_order(logits[r], *params, states[r])
            kept, _ = P.sampling_weights(logits[r], *params)
            assert got[r] in set(kept)
            if len(kept) <= 1000:                            # beyond that the order of a float32 sum decides
                assert got[r] == want, f"V={V} row {r}: kernel drew {got[r]}, the plain chain {want}"
    assert got[1] == V - 1


def test_sample_distribution():
    """Over many draws the kernel's frequencies follow softmax(logits / T) on a small vocabulary."""
    from picolm_b200 import ops
    V, n = 12, 4000
    logits = torch.linspace(-2, 2, V)[None, :].repeat(n, 1).contiguous()
    rng = torch.arange(1, n + 1, dtype=torch.int64, device=DEV) * 7919
    for _ in range(3):                                       # let the streams decorrelate from their seeds
        got = ops.sample(logits.to(DEV), rng, 0.7, 0, 1.0, 0.0)
    freq = torch.bincount(got.cpu().long(), minlength=V).double() / n
    p = torch.softmax(logits[0].double() / 0.7, dim=0)
    chi2 = (n * (freq - p) ** 2 / p).sum().item()
    assert chi2 < 40.0                                       # 11 degrees of freedom: 40 is beyond p = 1e-4


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (2048, 512, 256), (300, 640, 200), (1000, 1152, 2048), (129, 128, 72),
                                   (2048, 3072, 256), (2100, 2944, 192)])
def test_gemm_tc_pair(out_dtype, M, N, K, swiglu):
    """The product by pairs of CTAs (tcgen05.mma.cta_group::2, tiles of 256 x 256 or 256 x 192) against float64: whole
    and ragged tiles in both directions (a pair whose second CTA has no rows or no features left), K
    tails, more tiles than pairs, both epilogues."""
    from picolm_b200 import ops
    if swiglu and out_dtype == "float32":
        pytest.skip("the SwiGLU epilogue writes bfloat16")
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K) / K ** 0.25).to(torch.bfloat16)
    w = (torch.randn(N, K) / K ** 0.25).to(torch.bfloat16)
    a[:, K // 3] += 2.0
    w[N // 2, :] *= 3.0
    y = a.double() @ w.double().t()
    if swiglu:
        wd = ops.interleave_gate_up(w[: N // 2].contiguous().to(DEV), w[N // 2:].contiguous().to(DEV))
        got = ops.gemm_tc_wide(a.to(DEV), wd, torch.bfloat16, swiglu=True, pair=True)
        g, u = y[:, : N // 2].bfloat16().double(), y[:, N // 2:].bfloat16().double()
        ref = g / (1 + torch.exp(-g)) * u
        assert got.shape == (M, N // 2)
    else:
        got = ops.gemm_tc_wide(a.to(DEV), w.to(DEV), DT[out_dtype], pair=True)
        ref = y
        assert got.shape == (M, N)
    ops.check_status(DEV)
    if out_dtype == "float32":
        assert torch.allclose(got.double().cpu(), ref, atol=2e-3, rtol=1e-4)
    else:
        assert torch.allclose(got.double().cpu(), ref, atol=3e-2, rtol=2e-2)
    # the single-CTA kernel accumulates in the same order: the same bits (unless it cuts K into parts,
    # which it does where the tiles are few)
    if not swiglu:
        single = ops.gemm_tc_wide(a.to(DEV), w.to(DEV), DT[out_dtype])
        if (M, N, K) == (1000, 1152, 2048):
            assert torch.allclose(got.double(), single.double(), atol=2e-3 if out_dtype == "float32" else 3e-2, rtol=1e-2)
        else:
            assert torch.equal(got, single)


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(100, 2048, 2048), (300, 2048, 8192), (256, 3072, 2048), (65, 2052, 520)])
def test_gemm_tc_wide_with_k_in_parts(out_dtype, M, N, K):
    """Prompts of a few hundred tokens: few tiles, so the prompt-shaped product cuts K into parts that pass
    through scratch memory and a second kernel; against float64, and the same bits on a second call."""
    from picolm_b200 import ops
    from picolm_b200.ops._lib import _fn
    assert _fn("gemm_tc_wide", "plm_gemm_tc_wide_splits")(M, N, K) > 1
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K) / K ** 0.25).to(torch.bfloat16)
    w = (torch.randn(N, K) / K ** 0.25).to(torch.bfloat16)
    a[:, K // 3] += 2.0
    w[N // 2, :] *= 3.0
    ref = a.double() @ w.double().t()
    got = ops.linear(a.to(DEV), w.to(DEV), DT[out_dtype])
    ops.check_status(DEV)
    if out_dtype == "float32":
        assert torch.allclose(got.double().cpu(), ref, atol=2e-3, rtol=1e-4)
    else:
        assert torch.allclose(got.double().cpu(), ref, atol=3e-2, rtol=2e-2)
    assert torch.equal(got, ops.linear(a.to(DEV), w.to(DEV), DT[out_dtype]))


@pytest.mark.parametrize("M,N,K", [(2048, 2048, 512), (2304, 2562, 264), (1100, 2100, 328), (4100, 2400, 72),
                                   (3000, 3340, 136), (2900, 3333, 64), (20000, 130, 64), (2048, 3072, 128),
                                   (2100, 3000, 192)])
def test_product_added_to_the_stream_in_its_epilogue(M, N, K):
    """x += a @ w^T with the add in the product's epilogue (single CTAs and pairs, as the shape decides):
    against float64, ragged tiles in both directions, widths that are no multiple of 4 or 32 (the
    element-wise tail), and every element outside the product's rows untouched."""
    from picolm_b200 import ops
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K) / K ** 0.25).to(torch.bfloat16)
    w = (torch.randn(N, K) / K ** 0.25).to(torch.bfloat16)
    a[:, K // 3] += 2.0
    w[N // 2, :] *= 3.0
    x0 = torch.randn(M + 1, N) * 3
    x = x0.to(DEV)
    pending = ops.PendingLinear(a.to(DEV), w.to(DEV))
    assert pending.adds_in_place(x[:M])
    pending.add_into(x[:M])
    ops.check_status(DEV)
    ref = x0[:M].double() + a.double() @ w.double().t()
    assert torch.allclose(x[:M].double().cpu(), ref, atol=2e-3, rtol=1e-4)
    assert torch.equal(x[M].cpu(), x0[M])
    # the norm takes the same road: the sum lands in the stream, the rows are normalised
    x2 = x0[:M].to(DEV).contiguous()
    wn = (1 + 0.1 * torch.randn(N)).to(torch.bfloat16)
    h = ops.rmsnorm(x2, wn.to(DEV), 1e-5, torch.bfloat16, delta=ops.PendingLinear(a.to(DEV), w.to(DEV)))
    assert torch.equal(x2, x[:M])
    want = ref.float() * torch.rsqrt(ref.float().pow(2).mean(-1, keepdim=True) + 1e-5) * wn.float()
    assert torch.allclose(h.float().cpu(), want, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,d", [(300, 2048), (70, 130), (5, 6)])
def test_gather_rows(dtype, T, d):
    """Rows picked out of a matrix, in the order asked for, repeats included; widths that allow 16-byte copies
    and widths that do not; a source whose rows are wider than what is taken."""
    from picolm_b200 import ops
    torch.manual_seed(T + d)
    x = torch.randn(T, d + 2).to(DT[dtype])
    if dtype == "bfloat16" and d % 2:
        pytest.skip("rows are copied four bytes at a time")
    rows = torch.tensor([T - 1, 0, 3, 3, T // 2], dtype=torch.int32)
    got = ops.gather_rows(x.to(DEV)[:, :d], rows.to(DEV))
    assert torch.equal(got.cpu(), x[rows.long(), :d])
    got = ops.gather_rows(x.to(DEV), rows.to(DEV))
    assert torch.equal(got.cpu(), x[rows.long()])


@pytest.mark.parametrize("window", [None, 90])
@pytest.mark.parametrize("scratch", [False, True])
@pytest.mark.parametrize("H,G,hd", [(8, 2, 64), (40, 2, 16), (6, 3, 128), (4, 4, 48)])
def test_attention_decode_with_the_rotation_folded_in(H, G, hd, scratch, window):
    """The decode kernel that rotates queries and the new keys and writes the cache itself, against the
    two kernels it replaces (RoPE + cache write, then attention): the same output bit for bit, the same
    cache.  Positions at the first and the last place of a page, a sequence of one token, 20 query heads
    on a KV head (two row groups: one of them writes the cache)."""
    from types import SimpleNamespace
    from picolm_b200 import ops
    torch.manual_seed(H + hd)
    lens = [129, 1, 64, 700, 65, 320]                    # lengths after the step: the new token sits at len - 1
    B = len(lens)
    ks = [torch.randn(n, G, hd) * 0.5 for n in lens]
    vs = [torch.randn(n, G, hd) for n in lens]
    kc, vc, table = _paged(ks, vs, lens, 40, torch.bfloat16, 5)
    qkv = (torch.randn(B, (H + 2 * G) * hd) * 0.7).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    ang = torch.arange(1024, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    scale = 1.0 / math.sqrt(hd)
    step = SimpleNamespace(tok_pos=pos, tok_seq=seq, max_position=max(lens) - 1)
    # the two kernels
    k1, v1 = kc.clone().to(DEV), vc.clone().to(DEV)
    q = torch.empty((B, H, hd), dtype=torch.bfloat16, device=DEV)
    ops.rope_store(qkv, q, k1, v1, cos, sin, pos, seq, table.to(DEV), H, G, hd, hd, "half")
    n_splits = ops.decode_splits(B, H, G, max(lens))
    want = ops.attention_decode(q, k1, v1, pos, seq, table.to(DEV), G, scale, n_splits, window=window, scratch=scratch)
    # the one kernel
    k2, v2 = kc.clone().to(DEV), vc.clone().to(DEV)
    kv = SimpleNamespace(k=k2, v=v2, block_table=table.to(DEV), window=window, writable=True)
    rot = ops.Rotation(cos, sin, hd, "half")
    assert ops.attention_decode_rope_supported(qkv, kv, rot, hd)
    got = ops.attention_decode_rope(qkv, kv, step, H, G, hd, scale, rot, scratch=scratch)
    assert torch.isfinite(got).all()
    assert torch.equal(got, want)
    # the cache: the same values wherever the first way wrote some (unused places hold NaN in both)
    assert torch.equal(torch.nan_to_num(k2.float(), nan=7.0), torch.nan_to_num(k1.float(), nan=7.0))
    assert torch.equal(torch.nan_to_num(v2.float(), nan=7.0), torch.nan_to_num(v1.float(), nan=7.0))


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("T,F,K,N2", [(1, 128, 64, 256), (8, 2048, 512, 3072), (17, 200, 264, 384), (33, 136, 1024, 128),
                                       (64, 328, 192, 640)])
def test_norm_split_over_two_products(T, F, K, N2, swiglu):
    """An RMSNorm between two products, done by their epilogues: the first adds its result to the
    residual stream, applies the norm's weight and leaves the rows' sums of squares; the second scales
    its results.  Against x + a w^T, its RMSNorm and the product of that, in float64."""
    from picolm_b200 import ops
    torch.manual_seed(T + F + K)
    eps = 1e-5
    a = (torch.randn(T, K) / K ** 0.25).to(torch.bfloat16)
    w = (torch.randn(F, K) / K ** 0.25).to(torch.bfloat16)
    x = torch.randn(T, F) * torch.linspace(0.2, 5.0, T)[:, None]          # rows of very different size
    nw = (1.0 + 0.3 * torch.randn(F)).to(torch.bfloat16)
    w2 = (torch.randn(N2, F) / F ** 0.5).to(torch.bfloat16)
    xn = x.double() + a.double() @ w.double().t()
    h = xn / torch.sqrt((xn * xn).mean(dim=1, keepdim=True) + eps) * nw.double()
    y = h @ w2.double().t()
    xd = x.to(DEV)
    pending = ops.linear(a.to(DEV), w.to(DEV), torch.float32, defer=True)
    assert isinstance(pending, ops.PendingLinear)
    rows = ops.linear_residual_norm(pending, xd, nw.to(DEV), eps)
    rows.ready()                                                            # (the product may be held back for a chain)
    assert torch.allclose(xd.double().cpu(), xn, atol=2e-3, rtol=1e-4)      # the stream, updated in place
    assert torch.allclose(rows.materialize().double().cpu(), h, atol=3e-2, rtol=2e-2)
    if swiglu:
        w2d = ops.interleave_gate_up(w2[: N2 // 2].contiguous().to(DEV), w2[N2 // 2:].contiguous().to(DEV))
        got = ops.linear_swiglu(rows, w2d).double().cpu()
        g, u = y[:, : N2 // 2], y[:, N2 // 2:]
        ref = g / (1 + torch.exp(-g)) * u
    else:
        got = ops.linear(rows, w2.to(DEV), torch.bfloat16).double().cpu()
        ref = y
    ops.check_status(DEV)
    assert torch.allclose(got, ref, atol=4e-2, rtol=3e-2)
    # the same rows in another batch give the same values: the sums run in a fixed order
    if T > 1:
        x1 = x[-1:].contiguous().to(DEV)
        rows1 = ops.linear_residual_norm(ops.linear(a[-1:].contiguous().to(DEV), w.to(DEV), torch.float32, defer=True),
                                         x1, nw.to(DEV), eps)
        rows1.ready()
        assert torch.equal(x1[0], xd[-1])
        assert torch.equal(rows1.materialize()[0], rows.materialize()[-1])


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [
    (1, 128, 64), (8, 3072, 2048), (16, 200, 264), (17, 256, 512), (33, 130, 1024), (64, 2048, 8192)])
def test_gemm_tc_with_a_workspace(out_dtype, M, N, K):
    """The exported split-K product for at most 64 rows (weights on the MMA's 128 rows, K split, partials
    summed from a caller's workspace) against a float64 product of the same bf16 inputs: ragged edges in
    every dimension, K tails that are no multiple of the 64-wide stage."""
    from util import gemm_tc_workspace
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K) / K ** 0.25).to(torch.bfloat16)
    w = (torch.randn(N, K) / K ** 0.25).to(torch.bfloat16)
    # structure that a transposed, shifted or partly skipped tile cannot reproduce
    a[:, K // 3] += 2.0
    w[N // 2, :] *= 3.0
    ref = a.double() @ w.double().t()
    out = gemm_tc_workspace(a.to(DEV), w.to(DEV), DT[out_dtype])
    assert out.dtype == DT[out_dtype] and out.shape == (M, N)
    got = out.double().cpu()
    if out_dtype == "float32":
        assert torch.allclose(got, ref, atol=2e-3, rtol=1e-4)          # fp32 accumulation of exact bf16 products
    else:
        assert torch.allclose(got, ref, atol=2e-2, rtol=1e-2)


def test_gemm_tc_refuses_what_tma_cannot_address():
    from picolm_b200 import ops
    a = torch.zeros(4, 172, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, 172, dtype=torch.bfloat16, device=DEV)
    assert not ops.gemm_tc_supported(a, w)                             # rows of 344 bytes: not 16-byte aligned
    with pytest.raises(ops.KernelError, match="supported"):
        ops.gemm_tc_skinny(a, w, torch.float32)
    assert not ops.gemm_tc_supported(a.float(), w.float())
    out = ops.linear(a, w, torch.float32)                              # the dispatcher falls to the any-size kernel
    assert out.shape == (4, 64)


def _attn_case(H, G, hd, lens, new, seed, far_scale=40.0):
    """Sequences of `lens` keys whose last `new` positions are the queries; in every sequence the key at
    len // 7 matches the last query of every head strongly."""
    torch.manual_seed(seed)
    ks, vs, qs = [], [], []
    for b, n in enumerate(lens):
        k, v = torch.randn(n, G, hd) * 0.3, torch.randn(n, G, hd)
        q = torch.randn(new[b], H, hd) * 0.5
        far = n // 7
        k[far] *= 3.0
        for h in range(H):
            kk = k[far, h // (H // G)]
            q[-1, h] = kk * (far_scale / kk.norm() ** 2) * math.sqrt(hd)
        ks.append(k.to(torch.bfloat16).float()), vs.append(v.to(torch.bfloat16).float())
        qs.append(q.to(torch.bfloat16).float())
    return ks, vs, qs


def _attn_ref(ks, vs, qs, lens, new, H, hd, scale, window=None):
    ref = []
    for b, n in enumerate(lens):
        full_q = torch.zeros(n, H, hd)
        full_q[n - new[b]:] = qs[b]
        ref.append(P.attention(full_q, ks[b], vs[b], scale, window)[n - new[b]:].reshape(new[b], H * hd))
    return torch.cat(ref)


@pytest.mark.parametrize("window", [None, 90])
@pytest.mark.parametrize("H,G,hd", [(8, 2, 64), (6, 2, 48), (5, 5, 16), (32, 1, 128), (3, 1, 32), (4, 2, 256)])
def test_attention_prefill_mma(H, G, hd, window):
    """Ragged prefill on the tensor cores: whole prompts, a one-token sequence, a chunk that continues a
    cached prefix (300 keys, 70 of them new), lengths that straddle pages and query tiles."""
    from picolm_b200 import ops
    lens, new = [300, 1, 65, 130, 64], [70, 1, 65, 130, 3]
    ks, vs, qs = _attn_case(H, G, hd, lens, new, H * 7 + hd)
    scale = 1.0 / math.sqrt(hd)
    ref = _attn_ref(ks, vs, qs, lens, new, H, hd, scale, window)
    kc, vc, table = _paged(ks, vs, lens, 20, torch.bfloat16, 11)
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    out = ops.attention_prefill(torch.cat(qs).to(torch.bfloat16).to(DEV), kc.to(DEV), vc.to(DEV),
                                torch.tensor(starts, dtype=torch.int32, device=DEV),
                                torch.tensor(lens, dtype=torch.int32, device=DEV), table.to(DEV), max(new), G, scale,
                                window=window)
    assert torch.isfinite(out).all()
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=3e-2)
    if window is None:                                   # the far key carries the last row of the first sequence
        row = out.float().cpu()[new[0] - 1].reshape(H, hd)
        for h in range(H):
            assert torch.allclose(row[h], vs[0][lens[0] // 7][h // (H // G)], atol=5e-2)


@pytest.mark.parametrize("window", [None, 90])
@pytest.mark.parametrize("n_splits,scratch", [(1, False), (2, False), (3, False), (3, True), (8, False), (16, True), (37, True)])
@pytest.mark.parametrize("H,G,hd", [(8, 2, 64), (6, 2, 48), (5, 5, 16), (40, 1, 128), (3, 1, 32), (4, 2, 256)])
def test_attention_decode_mma(H, G, hd, n_splits, scratch, window):
    """Decode on the tensor cores with the keys cut into ranges: sequences of very unequal lengths (some
    ranges stay empty), more heads per KV head than one row group holds, a far key that must be found.
    The ranges merge inside a thread-block cluster, or through a scratch buffer and a second kernel."""
    from picolm_b200 import ops
    lens = [700, 1, 65, 130, 64, 257]
    new = [1] * len(lens)
    ks, vs, qs = _attn_case(H, G, hd, lens, new, H * 3 + hd + n_splits)
    scale = 1.0 / math.sqrt(hd)
    ref = _attn_ref(ks, vs, qs, lens, new, H, hd, scale, window)
    kc, vc, table = _paged(ks, vs, lens, 30, torch.bfloat16, 13)
    out = ops.attention_decode(torch.cat(qs).to(torch.bfloat16).to(DEV), kc.to(DEV), vc.to(DEV),
                               torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV),
                               torch.arange(len(lens), dtype=torch.int32, device=DEV), table.to(DEV), G, scale,
                               n_splits, window=window, scratch=scratch)
    assert torch.isfinite(out).all()
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=3e-2)
    if window is None:
        row = out.float().cpu()[0].reshape(H, hd)
        for h in range(H):
            assert torch.allclose(row[h], vs[0][lens[0] // 7][h // (H // G)], atol=5e-2)


@pytest.mark.parametrize("H,G,hd,n_splits", [(8, 2, 64, 47), (4, 1, 128, 33), (6, 3, 48, 94), (2, 2, 256, 19)])
def test_attention_decode_many_ranges_of_a_long_sequence(H, G, hd, n_splits):
    """One long sequence cut into many ranges that a second kernel merges (the shape of a single request far
    into its context): groups of threads add up stretches of the ranges, so counts that leave stretches of
    unequal length and tails shorter than the unrolled eight; a far key must be found; the same bits twice."""
    from picolm_b200 import ops
    lens = [6000, 70]
    new = [1, 1]
    ks, vs, qs = _attn_case(H, G, hd, lens, new, H + hd + n_splits)
    scale = 1.0 / math.sqrt(hd)
    ref = _attn_ref(ks, vs, qs, lens, new, H, hd, scale, None)
    kc, vc, table = _paged(ks, vs, lens, 100, torch.bfloat16, 5)
    args = (torch.cat(qs).to(torch.bfloat16).to(DEV), kc.to(DEV), vc.to(DEV),
            torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV),
            torch.arange(len(lens), dtype=torch.int32, device=DEV), table.to(DEV), G, scale, n_splits)
    out = ops.attention_decode(*args, scratch=True)
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=3e-2)
    row = out.float().cpu()[0].reshape(H, hd)
    for h in range(H):
        assert torch.allclose(row[h], vs[0][lens[0] // 7][h // (H // G)], atol=5e-2)
    assert torch.equal(out, ops.attention_decode(*args, scratch=True))


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 3072, 2048), (16, 200, 264), (17, 256, 512), (33, 130, 1024),
                                   (64, 2048, 8192), (5, 16384, 2048), (64, 40000, 128), (3, 2048, 2112),
                                   (7, 77001, 200), (20, 38000, 72)])
def test_gemm_tc_skinny_cluster(out_dtype, M, N, K):
    """The decode-shaped product whose K splits meet in distributed shared memory: every cluster size
    (1, 2, 4, 8), all three token-tile widths, ragged feature edges, K ranges that leave a CTA of the
    cluster with fewer (or no) K blocks; and, with more than 296 tiles of 128 features, the CTAs that stay
    and walk over the tiles (some take one tile more than others, the last tile is ragged, K ends inside
    a block)."""
    from picolm_b200 import ops
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K) / K ** 0.25).to(torch.bfloat16)
    w = (torch.randn(N, K) / K ** 0.25).to(torch.bfloat16)
    a[:, K // 3] += 2.0
    w[N // 2, :] *= 3.0
    ref = a.double() @ w.double().t()
    out = ops.gemm_tc_skinny(a.to(DEV), w.to(DEV), DT[out_dtype])
    ops.check_status(DEV)
    tol_ = dict(atol=2e-3, rtol=1e-4) if out_dtype == "float32" else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(out.double().cpu(), ref, **tol_)
    again = ops.gemm_tc_skinny(a.to(DEV), w.to(DEV), DT[out_dtype])
    assert torch.equal(out, again)                          # a fixed order of the partial sums


@pytest.mark.parametrize("M", [1, 8, 40, 64, 65, 300, 2048])
@pytest.mark.parametrize("F,K", [(64, 64), (192, 328), (8192, 2048), (1088, 512)])
def test_linear_swiglu_fused(M, F, K):
    """SwiGLU in the product's epilogue (skinny and wide paths) against gate/up products and the plain
    activation, with the rounding of gate and up to bf16 that the unfused path has."""
    from picolm_b200 import ops
    torch.manual_seed(M + F + K)
    a = torch.randn(M, K).to(torch.bfloat16)
    gate = (torch.randn(F, K) / K ** 0.5).to(torch.bfloat16)
    up = (torch.randn(F, K) / K ** 0.5).to(torch.bfloat16)
    w = ops.interleave_gate_up(gate.to(DEV), up.to(DEV))
    assert w.shape == (2 * F, K) and torch.equal(w[:64].cpu(), gate[:64]) and torch.equal(w[64:128].cpu(), up[:64])
    out = ops.linear_swiglu(a.to(DEV), w)
    ops.check_status(DEV)
    g = (a.double() @ gate.double().t()).to(torch.bfloat16).float()
    u = (a.double() @ up.double().t()).to(torch.bfloat16).float()
    ref = P.swiglu(g, u)
    assert out.shape == (M, F) and out.dtype == torch.bfloat16
    # a gate or up value that sits on a bf16 rounding boundary may round the other way: allow one such step
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("window", [None, 90])
@pytest.mark.parametrize("H,G,hd", [(8, 2, 64), (32, 1, 128), (6, 3, 64), (4, 4, 128)])
def test_attention_prefill_tcgen05(H, G, hd, window):
    """The tcgen05 prefill attention in the same ragged setting as the mma.sync kernel: whole prompts, a
    one-token sequence, a chunk after a cached prefix, lengths that straddle pages and 128-row query
    tiles, a last page that is partly unwritten (NaN there must not reach the result), a far key that
    carries a row, and a window's edge."""
    from picolm_b200 import ops
    lens, new = [300, 1, 65, 130, 64, 520], [70, 1, 65, 130, 3, 520]
    ks, vs, qs = _attn_case(H, G, hd, lens, new, H * 11 + hd)
    scale = 1.0 / math.sqrt(hd)
    ref = _attn_ref(ks, vs, qs, lens, new, H, hd, scale, window)
    kc, vc, table = _paged(ks, vs, lens, 30, torch.bfloat16, 17)
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    args = (torch.cat(qs).to(torch.bfloat16).to(DEV), kc.to(DEV), vc.to(DEV),
            torch.tensor(starts, dtype=torch.int32, device=DEV), torch.tensor(lens, dtype=torch.int32, device=DEV),
            table.to(DEV), max(new), G, scale)
    out = ops.attention_prefill_tc(*args, window=window)
    ops.check_status(DEV)
    assert torch.isfinite(out).all()
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=3e-2)
    mma = ops.attention_prefill(*args, window=window)
    assert torch.allclose(out.float(), mma.float(), atol=3e-2, rtol=3e-2)
    if window is None:
        row = out.float().cpu()[new[0] - 1].reshape(H, hd)
        for h in range(H):
            assert torch.allclose(row[h], vs[0][lens[0] // 7][h // (H // G)], atol=5e-2)


def test_attention_prefill_tcgen05_with_one_slow_warp():
    """A long prompt in which the first 32 rows of every query tile meet a larger score on every page (their
    running maximum rises by more than the kernel's lazy rescaling tolerates, so their warp rescales the
    output page after page and waits for the tensor cores each time) while the other rows never rescale:
    the softmax warps of a CTA drift apart, and a page must still get exactly its own 128 rows (the kernel
    lets nobody arrive for a page before the page in front has all its arrivals; the long sequence of
    test_gpu_real_widths.py is the case that showed the fault when that was missing)."""
    from picolm_b200 import ops
    H, G, hd, n = 4, 1, 64, 2900
    torch.manual_seed(5)
    u = torch.randn(hd)
    u /= u.norm()
    k = torch.randn(n, G, hd) * 0.3 + u * (torch.arange(n) // PAGE).float()[:, None, None]
    v = torch.randn(n, G, hd)
    q = torch.randn(n, H, hd) * 0.5
    hot = (torch.arange(n) % 128) < 32
    q[hot] = u * 64.0 + torch.randn(int(hot.sum()), H, hd) * 0.5          # 8 nats more per page at scale 1/8
    ks, vs, qs = [k.to(torch.bfloat16).float()], [v.to(torch.bfloat16).float()], [q.to(torch.bfloat16).float()]
    scale = 1.0 / math.sqrt(hd)
    ref = _attn_ref(ks, vs, qs, [n], [n], H, hd, scale)
    kc, vc, table = _paged(ks, vs, [n], 50, torch.bfloat16, 3)
    args = (qs[0].to(torch.bfloat16).to(DEV), kc.to(DEV), vc.to(DEV), torch.tensor([0, n], dtype=torch.int32, device=DEV),
            torch.tensor([n], dtype=torch.int32, device=DEV), table.to(DEV), n, G, scale)
    for _ in range(3):
        out = ops.attention_prefill_tc(*args)
        ops.check_status(DEV)
        assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("epilogue", ["float32", "bfloat16", "swiglu", "add"])
@pytest.mark.parametrize("M,N,K", [(1100, 2100, 6144), (130, 512, 8192), (1024, 2304, 6144), (128, 256, 8192)])
def test_gemm_tc_wide_stream_walk(epilogue, M, N, K):
    """The K blocks of all tiles handed out as one stream: tiles cut between two CTAs and among many (few
    tiles with a long K), with every epilogue, against float64; three launches in a row (the flags go down
    again) with the same bits; ragged edges."""
    import ctypes
    from picolm_b200 import ops
    from picolm_b200.ops._lib import _fn
    how = (ctypes.c_int * 3)()
    code = {"float32": 0, "bfloat16": 0, "swiglu": 1, "add": 2}[epilogue]
    if epilogue == "swiglu":
        N = N // 128 * 128
    _fn("gemm_tc_wide", "plm_gemm_tc_wide_how")(M, N, K, code, 148, ctypes.cast(how, ctypes.c_void_p))
    if how[1] > 1:
        pytest.skip("this shape cuts K through scratch memory with the store epilogue")
    assert how[2] > 0, "the shape was chosen to take the stream walk"
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K) / K ** 0.25).to(torch.bfloat16)
    w = (torch.randn(N, K) / K ** 0.25).to(torch.bfloat16)
    a[:, K // 3] += 2.0
    w[N // 2, :] *= 3.0
    a[M // 2, :] *= -2.0
    y = a.double() @ w.double().t()
    ad, wd = a.to(DEV), w.to(DEV)
    outs = []
    for _ in range(3):
        if epilogue == "swiglu":
            wi = ops.interleave_gate_up(wd[: N // 2].contiguous(), wd[N // 2:].contiguous())
            got = ops.gemm_tc_wide(ad, wi, torch.bfloat16, swiglu=True)
            g, u = y[:, : N // 2].bfloat16().double(), y[:, N // 2:].bfloat16().double()
            ref, tol_ = g / (1 + torch.exp(-g)) * u, dict(atol=3e-2, rtol=2e-2)
        elif epilogue == "add":
            x0 = torch.randn(M, N) * 3
            got = ops.gemm_tc_wide(ad, wd, torch.float32, out=x0.to(DEV), add=True)
            ref, tol_ = x0.double() + y, dict(atol=2e-3, rtol=1e-4)
        else:
            got = ops.gemm_tc_wide(ad, wd, DT[epilogue])
            ref, tol_ = y, dict(atol=2e-3, rtol=1e-4) if epilogue == "float32" else dict(atol=3e-2, rtol=2e-2)
        ops.check_status(DEV)
        assert torch.allclose(got.double().cpu(), ref, **tol_)
        outs.append(got)
    if epilogue != "add":
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    from picolm_b200.ops._lib import stream_space
    assert int(stream_space(DEV)[1].abs().sum()) == 0


@pytest.mark.parametrize("epilogue", ["float32", "bfloat16", "swiglu", "add"])
@pytest.mark.parametrize("M,N,K", [(1024, 2304, 6144), (512, 2048, 8192), (300, 700, 8192)])
def test_gemm_tc_pair_stream_walk(epilogue, M, N, K):
    """Pairs of CTAs that walk the stages of few tiles as one stream (each CTA of a pair leaves and adds the part
    of its own 128 rows): against float64, three launches with the same bits, ragged edges."""
    from picolm_b200 import ops
    from picolm_b200.ops._lib import _fn, stream_space
    if epilogue == "swiglu":
        N = N // 128 * 128
    assert _fn("gemm_tc_wide", "plm_gemm_tc_pair_streamed")(M, N, K, 148) > 0, "the shape was chosen to take the stream walk"
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K) / K ** 0.25).to(torch.bfloat16)
    w = (torch.randn(N, K) / K ** 0.25).to(torch.bfloat16)
    a[:, K // 3] += 2.0
    w[N // 2, :] *= 3.0
    a[M // 2, :] *= -2.0
    y = a.double() @ w.double().t()
    ad, wd = a.to(DEV), w.to(DEV)
    x0 = torch.randn(M, N) * 3
    outs = []
    for _ in range(3):
        if epilogue == "swiglu":
            wi = ops.interleave_gate_up(wd[: N // 2].contiguous(), wd[N // 2:].contiguous())
            got = ops.gemm_tc_wide(ad, wi, torch.bfloat16, swiglu=True, pair=True)
            g, u = y[:, : N // 2].bfloat16().double(), y[:, N // 2:].bfloat16().double()
            ref, tol_ = g / (1 + torch.exp(-g)) * u, dict(atol=3e-2, rtol=2e-2)
        elif epilogue == "add":
            got = ops.gemm_tc_wide(ad, wd, torch.float32, out=x0.to(DEV), add=True, pair=True)
            ref, tol_ = x0.double() + y, dict(atol=2e-3, rtol=1e-4)
        else:
            got = ops.gemm_tc_wide(ad, wd, DT[epilogue], pair=True)
            ref, tol_ = y, dict(atol=2e-3, rtol=1e-4) if epilogue == "float32" else dict(atol=3e-2, rtol=2e-2)
        ops.check_status(DEV)
        assert torch.allclose(got.double().cpu(), ref, **tol_)
        outs.append(got)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert int(stream_space(DEV)[1].abs().sum()) == 0


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(65, 128, 64), (128, 128, 128), (200, 136, 328), (300, 2048, 192),
                                   (256, 4096, 512), (1000, 264, 2048), (2048, 2560, 256), (5000, 2048, 64)])
def test_gemm_tc_wide_persistent(out_dtype, M, N, K):
    """The persistent prompt-shaped product: fewer tiles than SMs and many more, both tile widths, ragged
    edges in every dimension, several tiles per CTA so that both accumulators and the barrier phases
    across tiles are exercised."""
    from picolm_b200 import ops
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K) / K ** 0.25).to(torch.bfloat16)
    w = (torch.randn(N, K) / K ** 0.25).to(torch.bfloat16)
    a[:, K // 3] += 2.0
    w[N // 2, :] *= 3.0
    a[M // 2, :] *= -2.0
    ref = a.double() @ w.double().t()
    out = ops.gemm_tc_wide(a.to(DEV), w.to(DEV), DT[out_dtype])
    ops.check_status(DEV)
    tol_ = dict(atol=2e-3, rtol=1e-4) if out_dtype == "float32" else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(out.double().cpu(), ref, **tol_)
