"""Each CUDA kernel alone against a plain PyTorch float32 statement of the same operation,
at sizes other than the engine's tiny models (odd widths, head sizes in steps of 16, several
group sizes, vocabularies that are no power of two)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(autouse=True)
def guard_zones(guarded_allocations):
    """Every device buffer of these tests lies between guard zones, checked after each test."""
    yield guarded_allocations


def test_guard_zones_see_a_write_outside_a_buffer(guard_zones):
    """The checker itself: a buffer made under the fixture is usable, aligned and surrounded, and a
    byte written one place past its end, or one before its start, is found."""
    a = torch.empty(3, 5, device=DEV, dtype=torch.bfloat16)
    b = torch.full((7,), 2.0, device=DEV)
    c = torch.zeros(4, 4, device=DEV, dtype=torch.int32)
    assert a.data_ptr() % 256 == 0 and a.is_contiguous() and float(b.sum()) == 14.0 and int(c.abs().sum()) == 0
    assert guard_zones.check() >= 3
    raw, nbytes = guard_zones.held[0]
    raw[guard_zones.ZONE + nbytes] = 0
    with pytest.raises(AssertionError, match="past the end"):
        guard_zones.check()
    raw[guard_zones.ZONE + nbytes] = guard_zones.PATTERN
    raw[guard_zones.ZONE - 1] = 0
    with pytest.raises(AssertionError, match="before the start"):
        guard_zones.check()
    raw[guard_zones.ZONE - 1] = guard_zones.PATTERN


def tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,V", [(1, 16, 7), (37, 200, 1001), (5, 4096, 333)])
def test_embedding(dtype, T, H, V):
    from spyinfer_b200 import kernels
    table = torch.randn(V, H, device=DEV).to(dtype)
    ids = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    out = torch.empty(T, H, device=DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    kernels.embedding(table, ids, out, status)
    assert torch.equal(out, table.float()[ids.long()]) and status[0].item() == 0
    ids[T // 2] = V  # outside the vocabulary: reported, not read
    kernels.embedding(table, ids, out, status)
    assert status.tolist() == [1, T // 2]


@pytest.mark.parametrize("xd,dd,wd,od", [(torch.float32, torch.float32, torch.float32, torch.float32),
                                         (torch.float32, torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                         (torch.bfloat16, torch.bfloat16, torch.float32, torch.float32)])
@pytest.mark.parametrize("n,H,eps", [(1, 64, 1e-6), (19, 1000, 1e-5), (3, 5120, 1e-6), (2, 15000, 1e-3)])
def test_rmsnorm_with_residual_and_gather(xd, dd, wd, od, n, H, eps):
    from spyinfer_b200 import kernels
    x = (torch.randn(n, H, device=DEV) * 3).to(xd)
    delta = torch.randn(n, H, device=DEV).to(dd)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(wd)

    def ref(v):
        return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * w.float()

    out = torch.empty(n, H, device=DEV, dtype=od)
    kernels.rmsnorm(x, w, eps, out)
    torch.testing.assert_close(out.float(), ref(x.float()).to(od).float(), **tol(od))
    x2 = x.clone()
    kernels.rmsnorm(x2, w, eps, out, delta=delta, write_back=True)
    s = x.float() + delta.float()
    torch.testing.assert_close(out.float(), ref(s).to(od).float(), **tol(od))
    torch.testing.assert_close(x2.float(), s.to(xd).float(), rtol=0, atol=0)       # the residual sum is exact in 32-bit
    rows = torch.tensor([n - 1, 0, n - 1], device=DEV, dtype=torch.int32)
    out3 = torch.empty(3, H, device=DEV, dtype=od)
    x3 = x.clone()
    kernels.rmsnorm(x3, w, eps, out3, delta=delta, rows=rows)
    torch.testing.assert_close(out3.float(), ref(s)[rows.long()].to(od).float(), **tol(od))
    assert torch.equal(x3, x)                                                      # a gather writes nothing back


@pytest.mark.parametrize("dtypes", [(torch.float32, torch.float32, torch.float32), (torch.float32, torch.bfloat16, torch.float32),
                                    (torch.bfloat16, torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.bfloat16, torch.float32),
                                    (torch.bfloat16, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (3, 70, 50), (65, 129, 257), (130, 64, 1024), (2, 1187, 96)])
def test_gemm_simt(dtypes, M, N, K):
    from spyinfer_b200 import kernels
    ad, wd, cd = dtypes
    a = torch.randn(M, K, device=DEV).to(ad)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(wd)
    out = torch.empty(M, N, device=DEV, dtype=cd)
    kernels.gemm_simt(a, w, out)
    ref = (a.double() @ w.double().t()).float()
    torch.testing.assert_close(out.float(), ref.to(cd).float(), **tol(cd))
    # a row's result does not depend on the other rows of the batch
    if M > 1:
        one = torch.empty(1, N, device=DEV, dtype=cd)
        kernels.gemm_simt(a[M - 1:M].contiguous(), w, one)
        assert torch.equal(one[0], out[M - 1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,I", [(1, 8), (7, 224), (33, 1000)])
def test_swiglu(dtype, T, I):
    from spyinfer_b200 import kernels
    gu = (torch.randn(T, 2 * I, device=DEV) * 4).to(dtype)
    out = torch.empty(T, I, device=DEV, dtype=dtype)
    kernels.swiglu(gu, out)
    g, u = gu.float()[:, :I], gu.float()[:, I:]
    torch.testing.assert_close(out.float(), ((g / (1 + torch.exp(-g))) * u).to(dtype).float(), **tol(dtype))


def paged_setup(S, lens, nkv, hd, page_size, dtype, shuffle=True):
    """Random keys and values of S sequences scattered over shuffled pages."""
    width = max((l + page_size - 1) // page_size for l in lens)
    num_pages = S * width + 3
    perm = torch.randperm(num_pages) if shuffle else torch.arange(num_pages)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    nxt = 0
    for s, l in enumerate(lens):
        for lp in range((l + page_size - 1) // page_size):
            bt[s, lp] = perm[nxt]
            nxt += 1
    pages = torch.zeros(num_pages, 2, nkv, page_size, hd, device=DEV, dtype=dtype)
    ks = [torch.randn(l, nkv, hd, device=DEV).to(dtype) for l in lens]
    vs = [torch.randn(l, nkv, hd, device=DEV).to(dtype) for l in lens]
    for s, l in enumerate(lens):
        for p in range(l):
            page = int(bt[s, p // page_size])
            pages[page, 0, :, p % page_size] = ks[s][p]
            pages[page, 1, :, p % page_size] = vs[s][p]
    return pages, bt.to(DEV), ks, vs


def ref_attention(q, k, v, pos, scale, window):
    """q [nh, hd] at position pos over k, v [L, nkv, hd] in float64."""
    nh, nkv = q.shape[0], k.shape[1]
    lo = 0 if not window else max(0, pos - window + 1)
    out = torch.zeros_like(q, dtype=torch.float64)
    for h in range(nh):
        kvh = h // (nh // nkv)
        s = (k[lo:pos + 1, kvh].double() @ q[h].double()) * scale
        p = torch.softmax(s, dim=0)
        out[h] = p @ v[lo:pos + 1, kvh].double()
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page_size,window", [(4, 2, 16, 4, None), (6, 1, 48, 8, 20), (8, 8, 80, 16, None), (5, 5, 128, 16, 130),
                                                        (16, 2, 256, 32, None)])
def test_attention_generic_mixed_batch(dtype, nh, nkv, hd, page_size, window):
    from spyinfer_b200 import kernels
    torch.manual_seed(hd)
    lens = [1, 37, 300, 129]
    pages, bt, ks, vs = paged_setup(4, lens, nkv, hd, page_size, dtype)
    # a batch of: seq0 its only token; seq1 a portion of 5 in the middle; seq2 its last token; seq3 two tokens across a chunk edge
    toks = [(0, 0)] + [(1, p) for p in range(20, 25)] + [(2, 299)] + [(3, 127), (3, 128)]
    T = len(toks)
    q = torch.randn(T, nh * hd + 8, device=DEV).to(dtype)      # wider rows than nh*hd: only the first nh*hd columns are queries
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    seq_of = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    out = torch.empty(T, nh * hd, device=DEV, dtype=dtype)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    kernels.attention_generic(q, nh, hd, out, pages, bt, positions, seq_of, scale, window=window, status=status)
    assert status[0].item() == 0
    for i, (s, p) in enumerate(toks):
        ref = ref_attention(q[i, :nh * hd].view(nh, hd), ks[s], vs[s], p, scale, window)
        torch.testing.assert_close(out[i].view(nh, hd).double(), ref, **(dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16
                                                                         else dict(rtol=1e-4, atol=1e-5)))


def test_attention_generic_finds_one_far_key():
    """One key among hundreds is made to stand out (its score is far above the rest): the
    output must be that key's value row, wherever it lies: first slot of a page, last slot,
    the first key of all, the key just inside a window, and never the one just outside."""
    from spyinfer_b200 import kernels
    nh, nkv, hd, page_size, L = 2, 1, 32, 16, 700
    pages, bt, ks, vs = paged_setup(1, [L], nkv, hd, page_size, torch.float32)
    q = torch.randn(1, nh * hd, device=DEV)
    pos = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(1, nh * hd, device=DEV)
    for window, far in [(None, 0), (None, 15), (None, 16), (None, 127), (None, 128), (None, 511), (300, L - 300), (300, L - 301)]:
        pg = pages.clone()
        page, slot = int(bt[0, far // page_size]), far % page_size
        pg[page, 0, 0, slot] = 40.0 * q[0, :hd] / q[0, :hd].norm()     # aligned with head 0's query, large
        kernels.attention_generic(q, nh, hd, out, pg, bt, pos, seq, 1.0, window=window)
        hit = torch.allclose(out[0, :hd], vs[0][far, 0], atol=1e-3)
        inside = window is None or far > L - 1 - window
        assert hit == inside, f"window {window}, far key {far}: expected {'a hit' if inside else 'no hit'}"


@pytest.mark.parametrize("adtype,cdtype,wdtype", [(torch.float32, torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                                  (torch.float32, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
@pytest.mark.parametrize("nh,nkv,hd,rot,page_size", [(4, 2, 16, 16, 4), (3, 3, 48, 32, 8), (8, 2, 128, 128, 16), (2, 1, 80, 80, 5), (5, 1, 128, 64, 16)])
def test_qk_norm_rope_store(adtype, cdtype, wdtype, nh, nkv, hd, rot, page_size, pairing):
    from spyinfer_b200 import kernels
    torch.manual_seed(nh * hd)
    S, lens = 3, [9, 1, 30]
    starts = [4, 0, 27]                                   # this step brings positions [start, len) of each sequence
    width = 8
    perm = torch.randperm(S * width)
    bt = perm.view(S, width).to(torch.int32).to(DEV)
    pages = torch.zeros(S * width, 2, nkv, page_size, hd, device=DEV, dtype=cdtype)
    toks = [(s, p) for s in range(S) for p in range(starts[s], lens[s])]
    T = len(toks)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).to(adtype)
    qw = (1 + 0.2 * torch.randn(hd, device=DEV)).to(wdtype)
    kw = (1 + 0.2 * torch.randn(hd, device=DEV)).to(wdtype)
    eps, theta = 1e-5, 10000.0
    inv = torch.pow(torch.tensor(theta), -torch.arange(rot // 2, dtype=torch.float32) / (rot // 2)).to(DEV)
    table = kernels.build_rope_table(inv, 64)
    pos_f = torch.arange(64, dtype=torch.float32, device=DEV)[:, None] * inv[None, :]
    torch.testing.assert_close(table[..., 0], torch.cos(pos_f), rtol=0, atol=2e-6)
    torch.testing.assert_close(table[..., 1], torch.sin(pos_f), rtol=0, atol=2e-6)
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    seq_of = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    before = qkv.clone().float()
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    kernels.qk_rope_store(qkv, nh, nkv, hd, qw, kw, eps, table, positions, seq_of, bt, pages, store=True, status=status, pairing=pairing)
    assert status[0].item() == 0

    def norm_rope(x, w):                                    # x [T, heads, hd] float32
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()
        c, s = torch.cos(pos_f[positions.long()])[:, None, :], torch.sin(pos_f[positions.long()])[:, None, :]
        if pairing == "interleaved":                        # angle j turns the pair (2j, 2j + 1)
            lo, hi, rest = x[..., 0:rot:2], x[..., 1:rot:2], x[..., rot:]
            turned = torch.stack([lo * c - hi * s, lo * s + hi * c], dim=-1).flatten(-2)
            return torch.cat([turned, rest], dim=-1)
        lo, hi, rest = x[..., :rot // 2], x[..., rot // 2:rot], x[..., rot:]
        return torch.cat([lo * c - hi * s, lo * s + hi * c, rest], dim=-1)

    q_ref = norm_rope(before[:, :nh * hd].view(T, nh, hd), qw)
    k_ref = norm_rope(before[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd), kw)
    v_ref = before[:, (nh + nkv) * hd:].view(T, nkv, hd)
    t = tol(adtype)
    torch.testing.assert_close(qkv[:, :nh * hd].float().view(T, nh, hd), q_ref.to(adtype).float(), **t)
    assert torch.equal(qkv[:, nh * hd:].float(), before[:, nh * hd:])       # k and v columns are left as they were
    for i, (s, p) in enumerate(toks):
        page = int(bt[s, p // page_size])
        torch.testing.assert_close(pages[page, 0, :, p % page_size].float(), k_ref[i].to(cdtype).float(), **tol(cdtype))
        torch.testing.assert_close(pages[page, 1, :, p % page_size].float(), v_ref[i].to(cdtype).float(), rtol=0, atol=0)
    written = torch.zeros(S * width, page_size, dtype=torch.bool)
    for s, p in toks:
        written[int(bt[s, p // page_size]), p % page_size] = True
    assert (pages.float().abs().sum(dim=(1, 2, 4)).cpu()[~written] == 0).all()   # no other slot of any page was touched
    # store=False touches no page and still norms and rotates q
    qkv2 = before.to(adtype)
    pages2 = torch.zeros_like(pages)
    kernels.qk_rope_store(qkv2, nh, nkv, hd, qw, kw, eps, table, positions, seq_of, None, None, store=False, pairing=pairing)
    assert torch.equal(qkv2[:, :nh * hd], qkv[:, :nh * hd]) and pages2.abs().sum() == 0
    # a block-table entry that is no page is reported and skipped
    bad = bt.clone()
    bad[0, starts[0] // page_size] = S * width
    kernels.qk_rope_store(before.to(adtype), nh, nkv, hd, qw, kw, eps, table, positions, seq_of, bad, pages, store=True, status=status)
    assert status[0].item() == 3


def test_sampling_greedy_and_distribution():
    from spyinfer_b200 import kernels
    V = 1187
    logits = torch.randn(6, V, device=DEV)
    logits[2, 5] = logits[2, 900] = 50.0             # a tie: the lowest index wins
    tokens = torch.empty(6, dtype=torch.int32, device=DEV)
    kernels.sample(logits, tokens)
    want = logits.argmax(dim=-1)
    want[2] = 5
    assert tokens.tolist() == want.tolist()
    # temperature: frequencies of many seeded draws follow softmax(logits / T)
    V2, n, temp = 23, 20000, 0.7
    row = torch.randn(V2, device=DEV) * 2
    lg = row.expand(n, V2).contiguous()
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    t = torch.full((n,), temp, device=DEV)
    seed = torch.full((n,), 99, dtype=torch.int64, device=DEV)
    draw = torch.arange(n, dtype=torch.int64, device=DEV)
    kernels.sample(lg, out, t, seed, draw)
    freq = torch.bincount(out.long(), minlength=V2).double() / n
    p = torch.softmax(row.double() / temp, dim=0)
    assert (freq - p).abs().max() < 4 * math.sqrt(0.25 / n) + 1e-3
    again = torch.empty_like(out)
    kernels.sample(lg, again, t, seed, draw)
    assert torch.equal(out, again)                   # same seed and draw number: same token
    t0 = torch.zeros(n, device=DEV)                  # temperature 0 is greedy
    kernels.sample(lg, again, t0, seed, draw)
    assert (again == int(row.argmax())).all()


def test_sampling_top_k_draws_only_among_the_largest():
    """Top-k at a vocabulary that is no power of two and larger than one slice: frequencies follow
    the softmax over the k largest logits, nothing else is ever drawn; k = 1 is the argmax; ties at
    the k-th value stay; a row without top_k beside rows with it draws from the whole row; negative
    logits and equal bit patterns across the radix passes (values that share their top bytes)."""
    from spyinfer_b200 import kernels
    import plain_model
    torch.manual_seed(5)
    V, n, temp = 5003, 20000, 1.3
    row = torch.randn(V, device=DEV) * 0.01 - 3.0       # close values: they share the top bytes of their bit patterns
    top = torch.randperm(V, device=DEV)[:9]
    row[top] = torch.tensor([2.0, 1.5, 1.5, 1.0, 0.5, 0.0, -0.5, -1.0, -1.0], device=DEV)
    lg = row.expand(n, V).contiguous()
    t = torch.full((n,), temp, device=DEV)
    seed = torch.full((n,), 7, dtype=torch.int64, device=DEV)
    draw = torch.arange(n, dtype=torch.int64, device=DEV)
    for k in (1, 3, 5, 8, 40):
        out = torch.empty(n, dtype=torch.int32, device=DEV)
        kernels.sample(lg, out, t, seed, draw, torch.full((n,), k, dtype=torch.int32, device=DEV))
        freq = torch.bincount(out.long(), minlength=V).double() / n
        p = plain_model.top_k_probabilities(row.cpu(), temp, k).to(DEV)
        assert (freq[p == 0] == 0).all(), k
        assert (freq - p).abs().max() < 4 * math.sqrt(0.25 / n) + 1e-3, k
    # k = 8 cuts between the two equal values -1.0: both stay
    assert int((plain_model.top_k_probabilities(row.cpu(), temp, 8) > 0).sum()) == 9
    # rows with and without top_k in one call; k beyond the vocabulary means all
    ks = torch.tensor([2, 0, V + 5, 1], dtype=torch.int32, device=DEV).repeat(n // 4)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    kernels.sample(lg, out, t, seed, draw, ks)
    whole = torch.empty(n, dtype=torch.int32, device=DEV)
    kernels.sample(lg, whole, t, seed, draw)
    assert torch.equal(out[1::4], whole[1::4]) and torch.equal(out[2::4], whole[2::4])
    assert (out[3::4] == int(row.argmax())).all()
    two = set(top[:3].tolist())                          # 2.0 and the two 1.5: k = 2 keeps the tie
    assert set(out[0::4].tolist()) <= two


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (5, 200, 96), (16, 4096, 4096), (17, 1000, 520), (33, 136, 72), (64, 6144, 512),
                                   (65, 300, 136), (128, 256, 64), (100, 4096, 4096), (128, 6144, 4096), (90, 1187, 1032), (129, 1187, 1032), (200, 6144, 4096), (256, 4096, 12288), (160, 9000, 520), (300, 512, 4096), (1000, 24, 200), (2048, 1024, 12288), (512, 4096, 4096), (600, 3000, 4096),
                                   (2048, 4096, 512), (1500, 3000, 264), (4100, 2600, 72)])
def test_gemm_tcgen05(out_dtype, M, N, K):
    """Tensor-core product at sizes that exercise every tile class (16/32/64/128 tokens swapped, one and two
    token tiles; pairs with one row of 256 x 256 tiles, with and without K ranges; 128 x 256 tiles), tails in M, N and K, split-K, and the persistent kernel with one, two and
    several tiles per block."""
    from spyinfer_b200 import kernels
    torch.manual_seed(M * 7 + N)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    status = kernels.status_word(DEV)
    kernels.gemm_tcgen05(a, w, out)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    ref = a.float() @ w.float().t()
    assert torch.isfinite(out.float()).all()
    if out_dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=2e-4)
    else:
        torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), rtol=1.6e-2, atol=2e-3)
    if 1 < M <= 16:
        one = torch.empty(1, N, device=DEV, dtype=out_dtype)
        kernels.gemm_tcgen05(a[M - 1:M].contiguous(), w, one)
        assert torch.equal(one[0], out[M - 1])      # within a tile class a row does not depend on the batch


@pytest.mark.parametrize("K", [4096, 5120])
def test_gemm_tcgen05_output_head_at_its_real_size(K):
    """The output head of the benchmark shapes: 151,936 rows (1,187 tiles of 128, no multiple of 256)
    by 4,096 or 5,120, 32-bit logits, at every class of the number of wanted rows: one, a decoding
    batch of 8 and of 64, a few hundred, and a whole prompt of 2,048."""
    from spyinfer_b200 import kernels
    N = 151936
    torch.manual_seed(K)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    w32 = w.float()
    status = kernels.status_word(DEV)
    for M in (1, 8, 64, 300, 2048):
        a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
        out = torch.full((M, N), float("nan"), device=DEV, dtype=torch.float32)
        kernels.gemm_tcgen05(a, w, out)
        torch.cuda.synchronize()
        assert status[0].item() == 0
        ref = a.float() @ w32.t()
        err = (out - ref).abs().max().item()
        assert torch.isfinite(out).all() and err <= 2e-4 + 1e-4 * ref.abs().max().item(), f"M = {M}: largest error {err:.3g}"
        # the last tile (rows 151,808 to 151,935) and the first, exactly where a tail in N would go wrong
        torch.testing.assert_close(out[:, -128:], ref[:, -128:], rtol=1e-4, atol=2e-4)
        del out, ref


def test_a_wait_that_nothing_ends_gives_up_reports_and_leaves_the_engine_usable(tiny_models):
    """The tensor-core kernels wait on barriers with a time limit.  Here a barrier that nothing ever
    arrives at is waited on with a limit of one millisecond: the kernel returns by itself, the status
    word says so, the step function raises, and the engine generates as before afterwards."""
    import time

    from spyinfer_b200 import LLMEngine, SamplingParams, kernels
    from spyinfer_b200.engine import StepError
    folder, cfg, _ = tiny_models["d"]
    engine = LLMEngine(folder, dtype="bfloat16", max_num_seqs=2, max_model_len=64, num_kvcache_blocks=8, max_num_batched_tokens=64)
    sp = SamplingParams(max_new_tokens=4, ignore_eos=True)
    before = engine.generate([[5, 6, 7]], sp)
    t0 = time.perf_counter()
    waited = kernels.wait_selftest(1_000_000, engine.runner.stager.status)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert 1_000_000 <= waited < 50_000_000, f"the wait took {waited} ns against a limit of 1 ms"
    with pytest.raises(StepError, match="gave up.*time limit"):
        engine.runner.check_status()
    engine.runner.check_status()                          # the word is clear again
    assert engine.generate([[5, 6, 7]], sp) == before
    with pytest.raises(kernels.KernelError):
        kernels.wait_selftest(10**9)                      # limits above 100 ms are refused


def test_gemm_tcgen05_finds_one_large_product():
    """One input element and one weight element are made large: exactly one output element
    must stand out, wherever in K the pair lies (start of a 64-block, its end, the K tail)."""
    from spyinfer_b200 import kernels
    M, N, K = 70, 260, 328
    for k in (0, 63, 64, 127, 320, 327):
        a = torch.zeros(M, K, device=DEV, dtype=torch.bfloat16)
        w = torch.zeros(N, K, device=DEV, dtype=torch.bfloat16)
        a[69, k], w[259, k] = 3.0, 5.0
        out = torch.empty(M, N, device=DEV, dtype=torch.float32)
        kernels.gemm_tcgen05(a, w, out)
        want = torch.zeros(M, N, device=DEV)
        want[69, 259] = 15.0
        assert torch.equal(out, want), f"k = {k}"


def test_gemm_tcgen05_refuses_unaligned_k():
    from spyinfer_b200 import kernels
    a = torch.zeros(4, 60, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(8, 60, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(kernels.KernelError):
        kernels.gemm_tcgen05(a, w, torch.empty(4, 8, device=DEV, dtype=torch.bfloat16))
    assert not kernels.tensor_core_gemm_takes(8, 60) and kernels.tensor_core_gemm_takes(8, 64)


@pytest.mark.parametrize("nh,nkv,hd,page_size,window", [(8, 2, 128, 16, None), (10, 2, 64, 16, 150), (4, 4, 128, 8, None), (16, 1, 64, 32, None),
                                                        (6, 2, 128, 5, 33)])
def test_attention_mma_tiles_mixed_batch(nh, nkv, hd, page_size, window):
    """Tensor-core attention, tiles mode: portions, single tokens and a one-token sequence in
    one batch, group sizes 1, 3, 4, 5 and 16, page sizes that are no power of two."""
    from spyinfer_b200 import kernels
    torch.manual_seed(nh * hd)
    lens = [1, 70, 333, 129, 40]
    pages, bt, ks, vs = paged_setup(5, lens, nkv, hd, page_size, torch.bfloat16)
    # seq0 its only token; seq1 a portion of 23 tokens in the middle; seq2 its last token; seq3 two tokens across key 128; seq4 whole
    toks = [(0, 0)] + [(1, p) for p in range(30, 53)] + [(2, 332)] + [(3, 127), (3, 128)] + [(4, p) for p in range(40)]
    T = len(toks)
    q = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).to(torch.bfloat16)
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, 1, 24, 25, 27, 67], dtype=torch.int32, device=DEV)
    out = torch.full((T, nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    kernels.attention_mma(q, nh, hd, out, pages, bt, positions, q_start, 5, scale, window=window)
    torch.cuda.synchronize()
    assert kernels.status_word(DEV)[0].item() == 0
    for i, (s, p) in enumerate(toks):
        ref = ref_attention(q[i, :nh * hd].view(nh, hd), ks[s], vs[s], p, scale, window)
        torch.testing.assert_close(out[i].view(nh, hd).double(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nh,nkv,hd,page_size,window,split_keys", [(32, 8, 128, 16, None, 256), (10, 2, 64, 16, 300, 64), (8, 8, 128, 8, None, 128),
                                                                   (12, 4, 64, 16, None, 512)])
def test_attention_mma_split_decode(nh, nkv, hd, page_size, window, split_keys):
    """Tensor-core attention, split mode: one token per sequence, contexts from 1 to 1500 keys
    so that rows fall into one split, two splits and many, with and without a window."""
    from spyinfer_b200 import kernels
    torch.manual_seed(nh + hd)
    lens = [1, 17, split_keys, split_keys + 1, 700, 1500]
    S = len(lens)
    pages, bt, ks, vs = paged_setup(S, lens, nkv, hd, page_size, torch.bfloat16)
    q = torch.randn(S, (nh + 2 * nkv) * hd, device=DEV).to(torch.bfloat16)
    positions = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    q_start = torch.arange(S + 1, dtype=torch.int32, device=DEV)
    out = torch.full((S, nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    max_splits = (1500 + split_keys - 1) // split_keys
    kernels.attention_mma(q, nh, hd, out, pages, bt, positions, q_start, S, scale, window=window, split_keys=split_keys, max_splits=max_splits)
    torch.cuda.synchronize()
    assert kernels.status_word(DEV)[0].item() == 0
    for i, l in enumerate(lens):
        ref = ref_attention(q[i, :nh * hd].view(nh, hd), ks[i], vs[i], l - 1, scale, window)
        torch.testing.assert_close(out[i].view(nh, hd).double(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("split_keys", [0, 128])
def test_attention_mma_finds_one_far_key(split_keys):
    """As for the plain kernel: one key among hundreds stands out and the output must be its
    value row, at page and split edges and at a window's edge, in both launch modes."""
    from spyinfer_b200 import kernels
    nh, nkv, hd, page_size, L = 4, 1, 64, 16, 700
    pages, bt, ks, vs = paged_setup(1, [L], nkv, hd, page_size, torch.bfloat16)
    q = torch.randn(1, nh * hd, device=DEV).to(torch.bfloat16)
    pos = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    out = torch.empty(1, nh * hd, device=DEV, dtype=torch.bfloat16)
    for window, far in [(None, 0), (None, 15), (None, 16), (None, 127), (None, 128), (None, 511), (None, 699), (300, L - 300), (300, L - 301)]:
        pg = pages.clone()
        page, slot = int(bt[0, far // page_size]), far % page_size
        pg[page, 0, 0, slot] = (60.0 * q[0, :hd].float() / q[0, :hd].float().norm()).to(torch.bfloat16)
        kernels.attention_mma(q, nh, hd, out, pg, bt, pos, q_start, 1, 1.0, window=window, split_keys=split_keys, max_splits=6 if split_keys else 0)
        hit = torch.allclose(out[0, :hd].float(), vs[0][far, 0].float(), atol=2e-2)
        inside = window is None or far > L - 1 - window
        assert hit == inside, f"window {window}, far key {far}: expected {'a hit' if inside else 'no hit'}"


@pytest.mark.parametrize("M,N,K,epilogue,out_dtype", [
    (2048, 4096, 4096, None, torch.bfloat16),        # 128 tiles of 256 x 256 on 74 clusters: 54 tail tiles (the o projection at 2,048 tokens)
    (2048, 6144, 4096, None, torch.float32),         # 192 tiles: 44 tail tiles
    (1500, 5000, 1032, None, torch.bfloat16),        # tails in M, N and K as well: 6 x 20 tiles, 17 K blocks with 8 columns in the last
    (2048, 5120, 8192, None, torch.bfloat16),        # 160 tiles: 12 tail tiles of 128 K blocks, shared by default (the o projection of the 32B shape)
    (1200, 6400, 2048, "swiglu", torch.bfloat16),    # 5 x 25 tiles with the SwiGLU epilogue on the summed tile
    (2048, 3328, 2048, None, torch.float32),         # 104 tiles: 30 tail tiles, two main clusters a tile and 14 helpers with three turns each
])
def test_gemm_tcgen05_shares_the_last_round_of_tiles(M, N, K, epilogue, out_dtype, monkeypatch):
    """Many tokens on pairs of blocks: when the last round of 256 x 256 tiles would leave clusters idle,
    the K blocks of its tiles are shared out over all clusters and the partial tiles are summed by the
    block that arrives last.  The result is the one of whole tiles (same products, sums in K order),
    against a 32-bit reference, twice in a row (the arrival counters return to zero by themselves).
    The threshold that keeps small products on whole tiles is lowered to zero for the test."""
    from spyinfer_b200 import kernels
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    status = kernels.status_word(DEV)
    n_out = N // 2 if epilogue else N
    if epilogue:
        g, u = a.float() @ w[0::2].float().t(), a.float() @ w[1::2].float().t()
        ref = (g / (1 + torch.exp(-g))) * u
    else:
        ref = a.float() @ w.float().t()
    outs = []
    monkeypatch.setenv("SPYINFER_GEMM_TAIL_MIN", "0")
    for tail in ("1", "1", "0"):
        monkeypatch.setenv("SPYINFER_GEMM_TAIL", tail)
        out = torch.full((M, n_out), float("nan"), device=DEV, dtype=out_dtype)
        kernels.gemm_tcgen05(a, w, out, epilogue=epilogue)
        torch.cuda.synchronize()
        assert status[0].item() == 0 and torch.isfinite(out.float()).all()
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    if out_dtype == torch.float32:
        torch.testing.assert_close(outs[0], ref, rtol=1e-4, atol=3e-4)
        torch.testing.assert_close(outs[0], outs[2], rtol=1e-4, atol=2e-4)       # other order of the 32-bit sums over K
    else:
        torch.testing.assert_close(outs[0].float(), ref.to(torch.bfloat16).float(), rtol=1.6e-2, atol=4e-3)
        assert (outs[0].float() - outs[2].float()).abs().max().item() <= 2.0 ** -6 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("M,I,K", [(3, 100, 64), (16, 328, 200), (40, 1000, 136), (64, 6144, 512), (70, 520, 264), (128, 12288, 1024), (130, 520, 264), (300, 12288, 1024),
                                   (520, 1000, 136), (1100, 2304, 512)])   # 512 rows and more: pairs of blocks on 256 x 256 tiles
def test_gemm_tcgen05_swiglu_epilogue(M, I, K):
    """Gate and up rows interleaved in the weight; the product's epilogue applies SwiGLU."""
    from spyinfer_b200 import kernels
    torch.manual_seed(M + I)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    gate = (torch.randn(I, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    up = (torch.randn(I, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()
    out = kernels.gemm_tcgen05(a, w, epilogue="swiglu")
    assert out.shape == (M, I) and out.dtype == torch.bfloat16
    g, u = a.float() @ gate.float().t(), a.float() @ up.float().t()
    ref = (g / (1 + torch.exp(-g))) * u
    torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), rtol=1.6e-2, atol=2e-3)


@pytest.mark.parametrize("M,N,K,epilogue", [(200, 512, 4096, None), (65, 256, 64, None), (130, 4096, 4096, None), (640, 4096, 4096, "swiglu"),
                                              (1000, 1280, 12288, None), (2048, 4096, 4096, None), (300, 776, 1096, "swiglu")])
def test_gemm_tcgen05_shares_k_blocks_evenly(M, N, K, epilogue, monkeypatch):
    """Many tokens on single blocks (pairs switched off): the K blocks of all tiles are shared out
    evenly over the SMs, tiles that straddle two blocks are summed through the workspace; the result
    is the product, twice in a row (the flags have to come back to zero) and the same both times."""
    from spyinfer_b200 import kernels
    monkeypatch.setenv("SPYINFER_GEMM_PAIRS", "0")
    torch.manual_seed(M + N)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    ref = a.float() @ w.float().t()
    if epilogue == "swiglu":
        g, u = ref[:, 0::2], ref[:, 1::2]
        ref = ((g / (1 + torch.exp(-g))) * u).to(torch.bfloat16).float()
        outs = [kernels.gemm_tcgen05(a, w, epilogue="swiglu").float() for _ in range(2)]
        tol = dict(rtol=1.6e-2, atol=2e-3)
    else:
        outs = [kernels.gemm_tcgen05(a, w, out_dtype=torch.float32) for _ in range(2)]
        tol = dict(rtol=1e-4, atol=3e-4)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    torch.testing.assert_close(outs[0], ref, **tol)


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (24, 1024, 2048), (64, 384, 12288), (100, 4096, 4096), (128, 1024, 12288),
                                   (512, 4096, 4096), (600, 3000, 4096), (700, 1500, 12288)])
def test_gemm_tcgen05_deferred_reduction(M, N, K):
    """With defer=True a split-K product hands back its partial products; their sum is the product.  The last three
    are 512 tokens and more with too few 256 x 256 tiles for the pairs of blocks: K is cut into two to four ranges
    (32 tiles x 2, 36 x 2 with tails in both directions, 18 x 4)."""
    from spyinfer_b200 import kernels
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    stack = kernels.gemm_tcgen05(a, w, defer=True)
    assert stack.dim() == 3 and stack.shape[1:] == (M, N) and stack.dtype == torch.float32 and stack.shape[0] > 1
    direct = kernels.gemm_tcgen05(a, w, out_dtype=torch.float32)
    acc = stack[0].clone()
    for s in range(1, stack.shape[0]):
        acc += stack[s]
    assert torch.equal(acc, direct)          # the reduce kernel adds the splits in the same order
    torch.testing.assert_close(direct, a.float() @ w.float().t(), rtol=1e-4, atol=2e-4)
    # the fused consumers: rmsnorm adds the stack to the residual, qk_rope_store sums it on the way
    x = torch.randn(M, N, device=DEV)
    wn = torch.ones(N, device=DEV, dtype=torch.bfloat16)
    out1, out2 = torch.empty(M, N, device=DEV, dtype=torch.bfloat16), torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    x1, x2 = x.clone(), x.clone()
    kernels.rmsnorm(x1, wn, 1e-6, out1, delta=stack, write_back=True)
    kernels.rmsnorm(x2, wn, 1e-6, out2, delta=direct, write_back=True)
    torch.testing.assert_close(x1, x2, rtol=2e-6, atol=2e-6)     # x + (s0 + s1 + ...) against ((x + s0) + s1) + ...: one rounding apart
    torch.testing.assert_close(out1.float(), out2.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("hd,splits", [(64, 3), (128, 3), (128, 7)])
def test_qk_rope_store_sums_a_stack_of_partial_products(hd, splits):
    """A stack of float partial products gives what their sum gives: to the bit through the general
    kernel (head_dim 64), to one bfloat16 rounding through the register path of head_dim 128, whose
    sum of squares runs in another order."""
    from spyinfer_b200 import kernels
    nh, nkv, page_size, T = 4, 2, 16, 9
    width = (nh + 2 * nkv) * hd
    stack = torch.randn(splits, T, width, device=DEV)
    total = stack[0].clone()
    for s in range(1, splits):
        total += stack[s]
    qw = (1 + 0.1 * torch.randn(hd, device=DEV)).to(torch.bfloat16)
    kw = (1 + 0.1 * torch.randn(hd, device=DEV)).to(torch.bfloat16)
    inv = torch.pow(torch.tensor(10000.0), -torch.arange(hd // 2, dtype=torch.float32) / (hd // 2)).to(DEV)
    table = kernels.build_rope_table(inv, 64)
    positions = torch.arange(5, 5 + T, dtype=torch.int32, device=DEV)
    seq_of = torch.zeros(T, dtype=torch.int32, device=DEV)
    bt = torch.tensor([[2, 0, 1]], dtype=torch.int32, device=DEV)
    pages_a = torch.zeros(3, 2, nkv, page_size, hd, device=DEV, dtype=torch.bfloat16)
    pages_b = torch.zeros_like(pages_a)
    q_a = torch.empty(T, nh * hd, device=DEV, dtype=torch.bfloat16)
    kernels.qk_rope_store(stack, nh, nkv, hd, qw, kw, 1e-6, table, positions, seq_of, bt, pages_a, q_out=q_a)
    plain = total.clone()                                            # float32 in place
    kernels.qk_rope_store(plain, nh, nkv, hd, qw, kw, 1e-6, table, positions, seq_of, bt, pages_b)
    exact = dict(rtol=0, atol=0) if hd == 64 else dict(rtol=1e-2, atol=1e-3)
    torch.testing.assert_close(q_a.float(), plain[:, :nh * hd].to(torch.bfloat16).float(), **exact)
    torch.testing.assert_close(pages_a.float(), pages_b.float(), **exact)
    with pytest.raises(kernels.KernelError):
        kernels.qk_rope_store(stack, nh, nkv, hd, qw, kw, 1e-6, table, positions, seq_of, bt, pages_a)    # a stack cannot be rotated in place


@pytest.mark.parametrize("stacked", [False, True])
@pytest.mark.parametrize("nh,nkv", [(8, 2), (6, 1)])
def test_qk_rope_store_many_tokens_at_once_equal_few_at_a_time(stacked, nh, nkv):
    """A long prompt portion through the register paths of head size 128 gives bit for bit what the same
    tokens give in small portions; 1001 tokens so that the last block has warps without an item.
    Portions of 64 tokens and more of a bfloat16 array take the kernel with four heads a half warp,
    portions of 40 the one with one head (which the test above holds against the plain formulas); with
    6 query heads and one key/value head a group of four holds queries, the key and the value."""
    from spyinfer_b200 import kernels
    torch.manual_seed(5)
    hd, page_size, T = 128, 16, 1001
    width = (nh + 2 * nkv) * hd
    src = torch.randn(3, T, width, device=DEV) if stacked else torch.randn(T, width, device=DEV).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(hd, device=DEV)).to(torch.bfloat16)
    kw = (1 + 0.1 * torch.randn(hd, device=DEV)).to(torch.bfloat16)
    inv = torch.pow(torch.tensor(10000.0), -torch.arange(hd // 2, dtype=torch.float32) / (hd // 2)).to(DEV)
    table = kernels.build_rope_table(inv, T + 8)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    seq_of = torch.zeros(T, dtype=torch.int32, device=DEV)
    n_pages = (T + page_size - 1) // page_size
    bt = torch.randperm(n_pages).to(torch.int32).view(1, n_pages).to(DEV)
    outs = []
    for step in (T, 100, 40):
        pages = torch.zeros(n_pages, 2, nkv, page_size, hd, device=DEV, dtype=torch.bfloat16)
        q = torch.empty(T, nh * hd, device=DEV, dtype=torch.bfloat16)
        for a in range(0, T, step):
            b = min(T, a + step)
            part = src[:, a:b].contiguous() if stacked else src[a:b].clone()
            q[a:b] = kernels.qk_rope_store(part, nh, nkv, hd, qw, kw, 1e-6, table, positions[a:b].contiguous(), seq_of[a:b].contiguous(), bt, pages,
                                           q_out=torch.empty(b - a, nh * hd, device=DEV, dtype=torch.bfloat16) if stacked else None)[:, :nh * hd]
        outs.append((q, pages))
    assert kernels.status_word(DEV)[0].item() == 0
    for other in outs[1:]:
        assert torch.equal(outs[0][0], other[0]) and torch.equal(outs[0][1], other[1])
    assert outs[0][1].float().abs().sum() > 0


@pytest.mark.parametrize("nh,nkv,hd,page_size,window", [(8, 2, 128, 16, None), (10, 2, 64, 16, 150), (4, 4, 128, 8, None), (16, 1, 64, 32, None),
                                                        (6, 2, 128, 64, 33), (32, 8, 128, 16, None), (2, 1, 64, 128, None),
                                                        (6, 2, 96, 16, None), (4, 1, 80, 8, 100), (8, 4, 24, 16, None), (3, 3, 112, 32, 260), (2, 2, 8, 16, None)])
def test_attention_tc_mixed_batch(nh, nkv, hd, page_size, window):
    """tcgen05 attention: portions, single tokens, a one-token sequence and a 300-token portion
    (several 128-row blocks and several key tiles) in one batch; group sizes 1, 3, 4, 5, 16; head sizes
    that fill a tile of 64 or 128 columns and head sizes that are padded to one (8 ... 112)."""
    from spyinfer_b200 import kernels
    torch.manual_seed(nh * hd + 1)
    lens = [1, 70, 333, 129, 40, 700]
    pages, bt, ks, vs = paged_setup(6, lens, nkv, hd, page_size, torch.bfloat16)
    toks = ([(0, 0)] + [(1, p) for p in range(30, 53)] + [(2, 332)] + [(3, 127), (3, 128)] + [(4, p) for p in range(40)]
            + [(5, p) for p in range(400, 700)])
    T = len(toks)
    q = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).to(torch.bfloat16)
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, 1, 24, 25, 27, 67, 367], dtype=torch.int32, device=DEV)
    out = torch.full((T, nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    kernels.attention_tc(q, nh, hd, out, pages, bt, positions, q_start, 6, scale, window=window)
    torch.cuda.synchronize()
    assert kernels.status_word(DEV)[0].item() == 0
    assert torch.isfinite(out.float()).all()
    for i, (s, p) in enumerate(toks):
        if s == 5 and i % 7:          # check every 7th row of the long portion, and its first and last rows
            if i not in (67, T - 1):
                continue
        ref = ref_attention(q[i, :nh * hd].view(nh, hd), ks[s], vs[s], p, scale, window)
        torch.testing.assert_close(out[i].view(nh, hd).double(), ref, rtol=2e-2, atol=2e-2)


def test_attention_tc_blocks_of_one_query_tile_behind_blocks_of_two():
    """A mixed step as serving has them: two decoded tokens with long contexts beside a prompt of 1,400 tokens, at
    the 8B head counts.  There are more work items than SMs, so some blocks take a second item, and for some
    of them that item is a decoded token's: a block of rows whose second query tile is empty, with many key
    tiles, behind an item that used both tiles.  The idle half of the block then runs ahead of the working one."""
    from spyinfer_b200 import kernels
    torch.manual_seed(5)
    nh, nkv, hd, page_size = 32, 8, 128, 16
    lens = [1500, 700, 1400]
    pages, bt, ks, vs = paged_setup(3, lens, nkv, hd, page_size, torch.bfloat16)
    toks = [(0, 1499), (1, 699)] + [(2, p) for p in range(1400)]
    T = len(toks)
    q = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).to(torch.bfloat16)
    positions = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, 1, 2, T], dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    for _ in range(2):
        out = torch.full((T, nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
        kernels.attention_tc(q, nh, hd, out, pages, bt, positions, q_start, 3, scale)
        torch.cuda.synchronize()
        assert kernels.status_word(DEV)[0].item() == 0
        assert torch.isfinite(out.float()).all()
        for i in [0, 1, 2, 3, 65, 66, 129, 130] + list(range(97, T, 97)) + [T - 1]:
            s_, p_ = toks[i]
            ref = ref_attention(q[i, :nh * hd].view(nh, hd), ks[s_], vs[s_], p_, scale, None)
            torch.testing.assert_close(out[i].view(nh, hd).double(), ref, rtol=2e-2, atol=2e-2)


def test_attention_tc_refuses_pages_that_are_no_tma_box():
    from spyinfer_b200 import kernels
    pages, bt, ks, vs = paged_setup(1, [20], 1, 64, 5, torch.bfloat16)
    q = torch.zeros(1, 4 * 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(kernels.KernelError):
        kernels.attention_tc(q, 4, 64, torch.empty_like(q), pages, bt, torch.tensor([19], dtype=torch.int32, device=DEV),
                             torch.tensor([0, 1], dtype=torch.int32, device=DEV), 1, 1.0)


def test_attention_tc_finds_one_far_key_and_survives_large_scores():
    """One key stands out by a large score in a late tile (the running maximum jumps by far more
    than the rescale threshold after earlier tiles have accumulated): the output must be that
    key's value row; positions at tile and page edges, and a window's edge."""
    from spyinfer_b200 import kernels
    nh, nkv, hd, page_size, L = 4, 1, 64, 16, 700
    pages, bt, ks, vs = paged_setup(1, [L], nkv, hd, page_size, torch.bfloat16)
    q = torch.randn(1, nh * hd, device=DEV).to(torch.bfloat16)
    pos = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    out = torch.empty(1, nh * hd, device=DEV, dtype=torch.bfloat16)
    for window, far in [(None, 0), (None, 15), (None, 127), (None, 128), (None, 511), (None, 699), (300, L - 300), (300, L - 301)]:
        pg = pages.clone()
        page, slot = int(bt[0, far // page_size]), far % page_size
        pg[page, 0, 0, slot] = (60.0 * q[0, :hd].float() / q[0, :hd].float().norm()).to(torch.bfloat16)
        kernels.attention_tc(q, nh, hd, out, pg, bt, pos, q_start, 1, 1.0, window=window)
        hit = torch.allclose(out[0, :hd].float(), vs[0][far, 0].float(), atol=2e-2)
        inside = window is None or far > L - 1 - window
        assert hit == inside, f"window {window}, far key {far}: expected {'a hit' if inside else 'no hit'}"


@pytest.mark.parametrize("share", ["auto", "split", "whole"])
@pytest.mark.parametrize("nh,nkv,hd,page_size,window", [(32, 8, 128, 16, None), (10, 2, 64, 16, 300), (8, 8, 128, 8, None), (12, 4, 64, 32, None),
                                                        (16, 1, 128, 16, 700), (6, 1, 128, 128, None), (8, 2, 128, 64, 130),
                                                        (12, 4, 96, 16, None), (5, 5, 80, 8, 200), (4, 2, 40, 16, None), (2, 1, 8, 32, None)])
def test_attention_decode_contexts_from_one_key_to_thousands(nh, nkv, hd, page_size, window, share):
    """Persistent tcgen05 decode attention: one token per sequence, contexts at tile edges (127, 128,
    129 keys) and long ones, so that pairs are written whole by one block, cut over two blocks and over
    many; group sizes 1, 3, 4, 5, 6 and 16; with and without a window; head sizes that fill a tile of 64 or
    128 columns and head sizes that are padded to one."""
    from spyinfer_b200 import kernels
    torch.manual_seed(nh + hd + 5)
    lens = [1, 17, 127, 128, 129, 700, 1500, 3000]
    S = len(lens)
    pages, bt, ks, vs = paged_setup(S, lens, nkv, hd, page_size, torch.bfloat16)
    q = torch.randn(S, (nh + 2 * nkv) * hd, device=DEV).to(torch.bfloat16)
    positions = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    q_start = torch.arange(S + 1, dtype=torch.int32, device=DEV)
    out = torch.full((S, nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    kernels.attention_decode(q, nh, hd, out, pages, bt, positions, q_start, S, scale, window=window, share=share)
    torch.cuda.synchronize()
    assert kernels.status_word(DEV)[0].item() == 0
    for i, l in enumerate(lens):
        ref = ref_attention(q[i, :nh * hd].view(nh, hd), ks[i], vs[i], l - 1, scale, window)
        torch.testing.assert_close(out[i].view(nh, hd).double(), ref, rtol=2e-2, atol=2e-2)


def test_attention_decode_many_short_sequences():
    """More (sequence, kv head) pairs than blocks: every block walks several whole pairs and the
    borders of its share fall inside pairs; queries of up to four segments are in flight."""
    from spyinfer_b200 import kernels
    torch.manual_seed(11)
    nh, nkv, hd, page_size = 8, 2, 128, 16
    lens = [int(x) for x in torch.randint(1, 400, (150,))] + [128, 256, 1, 2]
    S = len(lens)
    pages, bt, ks, vs = paged_setup(S, lens, nkv, hd, page_size, torch.bfloat16)
    q = torch.randn(S, nh * hd, device=DEV).to(torch.bfloat16)
    positions = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    q_start = torch.arange(S + 1, dtype=torch.int32, device=DEV)
    out = torch.full((S, nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    for share in ("split", "whole", "auto"):   # several times: stale shared memory and scratch of an earlier run must not matter
        out.fill_(float("nan"))
        kernels.attention_decode(q, nh, hd, out, pages, bt, positions, q_start, S, scale, share=share)
    torch.cuda.synchronize()
    assert kernels.status_word(DEV)[0].item() == 0
    for i, l in enumerate(lens):
        ref = ref_attention(q[i].view(nh, hd), ks[i], vs[i], l - 1, scale, None)
        torch.testing.assert_close(out[i].view(nh, hd).double(), ref, rtol=2e-2, atol=2e-2)


def test_attention_decode_finds_one_far_key_and_survives_large_scores():
    """One key stands out by a large score (the running maximum jumps by far more than the rescale
    threshold after earlier tiles have accumulated): the output must be that key's value row; keys at
    tile and page edges, in the first and the last block of the pair, and at a window's edge."""
    from spyinfer_b200 import kernels
    nh, nkv, hd, page_size, L = 4, 1, 64, 16, 2000
    pages, bt, ks, vs = paged_setup(1, [L], nkv, hd, page_size, torch.bfloat16)
    q = torch.randn(1, nh * hd, device=DEV).to(torch.bfloat16)
    pos = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    out = torch.empty(1, nh * hd, device=DEV, dtype=torch.bfloat16)
    for window, far in [(None, 0), (None, 15), (None, 127), (None, 128), (None, 511), (None, 1999), (300, L - 300), (300, L - 301)]:
        pg = pages.clone()
        page, slot = int(bt[0, far // page_size]), far % page_size
        pg[page, 0, 0, slot] = (60.0 * q[0, :hd].float() / q[0, :hd].float().norm()).to(torch.bfloat16)
        kernels.attention_decode(q, nh, hd, out, pg, bt, pos, q_start, 1, 1.0, window=window)
        hit = torch.allclose(out[0, :hd].float(), vs[0][far, 0].float(), atol=2e-2)
        inside = window is None or far > L - 1 - window
        assert hit == inside, f"window {window}, far key {far}: expected {'a hit' if inside else 'no hit'}"
    # one sequence on a single block: a large score in a late tile after earlier tiles have accumulated
    nkv2, L2 = 1, 640
    S = 160   # enough other pairs that the long pair lies within one block's share
    lens = [L2] + [100] * (S - 1)
    pages, bt, ks, vs = paged_setup(S, lens, nkv2, hd, page_size, torch.bfloat16)
    q = torch.randn(S, nh * hd, device=DEV).to(torch.bfloat16)
    far = 600
    page, slot = int(bt[0, far // page_size]), far % page_size
    pages[page, 0, 0, slot] = (60.0 * q[0, :hd].float() / q[0, :hd].float().norm()).to(torch.bfloat16)
    out = torch.empty(S, nh * hd, device=DEV, dtype=torch.bfloat16)
    kernels.attention_decode(q, nh, hd, out, pages, bt, torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV),
                             torch.arange(S + 1, dtype=torch.int32, device=DEV), S, 1.0)
    assert torch.allclose(out[0, :hd].float(), vs[0][far, 0].float(), atol=2e-2)


def test_attention_decode_reports_bad_pages_and_positions_and_refuses_odd_pages():
    from spyinfer_b200 import kernels
    nh, nkv, hd, page_size = 4, 2, 64, 16
    pages, bt, ks, vs = paged_setup(2, [40, 300], nkv, hd, page_size, torch.bfloat16)
    q = torch.randn(2, nh * hd, device=DEV).to(torch.bfloat16)
    q_start = torch.arange(3, dtype=torch.int32, device=DEV)
    out = torch.zeros(2, nh * hd, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    bad = bt.clone()
    bad[1, 3] = pages.shape[0] + 7   # a page beyond the pool: skipped and reported
    kernels.attention_decode(q, nh, hd, out, pages, bad, torch.tensor([39, 299], dtype=torch.int32, device=DEV), q_start, 2, 1.0, status=status)
    assert status.tolist() == [3, 1]
    status.zero_()
    kernels.attention_decode(q, nh, hd, out, pages, bt, torch.tensor([39, bt.shape[1] * page_size], dtype=torch.int32, device=DEV), q_start, 2, 1.0,
                             status=status)
    assert status.tolist() == [2, 1]
    pages5, bt5, _, _ = paged_setup(1, [20], 1, 64, 5, torch.bfloat16)
    with pytest.raises(kernels.KernelError):
        kernels.attention_decode(q[:1], 4, 64, out[:1], pages5, bt5, torch.tensor([19], dtype=torch.int32, device=DEV), q_start[:2], 1, 1.0)
