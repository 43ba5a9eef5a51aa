"""Each kernel alone against its plain statement (tests/kernel_refs.py), in float32 and bfloat16, at
sizes other than the test models': widths and vocabularies that are no power of two, every head
size class, odd numbers of heads and groups, page edges, windows, and inputs made so that a single
wrong key, page or row shows."""

import math

import numpy as np
import pytest
import torch

import kernel_refs as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from tokasaurus_b200.kernels import ops as o
    return o


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-2)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,V", [(80, 509), (2048, 1000), (8, 3)])
def test_embed_gather(ops, dtype, H, V):
    g = torch.Generator(device="cpu").manual_seed(1)
    table = torch.randn(V, H, generator=g).to(dtype).to(DEV)
    ids = i32([0, V - 1, -1, 1 % V, -1, 2 % V])
    token_seq = i32([0, 0, 1, 2, 2, -1])  # the last row is padding
    seq_slot = i32([3, 1, 0])
    last = i32([2 % V, V - 1, 7, 1 % V])
    x = torch.full((6, H), 5.0, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed_gather(table, ids, token_seq, seq_slot, last, x, status)
    want = torch.stack([table[0], table[V - 1], table[int(last[1])], table[1 % V], table[int(last[0])],
                        torch.zeros(H, device=DEV, dtype=dtype)]).float()
    assert torch.equal(x, want) and int(status) == 0
    ops.embed_gather(table, i32([V, 0, 0, 0, 0, 0]), token_seq, seq_slot, last, x, status)
    assert int(status) & 1 and torch.equal(x[0], torch.zeros(H, device=DEV))  # refused, not read out of range


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,H,eps", [(5, 96, 1e-6), (3, 2048, 1e-5), (7, 4000, 1e-2), (1, 17, 1e-5), (2, 16384, 1e-5),
                                          (3, 10240, 1e-5)])
def test_add_rmsnorm(ops, dtype, rows, H, eps):
    g = torch.Generator().manual_seed(rows * H)
    x = (torch.randn(rows, H, generator=g) * 3).to(DEV)
    delta = torch.randn(rows, H, generator=g).to(dtype).to(DEV)
    w = (torch.rand(H, generator=g) + 0.5).to(DEV)
    for d in (delta, None):
        x1, x2 = x.clone(), x.clone()
        out = torch.empty(rows, H, dtype=dtype, device=DEV)
        want = torch.empty(rows, H, dtype=dtype, device=DEV)
        ops.add_rmsnorm(x1, d, w, eps, out)
        ref.add_rmsnorm(x2, d, w, eps, want)
        assert torch.equal(x1, x2)  # the residual sum is a float32 add
        torch.testing.assert_close(out.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,I", [(4, 160), (3, 8192), (9, 37)])
def test_silu_mul(ops, dtype, rows, I):
    gu = (torch.randn(rows, 2 * I, generator=torch.Generator().manual_seed(I)) * 4).to(dtype).to(DEV)
    out = torch.empty(rows, I, dtype=dtype, device=DEV)
    want = torch.empty_like(out)
    ops.silu_mul(gu, out)
    ref.silu_mul(gu, want)
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gather_rows(ops, dtype):
    for width in (96, 2048, 3):
        src = torch.randn(11, width).to(dtype).to(DEV)
        rows = i32([10, 0, 3, 3])
        out = torch.empty(4, width, dtype=dtype, device=DEV)
        ops.gather_rows(src, rows, out)
        assert torch.equal(out, src[rows.long()])


@pytest.mark.parametrize("M,N,K", [(1, 509, 96), (5, 64, 64), (64, 64, 16), (65, 129, 33), (130, 70, 257),
                                   (3, 2048, 8192), (200, 3, 7)])
def test_sgemm_true_fp32(ops, M, N, K):
    g = torch.Generator().manual_seed(M * N + K)
    a = torch.randn(M, K, generator=g).to(DEV)
    w = torch.randn(N, K, generator=g).to(DEV)
    out = torch.empty(M, N, device=DEV)
    ops.sgemm_tn(a, w, out)
    want = (a.double() @ w.double().T)
    err = (out.double() - want).abs().max().item()
    bound = 4 * K * 2 ** -24 * (a.abs().double() @ w.abs().double().T).max().item()
    assert err <= bound, (err, bound)
    # far inside what a 10-bit (tf32) or 8-bit (bfloat16) mantissa could give
    assert err < 2e-5 * math.sqrt(K) * 3
    # a row's result does not depend on the other rows of the batch
    if M > 1:
        one = torch.empty(1, N, device=DEV)
        ops.sgemm_tn(a[M - 1:M].contiguous(), w, one)
        assert torch.equal(one[0], out[M - 1])


def make_paged(dtype, n_seqs, lens, nkv, hd, ps, n_pages, seed, fill=1e3):
    """Random keys/values scattered over shuffled pages; unused slots hold large garbage."""
    g = torch.Generator().manual_seed(seed)
    kc = torch.full((n_pages, nkv, ps, hd), fill, dtype=dtype)
    vc = torch.full((n_pages, nkv, ps, hd), -fill, dtype=dtype)
    perm = torch.randperm(n_pages, generator=g).tolist()
    indptr, pages, K, V = [0], [], [], []
    for L in lens:
        npg = -(-L // ps)
        mine = [perm.pop() for _ in range(npg)]
        k = torch.randn(L, nkv, hd, generator=g).to(dtype)
        v = torch.randn(L, nkv, hd, generator=g).to(dtype)
        for j in range(L):
            kc[mine[j // ps], :, j % ps] = k[j]
            vc[mine[j // ps], :, j % ps] = v[j]
        pages += mine
        indptr.append(len(pages))
        K.append(k)
        V.append(v)
    return kc.to(DEV), vc.to(DEV), i32(indptr), i32(pages), K, V


def plain_attention(q, K, V, pos, scale, window):
    """float64 softmax attention of one query [nh, hd] at position pos over K, V [L, nkv, hd]."""
    nh, hd = q.shape
    nkv = K.shape[1]
    lo = max(0, pos - window + 1) if window else 0
    k = K[lo:pos + 1].double().repeat_interleave(nh // nkv, dim=1)
    v = V[lo:pos + 1].double().repeat_interleave(nh // nkv, dim=1)
    s = torch.einsum("hd,khd->hk", q.double(), k) * scale
    return torch.einsum("hk,khd->hd", torch.softmax(s, -1), v)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,nh,nkv,ps,window", [(16, 4, 2, 16, None), (32, 3, 1, 8, None), (48, 6, 3, 4, 7),
                                                  (64, 8, 2, 16, None), (80, 5, 5, 16, 33), (128, 8, 1, 32, None),
                                                  (256, 2, 1, 16, None), (112, 7, 1, 5, None)])
def test_attention_mixed_batch(ops, dtype, hd, nh, nkv, ps, window):
    """Three requests in one batch: a whole prompt, a portion in the middle of a request that ends
    just past a page edge, and a single decoded token far into its request."""
    lens = [37, 2 * ps + 1, 150]
    kc, vc, indptr, pages, K, V = make_paged(dtype, 3, lens, nkv, hd, ps, 64, seed=hd + nh)
    q_pos = [list(range(37)), list(range(ps - 1, 2 * ps + 1)), [149]]
    token_seq = i32([s for s, p in enumerate(q_pos) for _ in p])
    positions = i32([x for p in q_pos for x in p])
    T = token_seq.numel()
    g = torch.Generator().manual_seed(7)
    q = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype).to(DEV)
    scale = 1 / math.sqrt(hd)
    out = torch.zeros(T, nh * hd, dtype=dtype, device=DEV)
    ops.attn_paged(q, q.shape[1], out, kc, vc, token_seq, positions, indptr, pages, None, T, nh, nkv, hd, ps, scale,
                   window)
    t = 0
    for s, ps_ in enumerate(q_pos):
        for p in ps_:
            want = plain_attention(q[t, : nh * hd].view(nh, hd).cpu(), K[s], V[s], p, scale, window)
            torch.testing.assert_close(out[t].view(nh, hd).cpu().double(), want, **tol(dtype), check_dtype=False)
            t += 1
    # wanted rows only
    rows = i32([T - 1, 0, 40])
    some = torch.zeros(3, nh * hd, dtype=dtype, device=DEV)
    ops.attn_paged(q, q.shape[1], some, kc, vc, token_seq, positions, indptr, pages, rows, 3, nh, nkv, hd, ps, scale,
                   window)
    assert torch.equal(some, out[rows.long()])


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(ops, dtype):
    """One key among 700 is made to stand out for one query head: the output must be that key's
    value, wherever it lies (first slot of a page, last slot, the first key, the query's own)."""
    hd, nh, nkv, ps, L = 64, 4, 2, 16, 700
    for target in (0, 15, 16, 333, 687, 699):
        kc, vc, indptr, pages, K, V = make_paged(dtype, 1, [L], nkv, hd, ps, 50, seed=target)
        q = torch.zeros(1, (nh + 2 * nkv) * hd, dtype=dtype)
        direction = K[0][target, 1].float()
        q[0, 3 * hd:4 * hd] = (direction / direction.norm() * 60).to(dtype)  # head 3 reads kv head 1
        scale = 1.0
        out = torch.zeros(1, nh * hd, dtype=dtype, device=DEV)
        ops.attn_paged(q.to(DEV), q.shape[1], out, kc, vc, i32([0]), i32([L - 1]), indptr, pages, None, 1, nh, nkv, hd,
                       ps, scale, None)
        want = plain_attention(q[0, : nh * hd].view(nh, hd), K[0], V[0], L - 1, scale, None)
        assert (want[3] - V[0][target, 1].double()).abs().max() < 0.05  # the construction works
        torch.testing.assert_close(out[0].view(nh, hd).cpu().double(), want, **tol(dtype), check_dtype=False)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(ops, dtype):
    """The key just outside the window is made huge: it must not be seen; the one just inside must."""
    hd, nh, nkv, ps, L, W = 32, 2, 1, 8, 100, 24
    kc, vc, indptr, pages, K, V = make_paged(dtype, 1, [L], nkv, hd, ps, 20, seed=5)
    p = L - 1
    q = torch.randn(1, (nh + 2) * hd, generator=torch.Generator().manual_seed(2)).to(dtype)
    scale = 1 / math.sqrt(hd)
    for edge, seen in ((p - W, False), (p - W + 1, True)):
        k2 = [K[0].clone()]
        k2[0][edge, 0] = (q[0, :hd].float() * 30).to(dtype)
        kc2 = kc.clone()
        page = int(pages[edge // ps])
        kc2[page, 0, edge % ps] = k2[0][edge, 0].to(DEV)
        out = torch.zeros(1, nh * hd, dtype=dtype, device=DEV)
        ops.attn_paged(q.to(DEV), q.shape[1], out, kc2, vc, i32([0]), i32([p]), indptr, pages, None, 1, nh, nkv, hd, ps,
                       scale, W)
        want = plain_attention(q[0, : nh * hd].view(nh, hd), k2[0], V[0], p, scale, W)
        torch.testing.assert_close(out[0].view(nh, hd).cpu().double(), want, **tol(dtype), check_dtype=False)
        hit = (out[0, :hd].cpu().double() - V[0][edge, 0].double()).abs().max() < 0.05
        assert bool(hit) == seen


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,rot,nh,nkv,ps", [(16, 16, 4, 2, 16), (32, 32, 3, 1, 8), (64, 64, 8, 2, 16), (128, 64, 2, 2, 4),
                                              (48, 0, 2, 1, 16)])
def test_rope_kv_write(ops, dtype, hd, rot, nh, nkv, ps):
    from tokasaurus_b200.parts.rope import RotaryEncoding

    T = 9
    g = torch.Generator().manual_seed(hd)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype).to(DEV)
    positions = i32([0, 1, ps - 1, ps, 5000, 131071, 3, 7, 2])
    token_seq = i32([0, 0, 0, 0, 1, 2, -1, 3, 3])
    n_pages = 131072 // ps + 8
    tables = {0: [5, 6], 1: list(range(10, 10 + 5000 // ps + 1)), 2: [0] * (131071 // ps) + [7],
              3: list(range(n_pages - 8, n_pages - 8 + 7 // ps + 1))}
    indptr, pages = [0], []
    for s in range(4):
        pages += tables[s]
        indptr.append(len(pages))
    inv = RotaryEncoding(rot, 500000.0, "llama3", 32.0, 1.0, 4.0, 8192).inv_freq().to(DEV) if rot else None
    kc = torch.zeros(n_pages, nkv, ps, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    kc2, vc2 = kc.clone(), vc.clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    a, b = qkv.clone(), qkv.clone()
    ops.rope_kv_write(a, positions, token_seq, i32(indptr), i32(pages), inv, kc, vc, nh, nkv, hd, rot, ps, True, status)
    ref.rope_kv_write(b, positions, token_seq, i32(indptr), i32(pages), inv, kc2, vc2, nh, nkv, hd, rot, ps, True,
                      torch.zeros(1, dtype=torch.int32))
    assert int(status) == 0
    t = dict(rtol=1e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(a.float(), b.float(), **t)
    torch.testing.assert_close(kc.float(), kc2.float(), **t)
    assert torch.equal(vc, vc2)
    assert torch.equal(a[6], qkv[6])  # padding row untouched
    # write_cache=False rotates q and leaves the cache alone
    kc3 = torch.zeros_like(kc)
    c = qkv.clone()
    ops.rope_kv_write(c, positions, token_seq, i32(indptr), i32(pages), inv, kc3, vc.clone(), nh, nkv, hd, rot, ps, False,
                      status)
    assert torch.equal(c[:, : nh * hd], a[:, : nh * hd]) and not kc3.any()
    # a page id outside the pool is refused
    ops.rope_kv_write(qkv.clone(), positions, token_seq, i32(indptr), i32([n_pages + 3] * len(pages)), inv, kc3, vc.clone(),
                      nh, nkv, hd, rot, ps, True, status)
    assert int(status) & 2 and not kc3.any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,rot,nh,nkv,ps", [(16, 16, 4, 2, 16), (64, 64, 6, 2, 16), (128, 64, 2, 1, 8), (48, 32, 3, 3, 4)])
def test_rope_kv_write_with_the_elementwise_stage(ops, dtype, hd, rot, nh, nkv, ps):
    """Biases on q|k|v and an RMS norm of every q and k head before the rotation, alone and together, many tokens a
    block (more tokens than blocks the GPU holds would take too long here: the walk over tokens is the same)."""
    from tokasaurus_b200.parts.rope import RotaryEncoding

    T, n_pages = 300, 128
    g = torch.Generator().manual_seed(hd + nh)
    C = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, C, generator=g).to(dtype).to(DEV)
    bias = (torch.randn(C, generator=g) * 0.5).to(DEV)
    qk_norm = (torch.rand(2, hd, generator=g) + 0.5).to(DEV)
    positions = i32(list(range(T)))
    token_seq = i32([0 if t % 7 else -1 for t in range(T)])  # every seventh row is padding
    pages = torch.randperm(n_pages, generator=g).tolist()[: -(-T // ps)]
    inv = RotaryEncoding(rot, 10000.0).inv_freq().to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for b, n in ((bias, None), (None, qk_norm), (bias, qk_norm)):
        kc = torch.zeros(n_pages, nkv, ps, hd, dtype=dtype, device=DEV)
        vc, kc2 = torch.zeros_like(kc), torch.zeros_like(kc)
        vc2 = torch.zeros_like(kc)
        a, want = qkv.clone(), qkv.clone()
        ops.rope_kv_write(a, positions, token_seq, i32([0, len(pages)]), i32(pages), inv, kc, vc, nh, nkv, hd, rot, ps, True,
                          status, bias=b, qk_norm=n, norm_eps=1e-6)
        ref.rope_kv_write(want, positions, token_seq, i32([0, len(pages)]), i32(pages), inv, kc2, vc2, nh, nkv, hd, rot, ps,
                          True, torch.zeros(1, dtype=torch.int32), bias=b, qk_norm=n, norm_eps=1e-6)
        assert int(status) == 0
        t = dict(rtol=1e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)
        torch.testing.assert_close(a[:, : nh * hd].float(), want[:, : nh * hd].float(), **t)
        torch.testing.assert_close(kc.float(), kc2.float(), **t)
        torch.testing.assert_close(vc.float(), vc2.float(), **t)
        assert torch.equal(a[0], qkv[0])  # a padding row is untouched


def test_sampling_greedy_and_logprob(ops):
    for V in (509, 128256, 3):
        g = torch.Generator().manual_seed(V)
        logits = (torch.randn(5, V, generator=g) * 3).to(DEV)
        logits[1, V - 1] = 50.0
        logits[2, 0] = logits[2].max() + 1
        logits[3] = 0.25  # all equal: the first index wins
        ids = torch.full((5,), -1, dtype=torch.int32, device=DEV)
        lp = torch.zeros(5, device=DEV)
        last = torch.full((8,), -1, dtype=torch.int32, device=DEV)
        ops.sample(logits, torch.zeros(5, device=DEV), None, None, i32([4, -1, 0, 1, 2]), ids, lp, last)
        assert ids.tolist() == logits.argmax(-1).tolist() or V == 3
        assert int(ids[1]) == V - 1 and int(ids[2]) == 0 and int(ids[3]) == 0
        want_lp = torch.log_softmax(logits.double(), -1).gather(1, ids.long().view(-1, 1)).view(-1)
        torch.testing.assert_close(lp.double(), want_lp, rtol=1e-5, atol=1e-5)
        assert last.tolist() == [int(ids[2]), int(ids[3]), int(ids[4]), -1, int(ids[0]), -1, -1, -1]


@pytest.mark.parametrize("V", [1003, 150001])
def test_sampling_matches_plain_gumbel_draw(ops, V):
    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(6, V, generator=g) * 2).to(DEV)
    temp = torch.tensor([0.7, 1.0, 0.0, 1.5, 0.7, 0.7], device=DEV)
    keys = torch.tensor([11, -5, 3, 2**62, 11, 12], dtype=torch.int64, device=DEV)
    pos = i32([4, 4, 4, 100000, 5, 4])
    ids = torch.zeros(6, dtype=torch.int32, device=DEV)
    lp = torch.zeros(6, device=DEV)
    ops.sample(logits, temp, keys, pos, None, ids, lp, None)
    want_ids = torch.zeros(6, dtype=torch.int32)
    want_lp = torch.zeros(6)
    ref.sample(logits.cpu(), temp.cpu(), keys.cpu(), pos.cpu(), None, want_ids, want_lp, None)
    for r in range(6):
        if int(ids[r]) != int(want_ids[r]):  # only a near tie of the perturbed scores may differ
            T = float(temp[r]) or 1.0
            noise = ref.gumbel_noise(V, int(keys[r]) & (2**64 - 1), int(pos[r]))
            sc = logits[r].double().cpu().numpy() / T + noise
            assert abs(sc[int(ids[r])] - sc.max()) < 1e-4
    torch.testing.assert_close(lp.cpu(), want_lp, rtol=1e-4, atol=1e-4)
    # same key and position: the same draw whatever the row; another position or key: another stream
    again = torch.zeros(6, dtype=torch.int32, device=DEV)
    order = torch.tensor([5, 4, 3, 2, 1, 0], device=DEV)
    ops.sample(logits[order].contiguous(), temp[order].contiguous(), keys[order].contiguous(), pos[order].contiguous(), None, again, None, None)
    assert again.tolist() == ids[order].tolist()


def test_sampling_noise_at_the_extremes_of_the_random_bits(ops):
    """All bits set must not round the uniform number up to 1 (Gumbel value +inf: that entry would win whatever
    its logit), no bit set must not give 0; the kernel's float32 uniform equals the plain statement bit for bit."""
    patterns = np.array([0xFFFFFFFF, 0xFFFFFE00, 0xFFFFFDFF, 0, 1, 0x1FF, 0x200, 0x80000000, 0x7FFFFFFF, 12345678],
                        dtype=np.uint32)
    rnd = np.random.default_rng(0).integers(0, 2**32, size=4096, dtype=np.uint64).astype(np.uint32)
    bits = np.concatenate([patterns, rnd])
    u, gum = ops.noise_of_bits(torch.from_numpy(bits.view(np.int32)).to(DEV))
    u, gum = u.cpu().numpy(), gum.cpu().numpy()
    assert (u > 0).all() and (u < 1).all() and np.isfinite(gum).all()
    want = ref.uniform_open(bits)
    assert want.dtype == np.float32 and np.array_equal(u, want)
    np.testing.assert_allclose(gum, -np.log(-np.log(want.astype(np.float64))), rtol=2e-5, atol=2e-6)
    # a row whose every entry but one is far ahead: the far-behind entry never wins, whatever the noise can be
    assert gum.max() < 17 and gum.min() > -3


def test_sampling_follows_the_distribution(ops):
    """20,000 draws from a 7-way distribution at T = 0.8: chi-square against softmax(logits / T)."""
    V, N, T = 7, 20000, 0.8
    logits = torch.tensor([1.0, 0.2, -0.5, 2.0, 0.0, -3.0, 1.5], device=DEV).repeat(N, 1).contiguous()
    ids = torch.zeros(N, dtype=torch.int32, device=DEV)
    ops.sample(logits, torch.full((N,), T, device=DEV), torch.arange(N, dtype=torch.int64, device=DEV) * 7919 + 13,
               torch.zeros(N, dtype=torch.int32, device=DEV), None, ids, None, None)
    counts = torch.bincount(ids.long().cpu(), minlength=V).double()
    p = torch.softmax(logits[0].double().cpu() / T, -1)
    chi2 = (((counts - N * p) ** 2) / (N * p)).sum().item()
    assert chi2 < 24.1  # 99.95 % point of chi-square with 6 degrees of freedom


def test_topk_logprobs(ops):
    V, k = 509, 5
    logits = (torch.randn(4, V, generator=torch.Generator().manual_seed(9)) * 2).to(DEV)
    logits[2, 10] = logits[2, 20] = logits[2].max() + 1  # a tie: the smaller index first
    temp = torch.tensor([0.0, 0.5, 1.0, 2.0], device=DEV)
    idx = torch.zeros(4, k, dtype=torch.int32, device=DEV)
    lp = torch.zeros(4, k, device=DEV)
    ops.topk_logprobs(logits, temp, k, idx, lp)
    widx, wlp = torch.zeros(4, k, dtype=torch.int32), torch.zeros(4, k)
    ref.topk_logprobs(logits.cpu(), temp.cpu(), k, widx, wlp)
    assert torch.equal(idx.cpu(), widx)
    torch.testing.assert_close(lp.cpu(), wlp, rtol=1e-4, atol=1e-4)


def test_refusals(ops):
    with pytest.raises(ops.KernelError, match="multiples of 16"):
        ops.check_head_dim(24)
    with pytest.raises(ops.KernelError, match="CUDA"):
        ops.silu_mul(torch.zeros(2, 4), torch.zeros(2, 2))
    with pytest.raises(ops.KernelError):
        ops.sgemm_tn(torch.zeros(2, 4, device=DEV), torch.zeros(3, 5, device=DEV), torch.zeros(2, 3, device=DEV))
    with pytest.raises(ops.KernelError):
        ops.add_rmsnorm(torch.zeros(2, 4, device=DEV, dtype=torch.bfloat16), None, torch.ones(4, device=DEV), 1e-5,
                        torch.zeros(2, 4, device=DEV))


# ------------------------------------------------------------------------------------------------
# bfloat16 tensor-core attention (split-key kernel for single tokens, tiled kernel for portions)
def run_mma_attention(ops, lens_q, lens_kv, nh, nkv, hd, ps, window, seed, n_pages=None, fill=1e3, merged=True,
                      tc=False, single_heads=False):
    """A batch of requests with lens_q new tokens each at the end of lens_kv keys; returns (got, want)."""
    from types import SimpleNamespace
    from tokasaurus_b200.parts.attention import plan_attention

    dtype = torch.bfloat16
    n_pages = n_pages or sum(-(-L // ps) for L in lens_kv) + 7
    kc, vc, indptr, pages, K, V = make_paged(dtype, len(lens_kv), lens_kv, nkv, hd, ps, n_pages, seed=seed, fill=fill)
    q_start, pos, tseq = [], [], []
    for s, (n, kv) in enumerate(zip(lens_q, lens_kv)):
        q_start.append(len(pos))
        pos += list(range(kv - n, kv))
        tseq += [s] * n
    T = len(pos)
    host = SimpleNamespace(seq_q_len=np.asarray(lens_q, dtype=np.int32), seq_kv_len=np.asarray(lens_kv, dtype=np.int32))
    plan = plan_attention(host, window, query_tile=128 if tc else 64)
    g = torch.Generator().manual_seed(seed + 1)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype).to(DEV)
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    c = i32(plan["counts"])
    scale = 1 / math.sqrt(hd)
    n_items, n_dec, n_tiles = (int(x) for x in plan["counts"][:3])
    if n_dec:
        ops.attn_decode_mma(qkv, kc, vc, i32(q_start), i32(lens_kv), indptr, pages, i32(plan["items"]), c[0:1], n_items,
                            i32(plan["dec_seqs"]), i32(plan["dec_item_start"]), c[1:2], n_dec, out, nh, nkv, hd, ps, scale,
                            window, item_entry=i32(plan["item_entry"]) if merged else None)
    if n_tiles and tc:
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.attn_prefill_tc(qkv, out, kc, vc, i32(q_start), i32(lens_q), i32(lens_kv), indptr, pages, i32(plan["tiles"]),
                            c[2:3], n_tiles, nh, nkv, hd, ps, scale, window, status, single_heads=single_heads)
        assert int(status.item()) == 0
    elif n_tiles:
        ops.attn_prefill_mma(qkv, out, kc, vc, i32(q_start), i32(lens_q), i32(lens_kv), indptr, pages, i32(plan["tiles"]),
                             c[2:3], n_tiles, nh, nkv, hd, ps, scale, window)
    want = torch.zeros(T, nh, hd, dtype=torch.float64)
    for t in range(T):
        s = tseq[t]
        want[t] = plain_attention(qkv[t, : nh * hd].view(nh, hd).cpu(), K[s], V[s], pos[t], scale, window)
    return out.view(T, nh, hd).cpu().double(), want


@pytest.mark.parametrize("hd,nh,nkv,ps,window", [(64, 32, 8, 16, None), (16, 4, 2, 16, None), (32, 3, 1, 8, None),
                                                  (128, 8, 1, 32, None), (48, 6, 3, 4, 300), (80, 5, 5, 16, None),
                                                  (256, 2, 1, 16, None), (112, 34, 2, 5, None), (64, 4, 4, 64, 17)])
def test_mma_attention_mixed_batch(ops, hd, nh, nkv, ps, window):
    """Single tokens at short, page-edge and long contexts (several splits) beside portions that
    start in the middle of a request, span several 64-query tiles and end on odd lengths."""
    lens_q = [1, 1, 1, 1, 70, 2, 130, 1, 64]
    lens_kv = [1, 2 * ps, 2 * ps + 1, 777, 70, 259, 400, 256, 64]
    got, want = run_mma_attention(ops, lens_q, lens_kv, nh, nkv, hd, ps, window, seed=hd + nh)
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got, want, rtol=1.6e-2, atol=1.2e-2)
    # merge of the splits by a second kernel instead of inside the attention kernel: the same sums in the same order
    got2, _ = run_mma_attention(ops, lens_q, lens_kv, nh, nkv, hd, ps, window, seed=hd + nh, merged=False)
    assert torch.equal(got, got2)
    # and again: the arrival counters must have been left at zero
    got3, _ = run_mma_attention(ops, lens_q, lens_kv, nh, nkv, hd, ps, window, seed=hd + nh)
    assert torch.equal(got, got3)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("nh,nkv,ps,window", [(32, 8, 16, None), (3, 1, 8, None), (5, 5, 5, None), (4, 2, 64, 17),
                                              (6, 3, 4, 300), (8, 2, 16, 128), (4, 2, 256, None), (2, 1, 128, 200)])
def test_tc_attention_mixed_batch(ops, hd, nh, nkv, ps, window):
    """The tcgen05 kernels for portions (head sizes 64 and 128): portions that start in the middle of a request,
    span several 128-query tiles and several key tiles, end on odd lengths, or are two tokens long."""
    lens_q = [1, 70, 2, 130, 1, 64, 128, 300, 129]
    lens_kv = [777, 70, 259, 400, 256, 64, 128, 1000, 129]
    got, want = run_mma_attention(ops, lens_q, lens_kv, nh, nkv, hd, ps, window, seed=nh + ps, tc=True)
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got, want, rtol=1.6e-2, atol=1.2e-2)
    got2, _ = run_mma_attention(ops, lens_q, lens_kv, nh, nkv, hd, ps, window, seed=nh + ps, tc=True)
    assert torch.equal(got, got2)
    # one head a block instead of two (what a step with few query tiles asks for): the same arithmetic a head
    got3, _ = run_mma_attention(ops, lens_q, lens_kv, nh, nkv, hd, ps, window, seed=nh + ps, tc=True, single_heads=True)
    assert not torch.isnan(got3).any()
    torch.testing.assert_close(got3, want, rtol=1.6e-2, atol=1.2e-2)
    torch.testing.assert_close(got3.float(), got.float(), rtol=0, atol=2e-2 * want.abs().max().item())


@pytest.mark.parametrize("hd", [64, 128])
def test_tc_attention_never_reads_what_a_page_held_before(ops, hd):
    got, want = run_mma_attention(ops, [1, 37, 150], [100, 37, 333], 8, 2, hd, 16, None, seed=3, fill=float("nan"), tc=True)
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got, want, rtol=1.6e-2, atol=1.2e-2)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("slope", [0.02, 0.4, -0.4])
def test_tc_attention_with_scores_that_grow_along_the_keys(ops, hd, slope):
    """Keys whose scores rise (or fall) steadily with their position: the running reference of a row's
    exponentials has to move again and again, late in the row as well as early (the kernel that keeps its output
    in tensor memory rescales it only then), or never after the first tile."""
    from types import SimpleNamespace
    from tokasaurus_b200.parts.attention import plan_attention

    nh, nkv, ps, L, n = 4, 2, 16, 1100, 900
    kc, vc, indptr, pages, K, V = make_paged(torch.bfloat16, 1, [L], nkv, hd, ps, 90, seed=11)
    # every key gets a component along e_0 that grows with its position; queries have e_0 = 1 / scale
    table = pages.cpu().tolist()
    ramp = (torch.arange(L, dtype=torch.float32) * slope).to(torch.bfloat16)
    for i in range(L):
        kc[table[i // ps], :, i % ps, 0] = ramp[i].to(DEV)
        K[0][i, :, 0] = ramp[i]
    g = torch.Generator().manual_seed(5)
    qkv = (torch.randn(n, (nh + 2 * nkv) * hd, generator=g) * 0.5).to(torch.bfloat16)
    scale = 1 / math.sqrt(hd)
    qkv[:, 0:nh * hd:hd] = 1.0 / scale
    plan = plan_attention(SimpleNamespace(seq_q_len=np.asarray([n], dtype=np.int32), seq_kv_len=np.asarray([L], dtype=np.int32)),
                          None, query_tile=128)
    out = torch.zeros(n, nh * hd, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    c = i32(plan["counts"])
    ops.attn_prefill_tc(qkv.to(DEV), out, kc, vc, i32([0]), i32([n]), i32([L]), indptr, pages, i32(plan["tiles"]), c[2:3],
                        int(plan["counts"][2]), nh, nkv, hd, ps, scale, None, status)
    assert int(status.item()) == 0
    want = torch.zeros(n, nh, hd, dtype=torch.float64)
    for t in range(n):
        want[t] = plain_attention(qkv[t, : nh * hd].view(nh, hd), K[0], V[0], L - n + t, scale, None)
    torch.testing.assert_close(out.view(n, nh, hd).cpu().double(), want, rtol=1.6e-2, atol=1.2e-2)


def test_mma_attention_finds_one_far_key(ops):
    """One key among 1,500 stands out for one query head of a single-token request; and the same
    for the last query of a long portion.  The output must be that key's value."""
    nh, nkv, ps, L = 8, 2, 16, 1500
    for target in (0, 255, 256, 257, 1023, 1499):
        for lens_q in ([1], [200], [-200], [-200, 128]):
            hd = lens_q[1] if len(lens_q) > 1 else 64
            tc, lens_q = lens_q[0] < 0, [abs(lens_q[0])]
            kc, vc, indptr, pages, K, V = make_paged(torch.bfloat16, 1, [L], nkv, hd, ps, 100, seed=target)
            from types import SimpleNamespace
            from tokasaurus_b200.parts.attention import plan_attention
            n = lens_q[0]
            plan = plan_attention(SimpleNamespace(seq_q_len=np.asarray(lens_q, dtype=np.int32),
                                                  seq_kv_len=np.asarray([L], dtype=np.int32)), None,
                                  query_tile=128 if tc else 64)
            qkv = torch.zeros(n, (nh + 2 * nkv) * hd, dtype=torch.bfloat16)
            direction = K[0][target, 1].float()
            qkv[n - 1, 6 * hd:7 * hd] = (direction / direction.norm() * 60).to(torch.bfloat16)  # head 6 reads kv head 1
            out = torch.zeros(n, nh * hd, dtype=torch.bfloat16, device=DEV)
            c = i32(plan["counts"])
            if n == 1:
                ops.attn_decode_mma(qkv.to(DEV), kc, vc, i32([0]), i32([L]), indptr, pages, i32(plan["items"]), c[0:1],
                                    int(plan["counts"][0]), i32(plan["dec_seqs"]), i32(plan["dec_item_start"]), c[1:2], 1,
                                    out, nh, nkv, hd, ps, 1.0, None)
            elif tc:
                ops.attn_prefill_tc(qkv.to(DEV), out, kc, vc, i32([0]), i32(lens_q), i32([L]), indptr, pages,
                                    i32(plan["tiles"]), c[2:3], int(plan["counts"][2]), nh, nkv, hd, ps, 1.0, None,
                                    torch.zeros(1, dtype=torch.int32, device=DEV))
            else:
                ops.attn_prefill_mma(qkv.to(DEV), out, kc, vc, i32([0]), i32(lens_q), i32([L]), indptr, pages,
                                     i32(plan["tiles"]), c[2:3], int(plan["counts"][2]), nh, nkv, hd, ps, 1.0, None)
            got = out[n - 1].view(nh, hd)[6].cpu().double()
            assert (got - V[0][target, 1].double()).abs().max() < 0.06, (target, n)


def test_mma_attention_never_reads_what_a_page_held_before(ops):
    """Slots of the last page beyond the request's length hold NaN: nothing of them may show."""
    got, want = run_mma_attention(ops, [1, 37], [100, 37], 8, 2, 64, 16, None, seed=3, fill=float("nan"))
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got, want, rtol=1.6e-2, atol=1.2e-2)
    # long requests, whose whole tiles come by TMA and whose last tile is gathered; one ends on a tile's edge
    for hd, ps in ((64, 16), (128, 8), (128, 64), (64, 128)):
        got, want = run_mma_attention(ops, [1, 1, 1], [1000, 640, 333], 8, 2, hd, ps, None, seed=4, fill=float("nan"))
        assert not torch.isnan(got).any()
        torch.testing.assert_close(got, want, rtol=1.6e-2, atol=1.2e-2)


# ------------------------------------------------------------------------------------------------
# small-batch matrix products (K-split, float32 slices) and their consumers
@pytest.mark.parametrize("M,N,K", [(1, 3072, 2048), (8, 2048, 8192), (3, 509, 96), (17, 130, 160), (33, 64, 64),
                                   (64, 2048, 2048), (5, 128256, 2048), (2, 72, 8)])
def test_linear_smallm(ops, M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    for max_slices in (8, 1):
        parts = ops.linear_smallm(a, w, max_slices)
        assert parts.shape[1:] == (M, N) and parts.dtype == torch.float32 and (max_slices > 1 or parts.shape[0] == 1)
        want = a.double() @ w.double().T
        got = parts.double().sum(0)
        scale = (a.abs().double() @ w.abs().double().T).max().item()
        assert (got - want).abs().max().item() <= 2e-6 * scale * math.sqrt(K) + 1e-6, (parts.shape[0],)
    # a row does not depend on the others in the batch
    if M > 1:
        alone = ops.linear_smallm(a[M - 1:M].contiguous(), w, 8)
        torch.testing.assert_close(alone.sum(0)[0], ops.linear_smallm(a, w, 8).sum(0)[M - 1], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("M,I,K", [(1, 8192, 2048), (8, 160, 96), (20, 72, 64), (64, 256, 128)])
def test_linear_smallm_gated(ops, M, I, K):
    g = torch.Generator().manual_seed(M + I)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    up = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    w = ops.interleave_gate_up(gate, up)
    assert torch.equal(w[0:8], gate[0:8]) and torch.equal(w[8:16], up[0:8]) and torch.equal(w[16:24], gate[8:16])
    got = ops.linear_smallm_gated(a, w)
    want = torch.nn.functional.silu(a.double() @ gate.double().T) * (a.double() @ up.double().T)
    torch.testing.assert_close(got.double(), want, rtol=1.6e-2, atol=2e-3 * want.abs().max().item())
    # the unfused route over the same interleaved weights
    gu = ops.linear(a, w)
    act = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    ops.silu_mul(gu, act, 8)
    torch.testing.assert_close(act.double(), want, rtol=3e-2, atol=1e-2 * want.abs().max().item())


def test_partial_sums_reach_norm_and_rope(ops):
    from tokasaurus_b200.parts.rope import RotaryEncoding

    g = torch.Generator().manual_seed(4)
    rows, H = 5, 96
    x = torch.randn(rows, H, generator=g).to(DEV)
    parts = torch.randn(3, rows, H, generator=g).to(DEV)
    w = (torch.rand(H, generator=g) + 0.5).to(DEV)
    x1, x2 = x.clone(), x.clone()
    out = torch.empty(rows, H, dtype=torch.bfloat16, device=DEV)
    want = torch.empty_like(out)
    ops.add_rmsnorm(x1, parts, w, 1e-5, out)
    ref.add_rmsnorm(x2, parts, w, 1e-5, want)
    torch.testing.assert_close(x1, x2, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out.float(), want.float(), rtol=1.6e-2, atol=1e-2)
    # rope from slices equals rope from their bfloat16 sum
    nh, nkv, hd, ps = 6, 2, 48, 8
    C = (nh + 2 * nkv) * hd
    T = 4
    qparts = torch.randn(2, T, C, generator=g).to(DEV)
    qkv = qparts.sum(0).to(torch.bfloat16)
    positions, token_seq = i32([0, 9, 10, 300]), i32([0, 0, 0, 1])
    indptr, pages = i32([0, 2, 40]), i32(list(range(5, 7)) + list(range(10, 48)))
    inv = RotaryEncoding(hd, 10000.0).inv_freq().to(DEV)
    kc, vc = (torch.zeros(64, nkv, ps, hd, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    kc2, vc2 = kc.clone(), vc.clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    q_out = torch.empty(T, nh * hd, dtype=torch.bfloat16, device=DEV)
    ops.rope_kv_write_partials(qparts, q_out, positions, token_seq, indptr, pages, inv, kc, vc, nh, nkv, hd, hd, ps, True, status)
    ops.rope_kv_write(qkv, positions, token_seq, indptr, pages, inv, kc2, vc2, nh, nkv, hd, hd, ps, True, status)
    assert int(status) == 0
    torch.testing.assert_close(q_out.float(), qkv[:, : nh * hd].float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(kc.float(), kc2.float(), rtol=1e-2, atol=1e-2)
    assert torch.equal(vc, vc2)


# ------------------------------------------------------------------------------------------------
# fused products for at most 16 rows
@pytest.mark.parametrize("M,N,K", [(1, 3072, 2048), (8, 2048, 8192), (3, 509, 96), (16, 130, 160), (9, 64, 1024),
                                   (5, 128256, 2048), (2, 72, 8), (7, 40, 3000)])
def test_linear_decode_store_and_add(ops, M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    want = a.double() @ w.double().T
    scale = (a.abs().double() @ w.abs().double().T).max().item()
    f32 = ops.linear_decode(a, w, "f32")
    assert (f32.double() - want).abs().max().item() <= 2e-6 * scale * math.sqrt(K) + 1e-6
    b16 = ops.linear_decode(a, w, "bf16")
    torch.testing.assert_close(b16.double(), want, rtol=1e-2, atol=4e-3 * want.abs().max().item())
    x = torch.randn(M, N, generator=g).to(DEV)
    x0 = x.clone()
    ops.linear_decode(a, w, "add", out=x)
    torch.testing.assert_close(x.double(), x0.double() + want, rtol=1e-5, atol=1e-5 * max(1.0, scale))
    if M > 1:  # a row does not depend on the others
        alone = ops.linear_decode(a[M - 1:].contiguous(), w, "f32")
        assert torch.equal(alone[0], f32[M - 1])


@pytest.mark.parametrize("M,N,K,eps", [(1, 3072, 2048, 1e-5), (8, 509, 96, 1e-6), (13, 64, 160, 1e-2)])
def test_linear_decode_norm_prologue(ops, M, N, K, eps):
    g = torch.Generator().manual_seed(N)
    x = (torch.randn(M, K, generator=g) * 3).to(DEV)
    nw = (torch.rand(K, generator=g) + 0.5).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    xd = x.double()
    h = xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + eps) * nw.double()
    want = h @ w.double().T
    got = ops.linear_decode(x, w, "f32", nw, eps)
    torch.testing.assert_close(got.double(), want, rtol=1e-2, atol=6e-3 * want.abs().max().item())
    got16 = ops.linear_decode(x, w, "bf16", nw, eps)
    torch.testing.assert_close(got16.double(), want, rtol=2e-2, atol=1e-2 * want.abs().max().item())


@pytest.mark.parametrize("M,I,K", [(1, 8192, 2048), (8, 160, 96), (16, 72, 64)])
def test_linear_decode_gated(ops, M, I, K):
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, K, generator=g).to(DEV)
    nw = (torch.rand(K, generator=g) + 0.5).to(DEV)
    gate = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    up = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    w = ops.interleave_gate_up(gate, up)
    xd = x.double()
    h = xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + 1e-5) * nw.double()
    want = torch.nn.functional.silu(h @ gate.double().T) * (h @ up.double().T)
    got = ops.linear_decode(x, w, "gated", nw, 1e-5)
    assert got.shape == (M, I)
    torch.testing.assert_close(got.double(), want, rtol=2e-2, atol=1e-2 * want.abs().max().item())


@pytest.mark.parametrize("hd,nh,nkv,ps,rot,window", [(64, 32, 8, 16, 64, None), (16, 4, 2, 16, 16, None), (32, 3, 1, 8, 32, None),
                                                      (128, 8, 1, 32, 64, None), (48, 6, 3, 4, 0, 300), (80, 34, 2, 16, 80, None)])
@pytest.mark.parametrize("long_items", [False, True])
def test_fused_rope_decode_attention_equals_the_separate_kernels(ops, hd, nh, nkv, ps, rot, window, long_items):
    """``long_items``: few, long work items (their whole tiles come by TMA where the sizes allow), among them
    requests that end on a tile's edge, one key past it, and in the middle of a page."""
    from types import SimpleNamespace
    from tokasaurus_b200.parts.attention import plan_attention
    from tokasaurus_b200.parts.rope import RotaryEncoding

    lens_kv = [1600, 1024, 1025, 333, 2 * ps + 1] if long_items else [1, 2 * ps, 2 * ps + 1, 777, 256, 257, 513]
    B = len(lens_kv)
    dtype = torch.bfloat16
    n_pages = sum(-(-L // ps) for L in lens_kv) + 5
    kc, vc, indptr, pages, K, V = make_paged(dtype, B, lens_kv, nkv, hd, ps, n_pages, seed=hd)
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, generator=g).to(dtype).to(DEV)
    plan = plan_attention(SimpleNamespace(seq_q_len=np.ones(B, dtype=np.int32), seq_kv_len=np.asarray(lens_kv, dtype=np.int32)), window,
                          **(dict(slots=8 * 8) if long_items else {}))
    c = i32(plan["counts"])
    n_items, n_dec = int(plan["counts"][0]), int(plan["counts"][1])
    q_start, kv_len = i32(list(range(B))), i32(lens_kv)
    positions, token_seq = i32([L - 1 for L in lens_kv]), i32(list(range(B)))
    inv = RotaryEncoding(rot, 10000.0).inv_freq().to(DEV) if rot else None
    scale = 1 / math.sqrt(hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # separate kernels
    kc1, vc1, q1 = kc.clone(), vc.clone(), qkv.clone()
    ops.rope_kv_write(q1, positions, token_seq, indptr, pages, inv, kc1, vc1, nh, nkv, hd, rot, ps, True, status)
    want = torch.zeros(B, nh * hd, dtype=dtype, device=DEV)
    ops.attn_decode_mma(q1, kc1, vc1, q_start, kv_len, indptr, pages, i32(plan["items"]), c[0:1], n_items, i32(plan["dec_seqs"]),
                        i32(plan["dec_item_start"]), c[1:2], n_dec, want, nh, nkv, hd, ps, scale, window)
    # fused
    kc2, vc2 = kc.clone(), vc.clone()
    got = torch.zeros_like(want)
    ops.attn_decode_rope_mma(qkv, kc2, vc2, q_start, kv_len, indptr, pages, i32(plan["items"]), c[0:1], n_items,
                             i32(plan["dec_seqs"]), i32(plan["dec_item_start"]), c[1:2], n_dec, got, nh, nkv, hd, ps, scale,
                             window, inv, rot, True, status, item_entry=i32(plan["item_entry"]))
    assert int(status) == 0
    assert torch.equal(vc2, vc1)
    torch.testing.assert_close(kc2.float().nan_to_num(7.0), kc1.float().nan_to_num(7.0), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=1e-2)
    # the same rows given as three float32 slices that add up to them
    parts = torch.randn(3, *qkv.shape, generator=g).to(DEV)
    parts[2] = qkv.float() - parts[0] - parts[1]
    qsum = parts.sum(0).to(dtype)
    kc3, vc3 = kc.clone(), vc.clone()
    got3 = torch.zeros_like(want)
    ops.attn_decode_rope_mma(parts, kc3, vc3, q_start, kv_len, indptr, pages, i32(plan["items"]), c[0:1], n_items,
                             i32(plan["dec_seqs"]), i32(plan["dec_item_start"]), c[1:2], n_dec, got3, nh, nkv, hd, ps, scale,
                             window, inv, rot, True, status)
    if torch.equal(qsum, qkv):
        assert torch.equal(got3, got) and torch.equal(kc3.nan_to_num(7.0), kc2.nan_to_num(7.0))
    torch.testing.assert_close(got3.float(), want.float(), rtol=3e-2, atol=3e-2)
    # a layer call that reads another call's cache: nothing is written, the key already in the cache at the
    # token's position is the one that counts
    kc4, vc4 = kc1.clone(), vc1.clone()
    got4 = torch.zeros_like(want)
    ops.attn_decode_rope_mma(qkv, kc4, vc4, q_start, kv_len, indptr, pages, i32(plan["items"]), c[0:1], n_items,
                             i32(plan["dec_seqs"]), i32(plan["dec_item_start"]), c[1:2], n_dec, got4, nh, nkv, hd, ps, scale,
                             window, inv, rot, False, status)
    assert torch.equal(kc4.nan_to_num(7.0), kc1.nan_to_num(7.0)) and torch.equal(vc4, vc1)
    torch.testing.assert_close(got4.float(), want.float(), rtol=1.6e-2, atol=1e-2)
    # the element-wise stage before the rotation (biases, RMS norm of the q and k heads): the fused kernel against the
    # separate kernels given the same stage, from rows and from slices
    bias = (torch.randn(qkv.shape[1], generator=g) * 0.5).to(DEV)
    qk_norm = (torch.rand(2, hd, generator=g) + 0.5).to(DEV)
    stage = dict(bias=bias, qk_norm=qk_norm, norm_eps=1e-6)
    kc5, vc5, q5 = kc.clone(), vc.clone(), qkv.clone()
    ops.rope_kv_write(q5, positions, token_seq, indptr, pages, inv, kc5, vc5, nh, nkv, hd, rot, ps, True, status, **stage)
    want5 = torch.zeros_like(want)
    ops.attn_decode_mma(q5, kc5, vc5, q_start, kv_len, indptr, pages, i32(plan["items"]), c[0:1], n_items, i32(plan["dec_seqs"]),
                        i32(plan["dec_item_start"]), c[1:2], n_dec, want5, nh, nkv, hd, ps, scale, window)
    assert (want5.float() - want.float()).abs().max() > 0.05  # the stage changes the result
    for rows in (qkv, parts):
        kc6, vc6 = kc.clone(), vc.clone()
        got6 = torch.zeros_like(want)
        ops.attn_decode_rope_mma(rows, kc6, vc6, q_start, kv_len, indptr, pages, i32(plan["items"]), c[0:1], n_items,
                                 i32(plan["dec_seqs"]), i32(plan["dec_item_start"]), c[1:2], n_dec, got6, nh, nkv, hd, ps,
                                 scale, window, inv, rot, True, status, item_entry=i32(plan["item_entry"]), **stage)
        assert int(status) == 0
        torch.testing.assert_close(kc6.float().nan_to_num(7.0), kc5.float().nan_to_num(7.0), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(got6.float(), want5.float(), rtol=3e-2, atol=3e-2)


# ------------------------------------------------------------------------------------------------
# tcgen05 / TMA matrix product for many rows
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 128, 64), (256, 512, 128), (100, 300, 72), (1, 16, 8),
                                   (300, 509 * 8, 96), (2048, 3072, 2048), (130, 264, 2056), (640, 2048, 8192)])
def test_gemm_tcgen05(ops, M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.gemm_tcgen05(a, w, status)
    assert int(status) == 0
    want = a.double() @ w.double().T
    torch.testing.assert_close(out.double(), want, rtol=1e-2, atol=4e-3 * want.abs().max().item())
    # rows are independent of the batch they come in
    if M > 130:
        part = ops.gemm_tcgen05(a[128:130].contiguous(), w, status)
        assert torch.equal(part, out[128:130])


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (2048, 8192, 2048), (77, 72, 96), (300, 160, 2048)])
def test_gemm_tcgen05_gated(ops, M, I, K):
    g = torch.Generator().manual_seed(M + I)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    up = (torch.randn(I, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = ops.gemm_tcgen05(a, ops.interleave_gate_up(gate, up), status, gated=True)
    assert int(status) == 0 and got.shape == (M, I)
    want = torch.nn.functional.silu(a.double() @ gate.double().T) * (a.double() @ up.double().T)
    torch.testing.assert_close(got.double(), want, rtol=2e-2, atol=6e-3 * want.abs().max().item())


def test_gemm_tcgen05_refuses_what_tma_cannot_address(ops):
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    a = torch.zeros(4, 20, dtype=torch.bfloat16, device=DEV)  # K not a multiple of 8
    with pytest.raises(ops.KernelError):
        ops.gemm_tcgen05(a, torch.zeros(16, 20, dtype=torch.bfloat16, device=DEV), status)
    with pytest.raises(ops.KernelError):
        ops.gemm_tcgen05(torch.zeros(4, 16, device=DEV), torch.zeros(16, 16, device=DEV), status)  # float32


@pytest.mark.parametrize("M,N,K", [(8, 128, 64), (1, 256, 128), (16, 3072, 2048), (5, 509, 96), (8, 2048, 8192), (3, 130, 72),
                                   (17, 256, 128), (32, 2048, 2048), (33, 509, 96), (64, 3072, 2048), (50, 2048, 8192)])
def test_linear_tc_decode(ops, M, N, K):
    """The tcgen05 form of the small-batch product (weights on the 128-row side, TMA ring): same contract as
    linear_smallm."""
    g = torch.Generator().manual_seed(M * N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    parts = ops.linear_tc_decode(a, w, status)
    assert int(status) == 0 and parts.shape[1:] == (M, N)
    want = a.double() @ w.double().T
    scale = (a.abs().double() @ w.abs().double().T).max().item()
    assert (parts.double().sum(0) - want).abs().max().item() <= 2e-6 * scale * math.sqrt(K) + 1e-6
    if N % 16 == 0 and N >= 32:
        gate, up = w[: N // 2].contiguous(), w[N // 2:].contiguous()
        got = ops.linear_tc_decode(a, ops.interleave_gate_up(gate, up), status, gated=True)
        ref_ = torch.nn.functional.silu(a.double() @ gate.double().T) * (a.double() @ up.double().T)
        torch.testing.assert_close(got.double(), ref_, rtol=2e-2, atol=6e-3 * ref_.abs().max().item())
        assert int(status) == 0
