"""Each part alone on the GPU against the plain implementation's function for it, at sizes other
than the test models': norm, feed-forward, attention mixer (with its position encoding), block,
embedding and head; and a model whose run order names a block twice and lets a call read
another call's cache."""

import math

import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def rt(dtype):
    from tokasaurus_b200.engine.runtime import Runtime
    return Runtime(DEV, dtype)


def weights_for(part, dtype, seed=0, std=0.05):
    from tokasaurus_b200.weights import random_tensors
    host = random_tensors(part.weight_specs(), seed, std=std, norm_init="uniform")
    dev = {}
    for s in part.weight_specs():
        dev[s.name] = host[s.name].to(DEV, torch.float32 if s.role == "vector" else dtype)
    return host, dev


def context(needs, entries_spec, page_size=8, num_pages=64):
    """entries_spec: list of (request, tokens or None, start, want)."""
    from tokasaurus_b200.cache import CacheManager
    from tokasaurus_b200.engine.batch import Stager, StepContext, StepEntry, build_host_batch

    cm = context.cm if getattr(context, "reuse", False) else None
    if cm is None:
        cm = CacheManager(needs, page_size, num_pages, 8, dtype=context.dtype, device=DEV)
        context.cm = cm
        context.stager = Stager(DEV)
    entries = []
    for rid, toks, start, want in entries_spec:
        if rid not in cm.requests:
            cm.admit(rid)
        cm.ensure_capacity(rid, start + len(toks))
        entries.append(StepEntry(rid, toks, start, want))
    return StepContext(build_host_batch(entries, cm), cm, DEV, context.stager)


def tol(dtype, want=None):
    """Absolute tolerances are set against the size of the expected values: 1e-5 of the largest for
    float32, 2 % of the largest for bfloat16 (several roundings to 8 bits on the way)."""
    top = float(want.abs().max()) if want is not None else 1.0
    return dict(rtol=1e-4, atol=1e-5 * max(top, 1.0)) if dtype == torch.float32 else dict(rtol=3e-2, atol=2e-2 * max(top, 1.0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from tokasaurus_b200.parts import ResidualStream, RMSNorm

    n = RMSNorm(200, 3e-4, "n.weight")
    host, dev = weights_for(n, dtype)
    n.bind(dev, rt(dtype))
    x = torch.randn(6, 200)
    delta = torch.randn(6, 200).to(dtype)
    stream = ResidualStream(x.to(DEV), delta.to(DEV))
    out = n.forward(None, stream)
    want = plain.rms_norm(x.double() + delta.double(), host["n.weight"].double(), 3e-4)
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype, want))
    assert stream.delta is None
    torch.testing.assert_close(stream.x.cpu(), x + delta.float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from tokasaurus_b200.parts import GatedMLP

    m = GatedMLP(80, 208, "g", "u", "d")
    host, dev = weights_for(m, dtype, std=0.1)
    m.bind(dev, rt(dtype))
    h = torch.randn(7, 80).to(dtype)
    out = m.forward(None, h.to(DEV))
    if out.dim() == 3:  # few rows in bfloat16: float32 slices of a K-split product, added by the next norm
        out = out.sum(0)
    hd = h.double()
    want = (torch.nn.functional.silu(hd @ host["g"].double().T) * (hd @ host["u"].double().T)) @ host["d"].double().T
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype, want))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,scaled", [(6, 2, 48, True), (4, 4, 16, False), (5, 1, 80, True), (4, 2, 64, False),
                                                 (2, 1, 128, True)])
def test_attention_mixer_part_whole_and_cut(dtype, nh, nkv, hd, scaled):
    """The mixer alone: a whole sequence in one step equals the plain attention block's inner part;
    the same sequence cut into portions and single tokens gives the same rows."""
    from tokasaurus_b200.parts import PagedAttention, RotaryEncoding

    width = nh * hd
    pe = RotaryEncoding(hd, 500000.0, "llama3", 8.0, 1.0, 4.0, 16) if scaled else RotaryEncoding(hd, 10000.0)
    a = PagedAttention(width, nh, nkv, hd, pe, "q", "k", "v", "o")
    host, dev = weights_for(a, dtype, seed=hd, std=0.08)
    a.bind(dev, rt(dtype))
    T = 45
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(1)).to(dtype)
    # plain: projections, rotary, causal attention, output projection
    hd64 = h.double()
    q = (hd64 @ host["q"].double().T).view(T, nh, hd)
    k = (hd64 @ host["k"].double().T).view(T, nkv, hd)
    v = (hd64 @ host["v"].double().T).view(T, nkv, hd)
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=16) if scaled else None
    cos, sin = plain.rope_tables(torch.arange(T), plain.rope_inv_freq(hd, 500000.0 if scaled else 10000.0, sc))
    want = plain.causal_gqa_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v).reshape(T, -1)
    want = want @ host["o"].double().T
    context.dtype, context.reuse = dtype, False
    needs = {0: a.cache_need()}
    ctx = context(needs, [("w", list(range(T)), 0, [])])
    out = a.forward(ctx, h.to(DEV), ctx.layer_cache(0))
    out = out.sum(0) if out.dim() == 3 else out
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype, want))
    # cut: 7 + 2 + 20 + 1 + 1 + 14, a second request in between, wanted rows only at the end
    context.reuse = True
    at, got = 0, []
    for n in (7, 2, 20, 1, 1, 14):
        ctx = context(needs, [("other", [0] * 3, at // 2 * 0 + len(got) * 3, []), ("c", list(range(n)), at, [])])
        hh = torch.cat([torch.randn(3, width).to(dtype), h[at:at + n]]).to(DEV)
        rows = torch.arange(3, 3 + n, dtype=torch.int32, device=DEV)
        part = a.forward(ctx, hh, ctx.layer_cache(0), out_rows=rows)
        got.append(part.sum(0) if part.dim() == 3 else part)
        at += n
    torch.testing.assert_close(torch.cat(got).cpu().double(), want, **tol(dtype, want))
    context.reuse = False


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_head_and_block(dtype):
    from tokasaurus_b200.parts import (DecoderModel, GatedMLP, LayerCall, OutputHead, PagedAttention, PreNormBlock, RMSNorm,
                                       RotaryEncoding, TokenEmbedding)

    W, V, nh, nkv, hd, I = 96, 131, 2, 1, 48, 112
    pe = RotaryEncoding(hd, 10000.0)

    def block(i):
        return PreNormBlock(RMSNorm(W, 1e-5, f"b{i}.n1"), PagedAttention(W, nh, nkv, hd, pe, f"b{i}.q", f"b{i}.k", f"b{i}.v", f"b{i}.o"),
                            RMSNorm(W, 1e-5, f"b{i}.n2"), GatedMLP(W, I, f"b{i}.g", f"b{i}.u", f"b{i}.d"))

    # block 0 runs twice (second time on a cache entry of its own), block 1 reads the cache that call 0 wrote
    model = DecoderModel(TokenEmbedding(V, W, "emb"), [block(0), block(1)],
                         OutputHead(V, W, RMSNorm(W, 1e-5, "nf"), "emb"),
                         run_order=[LayerCall(0, cache=0), LayerCall(0, cache=1), LayerCall(1, cache=0, write_cache=False)])
    host, dev = weights_for(model, dtype, seed=3, std=0.08)
    model.bind(dev, rt(dtype))
    T = 21
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(4)).tolist()
    w = {k: t.double() for k, t in host.items()}

    def plain_block(x, i, k_from=None):
        h = plain.rms_norm(x, w[f"b{i}.n1"], 1e-5)
        q = (h @ w[f"b{i}.q"].T).view(T, nh, hd)
        k = (h @ w[f"b{i}.k"].T).view(T, nkv, hd)
        v = (h @ w[f"b{i}.v"].T).view(T, nkv, hd)
        cos, sin = plain.rope_tables(torch.arange(T), plain.rope_inv_freq(hd, 10000.0, None))
        q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
        if k_from is not None:
            k, v = k_from
        x = x + plain.causal_gqa_attention(q, k, v).reshape(T, -1) @ w[f"b{i}.o"].T
        h = plain.rms_norm(x, w[f"b{i}.n2"], 1e-5)
        x = x + (torch.nn.functional.silu(h @ w[f"b{i}.g"].T) * (h @ w[f"b{i}.u"].T)) @ w[f"b{i}.d"].T
        return x, (k, v)

    x = w["emb"][torch.tensor(ids)]
    x, kv0 = plain_block(x, 0)
    x, _ = plain_block(x, 0)
    x, _ = plain_block(x, 1, k_from=kv0)
    want = plain.rms_norm(x, w["nf"], 1e-5) @ w["emb"].T

    context.dtype, context.reuse = dtype, False
    needs = model.cache_entries()
    assert set(needs) == {0, 1}
    ctx = context(needs, [("a", ids, 0, list(range(T)))])
    logits = model.forward(ctx)
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.cpu().double(), want, **tol(dtype, want))
    # in two steps, wanting only some rows
    context.reuse = True
    ctx = context(needs, [("b", ids[:13], 0, [12])])
    l1 = model.forward(ctx)
    ctx = context(needs, [("b", ids[13:], 13, [0, 7])])
    l2 = model.forward(ctx)
    torch.testing.assert_close(torch.cat([l1, l2]).cpu().double(), want[[12, 13, 20]], **tol(dtype, want))
    context.reuse = False
