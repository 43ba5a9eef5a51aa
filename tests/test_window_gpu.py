"""Windowed attention through the whole engine.  A toy architecture, defined here and registered without a change to
the framework's files, runs the framework's paged attention with a window in every block (a query sees its own key
and the ``window - 1`` before it): one model with heads of 16 (FP32-pipe and mma.sync kernels) and one with heads of
64 (tcgen05 portions, split-key decode with whole tiles by TMA).  The window is no multiple of the page size, prompts
are longer than the window, and the cache manager gives pages back behind the window, so block tables hold -1, the
cached table arrays are dropped, and released pages go to other requests while their first owner still runs.

Compared with a plain windowed implementation (float64): trace replay in four cuttings and both precisions; the same
cuttings through the step graphs; generation through the entry point with graphs and the one-step run-ahead."""

import numpy as np
import pytest
import torch

import cuttings
import plain_llama as plain

pytestmark = pytest.mark.gpu

NAME = "ToyWindowLM"
SMALL = dict(architectures=[NAME], width=48, vocab_size=131, inner=72, heads=3, kv_heads=1, layers=2, eps=1e-5,
             window=21, theta=10000.0)
WIDE = dict(architectures=[NAME], width=128, vocab_size=211, inner=96, heads=2, kv_heads=1, layers=2, eps=1e-6,
            window=150, theta=50000.0)


def define_toy():
    from tokasaurus_b200.config import register_architecture
    from tokasaurus_b200.parts import (DecoderModel, GatedMLP, OutputHead, PagedAttention, PreNormBlock, RMSNorm,
                                       RotaryEncoding, TokenEmbedding)

    def build(c):
        W, V, hd = c["width"], c["vocab_size"], c["width"] // c["heads"]
        blocks = []
        for i in range(c["layers"]):
            blocks.append(PreNormBlock(
                RMSNorm(W, c["eps"], f"b{i}.n1"),
                PagedAttention(W, c["heads"], c["kv_heads"], hd, RotaryEncoding(hd, c["theta"]), f"b{i}.q", f"b{i}.k",
                               f"b{i}.v", f"b{i}.o", window=c["window"]),
                RMSNorm(W, c["eps"], f"b{i}.n2"), GatedMLP(W, c["inner"], f"b{i}.g", f"b{i}.u", f"b{i}.d")))
        return DecoderModel(TokenEmbedding(V, W, "emb"), blocks, OutputHead(V, W, RMSNorm(W, c["eps"], "nf"), "head"))

    register_architecture(NAME, dict, build, replace=True)


class PlainWindowed:
    """Whole sequences, no cache, float64 by default: every query sees keys (i - window, i]."""

    def __init__(self, folder, c, dtype=torch.float64):
        from safetensors import safe_open
        self.c, self.w = c, {}
        with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
            for k in f.keys():
                self.w[k] = f.get_tensor(k).to(dtype)

    def logits(self, ids):
        c, w = self.c, self.w
        T, nh, nkv, hd = len(ids), c["heads"], c["kv_heads"], c["width"] // c["heads"]
        x = w["emb"][torch.tensor(ids)]
        cos, sin = plain.rope_tables(torch.arange(T), plain.rope_inv_freq(hd, c["theta"], None))
        for i in range(c["layers"]):
            h = plain.rms_norm(x, w[f"b{i}.n1"], c["eps"])
            q, k, v = ((h @ w[f"b{i}.{n}"].T).view(T, m, hd) for n, m in (("q", nh), ("k", nkv), ("v", nkv)))
            a = plain.causal_gqa_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v,
                                           window=c["window"]).reshape(T, -1)
            x = x + a @ w[f"b{i}.o"].T
            h = plain.rms_norm(x, w[f"b{i}.n2"], c["eps"])
            x = x + (torch.nn.functional.silu(h @ w[f"b{i}.g"].T) * (h @ w[f"b{i}.u"].T)) @ w[f"b{i}.d"].T
        return plain.rms_norm(x, w["nf"], c["eps"]) @ w["head"].T

    def greedy(self, prompt, n):
        ids, out = list(prompt), []
        for _ in range(n):
            out.append(int(self.logits(ids)[-1].argmax()))
            ids.append(out[-1])
        return out


@pytest.fixture(scope="module")
def toys(tmp_path_factory):
    from tokasaurus_b200.config import unregister_architecture
    from tokasaurus_b200.weights import write_model_folder

    define_toy()
    root = tmp_path_factory.mktemp("window_models")
    out = {}
    for name, c, lengths, page in (("small", SMALL, [100, 37, 64, 5, 81, 128, 50], 8),
                                   ("wide", WIDE, [700, 289, 513, 64], 16)):
        folder = write_model_folder(root / name, c, seed=11, std=0.08, norm_init="uniform")
        reqs = {f"{name[0]}{i}": cuttings.random_tokens(n, c["vocab_size"], 900 + i) for i, n in enumerate(lengths)}
        p64 = PlainWindowed(folder, c)
        want = {rid: p64.logits(t).numpy() for rid, t in reqs.items()}
        p32 = PlainWindowed(folder, c, torch.float32)
        want32 = {rid: p32.logits(t).double().numpy() for rid, t in reqs.items()}
        out[name] = dict(folder=folder, cfg=c, reqs=reqs, want=want, want32=want32, page=page)
    yield out
    unregister_architecture(NAME)


def pool_for(steps, window, page):
    """Pages a trace needs when pages behind the window come back after every step: the largest, over the steps, of
    the sum over live requests of the pages they hold while the step runs."""
    held, peak = {}, 0
    for st in steps:
        during = 0
        for e in st["entries"]:
            before = held.get(e["id"], 0)
            after = before + len(e["tokens"])
            first_page = max(0, before - window + 1) // page  # pages behind it were given back after the step before
            during += -(-after // page) - first_page
            held[e["id"]] = after
        idle = sum(-(-n // page) - max(0, n - window + 1) // page for rid, n in held.items()
                   if rid not in {e["id"] for e in st["entries"]})
        peak = max(peak, during + idle)
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def replay(toy, dtype, steps):
    """Trace replay with exactly the pages the trace needs.  Returns the logits and, per page, the requests that held it."""
    from tokasaurus_b200.engine.trace import TraceReplayer

    page, window = toy["page"], toy["cfg"]["window"]
    rp = TraceReplayer(str(toy["folder"]), dtype, pool_for(steps, window, page) * page, page_size=page, max_requests=4)
    cache = rp.runner.cache
    assert cache.groups[0].need.window == window
    owners, outs = {}, []
    for st in steps:
        outs.append(rp.run_step(st))
        cache.check()
        for rid, rc in cache.requests.items():
            for p in rc.live_pages(0):
                owners.setdefault(p, set()).add(rid)
    assert not cache.requests and cache.num_free_pages() == [cache.num_pages]
    return cuttings.collect(steps, outs), owners


def compare(got, toy, dtype, what):
    for rid, ref in toy["want"].items():
        tol = cuttings.tolerance(dtype, ref, toy["want32"][rid])
        err = np.abs(got[rid] - ref).max(axis=1)
        bad = np.nonzero(err > tol)[0]
        assert bad.size == 0, (f"{dtype} {what}: request {rid}: first wrong token at position {bad[0]} "
                               f"(error {err[bad[0]]:.3g}, tolerance {tol:.3g}); {bad.size} of {len(err)} wrong")


CUTS = dict(whole=cuttings.whole, prefix_then_single=cuttings.prefix_then_single,
            changing_portions=cuttings.changing_portions, mixed=cuttings.mixed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("which", ["small", "wide"])
def test_windowed_cuttings_match_plain(toys, which, cut, dtype):
    toy = toys[which]
    steps = CUTS[cut](toy["reqs"])
    got, owners = replay(toy, dtype, steps)
    compare(got, toy, dtype, cut)
    if cut == "mixed":
        # pages came back behind the window and went to other requests
        assert any(len(v) > 1 for v in owners.values()), "no page was used by two requests"
        longest = max(len(t) for t in toy["reqs"].values())
        assert pool_for(steps, toy["cfg"]["window"], toy["page"]) < sum(-(-len(t) // toy["page"]) for t in toy["reqs"].values())
        assert longest > toy["cfg"]["window"]


def test_window_edge_shows(toys):
    """The comparison would not notice a window that is off by one if far keys carried no weight: check on the plain
    implementation that they do (the logits with window and window + 1 differ by much more than the tolerance)."""
    toy = toys["small"]
    rid, toks = max(toy["reqs"].items(), key=lambda kv: len(kv[1]))
    wider = PlainWindowed(toy["folder"], dict(toy["cfg"], window=toy["cfg"]["window"] + 1)).logits(toks).numpy()
    tol = cuttings.tolerance("bfloat16", toy["want"][rid])
    assert np.abs(wider - toy["want"][rid]).max() > 2 * tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["small", "wide"])
def test_windowed_cuttings_through_step_graphs(toys, which, dtype):
    """Steps replayed from CUDA graphs (decode graphs and graphs of padded mixed steps), pages released after every
    step as the scheduler does it."""
    from tokasaurus_b200.engine.batch import StepEntry
    from tokasaurus_b200.engine.engine import Engine

    toy = toys[which]
    page, window = toy["page"], toy["cfg"]["window"]
    for cut in ("prefix_then_single", "mixed"):
        steps = CUTS[cut](toy["reqs"])
        eng = Engine(model=str(toy["folder"]), dtype=dtype, page_size=page,
                     kv_cache_num_tokens=pool_for(steps, window, page) * page, max_seqs_per_forward=8,
                     cudagraph_max_size=8, cudagraph_step=4, graph_max_tokens=4096)
        cache, graphs = eng.runner.cache, eng.graphs
        lengths, n_graph = {}, 0
        for st in steps:
            entries = []
            for e in st["entries"]:
                if e["id"] not in lengths:
                    cache.admit(e["id"])
                    lengths[e["id"]] = 0
                cache.ensure_capacity(e["id"], lengths[e["id"]] + len(e["tokens"]))
                entries.append(StepEntry(e["id"], list(e["tokens"]), lengths[e["id"]], [len(e["tokens"]) - 1]))
            R = len(entries)
            extra = dict(temperature=np.zeros(R, dtype=np.float32), stream_key=np.zeros(R, dtype=np.int64),
                         sample_pos=np.zeros(R, dtype=np.int32), row_slot=np.full(R, -1, dtype=np.int32))
            prep = None
            if graphs.usable(entries):
                prep = graphs.prepare(entries, extra)
            elif graphs.usable_general(entries):
                prep = graphs.prepare_general(entries, extra)
            if prep is not None:
                graphs.launch(prep)
                logits = graphs.graphs[prep["key"]]["logits"][:R].float().cpu().numpy()
                n_graph += 1
            else:
                logits = eng.runner.step(entries).float().cpu().numpy()
            eng.runner.check_status()
            for en, row in zip(entries, logits):
                lengths[en.request] += en.n_tokens
                cache.release_behind_window(en.request, lengths[en.request])
                ref = toy["want"][en.request][lengths[en.request] - 1]
                tol = cuttings.tolerance(dtype, toy["want"][en.request], toy["want32"][en.request])
                err = float(np.abs(row - ref).max())
                assert err <= tol, (f"{dtype} {cut}: request {en.request} position {lengths[en.request] - 1}: "
                                    f"error {err:.3g}, tolerance {tol:.3g}")
            for rid in st["end"]:
                cache.free(rid)
                del lengths[rid]
            cache.check()
        assert n_graph > len(steps) // 2 and not cache.requests


@pytest.mark.parametrize("run_ahead", [True, False])
def test_windowed_generation_through_the_entry_point(toys, run_ahead):
    """Greedy generation in float32 with graphs and the one-step run-ahead: prompts longer than the window, decoding
    across several page releases, a pool too small for all requests at once and so small that a request is pushed out
    and fed again through the windowed group."""
    from tokasaurus_b200.engine.engine import Engine

    toy = toys["small"]
    c, page = toy["cfg"], toy["page"]
    p64 = PlainWindowed(toy["folder"], c)
    prompts = [cuttings.random_tokens(n, c["vocab_size"], 300 + n) for n in (45, 9, 30, 26, 52)]
    n_new = 40
    want = [p64.greedy(p, n_new) for p in prompts]
    for pool_tokens, opts in ((1024, {}), (104, dict(bump_city_population_me=True))):
        eng = Engine(model=str(toy["folder"]), dtype="float32", page_size=page, kv_cache_num_tokens=pool_tokens,
                     max_tokens_per_forward=24, max_seqs_per_forward=4, allocator_sanity_checks=True,
                     run_ahead=run_ahead, **opts)
        outs = eng.generate(prompts, max_num_tokens=n_new, ignore_eos=True)
        assert [o.completion_ids for o in outs] == want
        assert not eng.runner.cache.requests and eng.runner.cache.num_free_pages() == [g.allocator.num_pages for g in eng.runner.cache.groups]
        if opts:
            assert eng.scheduler.stats["bumps"] > 0
