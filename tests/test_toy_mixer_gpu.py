"""A toy mixer with state of its own, defined here, is registered, built, loaded and stepped
without a change to the framework's files.  The toy model's first block uses the toy mixer (a
running mean of its inputs, kept per request in the cache manager's state slots), its second
block the framework's paged attention: parts are chosen layer by layer."""

import numpy as np
import pytest
import torch

import cuttings
import plain_llama as plain

pytestmark = pytest.mark.gpu


def define_toy():
    from tokasaurus_b200.config import register_architecture
    from tokasaurus_b200.kernels import ops
    from tokasaurus_b200.parts import (DecoderModel, GatedMLP, Mixer, OutputHead, PagedAttention, PreNormBlock, RMSNorm,
                                       RotaryEncoding, StateNeed, TokenEmbedding, WeightSpec)

    class RunningMeanMixer(Mixer):
        """out_t = W @ mean(h_0 .. h_t).  State per request: the running sum [width] and the count."""

        def __init__(self, width, name):
            self.width, self.name = width, name

        def weight_specs(self):
            return (WeightSpec(self.name, (self.width, self.width)),)

        def cache_need(self):
            return StateNeed((self.width + 1,), "float32")

        def bind(self, weights, rt):
            self.w = weights[self.name]

        def forward(self, ctx, h, cache, out_rows=None):
            mean = torch.empty_like(h)
            hb = ctx.host
            for s in range(ctx.n_seqs):
                a, n, slot = int(hb.seq_q_start[s]), int(hb.seq_q_len[s]), int(hb.seq_slot[s])
                st = cache.state[slot]
                sums = torch.cumsum(h[a:a + n].float(), 0) + st[: self.width]
                counts = st[self.width] + torch.arange(1, n + 1, device=h.device)
                mean[a:a + n] = (sums / counts[:, None]).to(h.dtype)
                st[: self.width] = sums[-1]
                st[self.width] = counts[-1]
            if out_rows is not None:
                mean = mean[out_rows.long()].contiguous()
            return ops.linear(mean, self.w)

    def parse(d):
        return dict(d)

    def build(c):
        W, V, I = c["width"], c["vocab_size"], c["inner"]
        nh, nkv = c["heads"], c["kv_heads"]
        b0 = PreNormBlock(RMSNorm(W, c["eps"], "b0.n1"), RunningMeanMixer(W, "b0.mix"), RMSNorm(W, c["eps"], "b0.n2"),
                          GatedMLP(W, I, "b0.g", "b0.u", "b0.d"))
        b1 = PreNormBlock(RMSNorm(W, c["eps"], "b1.n1"),
                          PagedAttention(W, nh, nkv, W // nh, RotaryEncoding(W // nh, 10000.0), "b1.q", "b1.k", "b1.v", "b1.o"),
                          RMSNorm(W, c["eps"], "b1.n2"), GatedMLP(W, I, "b1.g", "b1.u", "b1.d"))
        b2 = PreNormBlock(RMSNorm(W, c["eps"], "b2.n1"), RunningMeanMixer(W, "b2.mix"), RMSNorm(W, c["eps"], "b2.n2"),
                          GatedMLP(W, I, "b2.g", "b2.u", "b2.d"))
        return DecoderModel(TokenEmbedding(V, W, "emb"), [b0, b1, b2], OutputHead(V, W, RMSNorm(W, c["eps"], "nf"), "head"))

    register_architecture("ToyRunningMeanLM", parse, build, replace=True)


TOY = dict(architectures=["ToyRunningMeanLM"], width=64, vocab_size=97, inner=80, heads=2, kv_heads=1, eps=1e-5)


def plain_toy(folder, ids):
    from safetensors import safe_open
    w = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).double()
    T = len(ids)
    x = w["emb"][torch.tensor(ids)]

    def ffn(x, i):
        h = plain.rms_norm(x, w[f"b{i}.n2"], 1e-5)
        return x + (torch.nn.functional.silu(h @ w[f"b{i}.g"].T) * (h @ w[f"b{i}.u"].T)) @ w[f"b{i}.d"].T

    def mean_block(x, i):
        h = plain.rms_norm(x, w[f"b{i}.n1"], 1e-5)
        m = torch.cumsum(h, 0) / torch.arange(1, T + 1).double()[:, None]
        return ffn(x + m @ w[f"b{i}.mix"].T, i)

    x = mean_block(x, 0)
    h = plain.rms_norm(x, w["b1.n1"], 1e-5)
    hd = 32
    q, k, v = (h @ w["b1.q"].T).view(T, 2, hd), (h @ w["b1.k"].T).view(T, 1, hd), (h @ w["b1.v"].T).view(T, 1, hd)
    cos, sin = plain.rope_tables(torch.arange(T), plain.rope_inv_freq(hd, 10000.0, None))
    a = plain.causal_gqa_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v).reshape(T, -1)
    x = ffn(x + a @ w["b1.o"].T, 1)
    x = mean_block(x, 2)
    return (plain.rms_norm(x, w["nf"], 1e-5) @ w["head"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state(tmp_path, dtype):
    from tokasaurus_b200.config import unregister_architecture
    from tokasaurus_b200.engine.trace import TraceReplayer
    from tokasaurus_b200.weights import write_model_folder

    define_toy()
    try:
        folder = write_model_folder(tmp_path / "toy", TOY, seed=5, std=0.08, norm_init="uniform")
        reqs = {f"t{i}": cuttings.random_tokens(n, 97, i) for i, n in enumerate([40, 23, 61, 9, 33, 50])}
        want = {rid: plain_toy(folder, toks) for rid, toks in reqs.items()}
        for cut in (cuttings.whole, cuttings.changing_portions, cuttings.mixed):
            steps = cut(reqs)
            rp = TraceReplayer(str(folder), dtype, cuttings.max_live_tokens(steps), page_size=16, max_requests=4)
            assert len(rp.runner.cache.groups) == 1 and len(rp.runner.cache._state) == 2  # one paged group, two state entries
            outs = [rp.run_step(st) for st in steps]
            rp.runner.cache.check()
            got = cuttings.collect(steps, outs)
            for rid in reqs:
                tol = (1e-4 if dtype == "float32" else 3e-2) * np.abs(want[rid]).max()
                err = np.abs(got[rid] - want[rid]).max(axis=1)
                assert err.max() <= tol, (cut.__name__, rid, int(err.argmax()), float(err.max()), tol)
    finally:
        unregister_architecture("ToyRunningMeanLM")
