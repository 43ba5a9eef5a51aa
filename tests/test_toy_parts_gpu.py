"""Two more toy parts, defined here and used without a change to the framework's files: a feed-forward
with routing (top-1 of four small experts, router logits and softmax in float32) and another position
encoding (learned absolute positions added to the token embedding, with an attention that rotates nothing).
The toy model's first block: attention without rotation + the framework's gated MLP; its second block: the
framework's rotary attention + the routed feed-forward.  Neither is, nor becomes, a model of anyone's."""

import numpy as np
import pytest
import torch

import cuttings
import plain_llama as plain

pytestmark = pytest.mark.gpu

EXPERTS, MAX_POS = 4, 128
TOY = dict(architectures=["ToyRoutedLM"], width=64, vocab_size=101, inner=48, expert_inner=32, heads=4, kv_heads=2,
           eps=1e-5)


def define_toy():
    from tokasaurus_b200.config import register_architecture
    from tokasaurus_b200.kernels import ops
    from tokasaurus_b200.parts import (DecoderModel, FeedForward, GatedMLP, NoPositionEncoding, OutputHead,
                                       PagedAttention, PreNormBlock, ResidualStream, RMSNorm, RotaryEncoding,
                                       TokenEmbedding, WeightSpec)

    class LearnedPositionEmbedding(TokenEmbedding):
        """Token embedding plus a learned vector for the token's position."""

        def __init__(self, vocab, width, weight_name, pos_name, max_pos):
            super().__init__(vocab, width, weight_name)
            self.pos_name, self.max_pos = pos_name, max_pos

        def weight_specs(self):
            return tuple(super().weight_specs()) + (WeightSpec(self.pos_name, (self.max_pos, self.width)),)

        def bind(self, weights, rt):
            super().bind(weights, rt)
            self.pos = weights[self.pos_name]

        def forward(self, ctx):
            stream = super().forward(ctx)
            stream.x += self.pos.index_select(0, ctx.positions[: ctx.n_tokens].long()).float()
            return ResidualStream(stream.x)

    class RoutedFFN(FeedForward):
        """Each token goes to the expert with the largest router logit; the expert's output is scaled by that
        expert's softmax probability.  Router logits, softmax and the scale are float32."""

        def __init__(self, width, inner, n_experts, prefix):
            self.width, self.inner, self.n, self.prefix = width, inner, n_experts, prefix

        def weight_specs(self):
            p = self.prefix
            specs = [WeightSpec(f"{p}.router", (self.n, self.width), keep_32bit=True)]
            for e in range(self.n):
                specs += [WeightSpec(f"{p}.e{e}.g", (self.inner, self.width)), WeightSpec(f"{p}.e{e}.u", (self.inner, self.width)),
                          WeightSpec(f"{p}.e{e}.d", (self.width, self.inner))]
            return tuple(specs)

        def bind(self, weights, rt):
            p = self.prefix
            self.router = weights[f"{p}.router"].float()
            self.g = [weights[f"{p}.e{e}.g"] for e in range(self.n)]
            self.u = [weights[f"{p}.e{e}.u"] for e in range(self.n)]
            self.d = [weights[f"{p}.e{e}.d"] for e in range(self.n)]

        def forward(self, ctx, h):
            logits = h.float() @ self.router.T
            prob = torch.softmax(logits, dim=-1)
            choice = logits.argmax(dim=-1)
            out = torch.zeros((h.shape[0], self.width), dtype=torch.float32, device=h.device)
            for e in range(self.n):  # a toy: every expert sees every row, rows of other experts are masked out
                act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
                ops.silu_mul(torch.cat([ops.linear(h, self.g[e]), ops.linear(h, self.u[e])], dim=1).contiguous(), act, 0)
                y = ops.linear(act, self.d[e]).float()
                out += y * (prob[:, e] * (choice == e))[:, None]
            return out.to(h.dtype)

    def build(c):
        W, V, hd = c["width"], c["vocab_size"], c["width"] // c["heads"]
        nh, nkv, eps = c["heads"], c["kv_heads"], c["eps"]
        b0 = PreNormBlock(RMSNorm(W, eps, "b0.n1"),
                          PagedAttention(W, nh, nkv, hd, NoPositionEncoding(), "b0.q", "b0.k", "b0.v", "b0.o"),
                          RMSNorm(W, eps, "b0.n2"), GatedMLP(W, c["inner"], "b0.g", "b0.u", "b0.d"))
        b1 = PreNormBlock(RMSNorm(W, eps, "b1.n1"),
                          PagedAttention(W, nh, nkv, hd, RotaryEncoding(hd, 10000.0), "b1.q", "b1.k", "b1.v", "b1.o"),
                          RMSNorm(W, eps, "b1.n2"), RoutedFFN(W, c["expert_inner"], EXPERTS, "b1.moe"))
        return DecoderModel(LearnedPositionEmbedding(V, W, "emb", "pos", MAX_POS), [b0, b1],
                            OutputHead(V, W, RMSNorm(W, eps, "nf"), "head"))

    register_architecture("ToyRoutedLM", dict, build, replace=True)


def plain_toy(folder, ids):
    """Logits [T, V] in float64 and each token's router margin (best minus second-best router logit, as a
    fraction of the largest router logit of the sequence)."""
    from safetensors import safe_open
    w = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).double()
    T, nh, nkv, hd = len(ids), TOY["heads"], TOY["kv_heads"], TOY["width"] // TOY["heads"]
    x = w["emb"][torch.tensor(ids)] + w["pos"][:T]

    def attention(x, i, rotary):
        h = plain.rms_norm(x, w[f"b{i}.n1"], 1e-5)
        q, k, v = ((h @ w[f"b{i}.{n}"].T).view(T, m, hd) for n, m in (("q", nh), ("k", nkv), ("v", nkv)))
        if rotary:
            cos, sin = plain.rope_tables(torch.arange(T), plain.rope_inv_freq(hd, 10000.0, None))
            q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
        return x + plain.causal_gqa_attention(q, k, v).reshape(T, -1) @ w[f"b{i}.o"].T

    x = attention(x, 0, False)
    h = plain.rms_norm(x, w["b0.n2"], 1e-5)
    x = x + (torch.nn.functional.silu(h @ w["b0.g"].T) * (h @ w["b0.u"].T)) @ w["b0.d"].T
    x = attention(x, 1, True)
    h = plain.rms_norm(x, w["b1.n2"], 1e-5)
    logits = h @ w["b1.moe.router"].T
    prob = torch.softmax(logits, -1)
    top2 = logits.topk(2, dim=-1).values
    y = torch.zeros_like(x)
    for t in range(T):
        e = int(logits[t].argmax())
        a = torch.nn.functional.silu(h[t] @ w[f"b1.moe.e{e}.g"].T) * (h[t] @ w[f"b1.moe.e{e}.u"].T)
        y[t] = prob[t, e] * (a @ w[f"b1.moe.e{e}.d"].T)
    x = x + y
    return (plain.rms_norm(x, w["nf"], 1e-5) @ w["head"].T).numpy(), ((top2[:, 0] - top2[:, 1]) / logits.abs().max()).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_learned_positions(tmp_path, dtype):
    from tokasaurus_b200.config import unregister_architecture
    from tokasaurus_b200.engine.trace import TraceReplayer
    from tokasaurus_b200.weights import write_model_folder

    define_toy()
    try:
        folder = write_model_folder(tmp_path / "toy", TOY, seed=9, std=0.08, norm_init="uniform")
        reqs = {f"t{i}": cuttings.random_tokens(n, 101, 7 * i + 1) for i, n in enumerate([40, 23, 61, 9, 33])}
        want = {rid: plain_toy(folder, toks) for rid, toks in reqs.items()}
        # a token whose two best router logits lie within rounding of each other may go to either expert: its row
        # is left out (the routed block is the last one, so no other token depends on it)
        margin = 1e-4 if dtype == "float32" else 2e-2
        compared = total = 0
        for cut in (cuttings.whole, cuttings.changing_portions, cuttings.mixed):
            steps = cut(reqs)
            rp = TraceReplayer(str(folder), dtype, cuttings.max_live_tokens(steps), page_size=16, max_requests=4)
            outs = [rp.run_step(st) for st in steps]
            rp.runner.cache.check()
            got = cuttings.collect(steps, outs)
            for rid in reqs:
                logits, gap = want[rid]
                clear = gap > margin
                tol = (1e-4 if dtype == "float32" else 3e-2) * np.abs(logits).max()
                err = np.abs(got[rid] - logits).max(axis=1)
                assert err[clear].max() <= tol, (cut.__name__, rid, int(err.argmax()), float(err[clear].max()), tol)
                compared += int(clear.sum())
                total += clear.shape[0]
        assert compared > 0.85 * total
    finally:
        unregister_architecture("ToyRoutedLM")


# ---------------------------------------------------------------------------------------------------------------------
# An attention whose projections carry biases and whose q and k heads are RMS-normalised before the rotation: the
# element-wise stage the framework's attention offers (``QkvStage``).  Such a mixer is "new parts and a registry
# entry", and it keeps every fast path: the decode steps below still run the fused rotary + cache write +
# split-key attention kernel, and the portions the tcgen05 kernel (heads of 64).

QKN = dict(architectures=["ToyQkNormLM"], width=256, vocab_size=113, inner=96, heads=4, kv_heads=2, layers=2, eps=1e-5,
           qk_eps=1e-6, theta=10000.0)


def define_qk_norm_toy():
    from tokasaurus_b200.config import register_architecture
    from tokasaurus_b200.parts import (DecoderModel, GatedMLP, OutputHead, PagedAttention, PreNormBlock, QkvStage, RMSNorm,
                                       RotaryEncoding, TokenEmbedding)

    def build(c):
        W, V, hd = c["width"], c["vocab_size"], c["width"] // c["heads"]
        blocks = []
        for i in range(c["layers"]):
            stage = QkvStage(bias_names=(f"b{i}.qb", f"b{i}.kb", f"b{i}.vb"), qk_norm_names=(f"b{i}.qn", f"b{i}.kn"),
                             norm_eps=c["qk_eps"])
            blocks.append(PreNormBlock(
                RMSNorm(W, c["eps"], f"b{i}.n1"),
                PagedAttention(W, c["heads"], c["kv_heads"], hd, RotaryEncoding(hd, c["theta"]), f"b{i}.q", f"b{i}.k",
                               f"b{i}.v", f"b{i}.o", qkv_stage=stage),
                RMSNorm(W, c["eps"], f"b{i}.n2"), GatedMLP(W, c["inner"], f"b{i}.g", f"b{i}.u", f"b{i}.d")))
        return DecoderModel(TokenEmbedding(V, W, "emb"), blocks, OutputHead(V, W, RMSNorm(W, c["eps"], "nf"), "head"))

    register_architecture("ToyQkNormLM", dict, build, replace=True)


def plain_qk_norm_toy(folder, ids, dtype=torch.float64):
    from safetensors import safe_open
    c, w = QKN, {}
    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).to(dtype)
    T, nh, nkv, hd = len(ids), c["heads"], c["kv_heads"], c["width"] // c["heads"]
    x = w["emb"][torch.tensor(ids)]
    cos, sin = plain.rope_tables(torch.arange(T), plain.rope_inv_freq(hd, c["theta"], None))
    for i in range(c["layers"]):
        h = plain.rms_norm(x, w[f"b{i}.n1"], c["eps"])
        q = (h @ w[f"b{i}.q"].T + w[f"b{i}.qb"]).view(T, nh, hd)
        k = (h @ w[f"b{i}.k"].T + w[f"b{i}.kb"]).view(T, nkv, hd)
        v = (h @ w[f"b{i}.v"].T + w[f"b{i}.vb"]).view(T, nkv, hd)
        q = plain.rms_norm(q, w[f"b{i}.qn"], c["qk_eps"])  # over the head size
        k = plain.rms_norm(k, w[f"b{i}.kn"], c["qk_eps"])
        a = plain.causal_gqa_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v).reshape(T, -1)
        x = x + a @ w[f"b{i}.o"].T
        h = plain.rms_norm(x, w[f"b{i}.n2"], c["eps"])
        x = x + (torch.nn.functional.silu(h @ w[f"b{i}.g"].T) * (h @ w[f"b{i}.u"].T)) @ w[f"b{i}.d"].T
    return (plain.rms_norm(x, w["nf"], c["eps"]) @ w["head"].T).double().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_with_biases_and_head_norms_keeps_the_fused_paths(tmp_path, monkeypatch, dtype):
    import test_replay_gpu as rp
    from tokasaurus_b200.config import unregister_architecture
    from tokasaurus_b200.kernels import ops
    from tokasaurus_b200.weights import write_model_folder

    define_qk_norm_toy()
    calls = dict(fused=0, tc=0)
    fused, tc = ops.attn_decode_rope_mma, ops.attn_prefill_tc

    def count_fused(*a, **k):
        calls["fused"] += 1
        assert k.get("bias") is not None and k.get("qk_norm") is not None
        return fused(*a, **k)

    def count_tc(*a, **k):
        calls["tc"] += 1
        return tc(*a, **k)

    monkeypatch.setattr(ops, "attn_decode_rope_mma", count_fused)
    monkeypatch.setattr(ops, "attn_prefill_tc", count_tc)
    try:
        folder = write_model_folder(tmp_path / "toy", QKN, seed=21, std=0.08, norm_init="uniform")
        reqs = {f"q{i}": cuttings.random_tokens(n, QKN["vocab_size"], 50 + i) for i, n in enumerate([150, 37, 64, 9, 201])}
        want = {rid: plain_qk_norm_toy(folder, toks) for rid, toks in reqs.items()}
        want32 = {rid: plain_qk_norm_toy(folder, toks, torch.float32) for rid, toks in reqs.items()} if dtype == "float32" else None
        # the stage is not a no-op for these weights: without the head norm the logits are far away
        for cut in ("whole", "prefix_then_single", "changing_portions", "mixed"):
            steps = rp.CUTS[cut](reqs)
            rp.compare(rp.replay(folder, dtype, steps, 16), want, want32, dtype)
        steps = cuttings.prefix_then_single(reqs)
        got, n_graph = rp.replay_through_graphs(folder, dtype, steps, 16)
        assert n_graph > len(steps) // 2
        for rid, ref in want.items():
            tol = cuttings.tolerance(dtype, ref, want32[rid] if want32 else None)
            for pos, row in got[rid].items():
                err = float(np.abs(row - ref[pos]).max())
                assert err <= tol, f"{dtype}: request {rid} position {pos}: error {err:.3g}, tolerance {tol:.3g}"
        if dtype == "bfloat16":
            assert calls["fused"] > 0, "decode steps left the fused rotary + attention kernel"
            assert calls["tc"] > 0, "portions left the tcgen05 kernel"
    finally:
        unregister_architecture("ToyQkNormLM")
