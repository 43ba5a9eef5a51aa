"""The plain Llama decoder with the reference's bfloat16 ROUNDING: every tensor that the reference holds in bfloat16
between two operations is rounded to bfloat16 here, at the same place, and everything else is computed exactly
(float64).  It states what "the reference's bfloat16 arithmetic" is, separately from how any kernel orders its sums:

* weights and the embedding rows are bfloat16 (tokasaurus/model/llama.py:514-518);
* RMSNorm computes in float32, casts x * rsqrt(var + eps) to bfloat16 and THEN multiplies by the bfloat16 weight, the
  product being bfloat16 again: two roundings (llama.py:44-54);
* each linear layer's output is bfloat16 (q, k, v :235-237; o :280; up, gate :329-330; down :332; the vocabulary
  projection :467, turned into float32 only afterwards);
* the rotary encoding multiplies bfloat16 q and k with float32 cos and sin and casts the result back (:243-259);
* the attention's output is bfloat16 (:261-269; what the attention library rounds inside itself is not modelled);
* silu(gate) is a bfloat16 tensor and so is its product with up (:331);
* both residual sums are bfloat16 + bfloat16 -> bfloat16 (:284, :336): the residual stream is rounded after every
  half-layer.

The engine under ``tokasaurus_b200`` rounds at fewer places (a float32 residual stream, one rounding in the norm, a
float32 product before the down projection's input is rounded); tests compare both with the float64 yardstick.
It shares no code with the engine; the exact operations come from ``plain_llama``.
"""

from __future__ import annotations

import torch

import plain_llama as pl


def r(x: torch.Tensor) -> torch.Tensor:
    """Round to bfloat16 (nearest even, as the cast does) and carry on in the input's dtype."""
    return x.to(torch.bfloat16).to(x.dtype)


def rms_norm(x, weight, eps):
    """tokasaurus/model/llama.py:44-54: float32 arithmetic, cast to the input dtype, then times the weight."""
    variance = x.pow(2).mean(-1, keepdim=True)
    return r(weight * r(x * torch.rsqrt(variance + eps)))


def attention_block(x, w, prefix, cfg, positions, inv_freq):
    """tokasaurus/model/llama.py:218-287 with the roundings listed in this file's header."""
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    hd = cfg["hidden_size"] // nh
    T = x.shape[0]
    h = rms_norm(x, w[f"{prefix}.input_layernorm.weight"], cfg["rms_norm_eps"])
    q = r(h @ w[f"{prefix}.self_attn.q_proj.weight"].T).view(T, nh, hd)
    k = r(h @ w[f"{prefix}.self_attn.k_proj.weight"].T).view(T, nkv, hd)
    v = r(h @ w[f"{prefix}.self_attn.v_proj.weight"].T).view(T, nkv, hd)
    cos, sin = pl.rope_tables(positions, inv_freq)
    q = r(pl.apply_rope(q, cos, sin))
    k = r(pl.apply_rope(k, cos, sin))
    a = r(pl.causal_gqa_attention(q, k, v)).reshape(T, nh * hd)
    return r(x + r(a @ w[f"{prefix}.self_attn.o_proj.weight"].T))


def mlp_block(x, w, prefix, cfg):
    """tokasaurus/model/llama.py:319-339 with the roundings listed in this file's header."""
    h = rms_norm(x, w[f"{prefix}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    up = r(h @ w[f"{prefix}.mlp.up_proj.weight"].T)
    gate = r(h @ w[f"{prefix}.mlp.gate_proj.weight"].T)
    prod = r(r(torch.nn.functional.silu(gate)) * up)
    return r(x + r(prod @ w[f"{prefix}.mlp.down_proj.weight"].T))


def lm_head(x, w, cfg):
    """tokasaurus/model/llama.py:465-467: final norm, bfloat16 logits."""
    h = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    name = "model.embed_tokens.weight" if cfg.get("tie_word_embeddings", False) else "lm_head.weight"
    return r(h @ w[name].T)


class PlainLlamaReferenceRounding(pl.PlainLlama):
    """``PlainLlama`` in float64 whose weights are rounded to bfloat16 once (a no-op for a folder stored in
    bfloat16, as the test models are) and whose intermediate tensors are rounded where the reference's are."""

    def __init__(self, folder, device: str = "cpu"):
        super().__init__(folder, torch.float64, device)
        self.w = {k: r(t) for k, t in self.w.items()}

    def logits(self, token_ids: list[int]) -> torch.Tensor:
        ids = torch.tensor(token_ids, dtype=torch.long, device=self.device)
        positions = torch.arange(len(token_ids), device=self.device)
        x = self.w["model.embed_tokens.weight"][ids]
        for i in range(self.cfg["num_hidden_layers"]):
            p = f"model.layers.{i}"
            x = attention_block(x, self.w, p, self.cfg, positions, self.inv_freq)
            x = mlp_block(x, self.w, p, self.cfg)
        return lm_head(x, self.w, self.cfg)

