"""A plain, slow implementation of the dense Llama decoder: whole sequences, no cache, one
function for each part, written from the reference's formulas.  It shares no code with the
engine under ``tokasaurus_b200`` (it reads config.json and model.safetensors by itself) and is
what the engine's logits are compared with.  ``tests/golden/make_reference_golden.py`` compares it
once with the reference's own model code on a tiny random model.

Every function takes and returns tensors of the ``dtype`` given to ``PlainLlama`` (float64 by
default: the yardstick; float32 gives the spread that 32-bit arithmetic alone causes).
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """tokasaurus/model/llama.py:44-51: variance = mean(x^2); x * rsqrt(variance + eps); times weight."""
    variance = x.pow(2).mean(-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """Inverse frequencies behind the reference's cos/sin tables (tokasaurus/model/llama.py:559-570
    builds them with LlamaRotaryEmbedding; tests/golden/make_reference_golden.py checks that this
    formula reproduces those tables).  Computed in float32 like the tables."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    if not scaling or scaling.get("rope_type", scaling.get("type", "default")) == "default":
        return inv
    factor = scaling["factor"]
    low = scaling["low_freq_factor"]
    high = scaling["high_freq_factor"]
    orig = scaling["original_max_position_embeddings"]
    # float32 tensor arithmetic throughout, as the tables are built
    wavelen = 2 * math.pi / inv
    stretched = torch.where(wavelen > orig / low, inv / factor, inv)
    smooth = (orig / wavelen - low) / (high - low)
    blended = (1 - smooth) * inv / factor + smooth * inv
    middle = (wavelen <= orig / low) & (wavelen >= orig / high)
    return torch.where(middle, blended, stretched)


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """cos, sin [T, head_dim] in float32: freqs = pos (x) inv_freq, emb = cat(freqs, freqs)
    (the tables of tokasaurus/model/llama.py:563-570, gathered by position at :576-578)."""
    freqs = torch.outer(positions.to(torch.float32), inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """tokasaurus/model/llama.py:247-256 (apply_rotary_pos_emb with unsqueeze_dim=1 over heads):
    x * cos + rotate_half(x) * sin; x is [T, heads, head_dim]."""
    cos = cos.to(x.dtype).unsqueeze(1)
    sin = sin.to(x.dtype).unsqueeze(1)
    return x * cos + rotate_half(x) * sin


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """q [T, nh, hd], k and v [T, nkv, hd] of ONE whole sequence.  Query i sees keys 0..i
    (tokasaurus/model/llama.py:716-729 plans causal attention; the scale is 1/sqrt(hd), the
    library default, no soft cap); query head j reads kv head j // (nh / nkv)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd)
    i = torch.arange(T, device=q.device).view(-1, 1)
    j = torch.arange(T, device=q.device).view(1, -1)
    hidden = j > i
    if window:
        hidden = hidden | (j <= i - window)
    scores = scores.masked_fill(hidden, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hqk,khd->qhd", probs, v)


def attention_block(x, w, prefix, cfg, positions, inv_freq):
    """tokasaurus/model/llama.py:218-287: norm, q/k/v projections (:235-237), views (:239-241),
    rotary (:243-256), attention, output projection (:280), residual (:284)."""
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    hd = cfg["hidden_size"] // nh
    T = x.shape[0]
    h = rms_norm(x, w[f"{prefix}.input_layernorm.weight"], cfg["rms_norm_eps"])
    q = (h @ w[f"{prefix}.self_attn.q_proj.weight"].T).view(T, nh, hd)
    k = (h @ w[f"{prefix}.self_attn.k_proj.weight"].T).view(T, nkv, hd)
    v = (h @ w[f"{prefix}.self_attn.v_proj.weight"].T).view(T, nkv, hd)
    cos, sin = rope_tables(positions, inv_freq)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    a = causal_gqa_attention(q, k, v).reshape(T, nh * hd)
    return x + a @ w[f"{prefix}.self_attn.o_proj.weight"].T


def mlp_block(x, w, prefix, cfg):
    """tokasaurus/model/llama.py:319-339: norm (:325), up and gate (:329-330), silu(gate) * up (:331),
    down (:332), residual (:336)."""
    h = rms_norm(x, w[f"{prefix}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    up = h @ w[f"{prefix}.mlp.up_proj.weight"].T
    gate = h @ w[f"{prefix}.mlp.gate_proj.weight"].T
    prod = torch.nn.functional.silu(gate) * up
    return x + prod @ w[f"{prefix}.mlp.down_proj.weight"].T


def lm_head(x, w, cfg):
    """tokasaurus/model/llama.py:465-467: final norm, vocabulary projection; tied weights read the
    embedding (:842-845)."""
    h = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    name = "model.embed_tokens.weight" if cfg.get("tie_word_embeddings", False) else "lm_head.weight"
    return h @ w[name].T


class PlainLlama:
    def __init__(self, folder: str | Path, dtype: torch.dtype = torch.float64, device: str = "cpu"):
        """``device``: where the arithmetic runs (the CPU by default; a model of real layer sizes in float64 is
        quicker with torch on the GPU, and is still this same plain arithmetic)."""
        folder = Path(folder)
        self.device = device
        with open(folder / "config.json") as f:
            self.cfg = json.load(f)
        self.cfg.setdefault("rms_norm_eps", 1e-6)
        self.dtype = dtype
        self.w: dict[str, torch.Tensor] = {}
        with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
            for k in f.keys():
                self.w[k] = f.get_tensor(k).to(device=device, dtype=dtype)
        hd = self.cfg["hidden_size"] // self.cfg["num_attention_heads"]
        self.inv_freq = rope_inv_freq(hd, self.cfg.get("rope_theta", 10000.0), self.cfg.get("rope_scaling")).to(device)

    def logits(self, token_ids: list[int]) -> torch.Tensor:
        """Logits [T, vocab] at every position of one whole sequence."""
        ids = torch.tensor(token_ids, dtype=torch.long, device=self.device)
        positions = torch.arange(len(token_ids), device=self.device)
        x = self.w["model.embed_tokens.weight"][ids]  # tokasaurus/model/llama.py:514-518
        for i in range(self.cfg["num_hidden_layers"]):  # llama.py:580-581
            p = f"model.layers.{i}"
            x = attention_block(x, self.w, p, self.cfg, positions, self.inv_freq)
            x = mlp_block(x, self.w, p, self.cfg)
        return lm_head(x, self.w, self.cfg)

    def greedy(self, prompt: list[int], n: int) -> list[int]:
        """n greedy tokens, recomputing the whole sequence each time (tokasaurus/model/llama.py:386-397
        with greedy_mask: argmax of the logits)."""
        ids = list(prompt)
        out = []
        for _ in range(n):
            nxt = int(self.logits(ids)[-1].argmax())
            out.append(nxt)
            ids.append(nxt)
        return out


def tiny_configs() -> list[dict]:
    """Two tiny configurations of the architecture that differ in every size and option."""
    return [
        dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=64,
             num_attention_heads=4, num_key_value_heads=2, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
             rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=128),
        dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=3, hidden_size=96,
             num_attention_heads=3, num_key_value_heads=1, intermediate_size=160, vocab_size=509, rope_theta=500000.0,
             rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                               original_max_position_embeddings=32),
             rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=256),
    ]


# seed, std of matrices, init of norm weights, page size: the other options the two test models differ in
TINY_WEIGHTS = [dict(seed=0, std=0.02, norm_init="ones", page_size=16),
                dict(seed=1, std=0.05, norm_init="uniform", page_size=8)]
