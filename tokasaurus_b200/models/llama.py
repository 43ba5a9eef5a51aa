"""The dense Llama decoder put together from parts, and its registry entry.

Tensor names are those of the checkpoint files, as the reference maps them in
tokasaurus/model/llama.py:824-847: ``model.embed_tokens.weight``; per layer
``model.layers.{i}.input_layernorm.weight``, ``.self_attn.{q,k,v,o}_proj.weight``,
``.post_attention_layernorm.weight``, ``.mlp.{gate,up,down}_proj.weight``; ``model.norm.weight``;
``lm_head.weight`` unless ``tie_word_embeddings`` (then the head reads the embedding tensor,
llama.py:842-845).
"""

from __future__ import annotations

from tokasaurus_b200.config.model_config import LlamaConfig
from tokasaurus_b200.config.registry import register_architecture
from tokasaurus_b200.parts import (
    DecoderModel,
    GatedMLP,
    OutputHead,
    PagedAttention,
    PreNormBlock,
    RMSNorm,
    RotaryEncoding,
    TokenEmbedding,
)


def build_llama(cfg: LlamaConfig) -> DecoderModel:
    H, hd = cfg.hidden_size, cfg.head_dim
    rs = cfg.rope_scaling
    if rs is not None and rs.rope_type == "llama3":
        position = RotaryEncoding(hd, cfg.rope_theta, "llama3", rs.factor, rs.low_freq_factor, rs.high_freq_factor,
                                  rs.original_max_position_embeddings)
    else:
        position = RotaryEncoding(hd, cfg.rope_theta)
    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        blocks.append(
            PreNormBlock(
                mixer_norm=RMSNorm(H, cfg.rms_norm_eps, f"{p}.input_layernorm.weight"),
                mixer=PagedAttention(
                    H, cfg.num_attention_heads, cfg.num_key_value_heads, hd, position,
                    q_name=f"{p}.self_attn.q_proj.weight", k_name=f"{p}.self_attn.k_proj.weight",
                    v_name=f"{p}.self_attn.v_proj.weight", o_name=f"{p}.self_attn.o_proj.weight",
                ),
                ffn_norm=RMSNorm(H, cfg.rms_norm_eps, f"{p}.post_attention_layernorm.weight"),
                ffn=GatedMLP(H, cfg.intermediate_size, gate_name=f"{p}.mlp.gate_proj.weight",
                             up_name=f"{p}.mlp.up_proj.weight", down_name=f"{p}.mlp.down_proj.weight"),
            )
        )
    embed_name = "model.embed_tokens.weight"
    head_name = embed_name if cfg.tie_word_embeddings else "lm_head.weight"
    # Tensors that Llama checkpoints may carry and that the reference, which reads only the names it wants
    # (tokasaurus/model/safetensors_utils.py:72-95, load_state_dict(strict=False) at llama.py:940), passes over: the
    # rotary tables' inverse frequencies of older exports, and a stored head beside tied embeddings.
    ignored = ["*.rotary_emb.inv_freq"] + (["lm_head.weight"] if cfg.tie_word_embeddings else [])
    return DecoderModel(
        embedding=TokenEmbedding(cfg.vocab_size, H, embed_name),
        blocks=blocks,
        head=OutputHead(cfg.vocab_size, H, RMSNorm(H, cfg.rms_norm_eps, "model.norm.weight"), head_name),
        ignored_weight_patterns=ignored,
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, build_llama, model_types=("llama",), replace=True)
