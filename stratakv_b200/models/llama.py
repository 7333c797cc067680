"""The dense Llama decoder as a list of parts.

Tensor names are the checkpoint's own, the ones the reference binds
(``src/generation/generator.cpp:331-343, 402-428, 461``): ``model.embed_tokens.weight``,
``model.layers.{i}.{input_layernorm, post_attention_layernorm}.weight``,
``model.layers.{i}.self_attn.{q,k,v,o}_proj.weight``, ``model.layers.{i}.mlp.{gate,up,down}_proj.weight``,
``model.norm.weight`` and ``lm_head.weight``.  The reference rejects tied
embeddings by requiring ``lm_head.weight``; here ``tie_word_embeddings`` makes
the head read the embedding table.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import (AttentionSpec, EmbeddingSpec, GatedMlpSpec, HeadSpec, LayerSpec,
                          ModelSpec, NormSpec, RopeSpec, ScheduleEntry)


def llama_spec(config: LlamaConfig) -> ModelSpec:
    rope = RopeSpec(head_dim=config.head_dim, theta=config.rope_theta)
    layers = []
    for i in range(config.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            mixer_norm=NormSpec(config.hidden_size, config.rms_norm_eps, p + "input_layernorm.weight"),
            mixer=AttentionSpec(
                hidden_size=config.hidden_size,
                num_heads=config.num_attention_heads,
                num_kv_heads=config.num_key_value_heads,
                head_dim=config.head_dim,
                scale=config.head_dim ** -0.5,     # src/layers/attention.cpp:262-263
                position=rope,
                q_weight=p + "self_attn.q_proj.weight",
                k_weight=p + "self_attn.k_proj.weight",
                v_weight=p + "self_attn.v_proj.weight",
                o_weight=p + "self_attn.o_proj.weight"),
            ffn_norm=NormSpec(config.hidden_size, config.rms_norm_eps,
                              p + "post_attention_layernorm.weight"),
            ffn=GatedMlpSpec(
                hidden_size=config.hidden_size,
                intermediate_size=config.intermediate_size,
                activation="silu",
                gate_weight=p + "mlp.gate_proj.weight",
                up_weight=p + "mlp.up_proj.weight",
                down_weight=p + "mlp.down_proj.weight"),
        ))
    embedding = EmbeddingSpec(config.vocab_size, config.hidden_size, "model.embed_tokens.weight")
    head_weight = embedding.weight if config.tie_word_embeddings else "lm_head.weight"
    return ModelSpec(
        architecture=config.architecture,
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        embedding=embedding,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(config.num_hidden_layers)),
        final_norm=NormSpec(config.hidden_size, config.rms_norm_eps, "model.norm.weight"),
        head=HeadSpec(config.vocab_size, config.hidden_size, head_weight),
        stop_token_ids=tuple(config.eos_token_ids),
        max_positions=config.max_position_embeddings,
        # A tied checkpoint may still carry a copy of the head; rotary tables are buffers.
        ignorable=(("lm_head.weight",) if config.tie_word_embeddings else ())
        + tuple(f"model.layers.{i}.self_attn.rotary_emb.inv_freq"
                for i in range(config.num_hidden_layers)),
    )


register_architecture("LlamaForCausalLM", LlamaConfig, llama_spec)
