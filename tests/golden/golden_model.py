"""Weights of the tiny model behind tests/golden/reference_logits_tiny_a.json.

Drawn with torch's CPU generator in a fixed order, so the test can rebuild them; the JSON
also stores the sum of their absolute values, and the test skips (instead of failing) if a
torch build ever draws other numbers.
"""
import torch

CONFIG = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=176, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256, rms_norm_eps=1e-5,
              rope_theta=10000.0, max_position_embeddings=64, tie_word_embeddings=False, hidden_act="silu")


def tensor_shapes(config):
    h, f, v = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    q = config["num_attention_heads"] * config["head_dim"]
    kv = config["num_key_value_heads"] * config["head_dim"]
    shapes = {"model.embed_tokens.weight": (v, h), "model.norm.weight": (h,), "lm_head.weight": (v, h)}
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shapes.update({p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
                       p + "self_attn.q_proj.weight": (q, h), p + "self_attn.k_proj.weight": (kv, h),
                       p + "self_attn.v_proj.weight": (kv, h), p + "self_attn.o_proj.weight": (h, q),
                       p + "mlp.gate_proj.weight": (f, h), p + "mlp.up_proj.weight": (f, h),
                       p + "mlp.down_proj.weight": (h, f)})
    return shapes


def golden_weights(config, seed):
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, shape in sorted(tensor_shapes(config).items()):
        values = torch.randn(shape, generator=generator, dtype=torch.float32) * 0.02
        if name.endswith("layernorm.weight") or name == "model.norm.weight":
            values = values + 1.0
        weights[name] = values
    return weights
