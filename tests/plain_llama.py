"""A plain, slow implementation of the dense Llama decoder, for comparison only.

Whole sequences, no cache, one function per part, float32 on the CPU (with the
double-precision steps the reference's CPU code has).  It shares no code with
the package: it reads ``config.json`` and the safetensors file through the
``safetensors`` library and plain ``json``.

It rests on the formulas of the reference's CPU classes; each function cites
them.  ``tests/golden/`` holds logits that the reference's own compiled CPU
classes produced for one tiny model, and ``tests/test_plain_reference.py``
compares this file with them.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch


def load_folder(model_dir, device="cpu"):
    """``(config dict, {name: float32 tensor})`` of a model folder.  ``device`` is where the tensors
    go: the arithmetic below runs wherever its weights are (large test models use a GPU for speed,
    in the same float32 and double steps)."""
    from safetensors import safe_open
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    weights = {}
    with safe_open(str(model_dir / "model.safetensors"), framework="pt") as handle:
        for name in handle.keys():
            weights[name] = handle.get_tensor(name).to(device=device, dtype=torch.float32)
    return config, weights


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """src/layers/rmsnorm.cpp:78-94: sum of squares in double, mean rounded to
    float, ``1/sqrt(mean + eps)`` in float, then ``x * inv * weight``."""
    mean_square = (x.double() ** 2).sum(dim=-1, keepdim=True) / x.shape[-1]
    mean_square = mean_square.float()
    inverse_rms = 1.0 / torch.sqrt(mean_square + torch.tensor(eps, dtype=torch.float32, device=x.device))
    return x * inverse_rms * weight


def rope_angles(head_dim: int, theta: float, positions: torch.Tensor):
    """src/layers/attention.cpp:63-69, 108-111: ``theta^(-2i/d)`` in double,
    stored as float; angle, cos and sin in double, rounded to float."""
    half = head_dim // 2
    exponent = -2.0 * np.arange(half, dtype=np.float64) / float(head_dim)
    inv_freq = np.power(np.float64(theta), exponent).astype(np.float32).astype(np.float64)
    angle = positions.double().cpu().numpy()[:, None] * inv_freq[None, :]
    return (torch.from_numpy(np.cos(angle)).float().to(positions.device),
            torch.from_numpy(np.sin(angle)).float().to(positions.device))


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """src/layers/attention.cpp:103-116: pairs ``(i, i + d/2)`` of every head;
    ``x`` is ``[tokens, heads, head_dim]``."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)


def attention(q, k, v, scale: float, window: int = 0):
    """src/layers/attention.cpp:261-338: for query head h the KV head is
    ``h // (heads / kv_heads)``; scores ``(q.k) * scale`` over positions
    ``0..p``; softmax with the maximum subtracted; weighted sum of values.
    ``q`` ``[T, heads, d]``, ``k``, ``v`` ``[T, kv_heads, d]`` of one sequence."""
    tokens, heads, _ = q.shape
    group = heads // k.shape[1]
    out = torch.zeros_like(q)
    for h in range(heads):
        g = h // group
        scores = (q[:, h, :] @ k[:, g, :].T) * scale                  # [T, T]
        index = torch.arange(tokens, device=q.device)
        mask = index[None, :] > index[:, None]
        if window > 0:
            mask = mask | (index[None, :] <= index[:, None] - window)
        scores = scores.masked_fill(mask, float("-inf"))
        weights = torch.softmax(scores, dim=-1)
        out[:, h, :] = weights @ v[:, g, :]
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """src/models/transformer_block.cpp:315-323: ``x * sigmoid(x)``."""
    return x * torch.sigmoid(x)


def feed_forward(h, gate_w, up_w, down_w):
    """src/models/transformer_block.cpp:312-325: ``down(silu(gate(h)) * up(h))``."""
    return (silu(h @ gate_w.T) * (h @ up_w.T)) @ down_w.T


def attention_block(h, weights, prefix, config, positions):
    """src/layers/attention.cpp:222-227, 341: projections, rotary encoding of
    queries and keys, attention, output projection."""
    heads = config["num_attention_heads"]
    kv_heads = config.get("num_key_value_heads", heads)
    head_dim = config.get("head_dim") or config["hidden_size"] // heads
    tokens = h.shape[0]
    q = (h @ weights[prefix + "self_attn.q_proj.weight"].T).view(tokens, heads, head_dim)
    k = (h @ weights[prefix + "self_attn.k_proj.weight"].T).view(tokens, kv_heads, head_dim)
    v = (h @ weights[prefix + "self_attn.v_proj.weight"].T).view(tokens, kv_heads, head_dim)
    cos, sin = rope_angles(head_dim, config["rope_theta"], positions)
    q, k = rope(q, cos, sin), rope(k, cos, sin)
    ctx = attention(q, k, v, 1.0 / math.sqrt(head_dim))
    return ctx.reshape(tokens, heads * head_dim) @ weights[prefix + "self_attn.o_proj.weight"].T


def decoder_layer(x, weights, layer: int, config, positions):
    """src/models/transformer_block.cpp:301-331: pre-norm block with two residual sums."""
    prefix = f"model.layers.{layer}."
    eps = config["rms_norm_eps"]
    h = rmsnorm(x, weights[prefix + "input_layernorm.weight"], eps)
    x = x + attention_block(h, weights, prefix, config, positions)
    h = rmsnorm(x, weights[prefix + "post_attention_layernorm.weight"], eps)
    return x + feed_forward(h, weights[prefix + "mlp.gate_proj.weight"],
                            weights[prefix + "mlp.up_proj.weight"],
                            weights[prefix + "mlp.down_proj.weight"])


def logits_of(config, weights, tokens) -> torch.Tensor:
    """Logits ``[len(tokens), vocab]`` at every position of one whole sequence
    (src/generation/generator.cpp:520-529 embedding, :554-568 layers, :773-774
    final norm and head)."""
    device = weights["model.embed_tokens.weight"].device
    ids = torch.tensor(list(tokens), dtype=torch.long, device=device)
    x = weights["model.embed_tokens.weight"][ids]
    positions = torch.arange(len(ids), device=device)
    for layer in range(config["num_hidden_layers"]):
        x = decoder_layer(x, weights, layer, config, positions)
    x = rmsnorm(x, weights["model.norm.weight"], config["rms_norm_eps"])
    head = (weights["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False)
            else weights["lm_head.weight"])
    return x @ head.T


def greedy(config, weights, prompt, max_new_tokens, stop_ids=()):
    """src/generation/generator.cpp:617-803 with temperature 0: returns prompt +
    generated ids; a stop id is kept and ends the sequence."""
    tokens = list(prompt)
    if max_new_tokens == 0 or (tokens and tokens[-1] in stop_ids):
        return tokens
    for _ in range(max_new_tokens):
        row = logits_of(config, weights, tokens)[-1]
        best = int(torch.argmax(row))          # first index among equals
        tokens.append(best)
        if best in stop_ids:
            break
    return tokens


def sample_reference(logits, temperature, top_k, top_p):
    """The distribution the reference's sampler draws from
    (src/generation/sampler.cpp:64-143): temperature, top-k (ties by lower
    index), softmax, top-p keeping the token that crosses the threshold,
    softmax again over the survivors.  Returns float64 probabilities ``[vocab]``."""
    values = np.asarray(logits, dtype=np.float32) / np.float32(temperature)
    vocab = len(values)
    order = sorted(range(vocab), key=lambda i: (-values[i], i))
    allowed = np.ones(vocab, dtype=bool)
    if 0 < top_k < vocab:
        allowed[order[top_k:]] = False
    weights = np.where(allowed, np.exp(values - values[allowed].max()), 0.0).astype(np.float32)
    total = weights.sum(dtype=np.float32)
    if top_p < 1.0:
        by_prob = sorted((i for i in range(vocab) if allowed[i]), key=lambda i: (-weights[i], i))
        cumulative, reached = np.float32(0.0), False
        for i in by_prob:
            if reached:
                allowed[i] = False
                continue
            cumulative += weights[i] / total
            if cumulative >= np.float32(top_p):
                reached = True
    final = np.where(allowed, np.exp(values.astype(np.float64) - values[allowed].max()), 0.0)
    return final / final.sum()
