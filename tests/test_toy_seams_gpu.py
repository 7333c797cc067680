"""Further parts that the framework does not know, defined here and registered without a change to
the package: a block arrangement with one norm and two branches, a layer without a feed-forward, an
embedding with a scale and a head that caps its logits, a feed-forward that routes each token to one
of two experts, and a position encoding with other pairs.  They are toys that show where another
architecture would plug in; none of them is a model of anyone's."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_llama
from helpers import random_tokens

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    vocab_size: int
    hidden_size: int
    weight: str
    scale: float
    kind: str = "toy_scaled_embedding"


@dataclass(frozen=True)
class CappedHeadSpec:
    vocab_size: int
    hidden_size: int
    weight: str
    cap: float
    kind: str = "toy_capped_head"


@dataclass(frozen=True)
class RoutedMlpSpec:
    """Each token goes to the expert whose router score is largest; ``x += expert(h) * score``."""
    hidden_size: int
    intermediate_size: int
    experts: int
    prefix: str
    kind: str = "toy_routed_mlp"


@dataclass(frozen=True)
class PairRopeSpec:
    """Rotary encoding over neighbouring pairs (2i, 2i+1) instead of (i, i + d/2)."""
    head_dim: int
    theta: float
    kind: str = "toy_rope_pairs"


def rotate_pairs(x, theta, positions):
    d = x.shape[-1]
    inv = theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
    angle = positions.double().cpu()[:, None] * inv[None, :]
    cos, sin = torch.cos(angle).float().to(x.device)[:, None], torch.sin(angle).float().to(x.device)[:, None]
    even, odd = x[..., 0::2], x[..., 1::2]
    return torch.stack([even * cos - odd * sin, even * sin + odd * cos], dim=-1).flatten(-2)


def register_toys():
    from stratakv_b200 import ops
    from stratakv_b200.parts import (FeedForward, Part, TensorRequest, part_class, register_arrangement,
                                     register_embedding, register_ffn, register_head, register_position)

    class ScaledEmbedding(part_class("embedding", "embedding")):
        graph_safe = True

        def forward(self, step, x, flags, stats=None):
            super().forward(step, x, flags, stats=None)
            x.mul_(self.spec.scale)
            if stats is not None:
                stats.invalidate()                    # the stream changed after the kernel wrote it

    class CappedHead(part_class("head", "linear_head")):
        folds_norm = False                            # takes finished rows only

        def forward(self, y, n_rows):
            logits = super().forward(y, n_rows)
            return torch.tanh(logits / self.spec.cap) * self.spec.cap

    class RoutedMlp(FeedForward):
        """Routing on the device, in float; the experts are the library's gated projections."""

        @classmethod
        def expected_tensors(cls, spec):
            found = {spec.prefix + "router": TensorRequest((spec.experts, spec.hidden_size))}
            for e in range(spec.experts):
                found[f"{spec.prefix}{e}.gate"] = TensorRequest((spec.intermediate_size, spec.hidden_size))
                found[f"{spec.prefix}{e}.up"] = TensorRequest((spec.intermediate_size, spec.hidden_size))
                found[f"{spec.prefix}{e}.down"] = TensorRequest((spec.hidden_size, spec.intermediate_size))
            return found

        def bind(self, tensors):
            from stratakv_b200.parts.ffn import pack_gate_up
            s = self.spec
            self.router = self.rt.upload(tensors[s.prefix + "router"], torch.float32)
            self.gate_up = [pack_gate_up(self.rt.upload(tensors[f"{s.prefix}{e}.gate"]),
                                         self.rt.upload(tensors[f"{s.prefix}{e}.up"])) for e in range(s.experts)]
            self.down = [self.rt.upload(tensors[f"{s.prefix}{e}.down"]) for e in range(s.experts)]

        def forward(self, step, h, x):
            kernels = self.rt.kernels()
            scores = torch.softmax(h.float() @ self.router.T, dim=-1)          # router logits in float
            weight, choice = scores.max(dim=-1)
            for e in range(self.spec.experts):
                rows = torch.nonzero(choice == e).flatten()
                if rows.numel() == 0:
                    continue
                mine = h[rows].contiguous()
                z = torch.empty(rows.numel(), self.spec.intermediate_size, dtype=h.dtype, device=h.device)
                kernels.linear(mine, self.gate_up[e], z, ops.MODE_GATED, "silu")
                out = torch.empty(rows.numel(), self.spec.hidden_size, dtype=torch.float32, device=h.device)
                kernels.linear(z, self.down[e], out, ops.MODE_STORE_F32)
                x[rows] += out * weight[rows, None]

    class PairRope:
        """No table to hand to the fused decode kernel: the attention part then uses the separate kernels."""
        role = "position"

        def __init__(self, spec, runtime):
            self.spec, self.rt = spec, runtime

        def ensure(self, positions):
            pass

        def rotate_and_store(self, step, qkv, q_out, k_cache, v_cache, block_table, num_heads, num_kv_heads,
                             head_dim, block_size, write_kv):
            n = qkv.shape[0]
            q_dim, kv_dim = num_heads * head_dim, num_kv_heads * head_dim
            q = rotate_pairs(qkv[:, :q_dim].view(n, num_heads, head_dim), self.spec.theta, step.positions)
            q_out.copy_(q.reshape(n, q_dim).to(q_out.dtype))
            if write_kv:
                k = rotate_pairs(qkv[:, q_dim:q_dim + kv_dim].view(n, num_kv_heads, head_dim), self.spec.theta,
                                 step.positions)
                v = qkv[:, q_dim + kv_dim:].view(n, num_kv_heads, head_dim)
                position = step.positions.long()
                block = block_table[step.token_seq.long(), position // block_size].long()
                k_cache[block, :, position % block_size] = k.to(k_cache.dtype)
                v_cache[block, :, position % block_size] = v.to(v_cache.dtype)

    def one_norm_two_branches(layer, step, x, entry):
        """x += mixer(norm(x)) + ffn(norm(x)): both branches read the same normalised rows."""
        if step.residual_stats is not None:
            step.residual_stats.expect(None)          # no norm of this block can be folded into a projection
        h = layer.mixer_norm.forward(x)
        branch = h.clone()                            # the mixer may use its input as scratch
        layer.mixer.forward(step, h, x, entry.cache, entry.writes_cache)
        layer.ffn.forward(step, branch, x)
        if step.residual_stats is not None:
            step.residual_stats.invalidate()

    def mixer_only(layer, step, x, entry):
        if step.residual_stats is not None:
            step.residual_stats.expect(None)
        layer.mixer.forward(step, layer.mixer_norm.forward(x), x, entry.cache, entry.writes_cache)
        if step.residual_stats is not None:
            step.residual_stats.invalidate()

    register_embedding("toy_scaled_embedding", ScaledEmbedding)
    register_head("toy_capped_head", CappedHead)
    register_ffn("toy_routed_mlp", RoutedMlp)
    register_position("toy_rope_pairs", PairRope)
    register_arrangement("toy_one_norm_two_branches", one_norm_two_branches)
    register_arrangement("toy_mixer_only", mixer_only)


HIDDEN, VOCAB, FFN, HEADS, KV_HEADS, HEAD_DIM, SCALE, CAP, THETA = 64, 150, 48, 4, 2, 16, 3.0, 0.5, 900.0


def toy_model(dtype):
    from stratakv_b200 import Engine, EngineConfig
    from stratakv_b200.engine.model import expected_tensors
    from stratakv_b200.parts import AttentionSpec, GatedMlpSpec, LayerSpec, ModelSpec, NormSpec, ScheduleEntry
    from stratakv_b200.weights import random_tensors
    register_toys()

    def attention(i):
        return AttentionSpec(HIDDEN, HEADS, KV_HEADS, HEAD_DIM, 0.25, PairRopeSpec(HEAD_DIM, THETA), f"l{i}.q", f"l{i}.k",
                             f"l{i}.v", f"l{i}.o")
    layers = (
        LayerSpec(NormSpec(HIDDEN, 1e-5, "l0.n"), attention(0), None,
                  GatedMlpSpec(HIDDEN, FFN, "silu", "l0.gate", "l0.up", "l0.down"), "toy_one_norm_two_branches"),
        LayerSpec(NormSpec(HIDDEN, 1e-5, "l1.n"), attention(1), arrangement="toy_mixer_only"),
        LayerSpec(NormSpec(HIDDEN, 1e-5, "l2.n1"), attention(2), NormSpec(HIDDEN, 1e-5, "l2.n2"),
                  RoutedMlpSpec(HIDDEN, FFN, 2, "l2.x.")),
    )
    spec = ModelSpec("ToySeams", HIDDEN, VOCAB, ScaledEmbeddingSpec(VOCAB, HIDDEN, "emb", SCALE), layers,
                     tuple(ScheduleEntry(i, i) for i in range(3)), NormSpec(HIDDEN, 1e-5, "norm"),
                     CappedHeadSpec(VOCAB, HIDDEN, "emb", CAP))
    tensors = random_tensors(expected_tensors(spec), seed=8, std=0.05, dtype=torch.bfloat16)
    engine = Engine(spec, tensors, EngineConfig(max_tokens=1024, dtype=dtype, block_size=16), verbose=False)
    return engine, tensors


def toy_plain(tensors, tokens):
    """The same model written out with the plain parts, whole sequence, float32 on the CPU."""
    w = {k: v.float() for k, v in tensors.items()}
    n = len(tokens)
    positions = torch.arange(n)
    x = w["emb"][torch.tensor(tokens)] * SCALE

    def attention(i, h):
        q = rotate_pairs((h @ w[f"l{i}.q"].T).view(n, HEADS, HEAD_DIM), THETA, positions)
        k = rotate_pairs((h @ w[f"l{i}.k"].T).view(n, KV_HEADS, HEAD_DIM), THETA, positions)
        v = (h @ w[f"l{i}.v"].T).view(n, KV_HEADS, HEAD_DIM)
        return plain_llama.attention(q, k, v, 0.25).reshape(n, HEADS * HEAD_DIM) @ w[f"l{i}.o"].T

    h = plain_llama.rmsnorm(x, w["l0.n"], 1e-5)
    x = x + attention(0, h) + plain_llama.feed_forward(h, w["l0.gate"], w["l0.up"], w["l0.down"])
    x = x + attention(1, plain_llama.rmsnorm(x, w["l1.n"], 1e-5))
    x = x + attention(2, plain_llama.rmsnorm(x, w["l2.n1"], 1e-5))
    h = plain_llama.rmsnorm(x, w["l2.n2"], 1e-5)
    scores = torch.softmax(h @ w["l2.x.router"].T, dim=-1)
    weight, choice = scores.max(dim=-1)
    routed = torch.zeros_like(x)
    for e in range(2):
        rows = choice == e
        routed[rows] = plain_llama.feed_forward(h[rows], w[f"l2.x.{e}.gate"], w[f"l2.x.{e}.up"], w[f"l2.x.{e}.down"])
    x = x + routed * weight[:, None]
    logits = plain_llama.rmsnorm(x, w["norm"], 1e-5) @ w["emb"].T
    return torch.tanh(logits / CAP) * CAP


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_seams_are_registered_built_and_stepped(dtype):
    from stratakv_b200 import StepEntry
    from helpers import tolerance
    engine, tensors = toy_model(dtype)
    a, b = random_tokens(VOCAB, 40, seed=1), random_tokens(VOCAB, 21, seed=2)
    ref_a, ref_b = toy_plain(tensors, a).numpy(), toy_plain(tensors, b).numpy()
    # router decisions on near-ties could differ in bfloat16; these sequences have none (checked by the margin)
    rtol, atol = tolerance(dtype, ref_a, noise=0.05)
    for round_ in range(2):
        sa, sb = engine.open_sequence(), engine.open_sequence()
        got = engine.step([StepEntry(sa, a[:30], [0, 29]), StepEntry(sb, b[:9], [8])]).float().cpu().numpy()
        np.testing.assert_allclose(got, np.stack([ref_a[0], ref_a[29], ref_b[8]]), rtol=rtol, atol=atol)
        for position in range(9, 19):
            got = engine.step([StepEntry(sa, [a[21 + position]], [0]), StepEntry(sb, [b[position]], [0])])
            np.testing.assert_allclose(got.float().cpu().numpy(), np.stack([ref_a[21 + position], ref_b[position]]),
                                       rtol=rtol, atol=atol)
        engine.close_sequence(sa)
        got = engine.step([StepEntry(sb, b[19:], [1])]).float().cpu().numpy()
        np.testing.assert_allclose(got[0], ref_b[20], rtol=rtol, atol=atol)
        engine.close_sequence(sb)
        assert engine.cache.all_free()
