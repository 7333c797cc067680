"""Parts alone, and a mixer that the framework does not know: a toy mixer with per-sequence
state of its own is defined here, registered, built into a model next to an attention layer
and stepped, with no change to the package's files."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_llama
from helpers import random_tokens

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class RunningMeanSpec:
    """x += (mean of h over this sequence's positions so far) . W^T"""
    hidden_size: int
    weight: str
    kind: str = "toy_running_mean"


def register_toy():
    from stratakv_b200.parts import CacheRequest, Mixer, TensorRequest, register_mixer

    class RunningMean(Mixer):
        @classmethod
        def expected_tensors(cls, spec):
            return {spec.weight: TensorRequest((spec.hidden_size, spec.hidden_size))}

        @classmethod
        def cache_request(cls, spec):
            return CacheRequest("none", state_bytes=4 * (spec.hidden_size + 1))      # running sum and count

        def bind(self, tensors):
            self.w = self.rt.upload(tensors[self.spec.weight], torch.float32)

        def forward(self, step, h, x, cache_entry, writes_cache=True):
            state = step.cache.state(cache_entry)
            start = 0
            for slot, q_len in zip(step.slots, step.q_lens):
                row = state[slot].view(torch.float32)
                rows = h[start:start + q_len].float()
                sums = row[:-1] + torch.cumsum(rows, dim=0)
                counts = row[-1] + torch.arange(1, q_len + 1, device=h.device, dtype=torch.float32)
                x[start:start + q_len] += (sums / counts[:, None]) @ self.w.T
                row[:-1] = sums[-1]
                row[-1] = counts[-1]
                start += q_len

    register_mixer("toy_running_mean", RunningMean)


def toy_model(dtype):
    from stratakv_b200 import Engine, EngineConfig
    from stratakv_b200.engine.model import expected_tensors
    from stratakv_b200.parts import (AttentionSpec, EmbeddingSpec, GatedMlpSpec, HeadSpec, LayerSpec, ModelSpec,
                                     NormSpec, RopeSpec, ScheduleEntry)
    from stratakv_b200.weights import random_tensors
    register_toy()
    hidden, vocab, ffn = 48, 120, 72
    def mlp(i):
        return GatedMlpSpec(hidden, ffn, "silu", f"l{i}.gate", f"l{i}.up", f"l{i}.down")
    layers = (
        LayerSpec(NormSpec(hidden, 1e-5, "l0.n1"),
                  AttentionSpec(hidden, 3, 1, 16, 0.25, RopeSpec(16, 777.0), "l0.q", "l0.k", "l0.v", "l0.o"),
                  NormSpec(hidden, 1e-5, "l0.n2"), mlp(0)),
        LayerSpec(NormSpec(hidden, 2e-5, "l1.n1"), RunningMeanSpec(hidden, "l1.mix"),
                  NormSpec(hidden, 2e-5, "l1.n2"), mlp(1)),
    )
    spec = ModelSpec("ToyForTests", hidden, vocab, EmbeddingSpec(vocab, hidden, "emb"), layers,
                     (ScheduleEntry(0, 0), ScheduleEntry(1, 1)), NormSpec(hidden, 1e-5, "norm"),
                     HeadSpec(vocab, hidden, "emb"))
    tensors = random_tensors(expected_tensors(spec), seed=5, dtype=torch.float32)
    engine = Engine(spec, tensors, EngineConfig(max_tokens=512, dtype=dtype, block_size=16), verbose=False)
    return engine, tensors


def toy_plain(tensors, tokens):
    """The same model from the plain parts, whole sequence."""
    w = {k: v.float() for k, v in tensors.items()}
    ids = torch.tensor(tokens)
    n = len(tokens)
    x = w["emb"][ids]
    h = plain_llama.rmsnorm(x, w["l0.n1"], 1e-5)
    cos, sin = plain_llama.rope_angles(16, 777.0, torch.arange(n))
    q = plain_llama.rope((h @ w["l0.q"].T).view(n, 3, 16), cos, sin)
    k = plain_llama.rope((h @ w["l0.k"].T).view(n, 1, 16), cos, sin)
    v = (h @ w["l0.v"].T).view(n, 1, 16)
    x = x + plain_llama.attention(q, k, v, 0.25).reshape(n, 48) @ w["l0.o"].T
    x = x + plain_llama.feed_forward(plain_llama.rmsnorm(x, w["l0.n2"], 1e-5), w["l0.gate"], w["l0.up"], w["l0.down"])
    h = plain_llama.rmsnorm(x, w["l1.n1"], 2e-5)
    means = torch.cumsum(h, dim=0) / torch.arange(1, n + 1)[:, None]
    x = x + means @ w["l1.mix"].T
    x = x + plain_llama.feed_forward(plain_llama.rmsnorm(x, w["l1.n2"], 2e-5), w["l1.gate"], w["l1.up"], w["l1.down"])
    return plain_llama.rmsnorm(x, w["norm"], 1e-5) @ w["emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    """In bfloat16 the decode steps fold the norms of the built-in parts into their projections; the toy
    mixer knows nothing of that, so the norm before it runs as a kernel and the one after it too."""
    from stratakv_b200 import StepEntry
    from helpers import tolerance
    engine, tensors = toy_model(dtype)
    if dtype == "bfloat16":
        tensors = {k: (v if v.dim() == 1 or k == "l1.mix" else v.to(torch.bfloat16).float()) for k, v in tensors.items()}
    assert engine.cache.state(1).shape == (engine.cache.max_slots, 4 * 49)
    assert len(engine.cache.groups) == 1 and engine.cache.entry_group[1] == (-1, -1)
    a, b = random_tokens(120, 30, seed=1), random_tokens(120, 11, seed=2)
    ref_a, ref_b = toy_plain(tensors, a).numpy(), toy_plain(tensors, b).numpy()
    rtol, atol = tolerance(dtype, ref_a)
    for round_ in range(2):                                  # the second round reuses slots: state must be zeroed
        sa, sb = engine.open_sequence(), engine.open_sequence()
        got = engine.step([StepEntry(sa, a[:20], [19]), StepEntry(sb, b[:4], [0, 3])]).cpu().numpy()
        np.testing.assert_allclose(got, np.stack([ref_a[19], ref_b[0], ref_b[3]]), rtol=rtol, atol=atol)
        for position in range(4, 11):
            got = engine.step([StepEntry(sa, [a[16 + position]], [0]), StepEntry(sb, [b[position]], [0])]).cpu().numpy()
            np.testing.assert_allclose(got, np.stack([ref_a[16 + position], ref_b[position]]), rtol=rtol, atol=atol)
        engine.close_sequence(sb)
        got = engine.step([StepEntry(sa, a[27:], [2])]).cpu().numpy()
        np.testing.assert_allclose(got[0], ref_a[29], rtol=rtol, atol=atol)
        engine.close_sequence(sa)
        assert engine.cache.all_free()


def test_parts_alone():
    """Each built-in part on its own: norm, feed-forward, attention mixer with its position encoding."""
    from stratakv_b200 import ops
    from stratakv_b200.cache import KVCache
    from stratakv_b200.parts import (AttentionSpec, CacheRequest, GatedMlpSpec, NormSpec, RopeSpec, Runtime,
                                     StepBatch, Workspace, part_class)
    device = torch.device("cuda")
    for dtype in (torch.float32, torch.bfloat16):
        rt = Runtime(dtype, device, Workspace(device), lambda d, hd: ops.kernels_for(d, hd, verbose=False), 32)
        tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
        g = torch.Generator().manual_seed(0)
        hidden, ffn, n = 40, 56, 9
        x = torch.randn(n, hidden, generator=g)
        # norm
        norm = part_class("norm", "rmsnorm")(NormSpec(hidden, 3e-4, "g"), rt)
        gamma = 1 + 0.1 * torch.randn(hidden, generator=g)
        norm.bind({"g": gamma})
        h = norm.forward(x.cuda())
        torch.testing.assert_close(h.float().cpu(), plain_llama.rmsnorm(x, gamma, 3e-4), **tol)
        # feed-forward adds into the residual stream
        mlp = part_class("ffn", "gated_mlp")(GatedMlpSpec(hidden, ffn, "silu", "g", "u", "d"), rt)
        w = {k: torch.randn(s, generator=g) * 0.2 for k, s in (("g", (ffn, hidden)), ("u", (ffn, hidden)), ("d", (hidden, ffn)))}
        mlp.bind(w)
        stream = x.cuda().clone()
        hq = h.float().cpu()
        mlp.forward(None, h, stream)
        wq = {k: v.to(dtype).float() for k, v in w.items()}
        torch.testing.assert_close(stream.cpu(), x + plain_llama.feed_forward(hq, wq["g"], wq["u"], wq["d"]), **tol)
        # attention over a fresh cache, two sequences
        spec = AttentionSpec(hidden, 4, 2, 32, 0.3, RopeSpec(32, 5000.0), "q", "k", "v", "o")
        attn = part_class("mixer", "attention")(spec, rt)
        aw = {k: torch.randn(s, generator=g) * 0.2 for k, s in (("q", (128, hidden)), ("k", (64, hidden)),
                                                                 ("v", (64, hidden)), ("o", (hidden, 128)))}
        attn.bind(aw)
        cache = KVCache([type(attn).cache_request(spec)], 8, 16, 2, dtype, device)
        s0, s1 = cache.acquire(), cache.acquire()
        cache.reserve({s0: 5, s1: 4})
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        step = StepBatch(2, 9, [s0, s1], [5, 4], [0, 0], 5, 5, i32([0] * 9), i32([0, 1, 2, 3, 4, 0, 1, 2, 3]),
                         i32([0] * 5 + [1] * 4), i32([0, 5, 9]), i32([5, 4]), i32([s0, s1]),
                         {0: i32(cache.block_table_rows(0, [s0, s1], 1))}, cache)
        stream = x.cuda().clone()
        attn.forward(step, h, stream, 0, True)
        aq = {k: v.to(dtype).float() for k, v in aw.items()}
        expect = x.clone()
        for lo, hi in ((0, 5), (5, 9)):
            t = hi - lo
            cos, sin = plain_llama.rope_angles(32, 5000.0, torch.arange(t))
            q = plain_llama.rope((hq[lo:hi] @ aq["q"].T).view(t, 4, 32), cos, sin)
            k = plain_llama.rope((hq[lo:hi] @ aq["k"].T).view(t, 2, 32), cos, sin)
            v = (hq[lo:hi] @ aq["v"].T).view(t, 2, 32)
            expect[lo:hi] += plain_llama.attention(q, k, v, 0.3).reshape(t, 128) @ aq["o"].T
        torch.testing.assert_close(stream.cpu(), expect, **tol)
