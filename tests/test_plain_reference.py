"""The plain implementation itself: closed-form cases from the reference's own tests, and
the logits the reference's compiled CPU classes produced for one tiny model (tests/golden)."""
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_rope_closed_form():
    """Identity projections, two tokens: position 1 rotates (1, 0) by one radian
    (tests/phase6_smoke.cpp:60-96)."""
    cos, sin = plain_llama.rope_angles(2, 10000.0, torch.arange(2))
    x = torch.tensor([[[1.0, 0.0]], [[1.0, 0.0]]])
    out = plain_llama.rope(x, cos, sin)
    assert torch.allclose(out[0, 0], torch.tensor([1.0, 0.0]))
    assert torch.allclose(out[1, 0], torch.tensor([math.cos(1.0), math.sin(1.0)]), atol=1e-7)
    # the second pair of a 4-wide head turns at theta^(-1/2)
    cos, sin = plain_llama.rope_angles(4, 10000.0, torch.tensor([3]))
    assert abs(float(cos[0, 1]) - math.cos(3 * 0.01)) < 1e-7


def test_swiglu_closed_form():
    """One block with unit weights: out = 1 + n * sigmoid(n) * n with n = 1/sqrt(1 + 1e-5)
    (tests/phase6_smoke.cpp:128-147)."""
    n = 1.0 / math.sqrt(1.0 + 1e-5)
    h = plain_llama.rmsnorm(torch.ones(1, 1), torch.ones(1), 1e-5)
    out = 1.0 + plain_llama.feed_forward(h, torch.ones(1, 1), torch.ones(1, 1), torch.ones(1, 1))
    assert abs(float(out) - (1.0 + n / (1.0 + math.exp(-n)) * n)) < 1e-6


def test_attention_groups_and_mask():
    """Two query heads share one KV head; a token sees itself and what came before
    (tests/phase6_smoke.cpp:98-126)."""
    q = torch.zeros(3, 2, 2)
    k = torch.zeros(3, 1, 2)
    v = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]], [[4.0, 4.0]]])
    out = plain_llama.attention(q, k, v, 1.0)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[1, 1], (v[0, 0] + v[1, 0]) / 2)
    assert torch.allclose(out[2, 0], v[:, 0].mean(0))
    windowed = plain_llama.attention(q, k, v, 1.0, window=2)
    assert torch.allclose(windowed[2, 0], (v[1, 0] + v[2, 0]) / 2)


def test_sampler_reference_properties():
    """top-k keeps the k largest; top-p keeps the crossing token (tests/phase7_smoke.cpp:69-92)."""
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    p = plain_llama.sample_reference(logits, 1.0, 2, 1.0)
    assert p[2] == p[3] == 0 and abs(p[0] - 0.625) < 1e-6
    p = plain_llama.sample_reference(logits, 1.0, 0, 0.6)
    assert p[2] == p[3] == 0 and p[1] > 0                     # 0.5 < 0.6: the token that crosses is kept
    p = plain_llama.sample_reference(logits, 1.0, 0, 0.4)
    assert p[0] == 1.0                                        # the top token alone exceeds top_p
    tie = plain_llama.sample_reference(np.zeros(4, dtype=np.float32), 1.0, 2, 1.0)
    assert tie[0] == tie[1] == 0.5                            # equal values: lower index first


@pytest.mark.skipif(not (GOLDEN / "reference_logits_tiny_a.json").exists(), reason="no golden file")
def test_against_the_reference_cpu_classes():
    """tests/golden/make_golden.py built the reference's CPU library, ran a tiny model through
    its TransformerBlock / RMSNorm / Linear classes and stored the logits."""
    golden = json.loads((GOLDEN / "reference_logits_tiny_a.json").read_text())
    import sys
    sys.path.insert(0, str(GOLDEN))
    from golden_model import golden_weights
    config, weights = golden["config"], golden_weights(golden["config"], golden["seed"])
    digest = float(sum(float(w.double().abs().sum()) for w in weights.values()))
    if abs(digest - golden["weights_abs_sum"]) > 1e-6 * golden["weights_abs_sum"]:
        pytest.skip("this torch build draws other random weights than the one that made the golden file")
    for case in golden["cases"]:
        got = plain_llama.logits_of(config, weights, case["tokens"]).numpy()
        want = np.array(case["logits"], dtype=np.float32).reshape(got.shape)
        np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-6)
