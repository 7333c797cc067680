"""The sampling kernels against the distribution the reference's sampler draws from."""
import numpy as np
import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu


def kernels():
    from stratakv_b200.ops import kernels_for
    return kernels_for(torch.float32, 64, verbose=False)


def draw(logits_row, n, temperature, top_k, top_p, seed=3):
    k = kernels()
    logits = torch.tensor(logits_row, dtype=torch.float32, device="cuda").repeat(n, 1).contiguous()
    out = torch.zeros(n, dtype=torch.int32, device="cuda")
    streams = torch.zeros(n, dtype=torch.int32, device="cuda")
    counters = torch.arange(n, dtype=torch.int32, device="cuda")
    k.sample(logits, out, temperature, top_k, top_p, seed, streams, counters)
    return out.cpu().numpy()


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.7, 5, 1.0), (1.3, 0, 0.8), (0.8, 40, 0.95),
                                                     (1.0, 1000, 0.999)])
def test_frequencies_match_the_reference_distribution(temperature, top_k, top_p):
    rng = np.random.default_rng(0)
    logits = (rng.standard_normal(331) * 2.0).astype(np.float32)
    expected = plain_llama.sample_reference(logits, temperature, top_k, top_p)
    n = 40000
    counts = np.bincount(draw(logits, n, temperature, top_k, top_p), minlength=331)
    assert counts[expected == 0].sum() == 0                   # nothing outside the kept set
    sigma = np.sqrt(n * expected * (1 - expected)) + 1.0
    assert (np.abs(counts - n * expected) < 5 * sigma).all()


def test_top_k_and_top_p_keep_what_the_reference_keeps():
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    assert set(draw(logits, 2000, 1.0, 2, 1.0)) == {0, 1}                 # tests/phase7_smoke.cpp:69-74
    assert set(draw(logits, 2000, 1.0, 0, 0.6)) == {0, 1}                 # the crossing token stays, :76-92
    assert set(draw(logits, 2000, 1.0, 0, 0.4)) == {0}
    assert set(draw(np.zeros(6, dtype=np.float32), 2000, 1.0, 2, 1.0)) == {0, 1}    # equal values: lower index first
    assert set(draw(logits, 200, 1.0, 1, 0.1)) == {0}


def test_draws_depend_on_seed_stream_and_counter_only():
    rng = np.random.default_rng(1)
    logits = torch.tensor(rng.standard_normal((6, 1000)), dtype=torch.float32, device="cuda")
    k = kernels()
    streams = torch.tensor([0, 1, 2, 3, 4, 5], dtype=torch.int32, device="cuda")
    counters = torch.tensor([9, 9, 9, 3, 3, 3], dtype=torch.int32, device="cuda")
    out = torch.zeros(6, dtype=torch.int32, device="cuda")
    k.sample(logits, out, 1.0, 0, 1.0, 11, streams, counters)
    first = out.clone()
    k.sample(logits, out, 1.0, 0, 1.0, 11, streams, counters)
    assert torch.equal(out, first)
    # a row alone gives the same token as in the batch
    one = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.sample(logits[4:5].contiguous(), one, 1.0, 0, 1.0, 11, streams[4:5].contiguous(), counters[4:5].contiguous())
    assert int(one) == int(first[4])
    k.sample(logits, out, 1.0, 0, 1.0, 12, streams, counters)
    assert not torch.equal(out, first)


def test_non_finite_logits_raise_the_flag():
    k = kernels()
    logits = torch.zeros(2, 50, device="cuda")
    logits[1, 3] = float("inf")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(2, dtype=torch.int32, device="cuda")
    zeros = torch.zeros(2, dtype=torch.int32, device="cuda")
    k.sample(logits, out, 1.0, 0, 1.0, 0, zeros, zeros, flag)
    assert int(flag) & 2


def test_long_rows_and_ties_take_the_other_paths_of_the_kernel():
    """Rows longer than the kernel keeps in shared memory are read again on every walk; many equal values make the
    passes over the index bits run; a top-k above what the list of elements in play holds keeps it from being made."""
    vocab = 50000
    rng = np.random.default_rng(5)
    logits = (-30.0 + 0.01 * rng.standard_normal(vocab)).astype(np.float32)
    logits[[7, 31000, 49999]] = [3.0, 2.5, 2.0]
    n = 6000
    drawn = draw(logits, n, 1.0, 3, 1.0)
    assert set(drawn) == {7, 31000, 49999}
    expected = np.exp([3.0, 2.5, 2.0]) / np.exp([3.0, 2.5, 2.0]).sum()
    counts = np.array([(drawn == i).sum() for i in (7, 31000, 49999)])
    assert (np.abs(counts - n * expected) < 5 * np.sqrt(n * expected * (1 - expected))).all()
    assert set(draw(logits, 500, 1.0, 0, 0.3)) == {7}                    # its share is 0.51: it crosses 0.3 alone
    assert set(draw(logits, 2000, 1.0, 0, 0.6)) == {7, 31000}            # 0.51 + 0.31 crosses 0.6
    # all values equal: the k lowest indices stay, whatever k
    flat = np.zeros(vocab, dtype=np.float32)
    assert set(draw(flat, 3000, 1.0, 5, 1.0)) == {0, 1, 2, 3, 4}
    assert set(draw(flat, 400, 0.7, 1, 1.0)) == {0}
    # more survivors than the list of elements in play holds
    slope = (-1e-4 * np.arange(vocab)).astype(np.float32)
    many = draw(slope, 4000, 1.0, 6000, 1.0)
    assert many.max() < 6000 and many.min() < 300 and (many > 3000).sum() > 1000
    # and the same three tokens on a row that does fit
    short = logits[:32000].copy()
    short[[7, 31000, 31999]] = [3.0, 2.5, 2.0]
    assert set(draw(short, 3000, 1.0, 3, 1.0)) == {7, 31000, 31999}
