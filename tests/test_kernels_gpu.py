"""Each kernel alone against a plain float32 computation of the same op, at sizes
other than the engine's (odd counts, sizes that are no power of two)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def lib(dtype, head_dim=64):
    from stratakv_b200.ops import kernels_for
    return kernels_for(dtype, head_dim, verbose=False)


def close(got, ref, dtype, scale=1.0):
    got, ref = got.float().cpu(), ref.float().cpu()
    if dtype == torch.float32:
        torch.testing.assert_close(got, ref, rtol=2e-5, atol=2e-6 * scale)
    else:
        torch.testing.assert_close(got, ref, rtol=1.6e-2, atol=1e-2 * scale)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,hidden,n", [(331, 80, 7), (1000, 2048, 33)])
def test_embed(dtype, vocab, hidden, n):
    k = lib(dtype)
    table = torch.randn(vocab, hidden, device="cuda").to(dtype)
    ids = torch.randint(0, vocab, (n,), device="cuda", dtype=torch.int32)
    out = torch.full((n, hidden), float("nan"), device="cuda")
    k.embed(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("build", DTYPES)
def test_convert_rounds_to_nearest_even(build):
    """Checkpoint tensors are converted on the device by the library's own kernel (the reference drops the low
    half of an FP32 weight, src/cuda/gemm_cuda.cu:74-83; this rounds to nearest even, as torch does)."""
    k = lib(build)
    generator = torch.Generator(device="cuda").manual_seed(3)
    values = torch.randn(100003, device="cuda", generator=generator) * 3
    # ties of the bfloat16 grid (the 16 bits below are exactly half), both parities, and special values
    ties = (torch.tensor([0x3F808000, 0x3F818000, 0xBF808000, 0x7F7F8000, 0x00008000, 0x00000001], dtype=torch.int64)
            .to(torch.int32).view(torch.float32).cuda())
    special = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), 65504.0, 70000.0, 1e-8, 3.4e38], device="cuda")
    source = torch.cat([values, ties, special])
    for src_dtype in (torch.float32, torch.float16, torch.bfloat16):
        stored = source.to(src_dtype)
        for dst_dtype in (torch.float32, torch.bfloat16, torch.float16):
            out = torch.full(stored.shape, 7.0, dtype=dst_dtype, device="cuda")
            k.convert(stored, out)
            assert torch.equal(out, stored.to(dst_dtype)), (src_dtype, dst_dtype)
    nan = torch.tensor([float("nan")], device="cuda")
    assert torch.isnan(k.convert(nan, torch.zeros(1, dtype=torch.bfloat16, device="cuda"))).all()
    with pytest.raises(Exception, match="float32, bfloat16 and float16 only"):
        k.convert(torch.zeros(4, dtype=torch.int32, device="cuda"), torch.zeros(4, device="cuda"))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden,eps", [(5, 80, 1e-5), (3, 2048, 1e-6), (9, 1000, 3e-3), (100, 264, 1e-5),
                                             (70, 2048, 1e-6), (65, 82, 1e-5)])
def test_rmsnorm(dtype, rows, hidden, eps):
    k = lib(dtype)
    x = torch.randn(rows, hidden, device="cuda") * 3.0
    gamma = 1.0 + 0.1 * torch.randn(hidden, device="cuda")
    out = torch.full((rows, hidden), float("nan"), device="cuda").to(dtype)
    k.rmsnorm(x, gamma, eps, out)
    xd = x.double()
    ref = (xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + eps) * gamma.double()).float()
    close(out, ref, dtype, scale=3.0)
    # with a row selection
    rows_index = torch.tensor([rows - 1, 0], device="cuda", dtype=torch.int32)
    picked = torch.full((2, hidden), float("nan"), device="cuda").to(dtype)
    k.rmsnorm(x, gamma, eps, picked, rows_index)
    close(picked, ref[rows_index.long()], dtype, scale=3.0)


def pack_gate_up(w):
    from stratakv_b200.parts.ffn import pack_gate_up as pack
    half = w.shape[0] // 2
    return pack(w[:half].contiguous(), w[half:].contiguous())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 48, 64), (3, 331, 80), (8, 256, 2048), (9, 100, 264), (17, 96, 96),
                                   (33, 80, 176), (64, 512, 512), (70, 130, 520), (200, 64, 72),
                                   (32, 2048, 5632), (64, 2560, 2048), (100, 1000, 1032), (128, 384, 4096),
                                   (5, 12288, 264),           # 768 row tiles of the small-step kernel
                                   (20, 48, 64), (40, 256, 192), (64, 256, 1280), (128, 512, 1344),   # two chunks a copy: one
                                                              # chunk in all, an odd count, parts of K of five and of seven chunks
                                   (20, 19000, 136), (64, 19072, 520), (100, 20000, 264)])   # more 128-row tiles than
                                                              # SMs: the swapped kernel's shallow rings, two blocks an SM
def test_linear_store_and_add(dtype, M, N, K):
    from stratakv_b200 import ops
    k = lib(dtype)
    a = torch.randn(M, K, device="cuda").to(dtype)
    w = (torch.randn(N, K, device="cuda") / math.sqrt(K)).to(dtype)
    ref = a.double() @ w.double().T
    bound = (a.double().abs() @ w.double().abs().T)
    out = torch.full((M, N), float("nan"), device="cuda")
    k.linear(a, w, out, ops.MODE_STORE_F32)
    # accumulation in float: error grows with the sum of |a||w| (tests/gemv_smoke.cu:259-272)
    assert ((out.double() - ref).abs() <= 2e-6 * (1 + bound)).all()
    out_t = torch.full((M, N), float("nan"), device="cuda").to(dtype)
    k.linear(a, w, out_t, ops.MODE_STORE)
    rounding = 0.0 if dtype == torch.float32 else 2.0 ** -8       # one rounding of the result to bfloat16
    assert ((out_t.double() - ref).abs() <= 2e-6 * (1 + bound) + rounding * ref.abs()).all()
    base = torch.randn(M, N, device="cuda")
    acc = base.clone()
    k.linear(a, w, acc, ops.MODE_ADD_F32)
    k.linear(a, w, acc, ops.MODE_ADD_F32)       # a second call must add again, not overwrite
    assert ((acc.double() - (base.double() + 2 * ref)).abs() <= 4e-6 * (1 + bound) + 1e-6 * base.abs()).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,F,K", [(1, 176, 64), (5, 104, 80), (8, 5632, 2048), (40, 256, 96), (130, 24, 72),
                                   (24, 72, 264), (64, 5632, 2048), (128, 200, 520), (48, 9600, 200)])   # (the last: shallow rings)
@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
def test_linear_gated(dtype, M, F, K, activation):
    """``act(gate) * up`` in the epilogue of one projection, for every activation the kernels name (the
    Llama feed-forward uses silu; the other one shows that the parameter is carried by every kernel)."""
    from stratakv_b200 import ops
    k = lib(dtype)
    a = torch.randn(M, K, device="cuda").to(dtype)
    w = (torch.randn(2 * F, K, device="cuda") / math.sqrt(K)).to(dtype)      # gate rows, then up rows
    out = torch.full((M, F), float("nan"), device="cuda").to(dtype)
    k.linear(a, pack_gate_up(w), out, ops.MODE_GATED, activation)
    gate = a.double() @ w[:F].double().T
    up = a.double() @ w[F:].double().T
    act = gated_activation(gate, activation)
    ref = act * up
    # float accumulation errs by at most ~2e-6 (1 + sum |a||w|) in gate and in up
    # (tests/gemv_smoke.cu:259-272); both activations have slopes below 1.2
    err_gate = 2e-6 * (1 + a.double().abs() @ w[:F].double().abs().T)
    err_up = 2e-6 * (1 + a.double().abs() @ w[F:].double().abs().T)
    rounding = 1e-6 if dtype == torch.float32 else 2.0 ** -8
    allowed = 1.2 * err_gate * up.abs() + act.abs() * err_up + rounding * ref.abs() + 1e-9
    assert ((out.double() - ref).abs() <= allowed).all()


def gated_activation(gate, name):
    if name == "silu":
        return gate * torch.sigmoid(gate)
    return torch.nn.functional.gelu(gate, approximate="tanh")


def _products(a, w, chunk=512):
    """``a . w^T`` and ``|a| . |w|^T`` in double on the GPU, a few hundred rows at a time."""
    wd = w.double()
    wa = wd.abs()
    ref = torch.cat([a[i:i + chunk].double() @ wd.T for i in range(0, a.shape[0], chunk)])
    bound = torch.cat([a[i:i + chunk].double().abs() @ wa.T for i in range(0, a.shape[0], chunk)])
    return ref, bound


# Shapes of the projections of real models (hidden 2048, feed-forward 5632, vocabulary 32000, and an odd
# vocabulary of 32001 whose rows are no multiple of 16 bytes, so that threads store instead of the copy
# engine).  They make the persistent tensor-memory kernel walk several tiles per block, wrap its ring of
# stages many times (K / 64 steps over four stages), use both tile widths and add into many row tiles.
@pytest.mark.parametrize("M,N,K,modes", [
    (129, 2048, 2048, "store_f32 store add"),        # 128-wide tiles, one tile per block, a tail of one row
    (300, 2560, 2048, "store_f32 store add"),        # the q|k|v projection of a short prompt
    (2048, 2560, 2048, "store_f32 add store"),       # 160-wide tiles for the float epilogues, 256-wide for bfloat16 (160 tiles on 148 blocks)
    (2048, 11264, 520, "gated"),                     # 256-wide tiles: 704 of them, five a block, a short inner size
    (2048, 2048, 5632, "store add"),                 # the down projection: 88 steps of K
    (4096, 2048, 5632, "add"),                       # 256 tiles, residual sum through the copy engine
    (2048, 11264, 2048, "gated"),                    # gate and up: 704 tiles, almost five per block
    (4096, 32000, 2048, "store_f32"),                # the output head over every position: 27 tiles per block
    (300, 32001, 2048, "store_f32 store add"),       # rows of an odd width: stored by the threads
    (2048, 32001, 2048, "store_f32"),
    (1000, 4112, 1032, "store_f32 store add gated"),  # tails in M, N and K at once
    (2048, 2500, 2048, "store_f32 add"),             # 160-wide tiles (256 of them, five stages), the last one clipped
    (1500, 2501, 520, "store_f32 store add"),        # 160-wide tiles whose rows the threads store themselves
    (1000, 4112, 5200, "store_f32 store add gated"),  # pairs of blocks on 256 x 256 tiles: tails in M (the pair's second
                                                     # block has 104 live rows in the last tile), N and K at once
    (1100, 2560, 6000, "store gated"),               # pairs: the second block of the last row tile has no live row
    (1500, 2501, 5208, "store_f32 store add"),       # pairs whose rows the threads store themselves
    (7000, 512, 5632, "store add"),                  # pairs: so many rows that they are walked in two bands (14 + 14 row tiles)
    (5000, 256, 8192, "store_f32 add"),              # 128-wide tiles in two bands (20 + 20 row tiles)
])
def test_linear_tiled_tensor_memory_kernel_at_model_sizes(M, N, K, modes):
    """tests/gemv_smoke.cu:329-357 takes the reference's kernels to the model's shapes with a bound from
    the sum of |a||w| (:259-272); the same here for steps of more than 128 tokens."""
    from stratakv_b200 import ops
    dtype = torch.bfloat16
    k = lib(dtype)
    a = torch.randn(M, K, device="cuda").to(dtype)
    w = (torch.randn(N, K, device="cuda") / math.sqrt(K)).to(dtype)
    ref, bound = _products(a, w)
    allowed = 2e-6 * (1 + bound)
    for mode in modes.split():
        if mode == "store_f32":
            out = torch.full((M, N), float("nan"), device="cuda")
            k.linear(a, w, out, ops.MODE_STORE_F32)
            assert ((out.double() - ref).abs() <= allowed).all(), mode
        elif mode == "store":
            out = torch.full((M, N), float("nan"), device="cuda").to(dtype)
            k.linear(a, w, out, ops.MODE_STORE)
            assert ((out.double() - ref).abs() <= allowed + 2.0 ** -8 * ref.abs()).all(), mode
        elif mode == "add":
            base = torch.randn(M, N, device="cuda")
            acc = base.clone()
            k.linear(a, w, acc, ops.MODE_ADD_F32)
            k.linear(a, w, acc, ops.MODE_ADD_F32)       # adds again
            assert ((acc.double() - (base.double() + 2 * ref)).abs() <= 2 * allowed + 1e-6 * base.abs()).all(), mode
        else:
            F = N // 2
            out = torch.full((M, F), float("nan"), device="cuda").to(dtype)
            gate, up = ref[:, :F], ref[:, F:]
            for activation in ("silu", "gelu_tanh"):
                k.linear(a, pack_gate_up(w), out, ops.MODE_GATED, activation)
                act = gated_activation(gate, activation)
                want = act * up
                slack = 1.2 * allowed[:, :F] * up.abs() + act.abs() * allowed[:, F:] + 2.0 ** -8 * want.abs() + 1e-9
                assert ((out.double() - want).abs() <= slack).all(), (mode, activation)
        torch.cuda.synchronize()
        assert int(k.error_flag.item()) == 0


def test_the_shapes_of_these_tests_reach_every_tensor_memory_kernel():
    """The launcher picks a kernel by a cost rule; if the rule moved, the tests above and below could lose a kernel
    without failing.  On a GPU of 148 SMs these shapes, which those tests bring, go where their comments say."""
    from stratakv_b200 import ops
    k = lib(torch.bfloat16)
    if torch.cuda.get_device_properties(0).multi_processor_count != 148:
        pytest.skip("the expectations are those of 148 SMs")
    assert k.linear_form(100, 2048, 2048, ops.MODE_STORE) == "few_tokens"
    assert k.linear_form(129, 2048, 2048, ops.MODE_STORE) == "tile_128"
    assert k.linear_form(2048, 2500, 2048, ops.MODE_ADD_F32) == "tile_160"
    assert k.linear_form(2048, 2560, 2048, ops.MODE_STORE) == "tile_256"
    assert k.linear_form(2048, 2560, 2048, ops.MODE_QKV_ROPE) == "tile_256"
    assert k.linear_form(2048, 11264, 520, ops.MODE_GATED) == "tile_256"            # a short inner size: no pair
    assert k.linear_form(2048, 2048, 2048, ops.MODE_ADD_F32) == "tile_256"      # one short tile a block: no pair
    assert k.linear_form(5000, 256, 8192, ops.MODE_STORE_F32) == "tile_128"
    for M, N, K, mode in [(2048, 11264, 2048, ops.MODE_GATED), (2048, 2048, 5632, ops.MODE_ADD_F32),
                          (1000, 4112, 5200, ops.MODE_GATED), (1000, 4112, 5200, ops.MODE_STORE),
                          (1100, 2560, 6000, ops.MODE_STORE), (1500, 2501, 5208, ops.MODE_ADD_F32),
                          (7000, 512, 5632, ops.MODE_ADD_F32),
                          (1000, 3072, 5120, ops.MODE_QKV_ROPE), (900, 3136, 5200, ops.MODE_QKV_ROPE)]:
        assert k.linear_form(M, N, K, mode) == "pair_256", (M, N, K, mode)


class _Norm:
    """Stands for a norm part: all the kernels want of it is its weight and eps."""
    def __init__(self, gamma, eps):
        from types import SimpleNamespace
        self.gamma, self.spec = gamma, SimpleNamespace(eps=eps)


def _stats(rows, width, dtype=torch.bfloat16, spare=0):
    from stratakv_b200.residual import ResidualStats
    nan = lambda *shape: torch.full(shape, float("nan"), device="cuda")
    return ResidualStats(nan(rows, width).to(dtype), nan(rows), nan(rows, (width + 15) // 16 + spare),
                         torch.zeros(1, device="cuda", dtype=torch.int32))


def _folded(stats, norm, rows=None):
    from stratakv_b200.residual import NormedRows
    assert stats.ready_for(norm)
    return NormedRows(stats.scaled, stats.row_scale, rows, stats.partials, stats.n_partials, norm.spec.eps)


@pytest.mark.parametrize("M,N,K,hidden_out", [(1, 176, 64, 72), (5, 104, 80, 40), (8, 2560, 2048, 2048),
                                              (16, 96, 1024, 1000), (33, 48, 96, 104), (64, 256, 4096, 512)])
def test_linear_with_folded_norm(M, N, K, hidden_out):
    """RMSNorm folded into the projections around it: the kernel that writes the stream (the embedding,
    a residual-add projection) leaves the row times the norm's weight and the row's factor, the
    projection after the norm applies the factor; together they are the norm, then the projection
    (src/layers/rmsnorm.cpp:63-97)."""
    from stratakv_b200 import ops
    dtype = torch.bfloat16
    k = lib(dtype)
    norm_a = _Norm((1 + 0.2 * torch.randn(K, device="cuda")).float(), 3e-5)
    norm_b = _Norm((1 + 0.2 * torch.randn(K, device="cuda")).float(), 2e-6)
    w = (torch.randn(N, K, device="cuda") / math.sqrt(K)).to(dtype)
    rows = torch.randperm(M, device="cuda").to(torch.int32)[: max(1, M // 2)]
    x = torch.empty(M, K, device="cuda")
    stats = _stats(M, K, spare=3)

    def check(norm):
        eps = norm.spec.eps
        if stats.consumer_sums:        # few rows: partial sums of squares for the consumer to add up
            assert stats.n_partials > 0
            sums = stats.partials[:, :stats.n_partials].double().sum(-1)
            assert torch.allclose(sums, (x.double() ** 2).sum(-1), rtol=1e-5, atol=0)
        else:                          # more: the writer's last block has made the factor
            assert stats.n_partials == 0
            factor = torch.rsqrt((x.double() ** 2).mean(-1) + eps)
            assert torch.allclose(stats.row_scale.double(), factor, rtol=1e-5, atol=0)
        assert torch.equal(stats.scaled, (x * norm.gamma).to(dtype))
        assert int(stats.counter) == 0
        for selected in (None, rows):
            m = M if selected is None else selected.numel()
            fused = torch.full((m, N), float("nan"), device="cuda")
            k.linear(_folded(stats, norm, selected), w, fused, ops.MODE_STORE_F32)
            xs = x.double() if selected is None else x.double()[selected.long()]
            exact_h = xs * torch.rsqrt((xs ** 2).mean(-1, keepdim=True) + eps) * norm.gamma.double()
            ref = exact_h @ w.double().T
            # the activations are rounded to bfloat16 once (half a unit in the last of 8 bits)
            bound = 2.0 ** -8 * (exact_h.abs() @ w.double().abs().T) + 1e-5
            assert ((fused.double() - ref).abs() <= bound).all()
            h = torch.empty(m, K, device="cuda", dtype=dtype)
            k.rmsnorm(x, norm.gamma, eps, h, selected)
            separate = torch.empty(m, N, device="cuda")
            k.linear(h, w, separate, ops.MODE_STORE_F32)
            assert ((fused - separate).abs().double() <= bound).all()

    # 1. the stream from the embedding
    vocab = 37
    table = torch.randn(vocab, K, device="cuda").to(dtype)
    ids = torch.randint(0, vocab, (M,), device="cuda", dtype=torch.int32)
    stats.expect(norm_a)
    k.embed(table, ids, x, stats=stats)
    assert stats.ready_for(norm_a) and not stats.ready_for(norm_b)
    assert torch.equal(x, table[ids.long()].float())
    check(norm_a)
    # 2. the stream after a residual-add projection, twice (the counter must come back to zero)
    for _ in range(2):
        a = torch.randn(M, hidden_out, device="cuda").to(dtype)
        w_add = (torch.randn(K, hidden_out, device="cuda") / math.sqrt(hidden_out)).to(dtype)
        plain = x.clone()
        k.linear(a, w_add, plain, ops.MODE_ADD_F32)
        stats.expect(norm_b)
        k.linear(a, w_add, x, ops.MODE_ADD_F32, stats=stats)
        if M <= 16:
            assert torch.equal(x, plain)                                 # the same kernel: the sum itself is unchanged
        else:                                                            # above 16 tokens the plain call is another kernel
            slack = 2e-6 * (1 + a.double().abs() @ w_add.double().abs().T) + 1e-6 * plain.double().abs()
            assert ((x.double() - plain.double()).abs() <= slack).all()
        assert stats.ready_for(norm_b)
        check(norm_b)
    # 3. a gated projection takes the folded norm too
    F = 64
    w_gu = (torch.randn(2 * F, K, device="cuda") / math.sqrt(K)).to(dtype)
    z = torch.empty(M, F, device="cuda", dtype=dtype)
    k.linear(_folded(stats, norm_b), pack_gate_up(w_gu), z, ops.MODE_GATED, "silu")
    xs = x.double()
    exact_h = xs * torch.rsqrt((xs ** 2).mean(-1, keepdim=True) + norm_b.spec.eps) * norm_b.gamma.double()
    gate, up = exact_h @ w_gu[:F].double().T, exact_h @ w_gu[F:].double().T
    ref = gate * torch.sigmoid(gate) * up
    # the activations' rounding moves gate and up by at most 2^-8 sum |h||w| each (silu has slope <= 1.1),
    # and the result is rounded to bfloat16
    err_gate = 2.0 ** -8 * (exact_h.abs() @ w_gu[:F].double().abs().T)
    err_up = 2.0 ** -8 * (exact_h.abs() @ w_gu[F:].double().abs().T)
    allowed = 1.1 * err_gate * (up.abs() + err_up) + (gate * torch.sigmoid(gate)).abs() * err_up + 2.0 ** -8 * ref.abs() + 1e-6
    assert ((z.double() - ref).abs() <= allowed).all()
    # 4. nobody to read the statistics: the kernel leaves none
    stats.expect(None)
    k.linear(a, w_add, x, ops.MODE_ADD_F32, stats=stats)
    assert not stats.ready_for(norm_b)


def test_folded_norm_refusals():
    from stratakv_b200 import ops
    from stratakv_b200.ops import KernelError
    from stratakv_b200.residual import NormedRows
    k = lib(torch.bfloat16)
    x = torch.zeros(80, 64, device="cuda")
    stats = _stats(80, 64)
    w = torch.zeros(32, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(KernelError, match="one factor per row"):
        k.linear(NormedRows(stats.scaled, stats.row_scale[:5]), w, torch.zeros(80, 32, device="cuda"),
                 ops.MODE_STORE_F32)
    with pytest.raises(KernelError, match="at most 64 tokens"):
        k.linear(NormedRows(stats.scaled, stats.row_scale), w, torch.zeros(80, 32, device="cuda"),
                 ops.MODE_STORE_F32)
    with pytest.raises(KernelError, match="partial sums do not match"):
        k.linear(NormedRows(stats.scaled[:8], stats.row_scale[:8], None, stats.partials[:8], 9, 1e-5), w,
                 torch.zeros(8, 32, device="cuda"), ops.MODE_STORE_F32)
    # more rows than the kernel folds a norm for: the sum is made, nothing is left for the norm
    norm = _Norm(torch.ones(64, device="cuda"), 1e-5)
    stats.expect(norm)
    stats.filled()
    a = torch.zeros(80, 32, device="cuda", dtype=torch.bfloat16)
    k.linear(a, torch.zeros(64, 32, device="cuda", dtype=torch.bfloat16), x, ops.MODE_ADD_F32, stats=stats)
    assert not stats.ready_for(norm)


def test_linear_refuses_bad_sizes():
    from stratakv_b200 import ops
    from stratakv_b200.ops import KernelError
    k = lib(torch.bfloat16)
    a = torch.zeros(2, 12, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(16, 12, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(KernelError, match="multiple of 8"):
        k.linear(a, w, torch.zeros(2, 16, device="cuda"), ops.MODE_STORE_F32)
    with pytest.raises(KernelError, match="CUDA tensor"):
        k.linear(a.cpu(), w, torch.zeros(2, 16, device="cuda"), ops.MODE_STORE_F32)


def paged_setup(dtype, lengths, new, heads, kv_heads, head_dim, block_size, seed):
    """Random q/k/v for sequences with ``lengths[i]`` cached tokens after a step that
    adds ``new[i]``; blocks are handed out in a scrambled order."""
    g = torch.Generator().manual_seed(seed)
    n_seq = len(lengths)
    width = max(-(-l // block_size) for l in lengths)
    n_blocks = n_seq * width + 3
    order = torch.randperm(n_blocks, generator=g).tolist()
    table = torch.zeros(n_seq, width, dtype=torch.int32)
    for s in range(n_seq):
        for b in range(-(-lengths[s] // block_size)):
            table[s, b] = order.pop()
    k_cache = torch.zeros(n_blocks, kv_heads, block_size, head_dim)
    v_cache = torch.zeros_like(k_cache)
    keys = [torch.randn(l, kv_heads, head_dim, generator=g) for l in lengths]
    values = [torch.randn(l, kv_heads, head_dim, generator=g) for l in lengths]
    for s in range(n_seq):
        for j in range(lengths[s]):
            k_cache[table[s, j // block_size], :, j % block_size] = keys[s][j]
            v_cache[table[s, j // block_size], :, j % block_size] = values[s][j]
    positions, token_seq = [], []
    for s in range(n_seq):
        positions += list(range(lengths[s] - new[s], lengths[s]))
        token_seq += [s] * new[s]
    q = torch.randn(len(positions), heads, head_dim, generator=g)
    to = lambda t: t.to("cuda").to(dtype)
    return dict(q=to(q), k_cache=to(k_cache), v_cache=to(v_cache), table=table.cuda(),
                positions=torch.tensor(positions, dtype=torch.int32).cuda(),
                token_seq=torch.tensor(token_seq, dtype=torch.int32).cuda(),
                keys=keys, values=values)


def attention_reference(setup, dtype, heads, kv_heads, scale, window=0):
    q = setup["q"].float().cpu()
    out = torch.zeros_like(q)
    group = heads // kv_heads
    for t in range(q.shape[0]):
        s, pos = int(setup["token_seq"][t]), int(setup["positions"][t])
        lo = max(0, pos - window + 1) if window else 0
        keys = setup["keys"][s][lo:pos + 1].to(dtype).double()
        values = setup["values"][s][lo:pos + 1].to(dtype).double()
        for h in range(heads):
            weights = torch.softmax((keys[:, h // group] @ q[t, h].double()) * scale, dim=0)
            out[t, h] = (weights @ values[:, h // group]).float()
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size,lengths,new,window", [
    (4, 2, 16, 16, [5, 40, 17], [5, 40, 17], 0),          # prompts from the start
    (6, 3, 48, 16, [33, 1, 100], [1, 1, 1], 0),           # one new token each
    (8, 1, 64, 64, [70, 129], [6, 65], 0),                # continuing a prompt
    (5, 5, 128, 32, [300], [1], 0),
    (4, 2, 32, 16, [90, 45], [90, 1], 20),                # a window of 20 keys
])
def test_attention(dtype, heads, kv_heads, head_dim, block_size, lengths, new, window):
    k = lib(dtype, head_dim)
    setup = paged_setup(dtype, lengths, new, heads, kv_heads, head_dim, block_size, seed=head_dim + heads)
    n = setup["q"].shape[0]
    out = torch.full((n, heads * head_dim), float("nan"), device="cuda").to(dtype)
    scale = 0.37 / math.sqrt(head_dim)
    k.attention(setup["q"].view(n, -1), setup["k_cache"], setup["v_cache"], setup["table"], setup["positions"],
                setup["token_seq"], out, heads, kv_heads, head_dim, block_size, scale, window)
    ref = attention_reference(setup, dtype, heads, kv_heads, scale, window).view(n, -1)
    close(out, ref, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(dtype):
    """One key among hundreds is made to dominate: the output must be that key's value."""
    heads, kv_heads, head_dim, block_size = 4, 2, 32, 16
    k = lib(dtype, head_dim)
    for far in (0, 15, 16, 257, 511):
        setup = paged_setup(dtype, [512], [1], heads, kv_heads, head_dim, block_size, seed=far)
        q = setup["q"].float()
        key = 8.0 * q[0, 0] / q[0, 0].norm()                   # aligned with head 0's query
        block = int(setup["table"][0, far // block_size])
        setup["k_cache"][block, 0, far % block_size] = key.to(dtype)
        setup["keys"][0][far, 0] = key.cpu()
        out = torch.zeros(1, heads * head_dim, device="cuda").to(dtype)
        k.attention(setup["q"].view(1, -1), setup["k_cache"], setup["v_cache"], setup["table"],
                    setup["positions"], setup["token_seq"], out, heads, kv_heads, head_dim, block_size,
                    4.0, 0)
        ref = attention_reference(setup, dtype, heads, kv_heads, 4.0).view(1, -1)
        close(out, ref, dtype)
        want = setup["values"][0][far, 0].to(dtype).float()
        torch.testing.assert_close(out[0, :head_dim].float().cpu(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size", [(4, 2, 16, 16), (3, 3, 80, 64), (8, 2, 128, 32)])
def test_rope_kv_write(dtype, heads, kv_heads, head_dim, block_size):
    from stratakv_b200.parts.position import rope_table
    k = lib(dtype, head_dim)
    lengths, new = [37, 5, 130], [37, 1, 66]
    setup = paged_setup(dtype, lengths, new, heads, kv_heads, head_dim, block_size, seed=3)
    n = setup["q"].shape[0]
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(n, (heads + 2 * kv_heads) * head_dim, generator=g).cuda()
    theta = 25000.0
    table = torch.from_numpy(rope_table(head_dim, theta, 256)).cuda()
    k_cache = torch.full_like(setup["k_cache"], 7.0)
    v_cache = torch.full_like(setup["v_cache"], 7.0)
    q_out = torch.full((n, heads * head_dim), float("nan"), device="cuda").to(dtype)
    k.rope_kv_write(qkv, table, setup["positions"], setup["token_seq"], setup["table"], q_out, k_cache, v_cache,
                    heads, kv_heads, head_dim, block_size, True)
    # plain: angles in double, rotation in float
    half = head_dim // 2
    pos = setup["positions"].cpu().double()
    inv = torch.tensor([theta ** (-2.0 * i / head_dim) for i in range(half)], dtype=torch.float64).float().double()
    angle = pos[:, None] * inv[None, :]
    cos, sin = torch.cos(angle).float(), torch.sin(angle).float()
    src = qkv.cpu()
    q = src[:, :heads * head_dim].view(n, heads, head_dim)
    kk = src[:, heads * head_dim:(heads + kv_heads) * head_dim].view(n, kv_heads, head_dim)
    vv = src[:, (heads + kv_heads) * head_dim:].view(n, kv_heads, head_dim)
    rot = lambda x: torch.cat([x[..., :half] * cos[:, None] - x[..., half:] * sin[:, None],
                               x[..., :half] * sin[:, None] + x[..., half:] * cos[:, None]], -1)
    exact = dtype == torch.float32
    got_q = q_out.float().cpu().view(n, heads, head_dim)
    torch.testing.assert_close(got_q, rot(q).to(dtype).float(), rtol=0 if exact else 8e-3, atol=1e-6 if exact else 1e-2)
    kc, vc = k_cache.float().cpu(), v_cache.float().cpu()
    touched = torch.zeros(kc.shape[0], block_size, dtype=torch.bool)
    for t in range(n):
        s, p = int(setup["token_seq"][t]), int(setup["positions"][t])
        block = int(setup["table"][s, p // block_size])
        touched[block, p % block_size] = True
        torch.testing.assert_close(kc[block, :, p % block_size], rot(kk)[t].to(dtype).float(),
                                   rtol=0 if exact else 8e-3, atol=1e-6 if exact else 1e-2)
        assert torch.equal(vc[block, :, p % block_size], vv[t].to(dtype).float())
    # rows no token of this step owns keep their old contents
    assert (kc.permute(0, 2, 1, 3)[~touched] == 7.0).all() and (vc.permute(0, 2, 1, 3)[~touched] == 7.0).all()


def test_argmax_lowest_index_among_equals():
    k = lib(torch.float32)
    logits = torch.randn(5, 1000, device="cuda")
    logits[0, 700] = logits[0, 20] = 50.0
    logits[3, 999] = 60.0
    out = torch.zeros(5, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.argmax(logits, out, flag)
    ref = torch.argmax(logits, dim=-1).cpu()
    ref[0] = 20
    assert out.cpu().tolist() == ref.tolist() and int(flag) == 0
    logits[2, 5] = float("nan")
    k.argmax(logits, out, flag)
    assert int(flag) & 2


@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size,lengths,window,splits", [
    (4, 2, 16, 16, [5, 40, 17, 1], 0, 1),
    (6, 3, 48, 16, [33, 1, 100], 0, 3),
    (32, 4, 64, 64, [700, 129, 2048, 64], 0, 8),          # the TinyLlama head layout
    (8, 8, 128, 32, [300, 31], 0, 2),                     # no sharing of KV heads
    (20, 1, 32, 16, [90, 45], 0, 4),                      # more than 16 query heads on one KV head
    (4, 2, 32, 16, [90, 45, 7], 20, 2),                   # a window of 20 keys
    (8, 2, 80, 64, [500], 0, 64),                         # more splits than there is work
])
def test_attention_decode(heads, kv_heads, head_dim, block_size, lengths, window, splits):
    dtype = torch.bfloat16
    k = lib(dtype, head_dim)
    setup = paged_setup(dtype, lengths, [1] * len(lengths), heads, kv_heads, head_dim, block_size, seed=heads)
    n = len(lengths)
    out = torch.full((n, heads * head_dim), float("nan"), device="cuda").to(dtype)
    scale = 0.37 / math.sqrt(head_dim)
    ctx_after = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    scratch_o = torch.full((n * heads * splits * head_dim,), float("nan"), device="cuda")
    scratch_ml = torch.full((n * heads * splits * 2,), float("nan"), device="cuda")
    k.attention_decode(setup["q"].view(n, -1), setup["k_cache"], setup["v_cache"], setup["table"], ctx_after, out,
                       heads, kv_heads, head_dim, block_size, scale, window, splits, scratch_o, scratch_ml)
    ref = attention_reference(setup, dtype, heads, kv_heads, scale, window).view(n, -1)
    close(out, ref, dtype)
    # the general kernel gives the same answer up to rounding
    other = torch.zeros_like(out)
    k.attention(setup["q"].view(n, -1), setup["k_cache"], setup["v_cache"], setup["table"], setup["positions"],
                setup["token_seq"], other, heads, kv_heads, head_dim, block_size, scale, window)
    close(out, other, dtype)


def test_attention_decode_finds_one_far_key_and_ignores_what_lies_beyond():
    """One key among two thousand dominates; rows of the last block beyond the length hold
    huge values that must not leak in."""
    dtype, heads, kv_heads, head_dim, block_size = torch.bfloat16, 8, 2, 64, 64
    k = lib(dtype, head_dim)
    for far, length in ((0, 2000), (1023, 2000), (1999, 2000), (64, 65)):
        setup = paged_setup(dtype, [length], [1], heads, kv_heads, head_dim, block_size, seed=far)
        q = setup["q"].float()
        key = 8.0 * q[0, 5] / q[0, 5].norm()                    # head 5 uses kv head 1
        block = int(setup["table"][0, far // block_size])
        setup["k_cache"][block, 1, far % block_size] = key.to(dtype)
        setup["keys"][0][far, 1] = key.cpu()
        last = int(setup["table"][0, (length - 1) // block_size])
        setup["k_cache"][last, :, length % block_size:] = 100.0   # stale rows past the end
        setup["v_cache"][last, :, length % block_size:] = 1e4
        for splits in (1, 5):
            out = torch.zeros(1, heads * head_dim, device="cuda").to(dtype)
            so = torch.zeros(heads * splits * head_dim, device="cuda")
            sm = torch.zeros(heads * splits * 2, device="cuda")
            k.attention_decode(setup["q"].view(1, -1), setup["k_cache"], setup["v_cache"], setup["table"],
                               torch.tensor([length], dtype=torch.int32, device="cuda"), out, heads, kv_heads,
                               head_dim, block_size, 4.0, 0, splits, so, sm)
            ref = attention_reference(setup, dtype, heads, kv_heads, 4.0).view(1, -1)
            close(out, ref, dtype)
            want = setup["values"][0][far, 1].to(dtype).float()
            torch.testing.assert_close(out[0, 5 * head_dim:6 * head_dim].float().cpu(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size,lengths,new,window", [
    (4, 2, 16, 16, [5, 40, 17], [5, 40, 17], 0),
    (6, 3, 48, 16, [33, 1, 100, 64], [33, 1, 100, 64], 0),
    (32, 4, 64, 64, [300, 129, 65], [300, 129, 65], 0),       # the TinyLlama head layout
    (8, 1, 64, 64, [70, 200], [6, 65], 0),                    # continuing prompts that are partly cached
    (5, 5, 128, 32, [130], [130], 0),
    (3, 3, 80, 64, [97, 31], [97, 30], 0),
    (4, 2, 32, 16, [150, 45], [150, 20], 20),                 # a window of 20 keys
    (4, 4, 32, 16, [200], [100], 70),                         # a window wider than a key tile
])
def test_attention_prefill(heads, kv_heads, head_dim, block_size, lengths, new, window):
    dtype = torch.bfloat16
    k = lib(dtype, head_dim)
    assert k.has_attention_prefill()
    setup = paged_setup(dtype, lengths, new, heads, kv_heads, head_dim, block_size, seed=heads + head_dim)
    n = setup["q"].shape[0]
    out = torch.full((n, heads * head_dim), float("nan"), device="cuda").to(dtype)
    scale = 0.37 / math.sqrt(head_dim)
    cu_q = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device="cuda")
    ctx_after = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    k.attention_prefill(setup["q"].view(n, -1), setup["k_cache"], setup["v_cache"], setup["table"], cu_q, ctx_after,
                        out, max(new), heads, kv_heads, head_dim, block_size, scale, window)
    ref = attention_reference(setup, dtype, heads, kv_heads, scale, window).view(n, -1)
    close(out, ref, dtype)


def test_attention_prefill_at_the_edges_of_tiles_and_windows():
    """Make single keys dominate at places where masks and tiles meet: the causal edge
    (the query's own key), the key before a tile boundary, the first key inside a window and
    the last one outside it (which must not be seen)."""
    dtype, heads, kv_heads, head_dim, block_size = torch.bfloat16, 2, 1, 32, 16
    k = lib(dtype, head_dim)
    length, window = 160, 48
    for query, far, visible in ((100, 100, True), (100, 63, True), (100, 64, True), (100, 53, True),
                                (100, 52, False), (128, 81, True), (128, 80, False), (159, 0, False)):
        setup = paged_setup(dtype, [length], [length], heads, kv_heads, head_dim, block_size, seed=query + far)
        q = setup["q"].float()
        key = 9.0 * q[query, 1] / q[query, 1].norm()
        block = int(setup["table"][0, far // block_size])
        setup["k_cache"][block, 0, far % block_size] = key.to(dtype)
        setup["keys"][0][far, 0] = key.cpu()
        out = torch.zeros(length, heads * head_dim, device="cuda").to(dtype)
        cu_q = torch.tensor([0, length], dtype=torch.int32, device="cuda")
        ctx_after = torch.tensor([length], dtype=torch.int32, device="cuda")
        k.attention_prefill(setup["q"].view(length, -1), setup["k_cache"], setup["v_cache"], setup["table"], cu_q,
                            ctx_after, out, length, heads, kv_heads, head_dim, block_size, 4.0, window)
        ref = attention_reference(setup, dtype, heads, kv_heads, 4.0, window).view(length, -1)
        close(out, ref, dtype)
        got = out[query, head_dim:].float().cpu()
        want = setup["values"][0][far, 0].to(dtype).float()
        assert torch.allclose(got, want, rtol=2e-2, atol=2e-2) == visible


@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size,lengths,window,splits,rotate", [
    (4, 2, 16, 16, [5, 40, 17, 1], 0, 1, True),
    (6, 3, 48, 16, [33, 1, 100], 0, 3, True),
    (32, 4, 64, 64, [700, 129, 2048, 64, 65], 0, 8, True),
    (8, 8, 128, 32, [300, 31], 0, 2, True),
    (20, 1, 32, 16, [90, 45], 0, 4, True),                 # more than 16 query heads on one KV head
    (4, 2, 32, 16, [90, 45, 7], 20, 2, True),              # a window
    (8, 2, 80, 64, [500, 16, 17], 0, 8, False),            # no rotation; more splits than work for some
    (2, 1, 32, 16, [9000, 300], 0, 4, True),               # a block table longer than the kernel keeps in shared memory
    (32, 4, 64, 64, [2048, 1500], 0, 4, True),             # few blocks: each stages its whole 512-key piece (four stages)
    (8, 2, 128, 64, [700, 40], 0, 2, True),                # head size 128: swizzled rows of 256 bytes, three stages hold the piece
])
def test_attention_decode_fused_equals_the_separate_kernels(heads, kv_heads, head_dim, block_size, lengths, window,
                                                            splits, rotate):
    """Rotation + cache write + split attention + merge in one kernel, against rope_kv_write followed by
    attention_decode; the cache must hold the same new rows afterwards and nothing else may change."""
    from stratakv_b200.parts.position import rope_table
    dtype = torch.bfloat16
    k = lib(dtype, head_dim)
    n = len(lengths)
    setup = paged_setup(dtype, lengths, [1] * n, heads, kv_heads, head_dim, block_size, seed=heads * 7 + head_dim)
    g = torch.Generator().manual_seed(99)
    qkv = torch.randn(n, (heads + 2 * kv_heads) * head_dim, generator=g).cuda()
    table = torch.from_numpy(rope_table(head_dim, 5000.0, max(2048, max(lengths) + 8))).cuda() if rotate else None
    ctx_after = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    scale = 0.5 / math.sqrt(head_dim)
    # the separate kernels
    k1, v1 = setup["k_cache"].clone(), setup["v_cache"].clone()
    q = torch.zeros(n, heads * head_dim, device="cuda").to(dtype)
    k.rope_kv_write(qkv, table, setup["positions"], setup["token_seq"], setup["table"], q, k1, v1, heads, kv_heads,
                    head_dim, block_size, True)
    expected = torch.zeros_like(q)
    so = torch.zeros(n * heads * 8 * head_dim, device="cuda")
    sm = torch.zeros(n * heads * 8 * 2, device="cuda")
    k.attention_decode(q, k1, v1, setup["table"], ctx_after, expected, heads, kv_heads, head_dim, block_size, scale,
                       window, splits, so, sm)
    # the fused kernel
    k2, v2 = setup["k_cache"].clone(), setup["v_cache"].clone()
    got = torch.full_like(q, float("nan"))
    k.attention_decode_fused(qkv, table, k2, v2, setup["table"], ctx_after, got, heads, kv_heads, head_dim, block_size,
                             scale, window, splits, True)
    torch.cuda.synchronize()
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    torch.testing.assert_close(got.float(), expected.float(), rtol=1.6e-2, atol=1e-2)
    # reading only: the cache stays as it was, and the result is the same over the rows already there
    k3, v3 = k1.clone(), v1.clone()
    again = torch.full_like(q, float("nan"))
    k.attention_decode_fused(qkv, table, k3, v3, setup["table"], ctx_after, again, heads, kv_heads, head_dim,
                             block_size, scale, window, splits, False)
    assert torch.equal(k3, k1) and torch.equal(v3, v1)
    torch.testing.assert_close(again.float(), expected.float(), rtol=1.6e-2, atol=1e-2)


@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size,lengths,new,window", [
    (32, 4, 64, 64, [300, 129, 65], [300, 129, 65], 0),       # the TinyLlama head layout
    (8, 1, 64, 64, [70, 200], [6, 65], 0),                    # continuing prompts that are partly cached
    (4, 2, 64, 16, [150, 45, 1, 128], [150, 20, 1, 128], 0),  # small cache blocks, tile-aligned and tiny lengths
    (5, 5, 128, 32, [130, 257], [130, 257], 0),
    (4, 4, 128, 128, [400], [300], 0),                        # blocks as large as a key tile
    (4, 2, 64, 16, [300, 45], [300, 20], 70),                 # a window
    (2, 1, 64, 64, [1000], [1000], 200),                      # a window wider than a key tile
])
def test_attention_prefill_tcgen05(heads, kv_heads, head_dim, block_size, lengths, new, window):
    dtype = torch.bfloat16
    k = lib(dtype, head_dim)
    assert k.has_attention_prefill_tc()
    setup = paged_setup(dtype, lengths, new, heads, kv_heads, head_dim, block_size, seed=3 * heads + head_dim)
    n = setup["q"].shape[0]
    out = torch.full((n, heads * head_dim), float("nan"), device="cuda").to(dtype)
    scale = 0.37 / math.sqrt(head_dim)
    cu_q = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device="cuda")
    ctx_after = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    k.attention_prefill_tc(setup["q"].view(n, -1).contiguous(), setup["k_cache"], setup["v_cache"], setup["table"], cu_q,
                           ctx_after, out, max(new), heads, kv_heads, head_dim, block_size, scale, window)
    torch.cuda.synchronize()
    assert int(k.error_flag.item()) == 0
    ref = attention_reference(setup, dtype, heads, kv_heads, scale, window).view(n, -1)
    close(out, ref, dtype)


def _rotate_plain(x, theta, positions):
    """Split-half rotation of ``x`` [n, heads, d] in float with angles taken in double
    (src/layers/attention.cpp:63-69, 96-135)."""
    half = x.shape[-1] // 2
    inv = torch.tensor([theta ** (-2.0 * i / x.shape[-1]) for i in range(half)], dtype=torch.float64).float().double()
    angle = positions.double()[:, None] * inv[None, :]
    cos, sin = torch.cos(angle).float()[:, None], torch.sin(angle).float()[:, None]
    return torch.cat([x[..., :half] * cos - x[..., half:] * sin, x[..., :half] * sin + x[..., half:] * cos], -1)


def _fused_decode_case(dtype, lengths, heads, kv_heads, head_dim, block_size, seed, theta=5000.0):
    """A paged cache with ``lengths[s] - 1`` keys per sequence and one new token each as a float q|k|v row;
    returns the kernel's inputs and a ``setup`` for ``attention_reference`` in which the rotated new key and
    the new value stand at the last position and the rotated queries are the queries."""
    from stratakv_b200.parts.position import rope_table
    n = len(lengths)
    setup = paged_setup(dtype, lengths, [1] * n, heads, kv_heads, head_dim, block_size, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    qkv = torch.randn(n, (heads + 2 * kv_heads) * head_dim, generator=g)
    positions = torch.tensor([l - 1 for l in lengths])
    q = _rotate_plain(qkv[:, :heads * head_dim].view(n, heads, head_dim), theta, positions)
    new_k = _rotate_plain(qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].view(n, kv_heads, head_dim), theta, positions)
    new_v = qkv[:, (heads + kv_heads) * head_dim:].view(n, kv_heads, head_dim)
    setup["q"] = q.to(dtype).cuda()
    for s, length in enumerate(lengths):
        setup["keys"][s][length - 1] = new_k[s]
        setup["values"][s][length - 1] = new_v[s]
    table = torch.from_numpy(rope_table(head_dim, theta, max(lengths) + 8)).cuda()
    return setup, qkv.cuda(), table, q


@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size,lengths,window,splits", [
    (4, 2, 16, 16, [5, 40, 17, 1], 0, 1),
    (32, 4, 64, 64, [700, 129, 2048, 64, 65], 0, 8),       # the TinyLlama head layout
    (32, 4, 64, 64, [2048] * 8, 0, 4),                     # the benchmark's step: whole 512-key pieces staged
    (32, 32, 128, 64, [300, 1000], 0, 2),                  # one query head per KV head, head size 128
    (32, 8, 128, 64, [2048, 77], 0, 8),
    (20, 1, 32, 16, [90, 45], 0, 4),                       # more than 16 query heads on one KV head
    (4, 2, 32, 16, [90, 45, 7], 20, 2),                    # a window
    (2, 1, 192, 32, [150], 0, 2),                          # the largest head size this kernel is built for
])
def test_attention_decode_fused_against_plain_attention(heads, kv_heads, head_dim, block_size, lengths, window, splits):
    """The fused kernel against attention written out in double (not against the other kernels)."""
    dtype = torch.bfloat16
    k = lib(dtype, head_dim)
    assert k.has_attention_decode_fused()
    setup, qkv, table, _ = _fused_decode_case(dtype, lengths, heads, kv_heads, head_dim, block_size, seed=heads + head_dim)
    n = len(lengths)
    scale = 0.5 / math.sqrt(head_dim)
    out = torch.full((n, heads * head_dim), float("nan"), device="cuda").to(dtype)
    k.attention_decode_fused(qkv, table, setup["k_cache"], setup["v_cache"], setup["table"],
                             torch.tensor(lengths, dtype=torch.int32, device="cuda"), out, heads, kv_heads, head_dim,
                             block_size, scale, window, splits, True)
    ref = attention_reference(setup, dtype, heads, kv_heads, scale, window).view(n, -1)
    close(out, ref, dtype)


@pytest.mark.parametrize("head_dim,splits", [(64, 1), (64, 4), (64, 8), (128, 2)])
def test_attention_decode_fused_finds_one_far_key_and_ignores_what_lies_beyond(head_dim, splits):
    """One key among two thousand dominates, wherever it lies (the first key, a piece's edge, the key just
    written); rows of the last block beyond the length hold huge values that must not leak in."""
    dtype, heads, kv_heads, block_size = torch.bfloat16, 8, 2, 64
    k = lib(dtype, head_dim)
    for far, length in ((0, 2000), (499, 2000), (500, 2000), (1023, 2000), (1998, 2000), (64, 66), (127, 129)):
        setup, qkv, table, q = _fused_decode_case(dtype, [length], heads, kv_heads, head_dim, block_size, seed=far)
        key = 8.0 * q[0, 5] / q[0, 5].norm()                    # head 5 uses kv head 1; q is already rotated
        block = int(setup["table"][0, far // block_size])
        setup["k_cache"][block, 1, far % block_size] = key.to(dtype)
        setup["keys"][0][far, 1] = key
        last = int(setup["table"][0, (length - 1) // block_size])
        setup["k_cache"][last, :, length % block_size:] = 100.0   # stale rows past the end
        setup["v_cache"][last, :, length % block_size:] = 1e4
        out = torch.zeros(1, heads * head_dim, device="cuda").to(dtype)
        k.attention_decode_fused(qkv, table, setup["k_cache"], setup["v_cache"], setup["table"],
                                 torch.tensor([length], dtype=torch.int32, device="cuda"), out, heads, kv_heads,
                                 head_dim, block_size, 4.0, 0, splits, True)
        ref = attention_reference(setup, dtype, heads, kv_heads, 4.0).view(1, -1)
        close(out, ref, dtype)
        want = setup["values"][0][far, 1].to(dtype).float()
        torch.testing.assert_close(out[0, 5 * head_dim:6 * head_dim].float().cpu(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("head_dim", [64, 128])
def test_attention_prefill_tcgen05_at_the_edges_of_tiles_and_windows(head_dim):
    """Single keys made to dominate where masks and tiles meet in the tensor-memory kernel: the causal edge
    (the query's own key), the last key of a 64-key tile and the first of the next, the edges of the
    128-query tiles, the first key inside a window and the last one outside it (which must not be seen),
    with part of the context cached by earlier steps."""
    dtype, heads, kv_heads, block_size = torch.bfloat16, 2, 1, 16
    k = lib(dtype, head_dim)
    length = 330
    cases = [(0, 200, 200, True), (0, 200, 63, True), (0, 200, 64, True), (0, 127, 127, True), (0, 128, 127, True),
             (0, 128, 128, True), (0, 329, 0, True), (0, 255, 191, True), (0, 256, 192, True),
             (100, 200, 101, True), (100, 200, 100, False), (100, 329, 230, True), (100, 329, 229, False),
             (100, 128, 29, True), (100, 128, 28, False), (70, 300, 0, False)]
    for cached in (0, 130, 201):                                 # tokens of the context that earlier steps brought
        for window, query, far, visible in cases:
            if query < cached:
                continue
            setup = paged_setup(dtype, [length], [length - cached], heads, kv_heads, head_dim, block_size,
                                seed=query + far + cached)
            q = setup["q"].float()
            row = query - cached
            key = 9.0 * q[row, 1] / q[row, 1].norm()
            block = int(setup["table"][0, far // block_size])
            setup["k_cache"][block, 0, far % block_size] = key.to(dtype)
            setup["keys"][0][far, 0] = key.cpu()
            n = length - cached
            out = torch.zeros(n, heads * head_dim, device="cuda").to(dtype)
            cu_q = torch.tensor([0, n], dtype=torch.int32, device="cuda")
            ctx_after = torch.tensor([length], dtype=torch.int32, device="cuda")
            k.attention_prefill_tc(setup["q"].view(n, -1).contiguous(), setup["k_cache"], setup["v_cache"],
                                   setup["table"], cu_q, ctx_after, out, n, heads, kv_heads, head_dim, block_size,
                                   4.0, window)
            ref = attention_reference(setup, dtype, heads, kv_heads, 4.0, window).view(n, -1)
            close(out, ref, dtype)
            got = out[row, head_dim:].float().cpu()
            want = setup["values"][0][far, 0].to(dtype).float()
            assert torch.allclose(got, want, rtol=2e-2, atol=2e-2) == visible, (cached, window, query, far)
    torch.cuda.synchronize()
    assert int(k.error_flag.item()) == 0


@pytest.mark.parametrize("heads,kv_heads,head_dim,hidden,block_size,lengths,new,rotate,write_kv", [
    (32, 4, 64, 2048, 64, [300, 129, 65], [300, 129, 65], True, True),     # the TinyLlama layout, whole prompts
    (5, 1, 64, 200, 16, [400, 200], [150, 110], True, True),               # a partly cached prompt, a tile that N cuts
    (8, 2, 128, 520, 32, [257], [257], True, True),                        # head size 128: two slabs a query head
    (6, 6, 128, 264, 64, [140, 90], [140, 90], False, True),               # no rotation
    (4, 2, 64, 328, 16, [200], [200], True, False),                        # a layer that reads another layer's cache
    (32, 4, 64, 2048, 64, [2041], [2041], True, True),                     # the TinyLlama layer on a long prompt: 160 tiles on 148 blocks
    (16, 4, 128, 5120, 32, [1000], [1000], True, True),                    # a long inner size: pairs of blocks, head size 128
    (41, 4, 64, 5200, 16, [600, 400], [500, 400], True, True),             # pairs: a partly cached prompt, a tile that N cuts, K's tail
])
def test_linear_qkv_rope_equals_the_projection_followed_by_rope_kv_write(heads, kv_heads, head_dim, hidden, block_size,
                                                                         lengths, new, rotate, write_kv):
    """The q|k|v projection with rotation and cache write in its epilogue against the same projection stored in float
    followed by rope_kv_write (which has its own test against plain arithmetic): same queries, same cache rows,
    nothing else touched."""
    from stratakv_b200 import ops
    from stratakv_b200.parts.position import rope_table
    dtype = torch.bfloat16
    k = lib(dtype, head_dim)
    assert k.has_linear_qkv_rope()
    setup = paged_setup(dtype, lengths, new, heads, kv_heads, head_dim, block_size, seed=heads + head_dim)
    n = setup["positions"].numel()
    width = (heads + 2 * kv_heads) * head_dim
    a = torch.randn(n, hidden, device="cuda").to(dtype)
    w = (torch.randn(width, hidden, device="cuda") / math.sqrt(hidden)).to(dtype)
    table = torch.from_numpy(rope_table(head_dim, 25000.0, max(lengths) + 8)).cuda() if rotate else None
    # in two steps
    qkv = torch.empty(n, width, device="cuda")
    k.linear(a, w, qkv, ops.MODE_STORE_F32)
    k1, v1 = torch.full_like(setup["k_cache"], 7.0), torch.full_like(setup["v_cache"], 7.0)
    q1 = torch.full((n, heads * head_dim), float("nan"), device="cuda").to(dtype)
    k.rope_kv_write(qkv, table, setup["positions"], setup["token_seq"], setup["table"], q1, k1, v1, heads, kv_heads,
                    head_dim, block_size, write_kv)
    # in one
    k2, v2 = torch.full_like(setup["k_cache"], 7.0), torch.full_like(setup["v_cache"], 7.0)
    q2 = torch.full((n, heads * head_dim), float("nan"), device="cuda").to(dtype)
    k.linear_qkv_rope(a, w, q2, table, setup["positions"], setup["token_seq"], setup["table"], k2, v2, heads, kv_heads,
                      head_dim, block_size, write_kv)
    torch.cuda.synchronize()
    assert int(k.error_flag.item()) == 0
    # the same float accumulators rotated by the same formula; the compilers may contract a*c - b*s differently
    torch.testing.assert_close(q2.float(), q1.float(), rtol=2.0 ** -7, atol=1e-6)
    torch.testing.assert_close(k2.float(), k1.float(), rtol=2.0 ** -7, atol=1e-6)
    assert torch.equal(v2, v1)
    if not write_kv:
        assert (k2 == 7.0).all() and (v2 == 7.0).all()
