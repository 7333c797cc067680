"""Who may fold a norm into a projection, decided on the host: the bookkeeping of
``residual.ResidualStats`` and of the ``pre_norm`` arrangement, with stand-in parts (no GPU)."""
from types import SimpleNamespace

import torch

from stratakv_b200.parts.attention import decode_splits, fused_decode_splits, wants_more_pieces
from stratakv_b200.parts.block import foldable, pre_norm
from stratakv_b200.residual import NormedRows, ResidualStats


def make_stats(rows=4, width=64):
    return ResidualStats(torch.zeros(rows, width), torch.zeros(rows), torch.zeros(rows, 4), torch.zeros(1, dtype=torch.int32))


class Norm:
    def __init__(self, log, name, folds=True):
        self.log, self.name, self.folds_norm = log, name, folds
        self.gamma, self.spec = torch.ones(64), SimpleNamespace(eps=1e-5)

    def forward(self, x, rows=None, out=None, name="normed", stats=None):
        if stats is not None and stats.ready_for(self):
            self.log.append((self.name, "folded"))
            return NormedRows(stats.scaled, stats.row_scale, rows, stats.partials, stats.n_partials, self.spec.eps)
        self.log.append((self.name, "kernel"))
        return x


class Writer:
    """A mixer or feed-forward; one that folds norms fills the statistics as the kernels' wrapper does."""
    def __init__(self, log, name, folds):
        self.log, self.name, self.folds_norm = log, name, folds

    def forward(self, step, h, x, *cache):
        self.log.append((self.name, "normed input" if isinstance(h, NormedRows) else "tensor input"))
        stats = step.residual_stats
        if self.folds_norm and stats is not None:
            stats.filled(4) if stats.next_norm is not None else stats.invalidate()


def run_layer(mixer_folds, ffn_folds, ffn_norm_folds=True):
    log = []
    layer = SimpleNamespace(mixer_norm=Norm(log, "norm1"), mixer=Writer(log, "mixer", mixer_folds),
                            ffn_norm=Norm(log, "norm2", ffn_norm_folds), ffn=Writer(log, "ffn", ffn_folds))
    after = Norm(log, "next")
    stats = make_stats()
    stats.expect(foldable(layer.mixer_norm, layer.mixer))
    stats.filled(1)                                       # as the embedding leaves them
    step = SimpleNamespace(residual_stats=stats, norm_after_layer=after)
    pre_norm(layer, step, torch.zeros(4, 64), SimpleNamespace(cache=0, writes_cache=True))
    return log, stats, after


def test_parts_that_fold_get_normed_rows_and_keep_the_statistics():
    log, stats, after = run_layer(True, True)
    assert log == [("norm1", "folded"), ("mixer", "normed input"), ("norm2", "folded"), ("ffn", "normed input")]
    assert stats.ready_for(after)


def test_a_mixer_that_does_not_fold_gets_a_tensor_and_the_norm_after_it_runs():
    log, stats, after = run_layer(False, True)
    assert log == [("norm1", "kernel"), ("mixer", "tensor input"), ("norm2", "kernel"), ("ffn", "tensor input")]
    assert stats.ready_for(after)                         # the feed-forward wrote the stream last and folds


def test_a_feed_forward_that_does_not_fold_leaves_the_statistics_unknown():
    log, stats, after = run_layer(True, False)
    assert log == [("norm1", "folded"), ("mixer", "normed input"), ("norm2", "kernel"), ("ffn", "tensor input")]
    assert not stats.ready_for(after) and stats.prepared_for is None


def test_a_norm_that_cannot_be_folded_is_not_prepared_for():
    log, stats, after = run_layer(True, True, ffn_norm_folds=False)
    assert ("norm2", "kernel") in log and ("ffn", "tensor input") in log


def test_statistics_are_for_one_norm_only():
    stats = make_stats()
    a, b = Norm([], "a"), Norm([], "b")
    assert not stats.ready_for(a)
    stats.expect(a)
    stats.filled(3)
    assert stats.ready_for(a) and not stats.ready_for(b) and not stats.ready_for(None) and stats.n_partials == 3
    stats.invalidate()
    assert not stats.ready_for(a)
    stats.expect(None)
    stats.filled()
    assert not stats.ready_for(a) and not stats.ready_for(None)


def test_few_rows_let_the_consumer_add_the_partial_sums():
    assert make_stats(rows=16).consumer_sums and not make_stats(rows=17).consumer_sums
    wide = ResidualStats(torch.zeros(4, 64), torch.zeros(4), torch.zeros(4, 2048), torch.zeros(1, dtype=torch.int32))
    assert not wide.consumer_sums
    assert ResidualStats(torch.zeros(8, 64), torch.zeros(8), torch.zeros(8, 512), torch.zeros(1, dtype=torch.int32)).consumer_sums
    assert not ResidualStats(torch.zeros(16, 64), torch.zeros(16), torch.zeros(16, 512), torch.zeros(1, dtype=torch.int32)).consumer_sums


SMS = 148        # the SM count is an argument of the policies; the engine passes the device's own


def test_context_splits_depend_on_sizes_only():
    for batch in (1, 2, 3, 5, 8, 12, 16, 24, 32, 48, 64, 200):
        for groups in (1, 4, 8, 32):
            for ctx in (16, 100, 128, 1000, 2048, 4096, 100000):
                fused = fused_decode_splits(batch, groups, ctx, SMS)
                assert fused in (1, 2, 4, 8)
                assert fused * 128 <= max(ctx, 128)                       # at least 128 keys a piece
                plain = decode_splits(batch, groups, ctx, SMS)
                assert 1 <= plain <= 64 and plain * 128 <= max(ctx, 128)
    assert fused_decode_splits(8, 4, 2048, SMS) == 4 and fused_decode_splits(8, 4, 4096, SMS) == 8
    assert fused_decode_splits(64, 4, 2048, SMS) == 1 and fused_decode_splits(1, 4, 2048, SMS) == 8
    assert fused_decode_splits(8, 4, 2048, 32) == 2               # a smaller GPU cuts contexts into fewer pieces


def test_only_few_long_sequences_leave_the_cluster_kernel():
    def leaves(batch, groups, ctx, per_sm=2):
        return wants_more_pieces(batch, groups, ctx, fused_decode_splits(batch, groups, ctx, SMS, per_sm=per_sm), SMS)
    assert leaves(1, 4, 32768) and leaves(2, 4, 32768)
    assert not leaves(1, 4, 8192) and not leaves(8, 4, 2048) and not leaves(8, 4, 16384)
    assert not leaves(8, 32, 2048, per_sm=1)              # many heads fill the GPU with one piece each
    assert not leaves(64, 4, 32768)
