"""Causal grouped-query attention over the paged cache.

``q, k, v = h.Wq^T, h.Wk^T, h.Wv^T`` (no bias); rotary encoding on every query
and key head before the key is cached; scores ``(q.k) * scale`` over the
sequence's own earlier positions and the token itself; softmax and the weighted
sum of values in float; ``x += ctx.Wo^T`` (``src/layers/attention.cpp:153-342``,
``src/models/transformer_block.cpp:301-309``).  The three projections are one
matrix ``[q | k | v]`` here, and the residual sum is the epilogue of the output
projection.
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from .base import CacheRequest, Mixer, TensorRequest
from .registry import part_class, register_mixer


def decode_splits(n_seqs: int, blocks_per_seq: int, max_ctx: int, sms: int) -> int:
    """Into how many pieces a decode step cuts each context: enough blocks to fill the
    GPU twice over, at least 128 keys (one group of 16 per warp) a piece.  It depends on
    the step's sizes only, never on which sequences are live."""
    by_length = max(1, max_ctx // 128)
    by_count = -(-2 * sms // max(1, n_seqs * blocks_per_seq))
    return max(1, min(by_length, by_count, 64))


def fused_decode_splits(n_seqs: int, blocks_per_seq: int, max_ctx: int, sms: int, per_sm: int = 2) -> int:
    """The same for the fused kernel, whose pieces are the blocks of one cluster: the largest
    power of two (other cluster sizes measured slower), at most 8, that keeps the grid within
    ``per_sm`` blocks per SM (2 up to head size 64, 1 above: the staged keys of a block take
    shared memory in proportion).  Half as many if that gives every block an SM to itself and
    a piece of at most 512 keys, which such a block fetches whole before its inputs are ready."""
    pairs = max(1, n_seqs * blocks_per_seq)
    by_length = max(1, max_ctx // 128)
    wanted = max(1, min(by_length, per_sm * sms // pairs, 8))
    wanted = 1 << (wanted.bit_length() - 1)
    if wanted > 1 and pairs * wanted > sms >= pairs * wanted // 2 and max_ctx * 2 <= 512 * wanted:
        wanted //= 2
    return wanted


def wants_more_pieces(n_seqs: int, blocks_per_seq: int, max_ctx: int, cluster_splits: int, sms: int) -> bool:
    """A cluster holds at most 8 pieces of a context.  Few long sequences want more: when the fused kernel's
    grid leaves SMs idle, its pieces are 2,048 keys or longer and the path through scratch memory would cut
    at least twice as many (batch 1 at 32,000 keys: 1.14 ms a step with 64 pieces and a combine kernel,
    1.72 ms with 8 pieces in one cluster)."""
    return (n_seqs * blocks_per_seq * cluster_splits < sms and max_ctx >= 2048 * cluster_splits
            and decode_splits(n_seqs, blocks_per_seq, max_ctx, sms) >= 2 * cluster_splits)


class PagedAttention(Mixer):
    graph_safe = True
    folds_norm = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError("attention: heads must be a multiple of kv heads")
        if spec.head_dim % 16 != 0:
            raise ValueError(f"attention: head size {spec.head_dim} is not supported "
                             "(the kernels take multiples of 16)")
        if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
            raise ValueError(f"attention: hidden size {spec.hidden_size} is not supported in bfloat16 "
                             "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
        self.q_dim = spec.num_heads * spec.head_dim
        self.kv_dim = spec.num_kv_heads * spec.head_dim
        position_spec = spec.position
        kind = position_spec.kind if position_spec is not None else "none"
        self.position = part_class("position", kind)(position_spec, runtime)

    @classmethod
    def expected_tensors(cls, spec):
        q_dim, kv_dim = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        return {spec.q_weight: TensorRequest((q_dim, spec.hidden_size)),
                spec.k_weight: TensorRequest((kv_dim, spec.hidden_size)),
                spec.v_weight: TensorRequest((kv_dim, spec.hidden_size)),
                spec.o_weight: TensorRequest((spec.hidden_size, q_dim))}

    @classmethod
    def cache_request(cls, spec):
        kind = "kv_window" if spec.window > 0 else "kv"
        return CacheRequest(kind, spec.num_kv_heads, spec.head_dim, spec.window)

    def bind(self, tensors):
        s = self.spec
        parts = [self.rt.upload(tensors[name]) for name in (s.q_weight, s.k_weight, s.v_weight)]
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        del parts
        self.w_o = self.rt.upload(tensors[s.o_weight])

    def forward(self, step, h, x, cache_entry, writes_cache=True):
        s, rt = self.spec, self.rt
        ops = rt.kernels(s.head_dim)
        n = h.shape[0]
        ctx = rt.workspace.get("attn_ctx", (n, self.q_dim), rt.dtype)
        if (rt.dtype == torch.bfloat16 and n > 128 and s.head_dim in (64, 128) and torch.is_tensor(h)
                and hasattr(self.position, "fusion_table") and ops.has_linear_qkv_rope()):
            # many tokens: the projection's epilogue rotates queries and keys and writes the cache itself
            q = rt.workspace.get("q", (n, self.q_dim), rt.dtype)
            k_cache, v_cache = step.cache.entry_kv(cache_entry)
            table = step.block_tables[step.cache.entry_group_index(cache_entry)]
            ops.linear_qkv_rope(h, self.w_qkv, q, self.position.fusion_table(step.max_ctx), step.positions,
                                step.token_seq, table, k_cache, v_cache, s.num_heads, s.num_kv_heads, s.head_dim,
                                step.cache.block_size, writes_cache)
            self._attend_rotated(step, q, ctx, k_cache, v_cache, table)
        else:
            qkv = rt.workspace.get("qkv", (n, self.q_dim + 2 * self.kv_dim), torch.float32)
            ops.linear(h, self.w_qkv, qkv, _ops.MODE_STORE_F32)
            self.attend(step, qkv, ctx, cache_entry, writes_cache)
        ops.linear(ctx, self.w_o, x, _ops.MODE_ADD_F32, stats=step.residual_stats)

    def attend(self, step, qkv, ctx, cache_entry, writes_cache=True):
        """From the float32 q|k|v rows of the step's tokens to the attention output ``ctx`` (compute dtype):
        position encoding, cache write, attention over each sequence's own keys."""
        s, rt = self.spec, self.rt
        ops = rt.kernels(s.head_dim)
        n = qkv.shape[0]
        k_cache, v_cache = step.cache.entry_kv(cache_entry)
        table = step.block_tables[step.cache.entry_group_index(cache_entry)]
        blocks_per_seq = s.num_kv_heads * (-(-(s.num_heads // s.num_kv_heads) // 16))
        fused = (step.is_decode and rt.dtype == torch.bfloat16 and hasattr(self.position, "fusion_table")
                 and ops.has_attention_decode_fused())
        if fused:
            splits = fused_decode_splits(n, blocks_per_seq, step.max_ctx, rt.sm_count, per_sm=2 if s.head_dim <= 64 else 1)
            fused = not wants_more_pieces(n, blocks_per_seq, step.max_ctx, splits, rt.sm_count)
        if fused:
            # one kernel: rotation, cache write, attention over the context in up to 8 pieces, merge
            ops.attention_decode_fused(qkv, self.position.fusion_table(step.max_ctx), k_cache, v_cache, table,
                                       step.ctx_after, ctx, s.num_heads, s.num_kv_heads, s.head_dim,
                                       step.cache.block_size, s.scale, s.window, splits, writes_cache)
            return
        q = rt.workspace.get("q", (n, self.q_dim), rt.dtype)
        self.position.rotate_and_store(step, qkv, q, k_cache, v_cache, table, s.num_heads, s.num_kv_heads,
                                       s.head_dim, step.cache.block_size, writes_cache)
        self._attend_rotated(step, q, ctx, k_cache, v_cache, table)

    def _attend_rotated(self, step, q, ctx, k_cache, v_cache, table):
        """Attention of the step's rotated queries ``q`` over the cache, which holds the step's keys and values."""
        s, rt = self.spec, self.rt
        ops = rt.kernels(s.head_dim)
        n = q.shape[0]
        blocks_per_seq = s.num_kv_heads * (-(-(s.num_heads // s.num_kv_heads) // 16))
        if step.is_decode and rt.dtype == torch.bfloat16:
            splits = decode_splits(n, blocks_per_seq, step.max_ctx, rt.sm_count)
            scratch_o = scratch_ml = None
            if splits > 1:
                scratch_o = rt.workspace.get("attn_split_o", (n * s.num_heads * splits * s.head_dim,), torch.float32)
                scratch_ml = rt.workspace.get("attn_split_ml", (n * s.num_heads * splits * 2,), torch.float32)
            ops.attention_decode(q, k_cache, v_cache, table, step.ctx_after, ctx, s.num_heads, s.num_kv_heads,
                                 s.head_dim, step.cache.block_size, s.scale, s.window, splits, scratch_o, scratch_ml)
        elif (rt.dtype == torch.bfloat16 and ops.has_attention_prefill_tc() and step.max_q_len > 32
              and step.cache.block_size & (step.cache.block_size - 1) == 0
              and step.n_seqs * -(-step.max_q_len // 128) <= 65535):
            ops.attention_prefill_tc(q, k_cache, v_cache, table, step.cu_q, step.ctx_after, ctx, step.max_q_len,
                                     s.num_heads, s.num_kv_heads, s.head_dim, step.cache.block_size, s.scale, s.window)
        elif rt.dtype == torch.bfloat16 and ops.has_attention_prefill():
            ops.attention_prefill(q, k_cache, v_cache, table, step.cu_q, step.ctx_after, ctx, step.max_q_len,
                                  s.num_heads, s.num_kv_heads, s.head_dim, step.cache.block_size, s.scale, s.window)
        else:
            ops.attention(q, k_cache, v_cache, table, step.positions, step.token_seq, ctx, s.num_heads,
                          s.num_kv_heads, s.head_dim, step.cache.block_size, s.scale, s.window)


register_mixer("attention", PagedAttention)
