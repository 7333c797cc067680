"""The allocation-free decode attention entry point, called through its exported C symbol.

Some hosts of these kernels are not allowed to allocate device memory while they run (a
plug-in inside another program's memory budget, a loop that must stay out of the allocator,
a process that gave all device memory to one pool at start).  For them the library exports
skv_attention_decode_no_alloc, which keeps the partial results of its context splits in an
array built into the library.  This test calls that symbol with ctypes, twice in a row on
different inputs (the second call finds the first call's leftovers in the array), and
compares each result with the regular entry point's, which gets its scratch from the caller.

The file is named so that pytest collects it last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, n_seqs, heads, kv_heads, head_dim, block_size, lengths):
    g = torch.Generator().manual_seed(seed)
    width = max(-(-l // block_size) for l in lengths)
    blocks = n_seqs * width + 1
    order = torch.randperm(blocks, generator=g)
    table = order[:n_seqs * width].view(n_seqs, width).to(torch.int32).cuda()
    k_cache = torch.randn(blocks, kv_heads, block_size, head_dim, generator=g).to(torch.bfloat16).cuda()
    v_cache = torch.randn(blocks, kv_heads, block_size, head_dim, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(n_seqs, heads * head_dim, generator=g).to(torch.bfloat16).cuda()
    ctx_after = torch.tensor(lengths, dtype=torch.int32).cuda()
    return q, k_cache, v_cache, table, ctx_after


def test_no_alloc_entry_point_matches_the_regular_one_twice():
    from stratakv_b200.ops import kernels_for
    heads, kv_heads, head_dim, block_size, splits = 8, 2, 64, 64, 4
    kernels = kernels_for(torch.bfloat16, head_dim, verbose=False)
    lib = ctypes.CDLL(str(kernels.path))                      # the symbol itself, not the Python wrapper
    entry = lib.skv_attention_decode_no_alloc
    entry.restype = ctypes.c_int
    lib.skv_last_error.restype = ctypes.c_char_p
    lib.skv_attention_decode_no_alloc_capacity.restype = ctypes.c_longlong
    capacity = lib.skv_attention_decode_no_alloc_capacity()
    assert capacity >= 3 * heads * splits * (head_dim + 2)
    scale = 1.0 / math.sqrt(head_dim)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    for call, lengths in enumerate(([700, 65, 1], [300, 1024, 129])):
        q, k_cache, v_cache, table, ctx_after = _inputs(40 + call, 3, heads, kv_heads, head_dim, block_size, lengths)
        expected = torch.zeros_like(q)
        scratch_o = torch.zeros(3 * heads * splits * head_dim, device="cuda")
        scratch_ml = torch.zeros(3 * heads * splits * 2, device="cuda")
        kernels.attention_decode(q, k_cache, v_cache, table, ctx_after, expected, heads, kv_heads, head_dim,
                                 block_size, scale, 0, splits, scratch_o, scratch_ml)
        got = torch.full_like(q, float("nan"))
        code = entry(ptr(q), ptr(k_cache), ptr(v_cache), ptr(table), table.shape[1], ptr(ctx_after), ptr(got),
                     3, heads, kv_heads, head_dim, block_size, ctypes.c_float(scale), 0, splits, stream)
        assert code == 0, lib.skv_last_error().decode()
        torch.cuda.synchronize()
        # the same two kernels with the same splits, only the scratch lies elsewhere: the same bits
        assert torch.equal(got, expected)
    # a request beyond the built-in array is refused, with both numbers in the message, and launches nothing
    too_many = int(capacity // (heads * (head_dim + 2))) + 1
    code = entry(ptr(q), ptr(k_cache), ptr(v_cache), ptr(table), table.shape[1], ptr(ctx_after), ptr(got),
                 3, heads, kv_heads, head_dim, block_size, ctypes.c_float(scale), 0, too_many, stream)
    message = lib.skv_last_error().decode()
    assert code != 0 and str(capacity) in message and "floats of scratch" in message
