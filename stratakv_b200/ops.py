"""The kernel library as Python calls: loads the compiled .so and checks arguments.

There is one backend: hand-written CUDA for sm_100a, loaded through ctypes.
If it cannot be compiled or loaded, or no CUDA device is present, the calls
raise; nothing falls back to the CPU or to library model code.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from .csrc.build import BuildError, build_library
from .residual import COLUMNS_PER_PARTIAL, KERNEL_FOLD_ROWS, NormedRows

MODE_STORE, MODE_STORE_F32, MODE_ADD_F32, MODE_GATED = 0, 1, 2, 3
MODE_QKV_ROPE = 4          # (linear_qkv_rope's own epilogue; named for Kernels.linear_form)
# activations of a gated feed-forward's gate that every projection kernel implements (csrc/common.cuh)
ACTIVATIONS = {"silu": 0, "swish": 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1}
_DTYPE_NAMES = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


class KernelError(RuntimeError):
    pass


def _ptr(tensor: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


_NULL = ctypes.c_void_p(0)
_NO_FOLD = (_NULL, _NULL, _NULL, 0, _NULL, ctypes.c_float(0.0), _NULL)
_SCOPED_STREAM = None


def _stream():
    if _SCOPED_STREAM is not None:
        return _SCOPED_STREAM
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Within the scope every kernel goes to the stream that was current when the scope began
    (asking torch for the current stream at each of a step's two hundred launches costs more
    than the launches themselves)."""

    def __enter__(self):
        global _SCOPED_STREAM
        self.previous = _SCOPED_STREAM
        _SCOPED_STREAM = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream) if torch.cuda.is_available() else None
        return self

    def __exit__(self, *exc):
        global _SCOPED_STREAM
        _SCOPED_STREAM = self.previous
        return False


class Kernels:
    """The kernels of one (compute dtype, head size) library."""

    launches = 0          # kernel launches issued through any library of this process

    def __init__(self, dtype: torch.dtype, head_dim: int, verbose: bool = True):
        if dtype not in _DTYPE_NAMES:
            raise KernelError(f"no kernels for dtype {dtype}")
        self.dtype = dtype
        self.head_dim = head_dim
        try:
            self.path = build_library(_DTYPE_NAMES[dtype], head_dim, verbose=verbose)
        except BuildError as error:
            raise KernelError(str(error)) from None
        try:
            self.lib = ctypes.CDLL(str(self.path))
        except OSError as error:
            raise KernelError(f"cannot load {self.path}: {error}") from None
        self.lib.skv_last_error.restype = ctypes.c_char_p
        if self.lib.skv_library_head_dim() != head_dim:
            raise KernelError(f"{self.path} was built for another head size")
        # A device word kernels raise bits in (4: a pipeline wait inside a kernel timed out).
        self.error_flag = torch.zeros(1, dtype=torch.int32, device="cuda") if torch.cuda.is_available() else None

    # ---- helpers -----------------------------------------------------------
    def _check(self, code: int, name: str) -> None:
        Kernels.launches += 1
        if code != 0:
            raise KernelError(f"{name}: {self.lib.skv_last_error().decode()}")

    def _want(self, tensor: torch.Tensor, dtype, name: str) -> None:
        if not tensor.is_cuda:
            raise KernelError(f"{name} must be a CUDA tensor: the kernels run on the GPU only")
        if tensor.dtype != dtype:
            raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
        if not tensor.is_contiguous():
            raise KernelError(f"{name} must be contiguous")

    # ---- kernels -------------------------------------------------------------
    _KINDS = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}

    def convert(self, src, out):
        """out = src in out's type (float32, bfloat16, float16), rounded to nearest even where bits are lost: how
        checkpoint tensors get from their stored type to the compute type once they are on the device."""
        if src.dtype not in self._KINDS or out.dtype not in self._KINDS:
            raise KernelError(f"convert: float32, bfloat16 and float16 only, not {src.dtype} -> {out.dtype}")
        if src.shape != out.shape or src.device != out.device or not src.is_cuda:
            raise KernelError("convert: source and result must have one shape and lie on the same GPU")
        if not (src.is_contiguous() and out.is_contiguous()):
            raise KernelError("convert: tensors must be contiguous")
        self.lib.skv_convert.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
                                         ctypes.c_void_p]
        self._check(self.lib.skv_convert(_ptr(src), self._KINDS[src.dtype], _ptr(out), self._KINDS[out.dtype],
                                         src.numel(), _stream()), "convert")
        return out

    def embed(self, table, ids, out, flag=None, stats=None):
        """out[t, :] = table[ids[t], :] as float32; with ``stats`` each row's sum of squares too."""
        self._want(table, self.dtype, "table"); self._want(ids, torch.int32, "ids")
        self._want(out, torch.float32, "out")
        n, hidden = out.shape
        vocab = table.shape[0]
        if table.shape[1] != hidden or ids.numel() != n:
            raise KernelError("embed: shapes do not agree")
        fold = self._fold_target(stats, n, hidden)
        self._check(self.lib.skv_embed(_ptr(table), _ptr(ids), _ptr(out), n, hidden, vocab, _ptr(flag),
                                       *(fold[:6] if fold else _NO_FOLD[:6]), _stream()), "embed")
        if stats is not None:
            stats.filled(1 if stats.consumer_sums else 0) if fold else stats.invalidate()

    def _fold_target(self, stats, rows: int, width: int):
        """Arguments (scaled rows, next norm's weight, partial sums, their stride, rows' factors, next norm's
        eps, counter) for a kernel that writes ``rows`` rows of the stream; None where it cannot fold."""
        if stats is None or stats.next_norm is None or self.dtype != torch.bfloat16 or rows > KERNEL_FOLD_ROWS:
            return None
        gamma = stats.next_norm.gamma
        self._want(gamma, torch.float32, "gamma"); self._want(stats.partials, torch.float32, "partials")
        self._want(stats.scaled, self.dtype, "scaled"); self._want(stats.row_scale, torch.float32, "row_scale")
        self._want(stats.counter, torch.int32, "counter")
        if (gamma.numel() != width or tuple(stats.scaled.shape) != (rows, width) or stats.row_scale.numel() != rows
                or stats.partials.shape[0] != rows
                or stats.partials.shape[1] * COLUMNS_PER_PARTIAL < width):
            raise KernelError("the buffers of the folded norm do not match the stream")
        return (_ptr(stats.scaled), _ptr(gamma), _ptr(stats.partials), stats.partials.shape[1], _ptr(stats.row_scale),
                ctypes.c_float(stats.next_norm.spec.eps), _NULL if stats.consumer_sums else _ptr(stats.counter))

    def rmsnorm(self, x, gamma, eps: float, out, rows=None):
        """out[r, :] = rmsnorm(x[rows[r] or r, :]) * gamma, in the compute dtype."""
        self._want(x, torch.float32, "x"); self._want(gamma, torch.float32, "gamma")
        self._want(out, self.dtype, "out")
        hidden = x.shape[-1]
        n_rows = out.shape[0]
        if gamma.numel() != hidden or out.shape[-1] != hidden:
            raise KernelError("rmsnorm: shapes do not agree")
        if rows is not None:
            self._want(rows, torch.int32, "rows")
            if rows.numel() != n_rows:
                raise KernelError("rmsnorm: one output row per index is needed")
        elif x.shape[0] != n_rows:
            raise KernelError("rmsnorm: shapes do not agree")
        self._check(self.lib.skv_rmsnorm(_ptr(x), _ptr(gamma), ctypes.c_float(eps), _ptr(out), _ptr(rows),
                                         n_rows, hidden, _stream()), "rmsnorm")

    def linear(self, a, w, out, mode: int = MODE_STORE, activation: str = "silu", flag=None, stats=None):
        """out = a[M,K] . w[N,K]^T with the epilogue ``mode``.

        ``a`` may be ``residual.NormedRows``: the norm is applied while the activations are
        loaded.  ``stats`` (residual-add mode): the statistics of ``out`` are brought up to date where
        the kernel can do that, and marked unknown where it cannot."""
        normed = a if isinstance(a, NormedRows) else None
        if normed is None:
            self._want(a, self.dtype, "a")
        else:
            self._want(normed.scaled, self.dtype, "scaled"); self._want(normed.row_scale, torch.float32, "row_scale")
            if normed.rows is not None:
                self._want(normed.rows, torch.int32, "rows")
            if normed.row_scale.numel() != normed.scaled.shape[0]:
                raise KernelError("linear: one factor per row of the normalised input is needed")
        self._want(w, self.dtype, "w")
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"linear: inner sizes differ ({K} and {w.shape[1]})")
        out_cols = N // 2 if mode == MODE_GATED else N
        out_dtype = self.dtype if mode in (MODE_STORE, MODE_GATED) else torch.float32
        self._want(out, out_dtype, "out")
        if tuple(out.shape) != (M, out_cols):
            raise KernelError(f"linear: out must be [{M}, {out_cols}], got {list(out.shape)}")
        if activation not in ACTIVATIONS:
            raise KernelError(f"linear: unknown activation '{activation}'")
        if stats is not None and mode != MODE_ADD_F32:
            raise KernelError("linear: statistics are kept by the residual-add mode only")
        if normed is not None:
            if stats is not None:
                raise KernelError("linear: a folded norm on the input and statistics of the output do not go together")
            if normed.n_partials > 0:
                self._want(normed.partials, torch.float32, "partials")
                if normed.partials.shape[0] != normed.scaled.shape[0] or normed.partials.shape[1] < normed.n_partials:
                    raise KernelError("linear: the partial sums do not match the normalised input")
                factor = (_NULL, _ptr(normed.partials), normed.n_partials, normed.partials.shape[1],
                          ctypes.c_float(normed.eps))
            else:
                factor = (_ptr(normed.row_scale), _NULL, 0, 0, ctypes.c_float(0.0))
            self._check(self.lib.skv_linear_normed(
                _ptr(normed.scaled), *factor, _ptr(normed.rows), _ptr(w), _ptr(out), M, N, K, mode,
                ACTIVATIONS[activation], _stream()), "linear")
            return
        fold = self._fold_target(stats, M, N)
        self._check(self.lib.skv_linear(_ptr(a), _ptr(w), _ptr(out), M, N, K, mode, ACTIVATIONS[activation],
                                        _ptr(flag if flag is not None else self.error_flag), *(fold or _NO_FOLD), _stream()),
                    "linear")
        if stats is not None:
            if fold:
                stats.filled((N + COLUMNS_PER_PARTIAL - 1) // COLUMNS_PER_PARTIAL if stats.consumer_sums else 0)
            else:
                stats.invalidate()

    def has_linear_qkv_rope(self) -> bool:
        return bool(self.lib.skv_has_linear_qkv_rope())

    def linear_form(self, M: int, N: int, K: int, mode: int) -> str:
        """Which tensor-memory kernel serves a projection of this shape and epilogue on this GPU (``mode`` 4 is the
        q|k|v projection with the rotary epilogue); for tests that must reach each of them."""
        code = int(self.lib.skv_linear_tcgen05_form(int(M), int(N), int(K), int(mode)))
        return {0: "few_tokens", 1: "tile_128", 2: "tile_160", 3: "tile_256", 4: "pair_256"}.get(code, "none")

    def linear_qkv_rope(self, a, w, q_out, cos_sin, positions, token_seq, block_table, k_cache, v_cache,
                        num_heads: int, num_kv_heads: int, head_dim: int, block_size: int, write_kv: bool, flag=None):
        """The q|k|v projection of a step of more than 128 tokens with ``rope_kv_write`` in its epilogue (bfloat16,
        head size 64 or 128): ``q_out`` [M, heads * head_dim] gets the rotated queries, the cache the rotated keys and
        the values of every token, at the row of its position in the block its sequence's table names."""
        self._want(a, self.dtype, "a"); self._want(w, self.dtype, "w"); self._want(q_out, self.dtype, "q_out")
        self._want(positions, torch.int32, "positions"); self._want(token_seq, torch.int32, "token_seq")
        self._want(block_table, torch.int32, "block_table")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        if cos_sin is not None:
            self._want(cos_sin, torch.float32, "cos_sin")
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or N != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError("linear_qkv_rope: the weight must be [(heads + 2 kv heads) * head_dim, K]")
        if tuple(q_out.shape) != (M, num_heads * head_dim) or positions.numel() != M or token_seq.numel() != M:
            raise KernelError("linear_qkv_rope: one query row, one position and one sequence index per token is needed")
        if tuple(k_cache.shape[1:]) != (num_kv_heads, block_size, head_dim) or k_cache.shape != v_cache.shape:
            raise KernelError("linear_qkv_rope: the cache must be [blocks, kv_heads, block_size, head_dim]")
        self._check(self.lib.skv_linear_qkv_rope(
            _ptr(a), _ptr(w), _ptr(q_out), M, N, K, _ptr(cos_sin), _ptr(positions), _ptr(token_seq), _ptr(block_table),
            block_table.shape[1], _ptr(k_cache), _ptr(v_cache), num_heads, num_kv_heads, head_dim, block_size,
            int(bool(write_kv)), _ptr(flag if flag is not None else self.error_flag), _stream()), "linear_qkv_rope")

    def rope_kv_write(self, qkv, cos_sin, positions, token_seq, block_table, q_out, k_cache, v_cache,
                      num_heads: int, num_kv_heads: int, head_dim: int, block_size: int, write_kv: bool):
        self._want(qkv, torch.float32, "qkv"); self._want(q_out, self.dtype, "q_out")
        self._want(positions, torch.int32, "positions"); self._want(token_seq, torch.int32, "token_seq")
        self._want(block_table, torch.int32, "block_table")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        if cos_sin is not None:
            self._want(cos_sin, torch.float32, "cos_sin")
        n = qkv.shape[0]
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError("rope_kv_write: qkv width does not match the head counts")
        self._check(self.lib.skv_rope_kv_write(
            _ptr(qkv), _ptr(cos_sin), _ptr(positions), _ptr(token_seq), _ptr(block_table),
            block_table.shape[1], _ptr(q_out), _ptr(k_cache), _ptr(v_cache), n, num_heads, num_kv_heads,
            head_dim, block_size, int(bool(write_kv)), _stream()), "rope_kv_write")

    def attention(self, q, k_cache, v_cache, block_table, positions, token_seq, out, num_heads: int,
                  num_kv_heads: int, head_dim: int, block_size: int, scale: float, window: int = 0):
        self._want(q, self.dtype, "q"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table")
        self._want(positions, torch.int32, "positions"); self._want(token_seq, torch.int32, "token_seq")
        n = q.shape[0]
        self._check(self.lib.skv_attention(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(positions),
            _ptr(token_seq), _ptr(out), n, num_heads, num_kv_heads, head_dim, block_size,
            ctypes.c_float(scale), window, _stream()), "attention")

    def has_attention_prefill(self) -> bool:
        return bool(self.lib.skv_has_attention_prefill())

    def attention_prefill(self, q, k_cache, v_cache, block_table, cu_q, ctx_after, out, max_q_len: int,
                          num_heads: int, num_kv_heads: int, head_dim: int, block_size: int, scale: float,
                          window: int = 0):
        """Many new tokens per sequence (bfloat16 build, head size up to 128): sequence ``s`` owns rows
        ``cu_q[s]..cu_q[s+1]-1`` of ``q``/``out``; ``ctx_after[s]`` keys are cached, this step's included."""
        self._want(q, self.dtype, "q"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table"); self._want(cu_q, torch.int32, "cu_q")
        self._want(ctx_after, torch.int32, "ctx_after")
        n_seqs = ctx_after.numel()
        if cu_q.numel() != n_seqs + 1 or block_table.shape[0] != n_seqs:
            raise KernelError("attention_prefill: one length, one offset pair and one table row per sequence is needed")
        self._check(self.lib.skv_attention_prefill(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(cu_q),
            _ptr(ctx_after), _ptr(out), n_seqs, max_q_len, num_heads, num_kv_heads, head_dim, block_size,
            ctypes.c_float(scale), window, _stream()), "attention_prefill")

    def has_attention_prefill_tc(self) -> bool:
        return bool(self.lib.skv_has_attention_prefill_tc())

    def attention_prefill_tc(self, q, k_cache, v_cache, block_table, cu_q, ctx_after, out, max_q_len: int,
                             num_heads: int, num_kv_heads: int, head_dim: int, block_size: int, scale: float,
                             window: int = 0, flag=None):
        """``attention_prefill`` with both products on the tcgen05 tensor cores (bfloat16, head size 64 or 128)."""
        self._want(q, self.dtype, "q"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table"); self._want(cu_q, torch.int32, "cu_q")
        self._want(ctx_after, torch.int32, "ctx_after")
        n_seqs = ctx_after.numel()
        if cu_q.numel() != n_seqs + 1 or block_table.shape[0] != n_seqs:
            raise KernelError("attention_prefill_tc: one length, one offset pair and one table row per sequence is needed")
        if tuple(k_cache.shape[1:]) != (num_kv_heads, block_size, head_dim) or k_cache.shape != v_cache.shape:
            raise KernelError("attention_prefill_tc: the cache must be [blocks, kv_heads, block_size, head_dim]")
        self._check(self.lib.skv_attention_prefill_tc(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(block_table), block_table.shape[1],
            _ptr(cu_q), _ptr(ctx_after), _ptr(out), n_seqs, q.shape[0], max_q_len, num_heads, num_kv_heads, head_dim,
            block_size, ctypes.c_float(scale), window, _ptr(flag if flag is not None else self.error_flag),
            _stream()), "attention_prefill_tc")

    def attention_decode(self, q, k_cache, v_cache, block_table, ctx_after, out, num_heads: int,
                         num_kv_heads: int, head_dim: int, block_size: int, scale: float, window: int = 0,
                         splits: int = 1, scratch_o=None, scratch_ml=None):
        """One new token per sequence (bfloat16 build): ``ctx_after[s]`` keys are cached for sequence
        ``s``, the newest being the query's own.  ``splits`` > 1 cuts each context across blocks and
        needs float scratch: ``scratch_o`` [seqs*heads*splits*head_dim], ``scratch_ml`` [seqs*heads*splits*2]."""
        self._want(q, self.dtype, "q"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table"); self._want(ctx_after, torch.int32, "ctx_after")
        n = q.shape[0]
        if ctx_after.numel() != n or block_table.shape[0] != n:
            raise KernelError("attention_decode: one length and one table row per sequence is needed")
        if splits > 1:
            self._want(scratch_o, torch.float32, "scratch_o"); self._want(scratch_ml, torch.float32, "scratch_ml")
            if scratch_o.numel() < n * num_heads * splits * head_dim or scratch_ml.numel() < n * num_heads * splits * 2:
                raise KernelError("attention_decode: scratch is too small for this many splits")
        self._check(self.lib.skv_attention_decode(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(ctx_after),
            _ptr(out), _ptr(scratch_o), _ptr(scratch_ml), n, num_heads, num_kv_heads, head_dim, block_size,
            ctypes.c_float(scale), window, splits, _stream()), "attention_decode")

    def has_attention_decode_fused(self) -> bool:
        return bool(self.lib.skv_has_attention_decode_fused())

    def attention_decode_fused(self, qkv, cos_sin, k_cache, v_cache, block_table, ctx_after, out, num_heads: int,
                               num_kv_heads: int, head_dim: int, block_size: int, scale: float, window: int = 0,
                               splits: int = 1, write_kv: bool = True):
        """One new token per sequence (bfloat16 build), from the float32 q|k|v projection: rotates queries
        and the new key (``cos_sin`` table, or ``None`` for no rotation), writes the new key and value into
        the cache, attends over ``ctx_after[s]`` keys and merges ``splits`` (1..8) context pieces in-kernel."""
        self._want(qkv, torch.float32, "qkv"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table"); self._want(ctx_after, torch.int32, "ctx_after")
        if cos_sin is not None:
            self._want(cos_sin, torch.float32, "cos_sin")
        n = qkv.shape[0]
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError("attention_decode_fused: qkv width does not match the head counts")
        if ctx_after.numel() != n or block_table.shape[0] != n:
            raise KernelError("attention_decode_fused: one length and one table row per sequence is needed")
        self._check(self.lib.skv_attention_decode_fused(
            _ptr(qkv), _ptr(cos_sin), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
            _ptr(ctx_after), _ptr(out), n, num_heads, num_kv_heads, head_dim, block_size, ctypes.c_float(scale),
            window, splits, int(bool(write_kv)), _stream()), "attention_decode_fused")

    def add_inplace(self, out, other):
        self._want(out, torch.float32, "out"); self._want(other, torch.float32, "other")
        if out.numel() != other.numel():
            raise KernelError("add_inplace: sizes differ")
        self._check(self.lib.skv_add_inplace(_ptr(out), _ptr(other), ctypes.c_longlong(out.numel()), _stream()),
                    "add_inplace")

    def argmax(self, logits, out, flag=None):
        self._want(logits, torch.float32, "logits"); self._want(out, torch.int32, "out")
        rows, vocab = logits.shape
        self._check(self.lib.skv_argmax(_ptr(logits), _ptr(out), rows, vocab, _ptr(flag), _stream()), "argmax")

    def sample(self, logits, out, temperature: float, top_k: int, top_p: float, seed: int, streams, counters,
               flag=None):
        """Temperature / top-k / top-p draw per row; row r uses random number (seed, streams[r], counters[r])."""
        self._want(logits, torch.float32, "logits"); self._want(out, torch.int32, "out")
        self._want(streams, torch.int32, "streams"); self._want(counters, torch.int32, "counters")
        rows, vocab = logits.shape
        if streams.numel() != rows or counters.numel() != rows or out.numel() != rows:
            raise KernelError("sample: one stream, counter and output per row is needed")
        self._check(self.lib.skv_sample(_ptr(logits), _ptr(out), rows, vocab, ctypes.c_float(temperature),
                                        int(top_k), ctypes.c_float(top_p), ctypes.c_ulonglong(seed),
                                        _ptr(streams), _ptr(counters), _ptr(flag), _stream()), "sample")


_LOADED: Dict[Tuple[torch.dtype, int], Kernels] = {}


def kernels_for(dtype: torch.dtype, head_dim: int, verbose: bool = True) -> Kernels:
    key = (dtype, head_dim)
    if key not in _LOADED:
        _LOADED[key] = Kernels(dtype, head_dim, verbose=verbose)
    return _LOADED[key]


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise KernelError(f"device {device}: this library runs on CUDA devices only")
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available: this library has no CPU path")
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise KernelError(f"device {device} has compute capability {major}.{minor}; "
                          "the kernels are built for sm_100a only")
    return device
