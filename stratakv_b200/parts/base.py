"""Interfaces every part implements, and what a part is handed when it runs.

A part is built from its spec and a ``Runtime`` (compute dtype, device, the
kernel library), says which checkpoint tensors it needs, receives them once in
``bind`` and then runs inside steps.  The residual stream ``x`` is a float32
``[tokens, hidden]`` tensor that mixers and feed-forwards add their result to
(the reference keeps the same stream in FP32, ``src/models/transformer_block.cpp:
301-331``); norms read it and emit the compute dtype.

Mixer:        ``forward(step, h, x, cache_entry, writes_cache)``  ->  ``x += mix(h)``
Feed-forward: ``forward(step, h, x)``                            ->  ``x += ffn(h)``
Norm:         ``forward(x, rows=None)``                          ->  ``h`` (compute dtype)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch


@dataclass(frozen=True)
class TensorRequest:
    """A checkpoint tensor a part needs.  ``init`` tells the random-weights mode
    how to fill it: ``normal`` is N(0, std), ``around_one`` is 1 + N(0, std)."""
    shape: Tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class CacheRequest:
    """What one run of a mixer needs from the cache.

    ``kind`` names a registered cache kind (``cache/kinds.py``): ``"kv"`` keeps
    every key and value; ``"kv_window"`` needs only the last ``window``;
    ``"none"`` keeps nothing per position.  ``v_head_dim`` is the width of a
    value where it differs from a key's (0: the same); ``extra`` carries sizes
    that a kind registered elsewhere wants.  ``state_bytes`` is fixed-size
    per-sequence state (zeroed when a sequence takes its slot).  Runs whose
    requests are equal share one group of storage."""
    kind: str = "none"
    num_kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_bytes: int = 0
    v_head_dim: int = 0
    extra: Tuple[int, ...] = ()

    def group_key(self):
        return (self.kind, self.num_kv_heads, self.head_dim, self.window, self.v_head_dim, self.extra)


class Runtime:
    """What parts share: compute dtype, device, scratch buffers and the kernel library."""

    def __init__(self, dtype: torch.dtype, device, workspace, kernel_loader, default_head_dim: int):
        self.dtype = dtype
        self.device = torch.device(device)
        self.workspace = workspace
        self._kernel_loader = kernel_loader          # (dtype, head_dim) -> kernels object
        self.default_head_dim = default_head_dim
        self._sm_count = None
        self._shared = {}                            # checkpoint tensor name -> its one copy on the device

    @property
    def sm_count(self) -> int:
        """SMs of the device the model runs on (parts size their grids by it); 1 off the GPU."""
        if self._sm_count is None:
            self._sm_count = (torch.cuda.get_device_properties(self.device).multi_processor_count
                              if self.device.type == "cuda" else 1)
        return self._sm_count

    def kernels(self, head_dim: Optional[int] = None):
        """The kernel library; attention parts name their head size, others take any build."""
        return self._kernel_loader(self.dtype, head_dim or self.default_head_dim)

    def upload(self, tensor: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """Copy a checkpoint tensor to the device in ``dtype`` (default: the
        compute dtype).  float32 -> bfloat16 rounds to nearest even; the
        reference truncates (``src/cuda/gemm_cuda.cu:74-83``)."""
        target = dtype or self.dtype
        floats = (torch.float32, torch.bfloat16, torch.float16)
        if self.device.type == "cuda" and tensor.dtype != target and tensor.dtype in floats and target in floats:
            # the stored bytes go up as they are and this library's own kernel converts them there
            stored = tensor.contiguous().to(device=self.device)
            return self.kernels().convert(stored, torch.empty(stored.shape, dtype=target, device=self.device))
        return tensor.to(device=self.device, dtype=target).contiguous()

    def upload_shared(self, name: str, tensor: torch.Tensor) -> torch.Tensor:
        """``upload`` for a checkpoint tensor that several parts may name (tied embedding and head):
        the first caller uploads it, the others get the same device tensor."""
        if name not in self._shared:
            self._shared[name] = self.upload(tensor)
        return self._shared[name]


@dataclass
class StepBatch:
    """One step's tokens: several sequences, each with ``q_len`` new tokens
    after ``ctx_before`` cached ones, packed back to back without padding.

    Host lists describe the batch; the device tensors are what kernels read.
    ``block_tables[g]`` is ``[n_seqs, width]`` int32 for cache group ``g``.
    """
    n_seqs: int
    n_tokens: int
    slots: List[int]
    q_lens: List[int]
    ctx_before: List[int]
    max_q_len: int
    max_ctx: int                       # longest context after this step
    token_ids: torch.Tensor            # [n_tokens] int32
    positions: torch.Tensor            # [n_tokens] int32, absolute position of each token
    token_seq: torch.Tensor            # [n_tokens] int32, which sequence of the batch
    cu_q: torch.Tensor                 # [n_seqs + 1] int32
    ctx_after: torch.Tensor            # [n_seqs] int32
    slot_ids: torch.Tensor             # [n_seqs] int32
    block_tables: Dict[int, torch.Tensor]
    cache: Any                         # cache.KVCache
    scratch: Dict[str, torch.Tensor] = field(default_factory=dict)
    residual_stats: Any = None         # residual.ResidualStats when norms may be folded into projections
    norm_after_layer: Any = None       # then: the foldable norm that reads the stream after the running layer

    @property
    def is_decode(self) -> bool:
        return self.max_q_len == 1


class Part:
    role = "part"
    # True if forward() only launches kernels on fixed device buffers (no host reads of
    # device data, no host-side per-sequence work), so a step can be captured in a CUDA graph.
    graph_safe = False
    # True if the part (a norm) can hand over ``residual.NormedRows`` instead of applying itself, or
    # (a mixer, a feed-forward) takes them as its input and keeps ``step.residual_stats`` up to date
    # when it adds to the stream.  The arrangement asks before it uses either.
    folds_norm = False

    def __init__(self, spec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime

    @classmethod
    def expected_tensors(cls, spec) -> Dict[str, TensorRequest]:
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receive the checkpoint tensors named by ``expected_tensors`` (CPU, stored dtype)."""


class Norm(Part):
    role = "norm"

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    role = "mixer"

    @classmethod
    def cache_request(cls, spec) -> CacheRequest:
        return CacheRequest()

    def forward(self, step: StepBatch, h: torch.Tensor, x: torch.Tensor,
                cache_entry: int, writes_cache: bool) -> None:
        raise NotImplementedError


class FeedForward(Part):
    role = "ffn"

    def forward(self, step: StepBatch, h: torch.Tensor, x: torch.Tensor) -> None:
        raise NotImplementedError
