"""A stand-in for the CUDA kernel library, used only by CPU tests of the engine's
bookkeeping (batch packing, cache slots and block tables, the order of parts).

It has the call signatures of ``stratakv_b200.ops.Kernels`` and computes each
call with plain torch on whatever device the tensors are on.  The package never
imports it; the product path has no CPU backend.
"""
from __future__ import annotations

import torch

MODE_STORE, MODE_STORE_F32, MODE_ADD_F32, MODE_GATED = 0, 1, 2, 3


class DoubleKernels:
    def __init__(self, dtype, head_dim):
        self.dtype = dtype
        self.head_dim = head_dim
        self.calls = []

    def embed(self, table, ids, out, flag=None, stats=None):
        self.calls.append("embed")
        out.copy_(table[ids.long()].float())

    def rmsnorm(self, x, gamma, eps, out, rows=None):
        self.calls.append("rmsnorm")
        src = x if rows is None else x[rows.long()]
        inv = 1.0 / torch.sqrt((src * src).mean(dim=-1, keepdim=True) + eps)
        out.copy_((src * inv * gamma).to(out.dtype))

    def linear(self, a, w, out, mode=MODE_STORE, activation="silu", flag=None, stats=None):
        self.calls.append("linear")
        result = a.float() @ w.float().T
        if mode == MODE_GATED:
            tiles = result.view(result.shape[0], -1, 2, 8)
            gate, up = tiles[:, :, 0, :], tiles[:, :, 1, :]
            out.copy_((gate * torch.sigmoid(gate) * up).reshape(result.shape[0], -1).to(out.dtype))
        elif mode == MODE_ADD_F32:
            out.add_(result)
        else:
            out.copy_(result.to(out.dtype))

    def rope_kv_write(self, qkv, cos_sin, positions, token_seq, block_table, q_out, k_cache, v_cache,
                      num_heads, num_kv_heads, head_dim, block_size, write_kv):
        self.calls.append("rope_kv_write")
        n = qkv.shape[0]
        q_dim, kv_dim, half = num_heads * head_dim, num_kv_heads * head_dim, head_dim // 2
        q = qkv[:, :q_dim].view(n, num_heads, head_dim)
        k = qkv[:, q_dim:q_dim + kv_dim].view(n, num_kv_heads, head_dim)
        v = qkv[:, q_dim + kv_dim:].view(n, num_kv_heads, head_dim)

        def rotate(x):
            if cos_sin is None:
                return x
            cs = cos_sin[positions.long()]                        # [n, half, 2]
            c, s = cs[:, None, :, 0], cs[:, None, :, 1]
            x1, x2 = x[..., :half], x[..., half:]
            return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)

        q_out.copy_(rotate(q).reshape(n, q_dim).to(q_out.dtype))
        if write_kv:
            k = rotate(k)
            for t in range(n):
                pos = int(positions[t])
                block = int(block_table[int(token_seq[t]), pos // block_size])
                k_cache[block, :, pos % block_size, :] = k[t].to(k_cache.dtype)
                v_cache[block, :, pos % block_size, :] = v[t].to(v_cache.dtype)

    def attention(self, q, k_cache, v_cache, block_table, positions, token_seq, out, num_heads,
                  num_kv_heads, head_dim, block_size, scale, window=0):
        self.calls.append("attention")
        n = q.shape[0]
        group = num_heads // num_kv_heads
        qh = q.view(n, num_heads, head_dim).float()
        result = torch.zeros(n, num_heads, head_dim)
        for t in range(n):
            pos, seq = int(positions[t]), int(token_seq[t])
            lo = max(0, pos - window + 1) if window > 0 else 0
            keys = torch.stack([k_cache[int(block_table[seq, j // block_size]), :, j % block_size, :]
                                for j in range(lo, pos + 1)]).float()       # [ctx, kv_heads, d]
            values = torch.stack([v_cache[int(block_table[seq, j // block_size]), :, j % block_size, :]
                                  for j in range(lo, pos + 1)]).float()
            for h in range(num_heads):
                g = h // group
                weights = torch.softmax((keys[:, g, :] @ qh[t, h]) * scale, dim=0)
                result[t, h] = weights @ values[:, g, :]
        out.copy_(result.reshape(n, num_heads * head_dim).to(out.dtype))

    def add_inplace(self, out, other):
        out.add_(other)

    def argmax(self, logits, out, flag=None):
        out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))


def double_loader():
    made = {}

    def load(dtype, head_dim):
        key = (dtype, head_dim)
        if key not in made:
            made[key] = DoubleKernels(dtype, head_dim)
        return made[key]
    return load
