"""Entry point of the tensor-core attention kernels (csrc/attn_mma.cu)."""
from __future__ import annotations

ENABLED = False


def accepts(q, kv, head_dim, n_heads, n_kv_heads) -> bool:
    return False


def attention(q, kv, out, batch, n_heads, n_kv_heads, head_dim, scale, rt):
    raise NotImplementedError
