"""Tensor-level entry points of the hand-written sm_100a kernels.

Every function takes CUDA tensors and launches on PyTorch's current stream; none has a CPU or
library stand-in.  Shapes use N = tokens of the step, H = width of the residual stream.
The residual stream is always float32; "activation type" is the model's dtype (float32 on the
32-bit path, bfloat16 on the serving path).
"""
from __future__ import annotations

from typing import Optional

import torch

from .library import (KernelError, call, check, declare, dtype_code, launch_count, library, pointer,
                      require_device, stream_handle, wait_error_flag)
from .stream import STREAM_ROWS, RowScaled, StreamSink

__all__ = ["KernelError", "embedding", "add_rmsnorm", "rmsnorm", "silu_mul", "sample", "qk_norm_rope_kv_write",
           "attention_generic", "gemm_f32", "linear", "qkv_projection", "gate_up_silu", "interleave_gate_up", "require_device", "library", "launch_count",
           "RowScaled", "StreamSink", "STREAM_ROWS", "unscaled_rows_supported"]


def embedding(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual[n] = table[ids[n]] widened to float32.  ids: int32 [N]."""
    check(table, "embedding table")
    check(ids, "token ids", torch.int32)
    vocab, hidden = table.shape
    tokens = ids.numel()
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    check(out, "embedding output", torch.float32, hidden)
    call("llm_embedding_gather", out.data_ptr(), table.data_ptr(), ids.data_ptr(), tokens, hidden, vocab,
         dtype_code(table.dtype), stream_handle())
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                write_residual: bool = True, act_dtype: Optional[torch.dtype] = None, unscaled: bool = False):
    """residual += delta (in place, 32-bit), then out = rmsnorm(residual) * weight in the activation
    type ``act_dtype`` (default: weight's dtype; the weight may be float32 beside bfloat16 activations).

    ``rows`` (int32) selects source rows: output row o comes from row rows[o]; then the residual is
    left untouched and ``delta`` is added on the fly.  ``unscaled``: the division by the root mean square is left to
    the product that consumes the result; returns a ``RowScaled`` (residual * weight and the rows' sums of squares)."""
    check(residual, "residual", torch.float32)
    width = residual.shape[-1]
    check(weight, "norm weight", last_dim=width)
    act = act_dtype or weight.dtype
    if delta is not None:
        check(delta, "delta", act, width)
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match residual {tuple(residual.shape)}")
    if rows is not None:
        check(rows, "rows", torch.int32)
        n_rows, write_residual = rows.numel(), False
    else:
        n_rows = residual.numel() // width
    if out is None:
        out = torch.empty((n_rows, width), dtype=act, device=residual.device)
    check(out, "norm output", act, width)
    squares = torch.empty((1, max(n_rows, 1)), dtype=torch.float32, device=residual.device) if unscaled else None
    call("llm_add_rmsnorm", residual.data_ptr(), pointer(delta), weight.data_ptr(), out.data_ptr(), pointer(rows),
         n_rows, width, float(eps), int(write_residual), dtype_code(act), dtype_code(weight.dtype), pointer(squares),
         stream_handle())
    return RowScaled(out, squares, eps) if unscaled else out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = rmsnorm(x) * weight over the last dimension; x in the activation type."""
    width = x.shape[-1]
    check(x, "x")
    check(weight, "norm weight", last_dim=width)
    if out is None:
        out = torch.empty_like(x)
    check(out, "norm output", x.dtype, width)
    call("llm_rmsnorm", x.data_ptr(), weight.data_ptr(), out.data_ptr(), x.numel() // width, width, float(eps),
         dtype_code(x.dtype), dtype_code(weight.dtype), stream_handle())
    return out


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, group: int = 0) -> torch.Tensor:
    """out[n, i] = silu(gate_up[n, i]) * gate_up[n, I + i]; gate_up is [N, 2 I], gate half first.  With ``group`` > 0
    gate and up columns are interleaved in groups of that many: output i finds its gate value at column
    (i // group) * 2 * group + i % group and its up value ``group`` columns further."""
    check(gate_up, "gate_up")
    rows, doubled = gate_up.shape
    if doubled % 2:
        raise KernelError(f"gate_up's last dimension must be even, got {doubled}")
    if out is None:
        out = torch.empty((rows, doubled // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(out, "silu_mul output", gate_up.dtype, doubled // 2)
    call("llm_silu_mul", gate_up.data_ptr(), out.data_ptr(), rows, doubled // 2, int(group), dtype_code(gate_up.dtype),
         stream_handle())
    return out


GATE_UP_GROUP = 64      # rows of gate and of up that share a 128-row tile of the fused weight


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int = GATE_UP_GROUP) -> torch.Tensor:
    """The fused [2 I, H] weight with gate and up rows interleaved in groups (see ``silu_mul``): a 128-row tile then
    holds 64 gate rows and their 64 up rows, so the product kernel can apply the gate in its epilogue."""
    inter, hidden = gate.shape
    if inter % group:
        raise KernelError(f"the intermediate size {inter} is no multiple of {group}")
    return torch.stack([gate.reshape(inter // group, group, hidden), up.reshape(inter // group, group, hidden)],
                       dim=1).reshape(2 * inter, hidden).contiguous()


def gate_up_silu(x, weight: torch.Tensor, group: int = 0) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for the fused weight ``weight`` [2 I, H] (halves when ``group`` is 0, else interleaved in
    groups): as one kernel where the product kernel can apply the gate in its epilogue (bfloat16, groups of 64, few
    rows), else as the product followed by ``silu_mul``.  ``x`` may be a ``RowScaled``."""
    if x.dtype == torch.bfloat16 and group == GATE_UP_GROUP:
        from . import gemm_bf16
        fused = gemm_bf16.gate_up_silu_fused(x, weight)
        if fused is not None:
            return fused
    return silu_mul(linear(x, weight), group=group)


def sample(logits: torch.Tensor, temperatures: Optional[torch.Tensor] = None, seeds: Optional[torch.Tensor] = None,
           steps: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V]: argmax where the temperature is 0, else the
    Gumbel-max draw keyed by (seeds[r], steps[r]).  Returns int32 [R]."""
    check(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    if temperatures is not None:
        check(temperatures, "temperatures", torch.float32)
        if seeds is None or steps is None:
            raise KernelError("temperature sampling needs seeds and steps")
        check(seeds, "seeds", torch.int64)
        check(steps, "steps", torch.int32)
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(out, "sampled tokens", torch.int32)
    slices = library().llm_sample_slices(rows, vocab)
    scores = indices = None
    if slices > 1:      # large vocabularies are scanned by several blocks per row, merged by a second kernel
        scores = torch.empty((rows, slices), dtype=torch.float32, device=logits.device)
        indices = torch.empty((rows, slices), dtype=torch.int32, device=logits.device)
    call("llm_sample", logits.data_ptr(), pointer(temperatures), pointer(seeds), pointer(steps), out.data_ptr(), rows,
         vocab, pointer(scores), pointer(indices), stream_handle())
    return out


def qk_norm_rope_kv_write(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                          inv_freq: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor,
                          block_tables: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, n_q_heads: int,
                          n_kv_heads: int, head_dim: int, eps: float, write_cache: bool,
                          error_flag: torch.Tensor, rotary_dim: Optional[int] = None, interleaved: bool = False) -> None:
    """In place on qkv [N, (Hq + 2 Hkv) D]: Q heads normalised and rotated where they are; K heads
    normalised, rotated and written to the K pages; V heads copied to the V pages.  Pages are
    [page, Hkv, page_size, D]; block_tables int32 [S, max_blocks].  ``rotary_dim`` (default: all of the head)
    elements of each head are rotated, by the angles position * inv_freq[i], i < rotary_dim / 2, paired as halves
    (i, i + rotary_dim / 2) or, ``interleaved``, as neighbours (2i, 2i + 1)."""
    if rotary_dim is None:
        rotary_dim = head_dim if inv_freq is None else 2 * inv_freq.numel()
    if rotary_dim % 2 or not 0 <= rotary_dim <= head_dim:
        raise KernelError(f"rotary_dim must be even and at most head_dim {head_dim}, got {rotary_dim}")
    check(qkv, "qkv", last_dim=(n_q_heads + 2 * n_kv_heads) * head_dim)
    tokens = qkv.shape[0]
    weight_dtype = qkv.dtype
    for name, tensor in (("q norm weight", q_weight), ("k norm weight", k_weight)):
        if tensor is not None:
            check(tensor, name, last_dim=head_dim)
            weight_dtype = tensor.dtype
    if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
        raise KernelError("q and k norm weights must share a dtype")
    if inv_freq is not None:
        check(inv_freq, "inv_freq", torch.float32, rotary_dim // 2)
    check(positions, "positions", torch.int32)
    check(seq_of_token, "seq_of_token", torch.int32)
    check(block_tables, "block_tables", torch.int32)
    check(k_pages, "k pages", qkv.dtype, head_dim)
    check(v_pages, "v pages", qkv.dtype, head_dim)
    if k_pages.shape != v_pages.shape or k_pages.dim() != 4 or k_pages.shape[1] != n_kv_heads:
        raise KernelError(f"pages must be [pages, {n_kv_heads}, page_size, {head_dim}], got {tuple(k_pages.shape)}")
    if positions.numel() != tokens or seq_of_token.numel() != tokens:
        raise KernelError("positions and seq_of_token need one entry per token")
    check(error_flag, "error flag", torch.int32)
    call("llm_qk_norm_rope_kv_write", qkv.data_ptr(), pointer(q_weight), pointer(k_weight), pointer(inv_freq),
         positions.data_ptr(), seq_of_token.data_ptr(), block_tables.data_ptr(), block_tables.shape[-1],
         k_pages.data_ptr(), v_pages.data_ptr(), tokens, n_q_heads, n_kv_heads, head_dim, k_pages.shape[2],
         k_pages.shape[0], float(eps), int(write_cache), error_flag.data_ptr(), int(rotary_dim), int(bool(interleaved)),
         dtype_code(qkv.dtype), dtype_code(weight_dtype), stream_handle())


def attention_generic(q: torch.Tensor, q_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_tables: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                      n_q_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                      out: Optional[torch.Tensor] = None, error_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal (optionally windowed) attention of every token over its sequence's pages, 32-bit
    arithmetic.  ``q`` holds head h of token n at q[n * q_stride + h * D]; returns [N, Hq * D].  A block-table entry
    that names no page of the pool is not followed: page 0 is read instead and ``error_flag`` (default: the device's
    shared flag) is set to 5."""
    check(q, "q")
    tokens = positions.numel()
    check(k_pages, "k pages", q.dtype, head_dim)
    check(v_pages, "v pages", q.dtype, head_dim)
    check(block_tables, "block_tables", torch.int32)
    check(seq_of_token, "seq_of_token", torch.int32)
    check(positions, "positions", torch.int32)
    if out is None:
        out = torch.empty((tokens, n_q_heads * head_dim), dtype=q.dtype, device=q.device)
    check(out, "attention output", q.dtype, n_q_heads * head_dim)
    call("llm_attention_generic", q.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(),
         block_tables.data_ptr(), block_tables.shape[-1], seq_of_token.data_ptr(), positions.data_ptr(),
         out.data_ptr(), tokens, n_q_heads, n_kv_heads, head_dim, k_pages.shape[2], k_pages.shape[0], float(scale),
         int(window), (error_flag if error_flag is not None else wait_error_flag(q.device)).data_ptr(), dtype_code(q.dtype),
         stream_handle())
    return out


def gemm_f32(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] times weight [N, K] transposed, all float32, FMA only (no tensor cores, no TF32)."""
    check(x, "x", torch.float32)
    check(weight, "weight", torch.float32, x.shape[-1])
    rows, inner = x.shape
    cols = weight.shape[0]
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.float32, device=x.device)
    check(out, "gemm output", torch.float32, cols)
    call("llm_gemm_f32", x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, cols, inner, inner, inner, cols,
         stream_handle())
    return out


def linear(x, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, sink: Optional[StreamSink] = None) -> Optional[torch.Tensor]:
    """y = x W^T for W stored [out, in] (utils/attention.py:119-124 uses nn.Linear for the same).

    float32: this package's FMA kernel.  bfloat16: the library matrix product (cuBLAS through
    PyTorch) where the reference's engine uses a library too, or this package's own kernels where
    they apply (see ``gemm_bf16``).  ``x`` may be a ``RowScaled``.  With a ``sink`` the product is added to the sink's
    residual stream by the product kernel itself where that kernel takes the case (``sink.added`` then says so and
    nothing is returned); otherwise the sink is left alone and the product is returned as usual."""
    if x.device.type != "cuda":
        raise KernelError("linear: there is no CPU path")
    if x.dtype == torch.float32:
        result = gemm_f32(x, weight, out)
        return result
    from . import gemm_bf16
    if sink is not None and out is None and not isinstance(x, RowScaled) and gemm_bf16.linear_into_stream(x, weight, sink):
        return None
    return gemm_bf16.linear_bf16(x, weight, out=out, out_dtype=out_dtype)


def unscaled_rows_supported(weight: torch.Tensor) -> bool:
    """Whether products with ``weight`` take ``RowScaled`` rows."""
    from . import gemm_bf16
    return gemm_bf16.unscaled_rows_supported(weight)


def qkv_projection(x, weight: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                   inv_freq: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor,
                   block_tables: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, n_q_heads: int, n_kv_heads: int,
                   head_dim: int, eps: float, write_cache: bool, error_flag: torch.Tensor, rotary_dim: Optional[int] = None,
                   interleaved: bool = False) -> torch.Tensor:
    """qkv = x W^T followed by ``qk_norm_rope_kv_write``: as one kernel where the product kernel can finish heads in its
    epilogue (bfloat16, heads of 128, up to 64 tokens, the whole head rotating in halves; from 17 tokens on only where
    that is measured to be faster), else as two.  ``x`` may be a ``RowScaled``."""
    whole_head = rotary_dim is None or rotary_dim == head_dim
    if x.dtype == torch.bfloat16 and whole_head and not interleaved and x.shape[0] <= 64:
        from . import gemm_bf16
        fused = gemm_bf16.qkv_rope_fused(x, weight, q_weight, k_weight, inv_freq, positions, seq_of_token, block_tables,
                                         k_pages, v_pages, n_q_heads, n_kv_heads, head_dim, eps, write_cache, error_flag)
        if fused is not None:
            return fused
    qkv = linear(x, weight)
    qk_norm_rope_kv_write(qkv, q_weight, k_weight, inv_freq, positions, seq_of_token, block_tables, k_pages, v_pages,
                          n_q_heads, n_kv_heads, head_dim, eps, write_cache, error_flag, rotary_dim, interleaved)
    return qkv


def attention(qkv: torch.Tensor, batch, block_tables: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
              n_q_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> torch.Tensor:
    """Attention of a step's tokens over the paged cache; ``qkv`` is the packed projection whose Q
    heads have been normalised and rotated in place.  Chooses the kernel by dtype, head size and the
    shape of the batch; every choice computes the same function."""
    q_stride = (n_q_heads + 2 * n_kv_heads) * head_dim
    if qkv.dtype == torch.bfloat16:
        from . import attention_bf16
        result = attention_bf16.try_attention(qkv, q_stride, batch, block_tables, k_pages, v_pages, n_q_heads,
                                              n_kv_heads, head_dim, scale, window)
        if result is not None:
            return result
    return attention_generic(qkv, q_stride, k_pages, v_pages, block_tables, batch.seq_of_token, batch.positions,
                             n_q_heads, n_kv_heads, head_dim, scale, window)
