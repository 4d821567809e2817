"""bfloat16 matrix products y = x W^T with 32-bit accumulation.

The reference's engine runs every projection through a library matrix product (nn.Linear on
cuBLAS: utils/attention.py:119-124,181; utils/layers.py:205-217; utils/model.py:170).  Here:

* up to 64 rows (decode steps, the output head): this package's tcgen05 / TMA kernel
  (``csrc/gemm_tcgen05.cu``), which streams the weights once and can write float32 directly, or the
  library product, whichever a one-time measurement per shape finds faster;
* more rows (prompt portions): the library product (cuBLAS through PyTorch).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .library import KernelError, call, check_wait_errors, library, stream_handle, wait_error_flag
from .stream import NO_SCALE, STREAM_ROWS, RowScaled, StreamSink, rows_of, scale_args_of

SMALL_M = 64
_use_small_m = os.environ.get("LLMSERVER_B200_SMALL_M_GEMM", "1") != "0"
error_flag = wait_error_flag        # the kernels of this package share one flag per device
check_errors = check_wait_errors


def small_m_supported(rows: int, cols: int, inner: int) -> bool:
    return _use_small_m and bool(library().llm_gemm_small_m_supports(rows, cols, inner))


# (row bucket, N, K, out dtype) -> split of K to use with this package's kernel, or 0 for the library product.
_choice = {}
SPLITS = (1, 2, 3, 4, 6, 8)
ROW_BUCKETS = (1, 2, 4, 8, 16, 32, 48, 64)
_tunings = 0


def tunings() -> int:
    """How many (row bucket, shape) choices were made by measurement in this process."""
    return _tunings


def _row_bucket(rows: int) -> int:
    for bucket in ROW_BUCKETS:
        if rows <= bucket:
            return bucket
    return SMALL_M


# The choices can be kept in a file (LLMSERVER_B200_GEMM_PLAN): what is in the file is used as it is, what is
# measured is added to it.  The choice fixes the order in which a product's partial sums are added, so two processes
# that read the same file give bit-identical bfloat16 results; without a file each process measures for itself and a
# close race may go either way.
PLAN_FILE = os.environ.get("LLMSERVER_B200_GEMM_PLAN")
_plan_loaded = False


OWN_KERNEL = "bf16-own"      # in place of the output type in a key: the choice among this package's variants only


def _key_text(key) -> str:
    bucket, cols, inner, out_dtype = key
    kind = out_dtype if isinstance(out_dtype, str) else ("f32" if out_dtype == torch.float32 else "bf16")
    return f"{bucket},{cols},{inner},{kind}"


def load_plan(path: Optional[str] = None) -> int:
    """Reads choices from ``path`` (default: the file named by LLMSERVER_B200_GEMM_PLAN); returns how many."""
    global _plan_loaded
    _plan_loaded = True
    path = path or PLAN_FILE
    if not path or not os.path.isfile(path):
        return 0
    count = 0
    with open(path) as handle:
        for line in handle:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            try:
                bucket, cols, inner, kind, split = line.split(",")
                key = (int(bucket), int(cols), int(inner),
                       {"f32": torch.float32, "bf16": torch.bfloat16}.get(kind, kind))
                _choice.setdefault(key, int(split))
                count += 1
            except ValueError as error:
                raise KernelError(f"{path}: cannot read the line {line!r} (row bucket,N,K,f32|bf16,split)") from error
    return count


def save_plan(path: Optional[str] = None) -> None:
    """Writes every known choice to ``path`` (default: the file named by LLMSERVER_B200_GEMM_PLAN)."""
    path = path or PLAN_FILE
    if not path:
        raise KernelError("no plan file was named (LLMSERVER_B200_GEMM_PLAN)")
    lines = ["# row bucket,N,K,output,split of K (0: library product)"]
    lines += [f"{_key_text(key)},{split}" for key, split in sorted(_choice.items(), key=lambda item: _key_text(item[0]))]
    temporary = f"{path}.{os.getpid()}.tmp"
    with open(temporary, "w") as handle:
        handle.write("\n".join(lines) + "\n")
    os.replace(temporary, path)


_flush_buffer = {}


_ROUNDS = 4
_empty_round = {}
# Between two small kernels the candidates often lie within a few percent of each other, and whole steps decide
# differently from that measurement at the two ends: up to 16 rows a step is faster with this package's kernel
# wherever the two are close (its weight stream starts before its predecessor ends, and it lets its successor launch
# early), from 32 rows on with the library's.  So a candidate of the other kind has to win by this much.
_CLOSE_FEW_ROWS = 0.10
_CLOSE_MANY_ROWS = 0.05
# Among the splits of this package's kernel, the ones within this much of the fastest count as equal, and the largest
# of them is taken: measured one product at a time, 6 and 8 parts of the 8B shape's q/k/v and output projections lie
# within 1 to 3.5 % of each other and the choice went either way from process to process, while whole steps are 1 to
# 2 % faster with 8 (more blocks keep more bytes in flight where one kernel hands over to the next).
_CLOSE_SPLITS = float(os.environ.get("LLMSERVER_B200_GEMM_CLOSE_SPLITS", "0.04"))


def _fastest_split(timed: list) -> int:
    """``timed``: (split, milliseconds) of this package's kernel; the largest split among the (nearly) fastest."""
    fastest = min(elapsed for _, elapsed in timed)
    return max(split for split, elapsed in timed if elapsed <= fastest * (1.0 + _CLOSE_SPLITS))


def _time_in_step(run, device, repeats: int = 10) -> float:
    """Time of ``run`` as a model step sees it: replayed from a CUDA graph between two small kernels of this package
    (so that a product which starts its weight stream while its predecessor still runs, and lets its successor
    launch early, gets the credit), with the weights coming from HBM (a buffer larger than L2 is overwritten before
    each round).  Milliseconds per round, less the time of a round without ``run``."""
    from . import rmsnorm
    if device not in _flush_buffer:
        _flush_buffer[device] = (torch.empty(256 << 20, dtype=torch.int8, device=device),
                                 torch.zeros((8, 1024), dtype=torch.bfloat16, device=device),
                                 torch.ones(1024, dtype=torch.bfloat16, device=device))
    flush, small_in, small_weight = _flush_buffer[device]
    small_out = torch.empty_like(small_in)

    def measure(body) -> float:
        def rounds():
            for _ in range(_ROUNDS):
                flush.zero_()
                rmsnorm(small_in, small_weight, 1e-6, out=small_out)
                body()
                rmsnorm(small_out, small_weight, 1e-6, out=small_in)

        rounds()
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            rounds()
        graph.replay()
        best = float("inf")
        for _ in range(repeats):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            graph.replay()
            end.record()
            end.synchronize()
            best = min(best, begin.elapsed_time(end))
        return best / _ROUNDS

    if device not in _empty_round:
        _empty_round[device] = measure(lambda: None)
    return measure(run) - _empty_round[device]


def _small_m(x, weight, out, split: int, scale: tuple = NO_SCALE) -> None:
    rows, inner = x.shape
    cols = weight.shape[0]
    call("llm_gemm_small_m", x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, cols, inner, cols,
         int(out.dtype == torch.float32), split, *scale, error_flag(x.device).data_ptr(), stream_handle())


def _plan_for(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, own_kernel_only: bool = False) -> int:
    """``own_kernel_only``: the best split of this package's kernel, the library's product not considered (for the
    products that finish their result in the kernel's epilogue, which the library's cannot; kept under a key of its own).

    Measures, once per (rows bucket, shape), this package's kernel with a few splits of K and the
    library product, each as a model step runs it, and remembers the fastest: a split (> 0) or 0 for the library.  All candidates read
    the same operands and give the same result up to rounding, so the choice changes speed only.
    While a CUDA graph is being captured nothing can be timed: an unknown shape then uses this
    package's kernel with its default split."""
    global _tunings
    rows, inner = x.shape
    cols = weight.shape[0]
    key = (_row_bucket(rows), cols, inner, OWN_KERNEL if own_kernel_only else out_dtype)
    known = _choice.get(key)
    if known is not None:
        return known
    if not _plan_loaded:
        load_plan()
        if key in _choice:
            return _choice[key]
    if torch.cuda.is_current_stream_capturing():
        return -1
    if out_dtype == torch.float32 or own_kernel_only:
        # 32-bit results always come from this package's kernel, straight from its accumulators; only the split is
        # measured (the library's product would have to be rounded to bfloat16 on the way)
        out = torch.empty((rows, cols), dtype=out_dtype, device=x.device)
        timed = []
        tiles, k_blocks = -(-cols // 128), -(-inner // 128)
        for split in SPLITS:
            if split > 1 and (tiles * split > 600 or k_blocks // split < 2):
                continue
            timed.append((split, _time_in_step(lambda: _small_m(x, weight, out, split), x.device)))
        best = _fastest_split(timed)
        _choice[key] = best
        _tunings += 1
        if PLAN_FILE:
            save_plan()
        return best
    out = torch.empty((rows, cols), dtype=out_dtype, device=x.device)

    def library_product():
        torch.matmul(x, weight.t(), out=out)

    favour_library = key[0] > 16
    best_time = _time_in_step(library_product, x.device) * ((1.0 - _CLOSE_MANY_ROWS) if favour_library else (1.0 + _CLOSE_FEW_ROWS))
    timed = []
    tiles, k_blocks = -(-cols // 128), -(-inner // 128)
    for split in SPLITS:
        if split > 1 and (tiles * split > 600 or k_blocks // split < 2):
            continue
        timed.append((split, _time_in_step(lambda: _small_m(x, weight, out, split), x.device)))
    best = _fastest_split(timed) if min(elapsed for _, elapsed in timed) < best_time else 0
    _choice[key] = best
    _tunings += 1
    if PLAN_FILE:
        save_plan()
    return best


def unscaled_rows_supported(weight: torch.Tensor) -> bool:
    """Whether products with ``weight`` [N, K] take ``RowScaled`` input (this package's kernel has to take the shape)."""
    return (STREAM_ROWS > 0 and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.is_contiguous()
            and small_m_supported(STREAM_ROWS, weight.shape[0], weight.shape[1]))


def linear_into_stream(x: torch.Tensor, weight: torch.Tensor, sink: StreamSink) -> bool:
    """sink.residual += x W^T in the product kernel's epilogue and, when the sink names a norm weight, the input of
    that norm (``sink.scaled``).  False, with nothing done, when the kernel does not take the case."""
    rows, inner = x.shape
    cols = weight.shape[0]
    residual = sink.residual
    if not (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.is_contiguous() and weight.is_contiguous()
            and rows <= STREAM_ROWS and small_m_supported(rows, cols, inner) and residual.dtype == torch.float32
            and residual.is_contiguous() and tuple(residual.shape) == (rows, cols)):
        return False
    norm_weight = sink.norm_weight
    if norm_weight is not None and (norm_weight.dtype not in (torch.bfloat16, torch.float32) or norm_weight.numel() != cols
                                    or not norm_weight.is_contiguous()):
        return False
    split = max(_plan_for(x, weight, torch.bfloat16, own_kernel_only=True), 0)
    scaled = parts = None
    if norm_weight is not None:
        scaled = torch.empty((rows, cols), dtype=torch.bfloat16, device=x.device)
        parts = torch.empty((library().llm_gemm_into_stream_parts(cols), max(STREAM_ROWS, rows)), dtype=torch.float32, device=x.device)
    call("llm_gemm_into_stream", x.data_ptr(), weight.data_ptr(), residual.data_ptr(), rows, cols, inner, split,
         0 if norm_weight is None else norm_weight.data_ptr(), int(norm_weight is not None and norm_weight.dtype == torch.float32),
         0 if scaled is None else scaled.data_ptr(), 0 if parts is None else parts.data_ptr(), 0 if parts is None else parts.shape[1],
         error_flag(x.device).data_ptr(), stream_handle())
    sink.added = True
    if norm_weight is not None:
        sink.scaled = RowScaled(scaled, parts, sink.eps)
    return True


def linear_bf16(x, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    if isinstance(x, RowScaled):
        # rows that still have to be divided by their root mean square: only this package's kernel can do that
        rows, inner = x.shape
        cols = weight.shape[0]
        out_dtype = out_dtype or torch.bfloat16
        if not (rows <= SMALL_M and unscaled_rows_supported(weight) and x.x.is_contiguous()):
            raise KernelError(f"linear_bf16: no product kernel takes unscaled rows for {rows} rows and a weight {tuple(weight.shape)}")
        if out is None:
            out = torch.empty((rows, cols), dtype=out_dtype, device=x.device)
        own_only = out_dtype != torch.float32
        _small_m(x.x, weight, out, max(_plan_for(x.x, weight, out_dtype, own_kernel_only=own_only), 0), x.scale_args())
        return out
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise KernelError(f"linear_bf16 takes bfloat16 operands, got {x.dtype} and {weight.dtype}")
    out_dtype = out_dtype or torch.bfloat16
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"linear_bf16 writes bfloat16 or float32, not {out_dtype}")
    rows, inner = x.shape
    cols = weight.shape[0]
    if out is not None and (out.dtype != out_dtype or not out.is_contiguous() or out.shape != (rows, cols)):
        raise KernelError("linear_bf16: the output tensor does not match")
    own_kernel = x.is_contiguous() and weight.is_contiguous() and small_m_supported(min(rows, SMALL_M), cols, inner)
    if out_dtype == torch.float32:
        # logits: 32-bit sums written as they are, whatever the number of rows (never a bfloat16 product widened
        # afterwards: rounding 150 thousand logits to 8 bits makes ties, and ties would then depend on the row count)
        if not own_kernel:
            return _float32_by_library(x, weight, out)
        if out is None:
            out = torch.empty((rows, cols), dtype=out_dtype, device=x.device)
        for begin in range(0, rows, SMALL_M):
            part = x[begin:begin + SMALL_M]
            _small_m(part, weight, out[begin:begin + SMALL_M], max(_plan_for(part, weight, out_dtype), 0))
        return out
    if rows <= SMALL_M and own_kernel:
        split = _plan_for(x, weight, out_dtype)
        if split != 0:
            if out is None:
                out = torch.empty((rows, cols), dtype=out_dtype, device=x.device)
            _small_m(x, weight, out, max(split, 0))
            return out
    if out is not None:
        return torch.matmul(x, weight.t(), out=out)
    return torch.matmul(x, weight.t())


def _float32_by_library(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor]) -> torch.Tensor:
    """For shapes this package's kernel does not take: the library's product with a 32-bit result (32-bit sums of
    bfloat16 products, not a rounded bfloat16 result widened)."""
    result = torch.mm(x, weight.t(), out_dtype=torch.float32)
    if out is not None:
        out.copy_(result)
        return out
    return result


def _plan_fused(kind: str, rows: int, cols: int, inner: int, fused, apart, device) -> int:
    """For 17 to 64 rows: the split with which the fused kernel ``fused(split)`` is fastest inside a step, or 0 when
    the library's product followed by the kernel of its own (``apart()``) is faster.  Measured once per (kind, row
    bucket, shape), kept with the other choices (and in the plan file).  While a graph is being captured nothing can
    be measured: an unknown shape then runs apart."""
    global _tunings
    key = (_row_bucket(rows), cols, inner, kind)
    known = _choice.get(key)
    if known is not None:
        return known
    if not _plan_loaded:
        load_plan()
        if key in _choice:
            return _choice[key]
    if torch.cuda.is_current_stream_capturing():
        return 0
    apart_time = _time_in_step(apart, device)
    timed = []
    tiles, k_blocks = -(-cols // 128), -(-inner // 128)
    for split in SPLITS:
        if split > 1 and (tiles * split > 600 or k_blocks // split < 2):
            continue
        timed.append((split, _time_in_step(lambda: fused(split), device)))
    best = _fastest_split(timed) if min(elapsed for _, elapsed in timed) < apart_time else 0
    _choice[key] = best
    _tunings += 1
    if PLAN_FILE:
        save_plan()
    return best


FUSE_QKV_ROPE = os.environ.get("LLMSERVER_B200_FUSE_QKV_ROPE", "1") != "0"


def qkv_rope_fused(x: torch.Tensor, weight: torch.Tensor, q_weight, k_weight, inv_freq, positions, seq_of_token,
                   block_tables, k_pages, v_pages, n_q_heads: int, n_kv_heads: int, head_dim: int, eps: float,
                   write_cache: bool, page_error: torch.Tensor) -> Optional[torch.Tensor]:
    """The fused q/k/v projection of a step with few tokens: x W^T, then, in the product kernel's epilogue, the per-head
    norms, the rotation and the cache write (see ``ops.qk_norm_rope_kv_write`` for the arithmetic).  Returns the packed
    [N, (Hq + 2 Hkv) D] tensor whose Q heads are finished (its K and V heads are not written: they went to the pages),
    or None when the fused kernel does not take the case; the caller then runs the two kernels one after the other."""
    scale, x = scale_args_of(x), rows_of(x)
    rows, inner = x.shape
    if not (FUSE_QKV_ROPE and _use_small_m and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and x.is_contiguous() and weight.is_contiguous() and k_pages.dtype == torch.bfloat16
            and library().llm_gemm_qkv_rope_supports(rows, n_q_heads, n_kv_heads, head_dim, inner)):
        return None
    if weight.shape[0] != (n_q_heads + 2 * n_kv_heads) * head_dim:
        return None
    if (q_weight is None) != (k_weight is None) or (q_weight is not None and q_weight.dtype != k_weight.dtype):
        return None
    if inv_freq is not None and inv_freq.numel() * 2 != head_dim:
        return None
    out = torch.empty((rows, weight.shape[0]), dtype=torch.bfloat16, device=x.device)

    def fused(split: int) -> None:
        call("llm_gemm_qkv_rope", x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, inner, weight.shape[0], split,
             0 if q_weight is None else q_weight.data_ptr(), 0 if k_weight is None else k_weight.data_ptr(),
             int(q_weight is not None and q_weight.dtype == torch.float32), 0 if inv_freq is None else inv_freq.data_ptr(),
             positions.data_ptr(), seq_of_token.data_ptr(), block_tables.data_ptr(), block_tables.shape[-1],
             k_pages.data_ptr(), v_pages.data_ptr(), n_q_heads, n_kv_heads, head_dim, k_pages.shape[2], k_pages.shape[0],
             float(eps), int(write_cache), page_error.data_ptr(), *scale, error_flag(x.device).data_ptr(), stream_handle())

    if rows <= 16:
        split = _plan_for(x, weight, torch.bfloat16, own_kernel_only=True)      # few rows: always this package's kernel
    else:
        def apart() -> None:      # what the caller would run instead (it writes the same values to the same places)
            from . import qk_norm_rope_kv_write
            torch.matmul(x, weight.t(), out=out)
            qk_norm_rope_kv_write(out, q_weight, k_weight, inv_freq, positions, seq_of_token, block_tables, k_pages, v_pages,
                                  n_q_heads, n_kv_heads, head_dim, eps, write_cache, page_error)

        split = _plan_fused("qkv-rope", rows, weight.shape[0], inner, fused, apart, x.device)
        if split == 0:
            return None
    fused(max(split, 0))
    return out


FUSE_GATE_UP_SILU = os.environ.get("LLMSERVER_B200_FUSE_GATE_UP_SILU", "1") != "0"


def gate_up_silu_fused(x: torch.Tensor, weight: torch.Tensor) -> Optional[torch.Tensor]:
    """silu(gate) * up in the epilogue of the product for few rows; ``weight`` is the fused [2 I, H] matrix with gate
    and up rows interleaved in groups of 64.  None when the product kernel does not take the case (the caller then
    runs the product and the activation kernel)."""
    scale, x = scale_args_of(x), rows_of(x)
    rows, inner = x.shape
    cols = weight.shape[0]
    if not (FUSE_GATE_UP_SILU and rows <= SMALL_M and cols % 128 == 0 and x.is_contiguous() and weight.is_contiguous()
            and weight.dtype == torch.bfloat16 and small_m_supported(rows, cols, inner)):
        return None
    out = torch.empty((rows, cols // 2), dtype=torch.bfloat16, device=x.device)

    def fused(split: int) -> None:
        call("llm_gemm_gate_up_silu", x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, cols, inner, cols // 2, split,
             *scale, error_flag(x.device).data_ptr(), stream_handle())

    # up to 16 rows this package's kernel, whatever a measurement of the bare products says (whole steps are faster with
    # it there, and the activation kernel goes away); with more rows whichever is measured faster: the fused kernel, or
    # the library's product followed by the activation kernel
    if rows <= 16:
        split = _plan_for(x, weight, torch.bfloat16, own_kernel_only=True)
    else:
        def apart() -> None:
            from . import silu_mul
            silu_mul(torch.matmul(x, weight.t()), out=out, group=64)

        split = _plan_fused("gate-up-silu", rows, cols, inner, fused, apart, x.device)
        if split == 0:
            return None
    fused(max(split, 0))
    return out
